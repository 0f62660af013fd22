"""Parity at the benchmark configurations' own sizes, through the C ABI.

* Gemma-3-1B shape (26 layers, hidden 1152, vocabulary 262144, Q4_0), 128-token prompt, 128
  greedy tokens: ids equal the UNMODIFIED reference decoder's ids (tests/golden/decode_1b.npz,
  written by tests/golden/make_golden.py --full-size from tests/diagnostics/diag_inference.py:917-1074),
  tied and untied LM head; and, with the fp16 paged cache and the sliding-window mask of the
  benchmark configuration, ids and teacher-forced logits equal the oracle's (flagged extensions).
* Q4_K GEMV at the 27B widths (5376x5376, 21504x5376, 5376x21504, 262144x5376), one and eight
  batch rows, against the C oracle with double-precision sums.
* Gemma-3-27B shape truncated to two layers plus the full LM head, Q4_K: logits and greedy ids
  against the oracle.
"""
import gc
import hashlib
import os

import numpy as np
import pytest

import adam_b200 as A
from adam_b200 import gguf_blocks as gb
from adam_b200 import synth
from adam_b200.config import GenerationConfig, gemma3_1b, gemma3_27b, with_layers
from adam_b200.engine import ADAMEngine
from oracle import cref
from oracle.decoder import OracleDecoder

from tests.golden.make_golden import FULL_SIZE_CASES

pytestmark = pytest.mark.gpu

GREEDY = dict(top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=())
WS, WT = 0, 1


def _rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


def _dequant_all(tensors):
    out = {}
    for k, t in tensors.items():
        out[k] = t if isinstance(t, np.ndarray) else cref.dequant(t.raw, t.ggml_type, t.rows, t.cols)
    return out


@pytest.mark.parametrize("case", FULL_SIZE_CASES, ids=[c[0] for c in FULL_SIZE_CASES])
def test_1b_shape_128_prompt_128_greedy_tokens(gpu, golden_dir, case):
    name, bkw, n_prompt, n_gen = case
    g = np.load(os.path.join(golden_dir, "decode_1b.npz"))
    cfg = gemma3_1b()
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, **bkw)
    h = hashlib.sha256()
    for k in sorted(tensors):
        t = tensors[k]
        h.update(t.tobytes() if isinstance(t, np.ndarray) else t.raw.tobytes())
    assert np.array_equal(np.frombuffer(h.digest(), np.uint8), g[f"{name}_sha256"]), "the model differs from the one the fixture was made from"
    prompt = g[f"{name}_prompt"]
    want_ref = g[f"{name}_tokens"].tolist()
    kv_cap = n_prompt + n_gen + 8

    # (a) the reference's own arithmetic: fp32 cache, every layer attends to every position
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=kv_cap, kv_dtype="f32", window=False)
    try:
        got, stats = eng.generate(prompt, GenerationConfig(max_tokens=n_gen, **GREEDY))
        assert stats["sampling_mode"] == "gpu_matvec_argmax"
        assert got == want_ref, f"first difference at step {next(i for i, (a, b) in enumerate(zip(got, want_ref)) if a != b)}"
        assert gpu.device_error() == 0
    finally:
        eng.close()

    # (b) the benchmark configuration: fp16 paged cache + sliding window on the local layers (oracle extensions)
    f32 = _dequant_all(tensors)
    dec = OracleDecoder(cfg, f32, kv_cap=kv_cap, window=True, kv_dtype=np.float16)
    want, want_logits = dec.generate(prompt, n_gen, keep_logits=True)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=kv_cap, kv_dtype="f16", window=True)
    try:
        got, _ = eng.generate(prompt, GenerationConfig(max_tokens=n_gen, **GREEDY))
        assert got == want
        # teacher-forced logits after positions n_prompt-1 .. n_prompt+n_gen-2 (1e-3 of the largest logit)
        seq = list(prompt) + want[:-1]
        out = eng.logits_trace(seq)
        worst = max(_rel(out[n_prompt - 1 + i], want_logits[i]) for i in range(n_gen))
        assert worst < 1e-3, worst
        assert all(int(out[n_prompt - 1 + i].argmax()) == want[i] for i in range(n_gen))
        assert gpu.device_error() == 0
    finally:
        eng.close()
    # (c) the same configuration with every token as ONE kernel launch (the persistent token kernel)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=kv_cap, kv_dtype="f16", window=True, single_launch=True)
    try:
        gpu.reset_native_stats()
        got, _ = eng.generate(prompt, GenerationConfig(max_tokens=n_gen, **GREEDY))
        assert got == want
        assert gpu.device_error() == 0
    finally:
        eng.close()
        del f32, dec, tensors
        gc.collect()


def _gemv_q4k(gpu, raw, N, K, x):
    B = x.shape[0]
    gpu.map_create_typed(WT, A.DTYPE_GGUF_Q4_K, 1, N * K)
    gpu.upload_gguf_blocks(WT, 12, 0, raw)
    gpu.tile_tensor(WT, 0, N, K)
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, B * K + B * N + 8)
    gpu.scatter_contiguous(WS, 0, x.reshape(-1))
    a_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    b_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    c_h, _ = gpu.upload_dev(np.array([B * K], np.uint32))
    gpu.batch_begin()
    gpu.map_matmul_t_xq4_dev(WS, WT, a_h, b_h, c_h, B, K, N)
    gpu.batch_end()
    y = gpu.gather(WS, np.arange(B * K, B * K + B * N, dtype=np.uint32)).view(np.float32).reshape(B, N)
    for hh in (a_h, b_h, c_h):
        gpu.free_handle(hh)
    gpu.map_destroy(WT)
    assert gpu.device_error() == 0
    return y


@pytest.mark.parametrize("N,K", [(5376, 5376), (21504, 5376), (5376, 21504), (262144, 5376)])
@pytest.mark.parametrize("B", [1, 8])
def test_q4_k_gemv_at_27b_widths(gpu, N, K, B):
    """Random Q4_K superblocks (fp16 d/dmin = |N(0,0.02)|/8, 6-bit scales and mins, 4-bit quants, all uniform),
    x ~ N(0,1): every output within 1e-3 of the double-precision product of the decoded weights."""
    rng = np.random.default_rng(N + 3 * K + B)
    raw = gb.random_q4_k_blocks(rng, N, K)
    x = rng.standard_normal((B, K), dtype=np.float32)
    y = _gemv_q4k(gpu, raw, N, K, x)
    ref = cref.gemv_f64(raw, 12, N, K, x)
    for b in range(B):
        scale = np.abs(ref[b]).max()
        assert np.abs(y[b] - ref[b]).max() < 5e-5 * scale
        big = np.abs(ref[b]) > 0.05 * scale
        assert (np.abs(y[b] - ref[b])[big] / np.abs(ref[b])[big]).max() < 1e-3


def test_27b_shape_two_layers_and_lm_head(gpu):
    """Hidden 5376, 32 query / 16 KV heads of 128, FFN 21504, vocabulary 262144, Q4_K, window 1024 with fp16 cache."""
    cfg = with_layers(gemma3_27b(), 2)
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_K, seed=41, tied=True)
    f32 = _dequant_all(tensors)
    n_prompt, n_gen = 24, 16
    prompt = synth.random_prompt(cfg.n_vocab, n_prompt, seed=141)
    dec = OracleDecoder(cfg, f32, kv_cap=64, window=True, kv_dtype=np.float16)
    want, want_logits = dec.generate(prompt, n_gen, keep_logits=True)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=64, kv_dtype="f16", window=True)
    try:
        got, _ = eng.generate(prompt, GenerationConfig(max_tokens=n_gen, **GREEDY))
        assert got == want
        out = eng.logits_trace(list(prompt) + want[:-1])
        worst = max(_rel(out[n_prompt - 1 + i], want_logits[i]) for i in range(n_gen))
        assert worst < 1e-3, worst
        assert gpu.device_error() == 0
    finally:
        eng.close()
        del f32, dec, tensors
        gc.collect()
