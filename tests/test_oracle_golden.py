"""The oracle against outputs of the unmodified reference (committed fixtures
made by tests/golden/make_golden.py).  CPU only."""
import hashlib
import os
from dataclasses import replace

import numpy as np
import pytest

from adam_b200 import gguf_blocks as gb
from adam_b200 import synth
from adam_b200.config import tiny_gemma3
from oracle import q4_blocks
from oracle.decoder import OracleDecoder, dequant_model

from tests.golden.make_golden import DECODE_CASES


def _bits_equal(a, b):
    a = np.asarray(a, np.float32); b = np.asarray(b, np.float32)
    return bool(((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all())


def test_q4_0_decode_bit_exact(golden_dir):
    g = np.load(os.path.join(golden_dir, "q4_dequant.npz"))
    assert _bits_equal(q4_blocks.dequant_q4_0(g["q4_0_raw"]), g["q4_0_out"])


def test_q4_k_decode_bit_exact(golden_dir):
    g = np.load(os.path.join(golden_dir, "q4_dequant.npz"))
    with np.errstate(invalid="ignore", over="ignore"):
        assert _bits_equal(q4_blocks.dequant_q4_k(g["q4_k_raw"]), g["q4_k_out"])


def test_q4_0_encoder_matches_gguf(golden_dir):
    g = np.load(os.path.join(golden_dir, "q4_0_quantize.npz"))
    assert np.array_equal(gb.quantize_q4_0(g["w"]), g["raw"])


@pytest.mark.parametrize("kind", ["q8_0", "q5_0"])
def test_q8_0_q5_0_decode_bit_exact(golden_dir, kind):
    """adam/loaders/gguf.py:282-288 (_dq8), :301-310 (_dq5_0): numpy and C restatements against the reference's output."""
    from oracle import cref
    g = np.load(os.path.join(golden_dir, "q8_q5_blocks.npz"))
    raw, want = g[f"{kind}_raw"], g[f"{kind}_out"]
    dec = q4_blocks.dequant_q8_0 if kind == "q8_0" else q4_blocks.dequant_q5_0
    with np.errstate(invalid="ignore", over="ignore"):
        assert _bits_equal(dec(raw), want)
        assert _bits_equal(cref.dequant(raw, 8 if kind == "q8_0" else 6, raw.shape[0], 32).reshape(-1), want)


def test_q8_0_q5_0_encoders_match_gguf(golden_dir):
    g = np.load(os.path.join(golden_dir, "q8_q5_blocks.npz"))
    assert np.array_equal(gb.quantize_q8_0(g["w"]), g["q8_0_enc"])
    assert np.array_equal(gb.quantize_q5_0(g["w"]), g["q5_0_enc"])


def test_q4_k_scale_pack_roundtrip():
    rng = np.random.default_rng(3)
    sc = rng.integers(0, 64, (50, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, (50, 8), dtype=np.uint8)
    s2, m2 = q4_blocks.unpack_q4_k_scales(gb.pack_q4_k_scales(sc, mn))
    assert np.array_equal(s2, sc) and np.array_equal(m2, mn)


def test_q4_k_encoder_reconstructs():
    rng = np.random.default_rng(4)
    w = rng.standard_normal((8, 512), dtype=np.float32) * np.float32(0.02)
    raw = gb.quantize_q4_k(w)
    assert raw.shape == (8, 2 * 144)
    deq = q4_blocks.dequant_q4_k(raw).reshape(8, 512)
    # 4-bit affine per 32: error at most about half a step of the widest sub-block
    assert np.abs(deq - w).max() < 0.012
    assert np.sqrt(np.mean((deq - w) ** 2)) < 0.004


def test_q4map_model_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "q4map_model.npz"))
    codes = q4_blocks.q4map_quantize(g["data"], g["scales"], g["zeros"], 32)
    deq = q4_blocks.q4map_dequantize(codes, g["scales"], g["zeros"], 32)
    assert _bits_equal(deq, g["deq"])


def test_q4k_to_q4map_is_lossless():
    rng = np.random.default_rng(5)
    raw = gb.random_q4_k_blocks(rng, 4, 512)
    codes, scales, zeros = q4_blocks.q4k_to_q4map_params(raw)
    a = q4_blocks.q4map_dequantize(codes, scales, zeros, 32)
    b = q4_blocks.dequant_q4_k(raw)
    # q*s + (-(m)) and q*s - m are the same float32 operation
    assert _bits_equal(a, b)


@pytest.mark.parametrize("case", DECODE_CASES, ids=[c[0] for c in DECODE_CASES])
def test_decoder_reproduces_reference_tokens(golden_dir, case):
    name, bkw, ckw, n_prompt, n_gen = case
    g = np.load(os.path.join(golden_dir, "decode_tiny.npz"))
    cfg = replace(tiny_gemma3(), **ckw)
    if "head_dim" in ckw:
        cfg = replace(cfg, head_dim_kv=ckw["head_dim"])
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, **bkw)
    h = hashlib.sha256()
    for k in sorted(tensors):
        t = tensors[k]
        h.update(t.tobytes() if isinstance(t, np.ndarray) else t.raw.tobytes())
    assert np.array_equal(np.frombuffer(h.digest(), np.uint8), g[f"{name}_sha256"]), "synthetic model changed"
    prompt = synth.random_prompt(cfg.n_vocab, n_prompt, seed=bkw["seed"] + 100)
    assert np.array_equal(prompt, g[f"{name}_prompt"])
    dec = OracleDecoder(cfg, dequant_model(tensors), kv_cap=n_prompt + n_gen + 1)
    toks, _ = dec.generate(prompt, n_gen)
    assert toks == g[f"{name}_tokens"].tolist()


def test_decoder_extensions_are_inert_when_off():
    """window / fp16-KV / TP flags change nothing when the sequence is shorter
    than the window, and stay close when on."""
    cfg = replace(tiny_gemma3(), sliding_window=8)
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=21, tied=False)
    f32 = dequant_model(tensors)
    prompt = synth.random_prompt(cfg.n_vocab, 6, seed=5)
    base = OracleDecoder(cfg, f32, 32)
    win = OracleDecoder(cfg, f32, 32, window=True)
    for i, t in enumerate(prompt):
        a = base.forward(int(t), i)
        b = win.forward(int(t), i)
    assert np.array_equal(a, b)          # 6 <= window 8
    for i in range(6, 14):
        a = base.forward(3, i)
        b = win.forward(3, i)
    assert not np.array_equal(a, b)      # window now truncates local layers
    tp = OracleDecoder(cfg, f32, 32, tp_size=2)
    h16 = OracleDecoder(cfg, f32, 32, kv_dtype=np.float16)
    base.reset()
    for i, t in enumerate(prompt):
        a = base.forward(int(t), i)
        c = tp.forward(int(t), i)
        d = h16.forward(int(t), i)
    assert np.abs(a - c).max() < 1e-4 * np.abs(a).max() + 1e-5
    assert np.abs(a - d).max() < 5e-3 * np.abs(a).max() + 1e-4
