"""GGUF Q8_0 / Q5_0 block storage and the GGUF file -> device path, through the C ABI.

* decode bit-exact against the UNMODIFIED reference loader's output (tests/golden/q8_q5_blocks.npz from
  adam/loaders/gguf.py:282-288, :301-310), uploads at an offset and from a device pointer;
* the reference's 8-bit operators on such maps -- row fetch (adamah.c:10189) and C = A @ B^T
  (adamah.c:9834) -- and the fused LM-head operators (arg-max, per-group top-k) against the oracle;
* the decoder with a Q8_0 / Q5_0 token embedding (tied and untied LM head) against the oracle decoder;
* a model read from a .gguf file: ids and logits equal the oracle's on the same blocks, and a tensor
  larger than the staging buffers lands byte for byte where a host upload puts it.
"""
import os

import numpy as np
import pytest

import adam_b200 as A
from adam_b200 import gguf_blocks as gb
from adam_b200 import synth
from adam_b200.config import GenerationConfig, tiny_gemma3
from adam_b200.engine import ADAMEngine
from oracle import cref
from oracle import q4_blocks
from oracle.decoder import OracleDecoder, dequant_model

from tests.golden.make_golden import GGUF_FILE_BUILD, GGUF_FILE_CFG, write_model_gguf

pytestmark = pytest.mark.gpu

GREEDY = dict(top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=())
WS, WT = 0, 1
KINDS = {"q8_0": (8, A.DTYPE_GGUF_Q8_0, 34, gb.random_q8_0_blocks), "q5_0": (6, A.DTYPE_GGUF_Q5_0, 22, gb.random_q5_0_blocks)}


def _bits_equal(a, b):
    a = np.asarray(a, np.float32); b = np.asarray(b, np.float32)
    return bool(((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all())


def _h(gpu, vals):
    return gpu.upload_dev(np.asarray(vals, np.uint32))[0]


def _rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


@pytest.mark.parametrize("kind", list(KINDS))
def test_decode_bit_exact_against_the_reference_loader(gpu, golden_dir, kind):
    ggml, dtype, bb, _ = KINDS[kind]
    g = np.load(os.path.join(golden_dir, "q8_q5_blocks.npz"))
    raw, want = g[f"{kind}_raw"], g[f"{kind}_out"]
    nb = raw.shape[0]
    gpu.map_create_typed(WT, dtype, 1, (nb + 8) * 32)
    # at a block offset, in two pieces
    gpu.upload_gguf_blocks(WT, ggml, 4 * 32, raw[:5].reshape(-1))
    gpu.upload_gguf_blocks(WT, ggml, 9 * 32, raw[5:].reshape(-1))
    with np.errstate(invalid="ignore", over="ignore"):
        assert _bits_equal(gpu.dequant_gguf(WT, 4 * 32, nb * 32), want)
        assert _bits_equal(gpu.dequant_gguf(WT, 6 * 32, 64), want[64:128])
    # untouched blocks read as zero; a type that does not match the map is refused
    assert not gpu.dequant_gguf(WT, 0, 4 * 32).any()
    assert gpu._lib.map_upload_gguf_blocks(WT, 2, 0, raw.ctypes.data, 18) == -3
    assert gpu._lib.map_upload_gguf_blocks(WT, ggml, 16, raw.ctypes.data, bb) == -3          # not on a block boundary
    assert gpu._lib.map_upload_gguf_blocks(WT, ggml, (nb + 7) * 32, raw.ctypes.data, 2 * bb) == -3   # beyond the map
    # blocks that already lie on the device
    import torch
    dev = torch.from_numpy(raw.reshape(-1).copy()).cuda()
    torch.cuda.synchronize()
    gpu.map_create_typed(WT, dtype, 1, nb * 32)
    gpu.upload_gguf_blocks(WT, ggml, 0, int(dev.data_ptr()), int(dev.numel()))
    with np.errstate(invalid="ignore", over="ignore"):
        assert _bits_equal(gpu.dequant_gguf(WT, 0, nb * 32), want)
    gpu.map_destroy(WT)
    assert gpu.device_error() == 0


@pytest.mark.parametrize("kind", list(KINDS))
def test_row_gather_xq8(gpu, kind):
    """map_row_gather_xq8.comp: one decoded row times the embedding scale (two roundings) into the float32 map."""
    ggml, dtype, _, gen = KINDS[kind]
    rng = np.random.default_rng(7)
    rows, cols = 50, 1152
    raw = gen(rng, rows, cols)
    w = q4_blocks.dequant(raw.reshape(-1), ggml, rows, cols)
    gpu.map_create_typed(WT, dtype, 1, 64 + rows * cols)
    gpu.upload_gguf_blocks(WT, ggml, 64, raw.reshape(-1))
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, 4096)
    scale = np.float32(np.sqrt(1152.0))
    for row in (0, 17, rows - 1):
        gpu.map_row_gather_xq8_dev(WS, WT, 64, 100, row, cols, float(scale))
        got = gpu.gather(WS, np.arange(100, 100 + cols, dtype=np.uint32)).view(np.float32)
        assert _bits_equal(got, w[row] * scale)
    assert gpu._lib.map_row_gather_xq8_dev(WS, WT, 64, 4000, 0, cols, 1.0) == -3      # destination beyond the map
    assert gpu._lib.map_row_gather_xq8_dev(WS, WT, 64, 0, rows, cols, 1.0) == -3      # row beyond the tensor
    assert gpu._lib.map_row_gather_xq8_dev(WS, WS, 0, 0, 0, 32, 1.0) == -3            # not a Q8_0 / Q5_0 map
    gpu.map_destroy(WT)
    assert gpu.device_error() == 0


def _matmul(gpu, ggml, dtype, raw, N, K, x, entry="xq8"):
    B = x.shape[0]
    gpu.map_create_typed(WT, dtype, 1, N * K)
    gpu.upload_gguf_blocks(WT, ggml, 0, raw.reshape(-1))
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, B * K + B * N + 8)
    gpu.scatter_contiguous(WS, 0, x.reshape(-1))
    hs = [_h(gpu, [0]), _h(gpu, [0]), _h(gpu, [B * K])]
    gpu.batch_begin()
    (gpu.map_matmul_t_xq8_dev if entry == "xq8" else gpu.map_matmul_t_xq4_dev)(WS, WT, hs[0], hs[1], hs[2], B, K, N)
    gpu.batch_end()
    y = gpu.gather(WS, np.arange(B * K, B * K + B * N, dtype=np.uint32)).view(np.float32).reshape(B, N)
    for h in hs:
        gpu.free_handle(h)
    gpu.map_destroy(WT)
    assert gpu.device_error() == 0
    return y


@pytest.mark.parametrize("kind", list(KINDS))
@pytest.mark.parametrize("N,K,B", [(1001, 1152, 1), (256, 32, 1), (4096, 5376, 3), (2050, 21504, 2), (262144, 1152, 1), (8192, 1152, 8), (37, 4096, 7)])
def test_matmul_t_xq8_against_the_oracle(gpu, kind, N, K, B):
    """Random blocks, x ~ N(0,1): every output within 1e-3 of the double-precision product of the decoded weights
    (ragged row counts, one block per row, the LM-head shape, several batch rows)."""
    ggml, dtype, _, gen = KINDS[kind]
    rng = np.random.default_rng(N + 3 * K + B + ggml)
    raw = gen(rng, N, K)
    x = rng.standard_normal((B, K), dtype=np.float32)
    y = _matmul(gpu, ggml, dtype, raw, N, K, x, entry="xq8" if B != 3 else "xq4")
    ref = cref.gemv_f64(raw.reshape(-1), ggml, N, K, x)
    for b in range(B):
        scale = np.abs(ref[b]).max()
        assert np.abs(y[b] - ref[b]).max() < 2e-5 * scale
        big = np.abs(ref[b]) > 0.05 * scale
        assert (np.abs(y[b] - ref[b])[big] / np.abs(ref[b])[big]).max() < 1e-3


def test_matmul_t_xq8_refuses_other_maps(gpu):
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, 256)
    gpu.map_create_typed(WT, A.DTYPE_GGUF_Q4_0, 1, 64)
    h = _h(gpu, [0])
    assert gpu._lib.map_matmul_t_xq8_dev(WS, WT, h, h, h, 1, 32, 2, 1) == -3
    assert gpu._lib.map_matmul_t_xq8_dev(WS, WT, h, h, h, 1, 32, 2, 0) == 0       # n_ops == 0 is a no-op (adamah.c:9856)
    gpu.free_handle(h)
    gpu.map_destroy(WT)


@pytest.mark.parametrize("kind", list(KINDS))
def test_fused_lm_head_operators_on_q8_q5_maps(gpu, kind):
    """map_matvec_argmax_t_xq4_dev and map_matvec_topk_t_xq4_ex_dev accept Q8_0 / Q5_0 maps: winner and per-group top-k
    equal those of the oracle's logits (ties to the lower row)."""
    ggml, dtype, _, gen = KINDS[kind]
    rng = np.random.default_rng(11 + ggml)
    N, K, k, rpg = 5000, 256, 8, 512
    raw = gen(rng, N, K)
    x = rng.standard_normal(K).astype(np.float32)
    ref = cref.gemv_f64(raw.reshape(-1), ggml, N, K, x[None])[0]
    gpu.map_create_typed(WT, dtype, 1, N * K)
    gpu.upload_gguf_blocks(WT, ggml, 0, raw.reshape(-1))
    groups = (N + rpg - 1) // rpg
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, K + 16 + 2 * groups * k)
    gpu.scatter_contiguous(WS, 0, x)
    a_h, b_h, d_h, tmp = _h(gpu, [0]), _h(gpu, [0]), _h(gpu, [K]), _h(gpu, [K + 1])
    gpu.map_matvec_argmax_t_xq4_dev(WS, WT, a_h, b_h, tmp, tmp, d_h, K, N)
    assert int(gpu.gather(WS, np.array([K], np.uint32)).view(np.float32)[0]) == int(ref.argmax())
    idx_h = _h(gpu, K + 16 + np.arange(groups * k))
    val_h = _h(gpu, K + 16 + groups * k + np.arange(groups * k))
    pen_h = _h(gpu, [0])
    gpu.map_matvec_topk_t_xq4_ex_dev(WS, WT, a_h, b_h, pen_h, idx_h, val_h, K, N, k, 0, 1.0, rpg)
    idx = gpu.gather(WS, (K + 16 + np.arange(groups * k)).astype(np.uint32)).view(np.float32).astype(np.int64).reshape(groups, k)
    val = gpu.gather(WS, (K + 16 + groups * k + np.arange(groups * k)).astype(np.uint32)).view(np.float32).reshape(groups, k)
    for gi in range(groups):
        rows = np.arange(gi * rpg, min(N, (gi + 1) * rpg))
        want = rows[np.argsort(-ref[rows], kind="stable")[:k]]
        assert idx[gi].tolist() == want.tolist()
        assert np.allclose(val[gi], ref[want], rtol=1e-4, atol=1e-6)
    for h in (a_h, b_h, d_h, tmp, idx_h, val_h, pen_h):
        gpu.free_handle(h)
    gpu.map_destroy(WT)
    assert gpu.device_error() == 0


@pytest.mark.parametrize("embd_type,tied", [(gb.GGML_TYPE_Q8_0, True), (gb.GGML_TYPE_Q8_0, False), (gb.GGML_TYPE_Q5_0, True)])
@pytest.mark.parametrize("layers", [gb.GGML_TYPE_Q4_0, gb.GGML_TYPE_Q4_K])
def test_decoder_with_q8_q5_embedding_matches_oracle(gpu, embd_type, tied, layers):
    """Token embedding (and the tied or untied LM head) in Q8_0 / Q5_0 next to Q4_0 / Q4_K layers, as real Gemma files
    have it: greedy ids equal the oracle's and teacher-forced logits agree within 1e-3; three sequences at once too."""
    cfg = tiny_gemma3(n_layer=3)
    tensors = synth.build_model(cfg, layers, seed=51 + embd_type, tied=tied, embd_type=embd_type)
    if not tied:       # an untied head of yet another kind: Q4 layers' type
        tensors["output.weight"] = synth.build_model(cfg, layers, seed=99, tied=False)["output.weight"]
    f32 = dequant_model(tensors)
    prompt = synth.random_prompt(cfg.n_vocab, 10, seed=5)
    want, want_logits = OracleDecoder(cfg, f32, kv_cap=64).generate(prompt, 20, keep_logits=True)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=64, kv_dtype="f32", max_batch=3)
    try:
        got, stats = eng.generate(prompt, GenerationConfig(max_tokens=20, **GREEDY))
        assert got == want and stats["sampling_mode"] == "gpu_matvec_argmax"
        out = eng.logits_trace(list(prompt) + want[:-1])
        assert max(_rel(out[len(prompt) - 1 + i], want_logits[i]) for i in range(20)) < 1e-3
        prompts = [prompt, synth.random_prompt(cfg.n_vocab, 7, seed=6), synth.random_prompt(cfg.n_vocab, 13, seed=7)]
        outs, _ = eng.generate_batch(prompts, GenerationConfig(max_tokens=12, **GREEDY))
        for p, o in zip(prompts, outs):
            assert o == OracleDecoder(cfg, f32, kv_cap=64).generate(p, 12)[0]
        assert gpu.device_error() == 0
    finally:
        eng.close()


def test_sampled_decoding_with_q8_embedding_stays_on_the_device(gpu):
    """top-k sampling reads the soft-capped logits the Q8_0 LM head leaves behind: the drawn ids are among the oracle's
    top-k at every step, and greedy sampling (top_k = 1 with a penalty) walks the oracle's penalised arg-max."""
    cfg = tiny_gemma3(n_layer=2)
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=61, tied=True, embd_type=gb.GGML_TYPE_Q8_0)
    prompt = synth.random_prompt(cfg.n_vocab, 8, seed=8)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=64, kv_dtype="f32")
    try:
        got, stats = eng.generate(prompt, GenerationConfig(max_tokens=16, top_k=8, top_p=0.9, temperature=0.7, repeat_penalty=1.0, seed=3, eos_token_ids=()))
        assert stats["sampling_mode"] == "gpu_fused_topk"
        dec = OracleDecoder(cfg, dequant_model(tensors), kv_cap=64)
        seq = list(prompt)
        for i, t in enumerate(seq):
            lg = dec.forward(int(t), i)
        for t in got:
            assert t in np.argsort(-lg, kind="stable")[:8].tolist()
            lg = dec.forward(int(t), len(seq))
            seq.append(t)
        assert gpu.device_error() == 0
    finally:
        eng.close()


def test_model_from_a_gguf_file_matches_oracle(gpu, golden_dir, tmp_path):
    """The committed tiny.gguf (Q4_0 layers, Q8_0 token_embd) and a larger file written here (Q4_K layers, Q5_0
    token_embd, untied Q4_K head): configuration from the file, blocks streamed from the file, ids and logits equal the
    oracle's on the decoded blocks of the model the file was written from."""
    gguf = pytest.importorskip("gguf")
    cases = [(os.path.join(golden_dir, "tiny.gguf"), GGUF_FILE_CFG(),
              synth.build_model(GGUF_FILE_CFG(), gb.GGML_TYPE_Q4_0, embd_type=gb.GGML_TYPE_Q8_0, **GGUF_FILE_BUILD))]
    cfg2 = tiny_gemma3(n_layer=3, sliding_window=8)
    t2 = synth.build_model(cfg2, gb.GGML_TYPE_Q4_K, seed=71, tied=False, embd_type=gb.GGML_TYPE_Q5_0)
    t2["output.weight"] = synth.build_model(cfg2, gb.GGML_TYPE_Q4_K, seed=72, tied=False)["output.weight"]
    p2 = str(tmp_path / "model.gguf")
    write_model_gguf(p2, cfg2, t2, gguf)
    cases.append((p2, cfg2, t2))
    for path, cfg, tensors in cases:
        f32 = dequant_model(tensors)
        prompt = synth.random_prompt(cfg.n_vocab, 9, seed=9)
        want, want_logits = OracleDecoder(cfg, f32, kv_cap=48, window=True).generate(prompt, 16, keep_logits=True)
        eng = ADAMEngine.from_gguf(gpu, path, kv_cap=48, kv_dtype="f32", window=True)
        try:
            for k in ("n_layer", "n_embd", "n_head", "n_head_kv", "head_dim", "n_ff", "n_vocab", "sliding_window"):
                assert getattr(eng.cfg, k) == getattr(cfg, k), k
            got, _ = eng.generate(prompt, GenerationConfig(max_tokens=16, **GREEDY))
            assert got == want
            out = eng.logits_trace(list(prompt) + want[:-1])
            assert max(_rel(out[len(prompt) - 1 + i], want_logits[i]) for i in range(16)) < 1e-3
            assert gpu.device_error() == 0
        finally:
            eng.close()


@pytest.mark.parametrize("ggml,dtype,gen", [(2, A.DTYPE_GGUF_Q4_0, gb.random_q4_0_blocks), (12, A.DTYPE_GGUF_Q4_K, gb.random_q4_k_blocks),
                                            (8, A.DTYPE_GGUF_Q8_0, gb.random_q8_0_blocks)])
def test_file_upload_larger_than_the_staging_buffers(gpu, tmp_path, ggml, dtype, gen):
    """A tensor of about 80 MB (three staging chunks) at an odd file offset: what adam_b200_upload_gguf_file places
    decodes bit for bit like the same bytes uploaded from host memory."""
    rng = np.random.default_rng(ggml)
    rows, cols = 36864 if ggml != 8 else 18432, 4096
    raw = gen(rng, rows, cols).reshape(-1)
    path = str(tmp_path / "blob.bin")
    with open(path, "wb") as f:
        f.write(b"\x5a" * 4098)
        f.write(raw.tobytes())
        f.write(b"\xa5" * 100)
    n = rows * cols
    gpu.map_create_typed(WT, dtype, 1, n + 256)
    gpu.upload_gguf_file(WT, ggml, 256, path, 4098, raw.size)
    gpu.map_create_typed(WT + 1, dtype, 1, n)
    gpu.upload_gguf_blocks(WT + 1, ggml, 0, raw)
    for off, cnt in ((0, 1 << 20), (n // 2 - 256 * 1000, 1 << 20), (n - (1 << 20), 1 << 20)):
        with np.errstate(invalid="ignore", over="ignore"):
            assert _bits_equal(gpu.dequant_gguf(WT, 256 + off, cnt), gpu.dequant_gguf(WT + 1, off, cnt))
    assert _bits_equal(gpu.dequant_gguf(WT + 1, 0, 4096), cref.dequant(raw[:4096 // gb.block_geometry(ggml)[0] * gb.block_geometry(ggml)[1]], ggml, 1, 4096).reshape(-1))
    # a file that ends before the tensor does, and a missing file, are refused
    assert gpu._lib.adam_b200_upload_gguf_file(WT, ggml, 256, os.fsencode(path), 4098 + 4096 * gb.block_geometry(ggml)[1], raw.size) == -3
    assert gpu._lib.adam_b200_upload_gguf_file(WT, ggml, 256, os.fsencode(path + ".none"), 0, raw.size) == -3
    gpu.map_destroy(WT)
    gpu.map_destroy(WT + 1)
    assert gpu.device_error() == 0
