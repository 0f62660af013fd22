"""CUDA GEMV / block decode against the oracle, called through the C ABI."""
import os

import numpy as np
import pytest

import adam_b200 as A
from adam_b200 import gguf_blocks as gb
from oracle import q4_blocks

pytestmark = pytest.mark.gpu

WS, WT = 0, 1          # map ids: float32 workspace, GGUF-block weights


def _bits_equal(a, b):
    a = np.asarray(a, np.float32); b = np.asarray(b, np.float32)
    return bool(((a.view(np.uint32) == b.view(np.uint32)) | (np.isnan(a) & np.isnan(b))).all())


def _gemv(gpu, ggml_type, raw, N, K, x, elem_off=0, pad_elems=0, tile=False):
    """y = W x through map_matmul_t_xq4_dev; x is [B,K].  ``tile`` registers the row-tiled
    copy first, which routes the call to the tensor-core kernel."""
    B = x.shape[0]
    dt = A.DTYPE_GGUF_Q4_0 if ggml_type == 2 else A.DTYPE_GGUF_Q4_K
    gpu.map_create_typed(WT, dt, 1, elem_off + N * K + pad_elems)
    gpu.upload_gguf_blocks(WT, ggml_type, elem_off, raw)
    if tile:
        gpu.tile_tensor(WT, elem_off, N, K)
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, B * K + B * N + 8)
    gpu.scatter_contiguous(WS, 0, x.reshape(-1))
    a_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    b_h, _ = gpu.upload_dev(np.array([elem_off], np.uint32))
    c_h, _ = gpu.upload_dev(np.array([B * K], np.uint32))
    gpu.batch_begin()
    gpu.map_matmul_t_xq4_dev(WS, WT, a_h, b_h, c_h, B, K, N)
    gpu.batch_end()
    y = gpu.gather(WS, np.arange(B * K, B * K + B * N, dtype=np.uint32)).view(np.float32).reshape(B, N)
    for h in (a_h, b_h, c_h):
        gpu.free_handle(h)
    assert gpu.device_error() == 0
    return y


def _check(y, W, x, tol=1e-3):
    ref = x.astype(np.float64) @ W.astype(np.float64).T
    scale = np.abs(ref).max()
    err = np.abs(y - ref).max() / scale
    assert err < tol * 0.05, f"max error {err:.3e} of max |y|"         # far inside the 1e-3 budget
    # element-wise: 1e-3 relative wherever the output is not tiny
    big = np.abs(ref) > 0.05 * scale
    assert (np.abs(y - ref)[big] / np.abs(ref)[big]).max() < tol


def test_dequant_q4_0_bit_exact_vs_reference(gpu, golden_dir):
    g = np.load(os.path.join(golden_dir, "q4_dequant.npz"))
    raw = g["q4_0_raw"]
    n = raw.shape[0] * 32
    gpu.map_create_typed(WT, A.DTYPE_GGUF_Q4_0, 1, n)
    gpu.upload_gguf_blocks(WT, 2, 0, raw)
    assert _bits_equal(gpu.dequant_gguf(WT, 0, n), g["q4_0_out"])


def test_dequant_q4_k_bit_exact_vs_reference(gpu, golden_dir):
    g = np.load(os.path.join(golden_dir, "q4_dequant.npz"))
    raw = g["q4_k_raw"]
    n = raw.shape[0] * 256
    gpu.map_create_typed(WT, A.DTYPE_GGUF_Q4_K, 1, n)
    gpu.upload_gguf_blocks(WT, 12, 0, raw)
    assert _bits_equal(gpu.dequant_gguf(WT, 0, n), g["q4_k_out"])


def test_dequant_at_offset_and_partial(gpu):
    rng = np.random.default_rng(7)
    raw = gb.random_q4_0_blocks(rng, 8, 256)
    gpu.map_create_typed(WT, A.DTYPE_GGUF_Q4_0, 1, 64 + 8 * 256)
    gpu.upload_gguf_blocks(WT, 2, 64, raw)
    ref = q4_blocks.dequant_q4_0(raw)
    assert _bits_equal(gpu.dequant_gguf(WT, 64 + 512, 256), ref[512:768])


def test_quantize_q4_0_kernel_matches_gguf(gpu, golden_dir):
    import torch
    g = np.load(os.path.join(golden_dir, "q4_0_quantize.npz"))
    w = torch.from_numpy(g["w"]).cuda().contiguous()
    raw = torch.empty(g["raw"].size, dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    gpu.quantize_q4_0_dev(w.data_ptr(), w.numel(), raw.data_ptr())
    assert np.array_equal(raw.cpu().numpy().reshape(g["raw"].shape), g["raw"])


@pytest.mark.parametrize("N,K", [(6912, 1152), (1152, 6912), (1024, 1152), (1152, 1024), (7, 32), (5, 96), (33, 4096), (130, 160)])
def test_q4_0_gemv(gpu, N, K):
    rng = np.random.default_rng(N * 31 + K)
    raw = gb.random_q4_0_blocks(rng, N, K)
    x = rng.standard_normal((1, K), dtype=np.float32)
    y = _gemv(gpu, 2, raw, N, K, x)
    _check(y, q4_blocks.dequant(raw.reshape(-1), 2, N, K), x)


@pytest.mark.parametrize("N,K,B", [(6912, 1152, 1), (1152, 6912, 1), (1536, 1152, 1), (1152, 1024, 1), (16, 64, 1), (48, 128, 1),
                                   (4096, 1152, 2), (2048, 1152, 3), (1024, 6912, 4), (512, 1152, 7), (64, 21504, 1), (32, 8192, 5)])
def test_q4_0_gemv_tensor_core_path(gpu, N, K, B):
    rng = np.random.default_rng(N * 7 + K + B)
    raw = gb.random_q4_0_blocks(rng, N, K)
    x = rng.standard_normal((B, K), dtype=np.float32)
    x[0, :5] = [1e-7, -3e4, 2.5e4, 0.0, -1e-3]            # wide dynamic range in one vector
    y = _gemv(gpu, 2, raw, N, K, x, tile=True)
    _check(y, q4_blocks.dequant(raw.reshape(-1), 2, N, K), x)
    y0 = _gemv(gpu, 2, raw, N, K, x, tile=False)             # same call without the tiled copy
    assert np.abs(y - y0).max() < 1e-4 * np.abs(y0).max()


@pytest.mark.parametrize("ggml_type,N,K,B", [(2, 256, 1152, 33), (12, 128, 1024, 37), (2, 64, 6912, 18)])
def test_tensor_core_path_many_batch_rows(gpu, ggml_type, N, K, B):
    """More than four batch rows: the row groups of one call run side by side in one launch."""
    rng = np.random.default_rng(N + K + B)
    raw = (gb.random_q4_0_blocks if ggml_type == 2 else gb.random_q4_k_blocks)(rng, N, K)
    x = rng.standard_normal((B, K), dtype=np.float32) * rng.uniform(0.01, 100.0, (B, 1)).astype(np.float32)   # a scale per row
    y = _gemv(gpu, ggml_type, raw, N, K, x, tile=True)
    W = q4_blocks.dequant(raw.reshape(-1), ggml_type, N, K)
    for b in range(B):          # every row against its own reference (rows differ in magnitude)
        _check(y[b:b + 1], W, x[b:b + 1])


@pytest.mark.parametrize("ggml_type,N,K,B", [(2, 1152, 1152, 64), (2, 300, 1152, 9), (2, 128, 6912, 33), (2, 1536, 256, 17), (2, 16, 32, 12),
                                             (12, 256, 1024, 64), (12, 2048, 5376, 40), (12, 72, 256, 10)])
def test_tcgen05_gemm_many_rows(gpu, ggml_type, N, K, B):
    """9..64 activation rows run as one tcgen05 GEMM (integer products in tensor memory, block scales in
    fp32): every row within 1e-3 of the dequantised reference, tile edges (N not a multiple of 128),
    a ragged last K chunk and K splits included; the call counter shows the path was taken."""
    rng = np.random.default_rng(7 * N + K + B)
    raw = (gb.random_q4_0_blocks if ggml_type == 2 else gb.random_q4_k_blocks)(rng, N, K)
    x = rng.standard_normal((B, K), dtype=np.float32) * rng.uniform(0.01, 100.0, (B, 1)).astype(np.float32)
    before = gpu.tc_gemm_count()
    gpu.tc_gemm_policy(2)               # small shapes too (by default they stay on the GEMV kernels)
    try:
        y = _gemv(gpu, ggml_type, raw, N, K, x)
    finally:
        gpu.tc_gemm_policy(1)
    assert gpu.tc_gemm_count() == before + 1
    W = q4_blocks.dequant(raw.reshape(-1), ggml_type, N, K)
    for b in range(B):
        _check(y[b:b + 1], W, x[b:b + 1])


def test_tensor_core_path_at_offset_and_bad_shapes(gpu):
    rng = np.random.default_rng(123)
    N, K = 96, 1152
    raw = gb.random_q4_0_blocks(rng, N, K)
    x = rng.standard_normal((1, K), dtype=np.float32)
    y = _gemv(gpu, 2, raw, N, K, x, elem_off=32 * 6, pad_elems=64, tile=True)
    _check(y, q4_blocks.dequant(raw.reshape(-1), 2, N, K), x)
    with pytest.raises(RuntimeError, match="code -3"):
        gpu.tile_tensor(WT, 32 * 6, 40, K)                   # rows not a multiple of 16
    with pytest.raises(RuntimeError, match="code -3"):
        gpu.tile_tensor(WT, 32 * 6, 96, 96)                  # cols not a multiple of 64


@pytest.mark.parametrize("N,K,B", [(5376, 5376, 1), (512, 21504, 1), (2048, 4096, 1), (16, 256, 1), (48, 768, 2), (64, 1024, 3),
                                   (1024, 5376, 4), (128, 2816, 7)])
def test_q4_k_gemv_tensor_core_path(gpu, N, K, B):
    rng = np.random.default_rng(N * 5 + K + B)
    raw = gb.random_q4_k_blocks(rng, N, K)
    x = rng.standard_normal((B, K), dtype=np.float32)
    x[0, :5] = [1e-7, -3e4, 2.5e4, 0.0, -1e-3]
    y = _gemv(gpu, 12, raw, N, K, x, tile=True)
    _check(y, q4_blocks.dequant(raw.reshape(-1), 12, N, K), x)
    y0 = _gemv(gpu, 12, raw, N, K, x, tile=False)
    assert np.abs(y - y0).max() < 1e-4 * np.abs(y0).max()


@pytest.mark.parametrize("N,K", [(5376, 5376), (512, 21504), (2048, 4096), (3, 256), (9, 768), (64, 1024)])
def test_q4_k_gemv(gpu, N, K):
    rng = np.random.default_rng(N * 17 + K)
    raw = gb.random_q4_k_blocks(rng, N, K)
    x = rng.standard_normal((1, K), dtype=np.float32)
    y = _gemv(gpu, 12, raw, N, K, x)
    _check(y, q4_blocks.dequant(raw.reshape(-1), 12, N, K), x)


@pytest.mark.parametrize("ggml_type,N,K,B", [(2, 300, 1152, 2), (2, 256, 6912, 3), (2, 64, 1024, 8), (12, 128, 5376, 8),
                                             (12, 40, 21504, 8), (12, 100, 512, 5), (2, 50, 64, 13)])
def test_gemv_batched(gpu, ggml_type, N, K, B):
    rng = np.random.default_rng(N + K + B)
    raw = (gb.random_q4_0_blocks if ggml_type == 2 else gb.random_q4_k_blocks)(rng, N, K)
    x = rng.standard_normal((B, K), dtype=np.float32)
    y = _gemv(gpu, ggml_type, raw, N, K, x)
    _check(y, q4_blocks.dequant(raw.reshape(-1), ggml_type, N, K), x)


def test_gemv_tensor_at_offset(gpu):
    rng = np.random.default_rng(99)
    N, K = 96, 1152
    raw = gb.random_q4_0_blocks(rng, N, K)
    x = rng.standard_normal((1, K), dtype=np.float32)
    y = _gemv(gpu, 2, raw, N, K, x, elem_off=32 * 5, pad_elems=64)
    _check(y, q4_blocks.dequant(raw.reshape(-1), 2, N, K), x)


def test_gemv_is_linear_in_x_at_full_size(gpu):
    """Size-independent property on the LM-head shape: W(ax + by) = aWx + bWy."""
    rng = np.random.default_rng(5)
    N, K = 262144, 1152
    raw = gb.random_q4_0_blocks(rng, N, K)
    x = rng.standard_normal((3, K), dtype=np.float32)
    x[2] = 0.5 * x[0] - 2.0 * x[1]
    y = _gemv(gpu, 2, raw, N, K, x)
    comb = 0.5 * y[0].astype(np.float64) - 2.0 * y[1].astype(np.float64)
    assert np.abs(y[2] - comb).max() < 2e-5 * np.abs(comb).max()
    rows = rng.integers(0, N, 64)
    W = q4_blocks.dequant(raw[rows].reshape(-1), 2, 64, K)
    ref = x.astype(np.float64) @ W.astype(np.float64).T
    assert np.abs(y[:, rows] - ref).max() < 5e-5 * np.abs(ref).max()


def test_gemv_rejects_bad_arguments(gpu):
    gpu.map_create_typed(WT, A.DTYPE_GGUF_Q4_0, 1, 64 * 32)
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, 256)
    a_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    with pytest.raises(RuntimeError, match="code -3"):
        gpu.map_matmul_t_xq4_dev(WS, WT, a_h, a_h, a_h, 1, 48, 4)        # K not a whole block
    with pytest.raises(RuntimeError, match="code -3"):
        gpu.map_matmul_t_xq4_dev(WS, WT, a_h, a_h, a_h, 1, 64, 64)       # weight range beyond the map
    with pytest.raises(RuntimeError, match="code -4"):
        gpu.map_matmul_t_xq4_dev(WS, 9, a_h, a_h, a_h, 1, 32, 4)         # no such map
    with pytest.raises(RuntimeError, match="code -4"):
        gpu.map_matmul_t_xq4_dev(WS, WT, 60000, a_h, a_h, 1, 32, 4)      # no such handle
    with pytest.raises(RuntimeError):
        gpu.upload_gguf_blocks(WT, 12, 0, np.zeros(144, np.uint8))        # type does not match the map
    gpu.free_handle(a_h)


@pytest.mark.parametrize("tile", [False, True])
def test_matvec_argmax_matches_full_logits(gpu, tile):
    rng = np.random.default_rng(11)
    N, K = 20000, 1152
    raw = gb.random_q4_0_blocks(rng, N, K)
    x = rng.standard_normal((1, K), dtype=np.float32)
    y = _gemv(gpu, 2, raw, N, K, x, tile=tile)[0]
    # same maps are still alive: fused LM head + arg-max writes the id as float32
    a_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    b_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    d_h, _ = gpu.upload_dev(np.array([K + 3], np.uint32))
    t_h, _ = gpu.upload_dev(np.zeros(4, np.uint32))
    gpu.batch_begin()
    gpu.map_matvec_argmax_t_xq4_dev(WS, WT, a_h, b_h, t_h, t_h, d_h, K, N, 256)
    gpu.batch_end()
    tok = int(gpu.gather(WS, np.array([K + 3], np.uint32)).view(np.float32)[0])
    assert tok == int(np.argmax(y))
    for h in (a_h, b_h, d_h, t_h):
        gpu.free_handle(h)


@pytest.mark.parametrize("tile", [False, True])
def test_fused_argmax_tie_goes_to_the_lower_index(gpu, tile):
    """Two identical rows share the largest product: the fused LM head + arg-max must name the lower one
    (the reference's `better`, map_argmax.comp; its known-answer test is tests/test_decode_primitives.py:17-29)."""
    rng = np.random.default_rng(21)
    N, K = 4096, 1152
    raw = gb.random_q4_0_blocks(rng, N, K)
    lo, hi = 700, 3001                                  # different 16-row groups, different CTAs
    raw[hi] = raw[lo]
    x = (q4_blocks.dequant(raw[lo].reshape(-1), 2, 1, K)[0] * 50.0).astype(np.float32)[None, :]
    y = _gemv(gpu, 2, raw, N, K, x, tile=tile)[0]
    assert y[lo] == y[hi] == y.max()
    a_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    b_h, _ = gpu.upload_dev(np.array([0], np.uint32))
    d_h, _ = gpu.upload_dev(np.array([K + 3], np.uint32))
    t_h, _ = gpu.upload_dev(np.zeros(4, np.uint32))
    gpu.batch_begin()
    gpu.map_matvec_argmax_t_xq4_dev(WS, WT, a_h, b_h, t_h, t_h, d_h, K, N, 256)
    gpu.batch_end()
    assert int(gpu.gather(WS, np.array([K + 3], np.uint32)).view(np.float32)[0]) == lo
    for h in (a_h, b_h, d_h, t_h):
        gpu.free_handle(h)
