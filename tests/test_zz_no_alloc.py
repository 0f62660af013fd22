"""The allocation-free LM-head arg-max entry point against the regular one.

Some users of the library cannot let a call allocate device memory: their own pool
owns the card, or they call from a place where cudaMalloc's device-wide
synchronisation is not acceptable.  ``map_matvec_argmax_t_xq4_static_dev`` serves
them from a fixed array inside the library.  This file is collected last on purpose
(zz): a run that stops at the first failure has then already run every other test.
It passes on its own in a fresh process and after the rest of the suite.
"""
import numpy as np
import pytest

import adam_b200 as A
from adam_b200 import gguf_blocks as gb
from oracle import cref

pytestmark = pytest.mark.gpu

WS, WT = 0, 1


def _setup(gpu, ggml_type, N, K, seed):
    rng = np.random.default_rng(seed)
    raw = (gb.random_q4_0_blocks if ggml_type == 2 else gb.random_q4_k_blocks)(rng, N, K)
    dt = A.DTYPE_GGUF_Q4_0 if ggml_type == 2 else A.DTYPE_GGUF_Q4_K
    gpu.map_create_typed(WT, dt, 1, N * K)
    gpu.upload_gguf_blocks(WT, ggml_type, 0, raw)
    gpu.map_create_typed(WS, A.DTYPE_F32, 1, K + 16)
    h = {k: gpu.upload_dev(np.array([v], np.uint32))[0] for k, v in dict(a=0, b=0, d0=K + 4, d1=K + 8, tmp=0).items()}
    return rng, h


def _both(gpu, h, K, N, x, rows_per_group=256):
    """Token id from the regular entry point and from the allocation-free one."""
    gpu.scatter_contiguous(WS, 0, x)
    gpu.batch_begin()
    gpu.map_matvec_argmax_t_xq4_dev(WS, WT, h["a"], h["b"], h["tmp"], h["tmp"], h["d0"], K, N, rows_per_group)
    gpu.map_matvec_argmax_t_xq4_static_dev(WS, WT, h["a"], h["b"], h["tmp"], h["tmp"], h["d1"], K, N, rows_per_group)
    gpu.batch_end()
    out = gpu.gather(WS, np.array([K + 4, K + 8], np.uint32)).view(np.float32)
    return int(out[0]), int(out[1])


@pytest.mark.parametrize("ggml_type,N,K", [(2, 40000, 1152), (12, 3000, 512), (2, 37, 64)])
def test_static_scratch_argmax_equals_regular_entry_point(gpu, ggml_type, N, K):
    import torch
    rng, h = _setup(gpu, ggml_type, N, K, seed=N)
    raw = (gb.random_q4_0_blocks if ggml_type == 2 else gb.random_q4_k_blocks)(np.random.default_rng(N), N, K)   # what _setup uploaded
    # two calls in a row: the second one finds the first one's leftovers in the shared array
    for _ in range(2):
        x = rng.standard_normal(K).astype(np.float32)
        ref, got = _both(gpu, h, K, N, x)
        assert got == ref                       # token ids: exact
        y = cref.gemv_f64(raw, ggml_type, N, K, x)[0]                  # the oracle's product: same winner
        top = np.sort(y)[-2:]
        if top[1] - top[0] > 1e-4 * np.abs(y).max():                   # (unless two rows tie within the kernel's tolerance)
            assert got == int(np.argmax(y))
    # the call itself must not allocate: free device memory is the same before and after
    x = rng.standard_normal(K).astype(np.float32)
    gpu.scatter_contiguous(WS, 0, x)
    gpu.sync()
    free0, _ = torch.cuda.mem_get_info(gpu.device_index)
    gpu.batch_begin()
    gpu.map_matvec_argmax_t_xq4_static_dev(WS, WT, h["a"], h["b"], h["tmp"], h["tmp"], h["d1"], K, N, 256)
    gpu.batch_end()
    free1, _ = torch.cuda.mem_get_info(gpu.device_index)
    assert free1 == free0
    # small groups: fewer CTAs than the regular launch, same winner
    x = rng.standard_normal(K).astype(np.float32)
    ref, got = _both(gpu, h, K, N, x, rows_per_group=max(16, N // 4000 + 1))
    assert got == ref
    assert gpu.device_error() == 0
    for v in h.values():
        gpu.free_handle(v)


def test_static_scratch_rejects_sizes_beyond_its_capacity(gpu):
    N, K = 8200, 64
    rng, h = _setup(gpu, 2, N, K, seed=1)
    with pytest.raises(RuntimeError, match="partial slots"):          # 8200 rows / 2 per group = 4100 > 4096 slots
        gpu.map_matvec_argmax_t_xq4_static_dev(WS, WT, h["a"], h["b"], h["tmp"], h["tmp"], h["d1"], K, N, 2)
    x = rng.standard_normal(K).astype(np.float32)
    ref, got = _both(gpu, h, K, N, x, rows_per_group=4)              # 2050 slots: fits
    assert got == ref
    for v in h.values():
        gpu.free_handle(v)
