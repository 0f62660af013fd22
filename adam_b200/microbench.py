"""GEMV micro-benchmarks through the C ABI.

    python -m adam_b200.microbench gemv  [--type 2|12] [--n N --k K] [--batch B]   # bandwidth sweep
    python -m adam_b200.microbench gemv-once --type 2 --n 262144 --k 1152 --reps 4  # a few launches (for ncu)

``gemv`` replays a CUDA graph whose launches walk over enough distinct copies of the weight matrix
to exceed L2 (cold HBM), times it with CUDA events on the library stream, and prints one JSON line per
shape: GB/s of algorithmic bytes (GGUF block bytes + fp32 x + fp32 y), the fraction of the measured
copy bandwidth (``MEASURED_PEAKS.json`` if present) and of the nominal 8 TB/s, and the warm
(L2-resident) per-launch latency.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import gguf_blocks as gb

SWEEP = [(2, 6912, 1152, 1), (2, 1152, 6912, 1), (2, 262144, 1152, 1), (12, 5376, 5376, 1), (12, 21504, 5376, 1),
         (12, 5376, 21504, 1), (12, 262144, 5376, 1), (12, 21504, 5376, 8), (2, 262144, 1152, 8)]


def _peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"])
    except Exception:
        return 6650.0


def _weights(gpu, A, t, N, K, copies, tile=False):
    dt = A.DTYPE_GGUF_Q4_0 if t == 2 else A.DTYPE_GGUF_Q4_K
    rng = np.random.default_rng(0)
    ru = min(N, 4096)
    raw_u = (gb.random_q4_0_blocks if t == 2 else gb.random_q4_k_blocks)(rng, ru, K)
    raw = np.tile(raw_u, (N // ru + 1, 1))[:N]
    gpu.map_create_typed(1, dt, 1, copies * N * K)
    for c in range(copies):
        gpu.upload_gguf_blocks(1, t, c * N * K, raw)
        if tile and N % 16 == 0 and K % (64 if t == 2 else 256) == 0:
            gpu.tile_tensor(1, c * N * K, N, K)
    return rng


def run_shape(gpu, A, t, N, K, B=1, target_bytes=600e6, reps=5, tile=False):
    wbytes = N * K * 0.5625
    copies = int(min(160, max(1, np.ceil(target_bytes / wbytes))))
    rng = _weights(gpu, A, t, N, K, copies, tile)
    gpu.map_create_typed(0, A.DTYPE_F32, 1, B * K + B * N + 8)
    gpu.scatter_contiguous(0, 0, rng.standard_normal(B * K).astype(np.float32))
    a_h = gpu.upload_dev(np.array([0], np.uint32))[0]
    c_h = gpu.upload_dev(np.array([B * K], np.uint32))[0]
    bhs = [gpu.upload_dev(np.array([c * N * K], np.uint32))[0] for c in range(copies)]
    tc0 = gpu.tc_gemm_count()
    gpu.map_matmul_t_xq4_dev(0, 1, a_h, bhs[0], c_h, B, K, N)       # eager once: workspaces are allocated outside the capture
    tc_path = gpu.tc_gemm_count() > tc0
    gpu.capture_begin()
    for c in range(copies):
        gpu.map_matmul_t_xq4_dev(0, 1, a_h, bhs[c], c_h, B, K, N)
    gid = gpu.capture_end()
    gpu.graph_launch(gid, 3)
    best = 1e30
    for _ in range(reps):
        gpu.batch_begin(); gpu.timer_begin(); gpu.graph_launch(gid, 1); ms = gpu.timer_end(); gpu.batch_end()
        best = min(best, ms)
    alg = wbytes + 4 * K * B + 4 * N * B
    gbs = alg * copies / (best * 1e-3) / 1e9
    gpu.capture_begin()
    for _ in range(20):
        gpu.map_matmul_t_xq4_dev(0, 1, a_h, bhs[0], c_h, B, K, N)
    gid2 = gpu.capture_end()
    gpu.graph_launch(gid2, 2)
    gpu.batch_begin(); gpu.timer_begin(); gpu.graph_launch(gid2, 1); ms2 = gpu.timer_end(); gpu.batch_end()
    peak = _peak()
    out = dict(type="Q4_0" if t == 2 else "Q4_K", kernel="tcgen05 GEMM" if tc_path else ("tensor-core (tiled)" if tile else "generic"), N=N, K=K, B=B, copies=copies, bytes_per_launch=int(alg),
               us_per_launch=round(best * 1e3 / copies, 3), GBs=round(gbs, 1), frac_of_measured=round(gbs / peak, 3),
               frac_of_8TBs=round(gbs / 8000, 3), warm_us_per_launch=round(ms2 * 1e3 / 20, 3))
    gpu.graph_destroy(gid); gpu.graph_destroy(gid2)
    for h in [a_h, c_h] + bhs:
        gpu.free_handle(h)
    gpu.map_destroy(1)
    return out


def run_once(gpu, A, t, N, K, B, reps, tile=False):
    rng = _weights(gpu, A, t, N, K, 1, tile)
    gpu.map_create_typed(0, A.DTYPE_F32, 1, B * K + B * N + 8)
    gpu.scatter_contiguous(0, 0, rng.standard_normal(B * K).astype(np.float32))
    a_h = gpu.upload_dev(np.array([0], np.uint32))[0]
    b_h = gpu.upload_dev(np.array([0], np.uint32))[0]
    c_h = gpu.upload_dev(np.array([B * K], np.uint32))[0]
    for _ in range(reps):
        gpu.map_matmul_t_xq4_dev(0, 1, a_h, b_h, c_h, B, K, N)
    gpu.sync()
    return gpu.device_error()


def main():
    import adam_b200 as A
    ap = argparse.ArgumentParser()
    ap.add_argument("cmd", choices=["gemv", "gemv-once"])
    ap.add_argument("--type", type=int, default=0)
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--tile", action="store_true", help="register row-tiled copies (tensor-core kernel for Q4_0)")
    a = ap.parse_args()
    gpu = A.init()
    try:
        if a.cmd == "gemv-once":
            err = run_once(gpu, A, a.type or 2, a.n or 262144, a.k or 1152, a.batch, a.reps, a.tile)
            print(json.dumps({"ok": err == 0}))
        else:
            shapes = [(a.type, a.n, a.k, a.batch)] if a.type and a.n and a.k else SWEEP
            for s in shapes:
                print(json.dumps(run_shape(gpu, A, *s, tile=a.tile)), flush=True)
    finally:
        gpu.shutdown()


if __name__ == "__main__":
    main()
