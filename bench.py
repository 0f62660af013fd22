#!/usr/bin/env python3
"""Decode benchmark for the Gemma-3-1B-shaped Q4_0 model (batch 1, 128-token
random prompt, greedy decode): one "step" is one decoded token.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  ``value`` is decode tok/s with everything resident in HBM
(K token steps timed with CUDA events on the library's stream); ``e2e`` is the
same metric through ``ADAMEngine.generate`` with host prompt ids: generated tokens divided by
the whole call's time, i.e. the host->device prompt copy, the chunked prefill, every decode step
and one device->host token read per step are all inside the timed region.
``roofline`` covers the timed region as a whole: the bytes one decoded token has to read (the model's
Q4_0 blocks, the norm vectors, the cached keys and values) over the CUDA-event time of a step, against the
measured HBM copy bandwidth.  A step is a CUDA graph of 133 per-operation kernels by default, or one launch
of the persistent token kernel (``ADAM_B200_SINGLE_LAUNCH=1``); the line carries the other path's time as
``other_step_path``.  ``lm_head_gemv`` is the dequant GEMV operator alone on the
stream (the metric's second half), measured on the LM-head shape, 262144 x 1152 Q4_0, whose 170 MB
exceed L2; ``gemv_sweep`` lists the other GEMV shapes of the benchmark configurations (cold HBM: each
launch of a graph reads a different copy of the weights).  ``cpu_baseline`` is the numpy
restatement of the reference's CPU decoder timed on this box's host cores on a bounded sample
(same weights, same prompt); its greedy ids are compared with the GPU arm's
(``ids_equal_oracle``).  ``tp`` is the Gemma-3-27B-shaped Q4_K model (random blocks, all 62
layers, batch 1) decoded tensor-parallel over the N GPUs of the run (N = 1: the same part-wise
path without collectives).  With N > 1 (torchrun, one rank per GPU) ``value`` comes from N
independent replicas of the 1B model: no collective on that path, weak scaling, value = all
ranks' tokens / slowest rank's time.

Other modes (one JSON line per result; what the summaries under profiles/ were made with):

    python bench.py --mode gemv [--type 2|12 --n N --k K --batch B] [--no-tile]   GEMV bandwidth, one shape or the sweep
    python bench.py --mode gemv-once --type 2 --n 262144 --k 1152 --reps 4          a few launches (for ncu)
    python bench.py --mode batch --batch 32 --prompt 512 --steps 256                batched decode + chunked prefill, 1B shape
    python bench.py --mode tp [--layers L --batch B --allreduce p2p|nccl --shard-of N]   27B-shape tensor-parallel decode
    python bench.py --mode token-once [--layers L] [--chain]                        a few token steps (for ncu): token kernel, or the graph of kernels
    python bench.py --mode token-trace [--layers L]                                 per-phase times inside the token kernel (SM clock stamps)
    ADAM_B200_LIB_PATH=adam_b200/libadam_b200_trace.so python bench.py --mode step-trace   phase times of one layer's five kernels in the default step
                                                                                    (needs `python -m adam_b200.build --step-trace`)
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PROMPT_LEN = 128
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one LM-head GEMV launch, from an ncu capture of
# `bench.py --mode gemv-once --type 2 --n 262144 --k 1152` (same kernel and shape; that
# entry point also stores the 1 MB of logits)
LMHEAD_DRAM_TRAFFIC = 169_949_184 + 4_576_256
# the same two counters for one launch of the token kernel (full 26-layer model, context 130), from an ncu
# capture of `bench.py --mode token-once --steps 4`
TOKEN_DRAM_TRAFFIC = 566_583_808 + 4_014_848
# and summed over the 133 kernels of one step of the CUDA-graph path, from an ncu capture of
# `bench.py --mode token-once --chain --steps 3` (metrics gpu__time_duration, dram__bytes_read, dram__bytes_write)
CHAIN_DRAM_TRAFFIC = 576_930_645 + 333_824


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])); mx = max(mx, float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(sm)}


def dist_env():
    from adam_b200.replicas import dist_env as _env
    return _env()


def set_blas_threads():
    """Use every host core for the numpy BLAS (torchrun exports OMP_NUM_THREADS=1 to its ranks)."""
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=os.cpu_count() or 1)
    except Exception:
        pass


def cpu_decode_sample(cfg, tensors, prompt, n_decode):
    """Numpy restatement of the reference's CPU decoder (tests/diagnostics/diag_inference.py:934-1061)
    on the given weights, with the cache rounding and window mask of the benchmark configuration:
    consumes ``prompt`` token by token, then decodes ``n_decode`` greedy tokens.  Returns (decode
    tok/s, seconds of decode, seconds of prompt, decoded ids)."""
    from oracle.decoder import OracleDecoder
    from oracle import cref
    from adam_b200 import synth
    set_blas_threads()
    f32 = {}
    for name, t in tensors.items():
        if isinstance(t, np.ndarray):
            f32[name] = t
        else:       # the reference pre-decodes every matrix to float32 (diag_inference.py:966-969)
            f32[name] = cref.dequant(synth.raw_to_host(t), t.ggml_type, t.rows, t.cols)
    dec = OracleDecoder(cfg, f32, kv_cap=len(prompt) + n_decode + 1, window=True, kv_dtype=np.float16)
    t0 = time.perf_counter()
    logits = None
    for i, t in enumerate(prompt):
        logits = dec.forward(int(t), i, want_logits=(i == len(prompt) - 1))
    t_prompt = time.perf_counter() - t0
    pos = len(prompt)
    ids = []
    t0 = time.perf_counter()
    for _ in range(n_decode):
        tok = int(np.argmax(logits))
        ids.append(tok)
        logits = dec.forward(tok, pos); pos += 1
    dt = time.perf_counter() - t0
    return n_decode / dt, dt, t_prompt, ids


def threads_used():
    try:
        from threadpoolctl import threadpool_info
        n = [p.get("num_threads", 1) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return max(n)
    except Exception:
        pass
    return os.cpu_count() or 1


# ---- GEMV bandwidth (the metric's second half; configs 1 and 4) ------------------------------------------

GEMV_SWEEP = [(2, 6912, 1152, 1), (2, 1152, 6912, 1), (12, 5376, 5376, 1), (12, 21504, 5376, 1), (12, 5376, 21504, 1),
              (12, 262144, 5376, 1), (12, 5376, 5376, 8), (12, 21504, 5376, 8), (12, 5376, 21504, 8), (12, 262144, 5376, 8),
              (8, 262144, 1152, 1), (6, 262144, 1152, 1)]      # Q8_0 / Q5_0: the token-embedding / LM-head table of the 1B shape
_BLOCK_NAME = {2: "Q4_0", 12: "Q4_K", 8: "Q8_0", 6: "Q5_0"}


def _gemv_weights(gpu, A, t, N, K, copies, tile):
    from adam_b200 import gguf_blocks as gb
    dt = A.GGUF_MAP_DTYPE[t]
    rng = np.random.default_rng(0)
    ru = min(N, 4096)
    raw_u = {2: gb.random_q4_0_blocks, 12: gb.random_q4_k_blocks, 8: gb.random_q8_0_blocks, 6: gb.random_q5_0_blocks}[t](rng, ru, K)
    raw = np.tile(raw_u, (N // ru + 1, 1))[:N]
    gpu.map_create_typed(1, dt, 1, copies * N * K)
    for c in range(copies):
        gpu.upload_gguf_blocks(1, t, c * N * K, raw)
        if tile and t in (2, 12) and N % 16 == 0 and K % (64 if t == 2 else 256) == 0:
            gpu.tile_tensor(1, c * N * K, N, K)
    return rng


def gemv_shape(gpu, A, t, N, K, B=1, target_bytes=600e6, reps=5, tile=True):
    """Cold-HBM bandwidth of y = W x for one shape: a CUDA graph whose launches walk over enough distinct
    copies of W to exceed L2, timed with CUDA events on the library stream (best of ``reps``); plus the warm
    (L2-resident) per-launch latency.  Algorithmic bytes = GGUF block bytes + fp32 x + fp32 y."""
    be, bb = {2: (32, 18), 12: (256, 144), 8: (32, 34), 6: (32, 22)}[t]
    wbytes = N * K // be * bb
    copies = int(min(160, max(1, np.ceil(target_bytes / wbytes))))
    rng = _gemv_weights(gpu, A, t, N, K, copies, tile)
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
    peak, _ = measured_peaks()
    kernel = "tcgen05 GEMM" if tc_path else ("CUDA-core GEMV (planes)" if t in (8, 6) else "tensor-core GEMV (tiled)" if tile else "CUDA-core GEMV")
    out = dict(type=_BLOCK_NAME[t], kernel=kernel,
               N=N, K=K, B=B, copies=copies, bytes_per_launch=int(alg), us_per_launch=round(best * 1e3 / copies, 3), GBs=round(gbs, 1),
               frac_of_measured=round(gbs / peak, 3), frac_of_8TBs=round(gbs / 8000, 3), warm_us_per_launch=round(ms2 * 1e3 / 20, 3))
    gpu.graph_destroy(gid); gpu.graph_destroy(gid2)
    for h in [a_h, c_h] + bhs:
        gpu.free_handle(h)
    gpu.map_destroy(1)
    return out


def gemv_once(gpu, A, t, N, K, B, reps, tile=True):
    rng = _gemv_weights(gpu, A, t, N, K, 1, tile)
    gpu.map_create_typed(0, A.DTYPE_F32, 1, B * K + B * N + 8)
    gpu.scatter_contiguous(0, 0, rng.standard_normal(B * K).astype(np.float32))
    a_h = gpu.upload_dev(np.array([0], np.uint32))[0]
    b_h = gpu.upload_dev(np.array([0], np.uint32))[0]
    c_h = gpu.upload_dev(np.array([B * K], np.uint32))[0]
    for _ in range(reps):
        gpu.map_matmul_t_xq4_dev(0, 1, a_h, b_h, c_h, B, K, N)
    gpu.sync()
    return gpu.device_error()


# ---- batched decode + chunked prefill on the 1B shape (config 3) -------------------------------------------

def batch_decode(args):
    import adam_b200 as A
    from adam_b200 import synth
    from adam_b200.config import gemma3_1b, with_layers
    from adam_b200.engine import ADAMEngine
    cfg = gemma3_1b()
    if args.layers:
        cfg = with_layers(cfg, args.layers)
    gpu = A.init()
    tensors = synth.build_model_cuda(gpu, cfg, seed=0)
    warmup = max(3, args.warmup)
    kv_cap = args.prompt + warmup + args.steps + 8
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=kv_cap, max_batch=args.batch, kv_dtype="f16", window=True)
    prompts = [list(map(int, synth.random_prompt(cfg.n_vocab, args.prompt, seed=10 + b))) for b in range(args.batch)]
    eng.begin(prompts, [kv_cap] * args.batch)
    gpu.batch_begin()
    gpu.timer_begin()
    if args.token_prefill:
        eng.step(args.prompt - 1, lm_head=False)
    else:
        eng.prefill(args.prompt - 1)
    pre_ms = gpu.timer_end()
    eng.step(warmup, lm_head=True)
    gpu.batch_end()
    gpu.batch_begin()
    gpu.timer_begin()
    eng.step(args.steps, lm_head=True)
    ms = gpu.timer_end()
    gpu.batch_end()
    err = gpu.device_error()
    launches = gpu.kernel_launches()
    eng.close()
    gpu.shutdown()
    w_bytes = synth.model_weight_elems(cfg) * 18 // 32
    print(json.dumps({"metric": "decode tok/s (Gemma-3-1B-shape Q4_0, batched)", "value": args.batch * args.steps / (ms * 1e-3), "unit": "tok/s",
                      "batch": args.batch, "steps": args.steps, "ms_per_step": ms / args.steps, "n_layer": cfg.n_layer, "window": True,
                      "prefill_tok_s": args.batch * (args.prompt - 1) / (pre_ms * 1e-3),
                      "prefill": "token by token, all sequences per step" if args.token_prefill else "chunks of (sequence, position) rows per pass",
                      "weight_bytes_per_step_if_read_once": int(w_bytes), "kernel_launches_total": int(launches), "device_error": int(err),
                      "data": "synthetic"}))


# ---- tensor-parallel decode on the 27B shape (config 5) ----------------------------------------------------

def _random_blocks_cuda(torch, dev, gen, rows, cols, ggml_type):
    """Seeded random GGUF blocks on the device: uniform quant/scale bytes, fp16 ``d`` (and ``dmin``) set to small
    positive values so every decoded weight is finite and of the usual magnitude."""
    from adam_b200 import gguf_blocks as gb
    from adam_b200.synth import QTensor
    from adam_b200.tp import block_bytes, block_elems
    be, bb = block_elems(ggml_type), block_bytes(ggml_type)
    n = rows * cols // be
    raw = torch.randint(0, 256, (n, bb), dtype=torch.uint8, device=dev, generator=gen)
    d = (torch.rand(n, device=dev, generator=gen) * 0.002 + 0.001).to(torch.float16).view(torch.uint8).view(n, 2)
    raw[:, 0:2] = d
    if ggml_type == gb.GGML_TYPE_Q4_K:
        raw[:, 0:2] = (d.view(torch.float16).view(n) / 32).to(torch.float16).view(torch.uint8).view(n, 2)   # d * 6-bit scale
        raw[:, 2:4] = raw[:, 0:2]
    return QTensor(ggml_type, rows, cols, raw.reshape(-1))


def _build_shard(torch, gpu, cfg, plan, ggml_type, seed):
    from adam_b200.synth import LAYER_MATS, LAYER_NORMS, QTensor, mat_shapes
    from adam_b200.tp import block_bytes, block_elems, local_config
    dev = torch.device("cuda", gpu.device_index)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    rng = np.random.default_rng(seed)
    lc = local_config(cfg, plan)
    shapes = mat_shapes(lc)
    shapes["attn_output"] = (cfg.n_embd, lc.n_head * lc.head_dim)     # K of the row-parallel matrices is local
    shapes["ffn_down"] = (cfg.n_embd, lc.n_ff)
    t = {}
    embd = _random_blocks_cuda(torch, dev, gen, cfg.n_vocab, cfg.n_embd, ggml_type)
    t["token_embd.weight"] = embd
    bpr = cfg.n_embd // block_elems(ggml_type) * block_bytes(ggml_type)
    t["output.weight"] = QTensor(ggml_type, len(plan.vocab), cfg.n_embd,
                                 embd.raw.view(cfg.n_vocab, bpr)[plan.vocab.start:plan.vocab.stop].contiguous().reshape(-1))

    def norm(n):
        return (np.float32(1) + np.float32(0.1) * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)

    t["output_norm.weight"] = norm(cfg.n_embd)
    for L in range(cfg.n_layer):
        p = f"blk.{L}"
        for n in LAYER_NORMS:
            t[f"{p}.{n}.weight"] = norm(cfg.n_embd)
        t[f"{p}.attn_q_norm.weight"] = norm(cfg.head_dim)
        t[f"{p}.attn_k_norm.weight"] = norm(cfg.head_dim_kv)
        for n in LAYER_MATS:
            t[f"{p}.{n}.weight"] = _random_blocks_cuda(torch, dev, gen, *shapes[n], ggml_type)
    return t


def tp_decode(gpu, rank, world, steps=32, warmup=4, layers=0, batch=1, prompt=16, ggml_type=12, token_prefill=False,
              use_graph=True, allreduce="p2p", shard_of=0):
    """Gemma-3-27B-shaped decode, tensor parallel over ``world`` ranks (one per GPU; an initialised NCCL process
    group when world > 1).  Every rank fills its own shard with seeded random GGUF blocks, consumes a short prompt,
    then ``steps`` decode steps are timed with CUDA events on the stream the step runs on; time = max over ranks.
    Returns the result dict on every rank."""
    import torch
    import torch.distributed as dist
    from adam_b200.config import gemma3_27b, with_layers
    from adam_b200.tp import ADAMEngineTP, block_bytes, block_elems, shard_plan
    cfg = gemma3_27b()
    if layers:
        cfg = with_layers(cfg, layers)
    tp_world = shard_of if (shard_of and world == 1) else world
    plan = shard_plan(cfg, rank, tp_world, ggml_type)
    tensors = _build_shard(torch, gpu, cfg, plan, ggml_type, seed=100 + rank)
    warmup = max(3, warmup)
    kv_cap = prompt + warmup + steps + 8
    eng = ADAMEngineTP(gpu, cfg, tensors, rank, tp_world, presharded=True, use_graph=use_graph, collectives=(tp_world == world),
                       allreduce=allreduce, kv_cap=kv_cap, max_batch=batch, kv_dtype="f16", window=True)
    del tensors
    prompts = [list(map(int, np.random.default_rng(b).integers(0, cfg.n_vocab, prompt))) for b in range(batch)]
    eng.begin(prompts, [kv_cap] * batch)
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.batch_begin()
    with torch.cuda.stream(eng._stream):
        pe0.record()
    eng.prefill(prompt - 1, chunked=not token_prefill)
    with torch.cuda.stream(eng._stream):
        pe1.record()
    eng.step(warmup, lm_head=True)
    gpu.batch_end()
    pe1.synchronize()
    pre_ms = pe0.elapsed_time(pe1)
    if world > 1:
        dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.batch_begin()
    with torch.cuda.stream(eng._stream):
        ev0.record()
    eng.step(steps, lm_head=True)
    with torch.cuda.stream(eng._stream):
        ev1.record()
    gpu.batch_end()
    ev1.synchronize()
    ms = ev0.elapsed_time(ev1)
    ids = eng.read_log(0, prompt + warmup, steps)
    ids_equal = True
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        mine = torch.from_numpy(np.asarray(ids, np.int64)).cuda()
        allids = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(allids, mine)
        ids_equal = all(bool(torch.equal(allids[0], x)) for x in allids)
    err = gpu.device_error()
    lc = eng.cfg
    w_elems = lc.n_layer * ((lc.n_head + 2 * lc.n_head_kv) * lc.head_dim * cfg.n_embd + cfg.n_embd * lc.n_head * lc.head_dim
                            + 3 * lc.n_ff * cfg.n_embd) + lc.n_vocab * cfg.n_embd
    w_bytes = w_elems * block_bytes(ggml_type) // block_elems(ggml_type)
    graph_used = bool(eng._graphs)
    ar_used = eng._ar is not None
    eng.close()
    ms_tok = ms / steps
    n_coll = 2 * cfg.n_layer + 2 if world > 1 else 0
    return {"metric": "decode tok/s (Gemma-3-27B-shape, tensor parallel)", "value": batch * steps / (ms * 1e-3), "unit": "tok/s",
            "n_gpus": world, "steps": steps, "ms_per_token": ms_tok, "batch": batch, "n_layer": cfg.n_layer,
            "weights": "Q4_K random blocks" if ggml_type == 12 else "Q4_0 random blocks",
            "parallelism": f"tp{tp_world}" + ("" if tp_world == world else " (one shard, no collectives)"),
            "weight_bytes_per_rank_per_token": int(w_bytes), "GBs_per_gpu": w_bytes / (ms_tok * 1e-3) / 1e9,
            "prefill_tok_s": batch * (prompt - 1) / (pre_ms * 1e-3) if prompt > 1 else None,
            "collectives_per_token": n_coll, "collective": (("peer-memory one-shot all-reduce (library kernel)" if ar_used else "NCCL all-reduce") + " x %d + arg-max all-gather" % (2 * cfg.n_layer)) if world > 1 else None,
            "graph": graph_used, "ids_equal_across_ranks": ids_equal, "device_error": int(err)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="adam_b200", choices=["adam_b200", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug: truncate the model depth (invalid as a benchmark number)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="skip the GEMV sweep of the default mode")
    ap.add_argument("--no-tp", action="store_true", help="skip the 27B-shape tensor-parallel decode of the default mode")
    ap.add_argument("--mode", default="decode", choices=["decode", "gemv", "gemv-once", "batch", "tp", "token-once", "token-trace", "step-trace"])
    ap.add_argument("--type", type=int, default=0, help="gemv / tp modes: GGML block type (2 = Q4_0, 12 = Q4_K)")
    ap.add_argument("--n", type=int, default=0)
    ap.add_argument("--k", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0)
    ap.add_argument("--prompt", type=int, default=0)
    ap.add_argument("--reps", type=int, default=4)
    ap.add_argument("--no-tile", action="store_true", help="gemv modes: CUDA-core kernel over plain GGUF blocks")
    ap.add_argument("--token-prefill", action="store_true", help="batch / tp modes: consume the prompt one position per step")
    ap.add_argument("--allreduce", default="p2p", choices=["p2p", "nccl"], help="tp mode: library peer-memory all-reduce or NCCL")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--shape", default="1b", choices=["1b", "27b"], help="step-trace mode: model shape (27b: Q4_0 blocks, give --layers)")
    ap.add_argument("--chain", action="store_true", help="token-once mode: the CUDA graph of per-operation kernels instead of the token kernel")
    ap.add_argument("--shard-of", type=int, default=0, help="tp mode, one process: rank 0's shard of an N-way split without collectives")
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    if args.mode in ("gemv", "gemv-once", "batch", "token-once", "token-trace", "step-trace"):
        return other_modes(args)
    if args.gpus > 1 and world == 1:
        # not under torchrun: relaunch one rank per GPU on this node
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(29500 + os.getpid() % 1000), os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)
    if args.mode == "tp":
        import torch
        torch.cuda.set_device(local_rank)
        if world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        os.environ.setdefault("ADAM_B200_DEVICE", str(local_rank))
        import adam_b200 as A
        gpu = A.init()
        res = tp_decode(gpu, rank, world, steps=steps, warmup=warmup, layers=args.layers, batch=args.batch or 1, prompt=args.prompt or 16,
                        ggml_type=args.type or 12, token_prefill=args.token_prefill, use_graph=not args.no_graph, allreduce=args.allreduce,
                        shard_of=args.shard_of)
        gpu.shutdown()
        if rank == 0:
            print(json.dumps(res))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    from adam_b200.config import gemma3_1b, with_layers
    cfg = gemma3_1b()
    if args.layers:
        cfg = with_layers(cfg, args.layers)
    workload = {"workload": "gemma3-1b-shape Q4_0 decode, batch 1, 128-token prompt, greedy", "n_layer": cfg.n_layer,
                "prompt_len": PROMPT_LEN, "kv": "fp16 paged", "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
                "l2": "each step streams 562 MB of weights (> 126 MB L2)"}

    if args.impl == "reference":
        # The reference's GPU path is Vulkan and cannot run on this box; its CPU path
        # (numpy decoder) is timed on the host cores.  Rank 0 only.
        if rank != 0:
            return
        from adam_b200 import gguf_blocks as gb
        from adam_b200 import synth
        # Seeded N(0, 0.02) weights quantized to Q4_0 on the host (numpy): this arm loads no CUDA library.
        tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=0)
        prompt = synth.random_prompt(cfg.n_vocab, PROMPT_LEN, seed=1)
        n_dec = min(steps, 128)
        tps, dt, t_prompt, _ = cpu_decode_sample(cfg, tensors, prompt, n_dec)
        cores = threads_used()
        sample = (f"full {cfg.n_layer}-layer model, {PROMPT_LEN}-token prompt consumed token by token ({t_prompt:.1f} s, untimed), then {n_dec} greedy "
                  f"tokens timed ({dt:.1f} s; --steps {steps}); numpy restatement of the reference's CPU decoder on float32 weights decoded from Q4_0")
        print(json.dumps({"impl": "reference", "metric": "decode tok/s (Gemma-3-1B-shape Q4, b=1)", "value": tps, "unit": "tok/s",
                          "n_gpus": world, "steps": n_dec, "warmup": 0, "ms_per_step": 1000.0 / tps, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload,
                          "cpu_baseline": {"value": tps, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
                          "e2e": {"value": tps, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import adam_b200 as A
    from adam_b200 import synth
    from adam_b200.config import GenerationConfig
    from adam_b200.engine import ADAMEngine

    os.environ.setdefault("ADAM_B200_DEVICE", str(local_rank))
    gpu = A.init()
    t_build = time.perf_counter()
    tensors = synth.build_model_cuda(gpu, cfg, seed=0)
    torch.cuda.synchronize()
    kv_cap = PROMPT_LEN + warmup + steps + 8
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=kv_cap, kv_dtype="f16", window=True)
    t_build = time.perf_counter() - t_build
    prompt = synth.random_prompt(cfg.n_vocab, PROMPT_LEN, seed=1)

    def barrier():
        gpu.sync()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    # ---- device-resident number: prefill, W warm-up tokens, K timed tokens -----------------
    eng.begin([prompt], [kv_cap - 4])
    gpu.batch_begin()
    t0 = time.perf_counter()
    eng.prefill(PROMPT_LEN - 1)              # 64 prompt positions per pass through the layers
    gpu.batch_end()
    prefill_s = time.perf_counter() - t0
    gpu.batch_begin(); eng.step(warmup, lm_head=True); gpu.batch_end()
    barrier()
    gpu.reset_native_stats()
    with ClockSampler(local_rank) as clk:
        gpu.batch_begin()
        gpu.timer_begin()
        eng.step(steps, lm_head=True)
        ms = gpu.timer_end()
        gpu.batch_end()
    barrier()
    launches = gpu.get_native_stats()["dispatch_count"]
    tokens_kernel = eng.read_log(0, PROMPT_LEN + warmup, steps)
    # the other way to run a one-sequence step, for the record: every token as one launch of the persistent token kernel
    other = None
    if world == 1:
        eng.begin([prompt], [kv_cap - 4])
        gpu.batch_begin(); eng.prefill(PROMPT_LEN - 1); eng.step(warmup, lm_head=True, chain=eng.single_launch); gpu.batch_end()
        gpu.reset_native_stats()
        gpu.batch_begin(); gpu.timer_begin(); eng.step(steps, lm_head=True, chain=eng.single_launch); ms_o = gpu.timer_end(); gpu.batch_end()
        other = {"path": "CUDA graph of per-operation kernels" if eng.single_launch else "single-launch token kernel (k_token)",
                 "ms_per_step": ms_o / steps, "tok_s": steps / (ms_o * 1e-3), "gpu_launches": int(gpu.get_native_stats()["dispatch_count"]),
                 "ids_equal": [int(t) for t in eng.read_log(0, PROMPT_LEN + warmup, steps)] == [int(t) for t in tokens_kernel]}

    # ---- end to end through the public API: host prompt in, one token read back per step ----
    gen_cfg = GenerationConfig(max_tokens=warmup + steps, top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=())
    eng.generate(prompt, GenerationConfig(max_tokens=4, top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=()))      # warm
    barrier()
    out, st = eng.generate(prompt, gen_cfg, sync_every=1)
    barrier()
    # the timed region of this figure starts before the prompt's host->device copy (begin) and ends after the
    # last token id has been read back: prompt copy, chunked prefill, every decode step and its 4-byte read
    e2e_tps = st["n_gen"] / st["total_s"]
    same_ids = [int(t) for t in tokens_kernel] == out[warmup:warmup + steps]

    # ---- dominant kernel: the dequant GEMV on the LM-head shape, alone on the stream --------
    hbm_peak, peak_kind = measured_peaks()
    m_embd = eng._mat_loc["token_embd.weight"]
    N, K = m_embd[2], m_embd[3]
    gpu.map_create_typed(200, A.DTYPE_F32, 1, K + 64)
    gpu.scatter_contiguous(200, 0, np.random.default_rng(2).standard_normal(K).astype(np.float32))
    a_h = gpu.upload_dev(np.array([0], np.uint32))[0]; b_h = gpu.upload_dev(np.array([m_embd[1]], np.uint32))[0]
    d_h = gpu.upload_dev(np.array([K + 8], np.uint32))[0]; t_h = gpu.upload_dev(np.zeros(4, np.uint32))[0]
    reps = 20
    gpu.capture_begin()
    for _ in range(reps):
        gpu.map_matvec_argmax_t_xq4_dev(200, m_embd[0], a_h, b_h, t_h, t_h, d_h, K, N, 256)
    gid = gpu.capture_end()
    gpu.graph_launch(gid, 2)
    best = 1e30
    for _ in range(5):
        gpu.batch_begin(); gpu.timer_begin(); gpu.graph_launch(gid, 1); kms = gpu.timer_end(); gpu.batch_end()
        best = min(best, kms)
    gemv_bytes = N * K * 18 // 32 + 4 * K + 4
    gemv_gbs = gemv_bytes / (best / reps * 1e-3) / 1e9
    step_bytes = synth.model_weight_elems(cfg) * 18 // 32
    # what one decoded token reads besides the weight blocks: the float32 norm vectors, and per layer the cached keys
    # and values of the positions it attends to (fp16; the sliding window on the local layers) plus the row it appends
    norm_bytes = 4 * (cfg.n_embd * (4 * cfg.n_layer + 1) + 2 * cfg.head_dim * cfg.n_layer)
    ctx_mean = PROMPT_LEN + warmup + steps / 2.0
    kv_row = 2 * cfg.n_head_kv * cfg.head_dim * 2
    kv_bytes = sum(kv_row * (min(ctx_mean, cfg.sliding_window) if (cfg.sliding_window and not cfg.is_global(L)) else ctx_mean) + kv_row
                   for L in range(cfg.n_layer))
    token_bytes = int(step_bytes + norm_bytes + kv_bytes)
    token_kernel = launches == steps          # one launch per token: the single-launch kernel ran (else the chain of per-operation kernels)

    # ---- the other GEMV shapes of the benchmark configurations (rank 0 of a single-GPU run) ---------
    sweep = None
    if world == 1 and not args.no_sweep and not args.layers:
        eng.close()
        sweep = [gemv_shape(gpu, A, *sh, target_bytes=300e6, reps=3) for sh in GEMV_SWEEP]
        eng = None

    # ---- the 27B shape, tensor parallel over the GPUs of this run --------------------------------------
    tp = None
    if not args.no_tp and not args.layers:
        if eng is not None:
            eng.close()
            eng = None
        tp = tp_decode(gpu, rank, world, steps=min(steps, 32), warmup=3)

    # ---- reduce over ranks -------------------------------------------------------------------
    from adam_b200.replicas import combine_timings
    comb = combine_timings(ms, steps, e2e_tps, world, device="cuda")     # a collective when world > 1
    ms, value = comb["ms"], comb["value"]

    line = None
    if rank == 0:
        cpu = None
        ids_equal_oracle = None
        if not args.no_cpu_baseline and world == 1:
            n_dec = min(len(out), 128)
            tps, dt, t_prompt, cpu_ids = cpu_decode_sample(cfg, tensors, prompt, n_dec)
            ids_equal_oracle = (cpu_ids == out[:n_dec])
            cpu = {"value": tps, "unit": "tok/s", "cores": threads_used(), "kind": "port",
                   "sample": f"full {cfg.n_layer}-layer model, same weights and {PROMPT_LEN}-token prompt as the GPU arm ({t_prompt:.1f} s, untimed), "
                             f"then {n_dec} greedy tokens timed ({dt:.1f} s); numpy restatement of the reference CPU decoder on float32 weights decoded from Q4_0"}
        line = {
            "metric": "decode tok/s (Gemma-3-1B-shape Q4, b=1)", "value": value, "unit": "tok/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 accumulate; weights int4 blocks; GEMV activations rounded to 23-bit block fixed point", "data": "synthetic", "config": workload,
            "e2e": {"value": comb["e2e"], "unit": "tok/s", "h2d_bytes_per_step": st["h2d_bytes"] / max(1, st["n_gen"]),
                    "d2h_bytes_per_step": st["d2h_bytes"] / max(1, st["n_gen"]), "ids_equal_device_run": same_ids,
                    "timed_region": "ADAMEngine.generate from the prompt's host-to-device copy to the last token read: "
                                    "prompt copy + chunked prefill + every decode step with its 4-byte token read",
                    "decode_only_tok_s": st["decode_tps"]},
            "ids_equal_oracle": ids_equal_oracle, "ids_compared": (len(cpu_ids) if cpu else 0),
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": token_bytes / (ms / steps * 1e-3) / 1e9, "peak": hbm_peak, "unit": "GB/s",
                         "frac": token_bytes / (ms / steps * 1e-3) / 1e9 / hbm_peak, "traffic": TOKEN_DRAM_TRAFFIC if token_kernel else CHAIN_DRAM_TRAFFIC,
                         "kernel": ("k_token<Q4_0, fp16 KV, head 256> (one launch per token: every layer, LM head, arg-max)" if token_kernel
                                    else "all %d kernels of a token step together (CUDA graph: 105 k_gemv_mma, 26 k_attention, embed, advance); "
                                         "the largest single kernel is under lm_head_gemv" % (launches // max(1, steps))),
                         "bytes_per_step": token_bytes, "us_per_step": ms / steps * 1e3,
                         "launches_in_timed_region": int(launches), "peak_kind": peak_kind,
                         "frac_of_8TBs": token_bytes / (ms / steps * 1e-3) / 1e9 / 8000.0,
                         "note": "latency-bound: 26 layers x 5 dependent kernels (or hand-overs between SMs inside the single launch); the bytes stream at this rate only on average"},
            "lm_head_gemv": {"bound": "hbm", "achieved": gemv_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gemv_gbs / hbm_peak,
                             "traffic": LMHEAD_DRAM_TRAFFIC, "kernel": "k_gemv_mma<4,false> (LM head %dx%d Q4_0 + arg-max, tensor-core path), alone on the stream" % (N, K),
                             "bytes_per_launch": gemv_bytes, "us_per_launch": best / reps * 1e3, "frac_of_8TBs": gemv_gbs / 8000.0},
            "step_hbm": {"bytes_per_step": step_bytes, "achieved_GBs": step_bytes / (ms / steps * 1e-3) / 1e9,
                         "frac": step_bytes / (ms / steps * 1e-3) / 1e9 / hbm_peak},
            "clocks": clk.summary(), "prefill_tok_s": (PROMPT_LEN - 1) / prefill_s, "build_s": t_build,
        }
        if other is not None:
            line["other_step_path"] = other
        if sweep is not None:
            line["gemv_sweep"] = sweep
        if tp is not None:
            line["tp"] = tp
        if cpu:
            line["cpu_baseline"] = cpu
    if eng is not None:
        eng.close()
    gpu.shutdown()
    if world > 1:
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line))


def token_trace(gpu, args):
    """Where the time of one token-kernel launch goes: every CTA stamps its SM clock at the phase boundaries of one
    layer and of the LM head (``adam_b200_decoder_token_trace``); the figures are means over the CTAs that take part,
    in microseconds at the SM clock read beside them, plus the launch time with and without the single-launch kernel."""
    from adam_b200 import synth
    from adam_b200.config import gemma3_1b, with_layers
    from adam_b200.engine import ADAMEngine
    cfg = gemma3_1b()
    if args.layers:
        cfg = with_layers(cfg, args.layers)
    tensors = synth.build_model_cuda(gpu, cfg, seed=0)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=PROMPT_LEN + 200, kv_dtype="f16", window=True)
    eng.begin([synth.random_prompt(cfg.n_vocab, PROMPT_LEN, seed=1)], [PROMPT_LEN + 190])
    gpu.batch_begin(); eng.prefill(PROMPT_LEN - 1); eng.step(8, lm_head=True); gpu.batch_end()
    try:
        mhz = float(subprocess.run(["nvidia-smi", "--query-gpu=clocks.sm", "--format=csv,noheader,nounits", "-i", "0"], capture_output=True, text=True).stdout.split()[0])
    except Exception:
        mhz = 1965.0
    names = ["", "residual update + input norm", "QKV product", "attention (QK-norm, RoPE, append, soft-max, PV)", "o-proj input staged", "o-proj product",
             "residual update + post-attention / FFN norms", "gate/up product + GeGLU", "down-proj input staged", "down-proj product",
             "", "final norm chain", "LM head product + arg-max", "finish"]
    layer = min(5, cfg.n_layer - 1)
    eng.token_trace(layer=layer)
    tr = eng.token_trace(layer=layer).astype(np.float64)
    phases = {}
    for i in list(range(1, 10)) + [11, 12, 13]:
        ok = (tr[:, i] > 0) & (tr[:, i - 1] > 0)
        if ok.any():
            d = (tr[ok, i] - tr[ok, i - 1]) / mhz
            phases[names[i]] = {"mean_us": round(float(d.mean()), 2), "max_us": round(float(d.max()), 2), "ctas": int(ok.sum())}
    ok = (tr[:, 9] > 0) & (tr[:, 0] > 0)
    layer_us = float(((tr[ok, 9] - tr[ok, 0]) / mhz).mean()) if ok.any() else None
    out = {"n_cta": int(tr.shape[0]), "traced_layer": layer, "sm_mhz": mhz, "layer_us": layer_us, "phases": phases}
    for chain in (False, True):
        gpu.batch_begin(); eng.step(8, lm_head=True, chain=chain); gpu.batch_end()
        gpu.batch_begin(); gpu.timer_begin(); eng.step(64, lm_head=True, chain=chain); ms = gpu.timer_end(); gpu.batch_end()
        out["ms_per_token_chain_of_kernels" if chain else "ms_per_token_single_launch"] = ms / 64
    out["device_error"] = gpu.device_error()
    eng.close()
    return out


def step_trace(gpu, args):
    """Where the time of one layer goes in the default one-sequence step (CUDA graph of per-operation kernels): the four
    products and the attention launch of one layer stamp the GPU's nanosecond timer at their phase boundaries
    (``adam_b200_decoder_step_trace``; needs the diagnostics library, see the module docstring).  The stamps are those of
    the last of ``--steps`` back-to-back steps, so clocks and caches are those of the benchmark's timed loop."""
    from adam_b200 import synth
    from adam_b200.config import gemma3_1b, with_layers
    from adam_b200.engine import ADAMEngine
    from adam_b200.config import gemma3_27b
    cfg = gemma3_27b() if args.shape == "27b" else gemma3_1b()
    if args.layers:
        cfg = with_layers(cfg, args.layers)
    steps = max(args.steps, 64)
    tensors = synth.build_model_cuda(gpu, cfg, seed=0)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=PROMPT_LEN + steps + 32, kv_dtype="f16", window=True)
    eng.begin([synth.random_prompt(cfg.n_vocab, PROMPT_LEN, seed=1)], [PROMPT_LEN + steps + 24])
    layer = min(5, cfg.n_layer - 1)
    eng.step_trace(layer)
    gpu.batch_begin(); eng.prefill(PROMPT_LEN - 1); eng.step(8, lm_head=True); gpu.batch_end()
    gpu.batch_begin(); gpu.timer_begin(); eng.step(steps, lm_head=True); ms = gpu.timer_end(); gpu.batch_end()
    prod, att = eng.step_trace()
    t0 = int(prod[0, 0, 2])                     # the moment the layer's first kernel may read its input
    names = ["qkv", "o_proj", "gate_up", "down"]
    out = {"shape": args.shape, "n_layer": cfg.n_layer, "traced_layer": layer, "context": PROMPT_LEN + 8 + steps, "ms_per_token": ms / steps, "unit": "us since the QKV kernel's dependency wait ended (CTA 0)", "kernels": {}}
    for k, nm in enumerate(names):
        r = prod[k, 0].astype(np.int64)
        out["kernels"][nm] = {"started": (r[0] - t0) / 1e3, "prologue_done": (r[1] - t0) / 1e3, "wait_over": (r[2] - t0) / 1e3,
                              "input_staged": (r[3] - t0) / 1e3, "products_done": (r[4] - t0) / 1e3}
        if r[5] > 0:        # inside the staging: norm chain -- branch RMS known, stream RMS and maximum known; long plain vector -- bulk copy landed, maximum known
            out["kernels"][nm].update({"staging_mark_1": (r[5] - t0) / 1e3, "staging_mark_2": (r[6] - t0) / 1e3})
    live = att[(att[:, 4] > 0)]
    if len(live):
        last = att[att[:, 7] > 0]
        out["kernels"]["attention"] = {
            "ctas_with_positions": int(len(live)), "started": float((live[:, 0].min() - t0) / 1e3), "rows_requested": float((live[:, 1].max() - t0) / 1e3),
            "wait_over": float((live[:, 2].max() - t0) / 1e3), "rows_normed_rotated": float((live[:, 3].max() - t0) / 1e3),
            "positions_done": float((live[:, 4].max() - t0) / 1e3), "partial_stored": float((live[:, 5].max() - t0) / 1e3) if (live[:, 5] > 0).any() else None,
            "ticket_taken": float((live[:, 6].max() - t0) / 1e3) if (live[:, 6] > 0).any() else None,
            "splits_merged": float((last[:, 7].max() - t0) / 1e3) if len(last) else None}
    out["device_error"] = gpu.device_error()
    eng.close()
    return out


def other_modes(args):
    """Single-GPU modes besides the decode benchmark (see the module docstring)."""
    if args.mode == "batch":
        args.batch = args.batch or 32
        args.prompt = args.prompt or 64
        return batch_decode(args)
    import adam_b200 as A
    gpu = A.init()
    try:
        if args.mode == "gemv-once":
            err = gemv_once(gpu, A, args.type or 2, args.n or 262144, args.k or 1152, args.batch or 1, args.reps, not args.no_tile)
            print(json.dumps({"ok": err == 0}))
        elif args.mode == "gemv":
            shapes = [(args.type, args.n, args.k, args.batch or 1)] if args.type and args.n and args.k else GEMV_SWEEP
            for sh in shapes:
                print(json.dumps(gemv_shape(gpu, A, *sh, tile=not args.no_tile)), flush=True)
        elif args.mode == "token-trace":
            print(json.dumps(token_trace(gpu, args)))
        elif args.mode == "step-trace":
            print(json.dumps(step_trace(gpu, args)))
        else:       # token-once: prompt, then a few single-launch token steps
            from adam_b200 import synth
            from adam_b200.config import gemma3_1b, with_layers
            from adam_b200.engine import ADAMEngine
            cfg = gemma3_1b()
            if args.layers:
                cfg = with_layers(cfg, args.layers)
            tensors = synth.build_model_cuda(gpu, cfg, seed=0)
            eng = ADAMEngine(gpu, cfg, tensors, kv_cap=PROMPT_LEN + 64, kv_dtype="f16", window=True, single_launch=not args.chain)
            eng.begin([synth.random_prompt(cfg.n_vocab, PROMPT_LEN, seed=1)], [PROMPT_LEN + 60])
            gpu.batch_begin(); eng.prefill(PROMPT_LEN - 1); eng.step(max(1, min(args.steps, 32)), lm_head=True); gpu.batch_end()
            print(json.dumps({"ok": gpu.device_error() == 0}))
            eng.close()
    finally:
        gpu.shutdown()


if __name__ == "__main__":
    main()
