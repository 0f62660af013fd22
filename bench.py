#!/usr/bin/env python3
"""Decode benchmark for the Gemma-3-1B-shaped Q4_0 model (batch 1, 128-token
random prompt, greedy decode): one "step" is one decoded token.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Prints ONE JSON line.  ``value`` is decode tok/s with everything resident in HBM
(K graph replays timed with CUDA events on the library's stream); ``e2e`` is the
same metric through ``ADAMEngine.generate`` with host prompt ids: generated tokens divided by
the whole call's time, i.e. the host->device prompt copy, the chunked prefill, every decode step
and one device->host token read per step are all inside the timed region.
``roofline`` is the dominant kernel (the dequant GEMV, measured on the LM-head
shape, 262144 x 1152 Q4_0, whose 170 MB exceed L2) against the measured HBM copy
bandwidth.  ``cpu_baseline`` is the numpy restatement of the reference's CPU decoder
timed on this box's host cores on a bounded sample (same weights, same prompt); its greedy ids
are compared with the GPU arm's (``ids_equal_oracle``).  With N > 1 (torchrun, one
rank per GPU) every rank runs an independent replica: no collective on the data
path, weak scaling, value = all ranks' tokens / slowest rank's time.
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
# dram__bytes_read.sum + dram__bytes_write.sum of one LM-head GEMV launch, from the ncu capture
# summarised in profiles/gemv_mma_q4_0_lmhead_262144x1152.md (same kernel and shape; that capture's
# entry point also stores the 1 MB of logits)
LMHEAD_DRAM_TRAFFIC = 169_949_184 + 4_576_256


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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="adam_b200", choices=["adam_b200", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="debug: truncate the model depth (invalid as a benchmark number)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank, local_rank, world = dist_env()
    if args.gpus > 1 and world == 1:
        # not under torchrun: relaunch one rank per GPU on this node
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}", "--master-addr", "127.0.0.1",
               "--master-port", str(29500 + os.getpid() % 1000), os.path.abspath(__file__)] + sys.argv[1:]
        sys.exit(subprocess.call(cmd))
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

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
            "roofline": {"bound": "hbm", "achieved": gemv_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": gemv_gbs / hbm_peak,
                         "traffic": LMHEAD_DRAM_TRAFFIC, "kernel": "k_gemv_mma<4,false> (LM head %dx%d Q4_0 + arg-max, tensor-core path)" % (N, K),
                         "bytes_per_launch": gemv_bytes, "us_per_launch": best / reps * 1e3, "peak_kind": peak_kind,
                         "frac_of_8TBs": gemv_gbs / 8000.0},
            "step_hbm": {"bytes_per_step": step_bytes, "achieved_GBs": step_bytes / (ms / steps * 1e-3) / 1e9,
                         "frac": step_bytes / (ms / steps * 1e-3) / 1e9 / hbm_peak},
            "clocks": clk.summary(), "prefill_tok_s": (PROMPT_LEN - 1) / prefill_s, "build_s": t_build,
        }
        if cpu:
            line["cpu_baseline"] = cpu
    eng.close()
    gpu.shutdown()
    if world > 1:
        dist.destroy_process_group()
    if line is not None:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
