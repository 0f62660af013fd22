"""Batched decode benchmark on the 1B shape (Q4_0): B independent sequences step together.

    python -m adam_b200.batch_bench --batch 32 --prompt 64 --steps 64

Seeded synthetic weights generated on the GPU, random prompt ids; the prompt is consumed token by
token (one step advances all sequences), then K decode steps are timed with the library's CUDA-event
timer around the graph replays.  Prints one JSON line: aggregate tokens/s, ms per step, and the
weight bytes a step streams if every batch row re-reads them (what the current kernels do: the GEMV
takes four batch rows per pass over the weights).
"""
from __future__ import annotations

import argparse
import json

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--prompt", type=int, default=64)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--token-prefill", action="store_true", help="consume the prompt one position per step instead of in 64-row chunks")
    a = ap.parse_args()
    import adam_b200 as A
    from adam_b200 import synth
    from adam_b200.config import gemma3_1b, with_layers
    from adam_b200.engine import ADAMEngine
    cfg = gemma3_1b()
    if a.layers:
        cfg = with_layers(cfg, a.layers)
    gpu = A.init()
    tensors = synth.build_model_cuda(gpu, cfg, seed=0)
    kv_cap = a.prompt + a.warmup + a.steps + 8
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=kv_cap, max_batch=a.batch, kv_dtype="f16")
    prompts = [list(map(int, synth.random_prompt(cfg.n_vocab, a.prompt, seed=10 + b))) for b in range(a.batch)]
    eng.begin(prompts, [kv_cap] * a.batch)
    gpu.batch_begin()
    gpu.timer_begin()
    if a.token_prefill:
        eng.step(a.prompt - 1, lm_head=False)
    else:
        eng.prefill(a.prompt - 1)
    pre_ms = gpu.timer_end()
    eng.step(max(3, a.warmup), lm_head=True)
    gpu.batch_end()
    gpu.batch_begin()
    gpu.timer_begin()
    eng.step(a.steps, lm_head=True)
    ms = gpu.timer_end()
    gpu.batch_end()
    err = gpu.device_error()
    launches = gpu.kernel_launches()
    eng.close()
    gpu.shutdown()
    w_bytes = synth.model_weight_elems(cfg) * 18 // 32
    print(json.dumps({"metric": "decode tok/s (Gemma-3-1B-shape Q4_0, batched)", "value": a.batch * a.steps / (ms * 1e-3), "unit": "tok/s",
                      "batch": a.batch, "steps": a.steps, "ms_per_step": ms / a.steps, "n_layer": cfg.n_layer,
                      "prefill_tok_s": a.batch * (a.prompt - 1) / (pre_ms * 1e-3), "prefill": "token by token, all sequences per step" if a.token_prefill else "64 rows (sequences x positions) per pass",
                      "weight_bytes_per_step_if_read_once": int(w_bytes), "passes_over_weights_per_step": (a.batch + 3) // 4,
                      "kernel_launches_total": int(launches), "device_error": int(err), "data": "synthetic"}))


if __name__ == "__main__":
    main()
