"""Tensor-parallel decode benchmark on the 27B shape (Q4_K), one rank per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P -m adam_b200.tp_bench --steps 32 [--layers L] [--batch B] [--type 12|2]
    python -m adam_b200.tp_bench --steps 32            # one GPU, the same part-wise path without collectives

Every rank fills its own shard with seeded random GGUF blocks on its GPU (valid scales, uniform
quants: no model file), consumes a short prompt, then K decode steps are timed with CUDA events
on the stream the step runs on; the time is the maximum over ranks.  Rank 0 prints one JSON line:
tokens/s, ms per token, the weight bytes each rank streams per token and the GB/s that is.
"""
from __future__ import annotations

import argparse
import json
import os

import numpy as np

from . import gguf_blocks as gb
from .config import GenerationConfig, gemma3_27b, with_layers
from .replicas import dist_env
from .synth import LAYER_MATS, LAYER_NORMS, QTensor, mat_shapes
from .tp import ADAMEngineTP, block_bytes, block_elems, local_config, shard_plan


def random_blocks_cuda(torch, dev, gen, rows: int, cols: int, ggml_type: int) -> QTensor:
    """Seeded random GGUF blocks on the device: uniform quant/scale bytes, fp16 ``d`` (and ``dmin``)
    set to small positive values so every decoded weight is finite and of the usual magnitude."""
    be, bb = block_elems(ggml_type), block_bytes(ggml_type)
    n = rows * cols // be
    raw = torch.randint(0, 256, (n, bb), dtype=torch.uint8, device=dev, generator=gen)
    d = (torch.rand(n, device=dev, generator=gen) * 0.002 + 0.001).to(torch.float16).view(torch.uint8).view(n, 2)
    raw[:, 0:2] = d
    if ggml_type == gb.GGML_TYPE_Q4_K:
        raw[:, 0:2] = (d.view(torch.float16).view(n) / 32).to(torch.float16).view(torch.uint8).view(n, 2)   # d * 6-bit scale
        raw[:, 2:4] = raw[:, 0:2]
    return QTensor(ggml_type, rows, cols, raw.reshape(-1))


def build_shard(torch, gpu, cfg, plan, ggml_type: int, seed: int):
    dev = torch.device("cuda", gpu.device_index)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    rng = np.random.default_rng(seed)
    lc = local_config(cfg, plan)
    shapes = mat_shapes(lc)
    # K of the row-parallel matrices is local, their output width is the whole n_embd
    shapes["attn_output"] = (cfg.n_embd, lc.n_head * lc.head_dim)
    shapes["ffn_down"] = (cfg.n_embd, lc.n_ff)
    t = {}
    embd = random_blocks_cuda(torch, dev, gen, cfg.n_vocab, cfg.n_embd, ggml_type)
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
            t[f"{p}.{n}.weight"] = random_blocks_cuda(torch, dev, gen, *shapes[n], ggml_type)
    return t


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="truncate the depth (say so when quoting the number)")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=16)
    ap.add_argument("--token-prefill", action="store_true", help="consume the prompt one position per step instead of in 64-row chunks")
    ap.add_argument("--type", type=int, default=gb.GGML_TYPE_Q4_K)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--allreduce", default="p2p", choices=["p2p", "nccl"], help="library peer-memory all-reduce or torch.distributed NCCL")
    ap.add_argument("--shard-of", type=int, default=0, help="one process: run rank 0's shard of an N-way split without collectives "
                                                            "(kernel time of a shard; the outputs are partial sums)")
    a = ap.parse_args()
    rank, local_rank, world = dist_env()
    import torch
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    os.environ.setdefault("ADAM_B200_DEVICE", str(local_rank))
    import adam_b200 as A
    cfg = gemma3_27b()
    if a.layers:
        cfg = with_layers(cfg, a.layers)
    gpu = A.init()
    tp_world = a.shard_of if (a.shard_of and world == 1) else world
    plan = shard_plan(cfg, rank, tp_world, a.type)
    tensors = build_shard(torch, gpu, cfg, plan, a.type, seed=100 + rank)
    kv_cap = a.prompt + a.warmup + a.steps + 8
    eng = ADAMEngineTP(gpu, cfg, tensors, rank, tp_world, presharded=True, use_graph=not a.no_graph, collectives=(tp_world == world), allreduce=a.allreduce,
                       kv_cap=kv_cap, max_batch=a.batch, kv_dtype="f16")
    del tensors
    prompts = [list(map(int, np.random.default_rng(b).integers(0, cfg.n_vocab, a.prompt))) for b in range(a.batch)]
    eng.begin(prompts, [kv_cap] * a.batch)
    pe0, pe1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.batch_begin()
    with torch.cuda.stream(eng._stream):
        pe0.record()
    eng.prefill(a.prompt - 1, chunked=not a.token_prefill)
    with torch.cuda.stream(eng._stream):
        pe1.record()
    eng.step(max(3, a.warmup), lm_head=True)
    gpu.batch_end()
    pe1.synchronize()
    pre_ms = pe0.elapsed_time(pe1)
    if world > 1:
        dist.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gpu.batch_begin()
    with torch.cuda.stream(eng._stream):
        ev0.record()
    eng.step(a.steps, lm_head=True)
    with torch.cuda.stream(eng._stream):
        ev1.record()
    gpu.batch_end()
    ev1.synchronize()
    ms = ev0.elapsed_time(ev1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    err = gpu.device_error()
    lc = eng.cfg
    w_elems = lc.n_layer * ((lc.n_head + 2 * lc.n_head_kv) * lc.head_dim * cfg.n_embd + cfg.n_embd * lc.n_head * lc.head_dim
                            + 3 * lc.n_ff * cfg.n_embd) + lc.n_vocab * cfg.n_embd
    w_bytes = w_elems * block_bytes(a.type) // block_elems(a.type)
    graph_used = bool(eng._graphs)
    ar_used = eng._ar is not None
    eng.close()
    gpu.shutdown()
    if rank == 0:
        ms_tok = ms / a.steps
        print(json.dumps({"metric": "decode tok/s (Gemma-3-27B-shape, tensor parallel)", "value": a.batch * a.steps / (ms * 1e-3), "unit": "tok/s",
                          "n_gpus": world, "steps": a.steps, "ms_per_step": ms_tok, "batch": a.batch, "n_layer": cfg.n_layer,
                          "weights": "Q4_K" if a.type == gb.GGML_TYPE_Q4_K else "Q4_0", "parallelism": f"tp{tp_world}" + ("" if tp_world == world else " (one shard, no collectives)"),
                          "weight_bytes_per_rank_per_step": int(w_bytes), "GBs_per_gpu": w_bytes / (ms_tok * 1e-3) / 1e9,
                          "prefill_tok_s": a.batch * (a.prompt - 1) / (pre_ms * 1e-3) if a.prompt > 1 else None,
                          "prefill": "token by token" if a.token_prefill else "64 rows per pass",
                          "collectives_per_step": 2 * cfg.n_layer + 2 if world > 1 else 0, "graph": graph_used, "allreduce": ("p2p" if ar_used else "nccl") if world > 1 else None, "device_error": int(err),
                          "data": "synthetic random blocks"}))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
