"""Tensor-parallel decode: shard arithmetic on CPU, the decoder's part-wise step on one
GPU, and two NCCL ranks against the oracle that sums shard partials in rank order.
The reference has no multi-GPU path, so the oracle side is a flagged extension."""
import json
import os
import socket
import subprocess
import sys
from dataclasses import replace

import numpy as np
import pytest

from adam_b200 import gguf_blocks as gb
from adam_b200 import synth
from adam_b200.config import GenerationConfig, gemma3_27b, tiny_gemma3
from adam_b200.tp import shard_plan, shard_tensors
from oracle.decoder import OracleDecoder, dequant_model
from oracle.q4_blocks import dequant_q4_0, dequant_q4_k

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GREEDY = dict(top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=())


def _deq(t):
    f = dequant_q4_0 if t.ggml_type == gb.GGML_TYPE_Q4_0 else dequant_q4_k
    return f(np.asarray(t.raw, np.uint8), t.rows * t.cols).reshape(t.rows, t.cols)


def _tp_cfg(ggml_type):
    # 4 query / 2 kv heads, head_dim 128 (a rank's two heads = one Q4_K superblock of the o-proj K); n_ff = 3 blocks of 256 so that two Q4_K ranks get uneven shards
    kw = dict(n_layer=2, n_embd=256, n_head=4, n_head_kv=2, head_dim=128, n_ff=768, n_vocab=512)
    cfg = replace(tiny_gemma3(), **kw)
    return replace(cfg, head_dim_kv=128)


def test_shard_plan_partitions_heads_ffn_and_vocab():
    cfg = gemma3_27b()
    for world in (1, 2, 4, 8):
        plans = [shard_plan(cfg, r, world, gb.GGML_TYPE_Q4_K) for r in range(world)]
        assert [h for p in plans for h in p.heads] == list(range(cfg.n_head))
        assert [h for p in plans for h in p.kv_heads] == list(range(cfg.n_head_kv))
        assert [v for p in plans for v in (p.vocab.start, p.vocab.stop)][0] == 0 and plans[-1].vocab.stop == cfg.n_vocab
        edges = [p.ff.start for p in plans] + [plans[-1].ff.stop]
        assert edges == list(plans[0].ff_bounds) and edges[0] == 0 and edges[-1] == cfg.n_ff
        assert all(e % 256 == 0 for e in edges)                     # whole Q4_K superblocks (84 of them: uneven at 8 ranks)
        sizes = [len(p.ff) for p in plans]
        assert max(sizes) - min(sizes) <= 256
    with pytest.raises(ValueError):
        shard_plan(cfg, 0, 3, gb.GGML_TYPE_Q4_K)                    # 32 heads over 3 ranks


@pytest.mark.parametrize("ggml_type", [gb.GGML_TYPE_Q4_0, gb.GGML_TYPE_Q4_K])
def test_shards_are_slices_and_partials_add_up(ggml_type):
    cfg = _tp_cfg(ggml_type)
    tensors = synth.build_model(cfg, ggml_type, seed=5)
    world = 2
    rng = np.random.default_rng(0)
    x_att = rng.standard_normal(cfg.n_head * cfg.head_dim).astype(np.float32)
    x_ff = rng.standard_normal(cfg.n_ff).astype(np.float32)
    full_o = _deq(tensors["blk.0.attn_output.weight"])
    full_d = _deq(tensors["blk.0.ffn_down.weight"])
    acc_o = np.zeros(cfg.n_embd, np.float32)
    acc_d = np.zeros(cfg.n_embd, np.float32)
    rows_q, rows_g, rows_lm = [], [], []
    for r in range(world):
        plan = shard_plan(cfg, r, world, ggml_type)
        local, lt = shard_tensors(cfg, tensors, plan)
        assert local.n_head == 2 and local.n_head_kv == 1 and local.n_ff == len(plan.ff) and local.n_vocab == len(plan.vocab)
        assert lt["token_embd.weight"].rows == cfg.n_vocab                       # table stays whole
        hd = cfg.head_dim
        q0, q1 = plan.heads.start * hd, plan.heads.stop * hd
        assert np.array_equal(_deq(lt["blk.0.attn_output.weight"]), full_o[:, q0:q1])
        assert np.array_equal(_deq(lt["blk.0.ffn_down.weight"]), full_d[:, plan.ff.start:plan.ff.stop])
        acc_o += _deq(lt["blk.0.attn_output.weight"]) @ x_att[q0:q1]
        acc_d += _deq(lt["blk.0.ffn_down.weight"]) @ x_ff[plan.ff.start:plan.ff.stop]
        rows_q.append(_deq(lt["blk.0.attn_q.weight"]))
        rows_g.append(_deq(lt["blk.1.ffn_gate.weight"]))
        rows_lm.append(_deq(lt["output.weight"]))
    assert np.allclose(acc_o, full_o @ x_att, rtol=1e-5, atol=1e-6)
    assert np.allclose(acc_d, full_d @ x_ff, rtol=1e-5, atol=1e-6)
    assert np.array_equal(np.concatenate(rows_q), _deq(tensors["blk.0.attn_q.weight"]))
    assert np.array_equal(np.concatenate(rows_g), _deq(tensors["blk.1.ffn_gate.weight"]))
    assert np.array_equal(np.concatenate(rows_lm), _deq(tensors["token_embd.weight"]))
    if ggml_type == gb.GGML_TYPE_Q4_K:
        assert [len(shard_plan(cfg, r, world, ggml_type).ff) for r in range(world)] == [512, 256]


def test_oracle_tp_sum_order_stays_within_tolerance():
    cfg = _tp_cfg(gb.GGML_TYPE_Q4_K)
    f32 = dequant_model(synth.build_model(cfg, gb.GGML_TYPE_Q4_K, seed=5))
    toks = synth.random_prompt(cfg.n_vocab, 6, seed=2)
    bounds = shard_plan(cfg, 0, 2, gb.GGML_TYPE_Q4_K).ff_bounds
    a = OracleDecoder(cfg, f32, kv_cap=8)
    b = OracleDecoder(cfg, f32, kv_cap=8, tp_size=2, tp_ff_bounds=bounds)
    for i, t in enumerate(toks):
        la, lb = a.forward(int(t), i), b.forward(int(t), i)
        assert np.abs(la - lb).max() <= 1e-3 * np.abs(la).max()


@pytest.mark.gpu
@pytest.mark.parametrize("use_graph", [False, True])
def test_part_wise_step_equals_reference_ids(gpu, golden_dir, use_graph):
    """World size 1: the same kernels, enqueued part by part on a torch stream (and recorded
    into a torch CUDA graph), must give the golden ids of the unmodified reference."""
    from adam_b200.tp import ADAMEngineTP
    from tests.golden.make_golden import DECODE_CASES
    name, bkw, ckw, n_prompt, n_gen = DECODE_CASES[0]
    g = np.load(os.path.join(golden_dir, "decode_tiny.npz"))
    cfg = replace(tiny_gemma3(), **ckw)
    if "head_dim" in ckw:
        cfg = replace(cfg, head_dim_kv=ckw["head_dim"])
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, **bkw)
    eng = ADAMEngineTP(gpu, cfg, tensors, 0, 1, use_graph=use_graph, kv_cap=64, kv_dtype="f32")
    try:
        toks, _ = eng.generate(g[f"{name}_prompt"], GenerationConfig(max_tokens=n_gen, **GREEDY))
        assert toks == g[f"{name}_tokens"].tolist()
        assert bool(eng._graphs) == use_graph
        assert gpu.device_error() == 0
    finally:
        eng.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.gpu
@pytest.mark.parametrize("ggml_type,allreduce", [(gb.GGML_TYPE_Q4_0, "p2p"), (gb.GGML_TYPE_Q4_K, "p2p"), (gb.GGML_TYPE_Q4_K, "nccl")])
def test_two_ranks_match_the_oracle(ggml_type, allreduce):
    """Two ranks (needs two GPUs), projections summed by the library's peer-memory all-reduce or by NCCL:
    greedy ids equal the rank-ordered oracle's, logits within 1e-3."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), os.path.join(ROOT, "tests", "tp_rank_main.py"), str(int(ggml_type)), allreduce]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert out.returncode == 0, (out.stdout[-1500:], out.stderr[-3000:])
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert res["ids_equal"], res
    assert res["long_ids_equal"] and res["long_equals_by_token"], res      # chunked prefill across ranks
    assert res["logit_rel_err"] < 1e-3
    assert res["graph_used"] and res["device_error"] == 0
    assert res["p2p_allreduce"] == (allreduce == "p2p")


_TP_GLOO_SCRIPT = '''
import json, os, sys
sys.path.insert(0, %r)
import numpy as np, torch, torch.distributed as dist
from dataclasses import replace
from adam_b200 import gguf_blocks as gb, synth
from adam_b200.config import tiny_gemma3
from adam_b200.tp import merge_argmax_pairs, shard_plan, shard_tensors
from oracle.q4_blocks import dequant_q4_k
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
cfg = replace(tiny_gemma3(), n_layer=1, n_embd=256, n_head=4, n_head_kv=2, head_dim=128, head_dim_kv=128, n_ff=768, n_vocab=512)
tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_K, seed=5)
deq = lambda t: dequant_q4_k(np.asarray(t.raw, np.uint8), t.rows * t.cols).reshape(t.rows, t.cols)
plan = shard_plan(cfg, rank, world, gb.GGML_TYPE_Q4_K)
local, lt = shard_tensors(cfg, tensors, plan)
rng = np.random.default_rng(0)
x_ff = rng.standard_normal(cfg.n_ff).astype(np.float32)          # same on every rank (seeded)
z = rng.standard_normal(cfg.n_embd).astype(np.float32)
# row-parallel down-proj: partial sums, all-reduce
part = torch.from_numpy(deq(lt["blk.0.ffn_down.weight"]) @ x_ff[plan.ff.start:plan.ff.stop])
dist.all_reduce(part)
# vocabulary-parallel LM head: local arg-max pair, gather, merge (with a forced tie across ranks)
logits = deq(lt["output.weight"]) @ z
logits[3] = 1e6                                                    # every rank's row 3 ties at the top
v = torch.tensor([float(logits.max())]); i = torch.tensor([int(logits.argmax()) + plan.vocab.start], dtype=torch.int32)
vs = [torch.empty_like(v) for _ in range(world)]; is_ = [torch.empty_like(i) for _ in range(world)]
dist.all_gather(vs, v); dist.all_gather(is_, i)
tok = int(merge_argmax_pairs(torch.stack(vs), torch.stack(is_))[0])
if rank == 0:
    full = deq(tensors["blk.0.ffn_down.weight"]) @ x_ff
    print(json.dumps({"down_err": float(np.abs(part.numpy() - full).max() / np.abs(full).max()), "tok": tok}))
dist.destroy_process_group()
'''


def test_two_gloo_ranks_reduce_and_merge_like_the_tp_engine(tmp_path):
    """The host side of tensor parallelism on CPU: shards from ``shard_tensors``, a gloo all-reduce of the
    row-parallel partial sums, and the arg-max merge with a tie across ranks (lower id wins)."""
    script = tmp_path / "tp_rank.py"
    script.write_text(_TP_GLOO_SCRIPT % ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(script)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert res["down_err"] < 1e-5
    assert res["tok"] == 3                          # rank 0's row 3, not rank 1's row 3 (global id 259)


@pytest.mark.gpu
def test_peer_allreduce_wait_runs_out_and_returns(gpu):
    """Two communicator ends in one process stand for two ranks; only rank 0 ever calls.  Its wait for rank 1's
    packets (memory nobody writes) must run out at the 30 ms limit, return, report error bit 2 and the sticky
    word; while the word is set calls do not wait; after a reset they wait (and run out) again."""
    import ctypes
    import time
    import torch
    lib = gpu._lib
    ids = (ctypes.c_uint32 * 2)()
    blob = ctypes.create_string_buffer(128)
    for r in range(2):
        cid = ctypes.c_uint32(0)
        assert lib.adam_b200_ar_create(2, r, 4096, ctypes.byref(cid), blob) == 0
        ids[r] = cid.value
    try:
        for r in range(2):
            assert lib.adam_b200_ar_open_local(ids[r], ids, 2) == 0
        assert lib.adam_b200_ar_set_wait_us(ids[0], 30000) == 0
        buf = torch.ones(256, dtype=torch.float32, device=f"cuda:{gpu.device_index}")
        torch.cuda.synchronize()
        gpu.device_error()
        t0 = time.perf_counter()
        assert lib.adam_b200_ar_allreduce(ids[0], buf.data_ptr(), 256) == 0
        gpu.sync()
        dt = time.perf_counter() - t0
        assert 0.02 < dt < 2.0, dt
        assert gpu.device_error() & 2
        assert lib.adam_b200_ar_timed_out(ids[0]) == 1
        t0 = time.perf_counter()
        assert lib.adam_b200_ar_allreduce(ids[0], buf.data_ptr(), 256) == 0      # sticky: no second wait
        gpu.sync()
        assert time.perf_counter() - t0 < 0.02
        assert lib.adam_b200_ar_reset(ids[0]) == 0 and lib.adam_b200_ar_timed_out(ids[0]) == 0
        t0 = time.perf_counter()
        assert lib.adam_b200_ar_allreduce(ids[0], buf.data_ptr(), 256) == 0
        gpu.sync()
        assert time.perf_counter() - t0 > 0.02 and lib.adam_b200_ar_timed_out(ids[0]) == 1
        gpu.device_error()
    finally:
        for r in range(2):
            lib.adam_b200_ar_destroy(ids[r])
