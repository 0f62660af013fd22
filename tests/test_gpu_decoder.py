"""Fused decoder against the oracle and against greedy ids produced by the
unmodified reference (tests/golden/decode_tiny.npz).  Through the C ABI."""
import os
from dataclasses import replace

import numpy as np
import pytest

from adam_b200 import gguf_blocks as gb
from adam_b200 import synth
from adam_b200.config import GenerationConfig, tiny_gemma3
from adam_b200.engine import ADAMEngine
from oracle.decoder import OracleDecoder, dequant_model

from tests.golden.make_golden import DECODE_CASES

pytestmark = pytest.mark.gpu

GREEDY = dict(top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=())


def _cfg(ckw):
    cfg = replace(tiny_gemma3(), **ckw)
    if "head_dim" in ckw:
        cfg = replace(cfg, head_dim_kv=ckw["head_dim"])
    return cfg


def _rel(a, b):
    return float(np.abs(a - b).max() / np.abs(b).max())


@pytest.mark.parametrize("case", DECODE_CASES, ids=[c[0] for c in DECODE_CASES])
def test_greedy_ids_equal_reference(gpu, golden_dir, case):
    """Token ids from the unmodified reference numpy decoder (fp32 KV, no window)."""
    name, bkw, ckw, n_prompt, n_gen = case
    g = np.load(os.path.join(golden_dir, "decode_tiny.npz"))
    cfg = _cfg(ckw)
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, **bkw)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=64, kv_dtype="f32")
    try:
        toks, stats = eng.generate(g[f"{name}_prompt"], GenerationConfig(max_tokens=n_gen, **GREEDY))
        assert toks == g[f"{name}_tokens"].tolist()
        assert stats["n_gen"] == n_gen and stats["sampling_mode"] == "gpu_matvec_argmax"
        assert gpu.device_error() == 0
    finally:
        eng.close()


@pytest.mark.parametrize("ggml_type,tied", [(gb.GGML_TYPE_Q4_0, True), (gb.GGML_TYPE_Q4_0, False), (gb.GGML_TYPE_Q4_K, False)])
def test_teacher_forced_logits_match_oracle(gpu, ggml_type, tied):
    """Every position's logits within 1e-3 (relative to the largest logit), fp32 KV."""
    cfg = _cfg(dict(n_layer=4))
    tensors = synth.build_model(cfg, ggml_type, seed=31, tied=tied)
    toks = synth.random_prompt(cfg.n_vocab, 20, seed=3)
    dec = OracleDecoder(cfg, dequant_model(tensors), kv_cap=32)
    ref = np.stack([dec.forward(int(t), i) for i, t in enumerate(toks)])
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=32, kv_dtype="f32")
    try:
        out = eng.logits_trace(toks)
        assert _rel(out, ref) < 1e-3
        assert _rel(out, ref) < 1e-4          # in practice far inside the budget
        assert np.array_equal(out.argmax(1), ref.argmax(1))
        # the hidden state of the last step as well
        dec.trace = {}
        dec.reset()
        for i, t in enumerate(toks):
            dec.forward(int(t), i)
        h = eng.read_buffer(0, cfg.n_embd)
        assert _rel(h, dec.trace[f"hidden.{cfg.n_layer - 1}"]) < 1e-4
        assert gpu.device_error() == 0
    finally:
        eng.close()


def test_fp16_kv_matches_oracle_extension(gpu):
    """KV rounded to fp16 when stored (extension; oracle flag kv_dtype=float16)."""
    cfg = _cfg(dict(n_layer=3))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=32, tied=False)
    toks = synth.random_prompt(cfg.n_vocab, 24, seed=4)
    f32 = dequant_model(tensors)
    ref16 = OracleDecoder(cfg, f32, kv_cap=32, kv_dtype=np.float16)
    ref = np.stack([ref16.forward(int(t), i) for i, t in enumerate(toks)])
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=32, kv_dtype="f16")
    try:
        out = eng.logits_trace(toks)
        assert _rel(out, ref) < 1e-3
        prompt = toks[:8]
        want, _ = OracleDecoder(cfg, f32, kv_cap=64, kv_dtype=np.float16).generate(prompt, 24)
        got, _ = eng.generate(prompt, GenerationConfig(max_tokens=24, **GREEDY))
        assert got == want
    finally:
        eng.close()


def test_sliding_window_matches_oracle_extension(gpu):
    """Window mask on non-global layers (extension; oracle flag window=True)."""
    cfg = _cfg(dict(n_layer=7, sliding_window=8))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=33, tied=False)
    toks = synth.random_prompt(cfg.n_vocab, 30, seed=5)
    f32 = dequant_model(tensors)
    dec = OracleDecoder(cfg, f32, kv_cap=32, window=True)
    ref = np.stack([dec.forward(int(t), i) for i, t in enumerate(toks)])
    nowin = OracleDecoder(cfg, f32, kv_cap=32)
    ref_nw = np.stack([nowin.forward(int(t), i) for i, t in enumerate(toks)])
    assert _rel(ref, ref_nw) > 1e-2                     # the mask matters at this length
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=32, kv_dtype="f32", window=True)
    try:
        assert _rel(eng.logits_trace(toks), ref) < 1e-4
    finally:
        eng.close()
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=32, kv_dtype="f32", window=False)   # reference behaviour: no mask
    try:
        assert _rel(eng.logits_trace(toks), ref_nw) < 1e-4
    finally:
        eng.close()


def test_long_context_uses_several_attention_splits_and_pages(gpu):
    cfg = _cfg(dict(n_layer=2, n_head=4, n_head_kv=2, head_dim=64))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=34, tied=True)
    n = 600                                               # > 2 splits of 256, 10 pages of 64
    toks = synth.random_prompt(cfg.n_vocab, n, seed=6)
    dec = OracleDecoder(cfg, dequant_model(tensors), kv_cap=n + 8)
    for i, t in enumerate(toks):
        ref = dec.forward(int(t), i, want_logits=(i == n - 1))
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=n + 8, kv_dtype="f32")
    try:
        eng.begin([toks], [n])
        eng.step(n - 1, lm_head=False)
        eng.step(1, lm_head=True, logits=True)
        assert _rel(eng.read_logits(0), ref) < 1e-4
        assert gpu.device_error() == 0
    finally:
        eng.close()


def test_clustered_and_independent_attention_splits_agree(gpu):
    """One sequence: a cache of at most 2048 positions runs the position splits of a head as one thread-block cluster that
    merges through shared memory, a larger one as independent CTAs that merge through global memory.  Same prompt, same
    weights: both match the oracle, and each other's ids."""
    cfg = _cfg(dict(n_layer=2, n_head=4, n_head_kv=2, head_dim=64))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=35, tied=True)
    n = 300                                               # several splits of 64 positions
    toks = synth.random_prompt(cfg.n_vocab, n, seed=7)
    dec = OracleDecoder(cfg, dequant_model(tensors), kv_cap=n + 40)
    for i, t in enumerate(toks):
        ref = dec.forward(int(t), i, want_logits=(i == n - 1))
    ids = []
    for kv_cap in (n + 40, 4096):
        eng = ADAMEngine(gpu, cfg, tensors, kv_cap=kv_cap, kv_dtype="f32")
        try:
            eng.begin([toks], [n + 32])
            eng.step(n - 1, lm_head=False)
            eng.step(1, lm_head=True, logits=True)
            assert _rel(eng.read_logits(0), ref) < 1e-4
            eng.step(24, lm_head=True)
            ids.append(eng.read_log(0, n, 25))
            assert gpu.device_error() == 0
        finally:
            eng.close()
    assert np.array_equal(ids[0], ids[1]) and (ids[0] >= 0).all()


def test_batch_of_ragged_prompts_equals_single_sequence_runs(gpu):
    cfg = _cfg(dict(n_layer=3))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=35, tied=False)
    f32 = dequant_model(tensors)
    prompts = [synth.random_prompt(cfg.n_vocab, n, seed=40 + n) for n in (5, 11, 8, 11, 1, 7)]
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=48, kv_dtype="f32", max_batch=6)
    try:
        outs, stats = eng.generate_batch(prompts, GenerationConfig(max_tokens=12, **GREEDY))
        for p, o in zip(prompts, outs):
            want, _ = OracleDecoder(cfg, f32, kv_cap=48).generate(p, 12)
            assert o == want
        assert stats["batch"] == 6 and stats["n_gen"] == 72
        # fewer host syncs give the same ids
        outs2, _ = eng.generate_batch(prompts, GenerationConfig(max_tokens=12, **GREEDY), sync_every=5)
        assert outs2 == outs
        # and a smaller batch on the same engine still works (graph is rebuilt)
        outs3, _ = eng.generate_batch(prompts[:2], GenerationConfig(max_tokens=12, **GREEDY))
        assert outs3 == outs[:2]
    finally:
        eng.close()


@pytest.mark.parametrize("tc", [False, True])
@pytest.mark.parametrize("ggml_type,kv_dtype,window", [(gb.GGML_TYPE_Q4_0, "f32", False), (gb.GGML_TYPE_Q4_0, "f16", True), (gb.GGML_TYPE_Q4_K, "f32", False)])
def test_chunked_prefill_equals_token_by_token(gpu, ggml_type, kv_dtype, window, tc):
    """The prompt consumed 64 rows (sequences x positions) at a time must leave the same state as single
    steps: same logits for the token after the prompt, same greedy continuation, ragged prompts included."""
    cfg = _cfg(dict(n_layer=3, sliding_window=8) if window else dict(n_layer=3))
    tensors = synth.build_model(cfg, ggml_type, seed=41)
    prompts = [synth.random_prompt(cfg.n_vocab, n, seed=50 + n) for n in (90, 71, 90)]      # > 64 rows: several chunks, 21 tokens each
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=128, kv_dtype=kv_dtype, max_batch=3, window=window)
    try:
        n_pre = min(len(p) for p in prompts) - 1
        eng.begin(prompts, [120] * 3)
        gpu.batch_begin(); eng.step(n_pre, lm_head=False); eng.step(1, lm_head=True, logits=True); gpu.batch_end()
        ref_logits = np.stack([eng.read_logits(b) for b in range(3)])
        gpu.batch_begin(); eng.step(8, lm_head=True); gpu.batch_end()
        ref_ids = [eng.read_log(b, n_pre + 1, 9) for b in range(3)]
        eng.begin(prompts, [120] * 3)
        # tc: the chunk's products on the tcgen05 GEMM (norm chain in, GeGLU out), which small shapes do not take by default
        gpu.tc_gemm_policy(2 if tc else 0)
        before = gpu.tc_gemm_count()
        try:
            gpu.batch_begin(); eng.prefill(n_pre); gpu.batch_end()
        finally:
            gpu.tc_gemm_policy(1)
        assert (gpu.tc_gemm_count() > before) == tc
        gpu.batch_begin(); eng.step(1, lm_head=True, logits=True); gpu.batch_end()
        got_logits = np.stack([eng.read_logits(b) for b in range(3)])
        gpu.batch_begin(); eng.step(8, lm_head=True); gpu.batch_end()
        got_ids = [eng.read_log(b, n_pre + 1, 9) for b in range(3)]
        # the chunk's products run on another kernel (other summation order); with an f16 cache a last-bit
        # difference can move a cached value by one f16 step, hence the wider bound there
        tol = 1e-3 if kv_dtype == "f16" else 2e-5
        assert np.abs(got_logits - ref_logits).max() <= tol * np.abs(ref_logits).max()
        for a, b in zip(ref_ids, got_ids):
            assert np.array_equal(a, b)
        assert gpu.device_error() == 0
        # asking for more prompt tokens than a sequence has left is refused
        eng.begin(prompts, [120] * 3)
        with pytest.raises(RuntimeError, match="prompt tokens left"):
            eng.prefill(80)
    finally:
        eng.close()


def test_host_sampling_mode(gpu):
    """Non-greedy configurations are sampled on the host from the logits (the reference's 'cpu' mode,
    engine.py:3711-3729): every drawn id lies in the oracle's top-k set after the repeat penalty, the same seed
    gives the same ids, and a one-candidate nucleus reduces to arg-max."""
    cfg = _cfg(dict(n_layer=2))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=44)
    f32 = dequant_model(tensors)
    prompt = [int(t) for t in synth.random_prompt(cfg.n_vocab, 7, seed=9)]
    gen = GenerationConfig(max_tokens=12, temperature=0.9, top_k=100, top_p=0.95, repeat_penalty=1.3, seed=123, eos_token_ids=())   # more than 64 candidates: host
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=32, kv_dtype="f32")
    try:
        ids, st = eng.generate(prompt, gen)
        assert st["sampling_mode"] == "cpu" and len(ids) == 12
        ids2, _ = eng.generate(prompt, gen)
        assert ids2 == ids
        dec = OracleDecoder(cfg, f32, kv_cap=32)
        seq = prompt + ids
        for i, t in enumerate(seq[:-1]):
            logits = dec.forward(t, i)
            if i >= len(prompt) - 1:
                lg = logits.copy()
                for h in set(seq[len(prompt):i + 1][-64:]):
                    lg[h] = lg[h] / 1.3 if lg[h] > 0 else lg[h] * 1.3
                assert seq[i + 1] in set(np.argsort(-lg)[:100].tolist())
        # a nucleus that keeps one candidate is arg-max of the penalised logits
        one, _ = eng.generate(prompt, GenerationConfig(max_tokens=6, temperature=0.7, top_k=40, top_p=1e-6, repeat_penalty=1.0, seed=1,
                                                       eos_token_ids=()))
        greedy, _ = eng.generate(prompt, GenerationConfig(max_tokens=6, **GREEDY))
        assert one == greedy
    finally:
        eng.close()


def test_prefix_reuse_continues_from_the_cache(gpu):
    """generate(reuse_prefix=n) (engine.py:3815-3833): a second turn that repeats the first turn's tokens
    gives the ids of a fresh run on the whole prompt, and only the new tokens are prefilled."""
    cfg = _cfg(dict(n_layer=3))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=43)
    p1 = [int(t) for t in synth.random_prompt(cfg.n_vocab, 23, seed=61)]
    p2 = [int(t) for t in synth.random_prompt(cfg.n_vocab, 9, seed=62)]
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=96, kv_dtype="f32", page_size=16)
    try:
        t1, _ = eng.generate(p1, GenerationConfig(max_tokens=6, **GREEDY))
        turn2 = p1 + t1 + p2
        cached = len(p1) + len(t1) - 1                      # the last sampled token was never fed back
        got, st = eng.generate(turn2, GenerationConfig(max_tokens=10, **GREEDY), reuse_prefix=cached)
        assert st["n_prompt_reused"] == cached and st["n_prompt_prefilled"] == len(turn2) - cached
        want, _ = eng.generate(turn2, GenerationConfig(max_tokens=10, **GREEDY))
        assert got == want
        oracle_ids, _ = OracleDecoder(cfg, dequant_model(tensors), kv_cap=96).generate(turn2, 10)   # and of the oracle
        assert got == oracle_ids
        # more reused positions than were ever computed are refused
        eng.generate(p1, GenerationConfig(max_tokens=2, **GREEDY))
        with pytest.raises(RuntimeError, match="are cached"):
            eng.generate(turn2, GenerationConfig(max_tokens=2, **GREEDY), reuse_prefix=len(p1) + 5)
        assert gpu.device_error() == 0
    finally:
        eng.close()


def test_graph_replay_equals_direct_launches(gpu):
    cfg = _cfg(dict(n_layer=2))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=36)
    prompt = synth.random_prompt(cfg.n_vocab, 6, seed=7)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=32)
    try:
        eng.begin([prompt], [30])
        eng.step(5, lm_head=False, direct=True, chain=True)
        eng.step(10, lm_head=True, direct=True, chain=True)
        a = eng.read_log(0, 6, 10)
        eng.begin([prompt], [30])
        gpu.reset_native_stats()
        eng.step(5, lm_head=False, chain=True)
        eng.step(10, lm_head=True, chain=True)
        b = eng.read_log(0, 6, 10)
        assert np.array_equal(a, b) and (a >= 0).all()
        assert gpu.get_native_stats()["dispatch_count"] >= 15 * 5 * cfg.n_layer     # graph nodes are counted (5 kernels per layer)
        # the single-launch token kernel: one launch per token, same ids
        eng.begin([prompt], [30])
        gpu.reset_native_stats()
        eng.step(5, lm_head=False, chain=False)
        eng.step(10, lm_head=True, chain=False)
        c = eng.read_log(0, 6, 10)
        assert np.array_equal(a, c)
        assert gpu.get_native_stats()["dispatch_count"] == 15
        assert gpu.device_error() == 0
    finally:
        eng.close()


def test_eos_stops_generation_and_kv_cap_is_enforced(gpu):
    cfg = _cfg(dict(n_layer=2))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=37, tied=False)
    prompt = synth.random_prompt(cfg.n_vocab, 6, seed=8)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=32)
    try:
        full, _ = eng.generate(prompt, GenerationConfig(max_tokens=10, **GREEDY))
        eos = full[4]
        cut, _ = eng.generate(prompt, GenerationConfig(max_tokens=10, top_k=1, temperature=0.0, repeat_penalty=1.0, eos_token_ids=(eos,)))
        assert cut == full[:full.index(eos)]
        with pytest.raises(RuntimeError, match="KV cache too small"):
            eng.generate(prompt, GenerationConfig(max_tokens=27, **GREEDY))
        with pytest.raises(RuntimeError, match="outside the vocabulary"):
            eng.begin([[cfg.n_vocab + 3]], [4])
    finally:
        eng.close()


def test_bounded_wait_runs_out_and_the_kernel_returns(gpu):
    """A device-side wait that nothing satisfies: the token kernel is launched once with its last CTA left
    out and a 20 ms limit.  The kernel must come back by itself, report the expired wait (error bit 2), make
    later steps return at once, and work again after the next begin()."""
    import time
    cfg = _cfg(dict(n_layer=3))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=41, tied=False)
    prompt = synth.random_prompt(cfg.n_vocab, 6, seed=9)
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=48, single_launch=True)
    try:
        good, _ = eng.generate(prompt, GenerationConfig(max_tokens=8, **GREEDY))
        eng.begin([prompt], [40])
        eng.step(5, lm_head=False)
        t0 = time.perf_counter()
        rc = eng._lib.adam_b200_decoder_test_wait_expiry(eng._dec, 20000)
        dt = time.perf_counter() - t0
        assert rc == 0
        assert dt < 2.0, f"the kernel took {dt:.2f} s to give up"
        assert gpu.device_error() & 2                     # DEVERR_WAIT (the read clears the word)
        pos_before, _ = eng.read_state()
        t0 = time.perf_counter()
        eng.step(3, lm_head=True)                         # sticky word: these launches return at once
        gpu.sync()
        assert time.perf_counter() - t0 < 0.5
        pos_after, _ = eng.read_state()
        assert pos_after[0] == pos_before[0] == 5         # nothing advanced
        gpu.device_error()
        again, _ = eng.generate(prompt, GenerationConfig(max_tokens=8, **GREEDY))    # begin() clears the word
        assert again == good
        assert gpu.device_error() == 0
    finally:
        eng.close()


def _splitmix_uniform(seed, seq, pos):
    """The device generator of sampled steps: splitmix64 of (seed, sequence, position), top 24 bits."""
    m = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15 * (((seq << 32) | pos) + 1)) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z ^= z >> 31
    return np.float32(z >> 40) * np.float32(1.0 / 16777216.0)


def test_device_sampling_mode(gpu):
    """Repeat penalty, top-k, nucleus and the draw on the device ('gpu_fused_topk', engine.py:3403-3512; rule of
    `_sample`, :3711-3729): the ids are reproduced on the host from the device's own logits by the same rule and
    the same counter-based uniform numbers; 4 bytes come back per token; greedy with a penalty takes the best
    penalised logit."""
    cfg = _cfg(dict(n_layer=2))
    tensors = synth.build_model(cfg, gb.GGML_TYPE_Q4_0, seed=45, tied=False)
    prompt = [int(t) for t in synth.random_prompt(cfg.n_vocab, 7, seed=9)]
    T, K, P, PEN, SEED = 0.9, 5, 0.9, 1.3, 123
    gen = GenerationConfig(max_tokens=14, temperature=T, top_k=K, top_p=P, repeat_penalty=PEN, seed=SEED, eos_token_ids=())
    eng = ADAMEngine(gpu, cfg, tensors, kv_cap=40, kv_dtype="f32")
    try:
        ids, st = eng.generate(prompt, gen)
        assert st["sampling_mode"] == "gpu_fused_topk" and len(ids) == 14 and st["d2h_bytes"] == 4 * 14
        ids2, _ = eng.generate(prompt, gen)
        assert ids2 == ids
        other, _ = eng.generate(prompt, GenerationConfig(max_tokens=14, temperature=T, top_k=K, top_p=P, repeat_penalty=PEN, seed=7, eos_token_ids=()))
        assert other != ids                                  # another seed, another draw
        logits = eng.logits_trace(prompt + ids[:-1])
        f32 = np.float32

        def penalised(lg, hist):
            lg = lg.copy()
            for t in set(hist[-64:]):
                lg[t] = lg[t] / f32(PEN) if lg[t] > 0 else lg[t] * f32(PEN)
            return lg

        for i in range(len(ids)):
            lg = penalised(logits[len(prompt) - 1 + i], ids[:i])
            order = np.lexsort((np.arange(lg.size), -lg))[:K]         # value descending, ties to the lower id
            l = lg[order]
            p = np.exp(((l - l[0]) / f32(T)).astype(f32)).astype(f32)
            tot = f32(0)
            for v in p:
                tot = f32(tot + v)
            keep, cs = K, f32(0)
            for r in range(K):
                cs = f32(cs + f32(p[r] / tot))
                if cs >= f32(P):
                    keep = r + 1
                    break
            ks = f32(0)
            for r in range(keep):
                ks = f32(ks + p[r])
            target = f32(_splitmix_uniform(SEED, 0, len(prompt) + i) * ks)
            acc, chosen, margin = f32(0), keep - 1, 1.0
            for r in range(keep):
                acc = f32(acc + p[r])
                margin = min(margin, abs(float(target) - float(acc)))
                if target < acc:
                    chosen = r
                    break
            if margin > 1e-5:                                 # (a draw that lands on a boundary may round either way)
                assert ids[i] == int(order[chosen]), f"step {i}"
        # greedy with a repeat penalty: the best penalised logit, still on the device
        gid, st = eng.generate(prompt, GenerationConfig(max_tokens=10, top_k=1, temperature=0.0, repeat_penalty=PEN, eos_token_ids=()))
        assert st["sampling_mode"] == "gpu_fused_topk"
        glog = eng.logits_trace(prompt + gid[:-1])
        for i in range(len(gid)):
            assert gid[i] == int(np.argmax(penalised(glog[len(prompt) - 1 + i], gid[:i])))
        # repeat_on_prompt widens the history to the prompt
        pid, _ = eng.generate(prompt, GenerationConfig(max_tokens=4, top_k=1, temperature=0.0, repeat_penalty=3.0, repeat_on_prompt=True, eos_token_ids=()))
        plog = eng.logits_trace(prompt + pid[:-1])
        lg0 = plog[len(prompt) - 1].copy()
        for t in set(prompt[-64:]):
            lg0[t] = lg0[t] / f32(3.0) if lg0[t] > 0 else lg0[t] * f32(3.0)
        assert pid[0] == int(np.argmax(lg0))
        assert gpu.device_error() == 0
    finally:
        eng.close()
