"""Registered decode plans (adamah.c:10253-10398; tests/test_decode_primitives.py:507-573) lowered to one CUDA graph
whose run-time arguments stay on the device: the same results as the operator calls made one by one with immediate
values, every step; one recording however many steps run; a re-recording when the sequence outgrows what the graph was
sized for; host-side substitution where an argument has no run-time form."""
import numpy as np
import pytest

import adam_b200 as A

pytestmark = pytest.mark.gpu

HD, ROWS = 64, 320                       # head size, cache rows
Q, KN, VN, QK, ROPED, NORMED, OUT = 0, 64, 128, 256, 384, 448, 512
KC, VC = 1024, 1024 + ROWS * HD          # K and V cache bases (multiples of HD)
SC = VC + ROWS * HD                      # scores
N_EL = SC + ROWS + 64
WMAP_N = 4 * HD


def _h(gpu, vals):
    return gpu.upload_dev(np.asarray(vals, np.uint32))[0]


def _read_all(gpu, mid):
    return gpu.gather(mid, np.arange(N_EL, dtype=np.uint32)).view(np.float32)


def _handles(gpu):
    return dict(q=_h(gpu, [Q]), k=_h(gpu, [KN]), qw=_h(gpu, [0]), kw=_h(gpu, [HD]), qk=_h(gpu, [QK]),
                kspec=_h(gpu, [0, KC // HD]), kbase=_h(gpu, [QK + HD]), vspec=_h(gpu, [0, VC // HD]), vbase=_h(gpu, [VN]),
                a=_h(gpu, [QK]), b=_h(gpu, [KC]), c=_h(gpu, [SC]), vals=_h(gpu, [VC]), out=_h(gpu, [OUT]),
                rs=_h(gpu, [VN]), rd=_h(gpu, [ROPED]), ns=_h(gpu, [OUT]), nw=_h(gpu, [2 * HD]), nd=_h(gpu, [NORMED]),
                e_src=_h(gpu, OUT + np.arange(HD)), e_dst=_h(gpu, NORMED + np.arange(HD)))


def _direct(gpu, mid, wmap, h, pos, seq):
    """The step as individual operator calls with immediate values."""
    gpu.batch_begin()
    gpu.map_qk_norm_rope_x_dev(mid, wmap, h["q"], h["qw"], h["k"], h["kw"], h["qk"], 1, HD, 1, HD, pos, 10000.0)
    gpu.map_row_copy_offset_dev(mid, h["kspec"], h["kbase"], pos, 1, HD)
    gpu.map_row_copy_offset_dev(mid, h["vspec"], h["vbase"], pos, 1, HD)
    gpu.map_matmul_t_dev(mid, h["a"], h["b"], h["c"], 1, HD, seq, 1)
    gpu.map_attn_softmax_value_dev(mid, h["c"], h["vals"], h["out"], 1, seq, HD, 0.125, 50.0)
    gpu.map_rope_dev(mid, h["rs"], h["rd"], 1, 1, HD, pos, 1000000.0)
    gpu.map_rmsnorm_x_dev(mid, wmap, h["ns"], h["nw"], h["nd"], 1, HD, 1e-6)
    gpu.map_op2_dev(mid, A.OP_ADD, h["e_src"], h["e_dst"], h["e_dst"], min(seq, HD))
    gpu.batch_end()


def _plan_ops(mid, wmap, h):
    P, S = A.DECODE_RUNTIME_POS, A.DECODE_RUNTIME_SEQ_LEN
    Op = A.DecodePlanOp
    return [
        Op(kind=A.DECODE_OP_QK_NORM_ROPE_X, map_id=mid, map_id2=wmap, h0=h["q"], h1=h["qw"], h2=h["k"], h3=h["kw"], h4=h["qk"],
           u0=1, u1=HD, u2=1, u3=HD, u4=P, f0=10000.0),
        Op(kind=A.DECODE_OP_ROW_COPY_OFFSET, map_id=mid, h0=h["kspec"], h1=h["kbase"], u0=P, u1=1, u2=HD),
        Op(kind=A.DECODE_OP_ROW_COPY_OFFSET, map_id=mid, h0=h["vspec"], h1=h["vbase"], u0=P, u1=1, u2=HD),
        Op(kind=A.DECODE_OP_MATMUL_T, map_id=mid, h0=h["a"], h1=h["b"], h2=h["c"], u0=1, u1=HD, u2=S, u3=1),
        Op(kind=A.DECODE_OP_ATTN_SOFTMAX_VALUE, map_id=mid, h0=h["c"], h1=h["vals"], h2=h["out"], u0=1, u1=S, u2=HD, f0=0.125, f1=50.0),
        Op(kind=A.DECODE_OP_ROPE, map_id=mid, h0=h["rs"], h1=h["rd"], u0=1, u1=1, u2=HD, u3=P, f0=1000000.0),
        Op(kind=A.DECODE_OP_RMSNORM_X, map_id=mid, map_id2=wmap, h0=h["ns"], h1=h["nw"], h2=h["nd"], u0=1, u1=HD, f0=1e-6),
        # n = seq_len while it is below the handles' 64 locs (the reference test's use of the sentinel)
        Op(kind=A.DECODE_OP_OP2, map_id=mid, op_code=A.OP_ADD, h0=h["e_src"], h1=h["e_dst"], h2=h["e_dst"], u0=S),
    ]


def test_plan_runs_as_one_graph_and_matches_immediate_calls(gpu):
    rng = np.random.default_rng(5)
    PLAN, DIRECT, WMAP = 7, 6, 9
    for mid in (PLAN, DIRECT):
        gpu.map_create_typed(mid, A.DTYPE_F32, 1, N_EL)
    gpu.map_create_typed(WMAP, A.DTYPE_F32, 1, WMAP_N)
    gpu.scatter_contiguous(WMAP, 0, (1 + 0.1 * rng.standard_normal(WMAP_N)).astype(np.float32))
    h = _handles(gpu)
    gpu.register_decode_plan(2, _plan_ops(PLAN, WMAP, h))
    try:
        for i, pos in enumerate(range(0, HD)):                     # seq_len stays within the element-wise op's 64-loc handles
            x = rng.standard_normal(3 * HD).astype(np.float32)
            for mid in (PLAN, DIRECT):
                gpu.scatter_contiguous(mid, 0, x)
            seq = pos + 1
            gpu.reset_native_stats()
            gpu.decode_step(2, pos, seq)
            launched = gpu.get_native_stats()["dispatch_count"]
            _direct(gpu, DIRECT, WMAP, h, pos, seq)
            assert np.array_equal(_read_all(gpu, PLAN), _read_all(gpu, DIRECT)), f"step {i} (pos {pos})"
            info = gpu.decode_plan_info(2)
            if i == 0:
                assert not info["runs_as_graph"] and info["host_steps"] == 1       # the first step runs eagerly
            else:
                assert info["runs_as_graph"] and info["recordings"] == 1 and info["graph_steps"] == i
                assert info["graph_kernels"] == 8 and launched == 1 + 8            # the setter + the graph's kernels: two host launches
        assert gpu.device_error() == 0
    finally:
        gpu.clear_decode_plan(2)


def test_plan_is_recorded_again_when_the_sequence_outgrows_it(gpu):
    rng = np.random.default_rng(6)
    PLAN, DIRECT, WMAP = 7, 6, 9
    for mid in (PLAN, DIRECT):
        gpu.map_create_typed(mid, A.DTYPE_F32, 1, N_EL)
    gpu.map_create_typed(WMAP, A.DTYPE_F32, 1, WMAP_N)
    gpu.scatter_contiguous(WMAP, 0, (1 + 0.1 * rng.standard_normal(WMAP_N)).astype(np.float32))
    h = _handles(gpu)
    ops = _plan_ops(PLAN, WMAP, h)[:-1]                            # without the element-wise op bounded by its handles
    gpu.register_decode_plan(3, ops)
    try:
        for i, pos in enumerate(list(range(0, 6)) + list(range(252, 262)) + [300, 319]):
            x = rng.standard_normal(3 * HD).astype(np.float32)
            for mid in (PLAN, DIRECT):
                gpu.scatter_contiguous(mid, 0, x)
            gpu.decode_step(3, pos, pos + 1)
            gpu.batch_begin()
            d = h
            gpu.map_qk_norm_rope_x_dev(DIRECT, WMAP, d["q"], d["qw"], d["k"], d["kw"], d["qk"], 1, HD, 1, HD, pos, 10000.0)
            gpu.map_row_copy_offset_dev(DIRECT, d["kspec"], d["kbase"], pos, 1, HD)
            gpu.map_row_copy_offset_dev(DIRECT, d["vspec"], d["vbase"], pos, 1, HD)
            gpu.map_matmul_t_dev(DIRECT, d["a"], d["b"], d["c"], 1, HD, pos + 1, 1)
            gpu.map_attn_softmax_value_dev(DIRECT, d["c"], d["vals"], d["out"], 1, pos + 1, HD, 0.125, 50.0)
            gpu.map_rope_dev(DIRECT, d["rs"], d["rd"], 1, 1, HD, pos, 1000000.0)
            gpu.map_rmsnorm_x_dev(DIRECT, WMAP, d["ns"], d["nw"], d["nd"], 1, HD, 1e-6)
            gpu.batch_end()
            assert np.array_equal(_read_all(gpu, PLAN), _read_all(gpu, DIRECT)), f"pos {pos}"
        info = gpu.decode_plan_info(3)
        assert info["runs_as_graph"] and info["recordings"] == 2 and info["cap"] == 512 and info["host_steps"] == 1
        assert gpu.device_error() == 0
    finally:
        gpu.clear_decode_plan(3)


def test_plan_with_an_argument_that_has_no_runtime_form_falls_back_to_host_substitution(gpu):
    """A sentinel as the row width of an RMSNorm cannot be resolved on the device: the plan keeps the reference's host-side
    substitution and still gives the right values."""
    rng = np.random.default_rng(7)
    gpu.map_create_typed(7, A.DTYPE_F32, 1, 256)
    x = rng.standard_normal(64).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(64)).astype(np.float32)
    gpu.scatter_contiguous(7, 0, np.concatenate([x, w]))
    s, wh, d = _h(gpu, [0]), _h(gpu, [64]), _h(gpu, [128])
    gpu.register_decode_plan(4, [A.DecodePlanOp(kind=A.DECODE_OP_RMSNORM, map_id=7, h0=s, h1=wh, h2=d, u0=1, u1=A.DECODE_RUNTIME_SEQ_LEN, f0=1e-6)])
    try:
        for _ in range(3):
            gpu.decode_step(4, 0, 64)
        got = gpu.gather(7, np.arange(128, 192, dtype=np.uint32)).view(np.float32)
        want = x / np.sqrt(np.mean(x.astype(np.float64) ** 2) + 1e-6) * w
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)
        info = gpu.decode_plan_info(4)
        assert info["state"] == -1 and info["host_steps"] == 3 and info["graph_steps"] == 0
        assert gpu.device_error() == 0
    finally:
        gpu.clear_decode_plan(4)


def test_step_trace_needs_the_diagnostics_build(gpu):
    """The regular library compiles no trace stamps: the diagnostics entry point says so instead of returning zeros."""
    from adam_b200 import synth
    from adam_b200.config import tiny_gemma3
    from adam_b200.engine import ADAMEngine
    cfg = tiny_gemma3(n_layer=2)
    eng = ADAMEngine(gpu, cfg, synth.build_model(cfg, seed=3), kv_cap=64)
    try:
        with pytest.raises(RuntimeError, match="STEP_TRACE"):
            eng.step_trace(0)
    finally:
        eng.close()
