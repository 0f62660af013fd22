"""Backend operators against the known-answer vectors of the reference's own
backend tests (tests/test_decode_primitives.py, tests/test_q4_roundtrip.py) and
against the numpy oracle.  All calls go through the C ABI."""
import os

import numpy as np
import pytest

import adam_b200 as A
from oracle import decoder as od
from oracle import q4_blocks

pytestmark = pytest.mark.gpu


def _f32map(gpu, mid, n, values=None):
    gpu.map_create_typed(mid, A.DTYPE_F32, 1, n)
    if values is not None:
        gpu.scatter(mid, np.arange(len(values), dtype=np.uint32), np.asarray(values, np.float32))


def _h(gpu, vals):
    return gpu.upload_dev(np.asarray(vals, np.uint32))[0]


def _read(gpu, mid, locs):
    return gpu.gather(mid, np.asarray(locs, np.uint32)).view(np.float32)


def test_scatter_gather_roundtrip_is_lossless(gpu):
    # tests/test_q4_roundtrip.py:74-90
    rng = np.random.default_rng(0)
    data = rng.standard_normal(1000).astype(np.float32)
    locs = rng.permutation(4096)[:1000].astype(np.uint32)
    _f32map(gpu, 2, 4096)
    gpu.scatter(2, locs, data)
    assert np.array_equal(_read(gpu, 2, locs), data)


def test_argmax_tie_goes_to_lower_index(gpu):
    # tests/test_decode_primitives.py:17-29
    logits = [-3.0, 5.5, 2.0, 5.5, 4.0, -1.0]
    _f32map(gpu, 8, 12, logits)
    src, dst = _h(gpu, np.arange(6)), _h(gpu, [10])
    gpu.map_argmax_dev(8, src, dst, 6)
    assert int(_read(gpu, 8, [10])[0]) == 1


def test_argmax_nan_and_large(gpu):
    rng = np.random.default_rng(1)
    v = rng.standard_normal(70000).astype(np.float32)
    v[123] = np.nan
    v[60001] = 9.0
    _f32map(gpu, 8, 70010, v)
    src, dst = _h(gpu, np.arange(70000)), _h(gpu, [70005])
    gpu.map_argmax_dev(8, src, dst, 70000)
    assert int(_read(gpu, 8, [70005])[0]) == 60001


def test_resolve_idx(gpu):
    # tests/test_decode_primitives.py:63-95 (the resolve step)
    vals = np.zeros(32, np.float32)
    vals[4:8] = [11.0, 22.0, 33.0, 44.0]
    vals[8:10] = [2.0, 0.0]
    _f32map(gpu, 16, 32, vals)
    base, sel, dst = _h(gpu, [4]), _h(gpu, [8, 9]), _h(gpu, [12, 13])
    gpu.batch_begin()
    gpu.map_resolve_idx_dev(16, base, sel, dst, 2)
    gpu.batch_end()
    assert _read(gpu, 16, [12, 13]).astype(np.int32).tolist() == [33, 11]


def test_matvec_t_xq4_on_q4_map_identity(gpu):
    # tests/test_decode_primitives.py:355-381
    ws_id, wt_id, M, K, N = 15, 14, 1, 8, 4
    gpu.map_create_typed(wt_id, A.DTYPE_Q4, 1, K * N, 32)
    gpu.set_qparams(wt_id, np.array([1.0 / 15.0], np.float32), np.array([0.0], np.float32))
    gpu.scatter(wt_id, np.arange(K * N, dtype=np.uint32), np.eye(N, K, dtype=np.float32).flatten())
    gpu.set_dtype(A.DTYPE_F32)
    gpu.map_create(ws_id, 1, K + N + 4)
    gpu.scatter(ws_id, np.arange(K, dtype=np.uint32), np.ones(K, np.float32))
    a_h, b_h, c_h = _h(gpu, [0]), _h(gpu, [0]), _h(gpu, [K])
    gpu.batch_begin()
    gpu.map_matmul_t_xq4_dev(ws_id, wt_id, a_h, b_h, c_h, 1, K, N)
    gpu.batch_end()
    assert np.allclose(_read(gpu, ws_id, np.arange(K, K + N)), np.ones(N), atol=0.05)


def test_q4_map_scatter_gather_matches_reference_cpu_model(gpu, golden_dir):
    # tests/test_q4_roundtrip.py:33-63 run on the reference, stored as a fixture
    g = np.load(os.path.join(golden_dir, "q4map_model.npz"))
    data, scales, zeros = g["data"], g["scales"], g["zeros"]
    gpu.map_create_typed(14, A.DTYPE_Q4, 1, data.size, 32)
    gpu.set_qparams(14, scales, zeros)
    gpu.scatter(14, np.arange(data.size, dtype=np.uint32), data)
    out = _read(gpu, 14, np.arange(data.size))
    assert np.array_equal(out.view(np.uint32), g["deq"].view(np.uint32))
    # mat-vec over the Q4 map against the CPU model of the same storage
    K, N = 32 * 8, 5
    W = g["deq"][:N * K].reshape(N, K)
    x = np.random.default_rng(2).standard_normal(K).astype(np.float32)
    _f32map(gpu, 15, K + N, x)
    a_h, b_h, c_h = _h(gpu, [0]), _h(gpu, [0]), _h(gpu, [K])
    gpu.map_matmul_t_xq4_dev(15, 14, a_h, b_h, c_h, 1, K, N)
    y = _read(gpu, 15, np.arange(K, K + N))
    ref = W.astype(np.float64) @ x
    assert np.abs(y - ref).max() < 1e-5 * np.abs(ref).max() + 1e-6


def test_q4_packed_contiguous_upload(gpu):
    rng = np.random.default_rng(3)
    raw = __import__("adam_b200.gguf_blocks", fromlist=["x"]).random_q4_k_blocks(rng, 2, 512)
    codes, scales, zeros = q4_blocks.q4k_to_q4map_params(raw)
    gpu.map_create_typed(14, A.DTYPE_Q4, 1, codes.size, 32)
    gpu.set_qparams(14, scales, zeros)
    packed = (codes[0::2] | (codes[1::2] << 4)).astype(np.uint8)
    gpu.scatter_q4_packed_contiguous(14, 0, packed)
    out = _read(gpu, 14, np.arange(codes.size))
    ref = q4_blocks.dequant_q4_k(raw)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))     # Q4_K -> Q4 map is lossless
    with pytest.raises(RuntimeError, match="code -3"):
        gpu.scatter_q4_packed_contiguous(14, 1, packed[:4])            # odd start


def test_batch_gather_scatter_dev(gpu):
    # tests/test_decode_primitives.py:384-398
    _f32map(gpu, 0, 8, [9.0, -2.0, 7.0, 1.5])
    _f32map(gpu, 1, 8)
    src, dst = _h(gpu, np.arange(4)), _h(gpu, np.arange(4))
    gpu.batch_begin()
    gh, _, n, _ = gpu.map_gather_dev(0, src, 4)
    gpu.map_scatter_dev(1, dst, 4, gh)
    gpu.batch_end()
    assert n == 4
    assert np.allclose(_read(gpu, 1, np.arange(4)), [9.0, -2.0, 7.0, 1.5])
    assert np.allclose(gpu.download_dev(gh, 4), [9.0, -2.0, 7.0, 1.5])


def test_row_copy_offset(gpu):
    # tests/test_decode_primitives.py:401-420
    data = np.zeros(40, np.float32)
    data[:8] = [1.0, 2.0, 3.0, 4.0, 10.0, 20.0, 30.0, 40.0]
    _f32map(gpu, 2, 40, data)
    spec, base = _h(gpu, [0, 3, 1, 5]), _h(gpu, [0])
    gpu.batch_begin()
    gpu.map_row_copy_offset_dev(2, spec, base, 2, 2, 4)
    gpu.batch_end()
    assert np.allclose(_read(gpu, 2, list(range(20, 24)) + list(range(28, 32))), data[:8])


def test_row_copy_then_matmul_t_in_one_batch(gpu):
    # tests/test_decode_primitives.py:423-446
    gpu.fusion_enable(True)
    data = np.zeros(32, np.float32)
    data[:8] = [1.0, 2.0, 3.0, 4.0, 10.0, 20.0, 30.0, 40.0]
    data[8:12] = 1.0
    _f32map(gpu, 16, 32, data)
    spec, sb = _h(gpu, [0, 0, 1, 1]), _h(gpu, [0])
    a, b, c = _h(gpu, [8]), _h(gpu, [20]), _h(gpu, [12])
    gpu.batch_begin()
    gpu.map_row_copy_offset_dev(16, spec, sb, 5, 2, 4)
    gpu.map_matmul_t_dev(16, a, b, c, 1, 4, 2)
    gpu.batch_end()
    assert np.allclose(_read(gpu, 16, [12, 13]), [10.0, 100.0])


def test_op2_then_argmax_then_op1(gpu):
    # tests/test_decode_primitives.py:481-504
    _f32map(gpu, 12, 12, [1.0, 2.0, 3.0])
    src, dbl, win, neg = _h(gpu, [0, 1, 2]), _h(gpu, [4, 5, 6]), _h(gpu, [8]), _h(gpu, [9, 10, 11])
    gpu.batch_begin()
    gpu.map_op2_dev(12, A.OP_ADD, src, src, dbl, 3)
    gpu.map_argmax_dev(12, dbl, win, 3)
    gpu.batch_end()
    assert int(_read(gpu, 12, [8])[0]) == 2
    gpu.batch_begin()
    gpu.map_op1_dev(12, A.OP_NEG, src, neg, 3)
    gpu.batch_end()
    assert np.allclose(_read(gpu, 12, [9, 10, 11]), [-1.0, -2.0, -3.0])


def test_decode_plan_runtime_sentinels(gpu):
    # tests/test_decode_primitives.py:507-573
    seed = np.zeros(24, np.float32)
    seed[0:6] = [1.0, 2.0, 3.0, 10.0, 20.0, 30.0]
    _f32map(gpu, 6, 24, seed)
    _f32map(gpu, 7, 24, seed)
    src, dst, spec, base = _h(gpu, [0, 1, 2]), _h(gpu, [12, 13, 14]), _h(gpu, [1, 0]), _h(gpu, [0])
    gpu.batch_begin()
    gpu.map_op2_dev(6, A.OP_ADD, src, src, dst, 3)
    gpu.map_row_copy_offset_dev(6, spec, base, 8, 1, 3)
    gpu.batch_end()
    ops = [A.DecodePlanOp(kind=A.DECODE_OP_OP2, map_id=7, op_code=A.OP_ADD, h0=src, h1=src, h2=dst, u0=A.DECODE_RUNTIME_SEQ_LEN),
           A.DecodePlanOp(kind=A.DECODE_OP_ROW_COPY_OFFSET, map_id=7, h0=spec, h1=base, u0=A.DECODE_RUNTIME_POS, u1=1, u2=3)]
    try:
        gpu.register_decode_plan(1, ops)
        gpu.decode_step(1, pos=8, seq_len=3)
    finally:
        gpu.clear_decode_plan(1)
    for probe in ([8, 9, 10], [12, 13, 14]):
        assert np.allclose(_read(gpu, 6, probe), _read(gpu, 7, probe))
    assert np.allclose(_read(gpu, 7, [12, 13, 14]), [2.0, 4.0, 6.0])
    with pytest.raises(RuntimeError, match="code -4"):
        gpu.decode_step(1, 0, 1)


def test_rmsnorm_variants_match_oracle(gpu):
    rng = np.random.default_rng(4)
    dim, rows = 1152, 3
    x = rng.standard_normal((rows, dim)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(dim)).astype(np.float32)
    r = rng.standard_normal((rows, dim)).astype(np.float32)
    buf = np.concatenate([x.ravel(), w, r.ravel(), np.zeros(rows * dim, np.float32)])
    _f32map(gpu, 3, buf.size, buf)
    off_w, off_r, off_d = rows * dim, rows * dim + dim, rows * dim + dim + rows * dim
    src = _h(gpu, [i * dim for i in range(rows)]); wt = _h(gpu, [off_w] * rows)
    res = _h(gpu, [off_r + i * dim for i in range(rows)]); dst = _h(gpu, [off_d + i * dim for i in range(rows)])
    gpu.map_rmsnorm_dev(3, src, wt, dst, rows, dim, 1e-6)
    out = _read(gpu, 3, np.arange(off_d, off_d + rows * dim)).reshape(rows, dim)
    ref = np.stack([od.rms_norm(x[i], w, 1e-6) for i in range(rows)])
    assert np.abs(out - ref).max() < 2e-6 * np.abs(ref).max()
    gpu.map_rmsnorm_add_dev(3, src, wt, res, dst, rows, dim, 1e-6)
    out = _read(gpu, 3, np.arange(off_d, off_d + rows * dim)).reshape(rows, dim)
    assert np.abs(out - (ref + r)).max() < 2e-6 * np.abs(ref + r).max()
    # weights in a second map
    _f32map(gpu, 4, dim, w)
    wt2 = _h(gpu, [0] * rows)
    gpu.map_rmsnorm_x_dev(3, 4, src, wt2, dst, rows, dim, 1e-6)
    out = _read(gpu, 3, np.arange(off_d, off_d + rows * dim)).reshape(rows, dim)
    assert np.abs(out - ref).max() < 2e-6 * np.abs(ref).max()


@pytest.mark.parametrize("pos,base", [(0, 1e4), (17, 1e4), (255, 1e6), (2047, 1e4)])
def test_rope_and_qk_norm_rope_match_oracle(gpu, pos, base):
    rng = np.random.default_rng(pos)
    H, KV, hd = 4, 1, 256
    q = rng.standard_normal((H, hd)).astype(np.float32)
    k = rng.standard_normal((KV, hd)).astype(np.float32)
    qw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    kw = (1 + 0.1 * rng.standard_normal(hd)).astype(np.float32)
    buf = np.concatenate([q.ravel(), k.ravel(), np.zeros((H + KV) * hd, np.float32)])
    _f32map(gpu, 3, buf.size, buf)
    _f32map(gpu, 4, 2 * hd, np.concatenate([qw, kw]))
    qs, qwl = _h(gpu, [i * hd for i in range(H)]), _h(gpu, [0] * H)
    ks, kwl = _h(gpu, [H * hd + i * hd for i in range(KV)]), _h(gpu, [hd] * KV)
    off = (H + KV) * hd
    dst = _h(gpu, [off])
    gpu.map_qk_norm_rope_x_dev(3, 4, qs, qwl, ks, kwl, dst, H, hd, KV, hd, pos, base)
    out = _read(gpu, 3, np.arange(off, off + (H + KV) * hd)).reshape(H + KV, hd)
    qn = np.stack([od.rms_norm(q[i], qw, 1e-6) for i in range(H)])
    kn = np.stack([od.rms_norm(k[i], kw, 1e-6) for i in range(KV)])
    ref = np.concatenate([od.rope_half(qn, pos, base), od.rope_half(kn, pos, base)])
    # This operator receives only freq_base, so the angle pos*base^(-2i/d) is formed
    # on the device; numpy's float32 pow is a few ulp off the correctly rounded
    # value and the angle error grows with pos.  (The fused decoder takes the
    # host-made angle table instead and is held to a tighter bound.)
    tol = (3e-6 + 4e-7 * pos) * np.abs(ref).max()
    assert np.abs(out - ref).max() < tol
    # plain rope over [tokens=1, heads, hd]
    src1, dst1 = _h(gpu, [0]), _h(gpu, [off])
    gpu.map_rope_dev(3, src1, dst1, 1, H, hd, pos, base)
    out = _read(gpu, 3, np.arange(off, off + H * hd)).reshape(H, hd)
    assert np.abs(out - od.rope_half(q, pos, base)).max() < (3e-6 + 4e-7 * pos) * np.abs(q).max()


def test_attention_ops_match_oracle(gpu):
    rng = np.random.default_rng(6)
    H, hd, seq, cap_rows = 4, 64, 37, 48
    q = rng.standard_normal((H, hd)).astype(np.float32)
    Kc = rng.standard_normal((cap_rows, hd)).astype(np.float32)
    Vc = rng.standard_normal((cap_rows, hd)).astype(np.float32)
    o_q, o_k, o_v = 0, H * hd, H * hd + cap_rows * hd
    o_s = o_v + cap_rows * hd
    o_o = o_s + H * cap_rows
    buf = np.zeros(o_o + H * hd, np.float32)
    buf[o_q:o_k] = q.ravel(); buf[o_k:o_v] = Kc.ravel(); buf[o_v:o_s] = Vc.ravel()
    _f32map(gpu, 3, buf.size, buf)
    a = _h(gpu, [o_q + h * hd for h in range(H)]); b = _h(gpu, [o_k] * H); c = _h(gpu, [o_s + h * cap_rows for h in range(H)])
    v = _h(gpu, [o_v] * H); o = _h(gpu, [o_o + h * hd for h in range(H)])
    scale = np.float32(1 / np.sqrt(hd))
    gpu.batch_begin()
    gpu.map_matmul_t_dev(3, a, b, c, 1, hd, seq, H)
    gpu.map_attn_softmax_value_dev(3, c, v, o, H, seq, hd, float(scale), 50.0)
    gpu.batch_end()
    out = _read(gpu, 3, np.arange(o_o, o_o + H * hd)).reshape(H, hd)
    ref = np.stack([od.attention_head(q[h], Kc[:seq], Vc[:seq], scale, 50.0) for h in range(H)])
    assert np.abs(out - ref).max() < 5e-6 * np.abs(ref).max() + 1e-6


def test_geglu_broadcast_and_softcap_ops(gpu):
    rng = np.random.default_rng(8)
    n = 6912
    gte = (3 * rng.standard_normal(n)).astype(np.float32)
    up = rng.standard_normal(n).astype(np.float32)
    buf = np.concatenate([gte, up, np.zeros(n, np.float32), np.array([30.0], np.float32)])
    _f32map(gpu, 3, buf.size, buf)
    la, lb, ld = _h(gpu, np.arange(n)), _h(gpu, np.arange(n, 2 * n)), _h(gpu, np.arange(2 * n, 3 * n))
    gpu.map_op2_dev(3, A.OP_GEGLU, la, lb, ld, n)
    out = _read(gpu, 3, np.arange(2 * n, 3 * n))
    ref = od.gelu_tanh(gte) * up
    assert np.abs(out - ref).max() < 2e-6 * np.abs(ref).max()
    # final soft-cap chain: x / cap -> tanh -> * cap  (engine.py:3517-3521)
    cap = _h(gpu, np.full(n, 3 * n))
    gpu.batch_begin()
    gpu.map_broadcast_dev(3, A.BROADCAST_DIV, la, cap, ld, n)
    gpu.map_op1_dev(3, A.OP_TANH, ld, ld, n)
    gpu.map_broadcast_dev(3, A.BROADCAST_MUL, ld, cap, ld, n)
    gpu.batch_end()
    out = _read(gpu, 3, np.arange(2 * n, 3 * n))
    ref = np.tanh(gte / np.float32(30)) * np.float32(30)
    assert np.abs(out - ref).max() < 3e-6 * 30


def test_out_of_range_loc_is_reported_not_faulted(gpu):
    _f32map(gpu, 3, 16, np.arange(16))
    bad, dst = _h(gpu, [3, 99]), _h(gpu, [0, 1])
    gpu.map_op1_dev(3, A.OP_NEG, bad, dst, 2)
    assert gpu.device_error() & 1
    assert gpu.device_error() == 0
    assert _read(gpu, 3, [0])[0] == -3.0


def test_off_path_symbols_return_invalid(gpu):
    assert gpu._lib.map_fma_dev(0, 0, 0, 0, 0, 0) == -3


def test_topk_reference_vector(gpu):
    """tests/test_decode_primitives.py:32-47 (ties to the lower index, indices as float32)."""
    _f32map(gpu, 3, 20, [-3.0, 5.5, 2.0, 5.5, 4.0, -1.0])
    src, idx, val = _h(gpu, np.arange(6)), _h(gpu, [8, 9, 10]), _h(gpu, [12, 13, 14])
    gpu.map_topk_dev(3, src, idx, val, 6, 3)
    assert _read(gpu, 3, [8, 9, 10]).astype(np.int32).tolist() == [1, 3, 4]
    assert np.allclose(_read(gpu, 3, [12, 13, 14]), [5.5, 5.5, 4.0], atol=1e-6)
    # NaN counts as the lowest value; k beyond 64 is refused
    _f32map(gpu, 3, 20, [np.nan, 1.0, np.nan, 0.5])
    gpu.map_topk_dev(3, _h(gpu, np.arange(4)), idx, val, 4, 3)
    assert _read(gpu, 3, [8, 9, 10]).astype(np.int32).tolist() == [1, 3, 0]
    assert gpu._lib.map_topk_dev(3, src, idx, val, 6, 65) == -3
    # against numpy on a larger input
    rng = np.random.default_rng(0)
    x = rng.standard_normal(5000).astype(np.float32)
    _f32map(gpu, 3, 5200, x)
    idx, val = _h(gpu, 5000 + np.arange(64)), _h(gpu, 5100 + np.arange(64))
    gpu.map_topk_dev(3, _h(gpu, np.arange(5000)), idx, val, 5000, 64)
    order = np.argsort(-x, kind="stable")[:64]
    assert _read(gpu, 3, 5000 + np.arange(64)).astype(np.int64).tolist() == order.tolist()
    assert np.array_equal(_read(gpu, 3, 5100 + np.arange(64)), x[order])


def test_topp_reference_vector(gpu):
    """tests/test_decode_primitives.py:50-63."""
    _f32map(gpu, 3, 16, [5.0, 4.0, 1.0, -1.0])
    gpu.map_topp_dev(3, _h(gpu, [0, 1, 2, 3]), _h(gpu, [8, 9, 10, 11]), 4, 1.0, 0.9)
    assert np.allclose(_read(gpu, 3, [8, 9, 10, 11]), [0.7310586, 0.26894143, 0.0, 0.0], atol=1e-5)
    # temperature sharpens the soft-max before the cut: at 0.5 the first two candidates reach 0.99
    gpu.map_topp_dev(3, _h(gpu, [0, 1, 2, 3]), _h(gpu, [8, 9, 10, 11]), 4, 0.5, 0.99)
    z = np.exp((np.array([5.0, 4.0, 1.0, -1.0]) - 5.0) / 0.5)
    assert np.allclose(_read(gpu, 3, [8, 9, 10, 11]), [z[0] / (z[0] + z[1]), z[1] / (z[0] + z[1]), 0.0, 0.0], atol=1e-6)
    # the shader leaves its loop at the first candidate when top_p >= 0.999999 (map_topp.comp:78-81): kept as is
    gpu.map_topp_dev(3, _h(gpu, [0, 1, 2, 3]), _h(gpu, [8, 9, 10, 11]), 4, 1.0, 1.0)
    assert _read(gpu, 3, [8, 9, 10, 11]).tolist() == [1.0, 0.0, 0.0, 0.0]
    assert gpu._lib.map_topp_dev(3, 1, 1, 65, 1.0, 0.9) == -3


def test_resolve_idx_and_categorical_reference_vector(gpu):
    """tests/test_decode_primitives.py:66-101: candidates 33 and 11 with p = (0.25, 0.75), r = 0.6 -> 11."""
    vals = np.zeros(32, np.float32)
    vals[4:8] = [11.0, 22.0, 33.0, 44.0]
    vals[8:10] = [2.0, 0.0]
    vals[16:18] = [0.25, 0.75]
    vals[20] = 0.6
    _f32map(gpu, 3, 32, vals)
    base = gpu.upload_dev(np.array([4], np.uint32))[0]
    gpu.map_resolve_idx_dev(3, base, _h(gpu, [8, 9]), _h(gpu, [12, 13]), 2)
    gpu.map_sample_categorical_dev(3, _h(gpu, [12, 13]), _h(gpu, [16, 17]), _h(gpu, [20]), _h(gpu, [21]), 2)
    assert _read(gpu, 3, [12, 13]).astype(np.int32).tolist() == [33, 11]
    assert int(_read(gpu, 3, [21])[0]) == 11
    # r below the first probability picks the first candidate; all-zero probabilities fall back to it too
    gpu.scatter(3, np.array([20], np.uint32), np.array([0.1], np.float32))
    gpu.map_sample_categorical_dev(3, _h(gpu, [12, 13]), _h(gpu, [16, 17]), _h(gpu, [20]), _h(gpu, [21]), 2)
    assert int(_read(gpu, 3, [21])[0]) == 33
    gpu.map_sample_categorical_dev(3, _h(gpu, [12, 13]), _h(gpu, [30, 31]), _h(gpu, [20]), _h(gpu, [21]), 2)
    assert int(_read(gpu, 3, [21])[0]) == 33


def test_repeat_penalty(gpu):
    """map_repeat_penalty.comp: positive logits are divided, the others multiplied; ids index the loc list."""
    _f32map(gpu, 3, 8, [2.0, -2.0, 0.0, 4.0, 1.0, 1.0, 1.0, 1.0])
    ids = gpu.upload_dev(np.array([0, 1, 3], np.uint32))[0]
    gpu.map_repeat_penalty_dev(3, _h(gpu, np.arange(8)), ids, 3, 2.0)
    assert _read(gpu, 3, np.arange(8)).tolist() == [1.0, -4.0, 0.0, 2.0, 1.0, 1.0, 1.0, 1.0]
    bad = gpu.upload_dev(np.array([99], np.uint32))[0]
    gpu.map_repeat_penalty_dev(3, _h(gpu, np.arange(8)), bad, 1, 2.0)
    assert gpu.device_error() & 1


def test_native_stats_count_launches(gpu):
    _f32map(gpu, 3, 16, np.arange(16))
    a = _h(gpu, [0, 1])
    gpu.reset_native_stats()
    gpu.batch_begin()
    for _ in range(5):
        gpu.map_op1_dev(3, A.OP_NEG, a, a, 2)
    gpu.batch_end()
    st = gpu.get_native_stats()
    assert st["dispatch_count"] == 5 and st["submit_count"] == 1 and st["scheduler_mode_name"] == "level_batched"


def test_matvec_topk_reference_vector(gpu):
    """tests/test_decode_primitives.py:260-301: rows diag(1,2,3,4) in a Q4 map, x = ones, row 3 penalised by 2:
    the two best are row 2 (3.0) and one of rows 1 / 3 (2.0)."""
    gpu.map_create_typed(13, A.DTYPE_Q4, 1, 16, 32)
    gpu.set_qparams(13, np.array([4.0 / 15.0], np.float32), np.array([0.0], np.float32))
    gpu.scatter(13, np.arange(16, dtype=np.uint32), np.diag([1.0, 2.0, 3.0, 4.0]).astype(np.float32).reshape(-1))
    _f32map(gpu, 14, 16, [1.0, 1.0, 1.0, 1.0])
    a_h, b_h, pen = _h(gpu, [0]), _h(gpu, [0]), _h(gpu, [3])
    idx, val = _h(gpu, [4, 5]), _h(gpu, [8, 9])
    gpu.batch_begin()
    gpu.map_matvec_topk_t_xq4_dev(14, 13, a_h, b_h, pen, idx, val, 4, 4, 2, 1, 2.0)
    gpu.batch_end()
    got_i = _read(gpu, 14, [4, 5]).astype(np.int32)
    assert got_i[0] == 2 and got_i[1] in (1, 3)
    assert np.allclose(_read(gpu, 14, [8, 9]), [3.0, 2.0], atol=0.15)
    assert gpu._lib.map_matvec_topk_t_xq4_dev(14, 13, a_h, b_h, pen, idx, val, 4, 4, 65, 1, 2.0) == -3      # k beyond 64


def test_matvec_topk_groups_match_numpy_on_gguf_blocks(gpu):
    """Partial top-k per group of rows over a GGUF Q4_0 matrix (tensor-core GEMV underneath): every group's list
    equals numpy's on the product of the decoded weights after the penalty; groups that hold fewer than k rows
    are padded with (0, -FLT_MAX) as the reference shader does."""
    from adam_b200 import gguf_blocks as gb
    rng = np.random.default_rng(17)
    N, K, k, rpg = 1000, 256, 7, 96
    raw = gb.random_q4_0_blocks(rng, N, K)
    gpu.map_create_typed(13, A.DTYPE_GGUF_Q4_0, 1, N * K)
    gpu.upload_gguf_blocks(13, 2, 0, raw)
    x = rng.standard_normal(K).astype(np.float32)
    groups = (N + rpg - 1) // rpg
    _f32map(gpu, 14, K + 2 * groups * k + 8, x)
    pen_ids = [5, 97, 500, 999]
    a_h, b_h, pen = _h(gpu, [0]), _h(gpu, [0]), _h(gpu, pen_ids)
    il, vl = K + np.arange(groups * k), K + groups * k + np.arange(groups * k)
    gpu.batch_begin()
    gpu.map_matvec_topk_t_xq4_ex_dev(14, 13, a_h, b_h, pen, _h(gpu, il), _h(gpu, vl), K, N, k, len(pen_ids), 1.7, rpg)
    gpu.batch_end()
    got_i = _read(gpu, 14, il).astype(np.int64).reshape(groups, k)
    got_v = _read(gpu, 14, vl).reshape(groups, k)
    y = (q4_blocks.dequant(raw.reshape(-1), 2, N, K).astype(np.float64) @ x).astype(np.float32)
    for t in pen_ids:
        y[t] = y[t] / np.float32(1.7) if y[t] > 0 else y[t] * np.float32(1.7)
    for g_ in range(groups):
        r0, r1 = g_ * rpg, min(N, (g_ + 1) * rpg)
        order = r0 + np.argsort(-y[r0:r1], kind="stable")[:k]
        n = len(order)
        assert got_i[g_, :n].tolist() == order.tolist()
        assert np.allclose(got_v[g_, :n], y[order], rtol=1e-4, atol=1e-5)
        assert (got_i[g_, n:] == 0).all() and (got_v[g_, n:] < -3e38).all()
    assert gpu.device_error() == 0
