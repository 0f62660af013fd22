// Operators of the reference backend's decode path, addressed through maps and
// loc handles exactly as the reference's C entry points are (one launch per
// call, on the context stream).  Each kernel names the reference shader whose
// behaviour it provides; arithmetic follows the reference's numpy decoder where
// the two differ (division by the RMS instead of a reciprocal multiply).
#include "common.cuh"
#include "gemv.cuh"
#include "gemv_mma.cuh"
#include "gemm_tc.cuh"
#include "blocks8.cuh"

#include <cstring>
#include <initializer_list>

namespace ab {

#define OOB(idx, n, err) if ((uint64_t)(idx) >= (n)) { atomicOr((err), DEVERR_OOB_MAP); return; }

// Decode-plan runtime arguments.  While a registered plan is lowered to a CUDA graph, an argument that holds one of the
// two sentinels (ADAMAH_DECODE_RUNTIME_POS / _SEQ_LEN) is handed to its kernel as it is, together with `rt`, the
// device address of {pos, seq_len}; the kernel resolves it when it runs, so one instantiated graph serves every step.
// rt == NULL: immediate call, values are what they say.
__device__ __forceinline__ uint32_t rtv(uint32_t v, const uint32_t* __restrict__ rt) {
    if (!rt) return v;
    return v == ADAMAH_DECODE_RUNTIME_POS ? rt[0] : (v == ADAMAH_DECODE_RUNTIME_SEQ_LEN ? rt[1] : v);
}
__global__ void k_set_runtime(uint32_t* rt, uint32_t pos, uint32_t seq_len) { rt[0] = pos; rt[1] = seq_len; }

// dst = (x / sqrt(mean(x^2) + eps)) * w  [+ resid]; one CTA per row.
// map_rmsnorm.comp / map_rmsnorm_x.comp / map_rmsnorm_add.comp.
__global__ void k_rmsnorm(float* __restrict__ act, uint64_t n_act, const float* __restrict__ wt, uint64_t n_wt,
                          const uint32_t* __restrict__ l_src, const uint32_t* __restrict__ l_wt,
                          const uint32_t* __restrict__ l_res, const uint32_t* __restrict__ l_dst,
                          uint32_t dim, float eps, uint32_t* err, uint32_t n_rows, const uint32_t* __restrict__ rt) {
    __shared__ float red[33];
    const uint32_t r = blockIdx.x;
    if (r >= rtv(n_rows, rt)) return;
    const uint64_t sb = l_src[r], wb = l_wt[r], db = l_dst[r], rb = l_res ? l_res[r] : 0;
    if (sb + dim > n_act || db + dim > n_act || wb + dim > n_wt || (l_res && rb + dim > n_act)) {
        if (threadIdx.x == 0) atomicOr(err, DEVERR_OOB_MAP);
        return;
    }
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) { float x = act[sb + i]; ss = fmaf(x, x, ss); }
    ss = block_sum(ss, red);
    const float rms = sqrtf(ss / (float)dim + eps);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = __fdiv_rn(act[sb + i], rms) * wt[wb + i];
        if (l_res) v += act[rb + i];
        act[db + i] = v;
    }
}

// Rotation angle table entry as the numpy decoder computes it
// (tests/diagnostics/diag_inference.py:948-954): float32 frequency, float32
// angle, then cos/sin of that float32 angle (evaluated in double, rounded once).
__device__ __forceinline__ void rope_cs(uint32_t pos, uint32_t i, uint32_t head_dim, float base, float& c, float& s) {
    const float e = (float)i * 2.0f / (float)head_dim;
    const float freq = 1.0f / (float)pow((double)base, (double)e);
    const float theta = (float)pos * freq;
    double sd, cd;
    sincos((double)theta, &sd, &cd);
    c = (float)cd; s = (float)sd;
}

// map_rope.comp: rotate pairs (d, d+half) of every head of every token.
__global__ void k_rope(float* __restrict__ m, uint64_t n, const uint32_t* __restrict__ l_src, const uint32_t* __restrict__ l_dst,
                       uint32_t n_tokens, uint32_t n_heads, uint32_t head_dim, uint32_t pos_offset, float base, uint32_t* err,
                       const uint32_t* __restrict__ rt) {
    n_tokens = rtv(n_tokens, rt); pos_offset = rtv(pos_offset, rt);
    const uint32_t half = head_dim / 2;
    const uint32_t pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair >= n_tokens * n_heads * half) return;
    const uint32_t tok = pair / (n_heads * half), rem = pair % (n_heads * half), head = rem / half, d = rem % half;
    float c, s;
    rope_cs(pos_offset + tok, d, head_dim, base, c, s);
    const uint64_t bs = (uint64_t)l_src[tok] + head * head_dim, bd = (uint64_t)l_dst[tok] + head * head_dim;
    OOB(bs + d + half, n, err); OOB(bd + d + half, n, err);
    const float x0 = m[bs + d], x1 = m[bs + d + half];
    m[bd + d] = x0 * c - x1 * s;
    m[bd + d + half] = x0 * s + x1 * c;
}

// map_qk_norm_rope_x.comp: per-head RMSNorm (eps 1e-6 as the shader hard-codes,
// equal to the model's norm_eps) then half-split RoPE, written to a contiguous
// q+k span.  One CTA per row.
__global__ void k_qk_norm_rope(float* __restrict__ act, uint64_t n_act, const float* __restrict__ wt, uint64_t n_wt,
                               const uint32_t* __restrict__ l_qs, const uint32_t* __restrict__ l_qw,
                               const uint32_t* __restrict__ l_ks, const uint32_t* __restrict__ l_kw,
                               const uint32_t* __restrict__ l_dst, uint32_t q_rows, uint32_t q_dim, uint32_t k_rows, uint32_t k_dim,
                               uint32_t pos, float base, uint32_t* err, const uint32_t* __restrict__ rt) {
    __shared__ float red[33];
    pos = rtv(pos, rt);
    const uint32_t row = blockIdx.x;
    const bool is_q = row < q_rows;
    const uint32_t lr = is_q ? row : row - q_rows, dim = is_q ? q_dim : k_dim, half = dim / 2;
    const uint64_t sb = is_q ? l_qs[lr] : l_ks[lr], wb = is_q ? l_qw[lr] : l_kw[lr];
    const uint64_t db = (uint64_t)l_dst[0] + (is_q ? (uint64_t)lr * q_dim : (uint64_t)q_rows * q_dim + (uint64_t)lr * k_dim);
    if (sb + dim > n_act || db + dim > n_act || wb + dim > n_wt) { if (threadIdx.x == 0) atomicOr(err, DEVERR_OOB_MAP); return; }
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) { float x = act[sb + i]; ss = fmaf(x, x, ss); }
    ss = block_sum(ss, red);
    const float rms = sqrtf(ss / (float)dim + 1e-6f);
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
        const float y0 = __fdiv_rn(act[sb + i], rms) * wt[wb + i];
        const float y1 = __fdiv_rn(act[sb + i + half], rms) * wt[wb + i + half];
        float c, s;
        rope_cs(pos, i, dim, base, c, s);
        __syncwarp();
        act[db + i] = y0 * c - y1 * s;
        act[db + i + half] = y0 * s + y1 * c;
    }
}

// map_row_copy.comp: copy_spec holds [src_row, dst_row] pairs.
__global__ void k_row_copy(float* __restrict__ m, uint64_t n, const uint32_t* __restrict__ spec, const uint32_t* __restrict__ src_base,
                           uint32_t dst_row_offset, uint32_t n_copies, uint32_t row_size, uint32_t* err, const uint32_t* __restrict__ rt) {
    dst_row_offset = rtv(dst_row_offset, rt); n_copies = rtv(n_copies, rt);
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= (uint64_t)n_copies * row_size) return;
    const uint32_t ci = (uint32_t)(tid / row_size), ei = (uint32_t)(tid % row_size);
    const uint64_t so = (uint64_t)src_base[0] + (uint64_t)spec[2 * ci] * row_size + ei;
    const uint64_t dd = ((uint64_t)spec[2 * ci + 1] + dst_row_offset) * row_size + ei;
    OOB(so, n, err); OOB(dd, n, err);
    m[dd] = m[so];
}

// map_matmul_t.comp: C[op][row][col] = sum_k A[op][row][k] * B[op][col][k]; a warp per output.
__global__ void k_matmul_t(float* __restrict__ m, uint64_t n, const uint32_t* __restrict__ la, const uint32_t* __restrict__ lb,
                           const uint32_t* __restrict__ lc, uint32_t M, uint32_t K, uint32_t N, uint32_t* err, const uint32_t* __restrict__ rt) {
    M = rtv(M, rt); K = rtv(K, rt); N = rtv(N, rt);
    const uint32_t op = blockIdx.z, row = blockIdx.y;
    const uint32_t col = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (col >= N || row >= M) return;
    const uint64_t ab_ = (uint64_t)la[op] + (uint64_t)row * K, bb = (uint64_t)lb[op] + (uint64_t)col * K;
    const uint64_t cb = (uint64_t)lc[op] + (uint64_t)row * N + col;
    if (ab_ + K > n || bb + K > n || cb >= n) { if (lane == 0) atomicOr(err, DEVERR_OOB_MAP); return; }
    float s = 0.f;
    for (uint32_t k = lane; k < K; k += 32) s = fmaf(m[ab_ + k], m[bb + k], s);
    s = warp_sum(s);
    if (lane == 0) m[cb] = s;
}

// map_attn_softmax_value.comp: p = softmax(cap*tanh(score*scale/cap)); out = p @ V.
__global__ void k_attn_softmax_value(float* __restrict__ m, uint64_t n, const uint32_t* __restrict__ l_sc, const uint32_t* __restrict__ l_v,
                                     const uint32_t* __restrict__ l_out, uint32_t row_size, uint32_t value_dim, float scale, float cap,
                                     uint32_t* err, uint32_t smem_rows, const uint32_t* __restrict__ rt) {
    extern __shared__ float prob[];
    __shared__ float red[33];
    row_size = rtv(row_size, rt);
    if (row_size > smem_rows) { if (threadIdx.x == 0) atomicOr(err, DEVERR_OOB_MAP); return; }      // beyond what the graph was sized for
    const uint32_t op = blockIdx.x;
    const uint64_t sb = l_sc[op], vb = l_v[op], ob = l_out[op];
    if (sb + row_size > n || vb + (uint64_t)row_size * value_dim > n || ob + value_dim > n) { if (threadIdx.x == 0) atomicOr(err, DEVERR_OOB_MAP); return; }
    float mx = -3.402823466e+38f;
    for (uint32_t t = threadIdx.x; t < row_size; t += blockDim.x) {
        float v = m[sb + t] * scale;
        if (cap > 0.f) v = tanhf(v / cap) * cap;
        prob[t] = v;
        mx = fmaxf(mx, v);
    }
    mx = block_max(mx, red);
    float sum = 0.f;
    for (uint32_t t = threadIdx.x; t < row_size; t += blockDim.x) { float p = expf(prob[t] - mx); prob[t] = p; sum += p; }
    sum = block_sum(sum, red);
    for (uint32_t t = threadIdx.x; t < row_size; t += blockDim.x) prob[t] = prob[t] / sum;
    __syncthreads();
    for (uint32_t d = threadIdx.x; d < value_dim; d += blockDim.x) {
        float acc = 0.f;
        for (uint32_t t = 0; t < row_size; ++t) acc = fmaf(prob[t], m[vb + (uint64_t)t * value_dim + d], acc);
        m[ob + d] = acc;
    }
}

__device__ float op1_eval(uint32_t op, float v) {
    switch (op) {                       // map_op1.comp
    case 0: return -v;
    case 1: return fabsf(v);
    case 2: return sqrtf(fmaxf(v, 0.f));
    case 3: return expf(v);
    case 4: return logf(fmaxf(v, 1e-7f));
    case 5: return tanhf(v);
    case 6: return fmaxf(0.f, v);
    case 7: return gelu_tanh(v);
    case 8: return sinf(v);
    case 9: return cosf(v);
    case 10: return tanf(v);
    case 11: return asinf(fminf(fmaxf(v, -1.f), 1.f));
    case 12: return acosf(fminf(fmaxf(v, -1.f), 1.f));
    case 13: return atanf(v);
    case 14: return sinhf(v);
    case 15: return coshf(v);
    case 16: return 1.f / (1.f + expf(-v));
    case 17: return v / (1.f + expf(-v));
    case 18: return v * tanhf(logf(1.f + expf(v)));
    case 19: return 1.05069995f * (v > 0.f ? v : 1.67325997f * (expf(v) - 1.f));
    case 20: return v > 0.f ? v : expf(v) - 1.f;
    case 21: return fmaxf(v, 0.01f * v);
    case 22: return ceilf(v);
    case 23: return floorf(v);
    case 24: return roundf(v);
    case 25: return v > 0.f ? 1.f : (v < 0.f ? -1.f : 0.f);
    case 26: return 1.f / v;
    case 27: return v * v;
    case 28: return v * v * v;
    case 29: return logf(1.f + expf(v));
    case 30: return fminf(fmaxf(0.2f * v + 0.5f, 0.f), 1.f);
    case 31: return v * fminf(fmaxf(0.2f * v + 0.5f, 0.f), 1.f);
    case 32: return expf(v) - 1.f;
    case 33: return logf(1.f + v);
    default: return v;
    }
}

__device__ float op2_eval(uint32_t op, float a, float b) {
    switch (op) {                       // map_op2.comp
    case 0: return a + b;
    case 1: return a - b;
    case 2: return a * b;
    case 3: return a / b;
    case 4: return powf(a, b);
    case 5: return fminf(a, b);
    case 6: return fmaxf(a, b);
    case 7: return fmodf(a, b);
    case 8: return a == b ? 1.f : 0.f;
    case 9: return a != b ? 1.f : 0.f;
    case 10: return a < b ? 1.f : 0.f;
    case 11: return a <= b ? 1.f : 0.f;
    case 12: return a > b ? 1.f : 0.f;
    case 13: return a >= b ? 1.f : 0.f;
    case 14: return (a != 0.f && b != 0.f) ? 1.f : 0.f;
    case 15: return (a != 0.f || b != 0.f) ? 1.f : 0.f;
    case 16: return ((a != 0.f) != (b != 0.f)) ? 1.f : 0.f;
    case 17: return atan2f(a, b);
    case 34: return gelu_tanh(a) * b;   // GeGLU
    case 35: return silu_clip(a) * b;   // SwiGLU
    default: return a;
    }
}

__global__ void k_op1(float* __restrict__ m, uint64_t n_el, uint32_t op, const uint32_t* __restrict__ ls, const uint32_t* __restrict__ ld,
                      uint32_t n, uint32_t* err, const uint32_t* __restrict__ rt) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rtv(n, rt)) return;
    const uint64_t s = ls[i], d = ld[i];
    OOB(s, n_el, err); OOB(d, n_el, err);
    m[d] = op1_eval(op, m[s]);
}
__global__ void k_op2(float* __restrict__ m, uint64_t n_el, uint32_t op, const uint32_t* __restrict__ la, const uint32_t* __restrict__ lb,
                      const uint32_t* __restrict__ ld, uint32_t n, uint32_t* err, const uint32_t* __restrict__ rt) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rtv(n, rt)) return;
    const uint64_t a = la[i], b = lb[i], d = ld[i];
    OOB(a, n_el, err); OOB(b, n_el, err); OOB(d, n_el, err);
    m[d] = op2_eval(op, m[a], m[b]);
}
// map_broadcast.comp: dst[i] = src[i] (op) scalar[i]
__global__ void k_broadcast(float* __restrict__ m, uint64_t n_el, uint32_t op, const uint32_t* __restrict__ ls, const uint32_t* __restrict__ lsc,
                            const uint32_t* __restrict__ ld, uint32_t n, uint32_t* err, const uint32_t* __restrict__ rt) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rtv(n, rt)) return;
    const uint64_t s = ls[i], c = lsc[i], d = ld[i];
    OOB(s, n_el, err); OOB(c, n_el, err); OOB(d, n_el, err);
    const float v = m[s], k = m[c];
    m[d] = op == 0 ? v * k : op == 1 ? v / k : op == 2 ? v + k : v - k;
}

// map_argmax.comp: index (into the loc list) of the maximum, ties to the lower
// index, NaN treated as -FLT_MAX; stored as float32.
__global__ void k_argmax(float* __restrict__ m, uint64_t n_el, const uint32_t* __restrict__ ls, const uint32_t* __restrict__ ld, uint32_t n, uint32_t* err) {
    __shared__ float sv[32];
    __shared__ int si[32];
    float bv = -3.402823466e+38f; int bi = -1;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const uint64_t s = ls[i];
        if (s >= n_el) { atomicOr(err, DEVERR_OOB_MAP); continue; }
        float v = m[s];
        if (!(v == v)) v = -3.402823466e+38f;
        if (better(v, (int)i, bv, bi)) { bv = v; bi = (int)i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
        const uint64_t d = ld[0];
        if (d >= n_el) { atomicOr(err, DEVERR_OOB_MAP); return; }
        m[d] = (float)(bi < 0 ? 0 : bi);
    }
}

// ---- sampled-decoding tail (map_topk.comp, map_topp.comp, map_sample_categorical.comp,
// map_repeat_penalty.comp; adamah.c:6787, :6978, :7095, :7286).  Small inputs (at most 64
// candidates after top-k), one CTA each. ----

// The k largest of n values with their indices into the loc list, largest first, ties to the
// lower index, NaN as -FLT_MAX; index stored as float32.  k <= 64.  Every thread keeps the best of the
// entries it owns that are still free (a bit per entry in shared memory marks the taken ones), a round is one
// block-wide arg-max, and only the thread that owned the winner rescans its entries.
constexpr uint32_t TOPK_BITMAP_WORDS = 4096;                 // entries 0 .. 131071 can be marked
__global__ void __launch_bounds__(1024) k_topk(float* __restrict__ m, uint64_t n_el, const uint32_t* __restrict__ ls, const uint32_t* __restrict__ li,
                                                const uint32_t* __restrict__ lv, uint32_t n, uint32_t k, uint32_t* err) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ uint32_t taken[TOPK_BITMAP_WORDS];
    __shared__ int s_win;
    for (uint32_t i = threadIdx.x; i < (n + 31) / 32; i += blockDim.x) taken[i] = 0u;
    __syncthreads();
    auto rescan = [&](float& bv, int& bi) {
        bv = -3.402823466e+38f; bi = -1;
        for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
            if (taken[i >> 5] & (1u << (i & 31))) continue;
            const uint64_t a = ls[i];
            if (a >= n_el) { atomicOr(err, DEVERR_OOB_MAP); continue; }
            float v = m[a];
            if (!(v == v)) v = -3.402823466e+38f;
            if (better(v, (int)i, bv, bi)) { bv = v; bi = (int)i; }
        }
    };
    float my_v; int my_i;
    rescan(my_v, my_i);
    for (uint32_t out = 0; out < k; ++out) {
        float bv = my_v; int bi = my_i;
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o); int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = bv; si[threadIdx.x >> 5] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (uint32_t w = 1; w < (blockDim.x >> 5); ++w) if (better(sv[w], si[w], bv, bi)) { bv = sv[w]; bi = si[w]; }
            s_win = bi;
            if (bi >= 0) taken[bi >> 5] |= 1u << (bi & 31);
            const uint64_t di = li[out], dv = lv[out];
            if (di >= n_el || dv >= n_el) atomicOr(err, DEVERR_OOB_MAP);
            else { m[di] = (float)(bi < 0 ? 0 : bi); m[dv] = bi < 0 ? -3.402823466e+38f : bv; }
        }
        __syncthreads();
        if (s_win >= 0 && s_win == my_i) rescan(my_v, my_i);       // only the winner's owner lost its candidate
        __syncthreads();
    }
}

// Soft-max with temperature over n <= 64 candidates (already sorted by the caller), nucleus cut at top_p,
// renormalised; the rest gets probability 0 (map_topp.comp).  One warp, two candidates per lane: loads,
// exponentials and the maximum run in parallel; the sums are formed in candidate order (each term fetched from
// its lane by a shuffle), so the results equal a sequential pass bit for bit.
__global__ void __launch_bounds__(32) k_topp(float* __restrict__ m, uint64_t n_el, const uint32_t* __restrict__ ls, const uint32_t* __restrict__ ld,
                                              uint32_t n, float temperature, float top_p, uint32_t* err) {
    const float NEG = -3.402823466e+38f;
    const uint32_t lane = threadIdx.x;
    float lg[2], pr[2];
    bool bad = false;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t i = lane + 32 * h;
        lg[h] = NEG;
        if (i < n) {
            if (ls[i] >= n_el || ld[i] >= n_el) bad = true;
            else { float v = m[ls[i]]; lg[h] = (!(v == v) || isinf(v)) ? NEG : v; }
        }
    }
    if (__any_sync(0xffffffffu, bad)) { if (lane == 0) atomicOr(err, DEVERR_OOB_MAP); return; }
    auto at = [&](const float (&x)[2], uint32_t i) { return __shfl_sync(0xffffffffu, x[i >> 5], i & 31); };
    const float temp = fmaxf(temperature, 1e-6f);
    const float keep_p = fminf(fmaxf(top_p, 0.f), 1.f);
    const float mx = warp_max(fmaxf(lg[0], lg[1]));
    if (mx == NEG) {
#pragma unroll
        for (int h = 0; h < 2; ++h) if (lane + 32 * h < n) m[ld[lane + 32 * h]] = 0.f;
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) pr[h] = (lane + 32 * h < n && lg[h] != NEG) ? expf(__fdiv_rn(lg[h] - mx, temp)) : 0.f;
    float sum = 0.f;
    for (uint32_t i = 0; i < n; ++i) sum += at(pr, i);
    if (sum <= 0.f) {
#pragma unroll
        for (int h = 0; h < 2; ++h) if (lane + 32 * h < n) m[ld[lane + 32 * h]] = (lane + 32 * h == 0) ? 1.f : 0.f;
        return;
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) pr[h] = __fdiv_rn(pr[h], sum);
    uint32_t keep = 0;
    float csum = 0.f;
    for (uint32_t i = 0; i < n; ++i) {
        csum += at(pr, i);
        keep = i + 1;
        if (keep_p >= 0.999999f || csum >= keep_p) break;
    }
    if (keep == 0 && n > 0) keep = 1;
    float ks = 0.f;
    for (uint32_t i = 0; i < keep; ++i) ks += at(pr, i);
    if (ks <= 0.f) ks = 1.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t i = lane + 32 * h;
        if (i < n) m[ld[i]] = i < keep ? __fdiv_rn(pr[h], ks) : 0.f;
    }
}

// Inverse-CDF draw: the first candidate whose running probability sum exceeds r * total
// (map_sample_categorical.comp).  One warp; probabilities are loaded in parallel, the running sums are formed in
// candidate order as above.
__global__ void __launch_bounds__(32) k_sample_categorical(float* __restrict__ m, uint64_t n_el, const uint32_t* __restrict__ lidx, const uint32_t* __restrict__ lprob,
                                                            const uint32_t* __restrict__ lrand, const uint32_t* __restrict__ ldst, uint32_t n, uint32_t* err) {
    const uint32_t lane = threadIdx.x;
    bool bad = lrand[0] >= n_el || ldst[0] >= n_el;
    float pr[2] = {0.f, 0.f};
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t i = lane + 32 * h;
        if (i < n) {
            if (lidx[i] >= n_el || lprob[i] >= n_el) bad = true;
            else { const float p = m[lprob[i]]; pr[h] = (!(p == p) || isinf(p) || p < 0.f) ? 0.f : p; }
        }
    }
    if (__any_sync(0xffffffffu, bad)) { if (lane == 0) atomicOr(err, DEVERR_OOB_MAP); return; }
    auto at = [&](uint32_t i) { return __shfl_sync(0xffffffffu, pr[i >> 5], i & 31); };
    float total = 0.f;
    for (uint32_t i = 0; i < n; ++i) total += at(i);
    uint32_t chosen = 0;
    if (total > 0.f) {
        float r = m[lrand[0]];
        if (!(r == r) || isinf(r)) r = 0.f;
        r = fminf(fmaxf(r, 0.f), 0.99999994f);
        const float target = r * total;
        float acc = 0.f;
        chosen = n - 1;
        for (uint32_t i = 0; i < n; ++i) {
            acc += at(i);
            if (target < acc) { chosen = i; break; }
        }
    }
    if (lane == 0) m[ldst[0]] = m[lidx[chosen]];
}

// logit[tok] = logit > 0 ? logit / penalty : logit * penalty for each listed token id.
__global__ void k_repeat_penalty(float* __restrict__ m, uint64_t n_el, const uint32_t* __restrict__ llogit, uint32_t n_logit_locs,
                                 const uint32_t* __restrict__ toks, uint32_t n_ids, float penalty, uint32_t* err) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_ids) return;
    const uint32_t tok = toks[i];
    if (tok >= n_logit_locs) { atomicOr(err, DEVERR_OOB_MAP); return; }
    const uint64_t a = llogit[tok];
    OOB(a, n_el, err);
    const float v = m[a];
    m[a] = v > 0.f ? __fdiv_rn(v, penalty) : v * penalty;
}

// map_resolve_idx.comp
__global__ void k_resolve_idx(float* __restrict__ m, uint64_t n_el, const uint32_t* __restrict__ lbase, const uint32_t* __restrict__ lsel,
                              const uint32_t* __restrict__ ld, uint32_t n, uint32_t* err) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const uint64_t s = lsel[i], d = ld[i];
    OOB(s, n_el, err); OOB(d, n_el, err);
    float sel = m[s];
    if (!(sel == sel) || isinf(sel) || sel < 0.f) sel = 0.f;
    const uint64_t t = (uint64_t)lbase[0] + (uint32_t)sel;
    OOB(t, n_el, err);
    float tok = m[t];
    if (!(tok == tok) || isinf(tok) || tok < 0.f) tok = 0.f;
    m[d] = tok;
}

// Mat-vec over the reference's own Q4-map storage: 8 nibbles per uint32 in
// logical order, value = code*scale + zero per group (map_matvec_t_xq4.comp
// load_q4).  One warp per output; kept for callers that still build Q4 maps.
__global__ void k_gemv_q4map(const float* __restrict__ x, const uint32_t* __restrict__ words, const float* __restrict__ qp,
                             uint32_t group, uint64_t w_off, float* __restrict__ y, uint32_t K, uint32_t N) {
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= N) return;
    const uint64_t base = w_off + (uint64_t)row * K;
    float acc = 0.f;
    for (uint32_t k = lane; k < K; k += 32) {
        const uint64_t e = base + k;
        const uint32_t code = (words[e >> 3] >> ((uint32_t)(e & 7) * 4)) & 0xFu;
        const uint64_t grp = e / group;
        acc = fmaf(x[k], fmaf((float)code, qp[grp * 2], qp[grp * 2 + 1]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) y[row] = acc;
}

static inline unsigned nblk(uint64_t n, unsigned t) { return (unsigned)((n + t - 1) / t); }

// y = W x for one row of activations over a Q4 map (for other translation units)
void launch_gemv_q4map(const float* x, const Map* w, uint64_t w_off, float* y, uint32_t K, uint32_t N) {
    k_gemv_q4map<<<nblk(N, 8), 256, 0, g.stream>>>(x, (const uint32_t*)w->buf, w->qparams, w->group_size, w_off, y, K, N);
    count_launch();
}

static Map* f32_map(uint32_t id, const char* op) {
    Map* m = get_map(id);
    if (!m) return nullptr;
    if (m->dtype != ADAMAH_DTYPE_F32 || m->pack_size != 1) { fail(ADAMAH_ERR_INVALID, "%s: map %u must be float32 with pack_size 1", op, id); return nullptr; }
    return m;
}

// ARGMAX scratch shared by every fused LM-head call.
static float* s_part_val = nullptr;
static int* s_part_idx = nullptr;
static unsigned int* s_ticket = nullptr;
static int* s_tok = nullptr;

int logits_scratch(size_t n, float** out);      // sample.cu

int argmax_scratch(float** pv, int** pi, unsigned int** tk) {
    if (!s_part_val) {
        // per-CTA partial winners for up to 64 batch rows of one launch (16 row groups of 4), one ticket per group
        size_t n = (size_t)64 * gemv_max_grid();
        if (cudaMalloc((void**)&s_part_val, n * 4) != cudaSuccess || cudaMalloc((void**)&s_part_idx, n * 4) != cudaSuccess ||
            cudaMalloc((void**)&s_ticket, 16 * 4) != cudaSuccess || cudaMalloc((void**)&s_tok, 64 * 4) != cudaSuccess)
            return fail(ADAMAH_ERR_MEMORY, "out of device memory for argmax scratch");
        cudaMemset(s_ticket, 0, 16 * 4);
    }
    *pv = s_part_val; *pi = s_part_idx; *tk = s_ticket;
    return ADAMAH_OK;
}

// Resolve a weight tensor at element offset `off` of a GGUF-block map.
int weight_ref(const Map* m, uint64_t off, uint64_t n_elems, int* wtype, WeightRef* w) {
    if (off + n_elems > m->n_elems) return fail(ADAMAH_ERR_INVALID, "weight tensor [%llu, +%llu) lies beyond its map", (unsigned long long)off, (unsigned long long)n_elems);
    if (m->dtype == ADAMAH_DTYPE_GGUF_Q4_0) {
        if (off % 32) return fail(ADAMAH_ERR_INVALID, "Q4_0 tensor offset must be a multiple of 32");
        *wtype = WT_Q4_0; w->q = m->q40_qs + off / 32; w->d = m->q40_d + off / 32;
        return ADAMAH_OK;
    }
    if (m->dtype == ADAMAH_DTYPE_GGUF_Q4_K) {
        if (off % 256) return fail(ADAMAH_ERR_INVALID, "Q4_K tensor offset must be a multiple of 256");
        *wtype = WT_Q4_K; w->q = (const uint4*)((const uint8_t*)m->buf + off / 256 * 144); w->d = nullptr;
        return ADAMAH_OK;
    }
    if (m->dtype == ADAMAH_DTYPE_GGUF_Q8_0 || m->dtype == ADAMAH_DTYPE_GGUF_Q5_0) {
        if (off % 32) return fail(ADAMAH_ERR_INVALID, "Q8_0 / Q5_0 tensor offset must be a multiple of 32");
        const bool q8 = m->dtype == ADAMAH_DTYPE_GGUF_Q8_0;
        *wtype = q8 ? WT_Q8_0 : WT_Q5_0;
        w->q = m->b8_q + off / 32 * (q8 ? 2 : 1); w->d = m->b8_d + off / 32; w->h = q8 ? nullptr : m->b8_h + off / 32;
        return ADAMAH_OK;
    }
    return fail(ADAMAH_ERR_INVALID, "map does not hold GGUF blocks");
}

// Run a GEMV on the tensor at (map, off): the tensor-core kernel when a row-tiled
// copy of exactly this tensor is registered and the shape fits, the generic one otherwise.
int run_gemv(uint32_t map_id, uint64_t off, int wtype, GemvArgs& ga) {
    if (wt_is_b8(wtype)) {
        // Q8_0 / Q5_0: plain products from their own kernel; an arg-max is a second small kernel over the logits
        if (ga.h_in || ga.epi == EPI_GEGLU || ga.epi == EPI_SWIGLU) return fail(ADAMAH_ERR_INVALID, "Q8_0 / Q5_0 tensors take plain products and arg-max only");
        float* y = ga.y;
        if (ga.epi == EPI_ARGMAX && !y) { int rc = logits_scratch((size_t)ga.B * ga.N, &y); if (rc) return rc; }
        const int ldy = ga.y ? ga.ldy : ga.N;
        int rc = launch_gemv_b8(wtype, ga.w0, ga.x, ga.ldx, y, ldy, ga.N, ga.K, ga.B, g.stream);
        if (rc || ga.epi != EPI_ARGMAX) return rc;
        if (ldy != ga.N) return fail(ADAMAH_ERR_INVALID, "arg-max over Q8_0 / Q5_0 products needs densely stored logits");
        return launch_argmax_rows(y, ga.N, ga.B, ga.softcap, ga.y != nullptr, ga.out_tok, ga.out_val, ga.out_tok_f32, g.stream, false);
    }
    if (ga.B >= TC_MIN_ROWS) {
        // many rows: the tcgen05 GEMM (its workspace is allocated on first use, never inside a capture)
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(g.stream, &cs) == cudaSuccess && cs == cudaStreamCaptureStatusNone) gemm_tc_prepare();
        if (gemm_tc_supports(wtype, ga)) return launch_gemm_tc(wtype, ga, g.stream);
    }
    if (ga.epi != EPI_GEGLU && ga.epi != EPI_SWIGLU) {
        const void* t = find_tiled(map_id, off, (uint32_t)ga.N, (uint32_t)ga.K);
        if (t && gemv_mma_supports(wtype, ga)) return launch_gemv_mma(wtype, (const uint8_t*)t, nullptr, ga, g.stream);
    }
    return launch_gemv(wtype, ga, g.stream);
}

}  // namespace ab

using namespace ab;

#define REQ_READY() if (!ready()) return ADAMAH_ERR_INVALID
#define REQ_H(h, bytes) if (!handle_ok((h), (uint32_t)(bytes))) return ADAMAH_ERR_NOT_FOUND
#define DONE(name) do { count_launch(); int rc__ = check_launch(name); end_of_op(); return rc__; } while (0)

// ---- decode-plan lowering: host side of the runtime arguments ------------------------------------------------
// Set while adamah_decode_step records a plan into a graph.  An operator that meets a sentinel in an argument it can
// take at run time sizes its launch for an upper bound (what its loc handles hold, or `cap` positions) and passes the
// sentinel on; a sentinel anywhere else makes the recording fail and the plan falls back to host-side substitution.
namespace ab {
struct PlanRecording { bool active; uint32_t cap; uint32_t* dev; bool unsupported; };
static PlanRecording g_rec = {};
static inline bool is_rt(uint32_t v) { return g_rec.active && (v == ADAMAH_DECODE_RUNTIME_POS || v == ADAMAH_DECODE_RUNTIME_SEQ_LEN); }
static inline const uint32_t* rt_ptr() { return g_rec.active ? g_rec.dev : nullptr; }
// arguments that have no run-time form: a sentinel there ends the recording
static inline bool rt_refuse(std::initializer_list<uint32_t> vals) {
    for (uint32_t v : vals) if (is_rt(v)) { g_rec.unsupported = true; return true; }
    return false;
}
static inline uint32_t handle_locs(uint32_t h) { return h < MAX_HANDLES && g.handles[h].used ? g.handles[h].nbytes / 4 : 0; }
static inline uint32_t min_locs(std::initializer_list<uint32_t> hs) {
    uint32_t m = 0xFFFFFFFFu;
    for (uint32_t h : hs) { const uint32_t n = handle_locs(h); if (n < m) m = n; }
    return m;
}
}
#define RT_REFUSE(...) if (rt_refuse({__VA_ARGS__})) return fail(ADAMAH_ERR_INVALID, "decode plan: this argument cannot be a run-time value")

static int rmsnorm_impl(uint32_t map_act, uint32_t map_wt, uint32_t src_h, uint32_t wt_h, uint32_t res_h, uint32_t dst_h,
                        uint32_t n_rows, uint32_t dim, float eps) {
    Map* a = f32_map(map_act, "rmsnorm"); Map* w = f32_map(map_wt, "rmsnorm");
    if (!a || !w) return ADAMAH_ERR_NOT_FOUND;
    RT_REFUSE(dim);
    const uint32_t rows_ub = is_rt(n_rows) ? (res_h ? min_locs({src_h, wt_h, dst_h, res_h}) : min_locs({src_h, wt_h, dst_h})) : n_rows;
    if (rows_ub == 0 || dim == 0) return fail(ADAMAH_ERR_INVALID, "rmsnorm: empty shape");
    REQ_H(src_h, rows_ub * 4); REQ_H(wt_h, rows_ub * 4); REQ_H(dst_h, rows_ub * 4);
    if (res_h) REQ_H(res_h, rows_ub * 4);
    k_rmsnorm<<<rows_ub, 256, 0, g.stream>>>((float*)a->buf, a->n_elems, (const float*)w->buf, w->n_elems, hlocs(src_h), hlocs(wt_h),
                                             res_h ? hlocs(res_h) : nullptr, hlocs(dst_h), dim, eps, g.dev_err, n_rows, rt_ptr());
    DONE("map_rmsnorm");
}

extern "C" int map_rmsnorm_dev(uint32_t map, uint32_t src_h, uint32_t wt_h, uint32_t dst_h, uint32_t n_rows, uint32_t dim, float eps) {
    REQ_READY();
    return rmsnorm_impl(map, map, src_h, wt_h, 0, dst_h, n_rows, dim, eps);
}
extern "C" int map_rmsnorm_x_dev(uint32_t map_act, uint32_t map_wt, uint32_t src_h, uint32_t wt_h, uint32_t dst_h,
                                 uint32_t n_rows, uint32_t dim, float eps) {
    REQ_READY();
    return rmsnorm_impl(map_act, map_wt, src_h, wt_h, 0, dst_h, n_rows, dim, eps);
}
extern "C" int map_rmsnorm_add_dev(uint32_t map, uint32_t src_h, uint32_t wt_h, uint32_t resid_h, uint32_t dst_h,
                                   uint32_t n_rows, uint32_t dim, float eps) {
    REQ_READY();
    if (!resid_h) return fail(ADAMAH_ERR_INVALID, "rmsnorm_add: residual handle is 0");
    return rmsnorm_impl(map, map, src_h, wt_h, resid_h, dst_h, n_rows, dim, eps);
}

extern "C" int map_rope_dev(uint32_t map, uint32_t src_h, uint32_t dst_h, uint32_t n_tokens, uint32_t n_heads,
                            uint32_t head_dim, uint32_t pos_offset, float freq_base) {
    REQ_READY();
    Map* m = f32_map(map, "rope");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    RT_REFUSE(n_heads, head_dim);
    const uint32_t tok_ub = is_rt(n_tokens) ? min_locs({src_h, dst_h}) : n_tokens;
    if (!tok_ub || !n_heads || head_dim < 2 || (head_dim & 1)) return fail(ADAMAH_ERR_INVALID, "rope: bad shape");
    REQ_H(src_h, tok_ub * 4); REQ_H(dst_h, tok_ub * 4);
    const uint64_t pairs = (uint64_t)tok_ub * n_heads * (head_dim / 2);
    k_rope<<<nblk(pairs, 256), 256, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(src_h), hlocs(dst_h), n_tokens, n_heads, head_dim,
                                                   pos_offset, freq_base, g.dev_err, rt_ptr());
    DONE("map_rope");
}

extern "C" int map_qk_norm_rope_x_dev(uint32_t map_act, uint32_t map_wt, uint32_t qsrc_h, uint32_t qwt_h, uint32_t ksrc_h, uint32_t kwt_h,
                                      uint32_t qkdst_h, uint32_t q_rows, uint32_t q_dim, uint32_t k_rows, uint32_t k_dim,
                                      uint32_t pos_offset, float freq_base) {
    REQ_READY();
    Map* a = f32_map(map_act, "qk_norm_rope"); Map* w = f32_map(map_wt, "qk_norm_rope");
    if (!a || !w) return ADAMAH_ERR_NOT_FOUND;
    RT_REFUSE(q_rows, q_dim, k_rows, k_dim);
    if (q_rows + k_rows == 0 || (q_rows && (q_dim < 2 || (q_dim & 1))) || (k_rows && (k_dim < 2 || (k_dim & 1))))
        return fail(ADAMAH_ERR_INVALID, "qk_norm_rope: bad shape");
    if (q_rows) { REQ_H(qsrc_h, q_rows * 4); REQ_H(qwt_h, q_rows * 4); }
    if (k_rows) { REQ_H(ksrc_h, k_rows * 4); REQ_H(kwt_h, k_rows * 4); }
    REQ_H(qkdst_h, 4);
    k_qk_norm_rope<<<q_rows + k_rows, 128, 0, g.stream>>>((float*)a->buf, a->n_elems, (const float*)w->buf, w->n_elems,
        q_rows ? hlocs(qsrc_h) : nullptr, q_rows ? hlocs(qwt_h) : nullptr, k_rows ? hlocs(ksrc_h) : nullptr, k_rows ? hlocs(kwt_h) : nullptr,
        hlocs(qkdst_h), q_rows, q_dim, k_rows, k_dim, pos_offset, freq_base, g.dev_err, rt_ptr());
    DONE("map_qk_norm_rope_x");
}

extern "C" int map_row_copy_offset_dev(uint32_t map, uint32_t spec_h, uint32_t src_base_h, uint32_t dst_row_offset,
                                       uint32_t n_copies, uint32_t row_size) {
    REQ_READY();
    Map* m = f32_map(map, "row_copy");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    RT_REFUSE(row_size);
    const uint32_t copies_ub = is_rt(n_copies) ? handle_locs(spec_h) / 2 : n_copies;
    if (!copies_ub || !row_size) return fail(ADAMAH_ERR_INVALID, "row_copy: empty shape");
    REQ_H(spec_h, copies_ub * 8); REQ_H(src_base_h, 4);
    k_row_copy<<<nblk((uint64_t)copies_ub * row_size, 256), 256, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(spec_h), hlocs(src_base_h),
                                                                                dst_row_offset, n_copies, row_size, g.dev_err, rt_ptr());
    DONE("map_row_copy_offset");
}
extern "C" int map_row_copy_dev(uint32_t map, uint32_t spec_h, uint32_t src_base_h, uint32_t n_copies, uint32_t row_size) {
    return map_row_copy_offset_dev(map, spec_h, src_base_h, 0, n_copies, row_size);
}

extern "C" int map_matmul_t_dev(uint32_t map, uint32_t a_h, uint32_t b_h, uint32_t c_h, uint32_t M, uint32_t K, uint32_t N, uint32_t n_ops) {
    REQ_READY();
    Map* m = f32_map(map, "matmul_t");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    RT_REFUSE(n_ops);
    const uint32_t M_ub = is_rt(M) ? g_rec.cap : M, N_ub = is_rt(N) ? g_rec.cap : N;      // K only bounds a loop
    if (!M_ub || !K || !N_ub || !n_ops || M_ub > 65535 || n_ops > 65535) return fail(ADAMAH_ERR_INVALID, "matmul_t: bad shape");
    REQ_H(a_h, n_ops * 4); REQ_H(b_h, n_ops * 4); REQ_H(c_h, n_ops * 4);
    dim3 grid(nblk(N_ub, 8), M_ub, n_ops);
    k_matmul_t<<<grid, 256, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(a_h), hlocs(b_h), hlocs(c_h), M, K, N, g.dev_err, rt_ptr());
    DONE("map_matmul_t");
}

extern "C" int map_attn_softmax_value_dev(uint32_t map, uint32_t scores_h, uint32_t values_h, uint32_t out_h, uint32_t n_ops,
                                          uint32_t row_size, uint32_t value_dim, float scale, float cap) {
    REQ_READY();
    Map* m = f32_map(map, "attn_softmax_value");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    RT_REFUSE(n_ops, value_dim);
    const uint32_t rows_ub = is_rt(row_size) ? (g_rec.cap < 49152u ? g_rec.cap : 49152u) : row_size;
    if (!n_ops || !rows_ub || !value_dim) return fail(ADAMAH_ERR_INVALID, "attn_softmax_value: empty shape");
    if (rows_ub > 49152) return fail(ADAMAH_ERR_INVALID, "attn_softmax_value: row_size %u exceeds 49152", rows_ub);
    REQ_H(scores_h, n_ops * 4); REQ_H(values_h, n_ops * 4); REQ_H(out_h, n_ops * 4);
    const size_t smem = (size_t)rows_ub * 4;
    static size_t raised = 48 * 1024;
    if (smem > raised) {
        if (cudaFuncSetAttribute(k_attn_softmax_value, cudaFuncAttributeMaxDynamicSharedMemorySize, 196608) != cudaSuccess)
            return fail(ADAMAH_ERR_BACKEND, "attn_softmax_value: cannot raise the shared-memory limit");
        raised = 196608;
    }
    k_attn_softmax_value<<<n_ops, 256, smem, g.stream>>>((float*)m->buf, m->n_elems, hlocs(scores_h), hlocs(values_h), hlocs(out_h),
                                                         row_size, value_dim, scale, cap, g.dev_err, rows_ub, rt_ptr());
    DONE("map_attn_softmax_value");
}

extern "C" int map_op1_dev(uint32_t map, uint32_t op, uint32_t src_h, uint32_t dst_h, uint32_t n) {
    REQ_READY();
    Map* m = f32_map(map, "op1");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n) return ADAMAH_OK;
    if (op > 33) return fail(ADAMAH_ERR_INVALID, "op1: unknown op %u", op);
    const uint32_t n_ub = is_rt(n) ? min_locs({src_h, dst_h}) : n;
    REQ_H(src_h, (uint64_t)n_ub * 4); REQ_H(dst_h, (uint64_t)n_ub * 4);
    k_op1<<<nblk(n_ub, 256), 256, 0, g.stream>>>((float*)m->buf, m->n_elems, op, hlocs(src_h), hlocs(dst_h), n, g.dev_err, rt_ptr());
    DONE("map_op1");
}
extern "C" int map_op2_dev(uint32_t map, uint32_t op, uint32_t a_h, uint32_t b_h, uint32_t dst_h, uint32_t n) {
    REQ_READY();
    Map* m = f32_map(map, "op2");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n) return ADAMAH_OK;
    if (op > 17 && op != 34 && op != 35) return fail(ADAMAH_ERR_INVALID, "op2: unknown op %u", op);
    const uint32_t n_ub = is_rt(n) ? min_locs({a_h, b_h, dst_h}) : n;
    REQ_H(a_h, (uint64_t)n_ub * 4); REQ_H(b_h, (uint64_t)n_ub * 4); REQ_H(dst_h, (uint64_t)n_ub * 4);
    k_op2<<<nblk(n_ub, 256), 256, 0, g.stream>>>((float*)m->buf, m->n_elems, op, hlocs(a_h), hlocs(b_h), hlocs(dst_h), n, g.dev_err, rt_ptr());
    DONE("map_op2");
}
extern "C" int map_broadcast_dev(uint32_t map, uint32_t op, uint32_t src_h, uint32_t scalar_h, uint32_t dst_h, uint32_t n) {
    REQ_READY();
    Map* m = f32_map(map, "broadcast");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n) return ADAMAH_OK;
    if (op > 3) return fail(ADAMAH_ERR_INVALID, "broadcast: unknown op %u", op);
    const uint32_t n_ub = is_rt(n) ? min_locs({src_h, scalar_h, dst_h}) : n;
    REQ_H(src_h, (uint64_t)n_ub * 4); REQ_H(scalar_h, (uint64_t)n_ub * 4); REQ_H(dst_h, (uint64_t)n_ub * 4);
    k_broadcast<<<nblk(n_ub, 256), 256, 0, g.stream>>>((float*)m->buf, m->n_elems, op, hlocs(src_h), hlocs(scalar_h), hlocs(dst_h), n, g.dev_err, rt_ptr());
    DONE("map_broadcast");
}
extern "C" int map_argmax_dev(uint32_t map, uint32_t src_h, uint32_t dst_h, uint32_t n) {
    REQ_READY();
    Map* m = f32_map(map, "argmax");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n) return fail(ADAMAH_ERR_INVALID, "argmax: empty input");
    REQ_H(src_h, (uint64_t)n * 4); REQ_H(dst_h, 4);
    k_argmax<<<1, 1024, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(src_h), hlocs(dst_h), n, g.dev_err);
    DONE("map_argmax");
}
extern "C" int map_topk_dev(uint32_t map, uint32_t src_h, uint32_t idx_dst_h, uint32_t val_dst_h, uint32_t n, uint32_t k) {
    REQ_READY();
    Map* m = f32_map(map, "topk");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n || !k) return ADAMAH_OK;
    if (k > 64) return fail(ADAMAH_ERR_INVALID, "topk: k must be at most 64");
    if (n > TOPK_BITMAP_WORDS * 32u) return fail(ADAMAH_ERR_INVALID, "topk: at most %u candidates", TOPK_BITMAP_WORDS * 32u);
    REQ_H(src_h, (uint64_t)n * 4); REQ_H(idx_dst_h, (uint64_t)k * 4); REQ_H(val_dst_h, (uint64_t)k * 4);
    k_topk<<<1, 1024, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(src_h), hlocs(idx_dst_h), hlocs(val_dst_h), n, k, g.dev_err);
    DONE("map_topk");
}
extern "C" int map_topp_dev(uint32_t map, uint32_t src_h, uint32_t dst_h, uint32_t n, float temperature, float top_p) {
    REQ_READY();
    Map* m = f32_map(map, "topp");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n) return ADAMAH_OK;
    if (n > 64) return fail(ADAMAH_ERR_INVALID, "topp: at most 64 candidates");
    REQ_H(src_h, (uint64_t)n * 4); REQ_H(dst_h, (uint64_t)n * 4);
    k_topp<<<1, 32, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(src_h), hlocs(dst_h), n, temperature, top_p, g.dev_err);
    DONE("map_topp");
}
extern "C" int map_sample_categorical_dev(uint32_t map, uint32_t idx_h, uint32_t prob_h, uint32_t rand_h, uint32_t dst_h, uint32_t n) {
    REQ_READY();
    Map* m = f32_map(map, "sample_categorical");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n) return ADAMAH_OK;
    if (n > 64) n = 64;
    REQ_H(idx_h, (uint64_t)n * 4); REQ_H(prob_h, (uint64_t)n * 4); REQ_H(rand_h, 4); REQ_H(dst_h, 4);
    k_sample_categorical<<<1, 32, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(idx_h), hlocs(prob_h), hlocs(rand_h), hlocs(dst_h), n, g.dev_err);
    DONE("map_sample_categorical");
}
// token_ids_h holds raw uint32 token ids (not locs); src_h lists the logits' locs.
extern "C" int map_repeat_penalty_dev(uint32_t map, uint32_t src_h, uint32_t token_ids_h, uint32_t n_ids, float penalty) {
    REQ_READY();
    Map* m = f32_map(map, "repeat_penalty");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n_ids) return ADAMAH_OK;
    if (n_ids > 64) return fail(ADAMAH_ERR_INVALID, "repeat_penalty: at most 64 token ids");
    REQ_H(src_h, 4); REQ_H(token_ids_h, (uint64_t)n_ids * 4);
    const uint32_t n_logit_locs = (uint32_t)(g.handles[src_h].nbytes / 4);
    k_repeat_penalty<<<1, 64, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(src_h), n_logit_locs, hlocs(token_ids_h), n_ids, penalty, g.dev_err);
    DONE("map_repeat_penalty");
}
extern "C" int map_resolve_idx_dev(uint32_t map, uint32_t base_h, uint32_t sel_h, uint32_t dst_h, uint32_t n) {
    REQ_READY();
    Map* m = f32_map(map, "resolve_idx");
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (!n) return ADAMAH_OK;
    REQ_H(base_h, 4); REQ_H(sel_h, (uint64_t)n * 4); REQ_H(dst_h, (uint64_t)n * 4);
    k_resolve_idx<<<nblk(n, 64), 64, 0, g.stream>>>((float*)m->buf, m->n_elems, hlocs(base_h), hlocs(sel_h), hlocs(dst_h), n, g.dev_err);
    DONE("map_resolve_idx");
}

// y[M,N] = x[M,K] * W[N,K]^T for n_ops problems; weights in a Q4 map or a GGUF-block map.
extern "C" int map_matmul_t_xq4_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t c_h,
                                    uint32_t M, uint32_t K, uint32_t N, uint32_t n_ops) {
    REQ_READY();
    Map* a = f32_map(map_act, "matmul_t_xq4");
    Map* w = get_map(map_wt);
    if (!a || !w) return ADAMAH_ERR_NOT_FOUND;
    RT_REFUSE(M, K, N, n_ops);
    if (!M || !K || !N || !n_ops) return fail(ADAMAH_ERR_INVALID, "matmul_t_xq4: empty shape");
    REQ_H(a_h, n_ops * 4); REQ_H(b_h, n_ops * 4); REQ_H(c_h, n_ops * 4);
    for (uint32_t op = 0; op < n_ops; ++op) {
        uint32_t ab_, bb, cb;
        if (n_ops == 1) { if (!hfirst(a_h, &ab_) || !hfirst(b_h, &bb) || !hfirst(c_h, &cb)) return ADAMAH_ERR_NOT_FOUND; }
        else {
            if (!g.handles[a_h].shadow || !g.handles[b_h].shadow || !g.handles[c_h].shadow)
                return fail(ADAMAH_ERR_INVALID, "matmul_t_xq4: batched problems need host-uploaded loc handles");
            ab_ = g.handles[a_h].shadow[op]; bb = g.handles[b_h].shadow[op]; cb = g.handles[c_h].shadow[op];
        }
        if ((uint64_t)ab_ + (uint64_t)M * K > a->n_elems || (uint64_t)cb + (uint64_t)M * N > a->n_elems)
            return fail(ADAMAH_ERR_INVALID, "matmul_t_xq4: activation range beyond map %u", map_act);
        const float* x = (const float*)a->buf + ab_;
        float* y = (float*)a->buf + cb;
        if (w->dtype == ADAMAH_DTYPE_Q4) {
            if ((uint64_t)bb + (uint64_t)N * K > w->n_elems) return fail(ADAMAH_ERR_INVALID, "matmul_t_xq4: weight range beyond map %u", map_wt);
            for (uint32_t r = 0; r < M; ++r) {
                k_gemv_q4map<<<nblk(N, 8), 256, 0, g.stream>>>(x + (size_t)r * K, (const uint32_t*)w->buf, w->qparams, w->group_size, bb,
                                                                y + (size_t)r * N, K, N);
                count_launch();
            }
        } else {
            int wtype; GemvArgs ga = {};
            int rc = weight_ref(w, bb, (uint64_t)N * K, &wtype, &ga.w0);
            if (rc) return rc;
            if (ab_ % 4 || K % 4) return fail(ADAMAH_ERR_INVALID, "matmul_t_xq4: activation offset must be a multiple of 4 elements");
            ga.x = x; ga.ldx = K; ga.y = y; ga.ldy = N; ga.N = N; ga.K = K; ga.B = M; ga.epi = EPI_STORE;
            rc = run_gemv(map_wt, bb, wtype, ga);
            if (rc) return rc;
        }
    }
    int rc = check_launch("map_matmul_t_xq4");
    end_of_op();
    return rc;
}

// LM head fused with arg-max (map_matvec_argmax_t_xq4.comp + map_argmax_pairs.comp):
// the winning row index is stored as float32 at locs_dst[0].  The reference's
// partial buffers (idx_tmp, val_tmp) are accepted and left untouched: partials
// live in the library's own scratch.
extern "C" int map_matvec_argmax_t_xq4_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t idx_tmp_h,
                                           uint32_t val_tmp_h, uint32_t dst_h, uint32_t K, uint32_t N, uint32_t rows_per_group) {
    REQ_READY();
    (void)rows_per_group;
    Map* a = f32_map(map_act, "matvec_argmax");
    Map* w = get_map(map_wt);
    if (!a || !w) return ADAMAH_ERR_NOT_FOUND;
    if (!K || !N) return fail(ADAMAH_ERR_INVALID, "matvec_argmax: empty shape");
    REQ_H(idx_tmp_h, 4); REQ_H(val_tmp_h, 4);
    uint32_t ab_, bb, db;
    if (!hfirst(a_h, &ab_) || !hfirst(b_h, &bb) || !hfirst(dst_h, &db)) return ADAMAH_ERR_NOT_FOUND;
    if ((uint64_t)ab_ + K > a->n_elems || db >= a->n_elems) return fail(ADAMAH_ERR_INVALID, "matvec_argmax: activation range beyond map");
    if (w->dtype != ADAMAH_DTYPE_GGUF_Q4_0 && w->dtype != ADAMAH_DTYPE_GGUF_Q4_K && w->dtype != ADAMAH_DTYPE_GGUF_Q8_0 && w->dtype != ADAMAH_DTYPE_GGUF_Q5_0)
        return fail(ADAMAH_ERR_INVALID, "matvec_argmax: weights must be in a GGUF-block map");
    int wtype; GemvArgs ga = {};
    int rc = weight_ref(w, bb, (uint64_t)N * K, &wtype, &ga.w0);
    if (rc) return rc;
    if (ab_ % 4) return fail(ADAMAH_ERR_INVALID, "matvec_argmax: activation offset must be a multiple of 4 elements");
    rc = argmax_scratch(&ga.part_val, &ga.part_idx, &ga.ticket);
    if (rc) return rc;
    ga.x = (const float*)a->buf + ab_; ga.ldx = K; ga.y = nullptr; ga.ldy = N; ga.N = N; ga.K = K; ga.B = 1; ga.epi = EPI_ARGMAX;
    ga.out_tok = nullptr; ga.out_tok_f32 = (float*)a->buf + db;
    rc = run_gemv(map_wt, bb, wtype, ga);
    if (rc) return rc;
    rc = check_launch("map_matvec_argmax_t_xq4");
    end_of_op();
    return rc;
}

// The reference's 8-bit weight operators (adamah.c:9834 map_matmul_t_xq8_dev, :10189 map_row_gather_xq8_dev; shaders
// map_matvec_t_xq8.comp / map_matmul_t_xq8.comp / map_row_gather_xq8.comp).  There the weight map holds bytes plus a
// (scale, zero) pair per 32; here it is a GGUF-block map of Q8_0 or Q5_0 blocks as they are in the file, which is
// what the reference derives its bytes and pairs from (adam/models/engine.py:1142-1182).
extern "C" int map_matmul_t_xq8_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t c_h,
                                    uint32_t M, uint32_t K, uint32_t N, uint32_t n_ops) {
    REQ_READY();
    Map* w = get_map(map_wt);
    if (!w) return ADAMAH_ERR_NOT_FOUND;
    if (n_ops == 0) return ADAMAH_OK;                                        // adamah.c:9856
    if (w->dtype != ADAMAH_DTYPE_GGUF_Q8_0 && w->dtype != ADAMAH_DTYPE_GGUF_Q5_0)
        return fail(ADAMAH_ERR_INVALID, "matmul_t_xq8: map %u does not hold Q8_0 / Q5_0 blocks", map_wt);
    return map_matmul_t_xq4_dev(map_act, map_wt, a_h, b_h, c_h, M, K, N, n_ops);   // same contract; the map's type picks the kernel
}

// map_act[dst_base + i] = decode(map_wt[src_base + row_idx * row_size + i]) * scale, i < row_size: the token-embedding
// row fetch (adam/models/engine.py:2409-2413 for the Q4 map; the Q8 twin is used for Q8_0 / Q5_0 embeddings).
// Bases and the row index are immediates, as in the reference.
extern "C" int map_row_gather_xq8_dev(uint32_t map_act, uint32_t map_wt, uint32_t src_base, uint32_t dst_base, uint32_t row_idx,
                                      uint32_t row_size, float scale) {
    REQ_READY();
    Map* a = f32_map(map_act, "row_gather_xq8");
    Map* w = get_map(map_wt);
    if (!a || !w) return ADAMAH_ERR_NOT_FOUND;
    if (row_size == 0) return ADAMAH_OK;                                     // adamah.c:10196
    const uint64_t src = (uint64_t)src_base + (uint64_t)row_idx * row_size;
    if (row_size % 32 || src % 32) return fail(ADAMAH_ERR_INVALID, "row_gather_xq8: rows must be whole blocks of 32");
    if ((uint64_t)dst_base + row_size > a->n_elems) return fail(ADAMAH_ERR_INVALID, "row_gather_xq8: destination beyond map %u", map_act);
    int wtype; WeightRef wr = {};
    int rc = weight_ref(w, src, row_size, &wtype, &wr);
    if (rc) return rc;
    if (!wt_is_b8(wtype)) return fail(ADAMAH_ERR_INVALID, "row_gather_xq8: map %u does not hold Q8_0 / Q5_0 blocks", map_wt);
    launch_dequant_b8(wtype, wr, row_size, (float*)a->buf + dst_base, scale, true, g.stream);
    rc = check_launch("map_row_gather_xq8");
    end_of_op();
    return rc;
}

// ---- decode plan (adamah.c:10253-10398) -------------------------------------
// A registered plan is a flat list of operator calls whose arguments may hold the sentinels
// ADAMAH_DECODE_RUNTIME_POS / _SEQ_LEN.  The reference replays the list through its public entry points every step
// with the sentinels replaced on the host.  Here the list is lowered ONCE to a CUDA graph in which the sentinels stay
// symbolic: kernels read {pos, seq_len} from two device words that a one-thread kernel sets before each launch of the
// graph, so a step costs two launches whatever the length of the plan.  Launches that depend on a run-time size are
// sized for an upper bound (the loc handles' length, or `cap` positions, doubled and re-recorded when a step outgrows
// it).  The first step of a plan runs eagerly (operators create their scratch buffers then, not inside a capture);
// a plan the recorder cannot express (a sentinel in an argument with no run-time form, a device-produced base handle)
// keeps running by host-side substitution, as in the reference.

namespace ab {
bool capturing();                     // runtime.cu: inside adam_b200_capture_begin / _end
constexpr uint32_t MAX_PLANS = 16, MAX_PLAN_OPS = 4096;
struct Plan {
    AdamahDecodePlanOp* ops; uint32_t n; bool valid;
    int state;                        // 0 = not run yet, 1 = warmed (eager step done), 2 = graph, -1 = host substitution only
    cudaGraph_t graph; cudaGraphExec_t exec;
    uint32_t cap, nodes, compiles, graph_steps, host_steps;
};
static Plan g_plans[MAX_PLANS];
static uint32_t* g_rt_dev = nullptr;
static void plan_drop_graph(Plan& p) {
    if (p.exec) { cudaStreamSynchronize(g.stream); cudaGraphExecDestroy(p.exec); }
    if (p.graph) cudaGraphDestroy(p.graph);
    p.exec = nullptr; p.graph = nullptr; p.nodes = 0;
}
void plans_clear_all() {
    for (auto& p : g_plans) { plan_drop_graph(p); free(p.ops); p = Plan{}; }
    if (g_rt_dev) { cudaFree(g_rt_dev); g_rt_dev = nullptr; }
}

// The operator calls of a plan, with u0..u4 as given (`symbolic`) or with the sentinels replaced by pos / seq_len.
static int plan_replay(const Plan& p, bool symbolic, uint32_t pos, uint32_t seq_len) {
    auto rt = [&](uint32_t v) { return symbolic ? v : (v == ADAMAH_DECODE_RUNTIME_POS ? pos : (v == ADAMAH_DECODE_RUNTIME_SEQ_LEN ? seq_len : v)); };
    int rc = ADAMAH_OK;
    for (uint32_t i = 0; i < p.n && rc == ADAMAH_OK; ++i) {
        const AdamahDecodePlanOp& o = p.ops[i];
        const uint32_t u0 = rt(o.u0), u1 = rt(o.u1), u2 = rt(o.u2), u3 = rt(o.u3), u4 = rt(o.u4);
        switch (o.kind) {
        case 0: break;
        case 1: rc = adamah_fusion_flush(); break;
        case 2: adamah_fusion_enable(u0 != 0); break;
        case 10: rc = map_op1_dev(o.map_id, o.op_code, o.h0, o.h1, u0); break;
        case 11: rc = map_op2_dev(o.map_id, o.op_code, o.h0, o.h1, o.h2, u0); break;
        case 12: rc = map_rmsnorm_dev(o.map_id, o.h0, o.h1, o.h2, u0, u1, o.f0); break;
        case 13: rc = map_rmsnorm_x_dev(o.map_id, o.map_id2, o.h0, o.h1, o.h2, u0, u1, o.f0); break;
        case 14: rc = map_rmsnorm_add_dev(o.map_id, o.h0, o.h1, o.h2, o.h3, u0, u1, o.f0); break;
        case 15: rc = map_rope_dev(o.map_id, o.h0, o.h1, u0, u1, u2, u3, o.f0); break;
        case 16: rc = map_matmul_t_dev(o.map_id, o.h0, o.h1, o.h2, u0, u1, u2, u3); break;
        case 19: rc = map_matmul_t_xq4_dev(o.map_id, o.map_id2, o.h0, o.h1, o.h2, u0, u1, u2, u3); break;
        case 23: rc = map_qk_norm_rope_x_dev(o.map_id, o.map_id2, o.h0, o.h1, o.h2, o.h3, o.h4, u0, u1, u2, u3, u4, o.f0); break;
        case 24: rc = map_row_copy_offset_dev(o.map_id, o.h0, o.h1, u0, u1, u2); break;
        case 25: rc = map_attn_softmax_value_dev(o.map_id, o.h0, o.h1, o.h2, u0, u1, u2, o.f0, o.f1); break;
        default: rc = fail(ADAMAH_ERR_INVALID, "decode plan: op kind %u is not on the decode path", o.kind); break;
        }
    }
    return rc;
}

// Record the plan into a graph sized for `cap` positions.  Leaves p.state = 2 on success, -1 otherwise.
static void plan_record(Plan& p, uint32_t cap) {
    plan_drop_graph(p);
    p.state = -1;
    if (!g_rt_dev && cudaMalloc((void**)&g_rt_dev, 8) != cudaSuccess) { cudaGetLastError(); return; }
    // base handles that only exist on the device would be read back (a synchronisation) by the operators that need them
    for (uint32_t i = 0; i < p.n; ++i)
        if (p.ops[i].kind == 19)
            for (uint32_t h : {p.ops[i].h0, p.ops[i].h1, p.ops[i].h2}) if (h >= MAX_HANDLES || !g.handles[h].used || !g.handles[h].shadow) return;
    const uint64_t l0 = g.launches;
    if (cudaStreamSynchronize(g.stream) != cudaSuccess || cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) { cudaGetLastError(); return; }
    g_rec = PlanRecording{true, cap, g_rt_dev, false};
    const int rc = plan_replay(p, true, 0, 0);
    g_rec.active = false;
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(g.stream, &graph);
    const uint32_t nodes = (uint32_t)(g.launches - l0);
    g.launches = l0;
    if (rc != ADAMAH_OK || e != cudaSuccess || !graph) { cudaGetLastError(); if (graph) cudaGraphDestroy(graph); return; }
    if (cudaGraphInstantiate(&p.exec, graph, 0) != cudaSuccess) { cudaGetLastError(); cudaGraphDestroy(graph); p.exec = nullptr; return; }
    p.graph = graph; p.cap = cap; p.nodes = nodes; p.compiles++; p.state = 2;
}
}  // namespace ab

extern "C" int adamah_register_decode_plan(uint32_t plan_id, const AdamahDecodePlanOp* ops, uint32_t n_ops) {
    REQ_READY();
    if (plan_id >= MAX_PLANS || n_ops > MAX_PLAN_OPS || (n_ops && !ops)) return fail(ADAMAH_ERR_INVALID, "decode plan: bad arguments");
    Plan& p = g_plans[plan_id];
    plan_drop_graph(p);
    free(p.ops);
    p = Plan{};
    if (n_ops) {
        p.ops = (AdamahDecodePlanOp*)malloc(sizeof(AdamahDecodePlanOp) * n_ops);
        if (!p.ops) return fail(ADAMAH_ERR_MEMORY, "decode plan: out of host memory");
        memcpy(p.ops, ops, sizeof(AdamahDecodePlanOp) * n_ops);
    }
    p.n = n_ops; p.valid = true;
    static const bool graphs = !(getenv("ADAM_B200_PLAN_GRAPH") && atoi(getenv("ADAM_B200_PLAN_GRAPH")) == 0);
    if (!graphs) p.state = -1;
    return ADAMAH_OK;
}
extern "C" void adamah_clear_decode_plan(uint32_t plan_id) {
    if (plan_id >= MAX_PLANS) return;
    plan_drop_graph(g_plans[plan_id]);
    free(g_plans[plan_id].ops);
    g_plans[plan_id] = Plan{};
}
extern "C" int adamah_decode_step(uint32_t plan_id, uint32_t pos, uint32_t seq_len) {
    REQ_READY();
    if (plan_id >= MAX_PLANS) return fail(ADAMAH_ERR_INVALID, "decode plan id out of range");
    Plan& p = g_plans[plan_id];
    if (!p.valid) return fail(ADAMAH_ERR_NOT_FOUND, "decode plan %u is not registered", plan_id);
    const bool opened = g.batch_depth == 0;
    if (opened) batch_begin();
    int rc = ADAMAH_OK;
    const uint32_t need = (pos >= seq_len ? pos + 1 : seq_len);
    if (p.state == 1 || (p.state == 2 && need > p.cap)) {
        if (capturing()) p.state = p.state == 2 ? 2 : 1;          // inside a caller's capture: not now
        else { uint32_t cap = 256; while (cap < need && cap < (1u << 30)) cap <<= 1; plan_record(p, cap); }
    }
    if (p.state == 2 && need <= p.cap && !capturing()) {
        k_set_runtime<<<1, 1, 0, g.stream>>>(g_rt_dev, pos, seq_len);
        if (cudaGraphLaunch(p.exec, g.stream) != cudaSuccess) rc = fail(ADAMAH_ERR_BACKEND, "decode plan: graph launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        count_launch(1 + p.nodes);
        p.graph_steps++;
    } else {
        rc = plan_replay(p, false, pos, seq_len);
        p.host_steps++;
        if (p.state == 0 && rc == ADAMAH_OK) p.state = 1;
    }
    if (opened) batch_end();
    return rc;
}
// out[0..5] = state (2 = runs as a graph, -1 = host substitution only, 0 / 1 = not recorded yet), positions the graph is
// sized for, kernels in the graph, times recorded, steps run as a graph, steps run by host substitution.
extern "C" int adam_b200_decode_plan_info(uint32_t plan_id, uint32_t* out) {
    if (plan_id >= MAX_PLANS || !out) return fail(ADAMAH_ERR_INVALID, "decode plan id out of range");
    const Plan& p = g_plans[plan_id];
    if (!p.valid) return fail(ADAMAH_ERR_NOT_FOUND, "decode plan %u is not registered", plan_id);
    out[0] = (uint32_t)p.state; out[1] = p.cap; out[2] = p.nodes; out[3] = p.compiles; out[4] = p.graph_steps; out[5] = p.host_steps;
    return ADAMAH_OK;
}

// ---- symbols off the decode path (present so the reference binding loads) ----
#define OFFPATH(name, ...) extern "C" int name(__VA_ARGS__) { return fail(ADAMAH_ERR_INVALID, #name " is not on the decode path"); }
typedef uint32_t u32; typedef const uint32_t* cu32p;
OFFPATH(map_op1, u32, u32, cu32p, cu32p, u32)
OFFPATH(map_op2, u32, u32, cu32p, cu32p, cu32p, u32)
OFFPATH(map_matmul, u32, cu32p, cu32p, cu32p, u32, u32, u32, u32)
OFFPATH(map_softmax, u32, cu32p, cu32p, u32, u32)
OFFPATH(map_layernorm, u32, cu32p, cu32p, cu32p, cu32p, u32, u32, float)
OFFPATH(map_broadcast, u32, u32, cu32p, cu32p, cu32p, u32)
OFFPATH(map_reduce, u32, u32, cu32p, cu32p, u32)
OFFPATH(map_matmul_dev, u32, u32, u32, u32, u32, u32, u32, u32)
OFFPATH(map_softmax_dev, u32, u32, u32, u32, u32)
OFFPATH(map_softmax_abs_dev, u32, u32, u32, u32, u32)
OFFPATH(map_attn_softmax_abs_dev, u32, u32, u32, u32, u32, float, float)
OFFPATH(map_layernorm_dev, u32, u32, u32, u32, u32, u32, u32, float)
OFFPATH(map_reduce_dev, u32, u32, u32, u32, u32)
OFFPATH(map_fma_dev, u32, u32, u32, u32, u32, u32)
OFFPATH(map_matmul_t_x_dev, u32, u32, u32, u32, u32, u32, u32, u32, u32)
OFFPATH(map_matmul_x_dev, u32, u32, u32, u32, u32, u32, u32, u32, u32)
OFFPATH(map_matmul_xq4_dev, u32, u32, u32, u32, u32, u32, u32, u32, u32)
OFFPATH(map_matmul_xq8_dev, u32, u32, u32, u32, u32, u32, u32, u32, u32)
