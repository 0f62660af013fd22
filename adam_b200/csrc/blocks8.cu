// Kernels over GGUF Q8_0 / Q5_0 blocks kept in planes (see blocks8.cuh): upload repack, bit-exact decode
// and row fetch, a dequant-fused GEMV, and the two small kernels (norm chain, arg-max over logits) that
// let the decoder run its LM head on such a matrix.
//
// GEMV.  HBM-bound byte work: 34 (22) bytes of weights per 32 products, activations staged once per CTA
// in shared memory.  L lanes share a row (L picked on the host so that a lane walks about a dozen blocks),
// a lane owns TWO neighbouring rows so every activation it reads from shared memory is used twice, and a
// warp covers (32 / L) * 2 rows per pass; CTAs walk the passes grid-stride.  A weight byte becomes a float
// with one byte permute (the code lands in the low mantissa bits of 2^23) and one subtraction, both exact;
// a block's 32 products are summed in fp32 and scaled by the block's fp16 scale once.  Lanes of a row combine
// with xor shuffles, so results do not depend on the launch.
#include "blocks8.cuh"

namespace ab {

constexpr int B8_THREADS = 256;
constexpr int B8_XSTRIDE = 36;           // floats per staged activation block (32 + 4 pad: float4 reads of neighbouring lanes hit different banks)
constexpr float B8_SNEG = -3.402823466e+38f;

// ---- upload -------------------------------------------------------------------------------------------
// One thread per block; the file's blocks are only 2-byte aligned.
__global__ void k_repack_q8_0(const uint16_t* __restrict__ raw, uint4* __restrict__ q, __half* __restrict__ d, uint64_t n_blocks) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_blocks) return;
    const uint16_t* b = raw + i * 17;
    uint32_t w[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) w[k] = b[1 + 2 * k] | ((uint32_t)b[2 + 2 * k] << 16);
    d[i] = __ushort_as_half(b[0]);
    q[2 * i] = make_uint4(w[0], w[1], w[2], w[3]);
    q[2 * i + 1] = make_uint4(w[4], w[5], w[6], w[7]);
}
__global__ void k_repack_q5_0(const uint16_t* __restrict__ raw, uint4* __restrict__ q, uint32_t* __restrict__ h, __half* __restrict__ d, uint64_t n_blocks) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_blocks) return;
    const uint16_t* b = raw + i * 11;
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) w[k] = b[3 + 2 * k] | ((uint32_t)b[4 + 2 * k] << 16);
    d[i] = __ushort_as_half(b[0]);
    h[i] = b[1] | ((uint32_t)b[2] << 16);
    q[i] = make_uint4(w[0], w[1], w[2], w[3]);
}

int launch_repack_b8(int wt, const void* raw_dev, const WeightRef& w, uint64_t n_blocks, cudaStream_t st) {
    if ((uintptr_t)raw_dev & 1) return fail(ADAMAH_ERR_INVALID, "block source must be 2-byte aligned");
    const unsigned grid = (unsigned)((n_blocks + 255) / 256);
    if (wt == WT_Q8_0) k_repack_q8_0<<<grid, 256, 0, st>>>((const uint16_t*)raw_dev, (uint4*)w.q, (__half*)w.d, n_blocks);
    else k_repack_q5_0<<<grid, 256, 0, st>>>((const uint16_t*)raw_dev, (uint4*)w.q, (uint32_t*)w.h, (__half*)w.d, n_blocks);
    count_launch();
    return ADAMAH_OK;
}

// ---- bit-exact decode -----------------------------------------------------------------------------------
// The integer code times the fp16 scale is exact in float32 (at most 8 + 11 significant bits), so one
// rounding-free product reproduces the loader's value; `scale` (the embedding multiplier) rounds once more.
template <int WT>
__global__ void k_dequant_b8(const WeightRef w, float* __restrict__ out, uint64_t n_elems, float scale, int with_scale) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elems) return;
    const uint64_t blk = i >> 5;
    const uint32_t j = (uint32_t)(i & 31);
    const float d = __half2float(w.d[blk]);
    int q;
    if (WT == WT_Q8_0) {
        q = (int)reinterpret_cast<const int8_t*>(w.q)[blk * 32 + j];
    } else {
        const uint32_t byte = reinterpret_cast<const uint8_t*>(w.q)[blk * 16 + (j & 15)];
        const uint32_t lo = j < 16 ? (byte & 15u) : (byte >> 4);
        q = (int)(lo | (((w.h[blk] >> j) & 1u) << 4)) - 16;
    }
    float v = __fmul_rn((float)q, d);
    if (with_scale) v = __fmul_rn(v, scale);
    out[i] = v;
}

int launch_dequant_b8(int wt, const WeightRef& w, uint64_t n_elems, float* out, float scale, bool with_scale, cudaStream_t st) {
    const unsigned grid = (unsigned)((n_elems + 255) / 256);
    if (wt == WT_Q8_0) k_dequant_b8<WT_Q8_0><<<grid, 256, 0, st>>>(w, out, n_elems, scale, with_scale ? 1 : 0);
    else k_dequant_b8<WT_Q5_0><<<grid, 256, 0, st>>>(w, out, n_elems, scale, with_scale ? 1 : 0);
    count_launch();
    return ADAMAH_OK;
}

// ---- GEMV -------------------------------------------------------------------------------------------------
// Byte i of a word of codes -> a float that holds the code exactly:
//   B8_CODE_LO: 2^23 + code (the byte sits in the low mantissa bits; any byte value; the caller subtracts 2^23 + offset);
//   B8_CODE_HI: 128 + code  (the byte sits at mantissa bits 16..23: codes below 128 only).  This one goes straight
//               into the FMA; the constant leaves afterwards through the block's pre-summed activations.
#define B8_CODE_LO(v, i) __uint_as_float(__byte_perm((v), 0x4B000000u, 0x7540u | (i)))
#define B8_CODE_HI(v, i) __uint_as_float(__byte_perm((v), 0x43000000u, 0x7054u | ((i) << 8)))

// {d0, d1} += {a0, a1} * {b0, b1} and {d0, d1} = {a0, a1} + {b0, b1} as one packed instruction each (sm_100)
__device__ __forceinline__ void add2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
#if ADAM_B200_F32X2
    asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rc, ra, rb;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t}"
        : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
#else
    d0 = a0 + b0; d1 = a1 + b1;
#endif
}

// 4 codes of two rows (ca, cb) against 4 activations of NB batch rows, read from shared memory once for both rows.
// EXACT: the codes are converted exactly (subtracting `bias` = 2^23 + offset); otherwise the products carry 128 + code.
template <int NB, bool EXACT>
__device__ __forceinline__ void b8_dot4x2(uint32_t ca, uint32_t cb, float bias, const float* __restrict__ xs, int xrow, float (&pa)[NB], float (&pb)[NB]) {
    float a[4], c[4];
    if (EXACT) {
        add2(a[0], c[0], B8_CODE_LO(ca, 0), B8_CODE_LO(cb, 0), -bias, -bias);
        add2(a[1], c[1], B8_CODE_LO(ca, 1), B8_CODE_LO(cb, 1), -bias, -bias);
        add2(a[2], c[2], B8_CODE_LO(ca, 2), B8_CODE_LO(cb, 2), -bias, -bias);
        add2(a[3], c[3], B8_CODE_LO(ca, 3), B8_CODE_LO(cb, 3), -bias, -bias);
    } else {
        a[0] = B8_CODE_HI(ca, 0); a[1] = B8_CODE_HI(ca, 1); a[2] = B8_CODE_HI(ca, 2); a[3] = B8_CODE_HI(ca, 3);
        c[0] = B8_CODE_HI(cb, 0); c[1] = B8_CODE_HI(cb, 1); c[2] = B8_CODE_HI(cb, 2); c[3] = B8_CODE_HI(cb, 3);
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
        const float4 xv = *reinterpret_cast<const float4*>(xs + b * xrow);
        fma2(pa[b], pb[b], a[0], c[0], xv.x, xv.x);
        fma2(pa[b], pb[b], a[1], c[1], xv.y, xv.y);
        fma2(pa[b], pb[b], a[2], c[2], xv.z, xv.z);
        fma2(pa[b], pb[b], a[3], c[3], xv.w, xv.w);
    }
}
// Bits 0..3 of t -> bit 4 of bytes 0..3 (the partial products t << 4, 11, 18, 25 land on distinct bits, so nothing carries).
__device__ __forceinline__ uint32_t q5_high(uint32_t t) { return ((t & 15u) * 0x02040810u) & 0x10101010u; }

template <int WT, int NB>
__global__ void __launch_bounds__(B8_THREADS) k_gemv_b8(const WeightRef w, const float* __restrict__ x, int ldx, float* __restrict__ y, int ldy,
                                                        int N, int K, int L, int logL) {
    extern __shared__ __align__(16) float xs[];
    const int nblk = K >> 5, xrow = nblk * B8_XSTRIDE;
    for (int b = 0; b < NB; ++b)
        for (int i = threadIdx.x; i < (K >> 2); i += B8_THREADS) {
            const float4 v = reinterpret_cast<const float4*>(x + (size_t)b * ldx)[i];
            *reinterpret_cast<float4*>(xs + b * xrow + (i >> 3) * B8_XSTRIDE + (i & 7) * 4) = v;
        }
    if (WT == WT_Q5_0) {
        // pad slot 0 of every staged block: the sum of its 32 activations (removes the 128 + 16 the codes carry)
        __syncthreads();
        for (int i = threadIdx.x; i < NB * nblk; i += B8_THREADS) {
            float* xb = xs + (i / nblk) * xrow + (i % nblk) * B8_XSTRIDE;
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) { const float4 v = *reinterpret_cast<const float4*>(xb + 4 * j); s0 += v.x; s1 += v.y; s2 += v.z; s3 += v.w; }
            xb[32] = (s0 + s1) + (s2 + s3);
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sub = lane & (L - 1), grp = lane >> logL;
    const int rpp = (32 >> logL) * 2, n_pass = (N + rpp - 1) / rpp;
    for (int pass = blockIdx.x * (B8_THREADS / 32) + warp; pass < n_pass; pass += gridDim.x * (B8_THREADS / 32)) {
        const int rowA = pass * rpp + grp * 2, rowB = rowA + 1;
        const size_t bA = (size_t)min(rowA, N - 1) * nblk, bB = (size_t)min(rowB, N - 1) * nblk;
        float accA[NB], accB[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) { accA[b] = 0.f; accB[b] = 0.f; }
#pragma unroll 2
        for (int blk = sub; blk < nblk; blk += L) {
            const float* xb = xs + blk * B8_XSTRIDE;
            float pa[NB], pb[NB];
#pragma unroll
            for (int b = 0; b < NB; ++b) { pa[b] = 0.f; pb[b] = 0.f; }
            const float dA = __half2float(w.d[bA + blk]), dB = __half2float(w.d[bB + blk]);
            if (WT == WT_Q8_0) {
                const uint4 a0 = __ldcs(w.q + (bA + blk) * 2), a1 = __ldcs(w.q + (bA + blk) * 2 + 1);
                const uint4 c0 = __ldcs(w.q + (bB + blk) * 2), c1 = __ldcs(w.q + (bB + blk) * 2 + 1);
                const uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                const uint32_t wb[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
                for (int i = 0; i < 8; ++i)     // int8 + 128 = an unsigned byte
                    b8_dot4x2<NB, true>(wa[i] ^ 0x80808080u, wb[i] ^ 0x80808080u, 8388608.f + 128.f, xb + 4 * i, xrow, pa, pb);
            } else {
                const uint4 a0 = __ldcs(w.q + bA + blk), c0 = __ldcs(w.q + bB + blk);
                const uint32_t ha = w.h[bA + blk], hb = w.h[bB + blk];
                const uint32_t wa[4] = {a0.x, a0.y, a0.z, a0.w}, wb[4] = {c0.x, c0.y, c0.z, c0.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t la = (wa[i] & 0x0F0F0F0Fu) | q5_high(ha >> (4 * i)), lb = (wb[i] & 0x0F0F0F0Fu) | q5_high(hb >> (4 * i));
                    b8_dot4x2<NB, false>(la, lb, 0.f, xb + 4 * i, xrow, pa, pb);
                    const uint32_t ua = ((wa[i] >> 4) & 0x0F0F0F0Fu) | q5_high(ha >> (16 + 4 * i)), ub = ((wb[i] >> 4) & 0x0F0F0F0Fu) | q5_high(hb >> (16 + 4 * i));
                    b8_dot4x2<NB, false>(ua, ub, 0.f, xb + 16 + 4 * i, xrow, pa, pb);
                }
            }
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (WT == WT_Q5_0) { const float off = 144.f * xb[b * xrow + 32]; pa[b] -= off; pb[b] -= off; }     // codes carried 128 + 16
                accA[b] = fmaf(dA, pa[b], accA[b]); accB[b] = fmaf(dB, pb[b], accB[b]);
            }
        }
        for (int o = L >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int b = 0; b < NB; ++b) { accA[b] += __shfl_xor_sync(0xffffffffu, accA[b], o); accB[b] += __shfl_xor_sync(0xffffffffu, accB[b], o); }
        }
        if (sub == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (rowA < N) y[(size_t)b * ldy + rowA] = accA[b];
                if (rowB < N) y[(size_t)b * ldy + rowB] = accB[b];
            }
        }
    }
}

template <int WT, int NB>
static int gemv_b8_launch(const WeightRef& w, const float* x, int ldx, float* y, int ldy, int N, int K, cudaStream_t st) {
    const int nblk = K >> 5;
    int L = 4, logL = 2;
    while (L < 32 && nblk / L > 16) { L <<= 1; ++logL; }
    const size_t smem = (size_t)NB * nblk * B8_XSTRIDE * 4;
    auto kern = k_gemv_b8<WT, NB>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return fail(ADAMAH_ERR_INVALID, "gemv (Q8_0 / Q5_0): K = %d is too wide for the staged activations", K);
    }
    const int rpp = (32 / L) * 2, n_pass = (N + rpp - 1) / rpp, want = (n_pass + B8_THREADS / 32 - 1) / (B8_THREADS / 32);
    const int per_sm = smem > 96 * 1024 ? 1 : smem > 48 * 1024 ? 2 : 4;
    const int grid = want < g.sm_count * per_sm ? want : g.sm_count * per_sm;
    kern<<<grid, B8_THREADS, smem, st>>>(w, x, ldx, y, ldy, N, K, L, logL);
    count_launch();
    return ADAMAH_OK;
}

int launch_gemv_b8(int wt, const WeightRef& w, const float* x, int ldx, float* y, int ldy, int N, int K, int B, cudaStream_t st) {
    if (!wt_is_b8(wt)) return fail(ADAMAH_ERR_INVALID, "gemv (Q8_0 / Q5_0): wrong weight type");
    if (N <= 0 || K <= 0 || B <= 0 || (K & 31)) return fail(ADAMAH_ERR_INVALID, "gemv (Q8_0 / Q5_0): K must be a positive multiple of 32");
    if (((uintptr_t)x & 15) || (ldx & 3)) return fail(ADAMAH_ERR_INVALID, "gemv (Q8_0 / Q5_0): activations must be 16-byte aligned");
    // batch rows in chunks of 4 / 2 / 1 (the weights of a chunk's rows are read once per chunk); wide K takes smaller chunks
    const size_t row_bytes = (size_t)(K >> 5) * B8_XSTRIDE * 4;
    if (row_bytes > 200 * 1024) return fail(ADAMAH_ERR_INVALID, "gemv (Q8_0 / Q5_0): K = %d is too wide", K);
    int rc = ADAMAH_OK;
    for (int b0 = 0; b0 < B && rc == ADAMAH_OK;) {
        int nb = B - b0 >= 4 ? 4 : B - b0 >= 2 ? 2 : 1;
        while (nb > 1 && nb * row_bytes > 200 * 1024) nb >>= 1;
        const float* xb = x + (size_t)b0 * ldx;
        float* yb = y + (size_t)b0 * ldy;
        if (wt == WT_Q8_0) rc = nb == 4 ? gemv_b8_launch<WT_Q8_0, 4>(w, xb, ldx, yb, ldy, N, K, st) : nb == 2 ? gemv_b8_launch<WT_Q8_0, 2>(w, xb, ldx, yb, ldy, N, K, st)
                                                                                                  : gemv_b8_launch<WT_Q8_0, 1>(w, xb, ldx, yb, ldy, N, K, st);
        else rc = nb == 4 ? gemv_b8_launch<WT_Q5_0, 4>(w, xb, ldx, yb, ldy, N, K, st) : nb == 2 ? gemv_b8_launch<WT_Q5_0, 2>(w, xb, ldx, yb, ldy, N, K, st)
                                                                                        : gemv_b8_launch<WT_Q5_0, 1>(w, xb, ldx, yb, ldy, N, K, st);
        b0 += nb;
    }
    return rc;
}

// ---- norm chain and arg-max as kernels of their own ---------------------------------------------------------
__global__ void __launch_bounds__(256) k_chain_rows(const float* __restrict__ h_in, const float* __restrict__ add_src, const float* __restrict__ w_post,
                                                    const float* __restrict__ w_pre, float* __restrict__ h_out, float* __restrict__ x_out, int E, float eps) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t o = (size_t)blockIdx.x * E;
    float r_post = 1.f;
    if (add_src && w_post) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < E; i += 256) { const float v = add_src[o + i]; ss = fmaf(v, v, ss); }
        r_post = sqrtf(block_sum(ss, red) / (float)E + eps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < E; i += 256) {
        float h = h_in[o + i];
        if (add_src) h += w_post ? add_src[o + i] / r_post * w_post[i] : add_src[o + i];
        h_out[o + i] = h;
        ss = fmaf(h, h, ss);
    }
    if (!w_pre) {
        for (int i = threadIdx.x; i < E; i += 256) x_out[o + i] = h_out[o + i];
        return;
    }
    const float r_pre = sqrtf(block_sum(ss, red) / (float)E + eps);
    for (int i = threadIdx.x; i < E; i += 256) x_out[o + i] = h_out[o + i] / r_pre * w_pre[i];     // the thread's own stores
}

int launch_chain_rows(const float* h_in, const float* add_src, const float* w_post, const float* w_pre, float* h_out, float* x_out,
                      int E, int rows, float eps, cudaStream_t st, bool pdl) {
    if (!h_in || !h_out || !x_out || h_out == h_in) return fail(ADAMAH_ERR_INVALID, "norm chain: missing buffer or h_out aliases h_in");
    launch_k(k_chain_rows, dim3(rows), dim3(256), 0, st, pdl, h_in, add_src, w_post, w_pre, h_out, x_out, E, eps);
    count_launch();
    return ADAMAH_OK;
}

__global__ void __launch_bounds__(1024) k_argmax_rows(float* __restrict__ logits, int V, float cap, int store_capped, int32_t* __restrict__ tok,
                                                      float* __restrict__ val, float* __restrict__ tok_f32) {
    __shared__ float sv[32]; __shared__ int si[32];
    pdl_launch_dependents();
    pdl_wait();
    float* lg = logits + (size_t)blockIdx.x * V;
    float bv = B8_SNEG; int bi = -1;
    for (int i = threadIdx.x; i < V; i += 1024) {
        float v = lg[i];
        if (!(v == v)) v = B8_SNEG;
        if (better(v, i, bv, bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { sv[warp] = bv; si[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        bv = sv[lane]; bi = si[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) {
            const int t = bi < 0 ? 0 : bi;
            if (tok) tok[blockIdx.x] = t;
            if (val) val[blockIdx.x] = bv;
            if (tok_f32) tok_f32[blockIdx.x] = (float)t;
        }
    }
    if (store_capped && cap > 0.f)
        for (int i = threadIdx.x; i < V; i += 1024) lg[i] = tanhf(lg[i] / cap) * cap;
}

int launch_argmax_rows(float* logits, int V, int rows, float cap, bool store_capped, int32_t* tok, float* val, float* tok_f32,
                       cudaStream_t st, bool pdl) {
    launch_k(k_argmax_rows, dim3(rows), dim3(1024), 0, st, pdl, logits, V, cap, store_capped ? 1 : 0, tok, val, tok_f32);
    count_launch();
    return ADAMAH_OK;
}

}  // namespace ab
