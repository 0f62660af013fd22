// Tensor-core variant of the Q4_0 dequant GEMV over row-tiled weights (tile.cu).
//
// Why tensor cores in a memory-bound GEMV: on the plain CUDA-core path the unpack
// (one byte-permute per weight, on the half-rate integer pipe) and one FMA per weight
// cap the kernel at about half of HBM bandwidth.  Here a 16-row x 32-weight block is
// one integer MMA (mma.sync.m16n8k32, u8 x s8 -> s32) per activation operand:
//   * weights enter as the raw nibbles 0..15 (u8): two logic ops split a 32-bit word
//     into its four low and four high nibbles, which are exactly the A registers;
//   * the activation vector is scaled by a power of two s (chosen per vector so that
//     |x*s| <= 2^22), rounded to an integer and split into three signed bytes
//     x*s = hi*65536 + mid*256 + lo, i.e. 23 bits of every activation are kept; the
//     B operand of the first MMA holds the (hi, mid) columns, the second the lo column;
//   * the block's exact integer sums are recombined in fp32, the -8 offset of Q4_0 is
//     removed with the pre-summed activations of the block, and the result is scaled
//     by the block scale d and accumulated in fp32 on the CUDA cores.
// The tensor pipe stays almost idle: the kernel is a stream over the weight bytes.
//
// Columns of the 8-wide B operand: (2b, 2b+1) = (hi, mid) [first MMA] or (lo, 0)
// [second MMA] of batch row b, b < 4.  With one batch row only columns 0,1 are staged.
// A warp owns one 16-row group and a slice of K; the KS warps that share a row group
// combine through shared memory.  Lane (g, t) = (lane/4, lane%4) holds rows g and g+8
// for batch row t.  Weight tiles reach shared memory through a per-warp ring of bulk
// copies (cp.async.bulk + mbarrier), so no load scoreboard limits the bytes in flight.
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace ab {

struct MmaSlot { uint4 q; uint2 sc; };

// D = A(u8, 16x32) * B(s8, 32x8) with a zero accumulator input.
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Staged activation bytes: block u (32 activations), column c, quad lane t -> 8 bytes
// { k = 4t..4t+3 , k = 16+4t..16+4t+3 } which are the two B registers of lane (c, t).
template <int NCOL>
__device__ __forceinline__ int xb_index(int k, int col) {
    const int u = k >> 5, w = k & 31;
    return ((u * NCOL + col) * 4 + ((w & 15) >> 2)) * 8 + (w >> 4) * 4 + (w & 3);
}

// x*s rounded to an integer and split into three signed bytes (hi, mid, lo).
template <int NCOL>
__device__ __forceinline__ void put_x(signed char* xb1, signed char* xb2, int k, int b, float v_scaled) {
    const int xi = __float2int_rn(v_scaled);
    const int lo = ((xi + 128) & 0xFF) - 128;
    const int r = (xi - lo) >> 8;
    const int mid = ((r + 128) & 0xFF) - 128;
    const int hi = (r - mid) >> 8;
    xb1[xb_index<NCOL>(k, 2 * b)] = (signed char)hi;
    xb1[xb_index<NCOL>(k, 2 * b + 1)] = (signed char)mid;
    xb2[xb_index<NCOL>(k, 2 * b)] = (signed char)lo;
}

// Four consecutive activations (k0 a multiple of 4) at once: they share one 32-bit word
// in each of the three byte planes.
template <int NCOL>
__device__ __forceinline__ void put_x4(signed char* xb1, signed char* xb2, int k0, int b, float4 v) {
    const float f[4] = {v.x, v.y, v.z, v.w};
    uint32_t wh = 0, wm = 0, wl = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int xi = __float2int_rn(f[i]);
        const int lo = ((xi + 128) & 0xFF) - 128;
        const int r = (xi - lo) >> 8;
        const int mid = ((r + 128) & 0xFF) - 128;
        const int hi = (r - mid) >> 8;
        wh |= (uint32_t)(hi & 0xFF) << (8 * i); wm |= (uint32_t)(mid & 0xFF) << (8 * i); wl |= (uint32_t)(lo & 0xFF) << (8 * i);
    }
    *reinterpret_cast<uint32_t*>(xb1 + xb_index<NCOL>(k0, 2 * b)) = wh;
    *reinterpret_cast<uint32_t*>(xb1 + xb_index<NCOL>(k0, 2 * b + 1)) = wm;
    *reinterpret_cast<uint32_t*>(xb2 + xb_index<NCOL>(k0, 2 * b)) = wl;
}

// Power-of-two scale that brings amax to at most 2^22 (and its inverse).
__device__ __forceinline__ void pow2_scale(float amax, float& s, float& inv) {
    if (!(amax > 0.f) || !(amax < 3.0e38f)) { s = 1.f; inv = 1.f; return; }
    // amax = m * 2^e with m in [0.5, 1)  (denormals count as e = -126)
    int e = (int)((__float_as_uint(amax) >> 23) & 0xFFu) - 126;
    e = max(-100, min(100, 22 - e));
    s = __uint_as_float((uint32_t)(127 + e) << 23);
    inv = __uint_as_float((uint32_t)(127 - e) << 23);
}

// Block-wide sum of `sv` and maximum of `mv` in one pass (red: 66 floats).
__device__ __forceinline__ void block_sum_max(float& sv, float& mv, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sv += __shfl_xor_sync(0xffffffffu, sv, o);
        mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
    }
    __syncthreads();
    if (lane == 0) { red[warp] = sv; red[33 + warp] = mv; }
    __syncthreads();
    float a = 0.f, m = -3.402823466e+38f;
    for (int w = 0; w < nw; ++w) { a += red[w]; m = fmaxf(m, red[33 + w]); }
    sv = a; mv = m;
}

// ---- bulk-copy pipeline primitives (cp.async.bulk + mbarrier, all waits bounded) ----
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Wait for the phase with the given parity; gives up after a bounded number of polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (int spin = 0; spin < (1 << 20); ++spin) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

constexpr int MMA_CH = 3;                  // tile pairs per bulk copy
constexpr int MMA_TILE = 576;              // bytes per tile pair

template <int NCOL, bool PAIR>
__global__ void __launch_bounds__(256, 2) k_gemv_mma(const GemvArgs a, const uint8_t* __restrict__ t0, const uint8_t* __restrict__ t1, int KS) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float s_red[2][8][PAIR ? 2 : 1][16][4];
    __shared__ float s_inv[4];
    __shared__ float red[66];
    __shared__ float s_bv[8 * 4];
    __shared__ int   s_bi[8 * 4];
    __shared__ bool  s_last;
    constexpr int NB = NCOL / 2;
    constexpr int MMA_PF = PAIR ? 3 : 6;       // tile pairs in flight per warp and matrix
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int RG = n_warps / KS, rg_l = warp / KS, ks = warp % KS;
    const int pairs = a.K >> 6, units = a.K >> 5;
    const int n_rg = a.N >> 4;
    const int n_sets = (n_rg + RG - 1) / RG;
    const int p0 = (int)((long long)ks * pairs / KS), p1 = (int)((long long)(ks + 1) * pairs / KS), np = p1 - p0;
    const int my_sets = (n_sets > (int)blockIdx.x) ? (n_sets - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int T = my_sets * np;

    // ---- weight stream: every warp runs its own ring of bulk copies into shared memory ----
    // Stage = MMA_CH consecutive tile pairs of the warp's row group (contiguous in memory),
    // one cp.async.bulk per matrix, completion counted on the stage's mbarrier.
    constexpr int NSTAGE = PAIR ? 2 : 4;
    constexpr int STAGE_BYTES = MMA_CH * MMA_TILE * (PAIR ? 2 : 1);
    __shared__ __align__(8) uint64_t s_bar[8][NSTAGE];
    // staged activations: (hi, mid) bytes, lo bytes, per-block integer sums
    signed char* xb1 = reinterpret_cast<signed char*>(smem_raw);
    signed char* xb2 = xb1 + (size_t)units * NCOL * 32;
    float* s_sx = reinterpret_cast<float*>(smem_raw + (size_t)units * NCOL * 64);          // [units][NB]
    unsigned char* ring = smem_raw + (((size_t)units * (NCOL * 64 + NB * 4) + 127) & ~(size_t)127) + (size_t)warp * NSTAGE * STAGE_BYTES;
    const int nch = (np + MMA_CH - 1) / MMA_CH;             // chunks per row group for this warp
    const int n_chunks = my_sets * nch;
    if (lane == 0) {
#pragma unroll
        for (int st = 0; st < NSTAGE; ++st) mbar_init(&s_bar[warp][st], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    // issue cursor (lane 0): chunk `i_c` is chunk `i_j` of this warp's `i_set`-th row group
    int i_c = 0, i_j = 0, i_rg = (int)blockIdx.x * RG + rg_l;
    auto issue_next = [&]() {                                // lane 0 only
        const int rg = min(i_rg, n_rg - 1);                 // clamped: rows past the end are dropped later
        const int pp0 = p0 + i_j * MMA_CH, n = min(MMA_CH, p1 - pp0);
        const size_t off = ((size_t)rg * pairs + pp0) * MMA_TILE;
        const int st = i_c & (NSTAGE - 1);
        unsigned char* dst = ring + (size_t)st * STAGE_BYTES;
        mbar_expect_tx(&s_bar[warp][st], (uint32_t)(n * MMA_TILE * (PAIR ? 2 : 1)));
        bulk_g2s(dst, t0 + off, (uint32_t)(n * MMA_TILE), &s_bar[warp][st]);
        if (PAIR) bulk_g2s(dst + MMA_CH * MMA_TILE, t1 + off, (uint32_t)(n * MMA_TILE), &s_bar[warp][st]);
        ++i_c;
        if (++i_j == nch) { i_j = 0; i_rg += (int)gridDim.x * RG; }
    };
    if (lane == 0) {
#pragma unroll
        for (int c = 0; c < NSTAGE; ++c) if (i_c < n_chunks) issue_next();
    }

    // Norm weights of the input chain (read-only, like the matrix): fetched ahead of the wait.
    float4 vp[3], vw[3];
    {
        const float4 o4 = make_float4(1.f, 1.f, 1.f, 1.f);
        const int n4 = a.K >> 2;
        const bool chain = a.h_in && n4 <= 3 * (int)blockDim.x;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const int i = threadIdx.x + j * blockDim.x;
            const bool in = chain && i < n4;
            vp[j] = (in && a.add_src && a.w_post) ? reinterpret_cast<const float4*>(a.w_post)[i] : o4;
            vw[j] = (in && a.w_pre) ? reinterpret_cast<const float4*>(a.w_pre)[i] : o4;
        }
    }
    // Everything above touches only read-only weights; the activations come from the
    // previous kernel.
    pdl_launch_dependents();
    pdl_wait();
    // ---- stage activations as signed bytes (hi, mid | lo) in MMA operand order ----
    {
        const int n4 = a.K >> 2;
        for (int b = 0; b < NB && b < a.B; ++b) {
            const size_t row = (size_t)b * a.ldx;
            if (a.h_in && n4 <= 3 * (int)blockDim.x) {
                const float* hp = a.h_in + row;
                const float* ap = a.add_src ? a.add_src + row : nullptr;
                float4 va[3], vh[3];
                const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int i = threadIdx.x + j * blockDim.x;
                    const bool in = i < n4;
                    vh[j] = in ? reinterpret_cast<const float4*>(hp)[i] : z4;
                    va[j] = (in && ap) ? reinterpret_cast<const float4*>(ap)[i] : z4;
                }
                float rms_a = 1.f;
                if (ap && a.w_post) {
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < 3; ++j) { ss = fmaf(va[j].x, va[j].x, ss); ss = fmaf(va[j].y, va[j].y, ss); ss = fmaf(va[j].z, va[j].z, ss); ss = fmaf(va[j].w, va[j].w, ss); }
                    ss = block_sum(ss, red);
                    rms_a = sqrtf(ss / (float)a.K + a.eps);
                }
                const float rcp_a = __frcp_rn(rms_a);
                // h' and, in the same reduction, its sum of squares and max |h' * w_pre|
                float ss = 0.f, am = 0.f;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    if (ap) {
                        if (a.w_post) {
                            vh[j].x += div_by(va[j].x, rms_a, rcp_a) * vp[j].x; vh[j].y += div_by(va[j].y, rms_a, rcp_a) * vp[j].y;
                            vh[j].z += div_by(va[j].z, rms_a, rcp_a) * vp[j].z; vh[j].w += div_by(va[j].w, rms_a, rcp_a) * vp[j].w;
                        } else { vh[j].x += va[j].x; vh[j].y += va[j].y; vh[j].z += va[j].z; vh[j].w += va[j].w; }
                    }
                    ss = fmaf(vh[j].x, vh[j].x, ss); ss = fmaf(vh[j].y, vh[j].y, ss); ss = fmaf(vh[j].z, vh[j].z, ss); ss = fmaf(vh[j].w, vh[j].w, ss);
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(vh[j].x * vw[j].x), fabsf(vh[j].y * vw[j].y)), fmaxf(fabsf(vh[j].z * vw[j].z), fabsf(vh[j].w * vw[j].w))));
                    const int i = threadIdx.x + j * blockDim.x;
                    if (i < n4 && a.h_out && blockIdx.x == 0) reinterpret_cast<float4*>(a.h_out + row)[i] = vh[j];
                }
                block_sum_max(ss, am, red);
                float rms = 1.f;
                if (a.w_pre) {
                    rms = sqrtf(ss / (float)a.K + a.eps);
                    const float rcp = __frcp_rn(rms);
                    am = am * rcp * 1.000001f;             // bound on max |x| (the scale has a factor 2 to spare)
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        vh[j].x = div_by(vh[j].x, rms, rcp) * vw[j].x; vh[j].y = div_by(vh[j].y, rms, rcp) * vw[j].y;
                        vh[j].z = div_by(vh[j].z, rms, rcp) * vw[j].z; vh[j].w = div_by(vh[j].w, rms, rcp) * vw[j].w;
                    }
                }
                float s, inv;
                pow2_scale(am, s, inv);
                if (threadIdx.x == 0) s_inv[b] = inv;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int i = threadIdx.x + j * blockDim.x;
                    if (i < n4) put_x4<NCOL>(xb1, xb2, 4 * i, b, make_float4(vh[j].x * s, vh[j].y * s, vh[j].z * s, vh[j].w * s));
                }
            } else {
                // plain activations: read once into registers when they fit (K <= 8192), scale, pack
                const float4* src = reinterpret_cast<const float4*>(a.x + row);
                float am = 0.f;
                float s, inv;
                if (n4 <= 8 * (int)blockDim.x) {
                    float4 v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int i = threadIdx.x + j * blockDim.x;
                        v[j] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j) am = fmaxf(am, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
                    am = block_max(am, red);
                    pow2_scale(am, s, inv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int i = threadIdx.x + j * blockDim.x;
                        if (i < n4) put_x4<NCOL>(xb1, xb2, 4 * i, b, make_float4(v[j].x * s, v[j].y * s, v[j].z * s, v[j].w * s));
                    }
                } else {
#pragma unroll 4
                    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                        const float4 v = src[i];
                        am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                    }
                    am = block_max(am, red);
                    pow2_scale(am, s, inv);
#pragma unroll 4
                    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                        const float4 v = src[i];
                        put_x4<NCOL>(xb1, xb2, 4 * i, b, make_float4(v.x * s, v.y * s, v.z * s, v.w * s));
                    }
                }
                if (threadIdx.x == 0) s_inv[b] = inv;
            }
        }
        __syncthreads();
    }

    // per-block sums of the integer activations (they remove the -8 of Q4_0 later)
    for (int i = threadIdx.x; i < units * NB; i += blockDim.x) {
        const int u = i / NB, b = i % NB;
        int acc = 0;
        if (b < a.B) {
            const int* h = reinterpret_cast<const int*>(xb1 + (size_t)(u * NCOL + 2 * b) * 32);
            const int* m = h + 8;
            const int* l = reinterpret_cast<const int*>(xb2 + (size_t)(u * NCOL + 2 * b) * 32);
            int sh = 0, sm2 = 0, sl = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) { sh = __dp4a(h[e], 0x01010101, sh); sm2 = __dp4a(m[e], 0x01010101, sm2); sl = __dp4a(l[e], 0x01010101, sl); }
            acc = sm2 * 256 + sl;
            s_sx[i] = (float)sh * 65536.0f + (float)acc;
        } else s_sx[i] = 0.f;
    }
    __syncthreads();
    float best_v = -3.402823466e+38f; int best_i = -1;        // for batch row t
    float accA[2] = {0.f, 0.f}, accB[2] = {0.f, 0.f};
    int parity = 0;
    // Lanes g >= NCOL supply all-zero B columns: they read a zero block with stride 0.
    __shared__ __align__(16) uint4 s_zero[4];
    if (threadIdx.x < 4) s_zero[threadIdx.x] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    // Lane (g, t) supplies B column g.  Only columns < NCOL are staged; the other lanes
    // re-read a staged column: whatever lands in B columns >= 2*B only reaches output
    // columns that are never read.
    const uint2* xq1 = reinterpret_cast<const uint2*>(xb1) + (g % NCOL) * 4 + t;
    const uint2* xq2 = reinterpret_cast<const uint2*>(xb2) + (g % NCOL) * 4 + t;
    constexpr int xstep = NCOL * 4;                            // uint2 per block
    const float* sxp = s_sx + (t < NB ? t : 0);

    // One 16x32 block of one matrix: raw nibbles against (hi, mid) and against (lo, 0).
    auto block_imma = [&](uint32_t wg, uint32_t wh, const uint2& b1, const uint2& b2, uint32_t sc2, float sx, float& acc0, float& acc1) {
        const uint32_t a0 = wg & 0x0F0F0F0Fu, a2 = (wg >> 4) & 0x0F0F0F0Fu;
        const uint32_t a1 = wh & 0x0F0F0F0Fu, a3 = (wh >> 4) & 0x0F0F0F0Fu;
        int d1[4], d2[4];
        imma16832(d1, a0, a1, a2, a3, b1.x, b1.y);
        imma16832(d2, a0, a1, a2, a3, b2.x, b2.y);
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&sc2));
        const float s0 = fmaf((float)d1[0], 65536.0f, (float)(d1[1] * 256 + d2[0]));
        const float s1 = fmaf((float)d1[2], 65536.0f, (float)(d1[3] * 256 + d2[2]));
        acc0 = fmaf(d.x, fmaf(-8.0f, sx, s0), acc0);
        acc1 = fmaf(d.y, fmaf(-8.0f, sx, s1), acc1);
    };

    bool timed_out = false;
    int j = 0, c_rg = (int)blockIdx.x * RG + rg_l;
    for (int c = 0; c < n_chunks; ++c) {
        const int st = c & (NSTAGE - 1);
        if (!timed_out) {
            const bool ok = mbar_wait(&s_bar[warp][st], (uint32_t)((c / NSTAGE) & 1));
            if (!__all_sync(0xffffffffu, ok)) {
                // A copy never completed.  Record it and stop touching the ring; the warp keeps
                // walking its chunks so that it still meets its peers at every CTA barrier.
                timed_out = true;
                if (lane == 0) atomicOr(a.err, DEVERR_WAIT);
            }
        }
        if (!timed_out) {
            const unsigned char* buf = ring + (size_t)st * STAGE_BYTES;
            const int pp0 = p0 + j * MMA_CH, n = min(MMA_CH, p1 - pp0);
            const uint2* xp1 = xq1 + (size_t)pp0 * 2 * xstep;
            const uint2* xp2 = xq2 + (size_t)pp0 * 2 * xstep;
            const float* sx = sxp + (size_t)pp0 * 2 * NB;
#pragma unroll
            for (int k = 0; k < MMA_CH; ++k) {
                if (k < n) {
                    const uint4 q = reinterpret_cast<const uint4*>(buf + k * MMA_TILE)[lane];
                    const uint2 sc = reinterpret_cast<const uint2*>(buf + k * MMA_TILE + 512)[g];
                    const uint2 b10 = xp1[(2 * k) * xstep], b11 = xp1[(2 * k + 1) * xstep];
                    const uint2 b20 = xp2[(2 * k) * xstep], b21 = xp2[(2 * k + 1) * xstep];
                    const float sx0 = sx[(2 * k) * NB], sx1 = sx[(2 * k + 1) * NB];
                    block_imma(q.x, q.y, b10, b20, sc.x, sx0, accA[0], accA[1]);
                    block_imma(q.z, q.w, b11, b21, sc.y, sx1, accA[0], accA[1]);
                    if (PAIR) {
                        const uint4 q1 = reinterpret_cast<const uint4*>(buf + (MMA_CH + k) * MMA_TILE)[lane];
                        const uint2 sc1 = reinterpret_cast<const uint2*>(buf + (MMA_CH + k) * MMA_TILE + 512)[g];
                        block_imma(q1.x, q1.y, b10, b20, sc1.x, sx0, accB[0], accB[1]);
                        block_imma(q1.z, q1.w, b11, b21, sc1.y, sx1, accB[0], accB[1]);
                    }
                }
            }
            __syncwarp();                                   // every lane is done with this stage
            if (lane == 0 && i_c < n_chunks) issue_next();
        }
        if (++j == nch) {
            // ---- end of this warp's K slice for the row group ----
            const int rg = c_rg;
            j = 0;
            c_rg += (int)gridDim.x * RG;
            float vA[2] = {accA[0], accA[1]}, vB[2] = {accB[0], accB[1]};
            bool writer = true;
            if (KS > 1) {       // combine the KS slices through shared memory
                float* mine = &s_red[parity][warp][0][0][0];
                mine[g * 4 + t] = accA[0]; mine[(g + 8) * 4 + t] = accA[1];
                if (PAIR) { mine[64 + g * 4 + t] = accB[0]; mine[64 + (g + 8) * 4 + t] = accB[1]; }
                __syncthreads();
                writer = (ks == 0);
                if (writer) {
                    for (int k2 = 1; k2 < KS; ++k2) {
                        const float* o = &s_red[parity][warp + k2][0][0][0];
                        vA[0] += o[g * 4 + t]; vA[1] += o[(g + 8) * 4 + t];
                        if (PAIR) { vB[0] += o[64 + g * 4 + t]; vB[1] += o[64 + (g + 8) * 4 + t]; }
                    }
                }
                parity ^= 1;
            }
            if (writer && rg < n_rg && t < a.B) {
                const float inv = s_inv[t];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rg * 16 + g + 8 * h;
                    const float va = vA[h] * inv;
                    if (a.epi == EPI_STORE) a.y[(size_t)t * a.ldy + row] = va;
                    else if (a.epi == EPI_GEGLU) a.y[(size_t)t * a.ldy + row] = gelu_tanh(va) * (vB[h] * inv);
                    else if (a.epi == EPI_SWIGLU) a.y[(size_t)t * a.ldy + row] = silu_clip(va) * (vB[h] * inv);
                    else {
                        float v = va;
                        if (a.y) a.y[(size_t)t * a.ldy + row] = a.softcap > 0.f ? tanhf(v / a.softcap) * a.softcap : v;
                        if (!(v == v)) v = -3.402823466e+38f;
                        if (better(v, row, best_v, best_i)) { best_v = v; best_i = row; }
                    }
                }
            }
            accA[0] = accA[1] = accB[0] = accB[1] = 0.f;
        }
    }
    if (timed_out) {
        // give the copies still in flight a bounded chance to land before the CTA's shared memory is released
        for (int st = 0; st < NSTAGE; ++st) { mbar_wait(&s_bar[warp][st], 0u); mbar_wait(&s_bar[warp][st], 1u); }
    }

    if (a.epi != EPI_ARGMAX) return;
    // lanes that share a batch row (same t) -> lane g == 0; then across warps; then across CTAs
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
    }
    if (g == 0) { s_bv[warp * 4 + t] = best_v; s_bi[warp * 4 + t] = best_i; }
    __syncthreads();
    if ((int)threadIdx.x < a.B && threadIdx.x < 4) {
        const int b = threadIdx.x;
        float bv = s_bv[b]; int bi = s_bi[b];
        for (int w = 1; w < n_warps; ++w) if (better(s_bv[w * 4 + b], s_bi[w * 4 + b], bv, bi)) { bv = s_bv[w * 4 + b]; bi = s_bi[w * 4 + b]; }
        a.part_val[(size_t)b * gridDim.x + blockIdx.x] = bv;
        a.part_idx[(size_t)b * gridDim.x + blockIdx.x] = bi;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int b = 0; b < a.B && b < 4; ++b) {
        float bv = -3.402823466e+38f; int bi = -1;
        for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
            const float v = __ldcg(a.part_val + (size_t)b * gridDim.x + i);
            const int k = __ldcg(a.part_idx + (size_t)b * gridDim.x + i);
            if (better(v, k, bv, bi)) { bv = v; bi = k; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        __syncthreads();
        if (lane == 0) { s_bv[warp] = bv; s_bi[warp] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < n_warps; ++w) if (better(s_bv[w], s_bi[w], bv, bi)) { bv = s_bv[w]; bi = s_bi[w]; }
            const int tok = bi < 0 ? 0 : bi;
            if (a.out_tok) a.out_tok[b] = tok;
            if (a.out_tok_f32) a.out_tok_f32[b] = (float)tok;
        }
    }
    if (threadIdx.x == 0) *a.ticket = 0u;
}

// Launch on `stream` with tiled weights t0 (and t1 for GeGLU/SwiGLU).  Returns
// ADAMAH_ERR_INVALID without launching when the shape does not fit this kernel
// (the caller then uses the generic kernel): needs N % 16 == 0, K % 64 == 0, and
// either plain x or an input chain short enough for the register-resident path.
int launch_gemv_mma(const uint8_t* t0, const uint8_t* t1, GemvArgs a, cudaStream_t stream);
bool gemv_mma_supports(const GemvArgs& a);
const void* find_tiled(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols);
const void* find_tiled_prefix(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols);
int tile_tensor(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols);
void tiled_drop_map(uint32_t map_id);

}  // namespace ab
