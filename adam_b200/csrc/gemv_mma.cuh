// Tensor-core variant of the Q4_0 / Q4_K dequant GEMV over row-tiled weights (tile.cu).
//
// Why tensor cores in a memory-bound GEMV: on the plain CUDA-core path the unpack
// (one byte-permute per weight, on the half-rate integer pipe) and one FMA per weight
// cap the kernel at about half of HBM bandwidth.  Here a 16-row x 32-weight block is
// ONE integer MMA (mma.sync.m16n8k32, u8 x s8 -> s32):
//   * weights enter as the raw nibbles 0..15 (u8): three logic ops split a 32-bit word
//     into its four low and four high nibbles, which are exactly the A registers;
//   * the activation vector is scaled by a power of two s (chosen per vector so that
//     |x*s| <= 2^22), rounded to an integer and split into three signed bytes
//     x*s = hi*65536 + mid*256 + lo, i.e. 23 bits of every activation are kept.  The
//     8-wide B operand holds, for up to two batch rows, the columns (hi, mid, lo, 0);
//   * lane (g, t) = (lane/4, lane%4) receives rows g and g+8 of column pair t: an even
//     t sees (hi, mid), an odd t sees (lo, 0), and both form v = d0*256 + d1 in integer
//     arithmetic (exact), convert it once, remove the -8 offset of Q4_0 with the block's
//     pre-summed activations (kept in the same units), scale by the block scale d and
//     accumulate in fp32.  Even and odd lanes differ by the constant factor 65536, which
//     is applied once per row group when the two are added.
// The tensor pipe stays almost idle: the kernel is a stream over the weight bytes.
//
// Q4_K blocks go through the same MMA; their tile carries the 6-bit scale and min as bytes
// and the superblock's (d, dmin) per row, the block scale is d*sc and the offset term
// -(dmin*m)*sum(x) replaces -8*d*sum(x).
//
// Batch rows 2i and 2i+1 use MMA i of a block (NI = 1 or 2 MMAs per block, four rows per
// group); a call with more rows runs its groups as the fast grid dimension of one launch.
// A warp owns one 16-row group and a slice of K; the KS warps that share a row group
// combine through shared memory.  Weight tiles reach shared memory through a per-warp
// ring of bulk copies (cp.async.bulk + mbarrier), so no load scoreboard limits the
// bytes in flight; every wait on the ring is bounded.
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace ab {

// D = A(u8, 16x32) * B(s8, 32x8) with a zero accumulator input.
__device__ __forceinline__ void imma16832(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0), "r"(0), "r"(0), "r"(0));
}

// Staged activation bytes: block u (32 activations), column c, quad lane t -> 8 bytes
// { k = 4t..4t+3 , k = 16+4t..16+4t+3 } which are the two B registers of lane (c, t).
// NCOL columns are staged per block: 4 (one batch row), 8 (two) or 16 (up to four).
template <int NCOL>
__device__ __forceinline__ int xb_index(int k, int col) {
    const int u = k >> 5, w = k & 31;
    return ((u * NCOL + col) * 4 + ((w & 15) >> 2)) * 8 + (w >> 4) * 4 + (w & 3);
}

// Four scaled activations (integers of at most 23 bits after rounding) as three words of signed bytes: x = hi * 65536 +
// mid * 256 + lo with mid, lo in [-128, 127].  Adding 0x808080 makes every digit of the base-256 representation its value
// plus 128 (the carries of the signed digits are those of the addition); flipping bit 7 of each byte turns that into the
// two's-complement byte.  Then a 4 x 3 byte transpose.
__device__ __forceinline__ void split_x4(const float (&f)[4], bool active, uint32_t& wh, uint32_t& wm, uint32_t& wl) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = active ? (((uint32_t)__float2int_rn(f[i]) + 0x00808080u) ^ 0x00808080u) : 0u;
    wl = __byte_perm(__byte_perm(w[0], w[1], 0x0040), __byte_perm(w[2], w[3], 0x0040), 0x5410);
    wm = __byte_perm(__byte_perm(w[0], w[1], 0x0051), __byte_perm(w[2], w[3], 0x0051), 0x5410);
    wh = __byte_perm(__byte_perm(w[0], w[1], 0x0062), __byte_perm(w[2], w[3], 0x0062), 0x5410);
}

// Four consecutive scaled activations (k0 a multiple of 4) of batch row b: round to
// integers, split into three signed bytes each, and store one 32-bit word into each
// of the row's four columns (hi, mid, lo, zero).
template <int NCOL>
__device__ __forceinline__ void put_x4(signed char* xb, int k0, int b, float4 v) {
    const float f[4] = {v.x, v.y, v.z, v.w};
    uint32_t wh, wm, wl;
    split_x4(f, true, wh, wm, wl);
    const int c0 = 4 * b;
    const int i0 = xb_index<NCOL>(k0, c0);          // columns of one block are 32 bytes apart
    *reinterpret_cast<uint32_t*>(xb + i0) = wh;
    *reinterpret_cast<uint32_t*>(xb + i0 + 32) = wm;
    *reinterpret_cast<uint32_t*>(xb + i0 + 64) = wl;
    *reinterpret_cast<uint32_t*>(xb + i0 + 96) = 0u;
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

// CTA-wide reductions with ONE barrier each: warp results go to `buf` (32 floats that no other reduction in
// flight uses), every warp then folds them itself.
__device__ __forceinline__ float cta_sum1(float v, float* buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    return warp_sum(lane < nw ? buf[lane] : 0.f);
}
__device__ __forceinline__ float cta_max1(float v, float* buf) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (lane == 0) buf[warp] = v;
    __syncthreads();
    return warp_max(lane < nw ? buf[lane] : -3.402823466e+38f);
}
__device__ __forceinline__ void cta_sum_max1(float& sv, float& mv, float* bs, float* bm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sv += __shfl_xor_sync(0xffffffffu, sv, o);
        mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
    }
    if (lane == 0) { bs[warp] = sv; bm[warp] = mv; }
    __syncthreads();
    sv = lane < nw ? bs[lane] : 0.f; mv = lane < nw ? bm[lane] : -3.402823466e+38f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        sv += __shfl_xor_sync(0xffffffffu, sv, o);
        mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
    }
}

// put_x4 plus the block's pre-summed columns: the eight lanes that hold the 32 activations of one block add
// their bytes and lane 0 of the eight stores sxf * (256 * sum(hi) + sum(mid)) and sxf * 256 * sum(lo), the two
// values the MMA lanes of batch row b subtract (s_sx[u * NCOL/2 + 2b], [.. + 2b + 1]).  Called by whole warps
// (k0 = 4 * (float4 index), consecutive over the lanes); `active` is uniform over each group of eight lanes.
template <int NCOL>
__device__ __forceinline__ void put_x4_sums(signed char* xb, float* s_sx, int k0, int b, float4 v, bool active, float sxf) {
    const float f[4] = {v.x, v.y, v.z, v.w};
    uint32_t wh, wm, wl;
    split_x4(f, active, wh, wm, wl);
    if (active) {
        const int i0 = xb_index<NCOL>(k0, 4 * b);
        *reinterpret_cast<uint32_t*>(xb + i0) = wh;
        *reinterpret_cast<uint32_t*>(xb + i0 + 32) = wm;
        *reinterpret_cast<uint32_t*>(xb + i0 + 64) = wl;
        *reinterpret_cast<uint32_t*>(xb + i0 + 96) = 0u;
    }
    int sh = __dp4a((int)wh, 0x01010101, 0), sm = __dp4a((int)wm, 0x01010101, 0), sl = __dp4a((int)wl, 0x01010101, 0);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        sh += __shfl_xor_sync(0xffffffffu, sh, o);
        sm += __shfl_xor_sync(0xffffffffu, sm, o);
        sl += __shfl_xor_sync(0xffffffffu, sl, o);
    }
    if (active && (threadIdx.x & 7) == 0)
        *reinterpret_cast<float2*>(s_sx + (size_t)(k0 >> 5) * (NCOL / 2) + 2 * b) = make_float2(sxf * (float)(sh * 256 + sm), sxf * (float)(sl * 256));
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

// bytes per tile pair (16 rows x 64 weights): 512 nibble bytes + 32 fp16 scales (Q4_0), or
// + 64 bytes of 6-bit scales/mins as bytes + 64 bytes of fp16 (d, dmin) per row (Q4_K)
constexpr int mma_tile_bytes(int wt) { return wt == WT_Q4_0 ? 576 : 640; }
constexpr int MMA_NSTAGE = 3;              // ring stages per warp (2 in the instance for long activation vectors, which leave less shared memory)
constexpr int MMA_MAX_WARPS = 16;
template <bool PAIR, int WT> struct MmaGeo {
    static constexpr int TILE = mma_tile_bytes(WT);
    static constexpr int CH = WT == WT_Q4_0 ? (PAIR ? 3 : 6) : (PAIR ? 2 : 4);   // tile pairs per stage and matrix
    static constexpr int STAGE_BYTES = CH * TILE * (PAIR ? 2 : 1);               // 3456 (Q4_0), 2560 (Q4_K)
};
constexpr int mma_ring_bytes_per_warp(int wt, int n_stage = MMA_NSTAGE) { return n_stage * (wt == WT_Q4_0 ? 6 * 576 : 4 * 640); }

#ifdef ADAM_B200_STEP_TRACE
#define GM_STAMP(slot) do { if (threadIdx.x == 0 && blockIdx.y < 8 && blockIdx.x == 0) STEP_STAMP(a_in.trace, blockIdx.y * 8 + (slot)); } while (0)
#else
#define GM_STAMP(slot) do { } while (0)
#endif
template <int NCOL, bool PAIR, int WT, int NST = MMA_NSTAGE>      // NST: ring stages per warp
__global__ void __launch_bounds__(512, 1) k_gemv_mma(const GemvArgs a_in, const uint8_t* __restrict__ t0, const uint8_t* __restrict__ t1, int KS) {
    constexpr int NI = NCOL == 16 ? 2 : 1;      // MMAs per block
    constexpr int NBR = NCOL / 4;               // batch rows staged
    // blockIdx.x = group of NBR batch rows, blockIdx.y = CTA index within a group.  The groups of one
    // launch are independent problems over the same weights; running them side by side keeps the
    // SMs busy where one group alone is bound by latency, and because the group index is the fast
    // grid dimension the CTAs that stream the same tiles are scheduled together, so all groups but
    // the first find them in L2.
    GM_STAMP(0);
    const uint32_t bx = blockIdx.y, gx = gridDim.y, grp = blockIdx.x;
    GemvArgs a = a_in;
    {
        const int r0 = (int)grp * NBR;
        a.B = min(NBR, a_in.B - r0);
        if (r0) {
            if (a.x) a.x += (size_t)r0 * a.ldx;
            if (a.h_in) a.h_in += (size_t)r0 * a.ldx;
            if (a.add_src) a.add_src += (size_t)r0 * a.ldx;
            if (a.h_out) a.h_out += (size_t)r0 * a.ldx;
            if (a.y) a.y += (size_t)r0 * a.ldy;
            if (a.out_tok) a.out_tok += r0;
            if (a.out_tok_f32) a.out_tok_f32 += r0;
            if (a.out_val) a.out_val += r0;
            if (a.part_val) { a.part_val += (size_t)r0 * gx; a.part_idx += (size_t)r0 * gx; a.ticket += grp; }
        }
    }
    constexpr int NPR = NCOL / 2;               // column pairs per block (one pre-summed value each)
    constexpr int NM = PAIR ? 2 : 1;
    constexpr int CH = MmaGeo<PAIR, WT>::CH;
    constexpr int STAGE_BYTES = MmaGeo<PAIR, WT>::STAGE_BYTES;
    constexpr int MMA_TILE = MmaGeo<PAIR, WT>::TILE;
    constexpr float SXF = WT == WT_Q4_0 ? -8.0f : -1.0f;    // Q4_0: d*(q-8); Q4_K: (d*sc)*q - (dmin*m)
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float s_red[2][MMA_MAX_WARPS][NM][NI][16][2];
    __shared__ __align__(8) uint64_t s_bar[MMA_MAX_WARPS][NST];
    __shared__ __align__(8) uint64_t s_xbar;                // bulk copy of a long activation vector
    bool x_timed_out = false;
    __shared__ float s_inv[4];
    __shared__ float s_rd[2][3][32];            // scratch of the CTA-wide reductions of the staging (alternating per batch row)
    __shared__ float s_bv[MMA_MAX_WARPS * 4];
    __shared__ int   s_bi[MMA_MAX_WARPS * 4];
    __shared__ bool  s_last;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int RG = n_warps / KS, rg_l = warp / KS, ks = warp % KS;
    const int pairs = a.K >> 6, units = a.K >> 5;
    const int n_rg = a.N >> 4;
    const int n_sets = (n_rg + RG - 1) / RG;
    const int p0 = (int)((long long)ks * pairs / KS), p1 = (int)((long long)(ks + 1) * pairs / KS), np = p1 - p0;
    const int my_sets = (n_sets > (int)bx) ? (n_sets - (int)bx + (int)gx - 1) / (int)gx : 0;

    // ---- weight stream: every warp runs its own ring of bulk copies into shared memory ----
    // Stage = up to CH consecutive tile pairs of the warp's row group (contiguous in memory),
    // one cp.async.bulk per matrix, completion counted on the stage's mbarrier.
    signed char* xb = reinterpret_cast<signed char*>(smem_raw);                            // [units][NCOL][32]
    float* s_sx = reinterpret_cast<float*>(smem_raw + (size_t)units * NCOL * 32);          // [units][NPR], already times -8
    unsigned char* ring = smem_raw + (((size_t)units * (NCOL * 32 + NPR * 4) + 127) & ~(size_t)127) + (size_t)warp * NST * STAGE_BYTES;
    const int nch = (np + CH - 1) / CH;                     // chunks per row group for this warp
    const int n_chunks = my_sets * nch;
    if (lane == 0) {
#pragma unroll
        for (int st = 0; st < NST; ++st) mbar_init(&s_bar[warp][st], 1);
        if (NST == 2 && warp == 0) mbar_init(&s_xbar, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    // issue cursor (lane 0): the next chunk to request is chunk `i_j` of row group `i_rg`, into stage `i_st`
    int i_c = 0, i_j = 0, i_st = 0, i_rg = (int)bx * RG + rg_l;
    auto issue_next = [&]() {                                // lane 0 only
        const int rg = min(i_rg, n_rg - 1);                 // clamped: rows past the end are dropped later
        const int pp0 = p0 + i_j * CH, n = min(CH, p1 - pp0);
        const size_t off = ((size_t)rg * pairs + pp0) * MMA_TILE;
        unsigned char* dst = ring + (size_t)i_st * STAGE_BYTES;
        mbar_expect_tx(&s_bar[warp][i_st], (uint32_t)(n * MMA_TILE * NM));
        bulk_g2s(dst, t0 + off, (uint32_t)(n * MMA_TILE), &s_bar[warp][i_st]);
        if (PAIR) bulk_g2s(dst + CH * MMA_TILE, t1 + off, (uint32_t)(n * MMA_TILE), &s_bar[warp][i_st]);
        ++i_c;
        if (++i_st == NST) i_st = 0;
        if (++i_j == nch) { i_j = 0; i_rg += (int)gx * RG; }
    };
    if (lane == 0) {
#pragma unroll
        for (int c = 0; c < NST; ++c) if (i_c < n_chunks) issue_next();
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
    GM_STAMP(1);
    pdl_launch_dependents();
    pdl_wait();
    GM_STAMP(2);
    // ---- stage activations as signed bytes (hi, mid | lo) in MMA operand order, with the per-block sums the
    // MMA lanes subtract (in the units of the lane that uses them: 256 * first column + second column, times
    // the offset factor).  One barrier per CTA-wide reduction; loop bodies that hold no element are skipped. ----
    {
        const int n4 = a.K >> 2;
        const int nj = (n4 + (int)blockDim.x - 1) / (int)blockDim.x;          // float4 per thread
        for (int b = 0; b < NBR && b < a.B; ++b) {
            const size_t row = (size_t)b * a.ldx;
            float (*rd)[32] = s_rd[b & 1];
            if (a.h_in && n4 <= 3 * (int)blockDim.x) {
                const float* hp = a.h_in + row;
                const float* ap = a.add_src ? a.add_src + row : nullptr;
                float4 va[3], vh[3];
                const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int i = threadIdx.x + j * blockDim.x;
                    const bool in = j < nj && i < n4;
                    vh[j] = in ? reinterpret_cast<const float4*>(hp)[i] : z4;
                    va[j] = (in && ap) ? reinterpret_cast<const float4*>(ap)[i] : z4;
                }
                float rms_a = 1.f;
                if (ap && a.w_post) {
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < 3; ++j)
                        if (j < nj) { ss = fmaf(va[j].x, va[j].x, ss); ss = fmaf(va[j].y, va[j].y, ss); ss = fmaf(va[j].z, va[j].z, ss); ss = fmaf(va[j].w, va[j].w, ss); }
                    ss = cta_sum1(ss, rd[0]);
                    rms_a = sqrtf(ss / (float)a.K + a.eps);
                }
                GM_STAMP(5);
                const float rcp_a = __frcp_rn(rms_a);
                // h' and, in the same reduction, its sum of squares and max |h' * w_pre|
                float ss = 0.f, am = 0.f;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    if (j < nj) {
                        if (ap) {
                            if (a.w_post) {
                                vh[j].x += div_by(va[j].x, rms_a, rcp_a) * vp[j].x; vh[j].y += div_by(va[j].y, rms_a, rcp_a) * vp[j].y;
                                vh[j].z += div_by(va[j].z, rms_a, rcp_a) * vp[j].z; vh[j].w += div_by(va[j].w, rms_a, rcp_a) * vp[j].w;
                            } else { vh[j].x += va[j].x; vh[j].y += va[j].y; vh[j].z += va[j].z; vh[j].w += va[j].w; }
                        }
                        ss = fmaf(vh[j].x, vh[j].x, ss); ss = fmaf(vh[j].y, vh[j].y, ss); ss = fmaf(vh[j].z, vh[j].z, ss); ss = fmaf(vh[j].w, vh[j].w, ss);
                        am = fmaxf(am, fmaxf(fmaxf(fabsf(vh[j].x * vw[j].x), fabsf(vh[j].y * vw[j].y)), fmaxf(fabsf(vh[j].z * vw[j].z), fabsf(vh[j].w * vw[j].w))));
                        const int i = threadIdx.x + j * blockDim.x;
                        if (i < n4 && a.h_out && bx == 0) reinterpret_cast<float4*>(a.h_out + row)[i] = vh[j];
                    }
                }
                cta_sum_max1(ss, am, rd[1], rd[2]);
                GM_STAMP(6);
                float rms = 1.f;
                if (a.w_pre) {
                    rms = sqrtf(ss / (float)a.K + a.eps);
                    const float rcp = __frcp_rn(rms);
                    am = am * rcp * 1.000001f;             // bound on max |x| (the scale has a factor 2 to spare)
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        if (j < nj) {
                            vh[j].x = div_by(vh[j].x, rms, rcp) * vw[j].x; vh[j].y = div_by(vh[j].y, rms, rcp) * vw[j].y;
                            vh[j].z = div_by(vh[j].z, rms, rcp) * vw[j].z; vh[j].w = div_by(vh[j].w, rms, rcp) * vw[j].w;
                        }
                    }
                }
                float s, inv;
                pow2_scale(am, s, inv);
                if (threadIdx.x == 0) s_inv[b] = inv;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    if (j < nj) {
                        const int i = threadIdx.x + j * blockDim.x;
                        put_x4_sums<NCOL>(xb, s_sx, 4 * i, b, make_float4(vh[j].x * s, vh[j].y * s, vh[j].z * s, vh[j].w * s), i < n4, SXF);
                    }
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
                        v[j] = (j < nj && i < n4) ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        if (j < nj) am = fmaxf(am, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
                    am = cta_max1(am, rd[0]);
                    pow2_scale(am, s, inv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (j < nj) {
                            const int i = threadIdx.x + j * blockDim.x;
                            put_x4_sums<NCOL>(xb, s_sx, 4 * i, b, make_float4(v[j].x * s, v[j].y * s, v[j].z * s, v[j].w * s), i < n4, SXF);
                        }
                    }
                } else {
                    // Long vectors.  With one batch row per pass the staged form of 32 activations takes the same 128 bytes
                    // as the floats themselves: a bulk copy parks the floats where their bytes will go, one pass over
                    // shared memory finds the maximum, a second one splits them in place.  The eight lanes
                    // that share a block read their floats before any of them stores bytes.  With more rows per pass the
                    // second pass reads global memory again.
                    float4* park = reinterpret_cast<float4*>(xb);
                    if constexpr (NCOL == 4 && NST == 2) {       // the instance the launcher picks for long plain vectors
                        // the whole vector in one bulk copy: one memory round trip however long it is
                        __syncthreads();                        // s_xbar was initialised by thread 0
                        if (threadIdx.x == 0) {
                            mbar_expect_tx(&s_xbar, (uint32_t)n4 * 16u);
                            bulk_g2s(park, src, (uint32_t)n4 * 16u, &s_xbar);
                        }
                        if (!mbar_wait(&s_xbar, 0u)) { x_timed_out = true; if (threadIdx.x == 0) atomicOr(a.err, DEVERR_WAIT); }
                        GM_STAMP(5);
#pragma unroll 4
                        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                            const float4 v = park[i];
                            am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                        }
                        am = cta_max1(am, rd[0]);
                        GM_STAMP(6);
                        pow2_scale(am, s, inv);
                        // four blocks per lane at a time, so that their shuffle chains overlap
                        for (int j0 = 0; j0 < nj; j0 += 4) {
                            float4 v4[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const int i = threadIdx.x + (j0 + u) * blockDim.x;
                                v4[u] = (j0 + u < nj && i < n4) ? park[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
                            __syncwarp();
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                if (j0 + u < nj) {
                                    const int i = threadIdx.x + (j0 + u) * blockDim.x;
                                    put_x4_sums<NCOL>(xb, s_sx, 4 * i, b, make_float4(v4[u].x * s, v4[u].y * s, v4[u].z * s, v4[u].w * s), i < n4, SXF);
                                }
                            }
                        }
                    } else {
#pragma unroll 4
                        for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                            const float4 v = src[i];
                            am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                        }
                        am = cta_max1(am, rd[0]);
                        pow2_scale(am, s, inv);
                        // second pass in groups of four: the loads of a group are all requested before the first is used
                        for (int j0 = 0; j0 < nj; j0 += 4) {
                            float4 v4[4];
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                const int i = threadIdx.x + (j0 + u) * blockDim.x;
                                v4[u] = (j0 + u < nj && i < n4) ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                            }
#pragma unroll
                            for (int u = 0; u < 4; ++u) {
                                if (j0 + u < nj) {
                                    const int i = threadIdx.x + (j0 + u) * blockDim.x;
                                    put_x4_sums<NCOL>(xb, s_sx, 4 * i, b, make_float4(v4[u].x * s, v4[u].y * s, v4[u].z * s, v4[u].w * s), i < n4, SXF);
                                }
                            }
                        }
                    }
                }
                if (threadIdx.x == 0) s_inv[b] = inv;
            }
        }
        // batch rows of this pass that the call does not have: their pre-summed entries are read, never used
        if (a.B < NBR) {
            for (int i = threadIdx.x; i < units * NPR; i += blockDim.x) if (((i % NPR) >> 1) >= a.B) s_sx[i] = 0.f;
        }
        __syncthreads();
    }
    GM_STAMP(3);
    float best_v[NI]; int best_i[NI];                       // arg-max candidates of batch rows 2i + t/2
    float acc[NM][NI][2];
#pragma unroll
    for (int i = 0; i < NI; ++i) { best_v[i] = -3.402823466e+38f; best_i[i] = -1; }
#pragma unroll
    for (int m = 0; m < NM; ++m)
#pragma unroll
        for (int i = 0; i < NI; ++i) acc[m][i][0] = acc[m][i][1] = 0.f;
    int parity = 0;
    // Lane (g, t) supplies B column g of every MMA.  With one batch row only columns 0..3
    // are staged and lanes g >= 4 re-read them: what lands in B columns >= 4 only reaches
    // output columns that are never read.
    const uint2* xq = reinterpret_cast<const uint2*>(xb) + (g % (NCOL < 8 ? NCOL : 8)) * 4 + t;
    constexpr int xstep = NCOL * 4;                            // uint2 per block
    const float* sxp = s_sx + (t % (NPR < 4 ? NPR : 4));
    const float cm = (t & 1) ? (1.0f / 256.0f) : 256.0f;      // even lanes hold (hi, mid), odd lanes (lo, 0)

    // One 16x32 block of one matrix against the staged columns.
    auto block_imma = [&](uint32_t wg, uint32_t wh, const uint2* xu, const float* sxu, uint32_t sc2, float (&ac)[NI][2]) {
        const uint32_t a0 = wg & 0x0F0F0F0Fu, a2 = (wg >> 4) & 0x0F0F0F0Fu;
        const uint32_t a1 = wh & 0x0F0F0F0Fu, a3 = (wh >> 4) & 0x0F0F0F0Fu;
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&sc2));
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const uint2 b = xu[i * 32];
            int dd[4];
            imma16832(dd, a0, a1, a2, a3, b.x, b.y);
            const float sx = sxu[i * 4];
            ac[i][0] = fmaf(d.x, (float)(dd[0] * 256 + dd[1]) + sx, ac[i][0]);
            ac[i][1] = fmaf(d.y, (float)(dd[2] * 256 + dd[3]) + sx, ac[i][1]);
        }
    };
    // Same for Q4_K: sc4 = { sc[g], m[g], sc[g+8], m[g+8] } of this block as bytes, (d, dmin) of the two rows.
    auto block_imma_k = [&](uint32_t wg, uint32_t wh, const uint2* xu, const float* sxu, uint32_t sc4, float2 dm0, float2 dm1, float (&ac)[NI][2]) {
        const uint32_t a0 = wg & 0x0F0F0F0Fu, a2 = (wg >> 4) & 0x0F0F0F0Fu;
        const uint32_t a1 = wh & 0x0F0F0F0Fu, a3 = (wh >> 4) & 0x0F0F0F0Fu;
        const float es0 = dm0.x * (float)(sc4 & 0xFFu), em0 = dm0.y * (float)((sc4 >> 8) & 0xFFu);
        const float es1 = dm1.x * (float)((sc4 >> 16) & 0xFFu), em1 = dm1.y * (float)(sc4 >> 24);
#pragma unroll
        for (int i = 0; i < NI; ++i) {
            const uint2 b = xu[i * 32];
            int dd[4];
            imma16832(dd, a0, a1, a2, a3, b.x, b.y);
            const float sx = sxu[i * 4];                     // minus the block's activation sum
            ac[i][0] = fmaf(es0, (float)(dd[0] * 256 + dd[1]), fmaf(em0, sx, ac[i][0]));
            ac[i][1] = fmaf(es1, (float)(dd[2] * 256 + dd[3]), fmaf(em1, sx, ac[i][1]));
        }
    };
    // Tile pair k of the current stage (both 32-weight blocks, both matrices).
    auto do_pair = [&](const unsigned char* buf, int k, const uint2* xp, const float* sx) {
        const uint2* xu0 = xp + (2 * k) * xstep;
        const float* sx0 = sx + (2 * k) * NPR;
#pragma unroll
        for (int m = 0; m < NM; ++m) {
            const unsigned char* tile = buf + (m * CH + k) * MMA_TILE;
            const uint4 q = reinterpret_cast<const uint4*>(tile)[lane];
            const uint2 sc = reinterpret_cast<const uint2*>(tile + 512)[g];
            if constexpr (WT == WT_Q4_0) {
                block_imma(q.x, q.y, xu0, sx0, sc.x, acc[m]);
                block_imma(q.z, q.w, xu0 + xstep, sx0 + NPR, sc.y, acc[m]);
            } else {
                const uint2 hd = reinterpret_cast<const uint2*>(tile + 576)[g];
                const float2 dm0 = __half22float2(*reinterpret_cast<const __half2*>(&hd.x));
                const float2 dm1 = __half22float2(*reinterpret_cast<const __half2*>(&hd.y));
                block_imma_k(q.x, q.y, xu0, sx0, sc.x, dm0, dm1, acc[m]);
                block_imma_k(q.z, q.w, xu0 + xstep, sx0 + NPR, sc.y, dm0, dm1, acc[m]);
            }
        }
    };

    bool timed_out = false;
    int j = 0, st = 0, c_rg = (int)bx * RG + rg_l;
    uint32_t ph = 0;
    for (int c = 0; c < n_chunks; ++c) {
        if (!timed_out) {
            const bool ok = mbar_wait(&s_bar[warp][st], ph);
            if (!__all_sync(0xffffffffu, ok)) {
                // A copy never completed.  Record it and stop touching the ring; the warp keeps
                // walking its chunks so that it still meets its peers at every CTA barrier.
                timed_out = true;
                if (lane == 0) atomicOr(a.err, DEVERR_WAIT);
            }
        }
        if (!timed_out) {
            const unsigned char* buf = ring + (size_t)st * STAGE_BYTES;
            const int pp0 = p0 + j * CH, n = p1 - pp0;
            const uint2* xp = xq + (size_t)pp0 * 2 * xstep;
            const float* sx = sxp + (size_t)pp0 * 2 * NPR;
            if (n >= CH) {
#pragma unroll
                for (int k = 0; k < CH; ++k) do_pair(buf, k, xp, sx);
            } else {
                int k = 0;
                for (; k + 1 < n; k += 2) { do_pair(buf, k, xp, sx); do_pair(buf, k + 1, xp, sx); }
                if (k < n) do_pair(buf, k, xp, sx);
            }
            __syncwarp();                                   // every lane is done with this stage
            if (lane == 0 && i_c < n_chunks) issue_next();
        }
        if (++st == NST) { st = 0; ph ^= 1u; }
        if (++j == nch) {
            // ---- end of this warp's K slice for the row group ----
            const int rg = c_rg;
            j = 0;
            c_rg += (int)gx * RG;
            // even lanes: 256 * acc + (odd neighbour's acc) / 256  ->  batch row 2i + t/2
            float val[NM][NI][2];
#pragma unroll
            for (int m = 0; m < NM; ++m)
#pragma unroll
                for (int i = 0; i < NI; ++i)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float v = acc[m][i][h] * cm;
                        val[m][i][h] = v + __shfl_xor_sync(0xffffffffu, v, 1);
                        acc[m][i][h] = 0.f;
                    }
            bool writer = true;
            if (KS > 1) {       // combine the KS slices through shared memory
                if (!(t & 1)) {
#pragma unroll
                    for (int m = 0; m < NM; ++m)
#pragma unroll
                        for (int i = 0; i < NI; ++i) {
                            s_red[parity][warp][m][i][g][t >> 1] = val[m][i][0];
                            s_red[parity][warp][m][i][g + 8][t >> 1] = val[m][i][1];
                        }
                }
                __syncthreads();
                writer = (ks == 0);
                if (writer && !(t & 1)) {
                    for (int k2 = 1; k2 < KS; ++k2) {
#pragma unroll
                        for (int m = 0; m < NM; ++m)
#pragma unroll
                            for (int i = 0; i < NI; ++i) {
                                val[m][i][0] += s_red[parity][warp + k2][m][i][g][t >> 1];
                                val[m][i][1] += s_red[parity][warp + k2][m][i][g + 8][t >> 1];
                            }
                    }
                }
                parity ^= 1;
            }
            if (writer && rg < n_rg && !(t & 1)) {
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int bt = 2 * i + (t >> 1);
                    if (bt < a.B) {
                        const float inv = s_inv[bt];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int row = rg * 16 + g + 8 * h;
                            const float va = val[0][i][h] * inv;
                            if (a.epi == EPI_STORE) a.y[(size_t)bt * a.ldy + row] = va;
                            else if (a.epi == EPI_GEGLU) a.y[(size_t)bt * a.ldy + row] = gelu_tanh(va) * (val[NM - 1][i][h] * inv);
                            else if (a.epi == EPI_SWIGLU) a.y[(size_t)bt * a.ldy + row] = silu_clip(va) * (val[NM - 1][i][h] * inv);
                            else {
                                float v = va;
                                if (a.y) a.y[(size_t)bt * a.ldy + row] = a.softcap > 0.f ? tanhf(v / a.softcap) * a.softcap : v;
                                if (!(v == v)) v = -3.402823466e+38f;
                                if (better(v, row, best_v[i], best_i[i])) { best_v[i] = v; best_i[i] = row; }
                            }
                        }
                    }
                }
            }
        }
    }
    GM_STAMP(4);
    if (x_timed_out) mbar_wait(&s_xbar, 0u);
    if (timed_out) {
        // give the copies still in flight a bounded chance to land before the CTA's shared memory is released
        for (int s2 = 0; s2 < NST; ++s2) { mbar_wait(&s_bar[warp][s2], 0u); mbar_wait(&s_bar[warp][s2], 1u); }
    }

    if (a.epi != EPI_ARGMAX) return;
    // lanes that share a batch row (same t) -> lane g == 0; then across warps; then across CTAs
#pragma unroll
    for (int i = 0; i < NI; ++i) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v[i], o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i[i], o);
            if (better(ov, oi, best_v[i], best_i[i])) { best_v[i] = ov; best_i[i] = oi; }
        }
        if (g == 0 && !(t & 1)) { s_bv[warp * 4 + 2 * i + (t >> 1)] = best_v[i]; s_bi[warp * 4 + 2 * i + (t >> 1)] = best_i[i]; }
    }
    __syncthreads();
    if ((int)threadIdx.x < a.B && threadIdx.x < 4 && threadIdx.x < NBR) {
        const int b = threadIdx.x;
        float bv = s_bv[b]; int bi = s_bi[b];
        for (int w = 1; w < n_warps; ++w) if (better(s_bv[w * 4 + b], s_bi[w * 4 + b], bv, bi)) { bv = s_bv[w * 4 + b]; bi = s_bi[w * 4 + b]; }
        a.part_val[(size_t)b * gx + bx] = bv;
        a.part_idx[(size_t)b * gx + bx] = bi;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1u) == gx - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int b = 0; b < a.B && b < NBR; ++b) {
        float bv = -3.402823466e+38f; int bi = -1;
        for (int i = threadIdx.x; i < (int)gx; i += blockDim.x) {
            const float v = __ldcg(a.part_val + (size_t)b * gx + i);
            const int k = __ldcg(a.part_idx + (size_t)b * gx + i);
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
            if (a.out_val) a.out_val[b] = bv;
            if (a.out_tok_f32) a.out_tok_f32[b] = (float)tok;
        }
    }
    if (threadIdx.x == 0) *a.ticket = 0u;
}

// Launch on `stream` with tiled weights t0 (and t1 for GeGLU/SwiGLU).  Returns
// ADAMAH_ERR_INVALID without launching when the shape does not fit this kernel
// (the caller then uses the generic kernel): needs N % 16 == 0, K % 64 == 0, and
// either plain x or an input chain short enough for the register-resident path.
int launch_gemv_mma(int wtype, const uint8_t* t0, const uint8_t* t1, GemvArgs a, cudaStream_t stream);
bool gemv_mma_supports(int wtype, const GemvArgs& a);
const void* find_tiled(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols);
const void* find_tiled_prefix(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols);
int tile_tensor(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols);
void tiled_drop_map(uint32_t map_id);

}  // namespace ab
