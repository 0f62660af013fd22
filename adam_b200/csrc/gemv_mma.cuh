// Tensor-core variant of the Q4_0 dequant GEMV over row-tiled weights (tile.cu).
//
// Why tensor cores in a memory-bound GEMV: on the plain CUDA-core path the unpack
// (one byte-permute per weight, on the half-rate integer pipe) and one FMA per weight
// cap the kernel at about half of HBM bandwidth.  Here a 16-row x 32-weight block is
// two mma.sync.m16n8k16 (fp16 in, fp32 accumulate): weights enter as exact fp16
// integers q-8 (two nibbles per logic op, offset removed by one packed half op), the
// activation vector enters as the B operand split into fp16 high and low parts
// (x*s = hi + lo/2048 with a power-of-two scale s chosen per vector so hi never
// overflows), which keeps 22 bits of every activation; the block's fp32 sums are
// then scaled by the block scale d on the CUDA cores.  About 0.055 warp instructions
// per weight instead of 0.114.  The tensor pipe itself stays almost idle: the kernel
// is still a stream over the weight bytes, bound by HBM.
//
// Columns of the 8-wide B operand: (2b, 2b+1) = (hi, lo) of batch row b, b < 4.  With
// one batch row only columns 0,1 are staged (NCOL = 2) and the rest are zero.
// A warp owns one 16-row group and a slice of K; the KS warps that share a row group
// combine through shared memory.  Lane (g, t) = (lane/4, lane%4) holds rows g and g+8
// for batch row t.  k-order inside a block is permuted consistently in A and B so that
// each lane's A registers come from one 32-bit word of each of its two rows.
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace ab {

constexpr float MMA_LO_SCALE = 2048.0f;

struct MmaSlot { uint4 q; uint2 sc; };

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Same with a zero accumulator input (the zero operands become the zero register).
__device__ __forceinline__ void mma16816_z(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "f"(0.f));
}

// One 32-bit word of nibbles (low nibbles = weights 4t..4t+3, high = 16+4t..) -> four
// half2 registers holding q-8:  r0 = (w0, w2), r1 = (w1, w3), r2 = (w16, w18), r3 = (w17, w19)
// in units relative to 4t.
__device__ __forceinline__ void unpack_word(uint32_t w, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    const uint32_t w8 = w >> 8;
    uint32_t a0 = (w & 0x000F000Fu) | 0x64006400u;      // 1024 + q
    uint32_t a1 = (w8 & 0x000F000Fu) | 0x64006400u;
    uint32_t a2 = (w & 0x00F000F0u) | 0x64006400u;      // 1024 + 16 q
    uint32_t a3 = (w8 & 0x00F000F0u) | 0x64006400u;
    const __half2 m1032 = __floats2half2_rn(-1032.f, -1032.f);
    const __half2 sixteenth = __floats2half2_rn(0.0625f, 0.0625f), m72 = __floats2half2_rn(-72.f, -72.f);
    __half2 h0 = __hadd2(*reinterpret_cast<__half2*>(&a0), m1032);
    __half2 h1 = __hadd2(*reinterpret_cast<__half2*>(&a1), m1032);
    __half2 h2 = __hfma2(*reinterpret_cast<__half2*>(&a2), sixteenth, m72);
    __half2 h3 = __hfma2(*reinterpret_cast<__half2*>(&a3), sixteenth, m72);
    r0 = *reinterpret_cast<uint32_t*>(&h0); r1 = *reinterpret_cast<uint32_t*>(&h1);
    r2 = *reinterpret_cast<uint32_t*>(&h2); r3 = *reinterpret_cast<uint32_t*>(&h3);
}

// Offset (in halves) of activation element k of column `col` inside the staged buffer.
template <int NCOL>
__device__ __forceinline__ int xs16_index(int k, int col) {
    const int u = k >> 5, w = k & 31, tg = (w & 15) >> 2, i = w & 3, mm = w >> 4;
    return ((u * NCOL + col) * 4 + tg) * 8 + mm * 4 + (i & 1) * 2 + (i >> 1);
}

template <int NCOL>
__device__ __forceinline__ void put_x(__half* xs, int k, int b, float v_scaled) {
    const __half hi = __float2half_rn(v_scaled);
    const __half lo = __float2half_rn((v_scaled - __half2float(hi)) * MMA_LO_SCALE);
    xs[xs16_index<NCOL>(k, 2 * b)] = hi;
    xs[xs16_index<NCOL>(k, 2 * b + 1)] = lo;
}

// Power-of-two scale that brings amax to at most 2^14 (and its inverse).
__device__ __forceinline__ void pow2_scale(float amax, float& s, float& inv) {
    if (!(amax > 0.f) || !(amax < 3.0e38f)) { s = 1.f; inv = 1.f; return; }
    int e;
    frexpf(amax, &e);
    e = max(-100, min(100, 14 - e));
    s = ldexpf(1.f, e); inv = ldexpf(1.f, -e);
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
    __half* xs = reinterpret_cast<__half*>(smem_raw);
    __shared__ float s_red[2][8][PAIR ? 2 : 1][16][4];
    __shared__ float s_inv[4];
    __shared__ float red[33];
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
    unsigned char* ring = smem_raw + (((size_t)units * NCOL * 64 + 127) & ~(size_t)127) + (size_t)warp * NSTAGE * STAGE_BYTES;
    const int nch = (np + MMA_CH - 1) / MMA_CH;             // chunks per row group for this warp
    const int n_chunks = my_sets * nch;
    if (lane == 0) {
#pragma unroll
        for (int st = 0; st < NSTAGE; ++st) mbar_init(&s_bar[warp][st], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    auto issue_chunk = [&](int c) {                         // lane 0 only
        const int set_i = c / nch, j = c % nch;
        const int rg = min(((int)blockIdx.x + set_i * (int)gridDim.x) * RG + rg_l, n_rg - 1);   // clamped: rows past the end are dropped later
        const int pp0 = p0 + j * MMA_CH, n = min(MMA_CH, p1 - pp0);
        const size_t off = ((size_t)rg * pairs + pp0) * MMA_TILE;
        const int st = c % NSTAGE;
        unsigned char* dst = ring + (size_t)st * STAGE_BYTES;
        mbar_expect_tx(&s_bar[warp][st], (uint32_t)(n * MMA_TILE * (PAIR ? 2 : 1)));
        bulk_g2s(dst, t0 + off, (uint32_t)(n * MMA_TILE), &s_bar[warp][st]);
        if (PAIR) bulk_g2s(dst + MMA_CH * MMA_TILE, t1 + off, (uint32_t)(n * MMA_TILE), &s_bar[warp][st]);
    };
    if (lane == 0) {
#pragma unroll
        for (int c = 0; c < NSTAGE; ++c) if (c < n_chunks) issue_chunk(c);
    }

    // ---- stage activations as fp16 (hi, lo) pairs in MMA operand order ----
    {
        if (NCOL > 2) {     // unused batch columns must read as zero
            uint4* z = reinterpret_cast<uint4*>(xs);
            for (int i = threadIdx.x; i < units * NCOL * 4; i += blockDim.x) z[i] = make_uint4(0, 0, 0, 0);
            __syncthreads();
        }
        const int n4 = a.K >> 2;
        for (int b = 0; b < NB && b < a.B; ++b) {
            const size_t row = (size_t)b * a.ldx;
            if (a.h_in && n4 <= 3 * (int)blockDim.x) {
                const float* hp = a.h_in + row;
                const float* ap = a.add_src ? a.add_src + row : nullptr;
                float4 va[3], vh[3], vp[3], vw[3];
                const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f), o4 = make_float4(1.f, 1.f, 1.f, 1.f);
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int i = threadIdx.x + j * blockDim.x;
                    const bool in = i < n4;
                    vh[j] = in ? reinterpret_cast<const float4*>(hp)[i] : z4;
                    va[j] = (in && ap) ? reinterpret_cast<const float4*>(ap)[i] : z4;
                    vp[j] = (in && ap && a.w_post) ? reinterpret_cast<const float4*>(a.w_post)[i] : o4;
                    vw[j] = (in && a.w_pre) ? reinterpret_cast<const float4*>(a.w_pre)[i] : o4;
                }
                float rms_a = 1.f;
                if (ap && a.w_post) {
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < 3; ++j) { ss = fmaf(va[j].x, va[j].x, ss); ss = fmaf(va[j].y, va[j].y, ss); ss = fmaf(va[j].z, va[j].z, ss); ss = fmaf(va[j].w, va[j].w, ss); }
                    ss = block_sum(ss, red);
                    rms_a = sqrtf(ss / (float)a.K + a.eps);
                }
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    if (ap) {
                        if (a.w_post) {
                            vh[j].x += __fdiv_rn(va[j].x, rms_a) * vp[j].x; vh[j].y += __fdiv_rn(va[j].y, rms_a) * vp[j].y;
                            vh[j].z += __fdiv_rn(va[j].z, rms_a) * vp[j].z; vh[j].w += __fdiv_rn(va[j].w, rms_a) * vp[j].w;
                        } else { vh[j].x += va[j].x; vh[j].y += va[j].y; vh[j].z += va[j].z; vh[j].w += va[j].w; }
                    }
                    ss = fmaf(vh[j].x, vh[j].x, ss); ss = fmaf(vh[j].y, vh[j].y, ss); ss = fmaf(vh[j].z, vh[j].z, ss); ss = fmaf(vh[j].w, vh[j].w, ss);
                    const int i = threadIdx.x + j * blockDim.x;
                    if (i < n4 && a.h_out && blockIdx.x == 0) reinterpret_cast<float4*>(a.h_out + row)[i] = vh[j];
                }
                float rms = 1.f;
                if (a.w_pre) { ss = block_sum(ss, red); rms = sqrtf(ss / (float)a.K + a.eps); }
                float am = 0.f;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    if (a.w_pre) {
                        vh[j].x = __fdiv_rn(vh[j].x, rms) * vw[j].x; vh[j].y = __fdiv_rn(vh[j].y, rms) * vw[j].y;
                        vh[j].z = __fdiv_rn(vh[j].z, rms) * vw[j].z; vh[j].w = __fdiv_rn(vh[j].w, rms) * vw[j].w;
                    }
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(vh[j].x), fabsf(vh[j].y)), fmaxf(fabsf(vh[j].z), fabsf(vh[j].w))));
                }
                am = block_max(am, red);
                float s, inv;
                pow2_scale(am, s, inv);
                if (threadIdx.x == 0) s_inv[b] = inv;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int i = threadIdx.x + j * blockDim.x;
                    if (i < n4) {
                        put_x<NCOL>(xs, 4 * i, b, vh[j].x * s); put_x<NCOL>(xs, 4 * i + 1, b, vh[j].y * s);
                        put_x<NCOL>(xs, 4 * i + 2, b, vh[j].z * s); put_x<NCOL>(xs, 4 * i + 3, b, vh[j].w * s);
                    }
                }
            } else {
                // generic path: (optional) slow input chain into a float scratch view is not
                // supported here; the launcher only takes this kernel with plain x or the fast chain.
                const float4* src = reinterpret_cast<const float4*>(a.x + row);
                float am = 0.f;
#pragma unroll 4
                for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                    const float4 v = src[i];
                    am = fmaxf(am, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                }
                am = block_max(am, red);
                float s, inv;
                pow2_scale(am, s, inv);
                if (threadIdx.x == 0) s_inv[b] = inv;
#pragma unroll 4
                for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                    const float4 v = src[i];
                    put_x<NCOL>(xs, 4 * i, b, v.x * s); put_x<NCOL>(xs, 4 * i + 1, b, v.y * s);
                    put_x<NCOL>(xs, 4 * i + 2, b, v.z * s); put_x<NCOL>(xs, 4 * i + 3, b, v.w * s);
                }
            }
        }
        __syncthreads();
    }

    float best_v = -3.402823466e+38f; int best_i = -1;        // for batch row t
    float accA[2] = {0.f, 0.f}, accB[2] = {0.f, 0.f};
    int parity = 0;
    // Lanes g >= NCOL supply all-zero B columns: they read a zero block with stride 0.
    __shared__ __align__(16) uint4 s_zero[4];
    if (threadIdx.x < 4) s_zero[threadIdx.x] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    const bool xlive = g < NCOL;
    const uint4* xq = xlive ? reinterpret_cast<const uint4*>(xs) + g * 4 + t : s_zero + t;
    const int xstep = xlive ? NCOL * 4 : 0;                    // uint4 per block
    constexpr float LO = 1.0f / MMA_LO_SCALE;

    // One tile pair of one matrix: four independent MMAs (two blocks x two k-halves) are
    // issued before any result is used, then the block scales are applied.
    auto pair_mma = [&](const uint4& q, const uint2& sc, const uint4& xb0, const uint4& xb1, float& acc0, float& acc1) {
        uint32_t p0g[4], p0h[4], p1g[4], p1h[4];
        unpack_word(q.x, p0g[0], p0g[1], p0g[2], p0g[3]);
        unpack_word(q.y, p0h[0], p0h[1], p0h[2], p0h[3]);
        unpack_word(q.z, p1g[0], p1g[1], p1g[2], p1g[3]);
        unpack_word(q.w, p1h[0], p1h[1], p1h[2], p1h[3]);
        float c00[4], c01[4], c10[4], c11[4];
        { const uint32_t av[4] = {p0g[0], p0h[0], p0g[1], p0h[1]}; mma16816_z(c00, av, xb0.x, xb0.y); }
        { const uint32_t av[4] = {p0g[2], p0h[2], p0g[3], p0h[3]}; mma16816_z(c01, av, xb0.z, xb0.w); }
        { const uint32_t av[4] = {p1g[0], p1h[0], p1g[1], p1h[1]}; mma16816_z(c10, av, xb1.x, xb1.y); }
        { const uint32_t av[4] = {p1g[2], p1h[2], p1g[3], p1h[3]}; mma16816_z(c11, av, xb1.z, xb1.w); }
        const float2 d0 = __half22float2(*reinterpret_cast<const __half2*>(&sc.x));
        const float2 d1 = __half22float2(*reinterpret_cast<const __half2*>(&sc.y));
        acc0 = fmaf(d0.x, fmaf(c00[1] + c01[1], LO, c00[0] + c01[0]), acc0);
        acc1 = fmaf(d0.y, fmaf(c00[3] + c01[3], LO, c00[2] + c01[2]), acc1);
        acc0 = fmaf(d1.x, fmaf(c10[1] + c11[1], LO, c10[0] + c11[0]), acc0);
        acc1 = fmaf(d1.y, fmaf(c10[3] + c11[3], LO, c10[2] + c11[2]), acc1);
    };

    bool timed_out = false;
    for (int c = 0; c < n_chunks; ++c) {
        const int st = c % NSTAGE, j = c % nch, set_i = c / nch;
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
            const uint4* xp = xq + (size_t)pp0 * 2 * xstep;
#pragma unroll
            for (int k = 0; k < MMA_CH; ++k) {
                if (k < n) {
                    const uint4 q = reinterpret_cast<const uint4*>(buf + k * MMA_TILE)[lane];
                    const uint2 sc = reinterpret_cast<const uint2*>(buf + k * MMA_TILE + 512)[g];
                    const uint4 xb0 = xp[(2 * k) * xstep], xb1 = xp[(2 * k + 1) * xstep];
                    pair_mma(q, sc, xb0, xb1, accA[0], accA[1]);
                    if (PAIR) {
                        const uint4 q1 = reinterpret_cast<const uint4*>(buf + (MMA_CH + k) * MMA_TILE)[lane];
                        const uint2 sc1 = reinterpret_cast<const uint2*>(buf + (MMA_CH + k) * MMA_TILE + 512)[g];
                        pair_mma(q1, sc1, xb0, xb1, accB[0], accB[1]);
                    }
                }
            }
            __syncwarp();                                   // every lane is done with this stage
            if (lane == 0 && c + NSTAGE < n_chunks) issue_chunk(c + NSTAGE);
        }
        if (j == nch - 1) {
            // ---- end of this warp's K slice for the row group ----
            const int rg = ((int)blockIdx.x + set_i * (int)gridDim.x) * RG + rg_l;
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
