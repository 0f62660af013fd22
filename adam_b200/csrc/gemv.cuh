// Dequant-fused GEMV over GGUF Q4_0 / Q4_K blocks:  y[b][n] = sum_k W[n][k] x[b][k].
//
// Replaces the reference's Q4 mat-vec shader and its dispatch
// (adamah-MAIN/adamah/shaders/src/f32/map_matvec_t_xq4.comp;
// adamah.c:8606-8691 exec_matvec_t_xq_internal) and the fused variants built on
// it (map_fused_gateup_t_xq4.comp, map_matvec_argmax_t_xq4.comp + map_argmax_pairs.comp).
//
// Layout.  A "unit" is 16 bytes of packed nibbles = 32 weights; a row of K
// weights has K/32 units.
//   Q4_0: units live in a quant plane (one uint4 per 18-byte GGUF block, its 16
//         nibble bytes) and the fp16 block scales in a separate plane, so every
//         load is 16-byte aligned.  Byte j of a unit holds weight j (low nibble)
//         and weight j+16 (high nibble); value = d * (q - 8).
//   Q4_K: native 144-byte superblocks = 9 uint4: one header (d, dmin, 12 bytes of
//         6-bit scales/mins) + 8 units.  Unit c covers sub-blocks 2*(c/2) (low
//         nibbles) and 2*(c/2)+1 (high nibbles), elements (c%2)*16 .. +15;
//         value = (d*sc) * q - (dmin*m).
// Mapping.  L lanes share a row (L = 4..32, picked per K on the host), every lane
// owns TWO rows so the 32 activations it reads from shared memory are used twice,
// and a warp covers (32/L)*2 rows per pass.  Nibbles become floats without an
// int->float convert: a byte permute drops the nibble into the mantissa of 2^23,
// one subtraction makes it exact.  Accumulation is fp32 FMA; lanes combine with
// xor shuffles.  Activations are staged in shared memory once per CTA.
#pragma once
#include "common.cuh"

namespace ab {

enum { WT_Q4_0 = 0, WT_Q4_K = 1 };
enum { EPI_STORE = 0, EPI_GEGLU = 1, EPI_SWIGLU = 2, EPI_ARGMAX = 3 };

struct WeightRef {          // a [N,K] tensor inside a GGUF-block map
    const uint4*  q;        // Q4_0: first unit of the tensor in the quant plane
                            // Q4_K: first superblock (9 uint4 each)
    const __half* d;        // Q4_0: first block scale; unused for Q4_K
};

struct GemvArgs {
    WeightRef w0, w1;       // w1 only for GEGLU/SWIGLU (the "up" matrix)
    const float* x; int ldx;        // activations [B][ldx]
    float* y; int ldy;              // outputs [B][ldy] (may be NULL for ARGMAX)
    int N, K, B;
    int epi;
    int kc_units;                   // units of K staged per chunk
    // ARGMAX epilogue
    float* part_val; int* part_idx; // [B][gridDim.x] scratch
    unsigned int* ticket;           // one counter, zero between launches
    int* out_tok;                   // [B] winning row per batch entry
    float* out_tok_f32;             // optional: same id stored as float (reference convention)
    float softcap;                  // applied to stored logits only (monotone)
};

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

// 16 bytes of nibbles -> 32 floats (value - bias), low nibbles then high nibbles.
template <int BIAS>
__device__ __forceinline__ void unpack_unit(const uint4& q, float (&lo)[16], float (&hi)[16]) {
    const float magic = 8388608.0f + (float)BIAS;
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t l4 = w[i] & 0x0F0F0F0Fu, h4 = (w[i] >> 4) & 0x0F0F0F0Fu;
        lo[4*i+0] = __uint_as_float(__byte_perm(l4, 0x4B000000u, 0x7650)) - magic;
        lo[4*i+1] = __uint_as_float(__byte_perm(l4, 0x4B000000u, 0x7651)) - magic;
        lo[4*i+2] = __uint_as_float(__byte_perm(l4, 0x4B000000u, 0x7652)) - magic;
        lo[4*i+3] = __uint_as_float(__byte_perm(l4, 0x4B000000u, 0x7653)) - magic;
        hi[4*i+0] = __uint_as_float(__byte_perm(h4, 0x4B000000u, 0x7650)) - magic;
        hi[4*i+1] = __uint_as_float(__byte_perm(h4, 0x4B000000u, 0x7651)) - magic;
        hi[4*i+2] = __uint_as_float(__byte_perm(h4, 0x4B000000u, 0x7652)) - magic;
        hi[4*i+3] = __uint_as_float(__byte_perm(h4, 0x4B000000u, 0x7653)) - magic;
    }
}

__device__ __forceinline__ void ld_x16(const float* p, float (&x)[16]) {
    const float4* v = reinterpret_cast<const float4*>(p);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float4 f = v[i]; x[4*i] = f.x; x[4*i+1] = f.y; x[4*i+2] = f.z; x[4*i+3] = f.w; }
}

__device__ __forceinline__ float dot16(const float (&a)[16], const float (&b)[16], float acc) {
#pragma unroll
    for (int i = 0; i < 16; ++i) acc = fmaf(a[i], b[i], acc);
    return acc;
}
__device__ __forceinline__ float sum16(const float (&a)[16]) {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; i += 2) { s0 += a[i]; s1 += a[i+1]; }
    return s0 + s1;
}

// 6-bit scale / min of sub-block j from the 12 packed bytes held in three words.
__device__ __forceinline__ void q4k_sm(const uint32_t (&h)[3], int j, float& sc, float& mn) {
    auto byte = [&](int i) -> uint32_t { return (h[i >> 2] >> (8 * (i & 3))) & 0xFFu; };
    uint32_t s, m;
    if (j < 4) { s = byte(j) & 63u; m = byte(j + 4) & 63u; }
    else       { s = (byte(j + 4) & 0x0Fu) | ((byte(j - 4) >> 6) << 4); m = (byte(j + 4) >> 4) | ((byte(j) >> 6) << 4); }
    sc = (float)s; mn = (float)m;
}

struct BestRow { float v; int i; };
__device__ __forceinline__ bool better(float cv, int ci, float bv, int bi) {
    // higher value wins, ties go to the lower index (map_argmax.comp `better`)
    if (bi < 0) return ci >= 0;
    if (ci < 0) return false;
    return (cv > bv) || (cv == bv && ci < bi);
}

// One pass: this lane's two rows over units [u0,u1) of the staged chunk.
template <int WT, int L, int NB>
__device__ __forceinline__ void gemv_accumulate(const WeightRef& wa, const WeightRef& wb, size_t rowA, size_t rowB,
                                                int units_per_row, int u0, int u1, int l,
                                                const float* xs, int xs_ld, int xs_elem0,
                                                float (&accA)[NB], float (&accB)[NB]) {
    if (WT == WT_Q4_0) {
        const uint4* qa = wa.q + rowA * units_per_row;
        const uint4* qb = wb.q + rowB * units_per_row;
        const __half* da = wa.d + rowA * units_per_row;
        const __half* db = wb.d + rowB * units_per_row;
#pragma unroll 2
        for (int u = u0 + l; u < u1; u += L) {
            const uint4 ua = ld_stream(qa + u), ub = ld_stream(qb + u);
            const float sa = __half2float(da[u]), sb = __half2float(db[u]);
            float alo[16], ahi[16], blo[16], bhi[16];
            unpack_unit<8>(ua, alo, ahi);
            unpack_unit<8>(ub, blo, bhi);
            const float* xp = xs + (u * 32 - xs_elem0);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float xlo[16], xhi[16];
                ld_x16(xp + b * xs_ld, xlo);
                ld_x16(xp + b * xs_ld + 16, xhi);
                accA[b] = fmaf(sa, dot16(ahi, xhi, dot16(alo, xlo, 0.f)), accA[b]);
                accB[b] = fmaf(sb, dot16(bhi, xhi, dot16(blo, xlo, 0.f)), accB[b]);
            }
        }
    } else {
        const int sb_per_row = units_per_row >> 3;
        const uint4* qa = wa.q + rowA * (size_t)sb_per_row * 9;
        const uint4* qb = wb.q + rowB * (size_t)sb_per_row * 9;
#pragma unroll 2
        for (int u = u0 + l; u < u1; u += L) {
            const int sb = u >> 3, c = u & 7, grp = c >> 1;
            const uint4 ua = ld_stream(qa + sb * 9 + 1 + c), ub = ld_stream(qb + sb * 9 + 1 + c);
            const uint4 ha = __ldg(qa + sb * 9), hb = __ldg(qb + sb * 9);
            float alo[16], ahi[16], blo[16], bhi[16];
            unpack_unit<0>(ua, alo, ahi);
            unpack_unit<0>(ub, blo, bhi);
            float sA0, mA0, sA1, mA1, sB0, mB0, sB1, mB1;
            { const uint32_t h[3] = {ha.y, ha.z, ha.w}; q4k_sm(h, 2 * grp, sA0, mA0); q4k_sm(h, 2 * grp + 1, sA1, mA1); }
            { const uint32_t h[3] = {hb.y, hb.z, hb.w}; q4k_sm(h, 2 * grp, sB0, mB0); q4k_sm(h, 2 * grp + 1, sB1, mB1); }
            const float dA = __half2float(__ushort_as_half((unsigned short)(ha.x & 0xFFFF)));
            const float mA = __half2float(__ushort_as_half((unsigned short)(ha.x >> 16)));
            const float dB = __half2float(__ushort_as_half((unsigned short)(hb.x & 0xFFFF)));
            const float mB = __half2float(__ushort_as_half((unsigned short)(hb.x >> 16)));
            const int e_lo = sb * 256 + grp * 64 + (c & 1) * 16;
            const float* xp = xs + (e_lo - xs_elem0);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                float xlo[16], xhi[16];
                ld_x16(xp + b * xs_ld, xlo);
                ld_x16(xp + b * xs_ld + 32, xhi);
                const float sxlo = sum16(xlo), sxhi = sum16(xhi);
                float ta = (dA * sA0) * dot16(alo, xlo, 0.f) - (mA * mA0) * sxlo;
                ta += (dA * sA1) * dot16(ahi, xhi, 0.f) - (mA * mA1) * sxhi;
                float tb = (dB * sB0) * dot16(blo, xlo, 0.f) - (mB * mB0) * sxlo;
                tb += (dB * sB1) * dot16(bhi, xhi, 0.f) - (mB * mB1) * sxhi;
                accA[b] += ta;
                accB[b] += tb;
            }
        }
    }
}

template <int WT, int L, int NB>
__global__ void __launch_bounds__(256) k_gemv(const GemvArgs a) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float s_bv[8 * NB];
    __shared__ int   s_bi[8 * NB];
    __shared__ bool  s_last;
    constexpr int RPW = 32 / L;                 // row slots per warp pass
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sub = lane / L, l = lane % L;
    const int units = a.K >> 5;
    const bool pair_mats = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    const int n_slots = pair_mats ? a.N : (a.N + 1) / 2;
    const int n_pass = (n_slots + RPW - 1) / RPW;
    const int n_chunks = (units + a.kc_units - 1) / a.kc_units;
    const int xs_ld = min(units, a.kc_units) * 32;

    BestRow best[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) { best[b].v = -3.402823466e+38f; best[b].i = -1; }

    // One pass per warp when K is staged in chunks; a grid-stride loop otherwise.
    const int pass_stride = (n_chunks == 1) ? gridDim.x * 8 : n_pass + 1;
    bool staged = false;
    for (int pass0 = blockIdx.x * 8; pass0 < n_pass; pass0 += pass_stride) {
        const int pass = pass0 + warp;
        const int slot = pass * RPW + sub;
        const bool live = pass < n_pass && slot < n_slots;
        size_t rowA, rowB;
        if (pair_mats) { rowA = rowB = (size_t)(live ? slot : 0); }
        else { rowA = (size_t)(live ? 2 * slot : 0); rowB = (rowA + 1 < (size_t)a.N) ? rowA + 1 : rowA; }
        const WeightRef& wb = pair_mats ? a.w1 : a.w0;
        float accA[NB], accB[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) { accA[b] = 0.f; accB[b] = 0.f; }

        for (int ch = 0; ch < n_chunks; ++ch) {
            const int u0 = ch * a.kc_units, u1 = min(units, u0 + a.kc_units);
            if (!staged || n_chunks > 1) {
                if (n_chunks > 1) __syncthreads();
                const int n4 = (u1 - u0) * 8;      // float4 per batch row in this chunk
                for (int b = 0; b < NB; ++b) {
                    const float4* src = reinterpret_cast<const float4*>(a.x + (size_t)min(b, a.B - 1) * a.ldx + u0 * 32);
                    float4* dst = reinterpret_cast<float4*>(xs + b * xs_ld);
                    for (int i = threadIdx.x; i < n4; i += blockDim.x) dst[i] = src[i];
                }
                __syncthreads();
                staged = true;
            }
            if (live) gemv_accumulate<WT, L, NB>(a.w0, wb, rowA, rowB, units, u0, u1, l, xs, xs_ld, u0 * 32, accA, accB);
        }
#pragma unroll
        for (int b = 0; b < NB; ++b) {
#pragma unroll
            for (int o = L / 2; o > 0; o >>= 1) {
                accA[b] += __shfl_xor_sync(0xffffffffu, accA[b], o);
                accB[b] += __shfl_xor_sync(0xffffffffu, accB[b], o);
            }
        }
        if (live && l == 0) {
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                if (b >= a.B) break;
                if (a.epi == EPI_STORE) {
                    a.y[(size_t)b * a.ldy + rowA] = accA[b];
                    if (rowB != rowA) a.y[(size_t)b * a.ldy + rowB] = accB[b];
                } else if (a.epi == EPI_GEGLU) {
                    a.y[(size_t)b * a.ldy + slot] = gelu_tanh(accA[b]) * accB[b];
                } else if (a.epi == EPI_SWIGLU) {
                    a.y[(size_t)b * a.ldy + slot] = silu_clip(accA[b]) * accB[b];
                } else {
                    float va = accA[b], vb = accB[b];
                    if (a.y) {
                        float sa = va, sb2 = vb;
                        if (a.softcap > 0.f) { sa = tanhf(sa / a.softcap) * a.softcap; sb2 = tanhf(sb2 / a.softcap) * a.softcap; }
                        a.y[(size_t)b * a.ldy + rowA] = sa;
                        if (rowB != rowA) a.y[(size_t)b * a.ldy + rowB] = sb2;
                    }
                    if (!(va == va)) va = -3.402823466e+38f;
                    if (!(vb == vb)) vb = -3.402823466e+38f;
                    if (better(va, (int)rowA, best[b].v, best[b].i)) { best[b].v = va; best[b].i = (int)rowA; }
                    if (rowB != rowA && better(vb, (int)rowB, best[b].v, best[b].i)) { best[b].v = vb; best[b].i = (int)rowB; }
                }
            }
        }
    }

    if (a.epi != EPI_ARGMAX) return;
    // CTA-level winner -> scratch; the CTA that arrives last reduces all partials.
#pragma unroll
    for (int b = 0; b < NB; ++b) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, best[b].v, o);
            int   oi = __shfl_xor_sync(0xffffffffu, best[b].i, o);
            if (better(ov, oi, best[b].v, best[b].i)) { best[b].v = ov; best[b].i = oi; }
        }
        if (lane == 0) { s_bv[warp * NB + b] = best[b].v; s_bi[warp * NB + b] = best[b].i; }
    }
    __syncthreads();
    if (threadIdx.x < NB && (int)threadIdx.x < a.B) {
        const int b = threadIdx.x;
        float bv = s_bv[b]; int bi = s_bi[b];
        for (int w = 1; w < 8; ++w) if (better(s_bv[w * NB + b], s_bi[w * NB + b], bv, bi)) { bv = s_bv[w * NB + b]; bi = s_bi[w * NB + b]; }
        a.part_val[(size_t)b * gridDim.x + blockIdx.x] = bv;
        a.part_idx[(size_t)b * gridDim.x + blockIdx.x] = bi;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(a.ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (int b = 0; b < a.B && b < NB; ++b) {
        float bv = -3.402823466e+38f; int bi = -1;
        for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) {
            const float v = __ldcg(a.part_val + (size_t)b * gridDim.x + i);
            const int   k = __ldcg(a.part_idx + (size_t)b * gridDim.x + i);
            if (better(v, k, bv, bi)) { bv = v; bi = k; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            int   oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        __syncthreads();
        if (lane == 0) { s_bv[warp] = bv; s_bi[warp] = bi; }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < 8; ++w) if (better(s_bv[w], s_bi[w], bv, bi)) { bv = s_bv[w]; bi = s_bi[w]; }
            const int tok = bi < 0 ? 0 : bi;
            if (a.out_tok) a.out_tok[b] = tok;
            if (a.out_tok_f32) a.out_tok_f32[b] = (float)tok;
        }
    }
    if (threadIdx.x == 0) *a.ticket = 0u;      // ready for the next launch
}

// Host side: picks lanes-per-row and batch tile, launches on `stream`.
int launch_gemv(int wtype, GemvArgs a, cudaStream_t stream);
// Upper bound of the grid launch_gemv uses (for sizing ARGMAX scratch).
int gemv_max_grid();

}  // namespace ab
