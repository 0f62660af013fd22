// Dequant-fused GEMV over GGUF Q4_0 / Q4_K blocks:  y[b][n] = sum_k W[n][k] x[b][k].
//
// Replaces the reference's Q4 mat-vec shader and its dispatch
// (adamah-MAIN/adamah/shaders/src/f32/map_matvec_t_xq4.comp;
// adamah.c:8606-8691 exec_matvec_t_xq_internal) and the fused variants built on
// it (map_fused_gateup_t_xq4.comp, map_matvec_argmax_t_xq4.comp + map_argmax_pairs.comp).
//
// Layout.  A "unit" is 16 bytes of packed nibbles = 32 weights.
//   Q4_0: units live in a quant plane (one uint4 per 18-byte GGUF block, its 16
//         nibble bytes) and the fp16 block scales in a separate plane, so every
//         load is 16-byte aligned.  Byte j of a unit holds weight j (low nibble)
//         and weight j+16 (high nibble); value = d * (q - 8).  Work item = 1 unit.
//   Q4_K: native 144-byte superblocks = 9 uint4: one header (d, dmin, 12 bytes of
//         6-bit scales/mins) + 8 units.  Units 2g and 2g+1 hold sub-block 2g in
//         their low nibbles and sub-block 2g+1 in their high nibbles;
//         value = (d*sc) * q - (dmin*m).  Work item = such a pair (64 weights),
//         so one scale decode serves 64 weights.
// Mapping.  L lanes share a row (L = 4..32, picked per shape on the host), every
// lane owns TWO rows so the activations it reads from shared memory are used
// twice, and a warp covers (32/L)*2 rows per pass.  A warp walks its passes as one
// linear stream of (pass, item) steps with a PF-deep register prefetch ring, so
// weight loads for later steps are in flight while the current one is decoded.
// Arithmetic.  A nibble q becomes the float 128+q with ONE byte permute (the
// nibble lands in the top mantissa bits of 2^7), and goes straight into an FMA
// with its activation; the constant is removed afterwards per item with the
// pre-summed activations: sum((128+q) x) - (128+z) * sum(x).  The per-item
// result is then scaled by the block scale and added in fp32.  Lanes combine
// with xor shuffles.
// Activations are staged once per CTA in shared memory in groups of one item
// (32 or 64 floats) followed by 4 pad floats; the pad keeps the float4 reads of
// neighbouring lanes in different banks and holds the group's two half sums.
#pragma once
#include "common.cuh"

#ifndef ADAM_B200_F32X2
#define ADAM_B200_F32X2 1       // use packed fma.rn.f32x2 (sm_100) for the inner products
#endif

namespace ab {

enum { WT_Q4_0 = 0, WT_Q4_K = 1, WT_Q8_0 = 2, WT_Q5_0 = 3 };   // the last two: blocks8.cuh (own kernels, not the ones below)
enum { EPI_STORE = 0, EPI_GEGLU = 1, EPI_SWIGLU = 2, EPI_ARGMAX = 3 };

template <int WT> struct Geo;
template <> struct Geo<WT_Q4_0> { static constexpr int ELEMS = 32, STRIDE = 36, PF = 4; };
template <> struct Geo<WT_Q4_K> { static constexpr int ELEMS = 64, STRIDE = 68, PF = 2; };

struct WeightRef {          // a [N,K] tensor inside a GGUF-block map
    const uint4*  q;        // Q4_0: first unit of the tensor in the quant plane
                            // Q4_K: first superblock (9 uint4 each)
    const __half* d;        // Q4_0: first block scale; unused for Q4_K
    const uint32_t* h;      // Q5_0 only: first word of the high-bit plane (Q8_0 / Q5_0: q = quant plane, d = scale plane)
};

struct GemvArgs {
    WeightRef w0, w1;       // w1 only for GEGLU/SWIGLU (the "up" matrix)
    const float* x; int ldx;        // activations [B][ldx]
    float* y; int ldy;              // outputs [B][ldy] (may be NULL for ARGMAX)
    int N, K, B;
    int epi;
    // Optional fused input chain (replaces x; rows of length K, leading dimension ldx):
    //   h' = h_in + (add_src ? (w_post ? rms(add_src) * w_post : add_src) : 0)
    //   x  = w_pre ? rms(h') * w_pre : h'
    // with rms(v) * w = (v / sqrt(mean(v^2) + eps)) * w.  CTA 0 stores h' to h_out
    // (must not alias h_in: other CTAs still read it).  This is the reference's
    // map_rmsnorm_add + map_rmsnorm pair (engine.py:3259, :3267) folded into the
    // consumer instead of two single-CTA dispatches.
    const float* h_in; const float* add_src; const float* w_post; const float* w_pre; float* h_out; float eps;
    // ARGMAX epilogue
    float* part_val; int* part_idx; // [B][gridDim.x] scratch
    unsigned int* ticket;           // one counter, zero between launches
    int* out_tok;                   // [B] winning row per batch entry
    float* out_tok_f32;             // optional: same id stored as float (reference convention)
    float* out_val;                 // optional: the winning logit (before any softcap)
    float softcap;                  // applied to stored logits only (monotone)
    int max_grid;                   // 0 = launcher's choice; otherwise an upper bound on the CTAs launched
    uint32_t* err;                  // device error word (set by launch_gemv_mma)
#ifdef ADAM_B200_STEP_TRACE
    long long* trace;               // 8 stamps per CTA for the first 8 CTAs of the first batch group (NULL = off)
#endif
};

__device__ __forceinline__ uint4 ld_stream(const uint4* p) { return __ldcs(p); }

// acc{0,1} += a{0,1} * b{0,1}
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
#if ADAM_B200_F32X2
    asm("{\n\t.reg .b64 ra, rb, rc;\n\t"
        "mov.b64 ra, {%2, %3};\n\t"
        "mov.b64 rb, {%4, %5};\n\t"
        "mov.b64 rc, {%0, %1};\n\t"
        "fma.rn.f32x2 rc, ra, rb, rc;\n\t"
        "mov.b64 {%0, %1}, rc;\n\t}"
        : "+f"(d0), "+f"(d1) : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
#else
    d0 = fmaf(a0, b0, d0);
    d1 = fmaf(a1, b1, d1);
#endif
}

// Byte i of a word whose bytes are nibble values 0..15 -> the float 128 + value.
#define NIBF(m4, i) __uint_as_float(__byte_perm((m4), 0x43000000u, 0x7054u | ((i) << 8)))

// One unit (16 bytes) against 16 "low" and 16 "high" activations:
// plo += sum (128 + lo_nibble_j) * xlo[j],  phi += sum (128 + hi_nibble_j) * xhi[j].
// Each sum runs in two interleaved chains (even / odd j).
__device__ __forceinline__ void dot_unit(const uint4& q, const float* xlo_p, const float* xhi_p,
                                         float (&plo)[2], float (&phi)[2]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 xl = *reinterpret_cast<const float4*>(xlo_p + 4 * i);
        const float4 xh = *reinterpret_cast<const float4*>(xhi_p + 4 * i);
        const uint32_t l4 = w[i] & 0x0F0F0F0Fu, h4 = (w[i] >> 4) & 0x0F0F0F0Fu;
        fma2(plo[0], plo[1], NIBF(l4, 0), NIBF(l4, 1), xl.x, xl.y);
        fma2(phi[0], phi[1], NIBF(h4, 0), NIBF(h4, 1), xh.x, xh.y);
        fma2(plo[0], plo[1], NIBF(l4, 2), NIBF(l4, 3), xl.z, xl.w);
        fma2(phi[0], phi[1], NIBF(h4, 2), NIBF(h4, 3), xh.z, xh.w);
    }
}

// Same, but the activations are already in registers (batched path: the decoded
// nibbles are reused for every batch row).
__device__ __forceinline__ void unpack_unit128(const uint4& q, float (&lo)[16], float (&hi)[16]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t l4 = w[i] & 0x0F0F0F0Fu, h4 = (w[i] >> 4) & 0x0F0F0F0Fu;
        lo[4*i+0] = NIBF(l4, 0); lo[4*i+1] = NIBF(l4, 1); lo[4*i+2] = NIBF(l4, 2); lo[4*i+3] = NIBF(l4, 3);
        hi[4*i+0] = NIBF(h4, 0); hi[4*i+1] = NIBF(h4, 1); hi[4*i+2] = NIBF(h4, 2); hi[4*i+3] = NIBF(h4, 3);
    }
}
__device__ __forceinline__ void dot16x(const float (&wv)[16], const float* xp, float (&p)[2]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 x = *reinterpret_cast<const float4*>(xp + 4 * i);
        fma2(p[0], p[1], wv[4*i], wv[4*i+1], x.x, x.y);
        fma2(p[0], p[1], wv[4*i+2], wv[4*i+3], x.z, x.w);
    }
}

// Effective scales (d*sc) and mins (dmin*m) of sub-blocks 2g and 2g+1 from a
// Q4_K header (x = d | dmin<<16, y/z/w = the 12 packed bytes), branch-light
// restatement of the unpack at adam/loaders/gguf.py:325-328.
__device__ __forceinline__ void q4k_scales(const uint4& h, int g, float& s0, float& m0, float& s1, float& m1) {
    const int sh = (g & 1) * 16;
    const uint32_t s16 = (h.y >> sh) & 0xFFFFu, m16 = (h.z >> sh) & 0xFFFFu, t16 = (h.w >> sh) & 0xFFFFu;
    uint32_t sp, mp;
    if (g < 2) { sp = s16 & 0x3F3Fu; mp = m16 & 0x3F3Fu; }
    else { sp = (t16 & 0x0F0Fu) | ((s16 >> 2) & 0x3030u); mp = ((t16 >> 4) & 0x0F0Fu) | ((m16 >> 2) & 0x3030u); }
    const float d = __half2float(__ushort_as_half((unsigned short)(h.x & 0xFFFFu)));
    const float dm = __half2float(__ushort_as_half((unsigned short)(h.x >> 16)));
    s0 = d * (float)(sp & 0xFFu); s1 = d * (float)(sp >> 8);
    m0 = dm * (float)(mp & 0xFFu); m1 = dm * (float)(mp >> 8);
}

__device__ __forceinline__ bool better(float cv, int ci, float bv, int bi) {
    // higher value wins, ties go to the lower index (map_argmax.comp `better`)
    if (bi < 0) return ci >= 0;
    if (ci < 0) return false;
    return (cv > bv) || (cv == bv && ci < bi);
}

// What one ring slot holds: this lane's item for its two rows.
template <int WT> struct Slot;
template <> struct Slot<WT_Q4_0> { uint4 qa, qb; unsigned short da, db; };
template <> struct Slot<WT_Q4_K> { uint4 qa0, qa1, qb0, qb1, ha, hb; };

template <int WT>
__device__ __forceinline__ void fetch_slot(Slot<WT>& s, const WeightRef& wa, const WeightRef& wb, size_t rowA, size_t rowB,
                                           int items, int it) {
    if constexpr (WT == WT_Q4_0) {
        s.qa = ld_stream(wa.q + rowA * items + it);
        s.qb = ld_stream(wb.q + rowB * items + it);
        s.da = __ldcs(reinterpret_cast<const unsigned short*>(wa.d) + rowA * items + it);
        s.db = __ldcs(reinterpret_cast<const unsigned short*>(wb.d) + rowB * items + it);
    } else {
        const int sb = it >> 2, g = it & 3;
        const uint4* pa = wa.q + (rowA * (size_t)(items >> 2) + sb) * 9;
        const uint4* pb = wb.q + (rowB * (size_t)(items >> 2) + sb) * 9;
        s.qa0 = ld_stream(pa + 1 + 2 * g); s.qa1 = ld_stream(pa + 2 + 2 * g);
        s.qb0 = ld_stream(pb + 1 + 2 * g); s.qb1 = ld_stream(pb + 2 + 2 * g);
        s.ha = __ldg(pa);
        s.hb = __ldg(pb);
    }
}

template <int WT, int NB>
__device__ __forceinline__ void consume_slot(const Slot<WT>& s, int it, const float* xs, int xs_ld,
                                             float (&accA)[NB], float (&accB)[NB]) {
    const float* xp = xs + it * Geo<WT>::STRIDE;
    if constexpr (WT == WT_Q4_0) {
        const float sa = __half2float(__ushort_as_half(s.da)), sb = __half2float(__ushort_as_half(s.db));
        if constexpr (NB == 1) {
            float pa[2] = {0.f, 0.f}, pa2[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f}, pb2[2] = {0.f, 0.f};
            dot_unit(s.qa, xp, xp + 16, pa, pa2);
            dot_unit(s.qb, xp, xp + 16, pb, pb2);
            const float sx = xp[32] + xp[33];
            accA[0] = fmaf(sa, fmaf(-136.f, sx, (pa[0] + pa[1]) + (pa2[0] + pa2[1])), accA[0]);
            accB[0] = fmaf(sb, fmaf(-136.f, sx, (pb[0] + pb[1]) + (pb2[0] + pb2[1])), accB[0]);
        } else {
            float alo[16], ahi[16], blo[16], bhi[16];
            unpack_unit128(s.qa, alo, ahi);
            unpack_unit128(s.qb, blo, bhi);
#pragma unroll
            for (int b = 0; b < NB; ++b) {
                const float* xb = xp + b * xs_ld;
                float pa[2] = {0.f, 0.f}, pb[2] = {0.f, 0.f};
                dot16x(alo, xb, pa); dot16x(ahi, xb + 16, pa);
                dot16x(blo, xb, pb); dot16x(bhi, xb + 16, pb);
                const float sx = xb[32] + xb[33];
                accA[b] = fmaf(sa, fmaf(-136.f, sx, pa[0] + pa[1]), accA[b]);
                accB[b] = fmaf(sb, fmaf(-136.f, sx, pb[0] + pb[1]), accB[b]);
            }
        }
    } else {
        const int g = it & 3;
        float sA0, mA0, sA1, mA1, sB0, mB0, sB1, mB1;
        q4k_scales(s.ha, g, sA0, mA0, sA1, mA1);
        q4k_scales(s.hb, g, sB0, mB0, sB1, mB1);
        if constexpr (NB == 1) {
            float alo[2] = {0.f, 0.f}, ahi[2] = {0.f, 0.f}, blo[2] = {0.f, 0.f}, bhi[2] = {0.f, 0.f};
            dot_unit(s.qa0, xp, xp + 32, alo, ahi);
            dot_unit(s.qb0, xp, xp + 32, blo, bhi);
            dot_unit(s.qa1, xp + 16, xp + 48, alo, ahi);
            dot_unit(s.qb1, xp + 16, xp + 48, blo, bhi);
            const float s0 = xp[64], s1 = xp[65];
            const float qlo_a = fmaf(-128.f, s0, alo[0] + alo[1]), qhi_a = fmaf(-128.f, s1, ahi[0] + ahi[1]);
            const float qlo_b = fmaf(-128.f, s0, blo[0] + blo[1]), qhi_b = fmaf(-128.f, s1, bhi[0] + bhi[1]);
            accA[0] += (sA0 * qlo_a - mA0 * s0) + (sA1 * qhi_a - mA1 * s1);
            accB[0] += (sB0 * qlo_b - mB0 * s0) + (sB1 * qhi_b - mB1 * s1);
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float alo[16], ahi[16], blo[16], bhi[16];
                unpack_unit128(h ? s.qa1 : s.qa0, alo, ahi);
                unpack_unit128(h ? s.qb1 : s.qb0, blo, bhi);
#pragma unroll
                for (int b = 0; b < NB; ++b) {
                    const float* xb = xp + b * xs_ld + h * 16;
                    float pal[2] = {0.f, 0.f}, pah[2] = {0.f, 0.f}, pbl[2] = {0.f, 0.f}, pbh[2] = {0.f, 0.f};
                    dot16x(alo, xb, pal); dot16x(ahi, xb + 32, pah);
                    dot16x(blo, xb, pbl); dot16x(bhi, xb + 32, pbh);
                    // half sums of this unit's activations are not stored; remove the
                    // 128 offset with the group sums once, on the second half
                    float ta = sA0 * (pal[0] + pal[1]) + sA1 * (pah[0] + pah[1]);
                    float tb = sB0 * (pbl[0] + pbl[1]) + sB1 * (pbh[0] + pbh[1]);
                    if (h == 1) {
                        const float s0 = xp[b * xs_ld + 64], s1 = xp[b * xs_ld + 65];
                        ta -= (128.f * sA0 + mA0) * s0 + (128.f * sA1 + mA1) * s1;
                        tb -= (128.f * sB0 + mB0) * s0 + (128.f * sB1 + mB1) * s1;
                    }
                    accA[b] += ta;
                    accB[b] += tb;
                }
            }
        }
    }
}

template <int WT, int L, int NB>
__global__ void __launch_bounds__(256, (WT == WT_Q4_0 && NB == 1) ? 2 : 1) k_gemv(const GemvArgs a) {
    extern __shared__ __align__(16) float xs[];
    __shared__ float s_bv[8 * NB];
    __shared__ int   s_bi[8 * NB];
    __shared__ bool  s_last;
    constexpr int RPW = 32 / L;                 // row slots per warp pass
    constexpr int PF = Geo<WT>::PF;             // prefetch ring depth
    constexpr int GE = Geo<WT>::ELEMS, GS = Geo<WT>::STRIDE;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int sub = lane / L, l = lane % L;
    const int items = a.K / GE;
    const bool pair_mats = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    const int n_slots = pair_mats ? a.N : (a.N + 1) / 2;
    const int n_pass = (n_slots + RPW - 1) / RPW;
    const int U = (items + L - 1) / L;          // steps per pass for one lane
    const int xs_ld = items * GS;
    const WeightRef& wB = pair_mats ? a.w1 : a.w0;

    const int gw = blockIdx.x * n_warps + warp, gstride = gridDim.x * n_warps;
    const int my_passes = (n_pass > gw) ? (n_pass - gw + gstride - 1) / gstride : 0;
    const int T = my_passes * U;

    auto rows_of = [&](int pass, size_t& rowA, size_t& rowB, int& slot, bool& live) {
        slot = pass * RPW + sub;
        live = slot < n_slots;
        if (pair_mats) { rowA = rowB = (size_t)(live ? slot : 0); }
        else { rowA = (size_t)(live ? 2 * slot : 0); rowB = (rowA + 1 < (size_t)a.N) ? rowA + 1 : rowA; }
    };

    // Start the weight stream before the activations are staged: they are independent.
    Slot<WT> ring[PF];
    int f_pass = gw, f_ui = 0, f_cnt = 0;
    size_t f_rowA = 0, f_rowB = 0; int f_slot = 0; bool f_live = false;
    if (T > 0) rows_of(f_pass, f_rowA, f_rowB, f_slot, f_live);
    auto fetch_next = [&](Slot<WT>& s) {
        const int it = f_ui * L + l;
        if (f_live && it < items) fetch_slot<WT>(s, a.w0, wB, f_rowA, f_rowB, items, it);
        ++f_cnt;
        if (++f_ui == U) { f_ui = 0; f_pass += gstride; if (f_cnt < T) rows_of(f_pass, f_rowA, f_rowB, f_slot, f_live); }
    };
#pragma unroll
    for (int i = 0; i < PF; ++i) if (f_cnt < T) fetch_next(ring[i]);

    pdl_launch_dependents();
    pdl_wait();             // the weight prefetch above is independent of earlier kernels; the activations are not
    {   // stage activations: group g of GE floats lands at xs[g * GS], its half sums in the pad
        const int n4 = a.K >> 2;
        if (a.h_in) {
            __shared__ float red[33];
            for (int b = 0; b < NB; ++b) {
                const size_t row = (size_t)min(b, a.B - 1) * a.ldx;
                const float* hp = a.h_in + row;
                const float* ap = a.add_src ? a.add_src + row : nullptr;
                float* xb = xs + b * xs_ld;
                if (n4 <= 3 * (int)blockDim.x) {
                    // Fast path: every vector this chain touches is fetched up front (at most
                    // three float4 per thread and vector), so the chain costs two reductions
                    // and one memory round trip instead of a round trip per loop iteration.
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
                    const float rcp_a = __frcp_rn(rms_a);
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        if (ap) {
                            if (a.w_post) {
                                vh[j].x += div_by(va[j].x, rms_a, rcp_a) * vp[j].x; vh[j].y += div_by(va[j].y, rms_a, rcp_a) * vp[j].y;
                                vh[j].z += div_by(va[j].z, rms_a, rcp_a) * vp[j].z; vh[j].w += div_by(va[j].w, rms_a, rcp_a) * vp[j].w;
                            } else { vh[j].x += va[j].x; vh[j].y += va[j].y; vh[j].z += va[j].z; vh[j].w += va[j].w; }
                        }
                        ss = fmaf(vh[j].x, vh[j].x, ss); ss = fmaf(vh[j].y, vh[j].y, ss); ss = fmaf(vh[j].z, vh[j].z, ss); ss = fmaf(vh[j].w, vh[j].w, ss);
                        const int i = threadIdx.x + j * blockDim.x;
                        if (i < n4 && a.h_out && blockIdx.x == 0 && b < a.B) reinterpret_cast<float4*>(a.h_out + row)[i] = vh[j];
                    }
                    float rms = 1.f;
                    if (a.w_pre) { ss = block_sum(ss, red); rms = sqrtf(ss / (float)a.K + a.eps); }
                    const float rcp = __frcp_rn(rms);
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        const int i = threadIdx.x + j * blockDim.x;
                        if (i < n4) {
                            float4 v = vh[j];
                            if (a.w_pre) { v.x = div_by(v.x, rms, rcp) * vw[j].x; v.y = div_by(v.y, rms, rcp) * vw[j].y; v.z = div_by(v.z, rms, rcp) * vw[j].z; v.w = div_by(v.w, rms, rcp) * vw[j].w; }
                            const int e = i * 4;
                            *reinterpret_cast<float4*>(xb + (e / GE) * GS + (e % GE)) = v;
                        }
                    }
                    continue;
                }
                float rms_a = 1.f;
                if (ap && a.w_post) {
                    float ss = 0.f;
                    for (int i = threadIdx.x; i < a.K; i += blockDim.x) { const float v = ap[i]; ss = fmaf(v, v, ss); }
                    ss = block_sum(ss, red);
                    rms_a = sqrtf(ss / (float)a.K + a.eps);
                }
                float ss = 0.f;
                for (int i = threadIdx.x; i < a.K; i += blockDim.x) {
                    float v = hp[i];
                    if (ap) v = v + (a.w_post ? __fdiv_rn(ap[i], rms_a) * a.w_post[i] : ap[i]);
                    xb[(i / GE) * GS + (i % GE)] = v;
                    ss = fmaf(v, v, ss);
                    if (a.h_out && blockIdx.x == 0 && b < a.B) a.h_out[row + i] = v;
                }
                if (a.w_pre) {
                    ss = block_sum(ss, red);
                    const float rms = sqrtf(ss / (float)a.K + a.eps);
                    for (int i = threadIdx.x; i < a.K; i += blockDim.x) {
                        float* p = xb + (i / GE) * GS + (i % GE);
                        *p = __fdiv_rn(*p, rms) * a.w_pre[i];
                    }
                }
            }
        } else {
            for (int b = 0; b < NB; ++b) {
                const float4* src = reinterpret_cast<const float4*>(a.x + (size_t)min(b, a.B - 1) * a.ldx);
                for (int i = threadIdx.x; i < n4; i += blockDim.x) {
                    const int e = i * 4;
                    *reinterpret_cast<float4*>(xs + b * xs_ld + (e / GE) * GS + (e % GE)) = src[i];
                }
            }
        }
        __syncthreads();
        for (int i = threadIdx.x; i < NB * items * 2; i += blockDim.x) {
            const int b = i / (items * 2), r = i % (items * 2);
            float* grp = xs + b * xs_ld + (r >> 1) * GS;
            const float* p = grp + (r & 1) * (GE / 2);
            float s = 0.f;
#pragma unroll
            for (int k = 0; k < GE / 2; ++k) s += p[k];
            grp[GE + (r & 1)] = s;
        }
        __syncthreads();
    }

    float best_v[NB]; int best_i[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) { best_v[b] = -3.402823466e+38f; best_i[b] = -1; }
    float accA[NB], accB[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) { accA[b] = 0.f; accB[b] = 0.f; }

    int c_pass = gw, c_ui = 0;
    size_t rowA = 0, rowB = 0; int slot = 0; bool live = false;
    if (T > 0) rows_of(c_pass, rowA, rowB, slot, live);

    for (int t0 = 0; t0 < T; t0 += PF) {
#pragma unroll
        for (int i = 0; i < PF; ++i) {
            if (t0 + i < T) {
                const Slot<WT> cur = ring[i];
                if (f_cnt < T) fetch_next(ring[i]);
                const int it = c_ui * L + l;
                if (live && it < items) consume_slot<WT, NB>(cur, it, xs, xs_ld, accA, accB);
                if (++c_ui == U) {
                    // ---- end of a pass: combine the L lanes of each row, run the epilogue ----
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
                            if (b < a.B) {
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
                                    if (better(va, (int)rowA, best_v[b], best_i[b])) { best_v[b] = va; best_i[b] = (int)rowA; }
                                    if (rowB != rowA && better(vb, (int)rowB, best_v[b], best_i[b])) { best_v[b] = vb; best_i[b] = (int)rowB; }
                                }
                            }
                        }
                    }
#pragma unroll
                    for (int b = 0; b < NB; ++b) { accA[b] = 0.f; accB[b] = 0.f; }
                    c_ui = 0;
                    c_pass += gstride;
                    if (t0 + i + 1 < T) rows_of(c_pass, rowA, rowB, slot, live);
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
            float ov = __shfl_xor_sync(0xffffffffu, best_v[b], o);
            int   oi = __shfl_xor_sync(0xffffffffu, best_i[b], o);
            if (better(ov, oi, best_v[b], best_i[b])) { best_v[b] = ov; best_i[b] = oi; }
        }
        if (lane == 0) { s_bv[warp * NB + b] = best_v[b]; s_bi[warp * NB + b] = best_i[b]; }
    }
    __syncthreads();
    if (threadIdx.x < NB && (int)threadIdx.x < a.B) {
        const int b = threadIdx.x;
        float bv = s_bv[b]; int bi = s_bi[b];
        for (int w = 1; w < n_warps; ++w) if (better(s_bv[w * NB + b], s_bi[w * NB + b], bv, bi)) { bv = s_bv[w * NB + b]; bi = s_bi[w * NB + b]; }
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
            for (int w = 1; w < n_warps; ++w) if (better(s_bv[w], s_bi[w], bv, bi)) { bv = s_bv[w]; bi = s_bi[w]; }
            const int tok = bi < 0 ? 0 : bi;
            if (a.out_tok) a.out_tok[b] = tok;
            if (a.out_val) a.out_val[b] = bv;
            if (a.out_tok_f32) a.out_tok_f32[b] = (float)tok;
        }
    }
    if (threadIdx.x == 0) *a.ticket = 0u;      // ready for the next launch
}

// Host side: picks lanes-per-row, CTA size and batch tile, launches on `stream`.
int launch_gemv(int wtype, GemvArgs a, cudaStream_t stream);
// Upper bound of the grid launch_gemv uses (for sizing ARGMAX scratch).
int gemv_max_grid();

}  // namespace ab
