// The token kernel: see token.cuh for what it replaces.
//
// Structure.  grid = one CTA per SM (cooperative launch: all CTAs are resident), 16 warps each.
// A token is a fixed sequence of phases -- per layer: QKV product, attention, o-proj product,
// gate/up product with GeGLU, down product; then the LM head -- and every CTA walks that sequence.
//
//  * Weights.  Each warp owns a ring of shared-memory stages that bulk copies (cp.async.bulk +
//    mbarrier) fill with the row-tiled weight tiles (tile.cu) the warp will need, in the order it
//    will need them, ACROSS phases and layers: the copy stream of a warp never waits for
//    activations, so by the time a phase's input arrives its first tiles are already on chip.
//    The arithmetic on a tile is that of the tensor-core GEMV (gemv_mma.cuh): integer MMA over raw
//    nibbles and three signed byte planes of the activations, exact up to the fp32 accumulation.
//  * Activations.  CTAs hand vectors to each other through global-memory buffers of 8-byte packets
//    {fp32 bits, tag}: the producer stores each value together with a tag that is unique to the
//    (token step, layer), the consumer polls the packets it needs until every tag matches.  One
//    8-byte store / load is a single access, so a matching tag proves the value: there is no
//    separate flag, no fence and no grid-wide barrier, and a hand-over costs one trip through L2.
//    Buffers alternate between two halves by layer parity, so a producer two layers ahead can never
//    overwrite what a slower CTA still has to read (everything a CTA writes is needed, through the
//    chain of products, by every CTA of the next layer).
//  * Residual stream.  Every CTA keeps its own copy of the hidden state in shared memory and updates
//    it with the same arithmetic in the same order (bit-identical across CTAs), so the stream itself
//    is never exchanged: only the o-proj and down-proj outputs are.
//  * Every wait is bounded (mbarrier polls by count, packet polls by clock).  A wait that runs out
//    sets DEVERR_WAIT and a sticky per-decoder word; the CTA stops computing, lets its outstanding
//    copies land, and returns; other CTAs see the word in their own poll loops and do the same.
#pragma once
#include "token.cuh"
#include "gemv_mma.cuh"

namespace ab {

constexpr long long TK_WAIT_CYCLES = 600LL * 1000 * 1000;   // about 0.3 s at 2 GHz

__device__ __forceinline__ void st_pkt(uint2* p, float v, uint32_t tag) {
    const unsigned long long w = ((unsigned long long)tag << 32) | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" :: "l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ uint2 ld_pkt(const uint2* p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return make_uint2((uint32_t)w, (uint32_t)(w >> 32));
}

struct TkWait {
    long long deadline;
    const uint32_t* dead;
    bool failed;
    __device__ __forceinline__ bool give_up(uint32_t& spins) {      // call once per unsuccessful poll round
        if ((++spins & 63u) == 0u) {
            if (clock64() > deadline || *reinterpret_cast<const volatile uint32_t*>(dead) != 0u) { failed = true; return true; }
        }
        return false;
    }
};

// Poll N packets (NULL pointers are skipped) until every tag matches; values land in out[].
template <int N>
__device__ __forceinline__ void poll_pkts(const uint2* const (&ptr)[N], uint32_t tag, float (&out)[N], TkWait& wt) {
    uint32_t spins = 0;
    if (wt.failed) {
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = 0.f;
        return;
    }
    while (true) {
        uint2 v[N];
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = ptr[i] ? ld_pkt(ptr[i]) : make_uint2(0u, tag);
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; ++i) ok = ok && (v[i].y == tag);
#pragma unroll
        for (int i = 0; i < N; ++i) out[i] = __uint_as_float(v[i].x);
        if (ok) return;
        if (wt.give_up(spins)) return;
    }
}

// Wait for a stage of the weight ring; gives up at the deadline.
__device__ __forceinline__ bool tk_mbar_wait(uint64_t* bar, uint32_t parity, long long deadline) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0;; ++spin) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
        if ((spin & 15u) == 15u && clock64() > deadline) return false;
    }
}

struct TkWork { int active, sb, kpart, rg_l, ks, n_sets, p0, np, nch, part_p0; };

// Attention work split of one layer at position p (the same on the producing and the consuming side).
struct TkAttnSplit { uint32_t start, c_first, n_chunks, n_act; };
__device__ __forceinline__ TkAttnSplit tk_attn_split(int s_max, uint32_t window, int p) {
    TkAttnSplit s;
    const uint32_t seq = (uint32_t)p + 1;
    s.start = (window > 0 && seq > window) ? seq - window : 0;
    s.c_first = s.start / 8;
    s.n_chunks = (seq - 1) / 8 - s.c_first + 1;
    s.n_act = min((uint32_t)s_max, (s.n_chunks + TK_NW - 1) / TK_NW);
    return s;
}

template <int WT> struct TkGeo {
    static constexpr int TILE = mma_tile_bytes(WT);
    static constexpr int CH = WT == WT_Q4_0 ? 6 : 4;        // tile slots per stage
    static constexpr int NSTAGE = 3;
    static constexpr int STAGE_BYTES = CH * TILE;
    static constexpr int RING_BYTES = NSTAGE * STAGE_BYTES; // per warp
};

// Shared-memory layout (dynamic part), computed identically on the host (token.cu).
struct TkSmemLayout { size_t xb, sx, ml, h, wp, work, ring, total; };
__host__ __device__ inline TkSmemLayout tk_smem_layout(int units_max, int hd, int H, int s_max, int E, int n_layer, int ring_bytes_per_warp) {
    TkSmemLayout l;
    size_t o = 0;
    l.xb = o;
    size_t xb_bytes = (size_t)units_max * 4 * 32;                       // [units][4 columns][32 bytes]
    size_t sx_bytes = (size_t)units_max * 2 * 4;                        // [units][2] pre-summed activations
    size_t attn_bytes = ((size_t)(3 + TK_NW) * hd + 2 * TK_NW + 2 * TK_NW) * 4;   // s_q, s_kn, s_vn, s_o[NW], s_m, s_l, s_w + spare
    l.sx = l.xb + xb_bytes;
    size_t scratch = xb_bytes + sx_bytes;
    if (attn_bytes > scratch) scratch = attn_bytes;
    o = (o + scratch + 15) & ~(size_t)15;
    l.ml = o; o += (size_t)H * s_max * 2 * 4; o = (o + 15) & ~(size_t)15;
    l.h = o; o += (size_t)E * 4; o = (o + 15) & ~(size_t)15;
    l.wp = o; o += (size_t)n_layer * 5 * 8; o = (o + 15) & ~(size_t)15;
    l.work = o; o += (size_t)TK_NW * TK_PHASES * sizeof(TkWork); o = (o + 127) & ~(size_t)127;
    l.ring = o; o += (size_t)TK_NW * ring_bytes_per_warp;
    l.total = o;
    return l;
}

template <int WT, typename T, int HD>
__global__ void __launch_bounds__(TK_THREADS, 1) k_token(const __grid_constant__ TkArgs a) {
    using G = TkGeo<WT>;
    constexpr int CH = G::CH, NSTAGE = G::NSTAGE, STAGE_BYTES = G::STAGE_BYTES, TILE = G::TILE;
    constexpr int NCOL = 4, NPR = 2, xstep = NCOL * 4;
    constexpr float SXF = WT == WT_Q4_0 ? -8.0f : -1.0f;
    constexpr float NEG = -1.0e30f;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ float s_red[2][TK_NW][2][16];
    __shared__ __align__(8) uint64_t s_bar[TK_NW][NSTAGE];
    __shared__ float red[66];
    __shared__ float s_inv;
    __shared__ float s_bv[TK_NW];
    __shared__ int s_bi[TK_NW];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int bx = blockIdx.x;
    const int E = a.E;

    int units_max = E / 32;
    if (a.q_dim / 32 > units_max) units_max = a.q_dim / 32;
    {
        const TkPhase& P = a.ph[TK_DOWN];
        const int pu = ((P.pairs + P.cpr - 1) / P.cpr + 1) * 2;
        if (pu > units_max) units_max = pu;
    }
    const TkSmemLayout lay = tk_smem_layout(units_max, HD, a.H, a.s_max, E, a.n_layer, G::RING_BYTES);
    signed char* xb = reinterpret_cast<signed char*>(smem_raw + lay.xb);
    float* s_sx = reinterpret_cast<float*>(smem_raw + lay.sx);
    float* s_ml = reinterpret_cast<float*>(smem_raw + lay.ml);
    float* s_h = reinterpret_cast<float*>(smem_raw + lay.h);
    const uint8_t** s_wp = reinterpret_cast<const uint8_t**>(smem_raw + lay.wp);
    TkWork* s_work = reinterpret_cast<TkWork*>(smem_raw + lay.work);
    unsigned char* ring = smem_raw + lay.ring + (size_t)warp * G::RING_BYTES;

    TkWait wt;
    wt.deadline = clock64() + TK_WAIT_CYCLES;
    wt.dead = a.dead;
    wt.failed = false;
    if (*reinterpret_cast<const volatile uint32_t*>(a.dead) != 0u) return;      // an earlier step gave up: do nothing

    // ---- set-up: weight pointer table, per-warp work of every phase, barriers ----
    for (int i = tid; i < a.n_layer * 5; i += TK_THREADS) s_wp[i] = a.layers[i / 5].w[i % 5];
    if (lane < TK_PHASES) {
        const int p = lane;
        const TkPhase P = a.ph[p];
        TkWork w;
        w.active = 0; w.sb = 0; w.kpart = 0; w.rg_l = 0; w.ks = 0; w.n_sets = 0; w.p0 = 0; w.np = 0; w.nch = 0; w.part_p0 = 0;
        const int chp = (p == TK_GU) ? CH / 2 : CH;
        if (P.n_rg > 0 && bx < P.G * P.cpr && warp < P.RG * P.KS && !(p == TK_LM && !a.with_lm)) {
            w.sb = bx / P.cpr; w.kpart = bx % P.cpr; w.rg_l = warp / P.KS; w.ks = warp % P.KS;
            const int n_sets_total = (P.n_rg + P.RG - 1) / P.RG;
            w.n_sets = w.sb < n_sets_total ? (n_sets_total - w.sb + P.G - 1) / P.G : 0;
            const int slices = P.cpr * P.KS, s = w.kpart * P.KS + w.ks;
            w.p0 = (int)((long long)s * P.pairs / slices);
            const int p1 = (int)((long long)(s + 1) * P.pairs / slices);
            w.np = p1 - w.p0;
            w.nch = (w.np + chp - 1) / chp;
            w.part_p0 = (int)((long long)(w.kpart * P.KS) * P.pairs / slices);
            w.active = (w.n_sets > 0 && w.np > 0) ? 1 : 0;
        }
        s_work[warp * TK_PHASES + p] = w;
    }
    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < NSTAGE; ++s) mbar_init(&s_bar[warp][s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // ---- the warp's weight stream ----
    // issue cursor (lane 0): phase i_p of layer i_L, set i_set, chunk i_j; stage i_st
    int i_L = 0, i_p = -1, i_set = 0, i_j = 0, i_st = 0, issued = 0, consumed = 0;
    bool i_done = false;
    auto next_phase = [&]() {
        while (true) {
            if (i_p == TK_LM) { i_done = true; return; }
            if (i_p == TK_DOWN || i_p < 0) {
                if (i_p == TK_DOWN) ++i_L;
                i_p = (i_L < a.n_layer) ? TK_QKV : TK_LM;
            } else ++i_p;
            if (s_work[warp * TK_PHASES + i_p].active) return;
        }
    };
    auto issue_next = [&]() {                                // lane 0, !i_done
        const TkWork w = s_work[warp * TK_PHASES + i_p];
        const TkPhase& P = a.ph[i_p];
        const bool pr = (i_p == TK_GU);
        const int chp = pr ? CH / 2 : CH;
        const int rg = min((w.sb + i_set * P.G) * P.RG + w.rg_l, P.n_rg - 1);
        const int pp0 = w.p0 + i_j * chp, n = min(chp, w.p0 + w.np - pp0);
        const size_t off = ((size_t)rg * P.pairs + pp0) * TILE;
        const uint8_t* t0;
        const uint8_t* t1 = nullptr;
        if (i_p == TK_LM) t0 = a.lm_tiled;
        else if (i_p == TK_QKV) t0 = s_wp[i_L * 5 + 0];
        else if (i_p == TK_O) t0 = s_wp[i_L * 5 + 1];
        else if (i_p == TK_GU) { t0 = s_wp[i_L * 5 + 2]; t1 = s_wp[i_L * 5 + 3]; }
        else t0 = s_wp[i_L * 5 + 4];
        unsigned char* dst = ring + (size_t)i_st * STAGE_BYTES;
        mbar_expect_tx(&s_bar[warp][i_st], (uint32_t)(n * TILE * (pr ? 2 : 1)));
        bulk_g2s(dst, t0 + off, (uint32_t)(n * TILE), &s_bar[warp][i_st]);
        if (pr) bulk_g2s(dst + chp * TILE, t1 + off, (uint32_t)(n * TILE), &s_bar[warp][i_st]);
        ++issued;
        if (++i_st == NSTAGE) i_st = 0;
        if (++i_j == w.nch) { i_j = 0; if (++i_set == w.n_sets) { i_set = 0; next_phase(); } }
    };
    if (lane == 0) {
        next_phase();
#pragma unroll
        for (int c = 0; c < NSTAGE; ++c) if (!i_done) issue_next();
    }
    int c_st = 0; uint32_t c_ph = 0;                        // consumer: next stage and its parity
    bool timed_out = false;

    // ---- this step ----
    const uint32_t seq_no = *a.seq;
    const int p = a.pos[0];
    int tok = (p < a.prompt_len[0]) ? a.prompt_tok[p] : a.cur_tok[0];
    if (tok < 0 || tok >= a.V) { if (tid == 0 && bx == 0) atomicOr(a.err, DEVERR_BAD_TOKEN); tok = 0; }
    if ((uint32_t)p >= a.n_pos) { if (tid == 0 && bx == 0) atomicOr(a.err, DEVERR_OOB_MAP); }
    const uint32_t tag_base = seq_no * 128u;

    // embedding row -> private copy of the residual stream (k_embed's arithmetic)
    for (int i = tid; i < E / 4; i += TK_THREADS) {
        const int k0 = 4 * i;
        float4 v;
        if (a.embd_wt == WT_Q4_0) {
            const int nblk = E / 32, blk = k0 >> 5, w = k0 & 31;
            const uint32_t word = reinterpret_cast<const uint32_t*>(a.embd.q + (size_t)tok * nblk + blk)[(w & 15) >> 2];
            const float s = __half2float(a.embd.d[(size_t)tok * nblk + blk]);
            const uint32_t nib = (w & 16) ? (word >> 4) & 0x0F0F0F0Fu : word & 0x0F0F0F0Fu;
            v.x = __fmul_rn(__fmul_rn((float)(int)(nib & 0xFFu) - 8.f, s), a.emb_scale);
            v.y = __fmul_rn(__fmul_rn((float)(int)((nib >> 8) & 0xFFu) - 8.f, s), a.emb_scale);
            v.z = __fmul_rn(__fmul_rn((float)(int)((nib >> 16) & 0xFFu) - 8.f, s), a.emb_scale);
            v.w = __fmul_rn(__fmul_rn((float)(int)(nib >> 24) - 8.f, s), a.emb_scale);
        } else {
            const int nsb = E / 256, sb = k0 >> 8, r = k0 & 255, grp = r >> 6, j = r & 63;
            const uint8_t* blk = reinterpret_cast<const uint8_t*>(a.embd.q) + ((size_t)tok * nsb + sb) * 144;
            const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
            const int sh = (grp & 1) * 16;
            const uint32_t s16 = (hdr.y >> sh) & 0xFFFFu, m16 = (hdr.z >> sh) & 0xFFFFu, t16 = (hdr.w >> sh) & 0xFFFFu;
            uint32_t sp, mp;
            if (grp < 2) { sp = s16 & 0x3F3Fu; mp = m16 & 0x3F3Fu; }
            else { sp = (t16 & 0x0F0Fu) | ((s16 >> 2) & 0x3030u); mp = ((t16 >> 4) & 0x0F0Fu) | ((m16 >> 2) & 0x3030u); }
            const float dd = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
            const float dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
            const bool hi = j >= 32;
            const float sc = __fmul_rn(dd, (float)(hi ? (sp >> 8) : (sp & 0xFFu)));
            const float mn = __fmul_rn(dm, (float)(hi ? (mp >> 8) : (mp & 0xFFu)));
            const uint32_t word = *reinterpret_cast<const uint32_t*>(blk + 16 + grp * 32 + (j & 31));
            const uint32_t nib = hi ? (word >> 4) & 0x0F0F0F0Fu : word & 0x0F0F0F0Fu;
            v.x = __fmul_rn(__fsub_rn(__fmul_rn((float)(nib & 0xFFu), sc), mn), a.emb_scale);
            v.y = __fmul_rn(__fsub_rn(__fmul_rn((float)((nib >> 8) & 0xFFu), sc), mn), a.emb_scale);
            v.z = __fmul_rn(__fsub_rn(__fmul_rn((float)((nib >> 16) & 0xFFu), sc), mn), a.emb_scale);
            v.w = __fmul_rn(__fsub_rn(__fmul_rn((float)(nib >> 24), sc), mn), a.emb_scale);
        }
        reinterpret_cast<float4*>(s_h)[i] = v;
    }
    // (each thread reads back only the elements it wrote, so no barrier is needed before the chain)

    // ---- helpers -------------------------------------------------------------------------------
    // per-unit sums of the staged integer activations, in the units of the lane that uses them
    auto finish_staging = [&](int units) {
        __syncthreads();
        for (int i = tid; i < units * NPR; i += TK_THREADS) {
            const int u = i / NPR, pr = i % NPR;
            const int* c0 = reinterpret_cast<const int*>(xb + (size_t)(u * NCOL + 2 * pr) * 32);
            const int* c1 = c0 + 8;
            int s0 = 0, s1 = 0;
#pragma unroll
            for (int e = 0; e < 8; ++e) { s0 = __dp4a(c0[e], 0x01010101, s0); s1 = __dp4a(c1[e], 0x01010101, s1); }
            s_sx[i] = SXF * (float)(s0 * 256 + s1);
        }
        __syncthreads();
    };

    // Residual update + norm in front of a product (the reference's map_rmsnorm_add + map_rmsnorm pair,
    // engine.py:3259, :3267):  h += rms(sum of `parts` partial vectors) * w_post (plain add without w_post);
    // x = rms(h) * w_pre; x is staged for the MMAs when `stage`.
    auto chain = [&](const uint2* add_buf, int parts, uint32_t tag, const float* w_post, const float* w_pre, bool stage) {
        const int n4 = E >> 2;
        float4 vh[3], va[3];
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const int i = tid + j * TK_THREADS;
            vh[j] = i < n4 ? reinterpret_cast<const float4*>(s_h)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            va[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (add_buf) {
            const uint2* ptr[24];
            float val[24];
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int i = tid + j * TK_THREADS;
#pragma unroll
                for (int q = 0; q < 2; ++q)
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        ptr[(j * 2 + q) * 4 + e] = (i < n4 && q < parts) ? add_buf + (size_t)q * E + 4 * i + e : nullptr;
            }
            poll_pkts<24>(ptr, tag, val, wt);
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                va[j] = make_float4(val[j * 8 + 0], val[j * 8 + 1], val[j * 8 + 2], val[j * 8 + 3]);
                if (parts > 1) { va[j].x += val[j * 8 + 4]; va[j].y += val[j * 8 + 5]; va[j].z += val[j * 8 + 6]; va[j].w += val[j * 8 + 7]; }
            }
            float rms_a = 1.f;
            if (w_post) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < 3; ++j) { ss = fmaf(va[j].x, va[j].x, ss); ss = fmaf(va[j].y, va[j].y, ss); ss = fmaf(va[j].z, va[j].z, ss); ss = fmaf(va[j].w, va[j].w, ss); }
                ss = block_sum(ss, red);
                rms_a = sqrtf(ss / (float)E + a.eps);
            }
            const float rcp_a = __frcp_rn(rms_a);
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                const int i = tid + j * TK_THREADS;
                if (w_post) {
                    const float4 wp = i < n4 ? reinterpret_cast<const float4*>(w_post)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
                    vh[j].x += div_by(va[j].x, rms_a, rcp_a) * wp.x; vh[j].y += div_by(va[j].y, rms_a, rcp_a) * wp.y;
                    vh[j].z += div_by(va[j].z, rms_a, rcp_a) * wp.z; vh[j].w += div_by(va[j].w, rms_a, rcp_a) * wp.w;
                } else { vh[j].x += va[j].x; vh[j].y += va[j].y; vh[j].z += va[j].z; vh[j].w += va[j].w; }
                if (i < n4) reinterpret_cast<float4*>(s_h)[i] = vh[j];
            }
        }
        if (!stage) return;
        float4 vw[3];
        float ss = 0.f, am = 0.f;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const int i = tid + j * TK_THREADS;
            vw[j] = (i < n4 && w_pre) ? reinterpret_cast<const float4*>(w_pre)[i] : make_float4(1.f, 1.f, 1.f, 1.f);
            ss = fmaf(vh[j].x, vh[j].x, ss); ss = fmaf(vh[j].y, vh[j].y, ss); ss = fmaf(vh[j].z, vh[j].z, ss); ss = fmaf(vh[j].w, vh[j].w, ss);
            am = fmaxf(am, fmaxf(fmaxf(fabsf(vh[j].x * vw[j].x), fabsf(vh[j].y * vw[j].y)), fmaxf(fabsf(vh[j].z * vw[j].z), fabsf(vh[j].w * vw[j].w))));
        }
        block_sum_max(ss, am, red);
        if (w_pre) {
            const float rms = sqrtf(ss / (float)E + a.eps);
            const float rcp = __frcp_rn(rms);
            am = am * rcp * 1.000001f;
#pragma unroll
            for (int j = 0; j < 3; ++j) {
                vh[j].x = div_by(vh[j].x, rms, rcp) * vw[j].x; vh[j].y = div_by(vh[j].y, rms, rcp) * vw[j].y;
                vh[j].z = div_by(vh[j].z, rms, rcp) * vw[j].z; vh[j].w = div_by(vh[j].w, rms, rcp) * vw[j].w;
            }
        }
        float s, inv;
        pow2_scale(am, s, inv);
        if (tid == 0) s_inv = inv;
#pragma unroll
        for (int j = 0; j < 3; ++j) {
            const int i = tid + j * TK_THREADS;
            if (i < n4) put_x4<NCOL>(xb, 4 * i, 0, make_float4(vh[j].x * s, vh[j].y * s, vh[j].z * s, vh[j].w * s));
        }
        finish_staging(E / 32);
    };

    // Stage n plain values that arrive as packets (buf[0..n)), n a multiple of 64.
    auto stage_packets = [&](const uint2* buf, int n, uint32_t tag) {
        const int n4 = n >> 2;
        float am = 0.f;
        constexpr int J = 6;                         // float4 per thread held in registers between the two passes
        for (int base = 0; base < n4; base += J * TK_THREADS) {
            float4 v[J];
#pragma unroll
            for (int jj = 0; jj < J; jj += 3) {
                const uint2* ptr[12];
                float val[12];
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    const int i = base + tid + (jj + j) * TK_THREADS;
#pragma unroll
                    for (int e = 0; e < 4; ++e) ptr[j * 4 + e] = i < n4 ? buf + 4 * i + e : nullptr;
                }
                poll_pkts<12>(ptr, tag, val, wt);
#pragma unroll
                for (int j = 0; j < 3; ++j) v[jj + j] = make_float4(val[j * 4], val[j * 4 + 1], val[j * 4 + 2], val[j * 4 + 3]);
            }
#pragma unroll
            for (int j = 0; j < J; ++j) am = fmaxf(am, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
            if (n4 <= J * TK_THREADS) {
                // everything is in registers: one pass
                am = block_max(am, red);
                float s, inv;
                pow2_scale(am, s, inv);
                if (tid == 0) s_inv = inv;
#pragma unroll
                for (int j = 0; j < J; ++j) {
                    const int i = tid + j * TK_THREADS;
                    if (i < n4) put_x4<NCOL>(xb, 4 * i, 0, make_float4(v[j].x * s, v[j].y * s, v[j].z * s, v[j].w * s));
                }
                finish_staging(n / 32);
                return;
            }
        }
        // longer vectors: second pass re-reads the packets (they are complete by now)
        am = block_max(am, red);
        float s, inv;
        pow2_scale(am, s, inv);
        if (tid == 0) s_inv = inv;
        for (int i = tid; i < n4; i += TK_THREADS) {
            float4 v;
            v.x = __uint_as_float(ld_pkt(buf + 4 * i).x); v.y = __uint_as_float(ld_pkt(buf + 4 * i + 1).x);
            v.z = __uint_as_float(ld_pkt(buf + 4 * i + 2).x); v.w = __uint_as_float(ld_pkt(buf + 4 * i + 3).x);
            put_x4<NCOL>(xb, 4 * i, 0, make_float4(v.x * s, v.y * s, v.z * s, v.w * s));
        }
        finish_staging(n / 32);
    };

    // One 16x32 block of one matrix against the staged columns (see gemv_mma.cuh).
    const uint2* xq = reinterpret_cast<const uint2*>(xb) + (g % NCOL) * 4 + t;
    const float* sxp = s_sx + (t % NPR);
    const float cm = (t & 1) ? (1.0f / 256.0f) : 256.0f;
    auto block_imma = [&](uint32_t wg, uint32_t wh, const uint2* xu, const float* sxu, uint32_t sc2, float (&ac)[2]) {
        const uint32_t a0 = wg & 0x0F0F0F0Fu, a2 = (wg >> 4) & 0x0F0F0F0Fu;
        const uint32_t a1 = wh & 0x0F0F0F0Fu, a3 = (wh >> 4) & 0x0F0F0F0Fu;
        const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&sc2));
        const uint2 b = xu[0];
        int dd[4];
        imma16832(dd, a0, a1, a2, a3, b.x, b.y);
        const float sx = sxu[0];
        ac[0] = fmaf(d.x, (float)(dd[0] * 256 + dd[1]) + sx, ac[0]);
        ac[1] = fmaf(d.y, (float)(dd[2] * 256 + dd[3]) + sx, ac[1]);
    };
    auto block_imma_k = [&](uint32_t wg, uint32_t wh, const uint2* xu, const float* sxu, uint32_t sc4, float2 dm0, float2 dm1, float (&ac)[2]) {
        const uint32_t a0 = wg & 0x0F0F0F0Fu, a2 = (wg >> 4) & 0x0F0F0F0Fu;
        const uint32_t a1 = wh & 0x0F0F0F0Fu, a3 = (wh >> 4) & 0x0F0F0F0Fu;
        const float es0 = dm0.x * (float)(sc4 & 0xFFu), em0 = dm0.y * (float)((sc4 >> 8) & 0xFFu);
        const float es1 = dm1.x * (float)((sc4 >> 16) & 0xFFu), em1 = dm1.y * (float)(sc4 >> 24);
        const uint2 b = xu[0];
        int dd[4];
        imma16832(dd, a0, a1, a2, a3, b.x, b.y);
        const float sx = sxu[0];
        ac[0] = fmaf(es0, (float)(dd[0] * 256 + dd[1]), fmaf(em0, sx, ac[0]));
        ac[1] = fmaf(es1, (float)(dd[2] * 256 + dd[3]), fmaf(em1, sx, ac[1]));
    };
    auto do_tile = [&](const unsigned char* tile, const uint2* xu0, const float* sx0, float (&ac)[2]) {
        const uint4 q = reinterpret_cast<const uint4*>(tile)[lane];
        const uint2 sc = reinterpret_cast<const uint2*>(tile + 512)[g];
        if constexpr (WT == WT_Q4_0) {
            block_imma(q.x, q.y, xu0, sx0, sc.x, ac);
            block_imma(q.z, q.w, xu0 + xstep, sx0 + NPR, sc.y, ac);
        } else {
            const uint2 hd = reinterpret_cast<const uint2*>(tile + 576)[g];
            const float2 dm0 = __half22float2(*reinterpret_cast<const __half2*>(&hd.x));
            const float2 dm1 = __half22float2(*reinterpret_cast<const __half2*>(&hd.y));
            block_imma_k(q.x, q.y, xu0, sx0, sc.x, dm0, dm1, ac);
            block_imma_k(q.z, q.w, xu0 + xstep, sx0 + NPR, sc.y, dm0, dm1, ac);
        }
    };

    float best_v = -3.402823466e+38f; int best_i = -1;      // LM-head candidates of this lane

    // The product of phase ph for this warp.  mode 0: packets out[kpart * N + row]; 1: GeGLU / SwiGLU of the
    // two matrices; 2: LM head (arg-max candidates, optional soft-capped logits).
    auto product = [&](int ph, int mode, uint2* out, uint32_t tag) {
        const TkWork w = s_work[warp * TK_PHASES + ph];
        if (!w.active) return;
        const TkPhase& P = a.ph[ph];
        const bool pr = (ph == TK_GU);
        const int chp = pr ? CH / 2 : CH;
        const int N = P.n_rg * 16;
        const float inv = s_inv;
        int parity = 0;
        for (int si = 0; si < w.n_sets; ++si) {
            const int rg = (w.sb + si * P.G) * P.RG + w.rg_l;
            float acc0[2] = {0.f, 0.f}, acc1[2] = {0.f, 0.f};
            for (int j = 0; j < w.nch; ++j) {
                if (!timed_out) {
                    const bool ok = tk_mbar_wait(&s_bar[warp][c_st], c_ph, wt.deadline);
                    if (!__all_sync(0xffffffffu, ok)) { timed_out = true; wt.failed = true; }
                }
                if (!timed_out) {
                    const unsigned char* buf = ring + (size_t)c_st * STAGE_BYTES;
                    const int pp0 = w.p0 + j * chp, n = min(chp, w.p0 + w.np - pp0);
                    const uint2* xp = xq + (size_t)(pp0 - w.part_p0) * 2 * xstep;
                    const float* sx = sxp + (size_t)(pp0 - w.part_p0) * 2 * NPR;
                    if (n == chp) {
#pragma unroll
                        for (int k = 0; k < CH; ++k) {
                            if (k < chp) {
                                do_tile(buf + k * TILE, xp + (2 * k) * xstep, sx + (2 * k) * NPR, acc0);
                                if (pr) do_tile(buf + (chp + k) * TILE, xp + (2 * k) * xstep, sx + (2 * k) * NPR, acc1);
                            }
                        }
                    } else {
                        for (int k = 0; k < n; ++k) {
                            do_tile(buf + k * TILE, xp + (2 * k) * xstep, sx + (2 * k) * NPR, acc0);
                            if (pr) do_tile(buf + (chp + k) * TILE, xp + (2 * k) * xstep, sx + (2 * k) * NPR, acc1);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) { ++consumed; if (!i_done) issue_next(); }
                }
                if (++c_st == NSTAGE) { c_st = 0; c_ph ^= 1u; }
            }
            // even lanes: 256 * acc + (odd neighbour's acc) / 256
            float val0[2], val1[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v = acc0[h] * cm;
                val0[h] = v + __shfl_xor_sync(0xffffffffu, v, 1);
                v = acc1[h] * cm;
                val1[h] = v + __shfl_xor_sync(0xffffffffu, v, 1);
            }
            bool writer = true;
            if (P.KS > 1) {
                if (t == 0) {
                    s_red[parity][warp][0][g] = val0[0]; s_red[parity][warp][0][g + 8] = val0[1];
                    s_red[parity][warp][1][g] = val1[0]; s_red[parity][warp][1][g + 8] = val1[1];
                }
                asm volatile("bar.sync %0, %1;" :: "r"(1 + w.rg_l), "r"(P.KS * 32) : "memory");
                writer = (w.ks == 0);
                if (writer && t == 0) {
                    for (int k2 = 1; k2 < P.KS; ++k2) {
                        val0[0] += s_red[parity][warp + k2][0][g]; val0[1] += s_red[parity][warp + k2][0][g + 8];
                        val1[0] += s_red[parity][warp + k2][1][g]; val1[1] += s_red[parity][warp + k2][1][g + 8];
                    }
                }
                parity ^= 1;
            }
            if (writer && t == 0 && rg < P.n_rg && !timed_out) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rg * 16 + g + 8 * h;
                    const float va = val0[h] * inv;
                    if (mode == 0) st_pkt(out + (size_t)w.kpart * N + row, va, tag);
                    else if (mode == 1) st_pkt(out + row, (a.act == 0 ? gelu_tanh(va) : silu_clip(va)) * (val1[h] * inv), tag);
                    else {
                        float v = va;
                        if (a.logits) a.logits[row] = a.final_cap > 0.f ? tanhf(v / a.final_cap) * a.final_cap : v;
                        if (!(v == v)) v = -3.402823466e+38f;
                        if (better(v, row, best_v, best_i)) { best_v = v; best_i = row; }
                    }
                }
            }
        }
    };

    // ---- attention of one layer (QK-norm + RoPE + KV append + soft-max(QK^T)V for this CTA's (head, split)) ----
    auto attention = [&](const TkLayer& ly, int L, const uint2* qkv, uint2* att, uint32_t tag) {
        constexpr int DPL = HD / 32, CP = 8, NPQ = (HD / 2 + 31) / 32;
        const TkAttnSplit sp = tk_attn_split(a.s_max, ly.window, p);
        const uint32_t H = (uint32_t)a.H, gsz = H / (uint32_t)a.KV;
        if ((uint32_t)bx >= H * sp.n_act) return;
        const uint32_t head = (uint32_t)bx % H, split = (uint32_t)bx / H, kvh = head / gsz;
        const uint32_t seq = (uint32_t)p + 1;
        const uint32_t cpc = (sp.n_chunks + sp.n_act - 1) / sp.n_act;
        const uint32_t c0 = min(sp.c_first + split * cpc, sp.c_first + sp.n_chunks), c1 = min(sp.c_first + sp.n_chunks, c0 + cpc);
        const uint32_t c_new = (uint32_t)p / CP;
        const bool owner = c_new >= c0 && c_new < c1;
        const bool appender = owner && (head % gsz == 0);
        T* __restrict__ kv_pool = reinterpret_cast<T*>(a.kv_pool);
        const KvGeom& geo = a.geo;
        float* s_q = reinterpret_cast<float*>(smem_raw);        // [HD]           (aliases the activation staging area)
        float* s_kn = s_q + HD;                                  // [HD] newest key as stored
        float* s_vn = s_kn + HD;                                 // [HD] newest value as stored
        float* s_o = s_vn + HD;                                  // [NW][HD]
        float* s_m = s_o + TK_NW * HD;                           // [NW]
        float* s_l = s_m + TK_NW;                                // [NW]
        float* s_w = s_l + TK_NW;                                // [NW]
        const int32_t* bt = a.block_table;
        auto page_of = [&](uint32_t pn) -> int32_t { return pn < geo.max_pages ? bt[pn] : -1; };
        KvRow<T, DPL> kr[CP], vr[CP];
        auto load_rows = [&](uint32_t c, uint32_t kv, KvRow<T, DPL> (&rows)[CP]) {
            const uint32_t tp0 = c * CP;
            const uint32_t lo = max(tp0, sp.start), hi = min(tp0 + CP, seq) - 1;
            const uint32_t pn = tp0 / geo.page, slot0 = tp0 - pn * geo.page;
            const int32_t pg0 = max(page_of(pn), 0);
            const T* base = kv_pool + kv_index(geo, (uint32_t)pg0, (uint32_t)L, kv, kvh, slot0) + lane * DPL;
#pragma unroll
            for (int j = 0; j < CP; ++j) {
                const uint32_t tp = min(max(tp0 + j, lo), hi);
                rows[j].load(base + (size_t)(tp - tp0) * HD);
            }
        };
        uint32_t c = c0 + warp;
        if (c < c1) { load_rows(c, 0, kr); load_rows(c, 1, vr); }
        // rotary angles and norm weights of this position (read-only tables)
        const uint32_t half = HD / 2;
        const uint32_t pp = (uint32_t)p < a.n_pos ? (uint32_t)p : a.n_pos - 1;
        const float* ct = a.cos_t[ly.rope] + (size_t)pp * half;
        const float* st = a.sin_t[ly.rope] + (size_t)pp * half;
        // warp 0: query row; warp 1: newest key row; warp 2: newest value row (owner only)
        if (warp < 3 && (warp == 0 || owner)) {
            const bool is_q = warp == 0, is_k = warp == 1;
            const uint2* src = qkv + (is_q ? (size_t)head * HD : (size_t)a.q_dim + (is_k ? 0 : (size_t)a.k_dim) + (size_t)kvh * HD);
            const uint2* ptr[2 * NPQ];
            float val[2 * NPQ];
#pragma unroll
            for (int j = 0; j < NPQ; ++j) {
                const uint32_t i = lane + 32 * j;
                ptr[2 * j] = i < half ? src + i : nullptr;
                ptr[2 * j + 1] = i < half ? src + i + half : nullptr;
            }
            poll_pkts<2 * NPQ>(ptr, tag, val, wt);
            size_t kv_off = 0;
            bool ok = appender;
            if (!is_q && appender) {
                const int32_t page_id = page_of((uint32_t)p / geo.page);
                if (page_id < 0) { ok = false; if (lane == 0) atomicOr(a.err, DEVERR_OOB_MAP); }
                else kv_off = kv_index(geo, (uint32_t)page_id, (uint32_t)L, is_k ? 0u : 1u, kvh, (uint32_t)p % geo.page);
            }
            if (!is_q && !is_k) {
#pragma unroll
                for (int j = 0; j < NPQ; ++j) {
                    const uint32_t i = lane + 32 * j;
                    if (i < half) {
                        s_vn[i] = kv_round<T>(val[2 * j]); s_vn[i + half] = kv_round<T>(val[2 * j + 1]);
                        if (ok) { st_kv(kv_pool + kv_off + i, val[2 * j]); st_kv(kv_pool + kv_off + i + half, val[2 * j + 1]); }
                    }
                }
            } else {
                const float* wn = is_q ? ly.norm[TKN_Q] : ly.norm[TKN_K];
                float rms = 1.f;
                if (wn) {
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < NPQ; ++j) ss = fmaf(val[2 * j], val[2 * j], ss);
#pragma unroll
                    for (int j = 0; j < NPQ; ++j) ss = fmaf(val[2 * j + 1], val[2 * j + 1], ss);
                    ss = warp_sum(ss);
                    rms = sqrtf(ss / (float)HD + a.eps);
                }
                const float rcp = __frcp_rn(rms);
#pragma unroll
                for (int j = 0; j < NPQ; ++j) {
                    const uint32_t i = lane + 32 * j;
                    if (i < half) {
                        float a0 = val[2 * j], a1 = val[2 * j + 1];
                        if (wn) { a0 = div_by(a0, rms, rcp) * wn[i]; a1 = div_by(a1, rms, rcp) * wn[i + half]; }
                        const float cs = ct[i], sn = st[i];
                        const float y0 = __fsub_rn(__fmul_rn(a0, cs), __fmul_rn(a1, sn));
                        const float y1 = __fadd_rn(__fmul_rn(a0, sn), __fmul_rn(a1, cs));
                        if (is_q) { s_q[i] = y0; s_q[i + half] = y1; }
                        else {
                            s_kn[i] = kv_round<T>(y0); s_kn[i + half] = kv_round<T>(y1);
                            if (ok) { st_kv(kv_pool + kv_off + i, y0); st_kv(kv_pool + kv_off + i + half, y1); }
                        }
                    }
                }
            }
        }
        __syncthreads();
        float q[DPL], o[DPL], m_run = NEG, l_run = 0.f;
#pragma unroll
        for (int d = 0; d < DPL; ++d) { q[d] = s_q[lane * DPL + d]; o[d] = 0.f; }
        for (; c < c1; c += TK_NW) {
            if (c == c_new) {
                KvRow<T, DPL> nk, nv;
                nk.from_float(s_kn + lane * DPL); nv.from_float(s_vn + lane * DPL);
                const int jn = (int)((uint32_t)p % CP);
#pragma unroll
                for (int j = 0; j < CP; ++j) if (j == jn) { kr[j] = nk; vr[j] = nv; }
            }
            float sc[CP];
#pragma unroll
            for (int j = 0; j < CP; ++j) {
                float kf[DPL];
                kr[j].to_float(kf);
                if constexpr (DPL >= 2) {
                    float a0 = 0.f, a1 = 0.f;
#pragma unroll
                    for (int d = 0; d < DPL; d += 2) fma2(a0, a1, q[d], q[d + 1], kf[d], kf[d + 1]);
                    sc[j] = a0 + a1;
                } else sc[j] = q[0] * kf[0];
            }
            const uint32_t c_next = c + TK_NW;
            if (c_next < c1) load_rows(c_next, 0, kr);
            warp_reduce_scatter<CP>(sc, lane);                   // lane l holds the score of position l / 4
            const uint32_t tp = c * CP + lane / 4;
            const bool valid = tp >= sp.start && tp < seq;
            float sv = sc[0] * a.attn_scale;
            if (a.attn_cap > 0.f) sv = tanhf(sv / a.attn_cap) * a.attn_cap;
            sv = valid ? sv : NEG;
            float cmx = sv;
            cmx = fmaxf(cmx, __shfl_xor_sync(0xffffffffu, cmx, 4));
            cmx = fmaxf(cmx, __shfl_xor_sync(0xffffffffu, cmx, 8));
            cmx = fmaxf(cmx, __shfl_xor_sync(0xffffffffu, cmx, 16));
            const float m_new = fmaxf(m_run, cmx);
            const float alpha = expf(m_run - m_new);
            const float pz = valid ? expf(sv - m_new) : 0.f;
            float ps = pz;
            ps += __shfl_xor_sync(0xffffffffu, ps, 4);
            ps += __shfl_xor_sync(0xffffffffu, ps, 8);
            ps += __shfl_xor_sync(0xffffffffu, ps, 16);
            l_run = fmaf(l_run, alpha, ps);
            m_run = m_new;
#pragma unroll
            for (int d = 0; d < DPL; ++d) o[d] *= alpha;
#pragma unroll
            for (int j = 0; j < CP; ++j) {
                float vf[DPL];
                vr[j].to_float(vf);
                const float pv = __shfl_sync(0xffffffffu, pz, j * 4);
                if constexpr (DPL >= 2) {
#pragma unroll
                    for (int d = 0; d < DPL; d += 2) fma2(o[d], o[d + 1], pv, pv, vf[d], vf[d + 1]);
                } else o[0] = fmaf(pv, vf[0], o[0]);
            }
            if (c_next < c1) load_rows(c_next, 1, vr);
        }
        // merge the warps
#pragma unroll
        for (int d = 0; d < DPL; ++d) s_o[warp * HD + lane * DPL + d] = o[d];
        if (lane == 0) { s_m[warp] = m_run; s_l[warp] = l_run; }
        __syncthreads();
        float M = NEG;
#pragma unroll
        for (int w2 = 0; w2 < TK_NW; ++w2) M = fmaxf(M, s_m[w2]);
        if (tid < TK_NW) s_w[tid] = expf(s_m[tid] - M);
        __syncthreads();
        uint2* dst = att + ((size_t)head * a.s_max + split) * (HD + 2);
        if (tid < HD) {
            float v = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < TK_NW; ++w2) v = fmaf(s_w[w2], s_o[w2 * HD + tid], v);
            st_pkt(dst + tid, v, tag);
        } else if (tid == HD) {
            float Ls = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < TK_NW; ++w2) Ls = fmaf(s_w[w2], s_l[w2], Ls);
            st_pkt(dst + HD, M, tag);
            st_pkt(dst + HD + 1, Ls, tag);
        }
        __syncthreads();                                         // the staging area is reused right after
    };

    // Attention output of all heads (merged over the splits) staged as the o-proj input.
    auto stage_attention = [&](const TkLayer& ly, const uint2* att, uint32_t tag) {
        const TkAttnSplit sp = tk_attn_split(a.s_max, ly.window, p);
        const int H = a.H, S = (int)sp.n_act;
        for (int i = tid; i < H * S; i += TK_THREADS) {
            const int hh = i / S, s = i % S;
            const uint2* b = att + ((size_t)hh * a.s_max + s) * (HD + 2) + HD;
            const uint2* ptr[2] = {b, b + 1};
            float val[2];
            poll_pkts<2>(ptr, tag, val, wt);
            s_ml[(hh * a.s_max + s) * 2] = val[0]; s_ml[(hh * a.s_max + s) * 2 + 1] = val[1];
        }
        __syncthreads();
        const int n4 = a.q_dim >> 2;
        float4 x[2];
        float am = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = tid + j * TK_THREADS;
            x[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (i < n4) {
                const int hh = (4 * i) / HD, e0 = (4 * i) % HD;
                float M = NEG;
                for (int s = 0; s < S; ++s) M = fmaxf(M, s_ml[(hh * a.s_max + s) * 2]);
                float den = 0.f;
                float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int s = 0; s < S; ++s) {
                    const float wgt = expf(s_ml[(hh * a.s_max + s) * 2] - M);
                    const uint2* b = att + ((size_t)hh * a.s_max + s) * (HD + 2) + e0;
                    const uint2* ptr[4] = {b, b + 1, b + 2, b + 3};
                    float val[4];
                    poll_pkts<4>(ptr, tag, val, wt);
                    num.x = fmaf(wgt, val[0], num.x); num.y = fmaf(wgt, val[1], num.y);
                    num.z = fmaf(wgt, val[2], num.z); num.w = fmaf(wgt, val[3], num.w);
                    den = fmaf(wgt, s_ml[(hh * a.s_max + s) * 2 + 1], den);
                }
                x[j] = make_float4(num.x / den, num.y / den, num.z / den, num.w / den);
                am = fmaxf(am, fmaxf(fmaxf(fabsf(x[j].x), fabsf(x[j].y)), fmaxf(fabsf(x[j].z), fabsf(x[j].w))));
            }
        }
        am = block_max(am, red);
        float s, inv;
        pow2_scale(am, s, inv);
        if (tid == 0) s_inv = inv;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = tid + j * TK_THREADS;
            if (i < n4) put_x4<NCOL>(xb, 4 * i, 0, make_float4(x[j].x * s, x[j].y * s, x[j].z * s, x[j].w * s));
        }
        finish_staging(a.q_dim / 32);
    };

    auto cta_in = [&](int ph) { const TkPhase& P = a.ph[ph]; return P.n_rg > 0 && bx < P.G * P.cpr; };

    // ---- the token ----
    const int qkv_ld = a.q_dim + 2 * a.k_dim;
    const size_t att_half = (size_t)a.H * a.s_max * (HD + 2);
    bool bail = false;
    for (int L = 0; L < a.n_layer && !bail; ++L) {
        const TkLayer ly = a.layers[L];
        const int par = L & 1;
        const uint32_t tag = tag_base + (uint32_t)L + 1u;
        uint2* b_qkv = a.x_qkv + (size_t)par * qkv_ld;
        uint2* b_att = a.x_att + (size_t)par * att_half;
        uint2* b_po = a.x_po + (size_t)par * a.ph[TK_O].cpr * E;
        uint2* b_act = a.x_act + (size_t)par * a.FF;
        uint2* b_pd = a.x_pd + (size_t)par * a.ph[TK_DOWN].cpr * E;
        const uint2* prev_pd = a.x_pd + (size_t)(par ^ 1) * a.ph[TK_DOWN].cpr * E;
        // QKV: previous layer's FFN output joins the stream, input norm
        chain(L > 0 ? prev_pd : nullptr, a.ph[TK_DOWN].cpr, tag - 1u, L > 0 ? a.layers[L - 1].norm[TKN_POST_FFW] : nullptr,
              ly.norm[TKN_ATTN], cta_in(TK_QKV));
        if (__syncthreads_or(wt.failed ? 1 : 0)) { bail = true; break; }
        if (cta_in(TK_QKV)) product(TK_QKV, 0, b_qkv, tag);
        __syncthreads();
        attention(ly, L, b_qkv, b_att, tag);
        if (cta_in(TK_O)) {
            stage_attention(ly, b_att, tag);
            if (__syncthreads_or(wt.failed ? 1 : 0)) { bail = true; break; }
            product(TK_O, 0, b_po, tag);
            __syncthreads();
        }
        // gate/up: attention output joins the stream, FFN norm
        chain(b_po, a.ph[TK_O].cpr, tag, ly.norm[TKN_POST_ATTN], ly.norm[TKN_FFN], cta_in(TK_GU));
        if (__syncthreads_or(wt.failed ? 1 : 0)) { bail = true; break; }
        if (cta_in(TK_GU)) product(TK_GU, 1, b_act, tag);
        __syncthreads();
        if (cta_in(TK_DOWN)) {
            const TkPhase& P = a.ph[TK_DOWN];
            const int kpart = bx % P.cpr;
            const int pp0 = (int)((long long)(kpart * P.KS) * P.pairs / (P.cpr * P.KS));
            const int pp1 = (int)((long long)((kpart + 1) * P.KS) * P.pairs / (P.cpr * P.KS));
            stage_packets(b_act + (size_t)pp0 * 64, (pp1 - pp0) * 64, tag);
            if (__syncthreads_or(wt.failed ? 1 : 0)) { bail = true; break; }
            product(TK_DOWN, 0, b_pd, tag);
            __syncthreads();
        }
    }
    if (!bail) {
        // last layer's FFN output joins the stream; final norm in front of the LM head
        const int lastp = (a.n_layer - 1) & 1;
        const uint32_t tag = tag_base + (uint32_t)a.n_layer;
        const bool lm = a.with_lm && cta_in(TK_LM);
        chain(a.x_pd + (size_t)lastp * a.ph[TK_DOWN].cpr * E, a.ph[TK_DOWN].cpr, tag, a.layers[a.n_layer - 1].norm[TKN_POST_FFW], a.out_norm, lm);
        if (__syncthreads_or(wt.failed ? 1 : 0)) bail = true;
        if (!bail && bx == 0 && a.h_out) {
            for (int i = tid; i < E; i += TK_THREADS) a.h_out[i] = s_h[i];
        }
        if (!bail && lm) {
            product(TK_LM, 2, nullptr, tag);
            // lanes -> warp -> CTA -> packet
#pragma unroll
            for (int o = 4; o < 32; o <<= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
                const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (better(ov, oi, best_v, best_i)) { best_v = ov; best_i = oi; }
            }
            if (lane == 0) { s_bv[warp] = best_v; s_bi[warp] = best_i; }
            __syncthreads();
            if (tid == 0) {
                float bv = s_bv[0]; int bi = s_bi[0];
                for (int w2 = 1; w2 < TK_NW; ++w2) if (better(s_bv[w2], s_bi[w2], bv, bi)) { bv = s_bv[w2]; bi = s_bi[w2]; }
                if (!timed_out && !wt.failed) {
                    st_pkt(a.x_amax + 2 * bx, bv, tag);
                    st_pkt(a.x_amax + 2 * bx + 1, __int_as_float(bi), tag);
                }
            }
        }
        if (__syncthreads_or((wt.failed || timed_out) ? 1 : 0)) bail = true;
        // CTA 0 closes the step: global arg-max, token log, position and step counter
        if (!bail && bx == 0) {
            if (a.with_lm) {
                const int n_cta = a.ph[TK_LM].G * a.ph[TK_LM].cpr;
                float bv = -3.402823466e+38f; int bi = -1;
                for (int i = tid; i < n_cta; i += TK_THREADS) {
                    const uint2* ptr[2] = {a.x_amax + 2 * i, a.x_amax + 2 * i + 1};
                    float val[2];
                    poll_pkts<2>(ptr, tag, val, wt);
                    const int k = __float_as_int(val[1]);
                    if (better(val[0], k, bv, bi)) { bv = val[0]; bi = k; }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
                }
                __syncthreads();
                if (lane == 0) { s_bv[warp] = bv; s_bi[warp] = bi; }
                if (__syncthreads_or(wt.failed ? 1 : 0)) bail = true;
                if (!bail && tid == 0) {
                    for (int w2 = 1; w2 < TK_NW; ++w2) if (better(s_bv[w2], s_bi[w2], bv, bi)) { bv = s_bv[w2]; bi = s_bi[w2]; }
                    const int ntok = bi < 0 ? 0 : bi;
                    a.cur_tok[0] = ntok;
                    a.cur_val[0] = bv;
                    if ((uint32_t)(p + 1) < a.log_ld) a.gen_log[p + 1] = ntok;
                }
            }
            if (!bail && tid == 0) { a.pos[0] = p + 1; *a.seq = seq_no + 1u; }
        }
    }
    if (bail) {
        if (tid == 0) { atomicOr(a.err, DEVERR_WAIT); atomicExch(a.dead, 1u); }
    }
    // Copies still in flight must land before the CTA's shared memory is released.
    {
        int outstanding = __shfl_sync(0xffffffffu, issued - consumed, 0);
        const long long drain_deadline = clock64() + TK_WAIT_CYCLES / 4;
        while (outstanding > 0) {
            tk_mbar_wait(&s_bar[warp][c_st], c_ph, drain_deadline);
            if (++c_st == NSTAGE) { c_st = 0; c_ph ^= 1u; }
            --outstanding;
        }
    }
}

}  // namespace ab
