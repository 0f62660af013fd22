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
// Every CTA polls the same few kilobytes: without a pause between unsuccessful rounds the polls alone saturate
// the L2 slices that hold them and delay the very stores they wait for.
constexpr unsigned TK_POLL_SLEEP_NS = 100;

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
    uint32_t rounds;                                                // unsuccessful poll rounds so far (diagnostics)
    __device__ __forceinline__ bool give_up(uint32_t& spins) {      // call once per unsuccessful poll round
        ++rounds;
        if ((++spins & 63u) == 0u) {
            if (clock64() > deadline || *reinterpret_cast<const volatile uint32_t*>(dead) != 0u) { failed = true; return true; }
        }
        return false;
    }
};

// Poll packets p0[k * stride] and (when p1 is not NULL) p1[k * stride], k < n <= N, with all loads in
// flight together, until every tag matches.  Entries k >= n come back as 0.  No arrays of pointers:
// everything stays in registers.
template <int N>
__device__ __forceinline__ void poll2(const uint2* p0, const uint2* p1, int stride, int n, uint32_t tag,
                                      float (&o0)[N], float (&o1)[N], TkWait& wt) {
#pragma unroll
    for (int i = 0; i < N; ++i) { o0[i] = 0.f; o1[i] = 0.f; }
    if (wt.failed || n <= 0) return;
    uint32_t spins = 0;
    while (true) {
        uint2 v0[N], v1[N];
#pragma unroll
        for (int i = 0; i < N; ++i) {
            v0[i] = i < n ? ld_pkt(p0 + (size_t)i * stride) : make_uint2(0u, tag);
            v1[i] = (p1 && i < n) ? ld_pkt(p1 + (size_t)i * stride) : make_uint2(0u, tag);
        }
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; ++i) ok = ok && (v0[i].y == tag) && (v1[i].y == tag);
        if (ok) {
#pragma unroll
            for (int i = 0; i < N; ++i) { o0[i] = __uint_as_float(v0[i].x); o1[i] = __uint_as_float(v1[i].x); }
            return;
        }
        if (wt.give_up(spins)) return;
        __nanosleep(TK_POLL_SLEEP_NS);
    }
}

// Poll the N packets addr(0..N-1) (NULL = skip, reads as 0) with all loads in flight together.
template <int N, class F>
__device__ __forceinline__ void poll_fn(F addr, uint32_t tag, float (&out)[N], TkWait& wt) {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = 0.f;
    if (wt.failed) return;
    uint32_t spins = 0;
    while (true) {
        uint2 v[N];
#pragma unroll
        for (int i = 0; i < N; ++i) { const uint2* q = addr(i); v[i] = q ? ld_pkt(q) : make_uint2(0u, tag); }
        bool ok = true;
#pragma unroll
        for (int i = 0; i < N; ++i) ok = ok && (v[i].y == tag);
        if (ok) {
#pragma unroll
            for (int i = 0; i < N; ++i) out[i] = __uint_as_float(v[i].x);
            return;
        }
        if (wt.give_up(spins)) return;
        __nanosleep(TK_POLL_SLEEP_NS);
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
struct TkCursor { const uint8_t* t0; const uint8_t* t1; int L, ph, chp, np, p0, pairs, n_rg, rg_step, rg_next, sets_left; };

// Attention work split of one layer at position p (the same on the producing and the consuming side).
struct TkAttnSplit { uint32_t start, c_first, n_chunks, n_act; };
__device__ __forceinline__ TkAttnSplit tk_attn_split(int s_max, uint32_t window, int p, int cp) {
    TkAttnSplit s;
    const uint32_t seq = (uint32_t)p + 1;
    s.start = (window > 0 && seq > window) ? seq - window : 0;
    s.c_first = s.start / cp;
    s.n_chunks = (seq - 1) / cp - s.c_first + 1;
    // one chunk per warp while CTAs are left: every row a warp needs is then requested before its query arrives
    s.n_act = min((uint32_t)s_max, (s.n_chunks + TK_NW - 1) / TK_NW);
    return s;
}
// Positions per chunk: as many rows in flight per warp as the registers hold (K and V rows of a chunk
// are all requested before any is used).
template <typename T, int HD> struct TkAttn { static constexpr int CP = (HD / 32) * (int)sizeof(T) > 8 ? 4 : 8; };

template <int WT> struct TkGeo {
    static constexpr int TILE = mma_tile_bytes(WT);
    // tile slots per stage: a product over two matrices puts CH / 2 tile pairs of each into a stage.  Few large
    // stages rather than many small ones: every chunk costs a wait, a refill and loop overhead on the warp's
    // critical path, and two stages of 5 KB per warp already keep ~150 KB in flight per SM.
    static constexpr int CH = WT == WT_Q4_0 ? 9 : 8;
    static constexpr int NSTAGE = 2;
    static constexpr int STAGE_BYTES = CH * TILE;
    static constexpr int RING_BYTES = NSTAGE * STAGE_BYTES; // per warp
};

// Shared-memory layout (dynamic part), computed identically on the host (token.cu).
struct TkSmemLayout { size_t xb, sx, xbw, h, lay, work, ring, total; };
__host__ __device__ inline TkSmemLayout tk_smem_layout(int units_max, int hd, int wu_cap, int E, int n_layer, int ring_bytes_per_warp) {
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
    l.xbw = o; o += (size_t)TK_NW * wu_cap * 136; o = (o + 15) & ~(size_t)15;      // per warp: [wu_cap][4][32] staged bytes + [wu_cap][2] sums
    l.h = o; o += (size_t)E * 4; o = (o + 15) & ~(size_t)15;
    l.lay = o; o += (size_t)n_layer * sizeof(TkLayer); o = (o + 15) & ~(size_t)15;      // the layer table, copied once per launch
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
    __shared__ TkCursor s_cur[TK_NW];
    __shared__ float s_bv[TK_NW];
    __shared__ int s_bi[TK_NW];

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int bx = blockIdx.x;
    const int E = a.E;

    const TkSmemLayout lay = tk_smem_layout(E / 32, HD, a.wu_cap, E, a.n_layer, G::RING_BYTES);
    signed char* xb = reinterpret_cast<signed char*>(smem_raw + lay.xb);
    float* s_sx = reinterpret_cast<float*>(smem_raw + lay.sx);
    signed char* xbw = reinterpret_cast<signed char*>(smem_raw + lay.xbw) + (size_t)warp * a.wu_cap * 136;   // this warp's own staging region
    float* s_h = reinterpret_cast<float*>(smem_raw + lay.h);
    TkLayer* s_lay = reinterpret_cast<TkLayer*>(smem_raw + lay.lay);
    TkWork* s_work = reinterpret_cast<TkWork*>(smem_raw + lay.work);
    unsigned char* ring = smem_raw + lay.ring + (size_t)warp * G::RING_BYTES;

    TkWait wt;
    wt.deadline = clock64() + (a.wait_cycles > 0 ? a.wait_cycles : TK_WAIT_CYCLES);
    wt.dead = a.dead;
    wt.failed = false;
    wt.rounds = 0;
    if (*reinterpret_cast<const volatile uint32_t*>(a.dead) != 0u) return;      // an earlier step gave up: do nothing

    // ---- set-up: weight pointer table, per-warp work of every phase, barriers ----
    {   // 8-byte words of the layer table
        const unsigned long long* src = reinterpret_cast<const unsigned long long*>(a.layers);
        unsigned long long* dst = reinterpret_cast<unsigned long long*>(s_lay);
        for (int i = tid; i < (int)(a.n_layer * sizeof(TkLayer) / 8); i += TK_THREADS) dst[i] = src[i];
    }
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
    // Issue cursor (lane 0).  What changes per chunk lives in registers (offset into the matrix, tile pairs
    // left in this set's K slice, stage); what changes per phase lives in the warp's TkCursor in shared memory.
    TkCursor* cur = s_cur + warp;
    size_t i_off = 0;
    int i_rem = 0, i_st = 0, issued = 0, consumed = 0;
    bool i_done = false;
    auto next_phase = [&]() {                                // lane 0: advance to the next phase with work for this warp
        int L = cur->L, ph = cur->ph;
        while (true) {
            if (ph == TK_LM) { i_done = true; return; }
            if (ph == TK_DOWN || ph < 0) {
                if (ph == TK_DOWN) ++L;
                ph = (L < a.n_layer) ? (int)TK_QKV : (int)TK_LM;
            } else ++ph;
            if (s_work[warp * TK_PHASES + ph].active) break;
        }
        const TkWork w = s_work[warp * TK_PHASES + ph];
        const TkPhase& P = a.ph[ph];
        cur->L = L; cur->ph = ph;
        cur->t0 = ph == TK_LM ? a.lm_tiled : s_lay[L].w[ph == TK_QKV ? 0 : ph == TK_O ? 1 : ph == TK_GU ? 2 : 4];
        cur->t1 = ph == TK_GU ? s_lay[L].w[3] : nullptr;
        cur->chp = ph == TK_GU ? CH / 2 : CH;
        cur->np = w.np; cur->p0 = w.p0; cur->pairs = P.pairs; cur->n_rg = P.n_rg;
        cur->rg_step = P.G * P.RG;
        const int rg0 = w.sb * P.RG + w.rg_l;
        cur->rg_next = rg0 + cur->rg_step;
        cur->sets_left = w.n_sets;
        i_off = ((size_t)min(rg0, P.n_rg - 1) * P.pairs + w.p0) * TILE;
        i_rem = w.np;
    };
    auto issue_next = [&]() {                                // lane 0, !i_done
        const int n = min(cur->chp, i_rem);
        const uint8_t* t1 = cur->t1;
        unsigned char* dst = ring + (size_t)i_st * STAGE_BYTES;
        mbar_expect_tx(&s_bar[warp][i_st], (uint32_t)(n * TILE * (t1 ? 2 : 1)));
        bulk_g2s(dst, cur->t0 + i_off, (uint32_t)(n * TILE), &s_bar[warp][i_st]);
        if (t1) bulk_g2s(dst + (CH / 2) * TILE, t1 + i_off, (uint32_t)(n * TILE), &s_bar[warp][i_st]);
        ++issued;
        if (++i_st == NSTAGE) i_st = 0;
        i_rem -= n;
        i_off += (size_t)n * TILE;
        if (i_rem == 0) {
            const int left = cur->sets_left - 1;
            if (left == 0) next_phase();
            else {
                cur->sets_left = left;
                const int rg = cur->rg_next;
                cur->rg_next = rg + cur->rg_step;
                i_off = ((size_t)min(rg, cur->n_rg - 1) * cur->pairs + cur->p0) * TILE;
                i_rem = cur->np;
            }
        }
    };
    if (lane == 0) {
        cur->L = 0; cur->ph = -1;
        next_phase();
#pragma unroll 1
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
    // (loops over the vectors are kept rolled on purpose: this code runs once per layer and has to stay in
    // the instruction cache)
    // per-unit sums of the staged integer activations, in the units of the lane that uses them
    auto finish_staging = [&](int units) {
        __syncthreads();
#pragma unroll 1
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

    // Incoming vectors are first gathered into s_a, a float image that shares its bytes with the staging
    // area xb (4 bytes per value in both; the 32 values of a unit and its 128 staged bytes coincide).
    float* s_a = reinterpret_cast<float*>(xb);
    // s_a[i] = w * (P(i) + P1(i)), or += with `acc`; P(i) = buf[(i >> rshift) * rstride + (i & ((1 << rshift) - 1))]
    // (rshift >= 31: one row), P1 likewise from buf1 (NULL = none), w = wtab[i >> rshift] (NULL = 1).
    // Consecutive threads poll consecutive packets (a warp reads 256 contiguous bytes per load), up to 16 loads
    // in flight per thread.  Ends with a CTA barrier.
    auto gather = [&](const uint2* buf, const uint2* buf1, int rshift, size_t rstride, int n, uint32_t tag, const float* wtab, bool acc) {
        const bool rows = rshift < 31;
        const int stride = rows ? (int)((TK_THREADS >> rshift) * rstride) : TK_THREADS;
#pragma unroll 1
        for (int base = 0; base < n; base += 8 * TK_THREADS) {
            const int i0 = base + tid;
            const int cnt = i0 < n ? min(8, (n - i0 + TK_THREADS - 1) / TK_THREADS) : 0;
            const size_t off = rows ? (size_t)(i0 >> rshift) * rstride + (size_t)(i0 & ((1 << rshift) - 1)) : (size_t)i0;
            float v0[8], v1[8];
            poll2<8>(buf + off, buf1 ? buf1 + off : nullptr, stride, cnt, tag, v0, v1, wt);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (k < cnt) {
                    const int i = i0 + k * TK_THREADS;
                    float v = v0[k] + v1[k];
                    if (wtab) v *= wtab[i >> rshift];
                    s_a[i] = acc ? s_a[i] + v : v;
                }
            }
        }
        __syncthreads();
    };

    // Residual update + norm in front of a product (the reference's map_rmsnorm_add + map_rmsnorm pair,
    // engine.py:3259, :3267):  h += rms(sum of `parts` partial vectors) * w_post (plain add without w_post);
    // x = rms(h) * w_pre; x is staged for the MMAs when `stage`.
    auto chain = [&](const uint2* add_buf, int parts, uint32_t tag, const float* w_post, const float* w_pre, bool stage) {
        const int n4 = E >> 2;
        float rms_a = 1.f;
        // the norm weights of this thread's first elements are requested ahead of the poll (one trip through L2 each)
        const float4 one4 = make_float4(1.f, 1.f, 1.f, 1.f);
        const float4 wp_first = (w_post && add_buf && tid < n4) ? reinterpret_cast<const float4*>(w_post)[tid] : one4;
        const float4 vw_first = (w_pre && stage && tid < n4) ? reinterpret_cast<const float4*>(w_pre)[tid] : one4;
        if (add_buf) {
            gather(add_buf, parts > 1 ? add_buf + E : nullptr, 31, 0, E, tag, nullptr, false);
            if (w_post) {
                float ss = 0.f;
#pragma unroll 1
                for (int i = tid; i < n4; i += TK_THREADS) {
                    const float4 va = reinterpret_cast<const float4*>(s_a)[i];
                    ss = fmaf(va.x, va.x, ss); ss = fmaf(va.y, va.y, ss); ss = fmaf(va.z, va.z, ss); ss = fmaf(va.w, va.w, ss);
                }
                ss = block_sum(ss, red);
                rms_a = sqrtf(ss / (float)E + a.eps);
            }
        }
        const float rcp_a = __frcp_rn(rms_a);
        float ss = 0.f, am = 0.f;
#pragma unroll 1
        for (int i = tid; i < n4; i += TK_THREADS) {
            float4 vh = reinterpret_cast<const float4*>(s_h)[i];
            if (add_buf) {
                const float4 va = reinterpret_cast<const float4*>(s_a)[i];
                if (w_post) {
                    const float4 wp = i == tid ? wp_first : reinterpret_cast<const float4*>(w_post)[i];
                    vh.x += div_by(va.x, rms_a, rcp_a) * wp.x; vh.y += div_by(va.y, rms_a, rcp_a) * wp.y;
                    vh.z += div_by(va.z, rms_a, rcp_a) * wp.z; vh.w += div_by(va.w, rms_a, rcp_a) * wp.w;
                } else { vh.x += va.x; vh.y += va.y; vh.z += va.z; vh.w += va.w; }
                reinterpret_cast<float4*>(s_h)[i] = vh;
            }
            if (stage) {
                const float4 vw = i == tid ? vw_first : (w_pre ? reinterpret_cast<const float4*>(w_pre)[i] : one4);
                ss = fmaf(vh.x, vh.x, ss); ss = fmaf(vh.y, vh.y, ss); ss = fmaf(vh.z, vh.z, ss); ss = fmaf(vh.w, vh.w, ss);
                am = fmaxf(am, fmaxf(fmaxf(fabsf(vh.x * vw.x), fabsf(vh.y * vw.y)), fmaxf(fabsf(vh.z * vw.z), fabsf(vh.w * vw.w))));
            }
        }
        if (!stage) { __syncthreads(); return; }             // s_a may be rewritten by the next gather
        block_sum_max(ss, am, red);                           // its barriers also end every read of s_a
        float rms = 1.f, rcp = 1.f;
        if (w_pre) {
            rms = sqrtf(ss / (float)E + a.eps);
            rcp = __frcp_rn(rms);
            am = am * rcp * 1.000001f;
        }
        float s, inv;
        pow2_scale(am, s, inv);
        if (tid == 0) s_inv = inv;
#pragma unroll 1
        for (int i = tid; i < n4; i += TK_THREADS) {
            float4 vh = reinterpret_cast<const float4*>(s_h)[i];
            if (w_pre) {
                const float4 vw = i == tid ? vw_first : reinterpret_cast<const float4*>(w_pre)[i];
                vh.x = div_by(vh.x, rms, rcp) * vw.x; vh.y = div_by(vh.y, rms, rcp) * vw.y;
                vh.z = div_by(vh.z, rms, rcp) * vw.z; vh.w = div_by(vh.w, rms, rcp) * vw.w;
            }
            put_x4<NCOL>(xb, 4 * i, 0, make_float4(vh.x * s, vh.y * s, vh.z * s, vh.w * s));
        }
        finish_staging(E / 32);
    };

    // One 16x32 block of one matrix against the staged columns (see gemv_mma.cuh).
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

    int cur_L = 0;
    auto mark = [&](int L, int slot) {
        if (a.trace && tid == 0 && (L == a.trace_layer || L < 0)) a.trace[(size_t)bx * TK_TRACE_SLOTS + slot] = clock64();
    };
    auto fmark = [&](int ph, int slot) { if (a.trace && tid == 0 && cur_L == a.trace_layer && ph == a.trace_phase) a.trace[(size_t)bx * TK_TRACE_SLOTS + slot] = clock64(); };
    float best_v = -3.402823466e+38f; int best_i = -1;      // LM-head candidates of this lane

    // The product of phase ph for this warp.  mode 0: packets out[kpart * N + row]; 1: GeGLU / SwiGLU of the
    // two matrices; 2: LM head (arg-max candidates, optional soft-capped logits).
    auto product = [&](int ph, int mode, uint2* out, uint32_t tag, const uint2* in_buf, uint32_t window) {
        const TkWork w = s_work[warp * TK_PHASES + ph];
        if (!w.active) return;
        const TkPhase& P = a.ph[ph];
        const bool pr = (ph == TK_GU);
        const int chp = pr ? CH / 2 : CH;
        const int N = P.n_rg * 16;
        float inv = s_inv;
        int part_p0 = w.part_p0;
        const uint2* xq = reinterpret_cast<const uint2*>(xb) + (g % NCOL) * 4 + t;
        const float* sxp = s_sx + (t % NPR);
        fmark(ph, 15);
        const uint32_t rounds0 = wt.rounds;
        if (ph == TK_O || ph == TK_DOWN) {
            // The input of these products needs no norm over the whole vector, so every warp stages just its
            // own K slice (<= wu_cap units) in its own region, with its own scale and without any CTA barrier:
            // poll the slice's packets, merge the attention splits (o-proj), warp maximum, pack in place.
            float* saw = reinterpret_cast<float*>(xbw);
            float* sxw = reinterpret_cast<float*>(xbw + (size_t)a.wu_cap * 128);
            const int ng = w.np * 16;                        // float4 groups of the slice
            float am = 0.f;
            // (lane l polls packets l, l + 32, ...: a warp-wide load then reads 256 contiguous bytes; a lane
            // that read four neighbouring packets instead would cost four times the sectors, and the SM's
            // request rate towards L2, not L2 itself, is what bounds these polls)
            const int nv = w.np * 64;                        // values of the slice
            if (ph == TK_DOWN) {
                const uint2* src = in_buf + (size_t)w.p0 * 64;
                float val[16];
                poll_fn<16>([&](int i) -> const uint2* { const int idx = lane + 32 * i; return idx < nv ? src + idx : nullptr; }, tag, val, wt);
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    const int idx = lane + 32 * k;
                    if (idx < nv) { saw[idx] = val[k]; am = fmaxf(am, fabsf(val[k])); }
                }
            } else {
                constexpr int HSH = HD == 32 ? 5 : HD == 64 ? 6 : HD == 128 ? 7 : 8;
                const int S = (int)tk_attn_split(a.s_max, window, p, TkAttn<T, HD>::CP).n_act;      // <= 4
#pragma unroll 1
                for (int q = 0; q < w.np; ++q) {              // one tile pair = 64 values = two per lane
                    const int i0 = (w.p0 + q) * 64 + lane;
                    float val[24];                           // per split: value k = 0, 1; maximum k = 0, 1; denominator k = 0, 1
                    poll_fn<24>([&](int i) -> const uint2* {
                        const int sidx = i / 6, r = i % 6, k = r & 1;
                        if (sidx >= S) return nullptr;
                        const int ii = i0 + 32 * k;
                        const uint2* b = in_buf + ((size_t)sidx * a.H + (ii >> HSH)) * (HD + 2);
                        return r < 2 ? b + (ii & (HD - 1)) : b + HD + (r >> 1) - 1;
                    }, tag, val, wt);
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        float M = NEG;
#pragma unroll
                        for (int s2 = 0; s2 < 4; ++s2) if (s2 < S) M = fmaxf(M, val[6 * s2 + 2 + k]);
                        float den = 0.f, num = 0.f;
#pragma unroll
                        for (int s2 = 0; s2 < 4; ++s2) {
                            if (s2 < S) {
                                const float wgt = expf(val[6 * s2 + 2 + k] - M);
                                num = fmaf(wgt, val[6 * s2 + k], num);
                                den = fmaf(wgt, val[6 * s2 + 4 + k], den);
                            }
                        }
                        const float x = num / den;
                        saw[q * 64 + lane + 32 * k] = x;
                        am = fmaxf(am, fabsf(x));
                    }
                }
            }
            __syncwarp();
            am = warp_max(am);
            float sc;
            pow2_scale(am, sc, inv);
#pragma unroll 1
            for (int j = 0; j * 32 < ng; ++j) {
                const int g4 = lane + 32 * j;
                const float4 v = g4 < ng ? reinterpret_cast<const float4*>(saw)[g4] : make_float4(0.f, 0.f, 0.f, 0.f);
                __syncwarp();
                if (g4 < ng) put_x4<NCOL>(xbw, 4 * g4, 0, make_float4(v.x * sc, v.y * sc, v.z * sc, v.w * sc));
            }
            __syncwarp();
            for (int i = lane; i < w.np * 2 * NPR; i += 32) {
                const int u = i / NPR, prr = i % NPR;
                const int* c0 = reinterpret_cast<const int*>(xbw + (size_t)(u * NCOL + 2 * prr) * 32);
                const int* c1 = c0 + 8;
                int s0 = 0, s1 = 0;
#pragma unroll
                for (int e = 0; e < 8; ++e) { s0 = __dp4a(c0[e], 0x01010101, s0); s1 = __dp4a(c1[e], 0x01010101, s1); }
                sxw[i] = SXF * (float)(s0 * 256 + s1);
            }
            __syncwarp();
            xq = reinterpret_cast<const uint2*>(xbw) + (g % NCOL) * 4 + t;
            sxp = sxw + (t % NPR);
            part_p0 = w.p0;
        }
        int parity = 0, pend = 0;                           // pend: refills put off until the set's results are out
        fmark(ph, 16);
        if (a.trace && tid == 0 && cur_L == a.trace_layer && ph == a.trace_phase) a.trace[(size_t)bx * TK_TRACE_SLOTS + 23] = (long long)(wt.rounds - rounds0);
        for (int si = 0; si < w.n_sets; ++si) {
            const int rg = (w.sb + si * P.G) * P.RG + w.rg_l;
            float acc0[2] = {0.f, 0.f}, acc1[2] = {0.f, 0.f};
            for (int j = 0; j < w.nch; ++j) {
                if (!timed_out) {
                    const bool ok = tk_mbar_wait(&s_bar[warp][c_st], c_ph, wt.deadline);
                    if (!__all_sync(0xffffffffu, ok)) { timed_out = true; wt.failed = true; }
                }
                if (si == 0 && j == 0) fmark(ph, 17);
                if (!timed_out) {
                    const unsigned char* buf = ring + (size_t)c_st * STAGE_BYTES;
                    const int pp0 = w.p0 + j * chp, n = min(chp, w.p0 + w.np - pp0);
                    const uint2* xp = xq + (size_t)(pp0 - part_p0) * 2 * xstep;
                    const float* sx = sxp + (size_t)(pp0 - part_p0) * 2 * NPR;
#pragma unroll 2
                    for (int k = 0; k < n; ++k) {
                        do_tile(buf + k * TILE, xp + (2 * k) * xstep, sx + (2 * k) * NPR, acc0);
                        if (pr) do_tile(buf + (chp + k) * TILE, xp + (2 * k) * xstep, sx + (2 * k) * NPR, acc1);
                    }
                    __syncwarp();
                    if (si == 0 && j == 0) fmark(ph, 18);
                    if (lane == 0) { ++consumed; if (!i_done) { if (j + 1 < w.nch || P.KS == 1) issue_next(); else ++pend; } }
                    if (si == 0 && j == 0) fmark(ph, 19);
                }
                if (++c_st == NSTAGE) { c_st = 0; c_ph ^= 1u; }
            }
            if (si == 0) fmark(ph, 20);
            // even lanes: 256 * acc + (odd neighbour's acc) / 256
            float val0[2], val1[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v = acc0[h] * cm;
                val0[h] = (v + __shfl_xor_sync(0xffffffffu, v, 1)) * inv;      // inv is a power of two: exact
                v = acc1[h] * cm;
                val1[h] = (v + __shfl_xor_sync(0xffffffffu, v, 1)) * inv;
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
            if (si == 0) fmark(ph, 21);
            if (writer && t == 0 && rg < P.n_rg && !timed_out) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int row = rg * 16 + g + 8 * h;
                    const float va = val0[h];
                    if (mode == 0) st_pkt(out + (size_t)w.kpart * N + row, va, tag);
                    else if (mode == 1) st_pkt(out + row, (a.act == 0 ? gelu_tanh(va) : silu_clip(va)) * val1[h], tag);
                    else {
                        float v = va;
                        if (a.logits) a.logits[row] = a.final_cap > 0.f ? tanhf(v / a.final_cap) * a.final_cap : v;
                        if (!(v == v)) v = -3.402823466e+38f;
                        if (better(v, row, best_v, best_i)) { best_v = v; best_i = row; }
                    }
                }
            }
            if (si == 0) fmark(ph, 22);
            if (lane == 0) { while (pend > 0) { --pend; if (!i_done) issue_next(); } }
        }
    };

    // ---- attention of one layer (QK-norm + RoPE + KV append + soft-max(QK^T)V for this CTA's (head, split)) ----
    auto attention = [&](const TkLayer& ly, int L, const uint2* qkv, uint2* att, uint32_t tag) {
        constexpr int DPL = HD / 32, CP = TkAttn<T, HD>::CP, NPQ = (HD / 2 + 31) / 32, LPV = 32 / CP;
        const TkAttnSplit sp = tk_attn_split(a.s_max, ly.window, p, CP);
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
        KvRow<T, DPL> kr[CP], vr[CP];
        auto load_rows = [&](uint32_t c, uint32_t kv, KvRow<T, DPL> (&rows)[CP]) {
            const uint32_t tp0 = c * CP;
            const uint32_t lo = max(tp0, sp.start), hi = min(tp0 + CP, seq) - 1;
            const uint32_t pn = tp0 / geo.page, slot0 = tp0 - pn * geo.page;
            const int32_t pg0 = max(pn < geo.max_pages ? bt[pn] : -1, 0);
            const T* base = kv_pool + kv_index(geo, (uint32_t)pg0, (uint32_t)L, kv, kvh, slot0) + lane * DPL;
#pragma unroll
            for (int j = 0; j < CP; ++j) {
                const uint32_t tp = min(max(tp0 + j, lo), hi);
                rows[j].load(base + (size_t)(tp - tp0) * HD);
            }
        };
        uint32_t c = c0 + warp;
        if (c < c1) { load_rows(c, 0, kr); load_rows(c, 1, vr); }
        // warp 0: query row; warp 1: newest key row; warp 2: newest value row (owner only)
        if (warp < 3 && (warp == 0 || owner)) {
            const uint32_t half = HD / 2;
            const uint32_t pp = (uint32_t)p < a.n_pos ? (uint32_t)p : a.n_pos - 1;
            const float* ct = a.cos_t[ly.rope] + (size_t)pp * half;
            const float* st = a.sin_t[ly.rope] + (size_t)pp * half;
            const bool is_q = warp == 0, is_k = warp == 1;
            const uint2* src = qkv + (is_q ? (size_t)head * HD : (size_t)a.q_dim + (is_k ? 0 : (size_t)a.k_dim) + (size_t)kvh * HD);
            float x0[NPQ], x1[NPQ];
            const int cnt = (int)lane < (int)half ? (int)((half - lane + 31) / 32) : 0;
            const float* wn = is_q ? ly.norm[TKN_Q] : ly.norm[TKN_K];
            float csv[NPQ], snv[NPQ], wn0[NPQ], wn1[NPQ];          // requested ahead of the poll
#pragma unroll
            for (int j = 0; j < NPQ; ++j) {
                const uint32_t i = lane + 32 * j;
                const bool inr = i < half;
                csv[j] = inr ? ct[i] : 1.f; snv[j] = inr ? st[i] : 0.f;
                wn0[j] = (inr && wn) ? wn[i] : 1.f; wn1[j] = (inr && wn) ? wn[i + half] : 1.f;
            }
            poll2<NPQ>(src + lane, src + half + lane, 32, cnt, tag, x0, x1, wt);
            size_t kv_off = 0;
            bool ok = appender;
            if (!is_q && appender) {
                const uint32_t pn = (uint32_t)p / geo.page;
                const int32_t page_id = pn < geo.max_pages ? bt[pn] : -1;
                if (page_id < 0) { ok = false; if (lane == 0) atomicOr(a.err, DEVERR_OOB_MAP); }
                else kv_off = kv_index(geo, (uint32_t)page_id, (uint32_t)L, is_k ? 0u : 1u, kvh, (uint32_t)p % geo.page);
            }
            if (!is_q && !is_k) {
#pragma unroll
                for (int j = 0; j < NPQ; ++j) {
                    const uint32_t i = lane + 32 * j;
                    if (i < half) {
                        s_vn[i] = kv_round<T>(x0[j]); s_vn[i + half] = kv_round<T>(x1[j]);
                        if (ok) { st_kv(kv_pool + kv_off + i, x0[j]); st_kv(kv_pool + kv_off + i + half, x1[j]); }
                    }
                }
            } else {
                float rms = 1.f;
                if (wn) {
                    float ss = 0.f;
#pragma unroll
                    for (int j = 0; j < NPQ; ++j) ss = fmaf(x0[j], x0[j], ss);
#pragma unroll
                    for (int j = 0; j < NPQ; ++j) ss = fmaf(x1[j], x1[j], ss);
                    ss = warp_sum(ss);
                    rms = sqrtf(ss / (float)HD + a.eps);
                }
                const float rcp = __frcp_rn(rms);
#pragma unroll
                for (int j = 0; j < NPQ; ++j) {
                    const uint32_t i = lane + 32 * j;
                    if (i < half) {
                        float a0 = x0[j], a1 = x1[j];
                        if (wn) { a0 = div_by(a0, rms, rcp) * wn0[j]; a1 = div_by(a1, rms, rcp) * wn1[j]; }
                        const float cs = csv[j], sn = snv[j];
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
            warp_reduce_scatter<CP>(sc, lane);                   // lane l holds the score of position l / LPV
            const uint32_t tp = c * CP + lane / LPV;
            const bool valid = tp >= sp.start && tp < seq;
            float sv = sc[0] * a.attn_scale;
            if (a.attn_cap > 0.f) sv = tanhf(sv / a.attn_cap) * a.attn_cap;
            sv = valid ? sv : NEG;
            float cmx = sv;
#pragma unroll
            for (int off = LPV; off < 32; off <<= 1) cmx = fmaxf(cmx, __shfl_xor_sync(0xffffffffu, cmx, off));
            const float m_new = fmaxf(m_run, cmx);
            const float alpha = expf(m_run - m_new);
            const float pz = valid ? expf(sv - m_new) : 0.f;
            float ps = pz;
#pragma unroll
            for (int off = LPV; off < 32; off <<= 1) ps += __shfl_xor_sync(0xffffffffu, ps, off);
            l_run = fmaf(l_run, alpha, ps);
            m_run = m_new;
#pragma unroll
            for (int d = 0; d < DPL; ++d) o[d] *= alpha;
#pragma unroll
            for (int j = 0; j < CP; ++j) {
                float vf[DPL];
                vr[j].to_float(vf);
                const float pv = __shfl_sync(0xffffffffu, pz, j * LPV);
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
        uint2* dst = att + ((size_t)split * H + head) * (HD + 2);
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

    auto cta_in = [&](int ph) { const TkPhase& P = a.ph[ph]; return P.n_rg > 0 && bx < P.G * P.cpr; };

    // ---- the token ----
    // One loop over (layer, product) so that the code of the norm chain, of the staging helpers and of the
    // product exists once: the kernel must stay inside the instruction cache, every phase runs once per layer.
    const int qkv_ld = a.q_dim + 2 * a.k_dim;
    const size_t att_half = (size_t)a.H * a.s_max * (HD + 2);
    const int cpr_o = a.ph[TK_O].cpr, cpr_d = a.ph[TK_DOWN].cpr;
    bool bail = false;
    const int n_it = a.n_layer * 4 + (a.with_lm ? 1 : 0);
#pragma unroll 1
    for (int it = 0; it < n_it; ++it) {
        const bool is_lm = it == a.n_layer * 4;
        const int L = is_lm ? a.n_layer - 1 : (it >> 2);
        const int kind = is_lm ? (int)TK_LM : (it & 3);        // TK_QKV, TK_O, TK_GU, TK_DOWN in this order
        const int par = L & 1;
        const uint32_t tag = tag_base + (uint32_t)L + 1u;
        const bool in = cta_in(kind);
        const TkLayer* ly = s_lay + L;
        cur_L = L;
        if (kind == TK_QKV) mark(L, 0);
        if (kind == TK_O) {
            attention(*ly, L, a.x_qkv + (size_t)par * qkv_ld, a.x_att + (size_t)par * att_half, tag);
            mark(L, 3);
        }
        if (kind != TK_O && kind != TK_DOWN) {
            // a product that reads the residual stream: the pending projection joins it first
            const uint2* add; int parts; uint32_t atag; const float* w_post; const float* w_pre;
            if (kind == TK_QKV) {
                add = L > 0 ? a.x_pd + (size_t)(par ^ 1) * cpr_d * E : nullptr; parts = cpr_d; atag = tag - 1u;
                w_post = L > 0 ? s_lay[L - 1].norm[TKN_POST_FFW] : nullptr; w_pre = ly->norm[TKN_ATTN];
            } else if (kind == TK_GU) {
                add = a.x_po + (size_t)par * cpr_o * E; parts = cpr_o; atag = tag;
                w_post = ly->norm[TKN_POST_ATTN]; w_pre = ly->norm[TKN_FFN];
            } else {
                add = a.x_pd + (size_t)par * cpr_d * E; parts = cpr_d; atag = tag;
                w_post = ly->norm[TKN_POST_FFW]; w_pre = a.out_norm;
            }
            chain(add, parts, atag, w_post, w_pre, in);
        }
        // (o-proj and down-proj stage per warp inside the product: no CTA barrier on their path)
        if (kind != TK_O && kind != TK_DOWN) { if (__syncthreads_or(wt.failed ? 1 : 0)) { bail = true; break; } }
        mark(is_lm ? -1 : L, is_lm ? 11 : (kind == TK_QKV ? 1 : 2 + 2 * kind));                // 1, 4, 6, 8: input staged
        if (is_lm && bx == 0 && a.h_out) {
            for (int i = tid; i < E; i += TK_THREADS) a.h_out[i] = s_h[i];
        }
        if (in) {
            uint2* out = kind == TK_QKV ? a.x_qkv + (size_t)par * qkv_ld
                       : kind == TK_O ? a.x_po + (size_t)par * cpr_o * E
                       : kind == TK_GU ? a.x_act + (size_t)par * a.FF
                       : kind == TK_DOWN ? a.x_pd + (size_t)par * cpr_d * E : nullptr;
            const uint2* in_buf = kind == TK_O ? a.x_att + (size_t)par * att_half : a.x_act + (size_t)par * a.FF;
            product(kind, kind == TK_GU ? 1 : (kind == TK_LM ? 2 : 0), out, tag, in_buf, ly->window);
        }
        if (kind != TK_O && kind != TK_DOWN) __syncthreads();     // the shared staging area is reused by the next phase
        mark(is_lm ? -1 : L, is_lm ? 12 : (kind == TK_QKV ? 2 : 3 + 2 * kind));                // 2, 5, 7, 9: product done
    }
    if (!bail) {
        const uint32_t tag = tag_base + (uint32_t)a.n_layer;
        if (a.with_lm && cta_in(TK_LM)) {
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
                    float v0[1], v1[1];
                    poll2<1>(a.x_amax + 2 * i, a.x_amax + 2 * i + 1, 0, 1, tag, v0, v1, wt);
                    const int k = __float_as_int(v1[0]);
                    if (better(v0[0], k, bv, bi)) { bv = v0[0]; bi = k; }
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
            mark(-1, 13);
            if (!bail && tid == 0) { a.pos[0] = p + 1; *a.seq = seq_no + 1u; }
        }
    }
    if (bail) {
        // the step counter still moves on: packets this step left behind must never match a later step's tags
        if (tid == 0) { atomicOr(a.err, DEVERR_WAIT); atomicExch(a.dead, 1u); atomicMax(a.seq, seq_no + 1u); }
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
