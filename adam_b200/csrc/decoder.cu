// Fused decoder: one decoded token for a batch of sequences as a fixed sequence
// of kernels (captured once into a CUDA graph and replayed), with positions and
// token ids living in device memory so that consecutive tokens need no host work.
//
// It computes what the reference engine's per-token loop computes
// (adam/models/engine.py:2971-3706 `_forward`: embed, per layer RMSNorm -> QKV ->
// QK-norm + RoPE -> KV append -> attention -> o-proj -> post-norm + residual ->
// RMSNorm -> gate/up -> GeGLU -> down -> post-norm + residual, final norm, LM head
// + arg-max), with the arithmetic of the reference's numpy decoder
// (tests/diagnostics/diag_inference.py:973-1037).  Differences from the reference
// runtime, all additive: B independent sequences per step, a paged KV cache in
// fp16 or fp32, an optional sliding-window mask on non-global layers, rotary angles
// read from a table the host supplies, chunked prefill (many prompt positions per
// pass), prefix reuse, and a part-wise step for tensor-parallel callers.
#include "common.cuh"
#include "gemv.cuh"
#include "gemv_mma.cuh"
#include "gemm_tc.cuh"
#include "token.cuh"
#include "blocks8.cuh"

#include <cstdlib>
#include <cstring>
#include <vector>

namespace ab {

int weight_ref(const Map* m, uint64_t off, uint64_t n_elems, int* wtype, WeightRef* w);
int argmax_scratch(float** pv, int** pi, unsigned int** tk);
int launch_sample(const float* logits, uint32_t V, uint32_t batch, uint32_t k, float temperature, float top_p, float penalty, int on_prompt,
                  uint64_t seed, const int32_t* pos, const int32_t* prompt_len, const int32_t* prompt_tok, int32_t* gen_log, uint32_t ld,
                  int32_t* cur_tok, float* cur_val);
bool capturing();

enum { MAT_Q = 0, MAT_K, MAT_V, MAT_O, MAT_GATE, MAT_UP, MAT_DOWN, MAT_EMBD, MAT_OUTPUT, MAT_KINDS };
enum { NORM_ATTN = 0, NORM_POST_ATTN, NORM_FFN, NORM_POST_FFW, NORM_Q, NORM_K, NORM_OUTPUT, NORM_KINDS };

struct Mat { bool bound; int wtype; WeightRef w; uint32_t rows, cols; uint32_t map_id; uint64_t elem_off; const uint8_t* tiled; };

struct Layer {
    Mat m[7];
    const float* norm[6];       // NORM_ATTN .. NORM_K (NULL = absent)
    bool qkv_contiguous, gateup_pairable;
    const uint8_t* qkv_tiled;   // row-tiled copy of the q,k,v rows as one tensor
};

struct Decoder {
    bool used;
    adam_b200_decoder_desc d;
    std::vector<Layer> layers;
    Mat embd, output;
    const float* output_norm;
    float* rope_cos[2]; float* rope_sin[2]; uint32_t rope_pos[2];
    // device state
    int32_t* pos;  int32_t* cur_tok;  float* cur_val;  int32_t* prompt_len;  int32_t* prompt_tok;  int32_t* gen_log;
    int32_t* block_table; uint32_t max_pages_per_seq, n_pages;
    void* kv_pool; size_t page_elems;
    float *hbuf[2], *qkv, *attn_out, *proj, *act, *logits; int h_final;
    float *part_o, *part_ml; unsigned int* attn_ticket; uint32_t n_splits;
    int32_t *row_seq, *row_pos; // chunked prefill: (sequence, position) of every row of the chunk
    uint32_t rows_cap;          // rows the activation buffers hold: max(max_batch, PREFILL_ROWS)
    std::vector<uint32_t> hpos, hplen, hres;   // host mirror of positions, prompt lengths and reserved tokens (argument checks)
    std::vector<int32_t> hbt;            // host mirror of the block table
    int32_t* tok_ring[4]; cudaEvent_t tok_event[4]; uint32_t tok_next;   // pinned slots for asynchronous token reads
    uint32_t batch;             // active sequences
    bool use_tiles;             // build row-tiled weight copies for the tensor-core GEMV
    // device-side sampling (adam_b200_decoder_set_sampling; used by steps with flag bit4)
    uint32_t smp_k; float smp_temp, smp_top_p, smp_penalty; int smp_on_prompt; uint64_t smp_seed;
    std::vector<uint32_t> free_pages;
    cudaGraphExec_t graph[2]; cudaGraph_t graph_src[2]; uint32_t graph_batch[2]; uint64_t graph_kernels[2];
    // single-launch token kernel (token.cuh): 0 = not examined yet, 1 = ready, -1 = this model does not qualify
    int tk_state; TkArgs tk; int tk_grid; int tk_wt; void* tk_mem[9];
    cudaGraphExec_t tk_graph[2]; cudaGraph_t tk_graph_src[2]; int tk_graph_state[2];   // TK_GRAPH_N token kernels per replay (index = LM head or not); state -1 = capture refused
};

constexpr uint32_t MAX_DECODERS = 8;
constexpr uint32_t ATTN_SPLIT = 64;        // fewest tokens an attention CTA takes before another CTA is added
constexpr uint32_t ATTN_MAX_SPLITS = 64;   // attention CTAs per (sequence, kv head)
constexpr uint32_t PREFILL_ROWS = 64;      // rows (sequences x tokens) of one prefill chunk
static Decoder* g_dec[MAX_DECODERS];

static Decoder* get_dec(uint32_t id) {
    if (!ready()) return nullptr;
    if (id >= MAX_DECODERS || !g_dec[id]) { fail(ADAMAH_ERR_NOT_FOUND, "decoder %u does not exist", id); return nullptr; }
    return g_dec[id];
}

// ---- kernels ---------------------------------------------------------------
#ifdef ADAM_B200_STEP_TRACE
// step trace: [4 products][8 CTAs][8 stamps] then [32 attention CTAs][8 stamps] of layer g_step_trace_layer
static long long* g_step_trace = nullptr; static uint32_t g_step_trace_layer = 0; static int g_step_trace_slot = -1;
#endif

// h[b] = dequant(token_embd[row tok]) * emb_scale   (diag_inference.py:975-977)
template <int WT>
__global__ void k_embed(const WeightRef w, uint32_t n_embd, uint32_t n_vocab, float emb_scale,
                        const int32_t* __restrict__ pos, const int32_t* __restrict__ prompt_len, const int32_t* __restrict__ prompt_tok,
                        uint32_t prompt_ld, const int32_t* __restrict__ cur_tok, float* __restrict__ h,
                        const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_pos, uint32_t* err) {
    pdl_launch_dependents();
    pdl_wait();
    // decode: row = sequence at its own position; prefill: row r = (sequence row_seq[r], position row_pos[r])
    const uint32_t r = blockIdx.x;
    const uint32_t b = row_seq ? (uint32_t)row_seq[r] : r;
    const int32_t p = row_pos ? row_pos[r] : pos[b];
    int32_t tok = (p < prompt_len[b]) ? prompt_tok[(size_t)b * prompt_ld + p] : cur_tok[b];
    if (tok < 0 || (uint32_t)tok >= n_vocab) { if (threadIdx.x == 0) atomicOr(err, DEVERR_BAD_TOKEN); tok = 0; }
    float* out = h + (size_t)r * n_embd;
    if (WT == WT_Q8_0 || WT == WT_Q5_0) {
        // code * fp16 scale is exact in float32; the embedding multiplier rounds once (map_row_gather_xq8.comp)
        const size_t b0 = (size_t)tok * (n_embd / 32);
        for (uint32_t i = threadIdx.x; i < n_embd; i += blockDim.x) {
            const size_t blk = b0 + (i >> 5);
            const uint32_t j = i & 31;
            int q;
            if (WT == WT_Q8_0) q = (int)reinterpret_cast<const int8_t*>(w.q)[blk * 32 + j];
            else {
                const uint32_t byte = reinterpret_cast<const uint8_t*>(w.q)[blk * 16 + (j & 15)];
                q = (int)((j < 16 ? (byte & 15u) : (byte >> 4)) | (((w.h[blk] >> j) & 1u) << 4)) - 16;
            }
            out[i] = __fmul_rn(__fmul_rn((float)q, __half2float(w.d[blk])), emb_scale);
        }
    } else if (WT == WT_Q4_0) {
        const uint32_t nblk = n_embd / 32;
        const uint8_t* q = reinterpret_cast<const uint8_t*>(w.q + (size_t)tok * nblk);
        const __half* d = w.d + (size_t)tok * nblk;
        for (uint32_t i = threadIdx.x; i < nblk * 16; i += blockDim.x) {
            const uint32_t blk = i >> 4, j = i & 15;
            const float s = __half2float(d[blk]);
            const uint32_t byte = q[blk * 16 + j];
            out[blk * 32 + j]      = __fmul_rn(__fmul_rn((float)(int)(byte & 15) - 8.f, s), emb_scale);
            out[blk * 32 + 16 + j] = __fmul_rn(__fmul_rn((float)(int)(byte >> 4) - 8.f, s), emb_scale);
        }
    } else {
        const uint32_t nsb = n_embd / 256;
        const uint8_t* base = reinterpret_cast<const uint8_t*>(w.q) + (size_t)tok * nsb * 144;
        for (uint32_t i = threadIdx.x; i < nsb * 128; i += blockDim.x) {
            const uint32_t sb = i >> 7, bi = i & 127, grp = bi >> 5, j = bi & 31;
            const uint8_t* blk = base + (size_t)sb * 144;
            const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
            float s0, m0, s1, m1;
            // same products as the loader: (d*sc), (dmin*m), each rounded once
            {
                const int sh = (grp & 1) * 16;
                const uint32_t s16 = (hdr.y >> sh) & 0xFFFFu, m16 = (hdr.z >> sh) & 0xFFFFu, t16 = (hdr.w >> sh) & 0xFFFFu;
                uint32_t sp, mp;
                if (grp < 2) { sp = s16 & 0x3F3Fu; mp = m16 & 0x3F3Fu; }
                else { sp = (t16 & 0x0F0Fu) | ((s16 >> 2) & 0x3030u); mp = ((t16 >> 4) & 0x0F0Fu) | ((m16 >> 2) & 0x3030u); }
                const float dd = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
                const float dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
                s0 = __fmul_rn(dd, (float)(sp & 0xFFu)); s1 = __fmul_rn(dd, (float)(sp >> 8));
                m0 = __fmul_rn(dm, (float)(mp & 0xFFu)); m1 = __fmul_rn(dm, (float)(mp >> 8));
            }
            const uint32_t byte = blk[16 + bi];
            float* o = out + sb * 256 + grp * 64;
            o[j]      = __fmul_rn(__fsub_rn(__fmul_rn((float)(byte & 15), s0), m0), emb_scale);
            o[32 + j] = __fmul_rn(__fsub_rn(__fmul_rn((float)(byte >> 4), s1), m1), emb_scale);
        }
    }
}

// Cluster primitives of the attention launch whose position splits form one thread-block cluster: the splits'
// partial results go to the first CTA's shared memory and meet at the hardware cluster barrier (every thread of
// every CTA arrives exactly once per phase; a CTA may exit after its last arrive).
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }
__device__ __forceinline__ uint32_t dsmem_addr_rank0(const void* p) {          // address of `p` in the cluster's CTA 0
    uint32_t r;
    asm("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(p)), "r"(0));
    return r;
}
__device__ __forceinline__ void st_dsmem4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ void st_dsmem2(uint32_t addr, float2 v) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" :: "r"(addr), "f"(v.x), "f"(v.y) : "memory");
}

// Decode attention for one (split, kv head, sequence), all query heads that share
// the kv head, with the steps that precede it folded in:
//   * per-head RMSNorm + half-split RoPE of the query rows (map_qk_norm_rope_x.comp),
//     angles read from the host-made table;
//   * the CTA whose range holds the newest position does the same for the key row
//     and appends key and value to the paged cache (map_row_copy.comp);
//   * p = softmax(cap*tanh(q.k*scale/cap)) over positions [start, seq), o = p @ V
//     (map_matmul_t.comp + map_attn_softmax_value.comp; diag_inference.py:989-1012).
// Work split.  Positions are walked in chunks of ATTN_CP = 8 (aligned to absolute
// multiples of 8, so a chunk never straddles a page whose size is a multiple of 8).
// The active CTAs (at most gridDim.x, at least one per 8 chunks) take contiguous
// runs of chunks; inside a CTA the 8 warps take chunks round-robin.  A lane owns
// head_dim/32 consecutive dims of every K and V row, so one row is one coalesced
// warp load, and all 8+8 row loads of a chunk are issued before any is used; the
// next chunk's K rows are requested as soon as the scores are done and its V rows
// after the P@V accumulation.  The 8 x heads partial dot products of a chunk are
// summed over the lanes with a reduce-scatter (one shuffle per value) that leaves
// score (position j, head g) on one lane; the soft-max runs online per warp, and
// (max, sum, o) are merged across warps in shared memory, then across CTAs by the
// CTA that finishes last.
constexpr int ATTN_CP = 8;
constexpr uint32_t ATTN_CHUNKS_PER_CTA = 32;   // chunks a CTA takes (4 per warp) before another CTA joins, when the grid is already large;
                                               // launches with few (sequence, head) pairs pass a smaller number in the upper half of `hpc`

template <typename T, int GS_MAX, int HD>
__global__ void __launch_bounds__(256) k_attention(const float* __restrict__ qkv, uint32_t qkv_ld,
                                                   const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
                                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, uint32_t n_pos,
                                                   void* __restrict__ kv_pool_v, KvGeom geo,
                                                   const int32_t* __restrict__ block_table, const int32_t* __restrict__ pos,
                                                   uint32_t n_head, uint32_t layer, uint32_t window, float scale, float cap,
                                                   float* __restrict__ out, float* __restrict__ part_o, float* __restrict__ part_ml,
                                                   unsigned int* __restrict__ ticket, uint32_t n_splits_max, uint32_t hpc,
                                                   const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_pos, uint32_t* err STEP_TRACE_PARAM) {
#ifdef ADAM_B200_STEP_TRACE
#define AT_STAMP(slot) do { if (threadIdx.x == 0 && blockIdx.z == 0 && (blockIdx.y * gridDim.x + blockIdx.x) < 32) STEP_STAMP(trace, (blockIdx.y * gridDim.x + blockIdx.x) * 8 + (slot)); } while (0)
#else
#define AT_STAMP(slot) do { } while (0)
#endif
    AT_STAMP(0);
    // n_splits_max == 0: the gridDim.x splits of a (sequence, head group) are one thread-block cluster and merge
    // through CTA 0's shared memory instead of global memory, a ticket and the last CTA to arrive.
    const bool cmerge = n_splits_max == 0;
    if (cmerge) cluster_arrive();               // "this CTA runs": waited for before the first store into CTA 0
    // row_seq / row_pos != NULL: chunked prefill.  Row b of qkv/out belongs to sequence row_seq[b] at position
    // row_pos[b], and the keys and values of the whole chunk are already in the cache (k_kv_append ran before).
    const bool appended = row_pos != nullptr;
    const uint32_t cpc_min = (hpc >> 16) ? (hpc >> 16) : ATTN_CHUNKS_PER_CTA;     // chunks per CTA before another CTA joins
    hpc &= 0xFFFFu;
    T* __restrict__ kv_pool = reinterpret_cast<T*>(kv_pool_v);
    constexpr int DPL = HD / 32;                // dims per lane
    constexpr int CP = ATTN_CP;                 // positions per chunk
    constexpr int NV = CP * GS_MAX;             // scores per chunk
    constexpr int VPL = NV >= 32 ? NV / 32 : 1; // scores a lane holds after the reduce-scatter
    constexpr int LPV = NV >= 32 ? 1 : 32 / NV; // lanes that hold the same score
    constexpr float NEG = -1.0e30f;
    static_assert(DPL >= 1 && (GS_MAX == 1 || GS_MAX == 2 || GS_MAX == 4 || GS_MAX == 8), "unsupported attention shape");
    extern __shared__ __align__(16) float sm[];
    __shared__ float s_m[8][GS_MAX], s_l[8][GS_MAX];
    __shared__ float s_w[8][GS_MAX], s_M[GS_MAX];
    __shared__ bool s_last;
    // blockIdx.y = (kv head, group of `hpc` query heads that share it)
    const uint32_t hgn = (n_head / geo.n_kv) / hpc;
    const uint32_t split = blockIdx.x, kvh = blockIdx.y / hgn, hg = blockIdx.y % hgn, b = blockIdx.z;
    const uint32_t head0 = kvh * (n_head / geo.n_kv) + hg * hpc;
    const uint32_t slot_y = b * gridDim.y + blockIdx.y;        // scratch slot of this (sequence, head group)
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // The block table is written by the host before the step's first kernel, so it can be
    // read ahead of the dependency wait: up to 128 entries sit in registers across the warp.
    const uint32_t sq = row_seq ? (uint32_t)row_seq[b] : b;
    const int32_t* bt = block_table + (size_t)sq * geo.max_pages;
    const bool bt_regs = geo.max_pages <= 128;
    int32_t btr[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { const uint32_t i = lane + 32 * k; btr[k] = (bt_regs && i < geo.max_pages) ? bt[i] : -1; }
    auto page_of = [&](uint32_t pn) -> int32_t {        // pn is the same for the whole warp
        if (pn >= geo.max_pages) return -1;
        if (!bt_regs) return bt[pn];
        int32_t v = btr[0];
        if (pn >= 32) v = btr[1];
        if (pn >= 64) v = btr[2];
        if (pn >= 96) v = btr[3];
        return __shfl_sync(0xffffffffu, v, pn & 31);
    };
    // QK-norm weights are read-only too.
    constexpr int NP = (HD / 2 + 31) / 32;          // rotation pairs per lane
    float wq0[NP], wq1[NP], wk0[NP], wk1[NP];
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        const uint32_t i = lane + 32 * j;
        const bool in = i < HD / 2;
        wq0[j] = (in && q_norm) ? q_norm[i] : 1.f; wq1[j] = (in && q_norm) ? q_norm[i + HD / 2] : 1.f;
        wk0[j] = (in && k_norm) ? k_norm[i] : 1.f; wk1[j] = (in && k_norm) ? k_norm[i + HD / 2] : 1.f;
    }
    // Positions only change in the step's last kernel, and the step's first kernel is
    // launched with a full dependency on it, so the position, and everything in the cache
    // older than this step, can be read ahead of the wait as well.
    // In chunked prefill the chunk's own keys and values were written by the kernel just before
    // this one, so the wait comes first there.
    if (appended) { pdl_launch_dependents(); pdl_wait(); }
    const uint32_t hd = HD, half = HD / 2, gs = hpc;
    const int32_t p = appended ? row_pos[b] : pos[b];
    const uint32_t seq = (uint32_t)p + 1;
    const uint32_t start = (window > 0 && seq > window) ? seq - window : 0;
    const uint32_t c_first = start / CP, n_chunks = (seq - 1) / CP - c_first + 1;
    const uint32_t n_act = min((uint32_t)gridDim.x, (n_chunks + cpc_min - 1) / cpc_min);
    if (split >= n_act) { if (cmerge) { cluster_wait(); cluster_arrive(); } return; }
    const uint32_t cpc = (n_chunks + n_act - 1) / n_act;
    const uint32_t c0 = min(c_first + split * cpc, c_first + n_chunks), c1 = min(c_first + n_chunks, c0 + cpc);
    const uint32_t c_new = appended ? 0xFFFFFFFFu : (uint32_t)p / CP;      // chunk whose newest row comes from this step's q/k/v
    const bool owner = !appended && c_new >= c0 && c_new < c1;
    float* s_q = sm;                            // [gs][hd]
    float* s_kn = s_q + gs * hd;                // [hd] newest key (as stored)
    float* s_vn = s_kn + hd;                    // [hd] newest value (as stored)
    float* s_o = s_vn + hd;                     // [8 warps][gs][hd]
    float* s_cp = s_o + 8 * gs * hd;            // cluster merge, CTA 0 only: [split][gs * hd + 4 * gs] (16-byte aligned rows)
    const bool page8 = (geo.page % CP) == 0;

    // Rows of chunk c.  Every load is unconditional (a predicated load would have to be
    // merged with a zero right away, which serialises the loads): positions outside
    // [start, seq) read a neighbouring valid row instead, and their scores are masked
    // later; the cache is zero-filled at creation, so whatever is read is finite.
    KvRow<T, DPL> kr[CP], vr[CP];
    auto load_rows = [&](uint32_t c, uint32_t kv, KvRow<T, DPL> (&rows)[CP]) {
        const uint32_t tp0 = c * CP;
        if (page8) {
            // the chunk lies inside one page and its rows are consecutive
            const uint32_t lo = max(tp0, start), hi = min(tp0 + CP, seq) - 1;
            const uint32_t pn = tp0 / geo.page, slot0 = tp0 - pn * geo.page;
            const int32_t pg0 = max(page_of(pn), 0);
            const T* base = kv_pool + kv_index(geo, (uint32_t)pg0, layer, kv, kvh, slot0) + lane * DPL;
#pragma unroll
            for (int j = 0; j < CP; ++j) {
                const uint32_t tp = min(max(tp0 + j, lo), hi);
                rows[j].load(base + (size_t)(tp - tp0) * HD);
            }
        } else {
#pragma unroll
            for (int j = 0; j < CP; ++j) {
                const uint32_t tp = min(max(tp0 + j, start), seq - 1);
                const uint32_t pn = tp / geo.page;
                const int32_t pg = max(page_of(pn), 0);
                rows[j].load(kv_pool + kv_index(geo, (uint32_t)pg, layer, kv, kvh, tp - pn * geo.page) + lane * DPL);
            }
        }
    };
    // With one query head per CTA there are registers for a second chunk in flight, so a
    // warp that owns up to two chunks waits for memory only once.
    constexpr bool DB = (GS_MAX == 1) && (DPL * sizeof(T) <= 16);
    constexpr uint32_t CSTEP = DB ? 16 : 8;     // chunk stride of one loop iteration
    KvRow<T, DPL> kr2[DB ? CP : 1], vr2[DB ? CP : 1];
    uint32_t c = c0 + warp;
    if (c < c1) { load_rows(c, 0, kr); load_rows(c, 1, vr); }
    if constexpr (DB) { if (c + 8 < c1) { load_rows(c + 8, 0, kr2); load_rows(c + 8, 1, vr2); } }

    // ---- a warp per row: query heads, and (owner only) the newest key and value rows ----
    const uint32_t pp = (uint32_t)p < n_pos ? (uint32_t)p : n_pos - 1;
    if ((uint32_t)p >= n_pos && tid == 0) atomicOr(err, DEVERR_OOB_MAP);
    const float* ct = cos_t + (size_t)pp * half;
    const float* st = sin_t + (size_t)pp * half;
    float cs[NP], sn[NP];
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        const uint32_t i = lane + 32 * j;
        cs[j] = i < half ? ct[i] : 1.f;
        sn[j] = i < half ? st[i] : 0.f;
    }
    AT_STAMP(1);
    if (!appended) { pdl_launch_dependents(); pdl_wait(); }     // this step's q/k/v rows come from the previous kernel
    AT_STAMP(2);
    const float* row_q = qkv + (size_t)b * qkv_ld + (size_t)head0 * hd;
    const float* row_k = qkv + (size_t)b * qkv_ld + (size_t)n_head * hd + (size_t)kvh * hd;
    const float* row_v = row_k + (size_t)geo.n_kv * hd;
    const uint32_t n_rows = gs + (owner ? 2u : 0u);
    for (uint32_t r = warp; r < n_rows; r += 8) {
        const bool is_q = r < gs, is_k = (r == gs);
        const float* src = is_q ? row_q + (size_t)r * hd : (is_k ? row_k : row_v);
        size_t kv_off = 0;
        bool ok = true;
        if (!is_q) {
            const uint32_t page_no = (uint32_t)p / geo.page;
            const int32_t page_id = page_of(page_no);
            if (page_id < 0) { ok = false; if (lane == 0) atomicOr(err, DEVERR_OOB_MAP); }
            else if (hg != 0) ok = false;               // one head group appends to the cache; the others only need the rows
            if (ok) kv_off = kv_index(geo, (uint32_t)page_id, layer, is_k ? 0u : 1u, kvh, (uint32_t)p % geo.page);
        }
        if (!is_q && !is_k) {
            for (uint32_t i = lane; i < hd; i += 32) {
                const float v = src[i];
                s_vn[i] = kv_round<T>(v);
                if (ok) st_kv(kv_pool + kv_off + i, v);
            }
            continue;
        }
        const float* w = is_q ? q_norm : k_norm;
        float x0[NP], x1[NP], w0[NP], w1[NP];
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const uint32_t i = lane + 32 * j;
            const bool in = i < half;
            x0[j] = in ? src[i] : 0.f;
            x1[j] = in ? src[i + half] : 0.f;
            w0[j] = is_q ? wq0[j] : wk0[j];
            w1[j] = is_q ? wq1[j] : wk1[j];
        }
        float rms = 1.f;
        if (w) {
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < NP; ++j) ss = fmaf(x0[j], x0[j], ss);
#pragma unroll
            for (int j = 0; j < NP; ++j) ss = fmaf(x1[j], x1[j], ss);
            ss = warp_sum(ss);
            rms = sqrtf(ss / (float)hd + eps);
        }
        const float rcp = __frcp_rn(rms);
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const uint32_t i = lane + 32 * j;
            if (i < half) {
                float a0 = x0[j], a1 = x1[j];
                if (w) { a0 = div_by(a0, rms, rcp) * w0[j]; a1 = div_by(a1, rms, rcp) * w1[j]; }
                const float y0 = __fsub_rn(__fmul_rn(a0, cs[j]), __fmul_rn(a1, sn[j]));
                const float y1 = __fadd_rn(__fmul_rn(a0, sn[j]), __fmul_rn(a1, cs[j]));
                if (is_q) { s_q[r * hd + i] = y0; s_q[r * hd + i + half] = y1; }
                else {
                    s_kn[i] = kv_round<T>(y0); s_kn[i + half] = kv_round<T>(y1);
                    if (ok) { st_kv(kv_pool + kv_off + i, y0); st_kv(kv_pool + kv_off + i + half, y1); }
                }
            }
        }
    }
    __syncthreads();
    AT_STAMP(3);

    // ---- this warp's chunks: scores, online soft-max, P@V ----
    float q[GS_MAX][DPL], o[GS_MAX][DPL], m_run[VPL], l_run[VPL];
#pragma unroll
    for (int g = 0; g < GS_MAX; ++g)
#pragma unroll
        for (int d = 0; d < DPL; ++d) { q[g][d] = g < (int)gs ? s_q[g * hd + lane * DPL + d] : 0.f; o[g][d] = 0.f; }
#pragma unroll
    for (int r = 0; r < VPL; ++r) { m_run[r] = NEG; l_run[r] = 0.f; }
    auto process = [&](uint32_t c, KvRow<T, DPL> (&kr)[CP], KvRow<T, DPL> (&vr)[CP]) {
        if (c == c_new) {
            // the newest position's rows come from this step's q/k/v, not from the cache
            KvRow<T, DPL> nk, nv;
            nk.from_float(s_kn + lane * DPL); nv.from_float(s_vn + lane * DPL);
            const int jn = (int)((uint32_t)p % CP);
#pragma unroll
            for (int j = 0; j < CP; ++j) if (j == jn) { kr[j] = nk; vr[j] = nv; }
        }
        float sc[NV];
#pragma unroll
        for (int j = 0; j < CP; ++j) {
            float kf[DPL];
            kr[j].to_float(kf);
#pragma unroll
            for (int g = 0; g < GS_MAX; ++g) {
                if constexpr (DPL >= 2) {
                    float a0 = 0.f, a1 = 0.f;
#pragma unroll
                    for (int d = 0; d < DPL; d += 2) fma2(a0, a1, q[g][d], q[g][d + 1], kf[d], kf[d + 1]);
                    sc[j * GS_MAX + g] = a0 + a1;
                } else {
                    sc[j * GS_MAX + g] = q[g][0] * kf[0];
                }
            }
        }
        const uint32_t c_next = c + CSTEP;
        if (c_next < c1) load_rows(c_next, 0, kr);
        warp_reduce_scatter<NV>(sc, lane);
        float pz[VPL], alpha[VPL];
#pragma unroll
        for (int r = 0; r < VPL; ++r) {
            const uint32_t v = NV >= 32 ? lane * VPL + r : lane / LPV;
            const uint32_t j = v / GS_MAX, g = v % GS_MAX;
            const uint32_t tp = c * CP + j;
            const bool valid = tp >= start && tp < seq && g < gs;
            float sv = sc[r] * scale;
            if (cap > 0.f) sv = tanhf(sv / cap) * cap;
            sv = valid ? sv : NEG;
            float cm = sv;
            cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 4));
            cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 8));
            cm = fmaxf(cm, __shfl_xor_sync(0xffffffffu, cm, 16));
            const float m_new = fmaxf(m_run[r], cm);
            alpha[r] = expf(m_run[r] - m_new);
            pz[r] = valid ? expf(sv - m_new) : 0.f;
            float ps = pz[r];
            ps += __shfl_xor_sync(0xffffffffu, ps, 4);
            ps += __shfl_xor_sync(0xffffffffu, ps, 8);
            ps += __shfl_xor_sync(0xffffffffu, ps, 16);
            l_run[r] = fmaf(l_run[r], alpha[r], ps);
            m_run[r] = m_new;
        }
#pragma unroll
        for (int g = 0; g < GS_MAX; ++g) {
            // lane and slot that hold (position 0, head g)
            const float al = __shfl_sync(0xffffffffu, alpha[g % VPL], NV >= 32 ? g / VPL : g * LPV);
#pragma unroll
            for (int d = 0; d < DPL; ++d) o[g][d] *= al;
        }
#pragma unroll
        for (int j = 0; j < CP; ++j) {
            float vf[DPL];
            vr[j].to_float(vf);
#pragma unroll
            for (int g = 0; g < GS_MAX; ++g) {
                const int v = j * GS_MAX + g;
                const float pv = __shfl_sync(0xffffffffu, pz[v % VPL], NV >= 32 ? v / VPL : v * LPV);
                if constexpr (DPL >= 2) {
#pragma unroll
                    for (int d = 0; d < DPL; d += 2) fma2(o[g][d], o[g][d + 1], pv, pv, vf[d], vf[d + 1]);
                } else {
                    o[g][0] = fmaf(pv, vf[0], o[g][0]);
                }
            }
        }
        if (c_next < c1) load_rows(c_next, 1, vr);
    };
    for (; c < c1; c += CSTEP) {
        process(c, kr, vr);
        if constexpr (DB) { if (c + 8 < c1) process(c + 8, kr2, vr2); }
    }
    AT_STAMP(4);
    // ---- merge the warps ----
    {
        float* so = s_o + (size_t)warp * gs * hd + lane * DPL;
#pragma unroll
        for (int g = 0; g < GS_MAX; ++g) {
            if (g < (int)gs) {
                if constexpr (DPL % 4 == 0) {
#pragma unroll
                    for (int d = 0; d < DPL; d += 4) *reinterpret_cast<float4*>(so + g * hd + d) = make_float4(o[g][d], o[g][d + 1], o[g][d + 2], o[g][d + 3]);
                } else {
#pragma unroll
                    for (int d = 0; d < DPL; ++d) so[g * hd + d] = o[g][d];
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < VPL; ++r) {
        const uint32_t v = NV >= 32 ? lane * VPL + r : lane / LPV;
        if (v < GS_MAX && (NV >= 32 || (lane % LPV) == 0)) { s_m[warp][v] = m_run[r]; s_l[warp][v] = l_run[r]; }
    }
    __syncthreads();
    if (tid < 8 * GS_MAX) {                     // weight of warp w for head g
        const uint32_t w = tid / GS_MAX, g = tid % GS_MAX;
        float M = NEG;
#pragma unroll
        for (int w2 = 0; w2 < 8; ++w2) M = fmaxf(M, s_m[w2][g]);
        s_w[w][g] = expf(s_m[w][g] - M);
        if (w == 0) s_M[g] = M;
    }
    __syncthreads();
    // thread -> 4 consecutive outputs (all of one head)
    const uint32_t n_out4 = gs * hd / 4;
    float* po = part_o + ((size_t)slot_y * n_splits_max + split) * gs * hd;
    float* pml = part_ml + ((size_t)slot_y * n_splits_max + split) * gs * 2;
    float* orow = out + ((size_t)b * n_head + head0) * hd;
    if (cmerge && n_act > 1 && split != 0) cluster_wait();      // CTA 0 of the cluster is running: its shared memory can be written
    for (uint32_t i4 = tid; i4 < n_out4; i4 += blockDim.x) {
        const uint32_t g = (i4 * 4) / hd;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        float L = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float ww = s_w[w][g];
            const float4 x = *reinterpret_cast<const float4*>(s_o + (size_t)w * gs * hd + i4 * 4);
            v.x = fmaf(ww, x.x, v.x); v.y = fmaf(ww, x.y, v.y); v.z = fmaf(ww, x.z, v.z); v.w = fmaf(ww, x.w, v.w);
            L = fmaf(ww, s_l[w][g], L);
        }
        if (n_act == 1) { v.x /= L; v.y /= L; v.z /= L; v.w /= L; reinterpret_cast<float4*>(orow)[i4] = v; }
        else if (cmerge) {
            float* mine = s_cp + (size_t)split * (gs * hd + 4 * gs);
            if (split == 0) {
                reinterpret_cast<float4*>(mine)[i4] = v;
                if ((i4 * 4) % hd == 0) *reinterpret_cast<float2*>(mine + gs * hd + g * 2) = make_float2(s_M[g], L);
            } else {
                st_dsmem4(dsmem_addr_rank0(mine + i4 * 4), v);
                if ((i4 * 4) % hd == 0) st_dsmem2(dsmem_addr_rank0(mine + gs * hd + g * 2), make_float2(s_M[g], L));
            }
        } else {
            reinterpret_cast<float4*>(po)[i4] = v;
            if ((i4 * 4) % hd == 0) *reinterpret_cast<float2*>(pml + g * 2) = make_float2(s_M[g], L);
        }
    }
    if (cmerge) {
        // every thread is here exactly once, whatever n_act is
        if (n_act == 1) { cluster_wait(); cluster_arrive(); return; }
        if (split != 0) { cluster_arrive(); return; }
        cluster_wait();
        cluster_arrive();
        cluster_wait();                         // ---- every split's partial result is in this CTA's shared memory ----
        const uint32_t pstride = gs * hd + 4 * gs;
        for (uint32_t i4 = tid; i4 < n_out4; i4 += blockDim.x) {
            const uint32_t g = (i4 * 4) / hd;
            float M = NEG;
            for (uint32_t s0 = 0; s0 < n_act; ++s0) M = fmaxf(M, s_cp[(size_t)s0 * pstride + gs * hd + g * 2]);
            float den = 0.f;
            float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t s0 = 0; s0 < n_act; ++s0) {
                const float* ps = s_cp + (size_t)s0 * pstride;
                const float w = expf(ps[gs * hd + g * 2] - M);
                const float4 x = reinterpret_cast<const float4*>(ps)[i4];
                num.x = fmaf(w, x.x, num.x); num.y = fmaf(w, x.y, num.y); num.z = fmaf(w, x.z, num.z); num.w = fmaf(w, x.w, num.w);
                den = fmaf(w, ps[gs * hd + g * 2 + 1], den);
            }
            reinterpret_cast<float4*>(orow)[i4] = make_float4(num.x / den, num.y / den, num.z / den, num.w / den);
        }
        AT_STAMP(7);
        return;
    }
    if (n_act == 1) return;
    AT_STAMP(5);
    __threadfence();
    __syncthreads();
    unsigned int* tkt = ticket + slot_y;
    if (tid == 0) s_last = (atomicAdd(tkt, 1u) == n_act - 1);
    __syncthreads();
    AT_STAMP(6);
    if (!s_last) return;
    __threadfence();
    // ---- merge the splits (last CTA to arrive): all loads of a batch of 4 splits are
    // issued together, then folded in with a running maximum ----
    const float* po0 = part_o + ((size_t)slot_y * n_splits_max) * gs * hd;
    const float* pml0 = part_ml + ((size_t)slot_y * n_splits_max) * gs * 2;
    for (uint32_t i4 = tid; i4 < n_out4; i4 += blockDim.x) {
        const uint32_t g = (i4 * 4) / hd;
        float M = NEG, den = 0.f;
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t s0 = 0; s0 < n_act; s0 += 4) {
            float2 ml[4]; float4 x[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t sidx = min(s0 + k, n_act - 1);
                ml[k] = __ldcg(reinterpret_cast<const float2*>(pml0 + ((size_t)sidx * gs + g) * 2));
                x[k] = __ldcg(reinterpret_cast<const float4*>(po0 + (size_t)sidx * gs * hd) + i4);
            }
            float Mn = M;
#pragma unroll
            for (int k = 0; k < 4; ++k) if (s0 + k < n_act) Mn = fmaxf(Mn, ml[k].x);
            const float a0 = expf(M - Mn);
            num.x *= a0; num.y *= a0; num.z *= a0; num.w *= a0; den *= a0;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                if (s0 + k < n_act) {
                    const float w = expf(ml[k].x - Mn);
                    num.x = fmaf(w, x[k].x, num.x); num.y = fmaf(w, x[k].y, num.y);
                    num.z = fmaf(w, x[k].z, num.z); num.w = fmaf(w, x[k].w, num.w);
                    den = fmaf(w, ml[k].y, den);
                }
            }
            M = Mn;
        }
        reinterpret_cast<float4*>(orow)[i4] = make_float4(num.x / den, num.y / den, num.z / den, num.w / den);
    }
    AT_STAMP(7);
    if (tid == 0) *tkt = 0u;
}

// Chunked prefill: QK-norm + RoPE of the key row and append of key and value to the paged
// cache for every row of the chunk, one warp per (row, kv head, K|V); the same arithmetic as
// the key/value part of k_attention.
template <typename T, int HD>
__global__ void __launch_bounds__(256) k_kv_append(const float* __restrict__ qkv, uint32_t qkv_ld, const float* __restrict__ k_norm, float eps,
                                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, uint32_t n_pos,
                                                   void* __restrict__ kv_pool_v, KvGeom geo, const int32_t* __restrict__ block_table,
                                                   const int32_t* __restrict__ row_seq, const int32_t* __restrict__ row_pos,
                                                   uint32_t n_rows, uint32_t n_head, uint32_t layer, uint32_t* err) {
    T* __restrict__ kv_pool = reinterpret_cast<T*>(kv_pool_v);
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t lane = threadIdx.x & 31, w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (w >= n_rows * geo.n_kv * 2) return;
    const uint32_t kv = w & 1u, kvh = (w >> 1) % geo.n_kv, r = (w >> 1) / geo.n_kv;
    const uint32_t sq = (uint32_t)row_seq[r];
    const int32_t p = row_pos[r];
    const uint32_t page_no = (uint32_t)p / geo.page;
    const int32_t page_id = page_no < geo.max_pages ? block_table[(size_t)sq * geo.max_pages + page_no] : -1;
    if (page_id < 0 || (uint32_t)p >= n_pos) { if (lane == 0) atomicOr(err, DEVERR_OOB_MAP); return; }
    T* dst = kv_pool + kv_index(geo, (uint32_t)page_id, layer, kv, kvh, (uint32_t)p % geo.page);
    const float* src = qkv + (size_t)r * qkv_ld + (size_t)n_head * HD + (size_t)kv * geo.n_kv * HD + (size_t)kvh * HD;
    if (kv == 1) {
        for (uint32_t i = lane; i < HD; i += 32) st_kv(dst + i, src[i]);
        return;
    }
    constexpr uint32_t half = HD / 2;
    constexpr int NP = (HD / 2 + 31) / 32;
    const float* ct = cos_t + (size_t)p * half;
    const float* st = sin_t + (size_t)p * half;
    float x0[NP], x1[NP];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        const uint32_t i = lane + 32 * j;
        x0[j] = i < half ? src[i] : 0.f;
        x1[j] = i < half ? src[i + half] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < NP; ++j) ss = fmaf(x0[j], x0[j], ss);
#pragma unroll
    for (int j = 0; j < NP; ++j) ss = fmaf(x1[j], x1[j], ss);
    float rms = 1.f;
    if (k_norm) { ss = warp_sum(ss); rms = sqrtf(ss / (float)HD + eps); }
    const float rcp = __frcp_rn(rms);
#pragma unroll
    for (int j = 0; j < NP; ++j) {
        const uint32_t i = lane + 32 * j;
        if (i < half) {
            float a0 = x0[j], a1 = x1[j];
            if (k_norm) { a0 = div_by(a0, rms, rcp) * k_norm[i]; a1 = div_by(a1, rms, rcp) * k_norm[i + half]; }
            const float c = ct[i], sn = st[i];
            st_kv(dst + i, __fsub_rn(__fmul_rn(a0, c), __fmul_rn(a1, sn)));
            st_kv(dst + i + half, __fadd_rn(__fmul_rn(a0, sn), __fmul_rn(a1, c)));
        }
    }
}

// Chunked prefill: row r = (sequence r / T, position pos[sequence] + r % T).
__global__ void k_prefill_rows(const int32_t* __restrict__ pos, uint32_t batch, uint32_t T, int32_t* __restrict__ row_seq, int32_t* __restrict__ row_pos) {
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= batch * T) return;
    const uint32_t s = r / T;
    row_seq[r] = (int32_t)s;
    row_pos[r] = pos[s] + (int32_t)(r % T);
}
__global__ void k_advance_n(int32_t* __restrict__ pos, uint32_t batch, int32_t n) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < batch) pos[b] += n;
}

// End of a step: advance positions; when the LM head ran, log the sampled token.
__global__ void k_advance(int32_t* __restrict__ pos, const int32_t* __restrict__ cur_tok, int32_t* __restrict__ gen_log,
                          uint32_t log_ld, uint32_t batch, int with_lm) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= batch) return;
    const int32_t p = pos[b] + 1;
    pos[b] = p;
    if (with_lm && (uint32_t)p < log_ld) gen_log[(size_t)b * log_ld + p] = cur_tok[b];
}

__global__ void k_fill_i32(int32_t* p, int32_t v, size_t n) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

// ---- host side ---------------------------------------------------------------

constexpr uint32_t TK_GRAPH_N = 8;
static void free_token_kernel(Decoder* D) {
    if (D->tk_state == 1) cudaStreamSynchronize(g.stream);
    for (int i = 0; i < 2; ++i) {
        if (D->tk_graph[i]) { cudaGraphExecDestroy(D->tk_graph[i]); cudaGraphDestroy(D->tk_graph_src[i]); D->tk_graph[i] = nullptr; D->tk_graph_src[i] = nullptr; }
        D->tk_graph_state[i] = 0;
    }
    for (void*& m : D->tk_mem) { if (m) cudaFree(m); m = nullptr; }
    D->tk_state = 0;
}

static void free_graphs(Decoder* D) {
    for (int i = 0; i < 2; ++i) {
        if (D->graph[i]) { cudaGraphExecDestroy(D->graph[i]); cudaGraphDestroy(D->graph_src[i]); D->graph[i] = nullptr; D->graph_src[i] = nullptr; }
    }
    free_token_kernel(D);
}

static void destroy(Decoder* D) {
    cudaStreamSynchronize(g.stream);
    free_graphs(D);
    free_token_kernel(D);
    for (int i = 0; i < 4; ++i) { if (D->tok_ring[i]) cudaFreeHost(D->tok_ring[i]); if (D->tok_event[i]) cudaEventDestroy(D->tok_event[i]); }
    void* ptrs[] = {D->pos, D->cur_tok, D->cur_val, D->prompt_len, D->prompt_tok, D->gen_log, D->block_table, D->kv_pool, D->hbuf[0], D->hbuf[1], D->qkv,
                    D->attn_out, D->proj, D->act, D->logits, D->part_o, D->part_ml, D->attn_ticket, D->row_seq, D->row_pos,
                    D->rope_cos[0], D->rope_sin[0], D->rope_cos[1], D->rope_sin[1]};
    for (void* p : ptrs) cudaFree(p);
    delete D;
}

void decoder_destroy_all() {
    for (uint32_t i = 0; i < MAX_DECODERS; ++i) if (g_dec[i]) { destroy(g_dec[i]); g_dec[i] = nullptr; }
}

#define DCU(x) do { cudaError_t e__ = (x); if (e__ != cudaSuccess) return fail(e__ == cudaErrorMemoryAllocation ? ADAMAH_ERR_MEMORY : ADAMAH_ERR_BACKEND, "%s: %s", #x, cudaGetErrorString(e__)); } while (0)

static bool is_global_layer(const adam_b200_decoder_desc& d, uint32_t L) { return d.global_every == 0 || (L + 1) % d.global_every == 0; }

static size_t kv_elem_size(const adam_b200_decoder_desc& d) { return d.kv_dtype == 1 ? 2 : 4; }

typedef void (*AttnKernel)(const float*, uint32_t, const float*, const float*, float, const float*, const float*, uint32_t, void*, KvGeom,
                           const int32_t*, const int32_t*, uint32_t, uint32_t, uint32_t, float, float, float*, float*, float*,
                           unsigned int*, uint32_t, uint32_t, const int32_t*, const int32_t*, uint32_t* STEP_TRACE_PARAM);

template <typename T, int GS>
static AttnKernel pick_attn_hd(uint32_t hd) {
    switch (hd) {
    case 32: return k_attention<T, GS, 32>;
    case 64: return k_attention<T, GS, 64>;
    case 128: return k_attention<T, GS, 128>;
    default: return k_attention<T, GS, 256>;
    }
}

template <typename T>
static int launch_attn_t(Decoder* D, uint32_t L, uint32_t batch, bool prefill = false) {
    const adam_b200_decoder_desc& d = D->d;
    KvGeom geo{d.n_layer, d.n_head_kv, d.head_dim, d.page_size, D->max_pages_per_seq, D->page_elems};
    const uint32_t gs = d.n_head / d.n_head_kv;
    // Query heads per CTA: one while that still leaves SMs idle (lowest latency; the CTAs
    // of a kv head re-read its rows from L2), the whole group once the grid is large.
    // Measured at the 1B shape (4 query heads on 1 kv head): up to three sequences are fastest with a CTA per query head, eight
    // sequences with two heads per CTA, 16 or more sequences and prefill chunks with the whole group per CTA (the rows of a kv
    // head are then read once instead of once per query head).
    static const uint32_t hpc_env = getenv("ADAM_B200_ATTN_HPC") ? (uint32_t)atoi(getenv("ADAM_B200_ATTN_HPC")) : 0u;
    const uint32_t work = batch * d.n_head;                    // CTAs per position split with one head each
    const uint32_t hpc_auto = work <= 12u ? 1u : (work <= 32u ? (gs >= 2u ? 2u : 1u) : gs);
    const uint32_t hpc = (hpc_env && gs % hpc_env == 0 && hpc_env <= 8u) ? hpc_env : hpc_auto;
    const uint32_t window = ((d.flags & 1u) && d.sliding_window > 0 && !is_global_layer(d, L)) ? d.sliding_window : 0;
    const size_t smem = ((size_t)hpc * d.head_dim + 2 * (size_t)d.head_dim + (size_t)8 * hpc * d.head_dim) * 4;
    const int which = is_global_layer(d, L) ? 1 : 0;
    const Layer& ly = D->layers[L];
    const uint32_t qkv_ld = (d.n_head + 2 * d.n_head_kv) * d.head_dim;
    dim3 grid(D->n_splits, d.n_head_kv * (gs / hpc), batch);
    // Chunks of 8 positions a CTA takes before another CTA joins: with few (sequence, head) pairs the SMs are idle and a
    // CTA's chain of dependent chunk loads is the attention's whole time, so the positions are spread thinly (one chunk
    // per warp); with many pairs the grid is full anyway and every extra CTA only repeats the query prologue.
    static const uint32_t cpc_env = getenv("ADAM_B200_ATTN_CPC") ? (uint32_t)atoi(getenv("ADAM_B200_ATTN_CPC")) : 0u;
    const uint32_t pairs = grid.y * grid.z;
    const uint32_t cpc = cpc_env ? cpc_env : (work <= 64u ? 8u : ATTN_CHUNKS_PER_CTA);
    (void)pairs;
    AttnKernel kern = hpc <= 1 ? pick_attn_hd<T, 1>(d.head_dim) : hpc <= 2 ? pick_attn_hd<T, 2>(d.head_dim)
                    : hpc <= 4 ? pick_attn_hd<T, 4>(d.head_dim) : pick_attn_hd<T, 8>(d.head_dim);
    // Few (sequence, head) pairs in flight (at most 12): the position splits of a pair form one thread-block cluster of 8 CTAs and merge
    // through shared memory (no partial results in global memory, no ticket, no last-CTA pass: 3 us less per launch at the
    // 1B shape).  A cluster covers any context, its CTAs taking more chunks each, so layers that may attend to more than
    // 2048 positions keep the wider grid of independent splits.  (Clusters of 16 were measured slower: they start later,
    // and so does every kernel behind them.)  ADAM_B200_ATTN_CLUSTER=0 turns the path off, =16 allows clusters of 16.
    static const int cluster_env = getenv("ADAM_B200_ATTN_CLUSTER") ? atoi(getenv("ADAM_B200_ATTN_CLUSTER")) : 8;
    static const uint32_t cluster_work = getenv("ADAM_B200_ATTN_CLUSTER_WORK") ? (uint32_t)atoi(getenv("ADAM_B200_ATTN_CLUSTER_WORK")) : 12u;
    const uint32_t reach = window ? (window < d.kv_cap ? window : d.kv_cap) : d.kv_cap;
    // The kernels behind a cluster launch start later (their prologues no longer overlap it); that costs more than the merge
    // saves once the o-proj behind it has more than about a megabyte of tiles to request (27B shape, 4-way shard: 2 % slower).
    const size_t o_bytes = (size_t)ly.m[MAT_O].rows * ly.m[MAT_O].cols * 9 / 16;
    if (cluster_env != 0 && !prefill && work <= cluster_work && reach <= 2048u && o_bytes <= (1u << 20)) {
        struct Known { AttnKernel k; unsigned cs; };
        static Known known[16]; static int n_known = 0;
        int cs = -1;
        for (int i = 0; i < n_known; ++i) if (known[i].k == kern) cs = (int)known[i].cs;
        const auto smem_for = [&](unsigned c) { return smem + (size_t)c * hpc * (d.head_dim + 4) * 4; };
        if (cs < 0) {
            cs = 0;
            const unsigned c_max = cluster_env == 16 ? 16u : 8u;
            if (c_max > 8 && cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) cudaGetLastError();
            for (unsigned c = c_max; c >= 8 && !cs; c >>= 1) {
                if (cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_for(c)) != cudaSuccess) { cudaGetLastError(); continue; }
                cudaLaunchConfig_t cfg = {};
                cfg.gridDim = dim3(c, grid.y, 1); cfg.blockDim = dim3(256); cfg.dynamicSmemBytes = smem_for(c);
                cudaLaunchAttribute at[1];
                at[0].id = cudaLaunchAttributeClusterDimension;
                at[0].val.clusterDim.x = c; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
                cfg.attrs = at; cfg.numAttrs = 1;
                int n = 0;
                if (cudaOccupancyMaxActiveClusters(&n, (const void*)kern, &cfg) != cudaSuccess) { cudaGetLastError(); continue; }
                if (n >= (int)(grid.y * grid.z)) cs = (int)c;
            }
            if (n_known < 16) { known[n_known].k = kern; known[n_known].cs = (unsigned)cs; ++n_known; }
        }
        if (cs > 0) {
            grid.x = (unsigned)cs;
            if (launch_k_cluster(kern, grid, dim3(256), smem_for((unsigned)cs), g.stream, g.pdl, (unsigned)cs, D->qkv, qkv_ld, ly.norm[NORM_Q], ly.norm[NORM_K], d.norm_eps,
                                 D->rope_cos[which], D->rope_sin[which], D->rope_pos[which],
                                 D->kv_pool, geo, D->block_table, D->pos, d.n_head, L, window, d.attn_scale,
                                 d.attn_softcap, D->attn_out, D->part_o, D->part_ml, D->attn_ticket, 0u, hpc | (cpc << 16),
                                 (const int32_t*)nullptr, (const int32_t*)nullptr, g.dev_err STEP_TRACE_ARG((g_step_trace && L == g_step_trace_layer) ? g_step_trace + 4 * 64 : nullptr)) != cudaSuccess)
                return fail(ADAMAH_ERR_BACKEND, "attention: cluster launch failed: %s", cudaGetErrorString(cudaGetLastError()));
            count_launch();
            return ADAMAH_OK;
        }
    }
    if (smem > 48 * 1024) DCU(cudaFuncSetAttribute((const void*)kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    launch_k(kern, grid, dim3(256), smem, g.stream, g.pdl, D->qkv, qkv_ld, ly.norm[NORM_Q], ly.norm[NORM_K], d.norm_eps,
             D->rope_cos[which], D->rope_sin[which], D->rope_pos[which],
             D->kv_pool, geo, D->block_table, D->pos, d.n_head, L, window, d.attn_scale,
             d.attn_softcap, D->attn_out, D->part_o, D->part_ml, D->attn_ticket, D->n_splits, hpc | (cpc << 16),
             prefill ? D->row_seq : nullptr, prefill ? D->row_pos : nullptr, g.dev_err STEP_TRACE_ARG((g_step_trace && L == g_step_trace_layer && !prefill) ? g_step_trace + 4 * 64 : nullptr));
    count_launch();
    return ADAMAH_OK;
}

// The embedding kernel takes a full dependency on everything before it (no programmatic launch): later kernels
// of the step rely on the previous step's position update and cache writes being complete before any of them starts.
static void launch_embed(Decoder* D, uint32_t rows, const int32_t* row_seq, const int32_t* row_pos) {
    const adam_b200_decoder_desc& d = D->d;
    auto go = [&](auto kern) {
        launch_k(kern, dim3(rows), dim3(256), 0, g.stream, false, D->embd.w, d.n_embd, D->embd.rows, d.emb_scale, D->pos, D->prompt_len, D->prompt_tok,
                 d.kv_cap, D->cur_tok, D->hbuf[0], row_seq, row_pos, g.dev_err);
    };
    switch (D->embd.wtype) {
    case WT_Q4_0: go(k_embed<WT_Q4_0>); break;
    case WT_Q4_K: go(k_embed<WT_Q4_K>); break;
    case WT_Q8_0: go(k_embed<WT_Q8_0>); break;
    default:      go(k_embed<WT_Q5_0>); break;
    }
    count_launch();
}

static int gemv(const Mat& m, const Mat* m2, GemvArgs a, int B, int epi) {
#ifdef ADAM_B200_STEP_TRACE
    if (g_step_trace && g_step_trace_slot >= 0) { a.trace = g_step_trace + 64 * g_step_trace_slot; g_step_trace_slot = -1; }
#endif
    a.w0 = m.w; if (m2) a.w1 = m2->w;
    a.N = (int)m.rows; a.K = (int)m.cols; a.B = B; a.epi = epi;
    if (B >= TC_MIN_ROWS && (!m2 || m2->wtype == m.wtype) && gemm_tc_supports(m.wtype, a)) return launch_gemm_tc(m.wtype, a, g.stream);
    if (m.tiled && (!m2 || (m2->tiled && m2->wtype == m.wtype)) && gemv_mma_supports(m.wtype, a))
        return launch_gemv_mma(m.wtype, m.tiled, m2 ? m2->tiled : nullptr, a, g.stream);
    return launch_gemv(m.wtype, a, g.stream);
}

// Enqueue one token step for `batch` sequences on the context stream.  Five
// kernels per layer: QKV GEMV (input RMSNorm and, past layer 0, the previous
// layer's post-FFN norm + residual folded into its prologue), attention (QK-norm,
// RoPE, KV append folded in), o-proj GEMV, gate/up GEMV (post-attention norm +
// residual + FFN norm in the prologue, GeGLU in the epilogue), down GEMV.  The
// residual stream alternates between two buffers because a prologue's CTA 0
// writes the updated stream while the other CTAs still read the old one.
static int enqueue_step_impl(Decoder* D, uint32_t batch, bool with_lm, bool want_logits);
static int enqueue_step(Decoder* D, uint32_t batch, bool with_lm, bool want_logits) {
    static const bool allow = !(getenv("ADAM_B200_PDL") && atoi(getenv("ADAM_B200_PDL")) == 0);
    g.pdl = allow;
    const int rc = enqueue_step_impl(D, batch, with_lm, want_logits);
    g.pdl = false;
    return rc;
}
// One part of a token step.  Parts 2L and 2L+1 are the attention half (embedding for L = 0,
// QKV, attention, o-proj) and the FFN half (gate/up, down) of layer L; part 2*n_layer is the
// LM head, part 2*n_layer + 1 advances the positions.  A tensor-parallel caller all-reduces
// `proj` after every layer part and merges the arg-max pairs after the LM-head part.
static uint32_t n_parts(const Decoder* D) { return 2 * D->d.n_layer + 2; }
static int enqueue_part(Decoder* D, uint32_t batch, uint32_t part, bool with_lm, bool want_logits) {
    const adam_b200_decoder_desc& d = D->d;
    const uint32_t E = d.n_embd, q_dim = d.n_head * d.head_dim, k_dim = d.n_head_kv * d.head_dim, qkv_ld = q_dim + 2 * k_dim;
    int rc;
    if (part < 2 * d.n_layer && !(part & 1u)) {
        const uint32_t L = part / 2;
        const Layer& ly = D->layers[L];
        if (L == 0) launch_embed(D, batch, nullptr, nullptr);
        const int cur = L == 0 ? 0 : 1;             // residual stream buffer on entry
        GemvArgs in = {};
        in.ldx = (int)E; in.eps = d.norm_eps; in.h_in = D->hbuf[cur]; in.w_pre = ly.norm[NORM_ATTN];
        if (L > 0) { in.add_src = D->proj; in.w_post = D->layers[L - 1].norm[NORM_POST_FFW]; in.h_out = D->hbuf[cur ^ 1]; }
        in.y = D->qkv; in.ldy = (int)qkv_ld;
        if (ly.qkv_contiguous) {
            Mat qkv = ly.m[MAT_Q]; qkv.rows = qkv_ld; qkv.tiled = ly.qkv_tiled;
#ifdef ADAM_B200_STEP_TRACE
            if (L == g_step_trace_layer) g_step_trace_slot = 0;
#endif
            if ((rc = gemv(qkv, nullptr, in, batch, EPI_STORE))) return rc;
        } else {
            if ((rc = gemv(ly.m[MAT_Q], nullptr, in, batch, EPI_STORE))) return rc;
            GemvArgs in2 = in; in2.h_out = nullptr;
            in2.y = D->qkv + q_dim;
            if ((rc = gemv(ly.m[MAT_K], nullptr, in2, batch, EPI_STORE))) return rc;
            in2.y = D->qkv + q_dim + k_dim;
            if ((rc = gemv(ly.m[MAT_V], nullptr, in2, batch, EPI_STORE))) return rc;
        }
        rc = d.kv_dtype == 1 ? launch_attn_t<__half>(D, L, batch) : launch_attn_t<float>(D, L, batch);
        if (rc) return rc;
        GemvArgs o = {};
        o.x = D->attn_out; o.ldx = (int)q_dim; o.y = D->proj; o.ldy = (int)E;
#ifdef ADAM_B200_STEP_TRACE
        if (L == g_step_trace_layer) g_step_trace_slot = 1;
#endif
        if ((rc = gemv(ly.m[MAT_O], nullptr, o, batch, EPI_STORE))) return rc;
    } else if (part < 2 * d.n_layer) {
        const Layer& ly = D->layers[part / 2];
        // the stream is in buffer 0 here for every layer (layer 0 never flipped, the others flipped in their QKV)
        GemvArgs gu = {};
        gu.ldx = (int)E; gu.eps = d.norm_eps; gu.h_in = D->hbuf[0]; gu.add_src = D->proj; gu.w_post = ly.norm[NORM_POST_ATTN];
        gu.w_pre = ly.norm[NORM_FFN]; gu.h_out = D->hbuf[1]; gu.y = D->act; gu.ldy = (int)d.n_ff;
#ifdef ADAM_B200_STEP_TRACE
        if (part / 2 == g_step_trace_layer) g_step_trace_slot = 2;
#endif
        if ((rc = gemv(ly.m[MAT_GATE], &ly.m[MAT_UP], gu, batch, d.ffn_act == 0 ? EPI_GEGLU : EPI_SWIGLU))) return rc;
        GemvArgs dn = {};
        dn.x = D->act; dn.ldx = (int)d.n_ff; dn.y = D->proj; dn.ldy = (int)E;
#ifdef ADAM_B200_STEP_TRACE
        if (part / 2 == g_step_trace_layer) g_step_trace_slot = 3;
#endif
        if ((rc = gemv(ly.m[MAT_DOWN], nullptr, dn, batch, EPI_STORE))) return rc;
    } else if (part == 2 * d.n_layer) {
        if (with_lm) {
            const Mat& lm = D->output.bound ? D->output : D->embd;
            if (wt_is_b8(lm.wtype)) {
                // Q8_0 / Q5_0 LM head: the norm chain, the products and the arg-max as three kernels; the products land
                // in the logits buffer (soft-capped afterwards only when the caller wants them)
                if ((rc = launch_chain_rows(D->hbuf[1], D->proj, D->layers[d.n_layer - 1].norm[NORM_POST_FFW], D->output_norm, D->hbuf[0], D->act,
                                            (int)E, (int)batch, d.norm_eps, g.stream, g.pdl))) return rc;
                if ((rc = launch_gemv_b8(lm.wtype, lm.w, D->act, (int)E, D->logits, (int)lm.rows, (int)lm.rows, (int)E, (int)batch, g.stream))) return rc;
                if ((rc = launch_argmax_rows(D->logits, (int)lm.rows, (int)batch, d.final_softcap, want_logits, D->cur_tok, D->cur_val, nullptr, g.stream, false))) return rc;
                D->h_final = 0;
                return check_launch("decoder step");
            }
            GemvArgs a = {};
            a.ldx = (int)E; a.eps = d.norm_eps; a.h_in = D->hbuf[1]; a.add_src = D->proj;
            a.w_post = D->layers[d.n_layer - 1].norm[NORM_POST_FFW]; a.w_pre = D->output_norm; a.h_out = D->hbuf[0];
            a.y = want_logits ? D->logits : nullptr; a.ldy = (int)lm.rows; a.softcap = d.final_softcap;
            a.out_tok = D->cur_tok; a.out_val = D->cur_val;
            if ((rc = argmax_scratch(&a.part_val, &a.part_idx, &a.ticket))) return rc;
            if ((rc = gemv(lm, nullptr, a, batch, EPI_ARGMAX))) return rc;
            D->h_final = 0;
        }
    } else {
        launch_k(k_advance, dim3((batch + 63) / 64), dim3(64), 0, g.stream, g.pdl, D->pos, D->cur_tok, D->gen_log, d.kv_cap, batch, with_lm ? 1 : 0);
        count_launch();
    }
    return check_launch("decoder step");
}

static int enqueue_step_impl(Decoder* D, uint32_t batch, bool with_lm, bool want_logits) {
    for (uint32_t part = 0; part < n_parts(D); ++part) {
        const int rc = enqueue_part(D, batch, part, with_lm, want_logits);
        if (rc) return rc;
    }
    return ADAMAH_OK;
}

static int validate_bound(Decoder* D) {
    const adam_b200_decoder_desc& d = D->d;
    if (!D->embd.bound) return fail(ADAMAH_ERR_INVALID, "decoder: token_embd is not bound");
    if (!D->output_norm) return fail(ADAMAH_ERR_INVALID, "decoder: output_norm is not bound");
    if (!D->rope_cos[0] || !D->rope_cos[1]) return fail(ADAMAH_ERR_INVALID, "decoder: rotary tables are not set");
    for (uint32_t L = 0; L < d.n_layer; ++L) {
        Layer& ly = D->layers[L];
        for (int k = 0; k < 7; ++k) if (!ly.m[k].bound) return fail(ADAMAH_ERR_INVALID, "decoder: layer %u matrix %d is not bound", L, k);
        if (!ly.norm[NORM_ATTN] || !ly.norm[NORM_FFN]) return fail(ADAMAH_ERR_INVALID, "decoder: layer %u pre-norms are not bound", L);
        // q, k, v stored back to back -> one wider GEMV (adam/models/engine.py:1612-1661)
        const Mat &q = ly.m[MAT_Q], &k = ly.m[MAT_K], &v = ly.m[MAT_V];
        const size_t ipr = q.cols / (q.wtype == WT_Q4_0 ? 32 : 256) * (q.wtype == WT_Q4_0 ? 1 : 9);   // uint4 per row
        ly.qkv_contiguous = q.wtype == k.wtype && k.wtype == v.wtype && k.w.q == q.w.q + (size_t)q.rows * ipr &&
                            v.w.q == k.w.q + (size_t)k.rows * ipr;
        if (ly.qkv_contiguous && D->use_tiles && !ly.qkv_tiled) {
            const uint32_t rows = q.rows + k.rows + v.rows;
            if (rows % 16 == 0 && q.cols % 64 == 0 && tile_tensor(q.map_id, q.elem_off, rows, q.cols) == ADAMAH_OK)
                ly.qkv_tiled = (const uint8_t*)find_tiled(q.map_id, q.elem_off, rows, q.cols);
        }
    }
    return ADAMAH_OK;
}

// ---- single-launch token kernel: eligibility, work split, buffers -----------------------------

// Spread one product over the grid (see TkPhase): the estimate is the number of tile pairs the busiest
// warp walks plus fixed costs per row group, per K split inside the CTA and per K split across CTAs.
static bool tk_pick_phase(TkPhase& P, int n_rg, int pairs, int nm, int grid, int max_cpr) {
    double best = 1e300;
    bool found = false;
    for (int cpr = 1; cpr <= max_cpr; ++cpr) {
        for (int KS = 1; KS <= TK_NW; ++KS) {
            const int RG = TK_NW / KS;
            if (RG < 1 || KS * cpr > pairs) continue;
            if (KS > 1 && RG > 15) continue;                   // named barriers 1..15
            const int n_sets = (n_rg + RG - 1) / RG;
            int G = grid / cpr;
            if (G > n_sets) G = n_sets;
            if (G < 1) continue;
            const int sets_per_cta = (n_sets + G - 1) / G;
            const int per_warp = (pairs + KS * cpr - 1) / (KS * cpr);
            const double cost = (double)sets_per_cta * (per_warp * nm + 2.0) + (KS > 1 ? 1.0 : 0.0) + (cpr > 1 ? 1.0 : 0.0) + 0.01 * KS;
            if (cost < best) { best = cost; P.n_rg = n_rg; P.pairs = pairs; P.RG = RG; P.KS = KS; P.cpr = cpr; P.G = G; found = true; }
        }
    }
    return found;
}

static int prepare_token_kernel(Decoder* D) {
    const adam_b200_decoder_desc& d = D->d;
    D->tk_state = -1;
    static const bool allow = !(getenv("ADAM_B200_TOKEN_KERNEL") && atoi(getenv("ADAM_B200_TOKEN_KERNEL")) == 0);
    if (!allow || !D->use_tiles || d.tp_size > 1) return ADAMAH_OK;
    int coop = 0;
    cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, g.device);
    if (!coop) return ADAMAH_OK;
    const uint32_t E = d.n_embd, q_dim = d.n_head * d.head_dim, k_dim = d.n_head_kv * d.head_dim, FF = d.n_ff;
    if (!token_supported_hd((int)d.head_dim) || d.n_layer > (uint32_t)TK_MAX_LAYERS || d.page_size % 8) return ADAMAH_OK;
    if (E % 64 || q_dim % 64 || FF % 64 || E > (uint32_t)TK_MAX_E || q_dim > 2u * TK_THREADS * 4u) return ADAMAH_OK;
    const Mat& lm = D->output.bound ? D->output : D->embd;
    if (!lm.tiled || lm.rows % 16) return ADAMAH_OK;
    if (wt_is_b8(D->embd.wtype) || wt_is_b8(lm.wtype)) return ADAMAH_OK;     // Q8_0 / Q5_0 tables run on the chain of kernels
    const int wt = lm.wtype;
    if (wt == WT_Q4_K && (E % 256 || q_dim % 256 || FF % 256)) return ADAMAH_OK;
    auto al16 = [](const void* p) { return ((uintptr_t)p & 15u) == 0; };
    if (!al16(D->output_norm)) return ADAMAH_OK;
    for (uint32_t L = 0; L < d.n_layer; ++L) {
        const Layer& ly = D->layers[L];
        if (!ly.qkv_contiguous || !ly.qkv_tiled || !ly.m[MAT_O].tiled || !ly.m[MAT_GATE].tiled || !ly.m[MAT_UP].tiled || !ly.m[MAT_DOWN].tiled) return ADAMAH_OK;
        for (int k : {MAT_Q, MAT_O, MAT_GATE, MAT_UP, MAT_DOWN}) if (ly.m[k].wtype != wt) return ADAMAH_OK;
        for (int k : {NORM_ATTN, NORM_POST_ATTN, NORM_FFN, NORM_POST_FFW}) if (!al16(ly.norm[k])) return ADAMAH_OK;
    }
    TkArgs a = {};
    // the gate/up product decides the grid: every CTA must take part in it (it is what makes each CTA's
    // reads a precondition of the next layer, see token_kernel.cuh), so a product with fewer sets than SMs
    // shrinks the grid instead
    int grid = g.sm_count;
    {
        TkPhase best = {}; double best_cost = 1e300; int best_grid = 0;
        for (int KS = 1; KS <= TK_NW; ++KS) {
            const int RG = TK_NW / KS, pairs = (int)E / 64, n_rg = (int)FF / 16;
            if (KS > pairs || (KS > 1 && RG > 15)) continue;
            const int n_sets = (n_rg + RG - 1) / RG;
            const int gr = n_sets < g.sm_count ? n_sets : g.sm_count;
            const int sets_per_cta = (n_sets + gr - 1) / gr;
            const int per_warp = (pairs + KS - 1) / KS;
            // idle SMs cost LM-head bandwidth: weigh them in
            const double cost = ((double)sets_per_cta * (per_warp * 2 + 2.0) + (KS > 1 ? 1.0 : 0.0) + 0.01 * KS) * (1.0 + 2.0 * (g.sm_count - gr) / (double)g.sm_count);
            if (cost < best_cost) { best_cost = cost; best_grid = gr; best.n_rg = n_rg; best.pairs = pairs; best.RG = RG; best.KS = KS; best.cpr = 1; best.G = gr; }
        }
        if (best_grid < 1) return ADAMAH_OK;
        grid = best_grid;
        a.ph[TK_GU] = best;
    }
    if (grid < (int)d.n_head) return ADAMAH_OK;
    if (!tk_pick_phase(a.ph[TK_QKV], (int)(q_dim + 2 * k_dim) / 16, (int)E / 64, 1, grid, 1)) return ADAMAH_OK;
    if (!tk_pick_phase(a.ph[TK_O], (int)E / 16, (int)q_dim / 64, 1, grid, 1)) return ADAMAH_OK;
    if (!tk_pick_phase(a.ph[TK_DOWN], (int)E / 16, (int)FF / 64, 1, grid, 2)) return ADAMAH_OK;
    if (!tk_pick_phase(a.ph[TK_LM], (int)lm.rows / 16, (int)E / 64, 1, grid, 1)) return ADAMAH_OK;
    // attention CTAs per query head: what the grid offers, at most 8192 gathered values per o-proj CTA
    a.s_max = grid / (int)d.n_head;
    if (a.s_max > TK_MAX_SPLITS) a.s_max = TK_MAX_SPLITS;
    if (a.s_max > 4) a.s_max = 4;                         // the o-proj merges up to four splits in one poll
    {   // per-warp staging regions of the o-proj and down-proj inputs: the widest K slice of a warp
        int np = 0;
        for (int ph : {TK_O, TK_DOWN}) {
            const TkPhase& P = a.ph[ph];
            const int n = (P.pairs + P.KS * P.cpr - 1) / (P.KS * P.cpr);
            if (n > np) np = n;
        }
        if (np > 8) return ADAMAH_OK;                     // a warp's slice must fit sixteen loads per lane
        a.wu_cap = 2 * np;
    }
    a.n_layer = (int)d.n_layer; a.E = (int)E; a.q_dim = (int)q_dim; a.k_dim = (int)k_dim; a.FF = (int)FF; a.V = (int)lm.rows;
    a.H = (int)d.n_head; a.KV = (int)d.n_head_kv;
    a.embd = D->embd.w; a.embd_wt = D->embd.wtype; a.emb_scale = d.emb_scale;
    a.lm_tiled = lm.tiled; a.out_norm = D->output_norm;
    a.eps = d.norm_eps; a.attn_scale = d.attn_scale; a.attn_cap = d.attn_softcap; a.final_cap = d.final_softcap; a.act = (int)d.ffn_act;
    a.pos = D->pos; a.cur_tok = D->cur_tok; a.cur_val = D->cur_val; a.prompt_len = D->prompt_len; a.prompt_tok = D->prompt_tok;
    a.gen_log = D->gen_log; a.log_ld = d.kv_cap;
    a.block_table = D->block_table;
    a.geo = KvGeom{d.n_layer, d.n_head_kv, d.head_dim, d.page_size, D->max_pages_per_seq, D->page_elems};
    a.kv_pool = D->kv_pool;
    for (int w = 0; w < 2; ++w) { a.cos_t[w] = D->rope_cos[w]; a.sin_t[w] = D->rope_sin[w]; }
    a.n_pos = D->rope_pos[0] < D->rope_pos[1] ? D->rope_pos[0] : D->rope_pos[1];
    a.h_out = D->hbuf[0];
    a.err = g.dev_err;
    if (token_smem_bytes(wt, a, (int)d.head_dim) > 220 * 1024) return ADAMAH_OK;
    // device memory: layer table, exchange buffers (two halves each), step counter and the sticky word
    std::vector<TkLayer> hl(d.n_layer);
    for (uint32_t L = 0; L < d.n_layer; ++L) {
        const Layer& ly = D->layers[L];
        TkLayer& t = hl[L];
        t.w[0] = ly.qkv_tiled; t.w[1] = ly.m[MAT_O].tiled; t.w[2] = ly.m[MAT_GATE].tiled; t.w[3] = ly.m[MAT_UP].tiled; t.w[4] = ly.m[MAT_DOWN].tiled;
        t.norm[TKN_ATTN] = ly.norm[NORM_ATTN]; t.norm[TKN_POST_ATTN] = ly.norm[NORM_POST_ATTN]; t.norm[TKN_FFN] = ly.norm[NORM_FFN];
        t.norm[TKN_POST_FFW] = ly.norm[NORM_POST_FFW]; t.norm[TKN_Q] = ly.norm[NORM_Q]; t.norm[TKN_K] = ly.norm[NORM_K];
        t.window = ((d.flags & 1u) && d.sliding_window > 0 && !is_global_layer(d, L)) ? d.sliding_window : 0;
        t.rope = is_global_layer(d, L) ? 1u : 0u;
    }
    const size_t sizes[9] = {
        hl.size() * sizeof(TkLayer),
        2 * (size_t)(q_dim + 2 * k_dim) * 8,
        2 * (size_t)d.n_head * a.s_max * (d.head_dim + 2) * 8,
        2 * (size_t)a.ph[TK_O].cpr * E * 8,
        2 * (size_t)FF * 8,
        2 * (size_t)a.ph[TK_DOWN].cpr * E * 8,
        2 * (size_t)grid * 8,
        4, 4};
    for (int i = 0; i < 9; ++i) {
        if (cudaMalloc(&D->tk_mem[i], sizes[i]) != cudaSuccess) {
            cudaGetLastError();
            for (void*& m : D->tk_mem) { if (m) cudaFree(m); m = nullptr; }
            return fail(ADAMAH_ERR_MEMORY, "decoder: out of device memory for the token kernel's buffers");
        }
        cudaMemsetAsync(D->tk_mem[i], 0, sizes[i], g.stream);
    }
    cudaMemcpyAsync(D->tk_mem[0], hl.data(), sizes[0], cudaMemcpyHostToDevice, g.stream);
    cudaStreamSynchronize(g.stream);
    a.layers = (const TkLayer*)D->tk_mem[0];
    a.x_qkv = (uint2*)D->tk_mem[1]; a.x_att = (uint2*)D->tk_mem[2]; a.x_po = (uint2*)D->tk_mem[3]; a.x_act = (uint2*)D->tk_mem[4];
    a.x_pd = (uint2*)D->tk_mem[5]; a.x_amax = (uint2*)D->tk_mem[6]; a.seq = (uint32_t*)D->tk_mem[7]; a.dead = (uint32_t*)D->tk_mem[8];
    D->tk = a; D->tk_grid = grid; D->tk_wt = wt;
    D->tk_state = 1;
    return ADAMAH_OK;
}

static long long* g_tk_trace = nullptr;     // diagnostics buffer (device), see adam_b200_decoder_token_trace
static int g_tk_trace_layer = 0, g_tk_trace_phase = 2;

// One token of the single active sequence as one launch.
static int enqueue_token(Decoder* D, bool with_lm, bool want_logits) {
    TkArgs a = D->tk;
    a.trace = g_tk_trace; a.trace_layer = g_tk_trace_layer; a.trace_phase = g_tk_trace_phase;
    a.with_lm = with_lm ? 1 : 0;
    a.logits = want_logits ? D->logits : nullptr;
    const int rc = launch_token(D->tk_wt, D->d.kv_dtype == 1, (int)D->d.head_dim, a, D->tk_grid, g.stream);
    if (rc == ADAMAH_OK && with_lm) D->h_final = 0;
    return rc;
}

}  // namespace ab

using namespace ab;

extern "C" int adam_b200_decoder_create(const adam_b200_decoder_desc* desc, uint32_t* id_out) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    if (!desc || !id_out) return fail(ADAMAH_ERR_INVALID, "decoder_create: null argument");
    adam_b200_decoder_desc d = *desc;
    if (!d.n_layer || !d.n_embd || !d.n_head || !d.n_head_kv || !d.head_dim || !d.n_ff || !d.n_vocab || !d.max_batch || !d.kv_cap)
        return fail(ADAMAH_ERR_INVALID, "decoder_create: zero dimension");
    if (d.n_head % d.n_head_kv || d.n_head / d.n_head_kv > 8) return fail(ADAMAH_ERR_INVALID, "decoder_create: unsupported GQA group");
    if (d.head_dim != 32 && d.head_dim != 64 && d.head_dim != 128 && d.head_dim != 256)
        return fail(ADAMAH_ERR_INVALID, "decoder_create: head_dim must be 32, 64, 128 or 256");
    if (d.n_embd % 32 || d.n_ff % 32) return fail(ADAMAH_ERR_INVALID, "decoder_create: widths must be multiples of 32");
    if (d.kv_dtype > 1) return fail(ADAMAH_ERR_INVALID, "decoder_create: kv_dtype must be 0 (f32) or 1 (f16)");
    if (d.page_size == 0) d.page_size = 64;
    if (d.attn_scale == 0.f) d.attn_scale = 1.0f / sqrtf((float)d.head_dim);
    uint32_t id = MAX_DECODERS;
    for (uint32_t i = 0; i < MAX_DECODERS; ++i) if (!g_dec[i]) { id = i; break; }
    if (id == MAX_DECODERS) return fail(ADAMAH_ERR_MEMORY, "decoder table full");
    Decoder* D = new Decoder();
    D->d = d;
    D->use_tiles = !(d.flags & 2u);
    D->layers.resize(d.n_layer);
    D->max_pages_per_seq = (d.kv_cap + d.page_size - 1) / d.page_size;
    D->n_pages = d.n_pages ? d.n_pages : D->max_pages_per_seq * d.max_batch;
    D->d.n_pages = D->n_pages;
    D->page_elems = (size_t)d.n_layer * 2 * d.n_head_kv * d.page_size * d.head_dim;
    D->n_splits = (d.kv_cap + ATTN_SPLIT - 1) / ATTN_SPLIT;      // ATTN_SPLIT = ATTN_CP * ATTN_CHUNKS_PER_CTA
    if (D->n_splits > ATTN_MAX_SPLITS) D->n_splits = ATTN_MAX_SPLITS;
    D->rows_cap = d.max_batch > PREFILL_ROWS ? d.max_batch : PREFILL_ROWS;
    gemm_tc_prepare();                          // workspace of the many-row GEMM (without it those rows run on the GEMV kernels)
    const size_t B = d.max_batch, R = D->rows_cap, E = d.n_embd, q_dim = (size_t)d.n_head * d.head_dim, k_dim = (size_t)d.n_head_kv * d.head_dim;
    const uint32_t gs = d.n_head / d.n_head_kv;
    g_dec[id] = D;
#define DALLOC(p, bytes) do { cudaError_t e__ = cudaMalloc((void**)&(p), (bytes)); if (e__ != cudaSuccess) { destroy(D); g_dec[id] = nullptr; \
        return fail(ADAMAH_ERR_MEMORY, "decoder_create: cudaMalloc(%zu) failed: %s", (size_t)(bytes), cudaGetErrorString(e__)); } } while (0)
    DALLOC(D->pos, B * 4); DALLOC(D->cur_tok, B * 4); DALLOC(D->cur_val, B * 4); DALLOC(D->prompt_len, B * 4);
    DALLOC(D->prompt_tok, B * d.kv_cap * 4); DALLOC(D->gen_log, B * d.kv_cap * 4);
    DALLOC(D->block_table, B * D->max_pages_per_seq * 4);
    DALLOC(D->kv_pool, (size_t)D->n_pages * D->page_elems * kv_elem_size(d));
    DALLOC(D->hbuf[0], R * E * 4); DALLOC(D->hbuf[1], R * E * 4); DALLOC(D->qkv, R * (q_dim + 2 * k_dim) * 4);
    DALLOC(D->attn_out, R * q_dim * 4); DALLOC(D->proj, R * E * 4);
    DALLOC(D->act, R * d.n_ff * 4); DALLOC(D->logits, B * (size_t)d.n_vocab * 4);
    DALLOC(D->part_o, R * d.n_head_kv * D->n_splits * gs * d.head_dim * 4);
    DALLOC(D->part_ml, R * d.n_head_kv * D->n_splits * gs * 2 * 4);
    DALLOC(D->attn_ticket, R * d.n_head * 4);
    DALLOC(D->row_seq, R * 4); DALLOC(D->row_pos, R * 4);
#undef DALLOC
    cudaMemsetAsync(D->attn_ticket, 0, R * d.n_head * 4, g.stream);
    cudaMemsetAsync(D->pos, 0, B * 4, g.stream);
    cudaMemsetAsync(D->cur_tok, 0, B * 4, g.stream);
    cudaMemsetAsync(D->cur_val, 0, B * 4, g.stream);
    cudaMemsetAsync(D->prompt_len, 0, B * 4, g.stream);
    cudaMemsetAsync(D->kv_pool, 0, (size_t)D->n_pages * D->page_elems * kv_elem_size(d), g.stream);
    k_fill_i32<<<(unsigned)((B * D->max_pages_per_seq + 255) / 256), 256, 0, g.stream>>>(D->block_table, -1, B * D->max_pages_per_seq);
    cudaStreamSynchronize(g.stream);
    for (uint32_t p = 0; p < D->n_pages; ++p) D->free_pages.push_back(D->n_pages - 1 - p);
    *id_out = id;
    return ADAMAH_OK;
}

extern "C" int adam_b200_decoder_destroy(uint32_t id) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    destroy(D);
    g_dec[id] = nullptr;
    return ADAMAH_OK;
}

extern "C" int adam_b200_decoder_bind_matrix(uint32_t id, uint32_t layer, uint32_t kind, uint32_t map_wt, uint64_t elem_off,
                                             uint32_t rows, uint32_t cols) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    Map* m = get_map(map_wt);
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (kind >= MAT_KINDS || (kind < MAT_EMBD && layer >= D->d.n_layer)) return fail(ADAMAH_ERR_INVALID, "bind_matrix: bad layer/kind");
    const adam_b200_decoder_desc& d = D->d;
    const uint32_t q_dim = d.n_head * d.head_dim, k_dim = d.n_head_kv * d.head_dim;
    const uint32_t want_r[MAT_KINDS] = {q_dim, k_dim, k_dim, d.n_embd, d.n_ff, d.n_ff, d.n_embd, d.n_vocab, d.n_vocab};
    const uint32_t want_c[MAT_KINDS] = {d.n_embd, d.n_embd, d.n_embd, q_dim, d.n_embd, d.n_embd, d.n_ff, d.n_embd, d.n_embd};
    // A tensor-parallel shard looks tokens up in the whole embedding table while its LM head
    // (n_vocab) covers only the shard's vocabulary rows.
    const bool full_embd = kind == MAT_EMBD && d.tp_size > 1 && rows >= d.n_vocab && cols == d.n_embd;
    if (!full_embd && (rows != want_r[kind] || cols != want_c[kind]))
        return fail(ADAMAH_ERR_INVALID, "bind_matrix: kind %u expects [%u,%u], got [%u,%u]", kind, want_r[kind], want_c[kind], rows, cols);
    Mat mt = {};
    int rc = weight_ref(m, elem_off, (uint64_t)rows * cols, &mt.wtype, &mt.w);
    if (rc) return rc;
    if (mt.wtype == WT_Q4_K && cols % 256) return fail(ADAMAH_ERR_INVALID, "bind_matrix: Q4_K needs cols %% 256 == 0");
    if (wt_is_b8(mt.wtype) && ((kind != MAT_EMBD && kind != MAT_OUTPUT) || d.tp_size > 1 || d.n_ff < d.n_embd))
        return fail(ADAMAH_ERR_INVALID, "bind_matrix: Q8_0 / Q5_0 blocks are accepted for token_embd and output, on one GPU, with n_ff >= n_embd");
    mt.rows = rows; mt.cols = cols; mt.bound = true; mt.map_id = map_wt; mt.elem_off = elem_off; mt.tiled = nullptr;
    // q, k, v get one combined tiled copy later (validate_bound); token_embd is tiled only as the LM head
    const bool solo = kind == MAT_O || kind == MAT_GATE || kind == MAT_UP || kind == MAT_DOWN || kind == MAT_OUTPUT || kind == MAT_EMBD;
    if (D->use_tiles && solo && !wt_is_b8(mt.wtype) && rows % 16 == 0 && cols % 64 == 0) {
        if (tile_tensor(map_wt, elem_off, rows, cols) == ADAMAH_OK) mt.tiled = (const uint8_t*)find_tiled(map_wt, elem_off, rows, cols);
    }
    if (kind == MAT_EMBD) D->embd = mt; else if (kind == MAT_OUTPUT) D->output = mt; else D->layers[layer].m[kind] = mt;
    free_graphs(D);
    return ADAMAH_OK;
}

extern "C" int adam_b200_decoder_bind_norm(uint32_t id, uint32_t layer, uint32_t kind, uint32_t map_f32, uint64_t elem_off, uint32_t n) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    Map* m = get_map(map_f32);
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (m->dtype != ADAMAH_DTYPE_F32) return fail(ADAMAH_ERR_INVALID, "bind_norm: map %u is not float32", map_f32);
    if (kind >= NORM_KINDS || (kind != NORM_OUTPUT && layer >= D->d.n_layer)) return fail(ADAMAH_ERR_INVALID, "bind_norm: bad layer/kind");
    const uint32_t want = (kind == NORM_Q || kind == NORM_K) ? D->d.head_dim : D->d.n_embd;
    if (n != want) return fail(ADAMAH_ERR_INVALID, "bind_norm: kind %u expects %u weights, got %u", kind, want, n);
    if (elem_off + n > m->n_elems) return fail(ADAMAH_ERR_INVALID, "bind_norm: range beyond map %u", map_f32);
    const float* p = (const float*)m->buf + elem_off;
    if (kind == NORM_OUTPUT) D->output_norm = p; else D->layers[layer].norm[kind] = p;
    free_graphs(D);
    return ADAMAH_OK;
}

extern "C" int adam_b200_decoder_set_rope(uint32_t id, uint32_t which, const float* cos_t, const float* sin_t, uint32_t n_pos, uint32_t half) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (which > 1 || !cos_t || !sin_t || half != D->d.head_dim / 2 || n_pos < D->d.kv_cap)
        return fail(ADAMAH_ERR_INVALID, "set_rope: need which in {0,1}, half == head_dim/2 and n_pos >= kv_cap");
    cudaStreamSynchronize(g.stream);
    cudaFree(D->rope_cos[which]); cudaFree(D->rope_sin[which]);
    D->rope_cos[which] = D->rope_sin[which] = nullptr;
    const size_t bytes = (size_t)n_pos * half * 4;
    DCU(cudaMalloc((void**)&D->rope_cos[which], bytes));
    DCU(cudaMalloc((void**)&D->rope_sin[which], bytes));
    DCU(cudaMemcpy(D->rope_cos[which], cos_t, bytes, cudaMemcpyHostToDevice));
    DCU(cudaMemcpy(D->rope_sin[which], sin_t, bytes, cudaMemcpyHostToDevice));
    D->rope_pos[which] = n_pos;
    free_graphs(D);
    return ADAMAH_OK;
}

// Start `batch` sequences: prompts (ragged, concatenated) are copied to the
// device, positions reset to 0, and pages reserved for `reserve[b]` tokens each.
extern "C" int adam_b200_decoder_begin(uint32_t id, uint32_t batch, const int32_t* prompt_tokens, const uint32_t* prompt_lens,
                                       const uint32_t* reserve) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    const adam_b200_decoder_desc& d = D->d;
    if (batch == 0 || batch > d.max_batch || !prompt_lens || !reserve) return fail(ADAMAH_ERR_INVALID, "decoder_begin: bad batch");
    if (capturing()) return fail(ADAMAH_ERR_INVALID, "decoder_begin: not allowed while a graph is being captured");
    int rc = validate_bound(D);
    if (rc) return rc;
    DCU(cudaStreamSynchronize(g.stream));
    // return all pages, then reserve
    D->free_pages.clear();
    for (uint32_t p = 0; p < D->n_pages; ++p) D->free_pages.push_back(D->n_pages - 1 - p);
    std::vector<int32_t> bt((size_t)d.max_batch * D->max_pages_per_seq, -1), plen(d.max_batch, 0), ptok((size_t)batch * d.kv_cap, 0);
    size_t off = 0;
    for (uint32_t b = 0; b < batch; ++b) {
        if (prompt_lens[b] == 0 || prompt_lens[b] > d.kv_cap || reserve[b] < prompt_lens[b] || reserve[b] > d.kv_cap)
            return fail(ADAMAH_ERR_INVALID, "decoder_begin: sequence %u needs 1 <= prompt <= reserve <= kv_cap (%u)", b, d.kv_cap);
        const uint32_t need = (reserve[b] + d.page_size - 1) / d.page_size;
        if (need > D->free_pages.size()) return fail(ADAMAH_ERR_MEMORY, "decoder_begin: KV page pool exhausted (%u pages)", D->n_pages);
        for (uint32_t p = 0; p < need; ++p) { bt[(size_t)b * D->max_pages_per_seq + p] = (int32_t)D->free_pages.back(); D->free_pages.pop_back(); }
        plen[b] = (int32_t)prompt_lens[b];
        if (!prompt_tokens) return fail(ADAMAH_ERR_INVALID, "decoder_begin: null prompt");
        for (uint32_t t = 0; t < prompt_lens[b]; ++t) {
            const int32_t tk = prompt_tokens[off + t];
            if (tk < 0 || (uint32_t)tk >= D->embd.rows) return fail(ADAMAH_ERR_INVALID, "decoder_begin: token id %d outside the vocabulary", tk);
            ptok[(size_t)b * d.kv_cap + t] = tk;
        }
        off += prompt_lens[b];
    }
    DCU(cudaMemcpyAsync(D->block_table, bt.data(), bt.size() * 4, cudaMemcpyHostToDevice, g.stream));
    DCU(cudaMemcpyAsync(D->prompt_len, plen.data(), plen.size() * 4, cudaMemcpyHostToDevice, g.stream));
    DCU(cudaMemcpyAsync(D->prompt_tok, ptok.data(), ptok.size() * 4, cudaMemcpyHostToDevice, g.stream));
    DCU(cudaMemsetAsync(D->pos, 0, (size_t)d.max_batch * 4, g.stream));
    DCU(cudaMemsetAsync(D->cur_tok, 0, (size_t)d.max_batch * 4, g.stream));
    DCU(cudaMemsetAsync(D->gen_log, 0xFF, (size_t)d.max_batch * d.kv_cap * 4, g.stream));
    if (D->tk_state == 1) DCU(cudaMemsetAsync(D->tk_mem[8], 0, 4, g.stream));
    DCU(cudaStreamSynchronize(g.stream));
    D->batch = batch;
    D->hpos.assign(batch, 0);
    D->hplen.assign(prompt_lens, prompt_lens + batch);
    D->hres.assign(reserve, reserve + batch);
    D->hbt = bt;
    return ADAMAH_OK;
}

// Continue the single active sequence with a new prompt whose first n_reuse tokens are the ones
// whose keys and values are already in the cache (role of generate(reuse_prefix=..),
// adam/models/engine.py:3815-3833): positions restart at n_reuse, the cache pages are kept and
// extended to `reserve` tokens.  n_reuse must not exceed the positions computed so far.
extern "C" int adam_b200_decoder_continue(uint32_t id, const int32_t* prompt_tokens, uint32_t prompt_len, uint32_t reserve, uint32_t n_reuse) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    const adam_b200_decoder_desc& d = D->d;
    if (D->batch != 1) return fail(ADAMAH_ERR_INVALID, "decoder_continue: needs one active sequence");
    if (capturing()) return fail(ADAMAH_ERR_INVALID, "decoder_continue: not allowed while a graph is being captured");
    if (!prompt_tokens || prompt_len == 0 || prompt_len > d.kv_cap || reserve < prompt_len || reserve > d.kv_cap)
        return fail(ADAMAH_ERR_INVALID, "decoder_continue: needs 1 <= prompt <= reserve <= kv_cap (%u)", d.kv_cap);
    if (n_reuse >= prompt_len || n_reuse > D->hpos[0])
        return fail(ADAMAH_ERR_INVALID, "decoder_continue: %u reused positions, but %u are cached and the prompt has %u tokens", n_reuse, D->hpos[0], prompt_len);
    DCU(cudaStreamSynchronize(g.stream));
    std::vector<int32_t> ptok(prompt_len);
    for (uint32_t t = 0; t < prompt_len; ++t) {
        if (prompt_tokens[t] < 0 || (uint32_t)prompt_tokens[t] >= D->embd.rows) return fail(ADAMAH_ERR_INVALID, "decoder_continue: token id %d outside the vocabulary", prompt_tokens[t]);
        ptok[t] = prompt_tokens[t];
    }
    uint32_t have = 0;
    while (have < D->max_pages_per_seq && D->hbt[have] >= 0) ++have;
    const uint32_t need = (reserve + d.page_size - 1) / d.page_size;
    if (need > have) {
        if (need - have > D->free_pages.size()) return fail(ADAMAH_ERR_MEMORY, "decoder_continue: KV page pool exhausted (%u pages)", D->n_pages);
        for (uint32_t p = have; p < need; ++p) { D->hbt[p] = (int32_t)D->free_pages.back(); D->free_pages.pop_back(); }
        DCU(cudaMemcpyAsync(D->block_table, D->hbt.data(), (size_t)D->max_pages_per_seq * 4, cudaMemcpyHostToDevice, g.stream));
    }
    const int32_t plen = (int32_t)prompt_len, p0 = (int32_t)n_reuse;
    DCU(cudaMemcpyAsync(D->prompt_len, &plen, 4, cudaMemcpyHostToDevice, g.stream));
    DCU(cudaMemcpyAsync(D->prompt_tok, ptok.data(), (size_t)prompt_len * 4, cudaMemcpyHostToDevice, g.stream));
    DCU(cudaMemcpyAsync(D->pos, &p0, 4, cudaMemcpyHostToDevice, g.stream));
    DCU(cudaMemsetAsync(D->cur_tok, 0, 4, g.stream));
    DCU(cudaMemsetAsync(D->gen_log, 0xFF, (size_t)d.kv_cap * 4, g.stream));
    if (D->tk_state == 1) DCU(cudaMemsetAsync(D->tk_mem[8], 0, 4, g.stream));
    DCU(cudaStreamSynchronize(g.stream));
    D->hpos[0] = n_reuse;
    D->hplen[0] = prompt_len;
    D->hres[0] = reserve;
    return ADAMAH_OK;
}

// Run `n_steps` token steps.  flags bit0: run the LM head + arg-max (the sampled
// id feeds the next step once the prompt is consumed); bit1: also store the
// soft-capped logits; bit2: launch kernels directly instead of replaying a graph;
// bit4: draw the token with the rule of adam_b200_decoder_set_sampling instead of the arg-max;
// bit3: use the chain of per-operation kernels even where the single-launch token
// kernel (one sequence, row-tiled weights) would run.
// Returns without waiting unless called outside batch_begin/batch_end.
extern "C" int adam_b200_decoder_step(uint32_t id, uint32_t n_steps, uint32_t flags) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (D->batch == 0) return fail(ADAMAH_ERR_INVALID, "decoder_step: call decoder_begin first");
    const bool sample = (flags & 16u) != 0;
    const bool with_lm = flags & 1u, want_logits = (flags & 2u) != 0 || sample, direct = (flags & 4u) != 0, chain = (flags & 8u) != 0;
    if (want_logits && !with_lm) return fail(ADAMAH_ERR_INVALID, "decoder_step: logits need the LM head flag");
    if (sample && D->smp_k == 0) return fail(ADAMAH_ERR_INVALID, "decoder_step: call adam_b200_decoder_set_sampling before a sampled step");
    // the sampled token replaces the arg-max one right after every step (positions are already advanced)
    auto sample_step = [&]() -> int {
        if (!sample) return ADAMAH_OK;
        const Mat& lm = D->output.bound ? D->output : D->embd;
        return launch_sample(D->logits, lm.rows, D->batch, D->smp_k, D->smp_temp, D->smp_top_p, D->smp_penalty, D->smp_on_prompt, D->smp_seed,
                             D->pos, D->prompt_len, D->prompt_tok, D->gen_log, D->d.kv_cap, D->cur_tok, D->cur_val);
    };
    int rc = ADAMAH_OK;
    // a step past the reserved pages would only set a device error bit and return ids that look valid
    for (uint32_t b = 0; b < D->batch; ++b)
        if ((uint64_t)D->hpos[b] + n_steps > D->hres[b])
            return fail(ADAMAH_ERR_INVALID, "decoder_step: sequence %u is at position %u of %u reserved, cannot take %u more steps", b, D->hpos[b], D->hres[b], n_steps);
    for (uint32_t& hp : D->hpos) hp += n_steps;
    if (D->batch == 1 && !chain && D->tk_state == 0 && !capturing()) { if ((rc = prepare_token_kernel(D))) return rc; }
    if (D->batch == 1 && !chain && D->tk_state == 1 && !capturing()) {
        uint32_t s = 0;
        // Several steps at once replay a graph of TK_GRAPH_N launches: a cooperative launch costs the host
        // more than the kernel's start-up on the device, and back-to-back graph nodes close that gap.
        static const bool use_graph = !(getenv("ADAM_B200_TOKEN_GRAPH") && atoi(getenv("ADAM_B200_TOKEN_GRAPH")) == 0);
        const int gi = with_lm ? 1 : 0;
        if (use_graph && !want_logits && !direct && n_steps >= TK_GRAPH_N && D->tk_graph_state[gi] >= 0) {
            if (!D->tk_graph[gi]) {
                const uint64_t l0 = g.launches;
                DCU(cudaStreamSynchronize(g.stream));
                cudaGraph_t graph = nullptr;
                bool ok = cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
                for (uint32_t k = 0; ok && k < TK_GRAPH_N; ++k) ok = enqueue_token(D, with_lm, false) == ADAMAH_OK;
                if (cudaStreamEndCapture(g.stream, &graph) != cudaSuccess) ok = false;
                if (ok && cudaGraphInstantiate(&D->tk_graph[gi], graph, 0) != cudaSuccess) ok = false;
                g.launches = l0;
                if (ok) { D->tk_graph_src[gi] = graph; D->tk_graph_state[gi] = 1; }
                else { cudaGetLastError(); if (graph) cudaGraphDestroy(graph); D->tk_graph[gi] = nullptr; D->tk_graph_state[gi] = -1; }
            }
            if (D->tk_graph[gi]) {
                for (; s + TK_GRAPH_N <= n_steps; s += TK_GRAPH_N) DCU(cudaGraphLaunch(D->tk_graph[gi], g.stream));
                count_launch(s);
            }
        }
        for (; s < n_steps && rc == ADAMAH_OK; ++s) { rc = enqueue_token(D, with_lm, want_logits); if (rc == ADAMAH_OK) rc = sample_step(); }
        end_of_op();
        return rc;
    }
    if (direct || want_logits || capturing()) {
        for (uint32_t s = 0; s < n_steps && rc == ADAMAH_OK; ++s) { rc = enqueue_step(D, D->batch, with_lm, want_logits); if (rc == ADAMAH_OK) rc = sample_step(); }
    } else {
        const int gi = with_lm ? 1 : 0;
        if (!D->graph[gi] || D->graph_batch[gi] != D->batch) {
            if (D->graph[gi]) { cudaGraphExecDestroy(D->graph[gi]); cudaGraphDestroy(D->graph_src[gi]); D->graph[gi] = nullptr; }
            {   // scratch must exist before the capture starts (no allocation inside it)
                float* pv; int* pi; unsigned int* tk;
                if ((rc = argmax_scratch(&pv, &pi, &tk))) return rc;
            }
            const uint64_t l0 = g.launches;
            DCU(cudaStreamSynchronize(g.stream));
            DCU(cudaStreamBeginCapture(g.stream, cudaStreamCaptureModeRelaxed));
            rc = enqueue_step(D, D->batch, with_lm, false);
            cudaGraph_t graph = nullptr;
            cudaError_t e = cudaStreamEndCapture(g.stream, &graph);
            if (rc) { if (graph) cudaGraphDestroy(graph); return rc; }
            if (e != cudaSuccess) return fail(ADAMAH_ERR_BACKEND, "decoder_step: capture failed: %s", cudaGetErrorString(e));
            DCU(cudaGraphInstantiate(&D->graph[gi], graph, 0));
            D->graph_src[gi] = graph;
            D->graph_batch[gi] = D->batch;
            D->graph_kernels[gi] = g.launches - l0;
            g.launches = l0;
        }
        for (uint32_t s = 0; s < n_steps; ++s) DCU(cudaGraphLaunch(D->graph[gi], g.stream));
        count_launch(D->graph_kernels[gi] * n_steps);
    }
    end_of_op();
    return rc;
}

// Sampling rule of steps that carry flag bit4 (role of GenerationConfig, adam/models/engine.py:24-29, applied as
// `_sample` does, :3711-3729): repeat penalty on the distinct ids among the last 64 of the history (generated
// tokens, plus the prompt with repeat_on_prompt), temperature, the top_k (1..64) best, soft-max, nucleus top_p,
// one draw per step from a counter-based generator keyed by (seed, sequence, position).  temperature <= 0 or
// top_k == 1 picks the best penalised logit.
extern "C" int adam_b200_decoder_set_sampling(uint32_t id, uint32_t top_k, float top_p, float temperature, float repeat_penalty,
                                              uint32_t repeat_on_prompt, uint64_t seed) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (top_k == 0 || top_k > 64) return fail(ADAMAH_ERR_INVALID, "decoder_set_sampling: top_k must be 1..64");
    if (!(repeat_penalty > 0.f)) return fail(ADAMAH_ERR_INVALID, "decoder_set_sampling: repeat_penalty must be positive");
    D->smp_k = top_k; D->smp_top_p = top_p; D->smp_temp = temperature; D->smp_penalty = repeat_penalty;
    D->smp_on_prompt = repeat_on_prompt ? 1 : 0; D->smp_seed = seed;
    return ADAMAH_OK;
}

// Asynchronous read of the current tokens: tokens_async enqueues, behind everything issued so
// far, a copy of the current token ids into one of four pinned slots and returns the slot;
// tokens_wait blocks until that copy has landed (later work on the stream keeps running) and
// hands the ids out.  Lets a caller keep the next step queued while it looks at the last ids.
extern "C" int adam_b200_decoder_tokens_async(uint32_t id, uint32_t* slot_out) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (!slot_out || D->batch == 0) return fail(ADAMAH_ERR_INVALID, "decoder_tokens_async: no active sequences or null argument");
    if (capturing()) return fail(ADAMAH_ERR_INVALID, "decoder_tokens_async: not allowed while a graph is being captured");
    const uint32_t slot = D->tok_next;
    D->tok_next = (slot + 1) & 3u;
    if (!D->tok_ring[slot]) {
        DCU(cudaMallocHost((void**)&D->tok_ring[slot], (size_t)D->d.max_batch * 4));
        DCU(cudaEventCreateWithFlags(&D->tok_event[slot], cudaEventDisableTiming));
    }
    DCU(cudaMemcpyAsync(D->tok_ring[slot], D->cur_tok, (size_t)D->batch * 4, cudaMemcpyDeviceToHost, g.stream));
    DCU(cudaEventRecord(D->tok_event[slot], g.stream));
    *slot_out = slot;
    return ADAMAH_OK;
}
extern "C" int adam_b200_decoder_tokens_wait(uint32_t id, uint32_t slot, int32_t* out) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (slot > 3 || !out || !D->tok_ring[slot]) return fail(ADAMAH_ERR_INVALID, "decoder_tokens_wait: bad slot");
    DCU(cudaEventSynchronize(D->tok_event[slot]));
    memcpy(out, D->tok_ring[slot], (size_t)D->batch * 4);
    return ADAMAH_OK;
}

// Overwrite the current token of every active sequence (host-side sampling: the caller read the
// logits of the last step and drew its own tokens; they feed the next step).
extern "C" int adam_b200_decoder_set_tokens(uint32_t id, const int32_t* tokens) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (!tokens || D->batch == 0) return fail(ADAMAH_ERR_INVALID, "decoder_set_tokens: no active sequences or null argument");
    if (capturing()) return fail(ADAMAH_ERR_INVALID, "decoder_set_tokens: not allowed while a graph is being captured");
    for (uint32_t b = 0; b < D->batch; ++b)
        if (tokens[b] < 0 || (uint32_t)tokens[b] >= D->embd.rows) return fail(ADAMAH_ERR_INVALID, "decoder_set_tokens: token id %d outside the vocabulary", tokens[b]);
    DCU(cudaMemcpyAsync(D->cur_tok, tokens, (size_t)D->batch * 4, cudaMemcpyHostToDevice, g.stream));
    DCU(cudaStreamSynchronize(g.stream));
    return ADAMAH_OK;
}

// Chunked prefill: consume the next n_tokens prompt tokens of every active sequence, several
// positions per pass: the rows of a chunk (sequence x token) go through the GEMVs together as
// batch rows, their keys and values are appended first and attention then reads the whole
// chunk from the cache (causal by position).  No LM head: the token after the prompt's last one
// comes from a normal step.  Every sequence must still have n_tokens prompt tokens ahead.
// Same results as n_tokens single steps (the reference consumes prompts token by token,
// engine.py:3838-3847).
template <typename T>
static int launch_kv_append_t(Decoder* D, uint32_t L, uint32_t rows) {
    const adam_b200_decoder_desc& d = D->d;
    KvGeom geo{d.n_layer, d.n_head_kv, d.head_dim, d.page_size, D->max_pages_per_seq, D->page_elems};
    const int which = is_global_layer(d, L) ? 1 : 0;
    const uint32_t warps = rows * d.n_head_kv * 2, qkv_ld = (d.n_head + 2 * d.n_head_kv) * d.head_dim;
    const dim3 grid((warps * 32 + 255) / 256);
    const Layer& ly = D->layers[L];
#define KVA(HD_) launch_k(k_kv_append<T, HD_>, grid, dim3(256), 0, g.stream, g.pdl, (const float*)D->qkv, qkv_ld, ly.norm[NORM_K], d.norm_eps, \
        (const float*)D->rope_cos[which], (const float*)D->rope_sin[which], D->rope_pos[which], D->kv_pool, geo, (const int32_t*)D->block_table, \
        (const int32_t*)D->row_seq, (const int32_t*)D->row_pos, rows, d.n_head, L, g.dev_err)
    switch (d.head_dim) { case 32: KVA(32); break; case 64: KVA(64); break; case 128: KVA(128); break; default: KVA(256); break; }
#undef KVA
    count_launch();
    return ADAMAH_OK;
}

// One part of a prefill chunk of T tokens per sequence; parts as in enqueue_part (2L = attention half
// of layer L, preceded by the row set-up and the embedding for L = 0; 2L+1 = FFN half), and part
// 2*n_layer advances the positions by T.
static int enqueue_prefill_part(Decoder* D, uint32_t batch, uint32_t T, uint32_t part) {
    const adam_b200_decoder_desc& d = D->d;
    const uint32_t rows = batch * T;
    const uint32_t E = d.n_embd, q_dim = d.n_head * d.head_dim, k_dim = d.n_head_kv * d.head_dim, qkv_ld = q_dim + 2 * k_dim;
    int rc;
    if (part == 2 * d.n_layer) {
        launch_k(k_advance_n, dim3((batch + 63) / 64), dim3(64), 0, g.stream, g.pdl, D->pos, batch, (int32_t)T);
        count_launch();
        return check_launch("decoder prefill");
    }
    const uint32_t L = part / 2;
    const Layer& ly = D->layers[L];
    if (!(part & 1u)) {
        if (L == 0) {
            k_prefill_rows<<<(rows + 63) / 64, 64, 0, g.stream>>>(D->pos, batch, T, D->row_seq, D->row_pos);
            count_launch();
            launch_embed(D, rows, (const int32_t*)D->row_seq, (const int32_t*)D->row_pos);
        }
        const int cur = L == 0 ? 0 : 1;
        GemvArgs in = {};
        in.ldx = (int)E; in.eps = d.norm_eps; in.h_in = D->hbuf[cur]; in.w_pre = ly.norm[NORM_ATTN];
        if (L > 0) { in.add_src = D->proj; in.w_post = D->layers[L - 1].norm[NORM_POST_FFW]; in.h_out = D->hbuf[cur ^ 1]; }
        in.y = D->qkv; in.ldy = (int)qkv_ld;
        if (ly.qkv_contiguous) {
            Mat qkv = ly.m[MAT_Q]; qkv.rows = qkv_ld; qkv.tiled = ly.qkv_tiled;
            if ((rc = gemv(qkv, nullptr, in, rows, EPI_STORE))) return rc;
        } else {
            if ((rc = gemv(ly.m[MAT_Q], nullptr, in, rows, EPI_STORE))) return rc;
            GemvArgs in2 = in; in2.h_out = nullptr;
            in2.y = D->qkv + q_dim;
            if ((rc = gemv(ly.m[MAT_K], nullptr, in2, rows, EPI_STORE))) return rc;
            in2.y = D->qkv + q_dim + k_dim;
            if ((rc = gemv(ly.m[MAT_V], nullptr, in2, rows, EPI_STORE))) return rc;
        }
        rc = d.kv_dtype == 1 ? launch_kv_append_t<__half>(D, L, rows) : launch_kv_append_t<float>(D, L, rows);
        if (rc) return rc;
        rc = d.kv_dtype == 1 ? launch_attn_t<__half>(D, L, rows, true) : launch_attn_t<float>(D, L, rows, true);
        if (rc) return rc;
        GemvArgs o = {};
        o.x = D->attn_out; o.ldx = (int)q_dim; o.y = D->proj; o.ldy = (int)E;
        if ((rc = gemv(ly.m[MAT_O], nullptr, o, rows, EPI_STORE))) return rc;
    } else {
        GemvArgs gu = {};
        gu.ldx = (int)E; gu.eps = d.norm_eps; gu.h_in = D->hbuf[0]; gu.add_src = D->proj; gu.w_post = ly.norm[NORM_POST_ATTN];
        gu.w_pre = ly.norm[NORM_FFN]; gu.h_out = D->hbuf[1]; gu.y = D->act; gu.ldy = (int)d.n_ff;
        if ((rc = gemv(ly.m[MAT_GATE], &ly.m[MAT_UP], gu, rows, d.ffn_act == 0 ? EPI_GEGLU : EPI_SWIGLU))) return rc;
        GemvArgs dn = {};
        dn.x = D->act; dn.ldx = (int)d.n_ff; dn.y = D->proj; dn.ldy = (int)E;
        if ((rc = gemv(ly.m[MAT_DOWN], nullptr, dn, rows, EPI_STORE))) return rc;
    }
    return check_launch("decoder prefill");
}

static int enqueue_prefill_chunk(Decoder* D, uint32_t batch, uint32_t T) {
    for (uint32_t part = 0; part <= 2 * D->d.n_layer; ++part) {
        const int rc = enqueue_prefill_part(D, batch, T, part);
        if (rc) return rc;
    }
    return ADAMAH_OK;
}

// One part of one prefill chunk of n_tokens (<= 64 / batch) tokens per sequence, for tensor-parallel
// callers: parts 0 .. 2*n_layer-1 as in adam_b200_decoder_step_part (all-reduce the projection
// buffer, batch * n_tokens rows, after each), part 2*n_layer advances the positions.
extern "C" int adam_b200_decoder_prefill_part(uint32_t id, uint32_t n_tokens, uint32_t part) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (D->batch == 0) return fail(ADAMAH_ERR_INVALID, "decoder_prefill_part: call decoder_begin first");
    if (part > 2 * D->d.n_layer) return fail(ADAMAH_ERR_INVALID, "decoder_prefill_part: part %u of %u", part, 2 * D->d.n_layer + 1);
    if (n_tokens == 0 || (uint64_t)n_tokens * D->batch > D->rows_cap) return fail(ADAMAH_ERR_INVALID, "decoder_prefill_part: a chunk holds at most %u rows", D->rows_cap);
    if (part == 0)
        for (uint32_t b = 0; b < D->batch; ++b)
            if ((uint64_t)D->hpos[b] + n_tokens > D->hplen[b])
                return fail(ADAMAH_ERR_INVALID, "decoder_prefill_part: sequence %u has only %u prompt tokens left", b, D->hplen[b] - D->hpos[b]);
    static const bool allow = !(getenv("ADAM_B200_PDL") && atoi(getenv("ADAM_B200_PDL")) == 0);
    g.pdl = allow;
    const int rc = enqueue_prefill_part(D, D->batch, n_tokens, part);
    g.pdl = false;
    if (rc == ADAMAH_OK && part == 2 * D->d.n_layer) for (uint32_t& hp : D->hpos) hp += n_tokens;
    end_of_op();
    return rc;
}

extern "C" int adam_b200_decoder_prefill(uint32_t id, uint32_t n_tokens) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (D->batch == 0) return fail(ADAMAH_ERR_INVALID, "decoder_prefill: call decoder_begin first");
    if (capturing()) return fail(ADAMAH_ERR_INVALID, "decoder_prefill: not allowed while a graph is being captured");
    for (uint32_t b = 0; b < D->batch; ++b)
        if ((uint64_t)D->hpos[b] + n_tokens > D->hplen[b])
            return fail(ADAMAH_ERR_INVALID, "decoder_prefill: sequence %u has only %u prompt tokens left", b, D->hplen[b] - D->hpos[b]);
    const uint32_t t_max = D->rows_cap / D->batch;
    if (t_max == 0) return fail(ADAMAH_ERR_INVALID, "decoder_prefill: batch larger than the row buffers");
    static const bool allow = !(getenv("ADAM_B200_PDL") && atoi(getenv("ADAM_B200_PDL")) == 0);
    int rc = ADAMAH_OK;
    uint32_t left = n_tokens;
    while (left && rc == ADAMAH_OK) {
        const uint32_t T = left < t_max ? left : t_max;
        g.pdl = allow;
        rc = enqueue_prefill_chunk(D, D->batch, T);
        g.pdl = false;
        left -= T;
    }
    if (rc == ADAMAH_OK) for (uint32_t& hp : D->hpos) hp += n_tokens;
    end_of_op();
    return rc;
}

// Where the time of a one-sequence step on the graph of per-operation kernels goes (diagnostics build only):
// out == NULL arms the trace for `layer` (the step graphs are recorded again with the trace buffer attached);
// a later call with a buffer waits for the stream and copies 512 stamps of the most recent step: the four
// products of the layer (QKV, o-proj, gate/up, down) as [product][CTA 0..7][8] and its attention launch as
// [CTA 0..31][8], nanoseconds of the GPU's global timer (slot meanings: adam_b200.h).
extern "C" int adam_b200_decoder_step_trace(uint32_t id, uint32_t layer, long long* out, uint32_t n_words) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
#ifdef ADAM_B200_STEP_TRACE
    const size_t words = 4 * 64 + 32 * 8;
    if (!out) {
        if (layer >= D->d.n_layer) return fail(ADAMAH_ERR_INVALID, "decoder_step_trace: layer %u of %u", layer, D->d.n_layer);
        DCU(cudaStreamSynchronize(g.stream));
        if (!g_step_trace) DCU(cudaMalloc(&g_step_trace, words * 8));
        DCU(cudaMemset(g_step_trace, 0, words * 8));
        g_step_trace_layer = layer;
        free_graphs(D);
        return ADAMAH_OK;
    }
    if (!g_step_trace) return fail(ADAMAH_ERR_INVALID, "decoder_step_trace: not armed");
    DCU(cudaStreamSynchronize(g.stream));
    DCU(cudaMemcpy(out, g_step_trace, (n_words < words ? n_words : words) * 8, cudaMemcpyDeviceToHost));
    return ADAMAH_OK;
#else
    (void)layer; (void)out; (void)n_words;
    return fail(ADAMAH_ERR_INVALID, "decoder_step_trace: this library was built without ADAM_B200_STEP_TRACE (python -m adam_b200.build --step-trace)");
#endif
}

// One part of a token step, enqueued directly on the stream (no graph): see enqueue_part.
// For callers that interleave their own work between parts (tensor parallelism: an
// all-reduce of the projection buffer after every layer part, a merge of the arg-max
// pairs after the LM-head part).  flags as in adam_b200_decoder_step.
extern "C" int adam_b200_decoder_n_parts(uint32_t id) {
    Decoder* D = get_dec(id);
    return D ? (int)n_parts(D) : ADAMAH_ERR_NOT_FOUND;
}
extern "C" int adam_b200_decoder_step_part(uint32_t id, uint32_t part, uint32_t flags) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (!D->batch) return fail(ADAMAH_ERR_INVALID, "decoder_step_part: call decoder_begin first");
    if (part >= n_parts(D)) return fail(ADAMAH_ERR_INVALID, "decoder_step_part: part %u of %u", part, n_parts(D));
    const bool with_lm = flags & 1u, want_logits = (flags & 2u) != 0;
    if (part == 0)
        for (uint32_t b = 0; b < D->batch; ++b)
            if (D->hpos[b] + 1u > D->hres[b]) return fail(ADAMAH_ERR_INVALID, "decoder_step_part: sequence %u has used all %u reserved positions", b, D->hres[b]);
    static const bool allow = !(getenv("ADAM_B200_PDL") && atoi(getenv("ADAM_B200_PDL")) == 0);
    g.pdl = allow;
    const int rc = enqueue_part(D, D->batch, part, with_lm, want_logits);
    g.pdl = false;
    if (rc == ADAMAH_OK && part + 1 == n_parts(D)) for (uint32_t& hp : D->hpos) hp += 1;
    end_of_op();
    return rc;
}
// Diagnostics of the single-launch token kernel: run ONE token step (LM head included) of the active
// sequence with per-phase SM clock stamps of layer `layer` and of the LM head recorded by every CTA, and
// return them: out[cta * 16 + slot] (clock64 values of that CTA's SM; slots 0..9 = layer phases, 10..13 = LM
// head), n_cta_out = CTAs launched.  out must hold 16 * 256 values.
extern "C" int adam_b200_decoder_token_trace(uint32_t id, uint32_t layer, long long* out, uint32_t* n_cta_out) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (!out || !n_cta_out || D->batch != 1) return fail(ADAMAH_ERR_INVALID, "decoder_token_trace: needs one active sequence");
    if (D->tk_state == 0) { const int rc0 = prepare_token_kernel(D); if (rc0) return rc0; }
    if (D->tk_state != 1) return fail(ADAMAH_ERR_INVALID, "decoder_token_trace: this model does not run on the token kernel");
    if (D->hpos[0] + 1u > D->hres[0]) return fail(ADAMAH_ERR_INVALID, "decoder_token_trace: no reserved position left");
    const size_t bytes = (size_t)TK_TRACE_SLOTS * 256 * sizeof(long long);
    DCU(cudaMalloc((void**)&g_tk_trace, bytes));
    DCU(cudaMemsetAsync(g_tk_trace, 0, bytes, g.stream));
    g_tk_trace_layer = (int)(layer & 0xFFFFu); g_tk_trace_phase = (int)(layer >> 16);
    D->hpos[0] += 1;
    const int rc = enqueue_token(D, true, false);
    cudaMemcpyAsync(out, g_tk_trace, bytes, cudaMemcpyDeviceToHost, g.stream);
    cudaStreamSynchronize(g.stream);
    cudaFree(g_tk_trace);
    g_tk_trace = nullptr;
    *n_cta_out = (uint32_t)D->tk_grid;
    return rc;
}

// Exercises the bounded waits of the single-launch token kernel without any fault: ONE token step is launched
// with its last CTA left out and every wait limited to `wait_us` microseconds.  The packets that CTA would have
// produced never arrive, so the waits of the others run out; they record DEVERR_WAIT in the device error word,
// set the decoder's sticky word and return.  Later steps return at once until decoder_begin / decoder_continue
// clears the word.  Returns after the launch has finished.
extern "C" int adam_b200_decoder_test_wait_expiry(uint32_t id, uint32_t wait_us) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (D->batch != 1) return fail(ADAMAH_ERR_INVALID, "decoder_test_wait_expiry: needs one active sequence");
    if (D->tk_state == 0) { const int rc0 = prepare_token_kernel(D); if (rc0) return rc0; }
    if (D->tk_state != 1 || D->tk_grid < 2) return fail(ADAMAH_ERR_INVALID, "decoder_test_wait_expiry: this model does not run on the token kernel");
    if (wait_us == 0 || wait_us > 1000000u) return fail(ADAMAH_ERR_INVALID, "decoder_test_wait_expiry: wait_us must be 1 .. 1000000");
    TkArgs a = D->tk;
    a.with_lm = 1; a.logits = nullptr; a.trace = nullptr;
    a.wait_cycles = (long long)wait_us * 2000;              // SM clocks at about 2 GHz
    const int rc = launch_token(D->tk_wt, D->d.kv_dtype == 1, (int)D->d.head_dim, a, D->tk_grid - 1, g.stream);
    DCU(cudaStreamSynchronize(g.stream));
    return rc;
}

// Device address and size of one of the decoder's buffers, for callers that run their own
// kernels or collectives on them (same stream, see adam_b200_set_stream):
//   0 = projection output [rows][n_embd] f32 (what a tensor-parallel caller all-reduces; rows =
//       batch in a decode step, batch * n_tokens in a prefill chunk; sized for max(max_batch, 64) rows)
//   1 = current token ids [max_batch] i32     2 = their logit values [max_batch] f32
//   3 = positions [max_batch] i32
extern "C" int adam_b200_decoder_buffer_ptr(uint32_t id, uint32_t which, uint64_t* ptr_out, uint64_t* bytes_out) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (!ptr_out || !bytes_out) return fail(ADAMAH_ERR_INVALID, "decoder_buffer_ptr: null argument");
    const size_t B = D->d.max_batch;
    switch (which) {
    case 0: *ptr_out = (uint64_t)(uintptr_t)D->proj; *bytes_out = (size_t)D->rows_cap * D->d.n_embd * 4; break;
    case 1: *ptr_out = (uint64_t)(uintptr_t)D->cur_tok; *bytes_out = B * 4; break;
    case 2: *ptr_out = (uint64_t)(uintptr_t)D->cur_val; *bytes_out = B * 4; break;
    case 3: *ptr_out = (uint64_t)(uintptr_t)D->pos; *bytes_out = B * 4; break;
    default: return fail(ADAMAH_ERR_INVALID, "decoder_buffer_ptr: unknown buffer %u", which);
    }
    return ADAMAH_OK;
}

// Reads (after synchronising): positions, current sampled tokens, and the log of
// sampled tokens: out_log[b][p] = id sampled for position p (-1 where none).
extern "C" int adam_b200_decoder_read_state(uint32_t id, int32_t* pos_out, int32_t* cur_tok_out) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (pos_out) DCU(cudaMemcpyAsync(pos_out, D->pos, (size_t)D->d.max_batch * 4, cudaMemcpyDeviceToHost, g.stream));
    if (cur_tok_out) DCU(cudaMemcpyAsync(cur_tok_out, D->cur_tok, (size_t)D->d.max_batch * 4, cudaMemcpyDeviceToHost, g.stream));
    DCU(cudaStreamSynchronize(g.stream));
    return ADAMAH_OK;
}
extern "C" int adam_b200_decoder_read_log(uint32_t id, uint32_t seq, uint32_t first_pos, uint32_t n, int32_t* out) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (!out || seq >= D->d.max_batch || (uint64_t)first_pos + n > D->d.kv_cap) return fail(ADAMAH_ERR_INVALID, "decoder_read_log: bad range");
    DCU(cudaMemcpyAsync(out, D->gen_log + (size_t)seq * D->d.kv_cap + first_pos, (size_t)n * 4, cudaMemcpyDeviceToHost, g.stream));
    DCU(cudaStreamSynchronize(g.stream));
    return ADAMAH_OK;
}
extern "C" int adam_b200_decoder_read_logits(uint32_t id, uint32_t seq, float* out) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    if (!out || seq >= D->d.max_batch) return fail(ADAMAH_ERR_INVALID, "decoder_read_logits: bad sequence");
    DCU(cudaMemcpyAsync(out, D->logits + (size_t)seq * D->d.n_vocab, (size_t)D->d.n_vocab * 4, cudaMemcpyDeviceToHost, g.stream));
    DCU(cudaStreamSynchronize(g.stream));
    return ADAMAH_OK;
}
// Debug/verification read of an activation buffer of the last step:
// what = 0 hidden after the last layer [E] (steps that ran the LM head), 2 qkv, 4 attn_out, 5 proj [E], 6 act [FF].
extern "C" int adam_b200_decoder_read_buffer(uint32_t id, uint32_t what, uint32_t seq, float* out, uint32_t n) {
    Decoder* D = get_dec(id);
    if (!D) return ADAMAH_ERR_NOT_FOUND;
    const adam_b200_decoder_desc& d = D->d;
    const uint32_t q_dim = d.n_head * d.head_dim, k_dim = d.n_head_kv * d.head_dim;
    const float* bufs[7] = {D->hbuf[D->h_final], nullptr, D->qkv, nullptr, D->attn_out, D->proj, D->act};
    const uint32_t lds[7] = {d.n_embd, d.n_embd, q_dim + 2 * k_dim, q_dim, q_dim, d.n_embd, d.n_ff};
    if (what > 6 || !bufs[what] || !out || seq >= d.max_batch || n > lds[what]) return fail(ADAMAH_ERR_INVALID, "decoder_read_buffer: bad arguments");
    DCU(cudaMemcpyAsync(out, bufs[what] + (size_t)seq * lds[what], (size_t)n * 4, cudaMemcpyDeviceToHost, g.stream));
    DCU(cudaStreamSynchronize(g.stream));
    return ADAMAH_OK;
}
