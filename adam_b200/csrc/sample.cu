// Sampled decoding on the device: LM head + per-group top-k with repeat penalty
// (map_matvec_topk_t_xq4[_ex]_dev: adamah-MAIN/adamah/adamah.c:9727-9832 and
// shaders/src/f32/map_matvec_topk_t_xq4.comp), and the decoder's own sampling step that keeps
// non-greedy generation on the GPU (role of the reference engine's fused top-k branch,
// adam/models/engine.py:3403-3512, and of its host-side rule `_sample`, :3711-3729).
//
// Design.  The logits of one LM-head product (1 MB at a 262144-row vocabulary) are written once by the
// dequant GEMV and stay in L2; selection then works on them in two short parallel stages instead of a
// serial insertion list per work group as in the shader:
//   stage 1  one CTA per group of rows keeps each thread's values in registers and extracts the group's k
//            best by k rounds of a block-wide arg-max (warp shuffles + one shared-memory hop);
//   stage 2  (decoder only) one CTA per sequence extracts the k best of all groups' candidates the same
//            way, which leaves them sorted, then soft-max with temperature, nucleus cut and the draw run on
//            one warp.
// Ties go to the lower row index everywhere (map_argmax.comp `better`), NaN counts as -FLT_MAX.
#include "common.cuh"
#include "gemv.cuh"
#include "token.cuh"

#include <cstdlib>

namespace ab {

int weight_ref(const Map* m, uint64_t off, uint64_t n_elems, int* wtype, WeightRef* w);
int run_gemv(uint32_t map_id, uint64_t off, int wtype, GemvArgs& ga);
void launch_gemv_q4map(const float* x, const Map* w, uint64_t w_off, float* y, uint32_t K, uint32_t N);

constexpr float SNEG = -3.402823466e+38f;
constexpr int SEL_T = 256;                 // threads of a selection CTA
constexpr int SEL_V = 8;                   // values a thread keeps in registers (a group has at most SEL_T * SEL_V rows)
constexpr uint32_t TOPK_MAX = 64;

// Block-wide arg-max of (v, i) over SEL_T threads; every thread gets the winner.  sv/si: SEL_T / 32 slots.
__device__ __forceinline__ void block_best(float& v, int& i, float* sv, int* si) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { sv[warp] = v; si[warp] = i; }
    __syncthreads();
    v = sv[0]; i = si[0];
#pragma unroll
    for (int w = 1; w < SEL_T / 32; ++w) if (better(sv[w], si[w], v, i)) { v = sv[w]; i = si[w]; }
}

// The k best of this CTA's values: thread t holds values val[j] with keys key[j] (key < 0 = empty slot).
// Round r leaves the r-th best in (out_v[r], out_i[r]) (shared memory, k <= 64); a slot is emptied once taken.
__device__ __forceinline__ void block_topk(float (&val)[SEL_V], int (&key)[SEL_V], uint32_t k, float* out_v, int* out_i, float* sv, int* si) {
    for (uint32_t r = 0; r < k; ++r) {
        float bv = SNEG; int bi = -1;
#pragma unroll
        for (int j = 0; j < SEL_V; ++j) if (key[j] >= 0 && better(val[j], key[j], bv, bi)) { bv = val[j]; bi = key[j]; }
        block_best(bv, bi, sv, si);
#pragma unroll
        for (int j = 0; j < SEL_V; ++j) if (key[j] >= 0 && key[j] == bi) key[j] = -1;
        if (threadIdx.x == 0) { out_v[r] = bi < 0 ? SNEG : bv; out_i[r] = bi; }
    }
    __syncthreads();
}

__device__ __forceinline__ float penalised(float v, int row, const uint32_t* __restrict__ pen, uint32_t n_pen, float penalty) {
    if (!(v == v)) v = SNEG;
    for (uint32_t i = 0; i < n_pen; ++i)
        if (pen[i] == (uint32_t)row) return v > 0.f ? __fdiv_rn(v, penalty) : v * penalty;
    return v;
}

// Stage 1.  Group g = rows [g * rpg, min(N, (g + 1) * rpg)); candidates land at cand_v / cand_i [g * k + r]
// (decoder) or, through locs, in the activation map with the row index stored as float32 (operator).
__global__ void __launch_bounds__(SEL_T) k_group_topk(const float* __restrict__ logits, uint32_t N, uint32_t rpg, uint32_t k,
                                                      const uint32_t* __restrict__ pen, uint32_t n_pen, float penalty,
                                                      float* __restrict__ cand_v, int* __restrict__ cand_i,
                                                      float* __restrict__ map, uint64_t n_el, const uint32_t* __restrict__ li,
                                                      const uint32_t* __restrict__ lv, uint32_t* err) {
    __shared__ float sv[SEL_T / 32]; __shared__ int si[SEL_T / 32];
    __shared__ float out_v[TOPK_MAX]; __shared__ int out_i[TOPK_MAX];
    const uint32_t g = blockIdx.x, r0 = g * rpg, r1 = min(N, r0 + rpg);
    float val[SEL_V]; int key[SEL_V];
#pragma unroll
    for (int j = 0; j < SEL_V; ++j) {
        const uint32_t row = r0 + threadIdx.x + j * SEL_T;
        key[j] = row < r1 ? (int)row : -1;
        val[j] = row < r1 ? penalised(logits[row], (int)row, pen, n_pen, penalty) : SNEG;
    }
    block_topk(val, key, k, out_v, out_i, sv, si);
    if (threadIdx.x < k) {
        const uint32_t o = g * k + threadIdx.x;
        if (map) {
            const uint64_t di = li[o], dv = lv[o];
            if (di >= n_el || dv >= n_el) atomicOr(err, DEVERR_OOB_MAP);
            else { map[di] = (float)(out_i[threadIdx.x] < 0 ? 0 : out_i[threadIdx.x]); map[dv] = out_v[threadIdx.x]; }
        } else { cand_v[o] = out_v[threadIdx.x]; cand_i[o] = out_i[threadIdx.x]; }
    }
}

// ---- decoder sampling step ------------------------------------------------------------------------------
// uniform in [0, 1) from (seed, sequence, position): splitmix64 of the three, top 24 bits
__host__ __device__ inline float sample_uniform(uint64_t seed, uint32_t seq, uint32_t pos) {
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (((uint64_t)seq << 32 | pos) + 1ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// The ids whose logits get the repeat penalty: the distinct tokens among the last 64 of the history (prompt
// included with on_prompt, else generated tokens only), as the reference's `set(prev[-64:])` (engine.py:3713).
// Position q of sequence b holds prompt_tok[q] for q < prompt_len and the logged sample otherwise.
__device__ __forceinline__ uint32_t history_ids(const int32_t* prompt_tok, const int32_t* gen_log, int32_t plen, int32_t pos_new,
                                                int on_prompt, uint32_t* ids) {
    const int32_t lo = max(on_prompt ? 0 : plen, pos_new - 64);
    uint32_t n = 0;
    for (int32_t q = lo; q < pos_new; ++q) {
        const int32_t t = q < plen ? prompt_tok[q] : gen_log[q];
        if (t < 0) continue;
        bool seen = false;
        for (uint32_t j = 0; j < n; ++j) seen |= ids[j] == (uint32_t)t;
        if (!seen) ids[n++] = (uint32_t)t;
    }
    return n;
}

// Stage 1 for the decoder: grid (groups, batch); the penalty list is rebuilt by every CTA (<= 64 short loops).
__global__ void __launch_bounds__(SEL_T) k_sample_stage1(const float* __restrict__ logits, uint32_t V, uint32_t k,
                                                         const int32_t* __restrict__ pos, const int32_t* __restrict__ prompt_len,
                                                         const int32_t* __restrict__ prompt_tok, const int32_t* __restrict__ gen_log, uint32_t ld,
                                                         float penalty, int on_prompt, float* __restrict__ cand_v, int* __restrict__ cand_i) {
    __shared__ float sv[SEL_T / 32]; __shared__ int si[SEL_T / 32];
    __shared__ float out_v[TOPK_MAX]; __shared__ int out_i[TOPK_MAX];
    __shared__ uint32_t s_pen[64]; __shared__ uint32_t s_np;
    const uint32_t g = blockIdx.x, b = blockIdx.y, groups = gridDim.x;
    if (threadIdx.x == 0)
        s_np = penalty != 1.0f ? history_ids(prompt_tok + (size_t)b * ld, gen_log + (size_t)b * ld, prompt_len[b], pos[b], on_prompt, s_pen) : 0u;
    __syncthreads();
    const float* lg = logits + (size_t)b * V;
    const uint32_t rpg = SEL_T * SEL_V, r0 = g * rpg, r1 = min(V, r0 + rpg);
    float val[SEL_V]; int key[SEL_V];
#pragma unroll
    for (int j = 0; j < SEL_V; ++j) {
        const uint32_t row = r0 + threadIdx.x + j * SEL_T;
        key[j] = row < r1 ? (int)row : -1;
        val[j] = row < r1 ? penalised(lg[row], (int)row, s_pen, s_np, penalty) : SNEG;
    }
    block_topk(val, key, k, out_v, out_i, sv, si);
    if (threadIdx.x < k) {
        const size_t o = ((size_t)b * groups + g) * k + threadIdx.x;
        cand_v[o] = out_v[threadIdx.x]; cand_i[o] = out_i[threadIdx.x];
    }
}

// Stage 2: one CTA per sequence.  The k best of the n_cand candidates (sorted as a by-product), then on warp 0:
// p_i = exp((l_i - l_0) / T) / sum, nucleus = the shortest prefix whose probability reaches top_p
// (np.searchsorted(cumsum, top_p) + 1, engine.py:3724-3726), renormalise, inverse-CDF draw with the uniform u.
// temperature <= 0 takes the best candidate (engine.py:3719).  Writes the token where the next step reads it and
// into the log at the sequence's (already advanced) position.
__global__ void __launch_bounds__(SEL_T) k_sample_stage2(const float* __restrict__ cand_v, const int* __restrict__ cand_i, uint32_t n_cand, uint32_t k,
                                                         float temperature, float top_p, uint64_t seed,
                                                         const int32_t* __restrict__ pos, int32_t* __restrict__ cur_tok, float* __restrict__ cur_val,
                                                         int32_t* __restrict__ gen_log, uint32_t ld, float* __restrict__ dbg) {
    __shared__ float sv[SEL_T / 32]; __shared__ int si[SEL_T / 32];
    __shared__ float out_v[TOPK_MAX]; __shared__ int out_i[TOPK_MAX];
    const uint32_t b = blockIdx.x;
    const float* cv = cand_v + (size_t)b * n_cand;
    const int* ci = cand_i + (size_t)b * n_cand;
    // candidates beyond SEL_T * SEL_V are folded in by keeping the better of what a slot already holds (they
    // arrive in groups of k sorted values, so a simple strided pre-pass is enough for the sizes in use)
    float val[SEL_V]; int key[SEL_V];
#pragma unroll
    for (int j = 0; j < SEL_V; ++j) { val[j] = SNEG; key[j] = -1; }
    // keys must be unique for block_topk: use the row index (unique across groups)
    for (uint32_t base = 0; base < n_cand; base += SEL_T * SEL_V) {
#pragma unroll
        for (int j = 0; j < SEL_V; ++j) {
            const uint32_t c = base + threadIdx.x + j * SEL_T;
            if (c < n_cand) {
                const float v = cv[c]; const int i = ci[c];
                if (i >= 0 && better(v, i, val[j], key[j])) { val[j] = v; key[j] = i; }
            }
        }
    }
    block_topk(val, key, k, out_v, out_i, sv, si);
    if (threadIdx.x >= 32) return;
    const uint32_t lane = threadIdx.x;
    uint32_t n = 0;
    for (uint32_t r = 0; r < k; ++r) if (out_i[r] >= 0) n = r + 1;
    int chosen = 0;
    if (n > 1 && temperature > 0.f) {
        // two candidates per lane
        const float l0 = out_v[0];
        float p[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) { const uint32_t r = lane + 32 * h; p[h] = r < n ? expf(__fdiv_rn(out_v[r] - l0, temperature)) : 0.f; }
        // sums in candidate order (lane 0 walks the values): the same order as a sequential cumulative sum
        float sum = 0.f;
        for (uint32_t r = 0; r < n; ++r) sum += __shfl_sync(0xffffffffu, p[r >> 5], r & 31);
        uint32_t keep = n;
        if (top_p < 1.0f) {
            float cs = 0.f;
            for (uint32_t r = 0; r < n; ++r) {
                cs += __fdiv_rn(__shfl_sync(0xffffffffu, p[r >> 5], r & 31), sum);
                if (cs >= top_p) { keep = r + 1; break; }
            }
        }
        float ks = 0.f;
        for (uint32_t r = 0; r < keep; ++r) ks += __shfl_sync(0xffffffffu, p[r >> 5], r & 31);
        const float u = sample_uniform(seed, b, (uint32_t)pos[b]);
        const float target = u * ks;
        float acc = 0.f;
        chosen = (int)keep - 1;
        for (uint32_t r = 0; r < keep; ++r) {
            acc += __shfl_sync(0xffffffffu, p[r >> 5], r & 31);
            if (target < acc) { chosen = (int)r; break; }
        }
        if (dbg && lane == 0) { dbg[b * 4] = (float)keep; dbg[b * 4 + 1] = u; dbg[b * 4 + 2] = sum; dbg[b * 4 + 3] = (float)n; }
    }
    if (lane == 0) {
        const int tok = out_i[chosen] < 0 ? 0 : out_i[chosen];
        cur_tok[b] = tok;
        cur_val[b] = out_v[chosen];
        const int32_t q = pos[b];
        if ((uint32_t)q < ld) gen_log[(size_t)b * ld + q] = tok;
    }
}

static float* s_cand_v = nullptr; static int* s_cand_i = nullptr; static size_t s_cand_n = 0;

// Enqueue the sampling step for `batch` sequences whose soft-capped logits lie at logits[b * V .. ) and whose
// positions were already advanced.  k = 1..64.
int launch_sample(const float* logits, uint32_t V, uint32_t batch, uint32_t k, float temperature, float top_p, float penalty, int on_prompt,
                  uint64_t seed, const int32_t* pos, const int32_t* prompt_len, const int32_t* prompt_tok, int32_t* gen_log, uint32_t ld,
                  int32_t* cur_tok, float* cur_val) {
    if (k == 0 || k > TOPK_MAX) return fail(ADAMAH_ERR_INVALID, "sampling: top_k must be 1..64 on the device");
    const uint32_t groups = (V + SEL_T * SEL_V - 1) / (SEL_T * SEL_V);
    const size_t need = (size_t)batch * groups * k;
    if (s_cand_n < need) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(g.stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone)
            return fail(ADAMAH_ERR_INVALID, "sampling: the first sampled step must run outside a graph capture");
        cudaStreamSynchronize(g.stream);
        cudaFree(s_cand_v); cudaFree(s_cand_i); s_cand_v = nullptr; s_cand_i = nullptr; s_cand_n = 0;
        if (cudaMalloc((void**)&s_cand_v, need * 4) != cudaSuccess || cudaMalloc((void**)&s_cand_i, need * 4) != cudaSuccess) {
            cudaGetLastError();
            return fail(ADAMAH_ERR_MEMORY, "sampling: out of device memory");
        }
        s_cand_n = need;
    }
    k_sample_stage1<<<dim3(groups, batch), SEL_T, 0, g.stream>>>(logits, V, k, pos, prompt_len, prompt_tok, gen_log, ld, penalty, on_prompt, s_cand_v, s_cand_i);
    k_sample_stage2<<<batch, SEL_T, 0, g.stream>>>(s_cand_v, s_cand_i, groups * k, k, temperature, top_p, seed, pos, cur_tok, cur_val, gen_log, ld, nullptr);
    count_launch(2);
    return check_launch("decoder sampling");
}

static float* s_logits = nullptr; static size_t s_logits_n = 0;
int logits_scratch(size_t n, float** out) {
    if (s_logits_n < n) {
        if (s_logits) { cudaStreamSynchronize(g.stream); cudaFree(s_logits); s_logits = nullptr; s_logits_n = 0; }
        if (cudaMalloc((void**)&s_logits, n * 4) != cudaSuccess) { cudaGetLastError(); return fail(ADAMAH_ERR_MEMORY, "out of device memory for %zu logits", n); }
        s_logits_n = n;
    }
    *out = s_logits;
    return ADAMAH_OK;
}
void sample_free_all() {
    cudaFree(s_logits); s_logits = nullptr; s_logits_n = 0;
    cudaFree(s_cand_v); cudaFree(s_cand_i); s_cand_v = nullptr; s_cand_i = nullptr; s_cand_n = 0;
}

}  // namespace ab

using namespace ab;

// Reference signature and results (adamah.c:9727-9822): for every group of rows_per_group rows of W the k
// largest of W[n,:] . x after the repeat penalty, as (row index as float32, value) pairs stored at
// locs_idx_dst / locs_val_dst [group * k + r] of the activation map; unfilled entries are (0, -FLT_MAX).
// W may be a Q4 map (the reference's storage) or a GGUF-block map.
extern "C" int map_matvec_topk_t_xq4_ex_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t penalty_ids_h,
                                            uint32_t idx_dst_h, uint32_t val_dst_h, uint32_t K, uint32_t N, uint32_t k,
                                            uint32_t n_penalty, float repeat_penalty, uint32_t rows_per_group) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    Map* a = get_map(map_act);
    Map* w = get_map(map_wt);
    if (!a || !w) return ADAMAH_ERR_NOT_FOUND;
    if (a->dtype != ADAMAH_DTYPE_F32 || a->pack_size != 1) return fail(ADAMAH_ERR_INVALID, "matvec_topk: map %u must be float32 with pack_size 1", map_act);
    if (N == 0 || k == 0) return ADAMAH_OK;                                  // adamah.c:9737
    if (k > TOPK_MAX || n_penalty > 64) return fail(ADAMAH_ERR_INVALID, "matvec_topk: k and n_penalty are limited to 64");
    if (rows_per_group == 0 || !K) return fail(ADAMAH_ERR_INVALID, "matvec_topk: rows_per_group and K must not be 0");
    if (rows_per_group > (uint32_t)(SEL_T * SEL_V)) return fail(ADAMAH_ERR_INVALID, "matvec_topk: rows_per_group is limited to %d", SEL_T * SEL_V);
    const uint32_t groups = (N + rows_per_group - 1) / rows_per_group;
    if (!handle_ok(idx_dst_h, groups * k * 4) || !handle_ok(val_dst_h, groups * k * 4) || !handle_ok(penalty_ids_h, n_penalty * 4)) return ADAMAH_ERR_NOT_FOUND;
    uint32_t ab_, bb;
    if (!hfirst(a_h, &ab_) || !hfirst(b_h, &bb)) return ADAMAH_ERR_NOT_FOUND;
    if ((uint64_t)ab_ + K > a->n_elems) return fail(ADAMAH_ERR_INVALID, "matvec_topk: activation range beyond map %u", map_act);
    float* lg = nullptr;
    int rc = logits_scratch(N, &lg);
    if (rc) return rc;
    const float* x = (const float*)a->buf + ab_;
    if (w->dtype == ADAMAH_DTYPE_Q4) {
        if ((uint64_t)bb + (uint64_t)N * K > w->n_elems) return fail(ADAMAH_ERR_INVALID, "matvec_topk: weight range beyond map %u", map_wt);
        launch_gemv_q4map(x, w, bb, lg, K, N);
    } else {
        int wtype; GemvArgs ga = {};
        if ((rc = weight_ref(w, bb, (uint64_t)N * K, &wtype, &ga.w0))) return rc;
        if (ab_ % 4 || K % 4) return fail(ADAMAH_ERR_INVALID, "matvec_topk: activation offset must be a multiple of 4 elements");
        ga.x = x; ga.ldx = (int)K; ga.y = lg; ga.ldy = (int)N; ga.N = (int)N; ga.K = (int)K; ga.B = 1; ga.epi = EPI_STORE;
        if ((rc = run_gemv(map_wt, bb, wtype, ga))) return rc;
    }
    k_group_topk<<<groups, SEL_T, 0, g.stream>>>(lg, N, rows_per_group, k, hlocs(penalty_ids_h), n_penalty, repeat_penalty, nullptr, nullptr,
                                                 (float*)a->buf, a->n_elems, hlocs(idx_dst_h), hlocs(val_dst_h), g.dev_err);
    count_launch();
    rc = check_launch("map_matvec_topk_t_xq4");
    end_of_op();
    return rc;
}

extern "C" int map_matvec_topk_t_xq4_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t penalty_ids_h,
                                         uint32_t idx_dst_h, uint32_t val_dst_h, uint32_t K, uint32_t N, uint32_t k,
                                         uint32_t n_penalty, float repeat_penalty) {
    return map_matvec_topk_t_xq4_ex_dev(map_act, map_wt, a_h, b_h, penalty_ids_h, idx_dst_h, val_dst_h, K, N, k, n_penalty, repeat_penalty, 256);
}
