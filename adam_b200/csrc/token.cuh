// One decoded token of one sequence as ONE persistent kernel (cooperative launch, one CTA per SM).
//
// The per-op decode loop of the reference (adam/models/engine.py:2971-3706 `_forward`: ~400 dispatches
// per token) and this library's own chain of 133 dependent kernels are both bound by hand-over
// latency at batch 1, not by HBM bandwidth.  Here the whole token -- embedding row, every layer's
// norm chain, QKV / o-proj / gate-up / down products, QK-norm + RoPE + KV append + attention, final
// norm, LM head + arg-max, position advance -- runs inside one launch.  Shared declarations of the
// kernel (token_kernel.cuh), its launcher (token.cu) and the decoder that fills the arguments.
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace ab {

struct KvGeom {
    uint32_t n_layer, n_kv, hd, page, max_pages;   // page = tokens per page
    size_t page_elems;                              // elements of one page (all layers, K and V)
};
__device__ __forceinline__ size_t kv_index(const KvGeom& g, uint32_t page_id, uint32_t layer, uint32_t kv, uint32_t head, uint32_t slot) {
    return (size_t)page_id * g.page_elems + ((((size_t)layer * 2 + kv) * g.n_kv + head) * g.page + slot) * g.hd;
}

__device__ __forceinline__ float ld_kv(const float* p) { return *p; }
__device__ __forceinline__ float ld_kv(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ void st_kv(float* p, float v) { *p = v; }
__device__ __forceinline__ void st_kv(__half* p, float v) { *p = __float2half_rn(v); }


template <typename T, int DPL> struct KvRow {
    static constexpr int BYTES = DPL * (int)sizeof(T);
    static constexpr int NW = BYTES >= 4 ? BYTES / 4 : 1;
    uint32_t w[NW];
    __device__ __forceinline__ void zero() {
#pragma unroll
        for (int i = 0; i < NW; ++i) w[i] = 0u;
    }
    __device__ __forceinline__ void load(const T* p) {
        if constexpr (BYTES == 32) {
            const uint4 a = reinterpret_cast<const uint4*>(p)[0], b = reinterpret_cast<const uint4*>(p)[1];
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w; w[4] = b.x; w[5] = b.y; w[6] = b.z; w[7] = b.w;
        } else if constexpr (BYTES == 16) {
            const uint4 a = *reinterpret_cast<const uint4*>(p);
            w[0] = a.x; w[1] = a.y; w[2] = a.z; w[3] = a.w;
        } else if constexpr (BYTES == 8) {
            const uint2 a = *reinterpret_cast<const uint2*>(p);
            w[0] = a.x; w[1] = a.y;
        } else if constexpr (BYTES == 4) {
            w[0] = *reinterpret_cast<const uint32_t*>(p);
        } else {
            w[0] = *reinterpret_cast<const unsigned short*>(p);
        }
    }
    __device__ __forceinline__ void from_float(const float* f) {      // values already rounded to T
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int i = 0; i < DPL; ++i) w[i] = __float_as_uint(f[i]);
        } else if constexpr (DPL >= 2) {
#pragma unroll
            for (int i = 0; i < DPL / 2; ++i) {
                const __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
        } else {
            w[0] = __half_as_ushort(__float2half_rn(f[0]));
        }
    }
    __device__ __forceinline__ void to_float(float (&f)[DPL]) const {
        if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int i = 0; i < DPL; ++i) f[i] = __uint_as_float(w[i]);
        } else if constexpr (DPL >= 2) {
#pragma unroll
            for (int i = 0; i < DPL / 2; ++i) {
                const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                f[2 * i] = v.x; f[2 * i + 1] = v.y;
            }
        } else {
            f[0] = __half2float(__ushort_as_half((unsigned short)w[0]));
        }
    }
};
template <typename T> __device__ __forceinline__ float kv_round(float v);
template <> __device__ __forceinline__ float kv_round<__half>(float v) { return __half2float(__float2half_rn(v)); }
template <> __device__ __forceinline__ float kv_round<float>(float v) { return v; }

// Sum a[0..NV) over the 32 lanes.  NV >= 32: lane l ends with the totals of values
// l*NV/32 .. in a[0..NV/32).  NV < 32: the 32/NV lanes v*32/NV .. end with value v in a[0].
template <int NV>
__device__ __forceinline__ void warp_reduce_scatter(float (&a)[NV], uint32_t lane) {
    int n = NV;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        if (n > 1) {
            const int h = n >> 1;
            const bool up = (lane & off) != 0;
#pragma unroll
            for (int i = 0; i < NV / 2; ++i) {
                if (i < h) {
                    const float send = up ? a[i] : a[i + h];
                    const float keep = up ? a[i + h] : a[i];
                    a[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
                }
            }
            n = h;
        } else {
            a[0] += __shfl_xor_sync(0xffffffffu, a[0], off);
        }
    }
}


constexpr int TK_NW = 16;                 // warps per CTA
constexpr int TK_THREADS = TK_NW * 32;
constexpr int TK_MAX_LAYERS = 126;        // exchange tags hold layer + 1 in 7 bits
constexpr int TK_MAX_SPLITS = 16;         // attention CTAs per query head
constexpr int TK_MAX_E = 3 * TK_THREADS * 4;   // widest residual stream the norm chain holds in registers
enum { TK_QKV = 0, TK_O, TK_GU, TK_DOWN, TK_LM, TK_PHASES };
enum { TKN_ATTN = 0, TKN_POST_ATTN, TKN_FFN, TKN_POST_FFW, TKN_Q, TKN_K, TKN_KINDS };

// How one matrix product is spread over the grid.  A CTA works on "sets" of RG row groups (16 rows
// each), KS warps per row group splitting K between them; with cpr > 1 the K range is first split over
// cpr CTAs whose partial outputs the consumer adds in order.  CTA c takes part iff c < G * cpr:
// set c / cpr, then every G-th; K part c % cpr.
struct TkPhase { int n_rg, pairs, RG, KS, cpr, G; };

struct TkLayer {
    const uint8_t* w[5];          // row-tiled weights: qkv (q,k,v rows as one tensor), o, gate, up, down
    const float* norm[TKN_KINDS]; // NULL = absent
    uint32_t window;              // sliding window of this layer (0 = attends to everything)
    uint32_t rope;                // which rotary table: 0 local, 1 global
};

struct TkArgs {
    const TkLayer* layers; int n_layer;
    int E, q_dim, k_dim, FF, V, H, KV;
    TkPhase ph[TK_PHASES];
    int s_max;                    // attention splits per head (<= 4, H * s_max <= grid)
    int wu_cap;                   // units (32 values) of the per-warp staging regions of the o-proj / down-proj inputs
    WeightRef embd; int embd_wt; float emb_scale;
    const uint8_t* lm_tiled; const float* out_norm;
    float eps, attn_scale, attn_cap, final_cap; int act;      // act: 0 = GeGLU, 1 = SwiGLU
    // sequence state
    int32_t* pos; int32_t* cur_tok; float* cur_val; const int32_t* prompt_len; const int32_t* prompt_tok;
    int32_t* gen_log; uint32_t log_ld;
    const int32_t* block_table; KvGeom geo; void* kv_pool;
    const float* cos_t[2]; const float* sin_t[2]; uint32_t n_pos;
    // exchange buffers: 8-byte packets {fp32 bits, tag}; every buffer has two halves used by even / odd layers
    uint2 *x_qkv, *x_att, *x_po, *x_act, *x_pd, *x_amax;
    uint32_t* seq;                // number of token steps run so far (advanced by the kernel)
    uint32_t* dead;               // sticky: a bounded wait ran out in an earlier step
    float* logits;                // optional [V] (soft-capped), NULL = not wanted
    float* h_out;                 // [E] hidden state after the last layer (verification reads)
    uint32_t* err;
    int with_lm;
    // diagnostics: when set, thread 0 of every CTA stores its SM clock at TK_TRACE_SLOTS points of one layer
    // (trace_layer) and of the LM head: trace[cta * TK_TRACE_SLOTS + slot]
    long long* trace; int trace_layer; int trace_phase;
    long long wait_cycles;        // bound of every device-side wait of one launch, in SM clocks (0 = default, about 0.3 s)
};
constexpr int TK_TRACE_SLOTS = 32;

// Exchange buffer sizes in packets (one half).
inline size_t tk_att_packets(const TkArgs& a, int hd) { return (size_t)a.H * a.s_max * (hd + 2); }

int launch_token(int wt, bool kv_half, int hd, const TkArgs& a, int grid, cudaStream_t st);
size_t token_smem_bytes(int wt, const TkArgs& a, int hd);
bool token_supported_hd(int hd);

}  // namespace ab
