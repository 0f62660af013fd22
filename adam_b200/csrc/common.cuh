// Shared declarations of libadam_b200: global context, maps, loc handles, and
// small device helpers.  One context per process, single-threaded callers, as
// in the reference runtime (adamah-MAIN/adamah/adamah.c:510-644).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#include "../../include/adam_b200.h"

namespace ab {

constexpr uint32_t MAX_MAPS    = 256;     // reference: MAX_MAPS 16 (adamah.c:30)
constexpr uint32_t MAX_HANDLES = 1u << 16; // reference: MAX_RES 2048 (adamah.c:31)

// Bits a kernel may OR into the device error word instead of faulting.
constexpr uint32_t DEVERR_OOB_MAP   = 1u;   // a loc pointed outside its map
constexpr uint32_t DEVERR_WAIT      = 2u;   // a bounded device-side wait ran out
constexpr uint32_t DEVERR_BAD_TOKEN = 4u;   // token id outside the vocabulary

struct Map {
    bool     used;
    uint32_t dtype;        // ADAMAH_DTYPE_*
    uint32_t word_size;    // bytes per element for F32 maps
    uint32_t pack_size;    // elements per pack (locs address packs)
    uint32_t n_packs;
    uint32_t group_size;   // Q4 map: elements per (scale, zero) pair
    uint64_t n_elems;      // pack_size * n_packs
    void*    buf;          // F32: float[n]; Q4: uint32[ceil(n/8)];
                           // GGUF_Q4_K: raw 144-byte superblocks;
                           // GGUF_Q4_0: quant plane (uint4 per block) then scale plane (half per block)
                           // GGUF_Q8_0: quant plane (32 B per block) then scale plane
                           // GGUF_Q5_0: nibble plane (16 B per block), high-bit plane (uint32 per block), scale plane
    size_t   bytes;
    float*   qparams;      // Q4 map: interleaved [scale, zero] per group
    uint32_t n_groups;
    uint4*   q40_qs;       // GGUF_Q4_0 planes (inside buf)
    __half*  q40_d;
    uint4*    b8_q;        // GGUF_Q8_0 / GGUF_Q5_0 planes (inside buf)
    uint32_t* b8_h;
    __half*   b8_d;
};

struct Handle {
    void*     dev;
    uint32_t  nbytes;
    bool      used;
    uint32_t* shadow;      // host copy of what the host uploaded (NULL for device-produced data)
};

struct Context {
    bool         inited;
    int          device;
    int          sm_count;
    size_t       total_mem;
    cudaStream_t stream;        // where everything is enqueued (own_stream unless the caller lent one)
    cudaStream_t own_stream;
    Map          maps[MAX_MAPS];
    Handle*      handles;       // [MAX_HANDLES], index = handle id
    uint32_t     handle_cursor;
    uint32_t     active_dtype;
    int          batch_depth;
    int          fusion_enabled;
    int          sched_mode;
    uint64_t     ticket;
    uint64_t     launches;      // kernels launched (graph nodes counted one by one)
    uint64_t     submits;       // stream synchronisations that closed a batch
    uint64_t     flushes;
    uint32_t*    dev_err;       // device error word
    bool         pdl;           // launch with programmatic stream serialization (set by the decoder while it enqueues a step)
};

extern Context g;

int  fail(int code, const char* fmt, ...);          // records text, returns code
bool ready();                                       // context initialised?
Map* get_map(uint32_t id);                          // NULL (+ error text) if absent
bool handle_ok(uint32_t h, uint32_t min_bytes);     // exists and holds >= min_bytes
inline uint32_t* hlocs(uint32_t h) { return (uint32_t*)g.handles[h].dev; }
inline float*    hdata(uint32_t h) { return (float*)g.handles[h].dev; }
// First word of a loc handle (the base of single-base ops).  Served from the host
// copy kept at upload time; device-produced handles cost one small read-back.
bool hfirst(uint32_t h, uint32_t* out);
uint32_t handle_alloc(uint32_t n_bytes);            // 0 on failure
int  check_launch(const char* what);                // cudaGetLastError -> status
inline void count_launch(uint64_t n = 1) { g.launches += n; }
void end_of_op();                                   // sync when not inside a batch

// Launch `k` on `st`; with `pdl` the launch may begin before the previous kernel in the
// stream has finished (programmatic dependent launch).  Every kernel launched that way
// calls pdl_wait() before it touches anything an earlier kernel writes.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*k)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, k, KArgs(args)...);
}


// The same with the CTAs of a launch grouped into thread-block clusters of `cluster_x` along x (gridDim.x a multiple of it).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k_cluster(void (*k)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = cluster_x; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, k, KArgs(args)...);
}

// ---- step trace (diagnostics build only: -DADAM_B200_STEP_TRACE, `python -m adam_b200.build --step-trace`) ----
// Kernels of the decode step stamp the global nanosecond timer at their phase boundaries into a buffer the host
// reads back (adam_b200_decoder_step_trace).  The regular build compiles none of it: no field, no parameter, no test.
#ifdef ADAM_B200_STEP_TRACE
#define STEP_TRACE_PARAM , long long* trace
#define STEP_TRACE_ARG(x) , (x)
__device__ __forceinline__ long long step_trace_now() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define STEP_STAMP(buf, index) do { if (buf) (buf)[index] = step_trace_now(); } while (0)
#else
#define STEP_TRACE_PARAM
#define STEP_TRACE_ARG(x)
#define STEP_STAMP(buf, index) do { } while (0)
#endif

// ---- device helpers --------------------------------------------------------

// Programmatic dependent launch: let the next kernel in the stream start its
// independent prologue now / wait until every earlier kernel's writes are visible.
// Both are no-ops for kernels launched the ordinary way.
// x / d for many x and one d, without the branchy IEEE division sequence: r = RN(1/d)
// once, then one Newton correction of the quotient (correctly rounded whenever nothing
// under- or overflows on the way).
__device__ __forceinline__ float div_by(float x, float d, float r) {
    const float q = x * r;
    return fmaf(fmaf(-q, d, x), r, q);
}

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a whole CTA (blockDim.x a multiple of 32, at most 1024).  `red` is
// shared scratch of at least 33 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // protect `red` from a previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = (lane < nw) ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = (lane < nw) ? red[lane] : -3.402823466e+38f;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// tanh-approximated GELU exactly as the reference's numpy decoder writes it
// (tests/diagnostics/diag_inference.py:941-943).
__device__ __forceinline__ float gelu_tanh(float x) {
    const float k = 0.7978845608028654f;        // float32(sqrt(2/pi))
    float x3 = x * x * x;
    float inner = k * (x + 0.044715f * x3);
    return 0.5f * x * (1.0f + tanhf(inner));
}
__device__ __forceinline__ float silu_clip(float x) {
    float c = fminf(fmaxf(x, -80.f), 80.f);     // diag_inference.py:945-946
    return x * (1.0f / (1.0f + expf(-c)));
}

}  // namespace ab
