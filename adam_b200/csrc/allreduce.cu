// One-shot all-reduce (sum) of a small fp32 buffer over peer memory, for tensor-parallel decode.
//
// The reference has no multi-GPU path; this replaces an NCCL all-reduce of the 21 KB projection
// vector, which costs ~12 us per call inside a CUDA graph and is issued 2 x n_layer times per
// token.  One process per GPU; every rank owns a staging area and a flag array in its own memory
// and maps its peers' through CUDA IPC.
//
// Protocol of one call, per CTA c (CTA c of every rank handles the same slice and talks only to
// the CTAs c of the peers), with the call number s kept in device memory (so a replayed CUDA
// graph advances it by itself) and staging slot p = s & 1:
//   1. copy my slice of the buffer into my staging slot p;
//   2. fence, then store s into flag[c][my rank] of EVERY rank (peer stores);
//   3. wait until flag[c][q] >= s for all q in my own flag array (bounded number of polls; on expiry
//      set DEVERR_WAIT and carry on, so the kernel always ends);
//   4. read slice c of every rank's staging slot p (peer loads), add in rank order, write the buffer.
// Two slots are enough without an exit barrier: a rank can overwrite slot p only in call s + 2, and
// it passes the wait of call s + 1 only after every peer has started call s + 1, i.e. has finished
// reading for call s.  Sums are formed in rank order on every rank, so all ranks get the same bits.
// Launched like the decoder's kernels: it waits for the producer of the buffer with the
// programmatic-dependency wait and lets the next kernel (a GEMV) start its weight prefetch at once.
#include "common.cuh"

#include <cstring>

namespace ab {

constexpr uint32_t AR_MAX_RANKS = 8;
constexpr uint32_t AR_MAX_CTAS = 32;
constexpr uint32_t AR_MAX_COMMS = 4;
constexpr int AR_POLL_LIMIT = 1 << 20;      // about a second of polling

struct ArComm {
    bool used, open;
    uint32_t world, rank;
    size_t max_bytes;                       // capacity of one staging slot
    float* stage;                           // [2][max_bytes] in my memory
    uint32_t* flags;                        // [AR_MAX_CTAS][AR_MAX_RANKS] in my memory, then [AR_MAX_CTAS] call counters, then a
                                            // word that is set once a wait has run out (later calls do not wait again)
    float* peer_stage[AR_MAX_RANKS];        // mapped (my own entry = stage)
    uint32_t* peer_flags[AR_MAX_RANKS];
};
static ArComm g_ar[AR_MAX_COMMS];

struct ArPeers { float* stage[AR_MAX_RANKS]; uint32_t* flags[AR_MAX_RANKS]; };

__device__ __forceinline__ uint32_t ld_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" :: "l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_peer(const float4* p) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) k_allreduce(float* __restrict__ buf, uint32_t n4, ArPeers peers, uint32_t world, uint32_t rank,
                                                   size_t slot_floats, uint32_t* err) {
    __shared__ uint32_t s_seq;
    __shared__ int s_ok;
    const uint32_t c = blockIdx.x, tid = threadIdx.x;
    uint32_t* my_flags = peers.flags[rank];
    uint32_t* counter = my_flags + AR_MAX_CTAS * AR_MAX_RANKS + c;
    uint32_t* dead = my_flags + AR_MAX_CTAS * AR_MAX_RANKS + AR_MAX_CTAS;
    pdl_launch_dependents();
    pdl_wait();                                             // the buffer comes from the previous kernel
    if (tid == 0) { s_seq = *counter + 1u; s_ok = 1; }
    __syncthreads();
    const uint32_t s = s_seq, p = s & 1u;
    // slice of this CTA, in float4 units
    const uint32_t per = (n4 + gridDim.x - 1) / gridDim.x;
    const uint32_t i0 = min(c * per, n4), i1 = min(i0 + per, n4);
    float4* mine = reinterpret_cast<float4*>(peers.stage[rank] + (size_t)p * slot_floats);
    const float4* src = reinterpret_cast<const float4*>(buf);
    for (uint32_t i = i0 + tid; i < i1; i += blockDim.x) mine[i] = src[i];
    __threadfence_system();
    __syncthreads();
    if (tid < world) st_sys(peers.flags[tid] + c * AR_MAX_RANKS + rank, s);
    if (tid < world) {
        const uint32_t* f = my_flags + c * AR_MAX_RANKS + tid;
        int polls = *dead ? AR_POLL_LIMIT : 0;
        while ((int32_t)(ld_sys(f) - s) < 0) {
            if (++polls > AR_POLL_LIMIT) { atomicOr(err, DEVERR_WAIT); *dead = 1u; s_ok = 0; break; }
        }
    }
    __syncthreads();
    // Even after a timed-out wait the sum is formed (from whatever is there): the kernel must end.
    for (uint32_t i = i0 + tid; i < i1; i += blockDim.x) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (uint32_t q = 0; q < world; ++q) {
            const float4 v = ld_peer(reinterpret_cast<const float4*>(peers.stage[q] + (size_t)p * slot_floats) + i);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        reinterpret_cast<float4*>(buf)[i] = acc;
    }
    if (tid == 0) *counter = s;
}

static ArComm* get_ar(uint32_t id) { return (id < AR_MAX_COMMS && g_ar[id].used) ? &g_ar[id] : nullptr; }

void ar_destroy_all() {
    for (uint32_t i = 0; i < AR_MAX_COMMS; ++i) {
        ArComm& a = g_ar[i];
        if (!a.used) continue;
        for (uint32_t q = 0; q < a.world; ++q) {
            if (a.open && q != a.rank) { if (a.peer_stage[q]) cudaIpcCloseMemHandle(a.peer_stage[q]); if (a.peer_flags[q]) cudaIpcCloseMemHandle(a.peer_flags[q]); }
        }
        cudaFree(a.stage); cudaFree(a.flags);
        memset(&a, 0, sizeof a);
    }
}

}  // namespace ab

using namespace ab;

// Creates this rank's end of a communicator for buffers of up to max_bytes and returns the two
// 64-byte IPC handles (staging, flags) that the caller passes to every peer.
extern "C" int adam_b200_ar_create(uint32_t world, uint32_t rank, uint64_t max_bytes, uint32_t* id_out, void* handles_out) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    if (!id_out || !handles_out || world < 2 || world > AR_MAX_RANKS || rank >= world || max_bytes == 0)
        return fail(ADAMAH_ERR_INVALID, "ar_create: bad arguments (2..%u ranks)", AR_MAX_RANKS);
    uint32_t id = AR_MAX_COMMS;
    for (uint32_t i = 0; i < AR_MAX_COMMS; ++i) if (!g_ar[i].used) { id = i; break; }
    if (id == AR_MAX_COMMS) return fail(ADAMAH_ERR_MEMORY, "ar_create: communicator table full");
    ArComm& a = g_ar[id];
    memset(&a, 0, sizeof a);
    a.max_bytes = (size_t)((max_bytes + 255) & ~(uint64_t)255);
    const size_t flag_bytes = (AR_MAX_CTAS * AR_MAX_RANKS + AR_MAX_CTAS + 4) * 4;
    if (cudaMalloc(&a.stage, 2 * a.max_bytes) != cudaSuccess || cudaMalloc(&a.flags, flag_bytes) != cudaSuccess) {
        cudaGetLastError(); cudaFree(a.stage); cudaFree(a.flags); memset(&a, 0, sizeof a);
        return fail(ADAMAH_ERR_MEMORY, "ar_create: out of device memory");
    }
    cudaMemset(a.stage, 0, 2 * a.max_bytes);
    cudaMemset(a.flags, 0, flag_bytes);
    cudaDeviceSynchronize();
    cudaIpcMemHandle_t h[2];
    if (cudaIpcGetMemHandle(&h[0], a.stage) != cudaSuccess || cudaIpcGetMemHandle(&h[1], a.flags) != cudaSuccess) {
        const char* e = cudaGetErrorString(cudaGetLastError());
        cudaFree(a.stage); cudaFree(a.flags); memset(&a, 0, sizeof a);
        return fail(ADAMAH_ERR_BACKEND, "ar_create: cudaIpcGetMemHandle failed: %s", e);
    }
    memcpy(handles_out, h, sizeof h);
    a.used = true; a.world = world; a.rank = rank;
    *id_out = id;
    return ADAMAH_OK;
}

// all_handles: world x 128 bytes, rank q's pair as returned by its ar_create.  Every rank must have
// created its end (and zeroed its flags) before any rank's first all-reduce: barrier after this call.
extern "C" int adam_b200_ar_open(uint32_t id, const void* all_handles) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    if (!all_handles || a->open) return fail(ADAMAH_ERR_INVALID, "ar_open: bad arguments or already open");
    const cudaIpcMemHandle_t* h = (const cudaIpcMemHandle_t*)all_handles;
    for (uint32_t q = 0; q < a->world; ++q) {
        if (q == a->rank) { a->peer_stage[q] = a->stage; a->peer_flags[q] = a->flags; continue; }
        void *ps = nullptr, *pf = nullptr;
        if (cudaIpcOpenMemHandle(&ps, h[2 * q], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess ||
            cudaIpcOpenMemHandle(&pf, h[2 * q + 1], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
            return fail(ADAMAH_ERR_BACKEND, "ar_open: cannot map rank %u's memory: %s", q, cudaGetErrorString(cudaGetLastError()));
        a->peer_stage[q] = (float*)ps; a->peer_flags[q] = (uint32_t*)pf;
    }
    a->open = true;
    return ADAMAH_OK;
}

// In-place sum over all ranks of n_floats fp32 values at device address buf (n_floats % 4 == 0,
// buf 16-byte aligned), enqueued on the library's stream.  All ranks call it in the same order.
extern "C" int adam_b200_ar_allreduce(uint32_t id, uint64_t buf, uint32_t n_floats) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    if (!a->open) return fail(ADAMAH_ERR_INVALID, "ar_allreduce: call ar_open first");
    if (!buf || (buf & 15) || n_floats == 0 || (n_floats & 3) || (size_t)n_floats * 4 > a->max_bytes)
        return fail(ADAMAH_ERR_INVALID, "ar_allreduce: bad buffer (need 16-byte alignment, a multiple of 4 floats, at most %zu bytes)", a->max_bytes);
    ArPeers p;
    for (uint32_t q = 0; q < AR_MAX_RANKS; ++q) { p.stage[q] = a->peer_stage[q]; p.flags[q] = a->peer_flags[q]; }
    const uint32_t n4 = n_floats / 4;
    uint32_t grid = (n4 + 255) / 256;
    if (grid > AR_MAX_CTAS) grid = AR_MAX_CTAS;
    static const bool allow = !(getenv("ADAM_B200_PDL") && atoi(getenv("ADAM_B200_PDL")) == 0);
    launch_k(k_allreduce, dim3(grid), dim3(256), 0, g.stream, allow, (float*)(uintptr_t)buf, n4, p, a->world, a->rank, a->max_bytes / 4, g.dev_err);
    count_launch();
    int rc = check_launch("ar_allreduce");
    end_of_op();
    return rc;
}

extern "C" int adam_b200_ar_destroy(uint32_t id) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    cudaStreamSynchronize(g.stream);
    for (uint32_t q = 0; q < a->world; ++q)
        if (a->open && q != a->rank) { cudaIpcCloseMemHandle(a->peer_stage[q]); cudaIpcCloseMemHandle(a->peer_flags[q]); }
    cudaFree(a->stage); cudaFree(a->flags);
    memset(a, 0, sizeof *a);
    return ADAMAH_OK;
}
