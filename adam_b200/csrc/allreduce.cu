// One-shot all-reduce (sum) of a small fp32 buffer over peer memory, for tensor-parallel decode.
//
// The reference has no multi-GPU path; this replaces an NCCL all-reduce of the 21 KB projection
// vector, which costs ~12 us per call inside a CUDA graph and is issued 2 x n_layer times per
// token (and, in a prefill chunk, of up to 64 such rows).  One process per GPU; every rank owns a staging area in its own memory and maps its
// peers' through CUDA IPC.
//
// Protocol of one call (number s, kept in device memory so that a replayed CUDA graph advances it
// by itself; every CTA keeps a copy of the same number and CTA 0 also writes the copies of the CTAs
// a smaller call does not launch, so calls of different sizes may follow one another; staging slot
// p = s & 1).  Data and hand-shake travel together, as in a low-latency
// ring protocol: every pair of floats is sent as one 16-byte packet { x, s, y, s } whose two 8-byte
// halves each carry the call number, so the receiver needs no separate flag and no fence.
//   1. every thread reads its floats of the buffer and stores the packets into region
//      [p][my rank] of EVERY peer's staging area (posted peer stores);
//   2. it then polls region [p][q] of its OWN staging area for every peer q until both halves of
//      the packet carry s (bounded by the SM clock: a few seconds by default, settable per
//      communicator; on expiry DEVERR_WAIT is recorded, a sticky word stops later calls from
//      waiting again until adam_b200_ar_reset clears it, and the kernel carries on to its end);
//   3. it adds the contributions in rank order (its own from registers) and writes the buffer.
// Two slots are enough without an exit barrier: a peer overwrites my slot p only in its call
// s + 2, which it reaches only after my packets of call s + 1 arrived, i.e. after I finished call s.
// Sums are formed in rank order on every rank, so all ranks get the same bits.  Launched like the
// decoder's kernels: it waits for the producer of the buffer with the programmatic-dependency wait
// and lets the next kernel (a GEMV) start its weight prefetch at once.  A packet at a given
// place of a slot only ever carries growing call numbers, so a stale one is never taken for the
// expected one whatever the sizes of earlier calls were.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace ab {

constexpr uint32_t AR_MAX_RANKS = 8;
constexpr uint32_t AR_MAX_CTAS = 64;
constexpr uint32_t AR_MAX_COMMS = 4;
constexpr long long AR_WAIT_CYCLES_DEFAULT = 10LL * 1000 * 1000 * 1000;   // about 5 s at 2 GHz: rank skew on a shared host (graph instantiation, module load, a preempted host thread) can reach a second

struct ArComm {
    bool used, open;
    uint32_t world, rank;
    size_t max_floats;                      // capacity of one (slot, rank) region, in floats
    uint4* stage;                           // [2 slots][world][max_floats / 2] packets in my memory
    uint32_t* state;                        // [AR_MAX_CTAS] call counters, then the sticky "a wait ran out" word
    uint4* peer_stage[AR_MAX_RANKS];        // mapped (my own entry = stage)
    long long wait_cycles;                  // bound of the wait of one call, in SM clocks
    bool local_peers;                       // peers are other communicators of this process (test set-up): nothing to unmap
};
static ArComm g_ar[AR_MAX_COMMS];

struct ArPeers { uint4* stage[AR_MAX_RANKS]; };

__device__ __forceinline__ void st_packet(uint4* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_packet(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

__global__ void __launch_bounds__(256) k_allreduce(float* __restrict__ buf, uint32_t n2, ArPeers peers, uint32_t world, uint32_t rank,
                                                   size_t region, uint32_t* __restrict__ state, uint32_t* err, long long wait_cycles) {
    const uint32_t c = blockIdx.x, tid = threadIdx.x;
    uint32_t* counter = state + c;
    uint32_t* dead = state + AR_MAX_CTAS;
    pdl_launch_dependents();
    pdl_wait();                                             // the buffer comes from the previous kernel
    uint32_t s = *counter + 1u;
    if (s == 0u) s = 1u;                                    // 0 is what untouched staging memory holds
    const uint32_t p = s & 1u;
    bool gave_up = *dead != 0u;                            // an earlier call ran out of time: do not wait again
    const long long deadline = clock64() + wait_cycles;
    // slice of this CTA, in float2 units
    const uint32_t per = (n2 + gridDim.x - 1) / gridDim.x;
    const uint32_t i0 = min(c * per, n2), i1 = min(i0 + per, n2);
    float2* b2 = reinterpret_cast<float2*>(buf);
    for (uint32_t i = i0 + tid; i < i1; i += blockDim.x) {
        const float2 v = b2[i];
        const uint4 pk = make_uint4(__float_as_uint(v.x), s, __float_as_uint(v.y), s);
        for (uint32_t q = 0; q < world; ++q)
            if (q != rank) st_packet(peers.stage[q] + ((size_t)p * world + rank) * region + i, pk);
    }
    const uint4* mine = peers.stage[rank] + (size_t)p * world * region;
    for (uint32_t i = i0 + tid; i < i1; i += blockDim.x) {
        const float2 v = b2[i];
        float2 acc = make_float2(0.f, 0.f);
        for (uint32_t q = 0; q < world; ++q) {
            if (q == rank) { acc.x += v.x; acc.y += v.y; continue; }
            const uint4* src = mine + (size_t)q * region + i;
            uint4 pk = ld_packet(src);
            uint32_t polls = 0;
            while ((pk.y != s || pk.w != s) && !gave_up) {
                if ((++polls & 31u) == 0u && clock64() > deadline) { atomicOr(err, DEVERR_WAIT); *dead = 1u; gave_up = true; break; }
                pk = ld_packet(src);
            }
            acc.x += __uint_as_float(pk.x); acc.y += __uint_as_float(pk.z);
        }
        b2[i] = acc;
    }
    __syncthreads();
    if (tid == 0) *counter = s;
    if (c == 0 && tid >= gridDim.x && tid < AR_MAX_CTAS) state[tid] = s;   // copies of the CTAs this call did not launch
}

static ArComm* get_ar(uint32_t id) { return (id < AR_MAX_COMMS && g_ar[id].used) ? &g_ar[id] : nullptr; }

void ar_destroy_all() {
    for (uint32_t i = 0; i < AR_MAX_COMMS; ++i) {
        ArComm& a = g_ar[i];
        if (!a.used) continue;
        for (uint32_t q = 0; q < a.world; ++q)
            if (a.open && !a.local_peers && q != a.rank && a.peer_stage[q]) cudaIpcCloseMemHandle(a.peer_stage[q]);
        cudaFree(a.stage); cudaFree(a.state);
        memset(&a, 0, sizeof a);
    }
}

}  // namespace ab

using namespace ab;

// Creates this rank's end of a communicator for buffers of up to max_bytes and returns its
// 64-byte IPC handle (128 bytes are written, the second half is reserved and zero), which the
// caller passes to every peer.
extern "C" int adam_b200_ar_create(uint32_t world, uint32_t rank, uint64_t max_bytes, uint32_t* id_out, void* handles_out) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    if (!id_out || !handles_out || world < 2 || world > AR_MAX_RANKS || rank >= world || max_bytes == 0)
        return fail(ADAMAH_ERR_INVALID, "ar_create: bad arguments (2..%u ranks)", AR_MAX_RANKS);
    uint32_t id = AR_MAX_COMMS;
    for (uint32_t i = 0; i < AR_MAX_COMMS; ++i) if (!g_ar[i].used) { id = i; break; }
    if (id == AR_MAX_COMMS) return fail(ADAMAH_ERR_MEMORY, "ar_create: communicator table full");
    ArComm& a = g_ar[id];
    memset(&a, 0, sizeof a);
    a.max_floats = (size_t)(((max_bytes + 3) / 4 + 63) & ~(uint64_t)63);
    const size_t stage_bytes = 2 * (size_t)world * (a.max_floats / 2) * sizeof(uint4);
    const size_t state_bytes = (AR_MAX_CTAS + 4) * 4;
    if (cudaMalloc(&a.stage, stage_bytes) != cudaSuccess || cudaMalloc(&a.state, state_bytes) != cudaSuccess) {
        cudaGetLastError(); cudaFree(a.stage); cudaFree(a.state); memset(&a, 0, sizeof a);
        return fail(ADAMAH_ERR_MEMORY, "ar_create: out of device memory");
    }
    cudaMemset(a.stage, 0, stage_bytes);
    cudaMemset(a.state, 0, state_bytes);
    cudaDeviceSynchronize();
    cudaIpcMemHandle_t h[2];
    memset(h, 0, sizeof h);
    if (cudaIpcGetMemHandle(&h[0], a.stage) != cudaSuccess) {
        const char* e = cudaGetErrorString(cudaGetLastError());
        cudaFree(a.stage); cudaFree(a.state); memset(&a, 0, sizeof a);
        return fail(ADAMAH_ERR_BACKEND, "ar_create: cudaIpcGetMemHandle failed: %s", e);
    }
    memcpy(handles_out, h, sizeof h);
    a.used = true; a.world = world; a.rank = rank;
    a.wait_cycles = AR_WAIT_CYCLES_DEFAULT;
    if (const char* e = getenv("ADAM_B200_AR_WAIT_US")) { const long long us = atoll(e); if (us > 0) a.wait_cycles = us * 2000; }
    *id_out = id;
    return ADAMAH_OK;
}

// all_handles: world x 128 bytes, rank q's as returned by its ar_create.  Every rank must have
// created its end (staging zeroed) before any rank's first all-reduce: barrier after this call.
extern "C" int adam_b200_ar_open(uint32_t id, const void* all_handles) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    if (!all_handles || a->open) return fail(ADAMAH_ERR_INVALID, "ar_open: bad arguments or already open");
    const cudaIpcMemHandle_t* h = (const cudaIpcMemHandle_t*)all_handles;
    for (uint32_t q = 0; q < a->world; ++q) {
        if (q == a->rank) { a->peer_stage[q] = a->stage; continue; }
        void* ps = nullptr;
        if (cudaIpcOpenMemHandle(&ps, h[2 * q], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess)
            return fail(ADAMAH_ERR_BACKEND, "ar_open: cannot map rank %u's memory: %s", q, cudaGetErrorString(cudaGetLastError()));
        a->peer_stage[q] = (uint4*)ps;
    }
    a->open = true;
    return ADAMAH_OK;
}

// In-place sum over all ranks of n_floats fp32 values at device address buf (n_floats % 2 == 0,
// buf 8-byte aligned), enqueued on the library's stream.  All ranks call it in the same order.
extern "C" int adam_b200_ar_allreduce(uint32_t id, uint64_t buf, uint32_t n_floats) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    if (!a->open) return fail(ADAMAH_ERR_INVALID, "ar_allreduce: call ar_open first");
    if (!buf || (buf & 7) || n_floats == 0 || (n_floats & 1) || (size_t)n_floats > a->max_floats)
        return fail(ADAMAH_ERR_INVALID, "ar_allreduce: bad buffer (need 8-byte alignment, an even count, at most %zu floats)", a->max_floats);
    ArPeers p;
    for (uint32_t q = 0; q < AR_MAX_RANKS; ++q) p.stage[q] = a->peer_stage[q];
    const uint32_t n2 = n_floats / 2;
    uint32_t grid = (n2 + 255) / 256;
    if (grid > AR_MAX_CTAS) grid = AR_MAX_CTAS;
    static const bool allow = !(getenv("ADAM_B200_PDL") && atoi(getenv("ADAM_B200_PDL")) == 0);
    launch_k(k_allreduce, dim3(grid), dim3(256), 0, g.stream, allow, (float*)(uintptr_t)buf, n2, p, a->world, a->rank, a->max_floats / 2,
             a->state, g.dev_err, a->wait_cycles);
    count_launch();
    int rc = check_launch("ar_allreduce");
    end_of_op();
    return rc;
}

// Bound of the wait of one call, in microseconds (about 5 s by default; ADAM_B200_AR_WAIT_US at creation).
extern "C" int adam_b200_ar_set_wait_us(uint32_t id, uint64_t wait_us) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    if (wait_us == 0 || wait_us > 600ull * 1000 * 1000) return fail(ADAMAH_ERR_INVALID, "ar_set_wait_us: 1 .. 600000000");
    a->wait_cycles = (long long)wait_us * 2000;
    return ADAMAH_OK;
}

// Clears the sticky word a timed-out call leaves behind (calls made while it is set do not wait and so
// return sums of whatever lies in the staging area).  Every rank resets, then the ranks meet at a host
// barrier, before the next call; the call counters are left alone (they only ever grow).
extern "C" int adam_b200_ar_reset(uint32_t id) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    cudaStreamSynchronize(g.stream);
    if (cudaMemset(a->state + AR_MAX_CTAS, 0, 4) != cudaSuccess) return fail(ADAMAH_ERR_BACKEND, "ar_reset: %s", cudaGetErrorString(cudaGetLastError()));
    return ADAMAH_OK;
}

// 1 if a call on this communicator ran out of time since creation / the last reset, else 0.
extern "C" int adam_b200_ar_timed_out(uint32_t id) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    uint32_t v = 0;
    cudaStreamSynchronize(g.stream);
    if (cudaMemcpy(&v, a->state + AR_MAX_CTAS, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return fail(ADAMAH_ERR_BACKEND, "ar_timed_out: %s", cudaGetErrorString(cudaGetLastError()));
    return v ? 1 : 0;
}

// Test set-up: connects communicators created in THIS process on this GPU (ids[q] = the communicator that
// plays rank q) by plain pointers instead of IPC handles, which a process cannot open on its own memory.
// Lets one process call one "rank" while nobody plays the others, so that a bounded wait can be seen to
// run out and return.
extern "C" int adam_b200_ar_open_local(uint32_t id, const uint32_t* ids, uint32_t n) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    if (!ids || n != a->world || a->open) return fail(ADAMAH_ERR_INVALID, "ar_open_local: bad arguments or already open");
    for (uint32_t q = 0; q < n; ++q) {
        ArComm* b = get_ar(ids[q]);
        if (!b || b->world != a->world || b->rank != q || b->max_floats != a->max_floats) return fail(ADAMAH_ERR_INVALID, "ar_open_local: communicator %u does not play rank %u", ids[q], q);
        a->peer_stage[q] = b->stage;
    }
    a->open = true; a->local_peers = true;
    return ADAMAH_OK;
}

extern "C" int adam_b200_ar_destroy(uint32_t id) {
    ArComm* a = get_ar(id);
    if (!a) return ADAMAH_ERR_NOT_FOUND;
    cudaStreamSynchronize(g.stream);
    for (uint32_t q = 0; q < a->world; ++q)
        if (a->open && !a->local_peers && q != a->rank) cudaIpcCloseMemHandle(a->peer_stage[q]);
    cudaFree(a->stage); cudaFree(a->state);
    memset(a, 0, sizeof *a);
    return ADAMAH_OK;
}
