// LM head + arg-max without any allocation: map_matvec_argmax_t_xq4_static_dev.
//
// Who needs it.  Some callers of this library are not allowed to allocate device
// memory when they call in: a serving loop that has handed the whole card to its own
// pool and treats any cudaMalloc as a bug, a caller inside a latency-critical section
// where the implicit device-wide synchronisation of cudaMalloc/cudaFree would stall
// other streams, or a process running with a memory cap that is already reached.
// The regular entry point (map_matvec_argmax_t_xq4_dev in ops.cu) creates its
// partial-result scratch with cudaMalloc on first use; this variant keeps the same
// scratch in a fixed array that is part of the library image instead.
//
// The price.  The array below occupies NOALLOC_SCRATCH_BYTES (about 32 KB) of device
// memory on every GPU on which the library has been initialised, from that moment (the
// CUDA runtime loads the module that holds it when it is first touched, which
// adamah_init does through adam_b200_noalloc_prepare) until the process exits, used or
// not.  Its size fixes the largest problem: one (value, index) slot per group of
// `rows_per_group` rows, at most NOALLOC_MAX_GROUPS slots, so N may not exceed
// NOALLOC_MAX_GROUPS * rows_per_group (1,048,576 rows at the default 256).  Larger N is
// refused with ADAMAH_ERR_INVALID and a message; it is never silently truncated.
//
// Sharing.  Every call on a device uses the same array, and the array keeps whatever
// the previous call left in it.  The only word that has to start at zero, the arrival
// counter, is cleared on the stream before each launch; the partial slots are fully
// rewritten by the kernel before they are read.  Two calls that overlap on the GPU
// (different streams, or one call per thread) would race on the array: issue them from
// one thread, as every other entry point of this library already requires.
//
// Set-up.  Host code cannot use the array's name as an address -- in host code it is only
// a stand-in symbol -- so once per device the runtime is asked for the real device address
// (cudaGetSymbolAddress, with that device current; the caller's current device is put back)
// and the answer is kept.  adamah_init / adamah_init_ex do this (adam_b200_noalloc_prepare),
// so that no call on the hot path is the first touch of the module: that first touch may
// itself load the module and synchronise, which is exactly what these callers want to avoid.
// A process that skips the initialisation call gets the look-up on the first call of the
// entry point instead; make that call before starting any stream capture.
#include "common.cuh"
#include "gemv.cuh"

namespace ab {

int weight_ref(const Map* m, uint64_t off, uint64_t n_elems, int* wtype, WeightRef* w);
int run_gemv(uint32_t map_id, uint64_t off, int wtype, GemvArgs& ga);

constexpr uint32_t NOALLOC_MAX_GROUPS = 4096;
struct NoAllocScratch {
    float        val[NOALLOC_MAX_GROUPS];
    int          idx[NOALLOC_MAX_GROUPS];
    unsigned int ticket;
};
constexpr size_t NOALLOC_SCRATCH_BYTES = sizeof(NoAllocScratch);

static __device__ __align__(256) unsigned char g_noalloc_scratch[sizeof(NoAllocScratch)];

constexpr int MAX_DEVICES = 64;
static NoAllocScratch* g_scratch_addr[MAX_DEVICES];     // per device, resolved on first use

static int scratch_for_current_device(NoAllocScratch** out) {
    const int dev = g.device;
    if (dev < 0 || dev >= MAX_DEVICES) return fail(ADAMAH_ERR_INVALID, "no-alloc arg-max: device ordinal %d out of range", dev);
    if (!g_scratch_addr[dev]) {
        int before = -1;
        cudaGetDevice(&before);
        cudaError_t e = cudaSetDevice(dev);
        if (e != cudaSuccess) return fail(ADAMAH_ERR_BACKEND, "no-alloc arg-max: cudaSetDevice(%d): %s", dev, cudaGetErrorString(e));
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (before >= 0 && before != dev) cudaSetDevice(before);
        if (e != cudaSuccess || !p) return fail(ADAMAH_ERR_BACKEND, "no-alloc arg-max: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_scratch_addr[dev] = reinterpret_cast<NoAllocScratch*>(p);
    }
    *out = g_scratch_addr[dev];
    return ADAMAH_OK;
}

// Called by adamah_init_ex: resolves the array on the library's device ahead of any hot-path call.
int noalloc_prepare() {
    NoAllocScratch* s = nullptr;
    return scratch_for_current_device(&s);
}

}  // namespace ab

using namespace ab;

extern "C" int adam_b200_noalloc_prepare(void) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    return noalloc_prepare();
}

// Same arguments and result as map_matvec_argmax_t_xq4_dev: the index of the largest of
// the N dot products W[n,:] . x (ties to the lower index) is stored as float32 at
// locs_dst[0] of map_act.  Calls no cudaMalloc / cudaFree / allocating routine.
extern "C" int map_matvec_argmax_t_xq4_static_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h,
                                                  uint32_t idx_tmp_h, uint32_t val_tmp_h, uint32_t dst_h,
                                                  uint32_t K, uint32_t N, uint32_t rows_per_group) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    // the two scratch handles are not used, but both variants reject the same bad arguments
    if (!handle_ok(idx_tmp_h, 4) || !handle_ok(val_tmp_h, 4)) return ADAMAH_ERR_NOT_FOUND;
    Map* a = get_map(map_act);
    Map* w = get_map(map_wt);
    if (!a || !w) return ADAMAH_ERR_NOT_FOUND;
    if (a->dtype != ADAMAH_DTYPE_F32 || a->pack_size != 1) return fail(ADAMAH_ERR_INVALID, "no-alloc arg-max: map %u must be float32 with pack_size 1", map_act);
    if (w->dtype != ADAMAH_DTYPE_GGUF_Q4_0 && w->dtype != ADAMAH_DTYPE_GGUF_Q4_K)
        return fail(ADAMAH_ERR_INVALID, "no-alloc arg-max: weights must be in a GGUF-block map");
    if (!K || !N) return fail(ADAMAH_ERR_INVALID, "no-alloc arg-max: empty shape");
    if (rows_per_group == 0) rows_per_group = 256;
    const uint64_t n_groups = ((uint64_t)N + rows_per_group - 1) / rows_per_group;
    if (n_groups > NOALLOC_MAX_GROUPS)
        return fail(ADAMAH_ERR_INVALID, "no-alloc arg-max: N=%u needs %llu partial slots of %u rows, the fixed scratch holds %u "
                    "(max N = %llu); use map_matvec_argmax_t_xq4_dev for larger N", N, (unsigned long long)n_groups, rows_per_group,
                    NOALLOC_MAX_GROUPS, (unsigned long long)NOALLOC_MAX_GROUPS * rows_per_group);
    uint32_t ab_, bb, db;
    if (!hfirst(a_h, &ab_) || !hfirst(b_h, &bb) || !hfirst(dst_h, &db)) return ADAMAH_ERR_NOT_FOUND;
    if ((uint64_t)ab_ + K > a->n_elems || db >= a->n_elems) return fail(ADAMAH_ERR_INVALID, "no-alloc arg-max: activation range beyond map %u", map_act);
    if (ab_ % 4) return fail(ADAMAH_ERR_INVALID, "no-alloc arg-max: activation offset must be a multiple of 4 elements");
    int wtype; GemvArgs ga = {};
    int rc = weight_ref(w, bb, (uint64_t)N * K, &wtype, &ga.w0);
    if (rc) return rc;
    NoAllocScratch* s = nullptr;
    if ((rc = scratch_for_current_device(&s))) return rc;
    // the arrival counter must start at zero whatever the previous call left behind
    if (cudaMemsetAsync(&s->ticket, 0, sizeof(unsigned int), g.stream) != cudaSuccess)
        return fail(ADAMAH_ERR_BACKEND, "no-alloc arg-max: cannot clear the arrival counter");
    ga.part_val = s->val; ga.part_idx = s->idx; ga.ticket = &s->ticket;
    ga.max_grid = (int)n_groups;                 // one partial slot per CTA, never more than the slots that exist
    ga.x = (const float*)a->buf + ab_; ga.ldx = (int)K; ga.y = nullptr; ga.ldy = (int)N; ga.N = (int)N; ga.K = (int)K; ga.B = 1;
    ga.epi = EPI_ARGMAX; ga.out_tok = nullptr; ga.out_tok_f32 = (float*)a->buf + db;
    if ((rc = run_gemv(map_wt, bb, wtype, ga))) return rc;
    rc = check_launch("map_matvec_argmax_t_xq4_static_dev");
    end_of_op();
    return rc;
}
