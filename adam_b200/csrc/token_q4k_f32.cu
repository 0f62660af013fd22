// Instantiations of the token kernel for one weight block type and one KV-cache element type
// (kept in separate translation units so that they compile in parallel).
#include "token_kernel.cuh"

namespace ab {

int launch_token_q4k_f32(int hd, const TkArgs& a, int grid, size_t smem, cudaStream_t st) {
    void (*k)(const TkArgs) = nullptr;
    switch (hd) {
    case 32: k = k_token<WT_Q4_K, float, 32>; break;
    case 64: k = k_token<WT_Q4_K, float, 64>; break;
    case 128: k = k_token<WT_Q4_K, float, 128>; break;
    case 256: k = k_token<WT_Q4_K, float, 256>; break;
    default: return fail(ADAMAH_ERR_INVALID, "token kernel: head_dim %d", hd);
    }
    static bool attr[4] = {false, false, false, false};
    const int ai = hd == 32 ? 0 : hd == 64 ? 1 : hd == 128 ? 2 : 3;
    if (!attr[ai]) {
        if (cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024) != cudaSuccess)
            return fail(ADAMAH_ERR_BACKEND, "token kernel: cannot raise the shared-memory limit: %s", cudaGetErrorString(cudaGetLastError()));
        attr[ai] = true;
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)k, TK_THREADS, smem) != cudaSuccess || per_sm < 1)
        return fail(ADAMAH_ERR_BACKEND, "token kernel: does not fit on an SM with %zu bytes of shared memory", smem);
    if (grid > per_sm * g.sm_count) return fail(ADAMAH_ERR_BACKEND, "token kernel: %d CTAs cannot all be resident", grid);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(TK_THREADS); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;          // all CTAs resident at once, or the launch fails
    at[0].val.cooperative = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, k, a);
    if (e != cudaSuccess) return fail(ADAMAH_ERR_BACKEND, "token kernel: launch failed: %s", cudaGetErrorString(e));
    return ADAMAH_OK;
}

}  // namespace ab
