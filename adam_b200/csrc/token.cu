// Launcher of the token kernel (token_kernel.cuh; instantiated per weight type / cache type in token_*.cu).
#include "token_kernel.cuh"

namespace ab {

int launch_token_q40_f16(int hd, const TkArgs& a, int grid, size_t smem, cudaStream_t st);
int launch_token_q40_f32(int hd, const TkArgs& a, int grid, size_t smem, cudaStream_t st);
int launch_token_q4k_f16(int hd, const TkArgs& a, int grid, size_t smem, cudaStream_t st);
int launch_token_q4k_f32(int hd, const TkArgs& a, int grid, size_t smem, cudaStream_t st);

bool token_supported_hd(int hd) { return hd == 32 || hd == 64 || hd == 128 || hd == 256; }

size_t token_smem_bytes(int wt, const TkArgs& a, int hd) {
    const int ring = wt == WT_Q4_0 ? TkGeo<WT_Q4_0>::RING_BYTES : TkGeo<WT_Q4_K>::RING_BYTES;
    return tk_smem_layout(a.E / 32, hd, a.wu_cap, a.E, a.n_layer, ring).total;
}

int launch_token(int wt, bool kv_half, int hd, const TkArgs& a, int grid, cudaStream_t st) {
    const size_t smem = token_smem_bytes(wt, a, hd);
    int rc;
    if (wt == WT_Q4_0) rc = kv_half ? launch_token_q40_f16(hd, a, grid, smem, st) : launch_token_q40_f32(hd, a, grid, smem, st);
    else rc = kv_half ? launch_token_q4k_f16(hd, a, grid, smem, st) : launch_token_q4k_f32(hd, a, grid, smem, st);
    if (rc == ADAMAH_OK) count_launch();
    return rc;
}

}  // namespace ab
