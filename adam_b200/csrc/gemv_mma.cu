// Host-side launch logic of the tensor-core Q4_0 GEMV (kernel in gemv_mma.cuh).
#include "gemv_mma.cuh"

namespace ab {

constexpr int MMA_SMEM_LIMIT = 200 * 1024;

typedef void (*MmaKernel)(const GemvArgs, const uint8_t*, const uint8_t*, int);

bool gemv_mma_supports(const GemvArgs& a) {
    if (a.N <= 0 || a.K <= 0 || a.B <= 0) return false;
    if (a.N % 16 || a.K % 64) return false;
    if (a.h_in) { if ((a.K >> 2) > 3 * 256 || (a.ldx & 3)) return false; }
    else if (((uintptr_t)a.x & 15) || (a.ldx & 3)) return false;
    const size_t smem1 = (size_t)(a.K / 32) * (2 * 64 + 4) + 8 * 4 * 3 * 576 + 128;
    return smem1 <= (size_t)MMA_SMEM_LIMIT;
}

struct MmaInfo { bool attr; size_t occ_smem; int per_sm; };
static MmaInfo g_mma_info[2][2];

int launch_gemv_mma(const uint8_t* t0, const uint8_t* t1, GemvArgs a, cudaStream_t stream) {
    if (!gemv_mma_supports(a)) return fail(ADAMAH_ERR_INVALID, "gemv_mma: shape not supported");
    const bool pair = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    if (pair && !t1) return fail(ADAMAH_ERR_INVALID, "gemv_mma: second matrix missing");
    const int units = a.K / 32, pairs = a.K / 64, n_rg = a.N / 16;
    // batch rows per pass: 1 (two staged columns) or up to 4 (eight columns)
    int nb_max = 4;
    while (nb_max > 1 && (size_t)units * nb_max * (2 * 64 + 4) + 8 * 4 * 3 * 576 + 128 > (size_t)MMA_SMEM_LIMIT) nb_max >>= 1;
    for (int b0 = 0; b0 < a.B; b0 += nb_max) {
        GemvArgs g1 = a;
        g1.B = (a.B - b0 < nb_max) ? a.B - b0 : nb_max;
        if (a.x) g1.x = a.x + (size_t)b0 * a.ldx;
        if (a.h_in) g1.h_in = a.h_in + (size_t)b0 * a.ldx;
        if (a.add_src) g1.add_src = a.add_src + (size_t)b0 * a.ldx;
        if (a.h_out) g1.h_out = a.h_out + (size_t)b0 * a.ldx;
        if (a.y) g1.y = a.y + (size_t)b0 * a.ldy;
        if (a.out_tok) g1.out_tok = a.out_tok + b0;
        if (a.out_tok_f32) g1.out_tok_f32 = a.out_tok_f32 + b0;
        const int ncol = g1.B == 1 ? 2 : 8;
        const size_t ring_bytes = (size_t)8 * (pair ? 2 : 4) * 3 * 576 * (pair ? 2 : 1);
        const size_t smem = (((size_t)units * (ncol * 64 + (ncol / 2) * 4) + 127) & ~(size_t)127) + ring_bytes;
        g1.err = g.dev_err;
        MmaKernel k = ncol == 2 ? (pair ? k_gemv_mma<2, true> : k_gemv_mma<2, false>) : (pair ? k_gemv_mma<8, true> : k_gemv_mma<8, false>);
        MmaInfo& ki = g_mma_info[ncol == 2 ? 0 : 1][pair ? 1 : 0];
        if (!ki.attr) {
            if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM_LIMIT) != cudaSuccess)
                return fail(ADAMAH_ERR_BACKEND, "gemv_mma: cannot raise the shared-memory limit");
            ki.attr = true;
        }
        if (ki.occ_smem != smem) {
            int per_sm = 0;
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, 256, smem);
            ki.per_sm = per_sm < 1 ? 1 : per_sm; ki.occ_smem = smem;
        }
        // K slices per row group: the fewest that still give every SM two CTAs; small
        // problems take the most parallel split.
        int KS = 8;
        for (int c = 1; c <= 8; c <<= 1) {
            if (c > pairs) break;
            const int n_sets = (n_rg + 8 / c - 1) / (8 / c);
            if (n_sets >= 2 * g.sm_count) { KS = c; break; }
        }
        while (KS > pairs) KS >>= 1;
        if (KS < 1) KS = 1;
        const int n_sets = (n_rg + 8 / KS - 1) / (8 / KS);
        int grid = g.sm_count * ki.per_sm;
        if (grid > n_sets) grid = n_sets;
        if (a.epi == EPI_ARGMAX && grid > gemv_max_grid()) grid = gemv_max_grid();
        if (a.max_grid > 0 && grid > a.max_grid) grid = a.max_grid;
        if (grid < 1) grid = 1;
        if (launch_k(k, dim3(grid), dim3(256), smem, stream, g.pdl, g1, t0, t1, KS) != cudaSuccess) return fail(ADAMAH_ERR_BACKEND, "gemv_mma: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        count_launch();
    }
    return ADAMAH_OK;
}

}  // namespace ab
