// Host-side launch logic of the tensor-core Q4_0 GEMV (kernel in gemv_mma.cuh).
#include "gemv_mma.cuh"

namespace ab {

constexpr int MMA_SMEM_LIMIT = 200 * 1024;

typedef void (*MmaKernel)(const GemvArgs, const uint8_t*, const uint8_t*, int);

// staged bytes per 32-activation block: NCOL columns of 32 bytes + NCOL/2 pre-summed floats
static size_t x_bytes(int units, int ncol) { return (((size_t)units * (ncol * 32 + (ncol / 2) * 4)) + 127) & ~(size_t)127; }
static size_t ring_bytes(int n_warps) { return (size_t)n_warps * MMA_RING_BYTES_PER_WARP; }

bool gemv_mma_supports(const GemvArgs& a) {
    if (a.N <= 0 || a.K <= 0 || a.B <= 0) return false;
    if (a.N % 16 || a.K % 64) return false;
    if (a.h_in) { if ((a.K >> 2) > 3 * 256 || (a.ldx & 3)) return false; }
    else if (((uintptr_t)a.x & 15) || (a.ldx & 3)) return false;
    return x_bytes(a.K / 32, 4) + ring_bytes(8) <= (size_t)MMA_SMEM_LIMIT;
}

struct MmaInfo { bool attr; size_t occ_smem; int occ_threads; int per_sm; };
static MmaInfo g_mma_info[3][2];

int launch_gemv_mma(const uint8_t* t0, const uint8_t* t1, GemvArgs a, cudaStream_t stream) {
    if (!gemv_mma_supports(a)) return fail(ADAMAH_ERR_INVALID, "gemv_mma: shape not supported");
    const bool pair = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    if (pair && !t1) return fail(ADAMAH_ERR_INVALID, "gemv_mma: second matrix missing");
    const int units = a.K / 32, pairs = a.K / 64, n_rg = a.N / 16;
    // batch rows per pass: as many of 4, 2, 1 as shared memory allows
    int nb_max = 4;
    while (nb_max > 1 && x_bytes(units, 4 * nb_max) + ring_bytes(8) > (size_t)MMA_SMEM_LIMIT) nb_max >>= 1;
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
        const int ncol = g1.B == 1 ? 4 : (g1.B == 2 ? 8 : 16);
        // 16 warps per CTA when there are too few row groups to give every SM a CTA
        int n_warps = 8;
        if (n_rg < g.sm_count && pairs >= 32 && x_bytes(units, ncol) + ring_bytes(16) <= (size_t)MMA_SMEM_LIMIT) n_warps = 16;
        const size_t smem = x_bytes(units, ncol) + ring_bytes(n_warps);
        g1.err = g.dev_err;
        const int vi = ncol == 4 ? 0 : (ncol == 8 ? 1 : 2);
        MmaKernel k = vi == 0 ? (pair ? k_gemv_mma<4, true> : k_gemv_mma<4, false>)
                    : vi == 1 ? (pair ? k_gemv_mma<8, true> : k_gemv_mma<8, false>)
                              : (pair ? k_gemv_mma<16, true> : k_gemv_mma<16, false>);
        MmaInfo& ki = g_mma_info[vi][pair ? 1 : 0];
        if (!ki.attr) {
            if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM_LIMIT) != cudaSuccess)
                return fail(ADAMAH_ERR_BACKEND, "gemv_mma: cannot raise the shared-memory limit");
            ki.attr = true;
        }
        if (ki.occ_smem != smem || ki.occ_threads != n_warps * 32) {
            int per_sm = 0;
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, n_warps * 32, smem);
            ki.per_sm = per_sm < 1 ? 1 : per_sm; ki.occ_smem = smem; ki.occ_threads = n_warps * 32;
        }
        // K slices per row group: the fewest that still give every SM two CTAs; small
        // problems take the most parallel split.
        int KS = n_warps;
        for (int c = 1; c <= n_warps; c <<= 1) {
            if (c > pairs) break;
            const int n_sets = (n_rg + n_warps / c - 1) / (n_warps / c);
            if (n_sets >= 2 * g.sm_count) { KS = c; break; }
        }
        while (KS > pairs) KS >>= 1;
        if (KS < 1) KS = 1;
        const int n_sets = (n_rg + n_warps / KS - 1) / (n_warps / KS);
        int grid = g.sm_count * ki.per_sm;
        if (grid > n_sets) grid = n_sets;
        if (a.epi == EPI_ARGMAX && grid > gemv_max_grid()) grid = gemv_max_grid();
        if (a.max_grid > 0 && grid > a.max_grid) grid = a.max_grid;
        if (grid < 1) grid = 1;
        if (launch_k(k, dim3(grid), dim3(n_warps * 32), smem, stream, g.pdl, g1, t0, t1, KS) != cudaSuccess)
            return fail(ADAMAH_ERR_BACKEND, "gemv_mma: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        count_launch();
    }
    return ADAMAH_OK;
}

}  // namespace ab
