// Host-side launch logic of the tensor-core Q4_0 GEMV (kernel in gemv_mma.cuh).
#include "gemv_mma.cuh"

#include <cstdio>
#include <cstdlib>

namespace ab {

constexpr int MMA_SMEM_LIMIT = 200 * 1024;
constexpr int MMA_SMEM_LIMIT_LONG = 204 * 1024; // the instance for long plain vectors (two ring stages, 6 KB of static shared memory)
constexpr int MMA_MAX_PASSES = 16;          // batch-row groups per launch (arg-max scratch is sized for it)

typedef void (*MmaKernel)(const GemvArgs, const uint8_t*, const uint8_t*, int);

// staged bytes per 32-activation block: NCOL columns of 32 bytes + NCOL/2 pre-summed floats
static size_t x_bytes(int units, int ncol) { return (((size_t)units * (ncol * 32 + (ncol / 2) * 4)) + 127) & ~(size_t)127; }
static size_t ring_bytes(int wt, int n_warps, int n_stage = MMA_NSTAGE) { return (size_t)n_warps * mma_ring_bytes_per_warp(wt, n_stage); }
// fewest warps whose threads hold a fused input chain in registers (three float4 each)
static int chain_min_warps(const GemvArgs& a) { return a.h_in ? ((a.K >> 2) + 95) / 96 : 1; }

bool gemv_mma_supports(int wt, const GemvArgs& a) {
    if (a.N <= 0 || a.K <= 0 || a.B <= 0) return false;
    if (a.N % 16 || a.K % 64) return false;
    if (wt != WT_Q4_0 && wt != WT_Q4_K) return false;
    if (wt == WT_Q4_K && a.K % 256) return false;
    if (a.h_in) { if (chain_min_warps(a) > MMA_MAX_WARPS || (a.ldx & 3)) return false; }
    else if (((uintptr_t)a.x & 15) || (a.ldx & 3)) return false;
    int nw = chain_min_warps(a) <= 8 ? 8 : (chain_min_warps(a) <= 12 ? 12 : 16);
    const bool pair = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    const bool long_x = !a.h_in && a.K > 8192 && !pair;
    return x_bytes(a.K / 32, 4) + ring_bytes(wt, nw, long_x ? 2 : MMA_NSTAGE) <= (size_t)(long_x ? MMA_SMEM_LIMIT_LONG : MMA_SMEM_LIMIT);
}

struct MmaInfo { bool attr; size_t occ_smem[3]; int per_sm[3]; };   // per warp count 8, 12, 16
static MmaInfo g_mma_info[2][3][2];

template <int WT>
static MmaKernel pick_kernel(int vi, bool pair) {
    return vi == 0 ? (pair ? k_gemv_mma<4, true, WT> : k_gemv_mma<4, false, WT>)
         : vi == 1 ? (pair ? k_gemv_mma<8, true, WT> : k_gemv_mma<8, false, WT>)
                   : (pair ? k_gemv_mma<16, true, WT> : k_gemv_mma<16, false, WT>);
}

int launch_gemv_mma(int wt, const uint8_t* t0, const uint8_t* t1, GemvArgs a, cudaStream_t stream) {
    if (!gemv_mma_supports(wt, a)) return fail(ADAMAH_ERR_INVALID, "gemv_mma: shape not supported");
    const bool pair = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    if (pair && !t1) return fail(ADAMAH_ERR_INVALID, "gemv_mma: second matrix missing");
    const int units = a.K / 32, pairs = a.K / 64, n_rg = a.N / 16;
    // batch rows per pass: as many of 4, 2, 1 as shared memory allows
    // Batch rows per pass.  The passes of a launch run side by side (gridDim.x), each re-reading the weights from L2.
    // Matrices of a few MB are bound by latency, not by bytes: there more, thinner passes (more CTAs in flight) win --
    // measured at the 1B shape: 4 rows as 4 passes of one (0.94 against 1.41 ms per step), 8..32 rows as passes of two
    // (batch 8: 1.21 against 1.48 ms).  Large matrices (27B shapes, LM heads) and prefill chunks keep four rows per pass.
    static const int nb_env = getenv("ADAM_B200_MMA_ROWS") ? atoi(getenv("ADAM_B200_MMA_ROWS")) : 0;
    const double w_bytes = (double)a.N * a.K * 0.5625 * (pair ? 2 : 1);
    int nb_max = (nb_env == 1 || nb_env == 2 || nb_env == 4) ? nb_env : (w_bytes > 16.0e6 ? 4 : (a.B <= 4 ? 1 : (a.B <= 32 ? 2 : 4)));
    const int nw_min = chain_min_warps(a) <= 8 ? 8 : (chain_min_warps(a) <= 12 ? 12 : 16);
    while (nb_max > 1 && x_bytes(units, 4 * nb_max) + ring_bytes(wt, nw_min) > (size_t)MMA_SMEM_LIMIT) nb_max >>= 1;     // (one row: see long_x below)
    // One launch covers up to MMA_MAX_PASSES groups of nb_max batch rows (gridDim.y); more rows take more launches.
    const int rows_per_launch = a.B <= nb_max ? a.B : nb_max * MMA_MAX_PASSES;
    for (int b0 = 0; b0 < a.B; b0 += rows_per_launch) {
        GemvArgs g1 = a;
        g1.B = (a.B - b0 < rows_per_launch) ? a.B - b0 : rows_per_launch;
        if (a.x) g1.x = a.x + (size_t)b0 * a.ldx;
        if (a.h_in) g1.h_in = a.h_in + (size_t)b0 * a.ldx;
        if (a.add_src) g1.add_src = a.add_src + (size_t)b0 * a.ldx;
        if (a.h_out) g1.h_out = a.h_out + (size_t)b0 * a.ldx;
        if (a.y) g1.y = a.y + (size_t)b0 * a.ldy;
        if (a.out_tok) g1.out_tok = a.out_tok + b0;
        if (a.out_tok_f32) g1.out_tok_f32 = a.out_tok_f32 + b0;
        if (a.out_val) g1.out_val = a.out_val + b0;
        const int rows_per_pass = g1.B < nb_max ? g1.B : nb_max;
        const int n_pass = (g1.B + rows_per_pass - 1) / rows_per_pass;
        const int ncol = rows_per_pass == 1 ? 4 : (rows_per_pass == 2 ? 8 : 16);
        g1.err = g.dev_err;
        const int vi = ncol == 4 ? 0 : (ncol == 8 ? 1 : 2);
        MmaKernel k = wt == WT_Q4_0 ? pick_kernel<WT_Q4_0>(vi, pair) : pick_kernel<WT_Q4_K>(vi, pair);
        MmaInfo& ki = g_mma_info[wt == WT_Q4_0 ? 0 : 1][vi][pair ? 1 : 0];
        if (!ki.attr) {
            if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM_LIMIT) != cudaSuccess)
                return fail(ADAMAH_ERR_BACKEND, "gemv_mma: cannot raise the shared-memory limit");
            ki.attr = true;
        }
        // Shape of the launch: warps per CTA (8, 12 or 16) and K slices per row group (a
        // divisor of the warp count).  The estimate is the time of the busiest SM: tile pairs
        // per warp (plus a fixed cost per finished row group) times the larger of a lone
        // warp's latency per pair and the SM's issue time for all resident warps; ties go to
        // the smaller CTA and the smaller split.
        int n_warps = 8, KS = 1, best_per_sm = 1, n_stage = (!a.h_in && a.K > 8192 && ncol == 4 && !pair) ? 2 : MMA_NSTAGE;
        double best_cost = 1e300;
        const int nm = pair ? 2 : 1;
        const int sm_eff = g.sm_count / n_pass > 0 ? g.sm_count / n_pass : 1;   // the row groups of a launch share the SMs
        for (int nw = nw_min; nw <= 16; nw += 4) {
            // three ring stages per warp, two where a long activation vector leaves no room for three
            // long plain vectors, one batch row, one matrix: the instance that copies the vector to shared memory in
            // bulk and keeps two ring stages per warp, so that 16 warps fit beside it
            const bool long_x = !a.h_in && a.K > 8192 && ncol == 4 && !pair;
            const int nst = long_x ? 2 : MMA_NSTAGE;
            const size_t sm_bytes = x_bytes(units, ncol) + ring_bytes(wt, nw, nst);
            if (sm_bytes > (size_t)(long_x ? MMA_SMEM_LIMIT_LONG : MMA_SMEM_LIMIT)) break;
            int per_sm = ki.per_sm[nw / 4 - 2];
            if (ki.occ_smem[nw / 4 - 2] != sm_bytes) {
                per_sm = 0;
                cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, nw * 32, sm_bytes);
                if (per_sm < 1) per_sm = 1;
                ki.per_sm[nw / 4 - 2] = per_sm; ki.occ_smem[nw / 4 - 2] = sm_bytes;
            }
            for (int c = 1; c <= nw; ++c) {
                if (nw % c || c > pairs) continue;
                const int rgs = nw / c;                              // row groups per CTA pass
                const long long n_sets = (n_rg + rgs - 1) / rgs;
                long long ctas = (long long)sm_eff * per_sm;
                if (ctas > n_sets) ctas = n_sets;
                const long long passes = (n_sets + ctas - 1) / ctas;            // per CTA
                const long long resident = (ctas + sm_eff - 1) / sm_eff;           // CTAs on the busiest SM
                const int slice = (pairs + c - 1) / c;
                // a warp alone needs ~300 cycles per tile pair; an SM issues one per ~16 cycles
                const double busy = (double)resident * nw * 16.0;
                double cost = (double)passes * (slice * nm + 3.0 + 0.25 * c) * (busy > 300.0 ? busy : 300.0);
                // a long plain vector is staged by the CTA's own warps before the first product: ~500 cycles per 128 values and warp
                if (!a.h_in && a.K > 8192) cost += (double)a.K / 128.0 / nw * 500.0 * resident;
                if (cost < best_cost * 0.999) { best_cost = cost; n_warps = nw; KS = c; best_per_sm = per_sm; n_stage = nst; }
            }
        }
        {   // tuning aid: ADAM_B200_MMA_SHAPE="warps,k_slices" overrides the estimate (warps 8 / 12 / 16, k_slices a divisor)
            static const char* force = getenv("ADAM_B200_MMA_SHAPE");
            int fw = 0, fk = 0;
            if (force && sscanf(force, "%d,%d", &fw, &fk) == 2 && (fw == 8 || fw == 12 || fw == 16) && fw >= nw_min && fk >= 1 && fw % fk == 0 && fk <= pairs &&
                x_bytes(units, ncol) + ring_bytes(wt, fw, n_stage) <= (size_t)(n_stage == 2 ? MMA_SMEM_LIMIT_LONG : MMA_SMEM_LIMIT)) {
                n_warps = fw; KS = fk;
                cudaOccupancyMaxActiveBlocksPerMultiprocessor(&best_per_sm, k, fw * 32, x_bytes(units, ncol) + ring_bytes(wt, fw, n_stage));
                if (best_per_sm < 1) best_per_sm = 1;
            }
        }
        const size_t smem = x_bytes(units, ncol) + ring_bytes(wt, n_warps, n_stage);
        const int n_sets = (n_rg + n_warps / KS - 1) / (n_warps / KS);
        int grid = sm_eff * best_per_sm;
        if (grid > n_sets) grid = n_sets;
        if (a.epi == EPI_ARGMAX && grid > gemv_max_grid()) grid = gemv_max_grid();
        if (a.max_grid > 0 && grid > a.max_grid) grid = a.max_grid;
        if (grid < 1) grid = 1;
        if (getenv("ADAM_B200_DEBUG")) {
            static int seen_n[64], seen_k[64], n_seen = 0;
            bool seen = false;
            for (int i = 0; i < n_seen; ++i) seen |= seen_n[i] == a.N && seen_k[i] == a.K;
            if (!seen && n_seen < 64) {
                seen_n[n_seen] = a.N; seen_k[n_seen++] = a.K;
                fprintf(stderr, "[gemv_mma] N %d K %d B %d pair %d chain %d: %d warps, %d K slices, %d ring stages, grid %d x %d, %zu B shared, %d CTAs per SM\n",
                        a.N, a.K, g1.B, (int)pair, a.h_in != nullptr, n_warps, KS, n_stage, n_pass, grid, smem, best_per_sm);
            }
        }
        if (n_stage == 2) {
            k = wt == WT_Q4_0 ? (MmaKernel)k_gemv_mma<4, false, WT_Q4_0, 2> : (MmaKernel)k_gemv_mma<4, false, WT_Q4_K, 2>;
            static bool attr2[2];
            if (!attr2[wt == WT_Q4_0 ? 0 : 1]) {
                if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, MMA_SMEM_LIMIT_LONG) != cudaSuccess)
                    return fail(ADAMAH_ERR_BACKEND, "gemv_mma: cannot raise the shared-memory limit");
                attr2[wt == WT_Q4_0 ? 0 : 1] = true;
            }
        }
        if (launch_k(k, dim3(n_pass, grid), dim3(n_warps * 32), smem, stream, g.pdl, g1, t0, t1, KS) != cudaSuccess)
            return fail(ADAMAH_ERR_BACKEND, "gemv_mma: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        count_launch();
    }
    return ADAMAH_OK;
}

}  // namespace ab
