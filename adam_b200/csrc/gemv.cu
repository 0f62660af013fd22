// Host-side launch logic of the dequant-fused GEMV (kernel in gemv.cuh).
#include "gemv.cuh"

namespace ab {

constexpr int GEMV_SMEM_LIMIT = 96 * 1024;   // staged activations per CTA (2 CTAs fit an SM)
constexpr int GEMV_MAX_GRID = 4096;

int gemv_max_grid() { return GEMV_MAX_GRID; }

typedef void (*GemvKernel)(const GemvArgs);

template <int WT, int L>
static GemvKernel pick_nb(int nb) {
    switch (nb) {
    case 1: return k_gemv<WT, L, 1>;
    case 2: return k_gemv<WT, L, 2>;
    case 4: return k_gemv<WT, L, 4>;
    default: return k_gemv<WT, L, 8>;
    }
}
template <int WT>
static GemvKernel pick_l(int L, int nb) {
    switch (L) {
    case 4: return pick_nb<WT, 4>(nb);
    case 8: return pick_nb<WT, 8>(nb);
    case 16: return pick_nb<WT, 16>(nb);
    default: return pick_nb<WT, 32>(nb);
    }
}

// Lanes per row: at least four units per lane where K allows it, then the least
// idle lanes in the last sweep, then the widest (best coalescing).
static int choose_lanes(int units) {
    int bestL = 4; long bestWaste = -1;
    const int cand[4] = {32, 16, 8, 4};
    for (int i = 0; i < 4; ++i) {
        int L = cand[i], iters = (units + L - 1) / L;
        if (iters < 4 && L != 4) continue;
        long waste = (long)iters * L * 1000 / units;
        if (bestWaste < 0 || waste < bestWaste) { bestWaste = waste; bestL = L; }
    }
    return bestL;
}

struct KernelInfo { bool ready; int ctas_per_sm; };
static KernelInfo g_info[2][4][4];

static int l_index(int L) { return L == 4 ? 0 : L == 8 ? 1 : L == 16 ? 2 : 3; }
static int nb_index(int nb) { return nb == 1 ? 0 : nb == 2 ? 1 : nb == 4 ? 2 : 3; }

int launch_gemv(int wtype, GemvArgs a, cudaStream_t stream) {
    if (a.N <= 0 || a.K <= 0 || a.B <= 0) return fail(ADAMAH_ERR_INVALID, "gemv: empty shape");
    if (wtype == WT_Q4_0 ? (a.K % 32) : (a.K % 256)) return fail(ADAMAH_ERR_INVALID, "gemv: K=%d is not a whole number of blocks", a.K);
    if (((uintptr_t)a.x & 15) || (a.ldx & 3)) return fail(ADAMAH_ERR_INVALID, "gemv: activations must be 16-byte aligned");
    const int units = a.K / 32;
    const int L = choose_lanes(units);
    const bool pair = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    const int n_slots = pair ? a.N : (a.N + 1) / 2;
    const int n_pass = (n_slots + 32 / L - 1) / (32 / L);

    for (int b0 = 0; b0 < a.B; b0 += 8) {
        GemvArgs g1 = a;
        g1.B = (a.B - b0 < 8) ? a.B - b0 : 8;
        const int nb = g1.B == 1 ? 1 : g1.B == 2 ? 2 : g1.B <= 4 ? 4 : 8;
        g1.x = a.x + (size_t)b0 * a.ldx;
        if (a.y) g1.y = a.y + (size_t)b0 * a.ldy;
        if (a.out_tok) g1.out_tok = a.out_tok + b0;
        if (a.out_tok_f32) g1.out_tok_f32 = a.out_tok_f32 + b0;
        int kc_units = units;
        if ((size_t)nb * units * 128 > (size_t)GEMV_SMEM_LIMIT) {
            kc_units = GEMV_SMEM_LIMIT / (nb * 128);
            kc_units -= kc_units % 8;              // whole Q4_K superblocks, 16-byte rows
        }
        g1.kc_units = kc_units;
        const size_t smem = (size_t)nb * (kc_units < units ? kc_units : units) * 128;
        GemvKernel k = (wtype == WT_Q4_0) ? pick_l<WT_Q4_0>(L, nb) : pick_l<WT_Q4_K>(L, nb);
        KernelInfo& ki = g_info[wtype][l_index(L)][nb_index(nb)];
        if (!ki.ready) {
            if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM_LIMIT) != cudaSuccess)
                return fail(ADAMAH_ERR_BACKEND, "gemv: cannot raise the shared-memory limit");
            ki.ready = true;
        }
        int per_sm = 0;
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, 256, smem);
        if (per_sm < 1) per_sm = 1;
        int need = (n_pass + 7) / 8;
        int grid;
        if (kc_units < units) grid = need;                           // one pass per warp
        else { grid = g.sm_count * per_sm; if (grid > need) grid = need; }
        if (grid < 1) grid = 1;
        if (a.epi == EPI_ARGMAX && grid > GEMV_MAX_GRID) {
            if (kc_units < units) return fail(ADAMAH_ERR_INVALID, "gemv+argmax: K too large for the batch tile");
            grid = GEMV_MAX_GRID;
        }
        k<<<grid, 256, smem, stream>>>(g1);
        count_launch();
    }
    return ADAMAH_OK;
}

}  // namespace ab
