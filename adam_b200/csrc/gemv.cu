// Host-side launch logic of the dequant-fused GEMV (kernel in gemv.cuh).
#include "gemv.cuh"

namespace ab {

constexpr int GEMV_SMEM_LIMIT = 200 * 1024;  // staged activations per CTA
constexpr int GEMV_MAX_GRID = 4096;

int gemv_max_grid() { return GEMV_MAX_GRID; }

typedef void (*GemvKernel)(const GemvArgs);

template <int WT, int L>
static GemvKernel pick_nb(int nb) {
    switch (nb) {
    case 1: return k_gemv<WT, L, 1>;
    case 2: return k_gemv<WT, L, 2>;
    default: return k_gemv<WT, L, 4>;
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

static int l_index(int L) { return L == 4 ? 0 : L == 8 ? 1 : L == 16 ? 2 : 3; }
static int nb_index(int nb) { return nb == 1 ? 0 : nb == 2 ? 1 : 2; }

struct KernelInfo { bool attr_set; size_t occ_smem; int occ_block; int per_sm; };
static KernelInfo g_info[2][4][3];

// Lanes per row and CTA size.  Among the shapes that give the grid at least two
// CTAs per SM (so every SM streams weights), take the one with the fewest idle
// lanes in the last sweep of a row, widest first; small problems that cannot
// fill the machine take the most parallel shape.
static void choose_shape(int units, int n_slots, int sm_count, int* L_out, int* block_out) {
    const int cand[4] = {32, 16, 8, 4};
    int bestL = 32, bestBlock = 128;
    long bestWaste = -1;
    for (int pass = 0; pass < 2 && bestWaste < 0; ++pass) {
        const int block = pass == 0 ? 256 : 128;
        for (int i = 0; i < 4; ++i) {
            const int L = cand[i], rpw = 32 / L, warps = block / 32;
            const long n_pass = (n_slots + rpw - 1) / rpw;
            const long ctas = (n_pass + warps - 1) / warps;
            if (ctas < 2L * sm_count) continue;
            const int iters = (units + L - 1) / L;
            const long waste = (long)iters * L * 1000 / units;
            if (bestWaste < 0 || waste < bestWaste) { bestWaste = waste; bestL = L; bestBlock = block; }
        }
    }
    *L_out = bestL; *block_out = bestBlock;
}

int launch_gemv(int wtype, GemvArgs a, cudaStream_t stream) {
    if (a.N <= 0 || a.K <= 0 || a.B <= 0) return fail(ADAMAH_ERR_INVALID, "gemv: empty shape");
    if (wtype != WT_Q4_0 && wtype != WT_Q4_K) return fail(ADAMAH_ERR_INVALID, "gemv: this kernel reads Q4_0 / Q4_K blocks only");
    if (wtype == WT_Q4_0 ? (a.K % 32) : (a.K % 256)) return fail(ADAMAH_ERR_INVALID, "gemv: K=%d is not a whole number of blocks", a.K);
    if (!a.h_in && (((uintptr_t)a.x & 15) || (a.ldx & 3))) return fail(ADAMAH_ERR_INVALID, "gemv: activations must be 16-byte aligned");
    if (a.h_in && a.h_out == a.h_in) return fail(ADAMAH_ERR_INVALID, "gemv: h_out must not alias h_in");
    const int units = (wtype == WT_Q4_0) ? a.K / Geo<WT_Q4_0>::ELEMS : a.K / Geo<WT_Q4_K>::ELEMS;   // work items per row
    const bool pair = (a.epi == EPI_GEGLU || a.epi == EPI_SWIGLU);
    const int n_slots = pair ? a.N : (a.N + 1) / 2;
    int L, block;
    choose_shape(units, n_slots, g.sm_count, &L, &block);
    const int n_pass = (n_slots + 32 / L - 1) / (32 / L);
    const size_t x_bytes = (size_t)units * (wtype == WT_Q4_0 ? Geo<WT_Q4_0>::STRIDE : Geo<WT_Q4_K>::STRIDE) * 4;
    int nb_max = 4;
    while (nb_max > 1 && x_bytes * nb_max > (size_t)GEMV_SMEM_LIMIT) nb_max >>= 1;
    if (x_bytes > (size_t)GEMV_SMEM_LIMIT) return fail(ADAMAH_ERR_INVALID, "gemv: K=%d exceeds the shared-memory staging limit", a.K);

    for (int b0 = 0; b0 < a.B; b0 += nb_max) {
        GemvArgs g1 = a;
        g1.B = (a.B - b0 < nb_max) ? a.B - b0 : nb_max;
        const int nb = g1.B == 1 ? 1 : g1.B == 2 ? 2 : 4;
        if (a.x) g1.x = a.x + (size_t)b0 * a.ldx;
        if (a.h_in) g1.h_in = a.h_in + (size_t)b0 * a.ldx;
        if (a.add_src) g1.add_src = a.add_src + (size_t)b0 * a.ldx;
        if (a.h_out) g1.h_out = a.h_out + (size_t)b0 * a.ldx;
        if (a.y) g1.y = a.y + (size_t)b0 * a.ldy;
        if (a.out_tok) g1.out_tok = a.out_tok + b0;
        if (a.out_tok_f32) g1.out_tok_f32 = a.out_tok_f32 + b0;
        const size_t smem = x_bytes * nb;
        GemvKernel k = (wtype == WT_Q4_0) ? pick_l<WT_Q4_0>(L, nb) : pick_l<WT_Q4_K>(L, nb);
        KernelInfo& ki = g_info[wtype][l_index(L)][nb_index(nb)];
        if (!ki.attr_set) {
            if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMV_SMEM_LIMIT) != cudaSuccess)
                return fail(ADAMAH_ERR_BACKEND, "gemv: cannot raise the shared-memory limit");
            ki.attr_set = true;
        }
        if (ki.occ_smem != smem || ki.occ_block != block) {
            int per_sm = 0;
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, block, smem);
            ki.per_sm = per_sm < 1 ? 1 : per_sm; ki.occ_smem = smem; ki.occ_block = block;
        }
        const int warps = block / 32;
        int need = (n_pass + warps - 1) / warps;
        int grid = g.sm_count * ki.per_sm;
        if (grid > need) grid = need;
        if (grid < 1) grid = 1;
        if (a.epi == EPI_ARGMAX && grid > GEMV_MAX_GRID) grid = GEMV_MAX_GRID;
        if (a.max_grid > 0 && grid > a.max_grid) grid = a.max_grid;
        if (launch_k(k, dim3(grid), dim3(block), smem, stream, g.pdl, g1) != cudaSuccess) return fail(ADAMAH_ERR_BACKEND, "gemv: launch failed: %s", cudaGetErrorString(cudaGetLastError()));
        count_launch();
    }
    return ADAMAH_OK;
}

}  // namespace ab
