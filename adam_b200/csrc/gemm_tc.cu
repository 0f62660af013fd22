// Dequant-fused GEMM  y[b][n] = sum_k W[n][k] x[b][k]  for 9..64 activation rows b (a prefill chunk
// or a large decode batch) on the 5th-generation tensor cores: tcgen05.mma with the accumulator in
// tensor memory (TMEM).  Same operator as the GEMV kernels (the reference's Q4 mat-vec shader
// adamah-MAIN/adamah/shaders/src/f32/map_matvec_t_xq4.comp and map_fused_gateup_t_xq4.comp run once
// per row by adamah.c:8606-8691), same arithmetic idea: activations become integers of up to 23 bits
// with one power-of-two scale per row, the products with the 4-bit weights are formed exactly, and
// each 32-weight block's sum is scaled by the block's scale and accumulated in fp32.  Here the
// integers are split into two signed 11-bit planes, which fp16 holds exactly; a block's 32 products
// per plane add up exactly in the tensor core's fp32 accumulator (|sum| < 2^20).
//
// Two kernels:
//   k_quant_rows   one CTA per activation row: the optional input chain (residual add + RMS norms,
//                  as the GEMV prologue; the row stays in registers and all loads are issued before
//                  the first use), the row's scale, and the row's two fp16 planes written straight
//                  into the B-operand image in global memory: K-major with the 128-byte swizzle,
//                  two 32-wide K blocks per 128-byte operand row, 128 operand rows (row n = plane *
//                  64 + activation row) = 16 KB per block pair, and behind each chunk of four
//                  blocks the 4 x 64 per-row integer sums as floats (the term that carries the Q4_K
//                  block minimum).
//   k_gemm_tc      256 threads, two CTAs per SM (256 TMEM columns and 99 KB of shared memory each), a
//                  grid that fills the GPU twice over and takes work items (tile of 128 weight rows
//                  x K split) round-robin.  Per chunk of 4 K blocks: one bulk copy brings the B
//                  image (33 KB) into one of two buffers, the threads turn the chunk's nibbles
//                  (64-byte runs per weight row, requested one chunk ahead and held in registers)
//                  into fp16 (q - 8 for Q4_0, q for Q4_K: one byte permute per pair gives 1024 + q,
//                  one packed subtract removes the offset) in the swizzled A image, and then per K
//                  block one thread issues two tcgen05.mma (M 128 x N 128 x K 16 each, fp16 -> fp32
//                  in TMEM) and a commit whose completion arrives on an mbarrier.  TMEM holds two
//                  accumulators of 128 columns: block j + 1 is issued before block j is read.  The
//                  two warps of a TMEM lane quarter read 32 of the 64 columns each (tcgen05.ld),
//                  recombine the planes (hi * 2048 + lo), apply the block scale and accumulate 32
//                  fp32 outputs per thread.  K splits leave partial sums in a workspace; the last
//                  CTA of a tile (atomic ticket) adds them in split order and runs the epilogue
//                  (store, or GeGLU / SwiGLU over a tile of 64 gate rows + 64 up rows).
// Every wait (bulk copy, tensor-core completion) is bounded: when one runs out the kernel records
// DEVERR_WAIT, stops waiting, and still frees its tensor memory.  The shared-memory request keeps a
// third CTA off an SM, so a TMEM allocation never waits on a CTA that cannot run.
#include "gemm_tc.cuh"
#include "gemv_mma.cuh"

#include <cstdlib>

namespace ab {

constexpr int TC_PLANES = 2;
constexpr int TC_N = TC_PLANES * TC_COLS;                // 128 B-operand rows
constexpr int TC_CH = 4;                                 // K blocks per chunk
// Operand images, K-major with the 128-byte swizzle: a "pair" image holds two K blocks (64 fp16 = 128
// bytes per operand row) of 128 operand rows = 16 KB: 8-row groups of 1024 bytes, a row's 128 bytes
// contiguous, and the 16-byte piece c of row r stored at piece c ^ (r & 7).  Images start at
// multiples of 1024 bytes (the swizzle works on address bits).
constexpr int TC_PAIR_IMG = 128 * 128;                   // 16384
constexpr int TC_A_CHUNK = (TC_CH / 2) * TC_PAIR_IMG;    // 32768
constexpr int TC_B_SUMS = TC_A_CHUNK;                    // offset of the chunk's [4][64] row sums in the B chunk image
constexpr int TC_B_CHUNK = TC_A_CHUNK + TC_CH * TC_COLS * 4;        // 33792 = 33 * 1024
constexpr int TC_SMEM = TC_A_CHUNK + 2 * TC_B_CHUNK + 1024;         // A image + two B buffers (+ alignment slack); two CTAs per SM, never three (TMEM holds two allocations)
constexpr int TC_TMEM_COLS = 256;
constexpr int TC_THREADS = 256;                         // two warps per TMEM lane quarter: each takes 32 of the 64 columns
constexpr int TC_MYCOLS = TC_COLS / 2;
constexpr int TC_MAX_K = 32768;
constexpr int TC_MAX_CTAS = 1536;                        // workspace: 32 KB of partial sums per CTA
constexpr int TC_MAX_TILES = 4096;

struct TcWork { uint8_t* bimg; float* inv; float* part; unsigned int* tickets; bool ok; };
static TcWork g_tc = {};
static uint64_t g_tc_calls = 0;
static int g_tc_policy = -1;             // 0 never, 1 where it is expected to be faster, 2 whenever the shape allows; -1 = take it from ADAM_B200_TC

bool gemm_tc_prepare() {
    if (g_tc.ok) return true;
    const size_t bimg_bytes = (size_t)(TC_MAX_K / 32 / TC_CH) * TC_B_CHUNK;
    if (cudaMalloc(&g_tc.bimg, bimg_bytes) != cudaSuccess || cudaMalloc(&g_tc.inv, TC_COLS * 4) != cudaSuccess ||
        cudaMalloc(&g_tc.part, (size_t)TC_MAX_CTAS * TC_COLS * 128 * 4) != cudaSuccess ||
        cudaMalloc(&g_tc.tickets, TC_MAX_TILES * 4) != cudaSuccess) {
        cudaGetLastError();
        gemm_tc_release();
        return false;
    }
    cudaMemset(g_tc.tickets, 0, TC_MAX_TILES * 4);
    cudaMemset(g_tc.bimg, 0, bimg_bytes);
    g_tc.ok = true;
    return true;
}

void gemm_tc_release() {
    cudaFree(g_tc.bimg); cudaFree(g_tc.inv); cudaFree(g_tc.part); cudaFree(g_tc.tickets);
    g_tc = TcWork{};
}

// Byte offset of (operand row n, byte kb of the row's 128) in a pair image.
__device__ __forceinline__ int swz_off(int n, int kb) { return (n >> 3) * 1024 + (n & 7) * 128 + ((((kb >> 4) ^ n) & 7) << 4) + (kb & 15); }
// Byte offset in the B image of the 4 values k0 .. k0+3 (k0 a multiple of 4) of operand row n, and of block kb's row sums.
__device__ __forceinline__ size_t bimg_off(int n, int k0) {
    const int kb = k0 >> 5;
    return (size_t)(kb >> 2) * TC_B_CHUNK + ((kb >> 1) & 1) * TC_PAIR_IMG + swz_off(n, (kb & 1) * 64 + (k0 & 31) * 2);
}
__device__ __forceinline__ size_t bsum_off(int kb) { return (size_t)(kb >> 2) * TC_B_CHUNK + TC_B_SUMS + (kb & 3) * (TC_COLS * 4); }

// ---- activations: chain, scale, two fp16 planes in B-operand order -------------------------------
// Four consecutive activations (k = 4i .. 4i+3) of column `col`, already scaled: round to integers,
// split into the two planes, store them, and leave the block's integer sum behind the block's image.
// Called by all threads of a warp together (the eight threads of one 32-wide block are eight
// neighbouring lanes); threads with on == false only take part in the shuffles.
__device__ __forceinline__ void put_planes(uint8_t* __restrict__ bimg, int col, int i, bool on, float4 v, float s) {
    const float f[4] = {v.x * s, v.y * s, v.z * s, v.w * s};
    __align__(8) __half hi[4], lo[4];
    int sum = 0;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const int xi = on ? __float2int_rn(f[e]) : 0;       // |xi| <= 2^22
        const int l = ((xi + 1024) & 2047) - 1024;          // [-1024, 1023]
        const int h = (xi - l) >> 11;                       // [-2048, 2048]: exact in fp16
        hi[e] = __int2half_rn(h); lo[e] = __int2half_rn(l);
        sum += xi;
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if (on) {
        const int k0 = 4 * i;
        *reinterpret_cast<uint2*>(bimg + bimg_off(col, k0)) = *reinterpret_cast<const uint2*>(hi);
        *reinterpret_cast<uint2*>(bimg + bimg_off(TC_COLS + col, k0)) = *reinterpret_cast<const uint2*>(lo);
        if ((k0 & 31) == 0) reinterpret_cast<float*>(bimg + bsum_off(k0 >> 5))[col] = (float)sum;
    }
}

constexpr int QR_THREADS = 512;
constexpr int QR_MAXV = 4;             // float4 per thread held in registers: rows of up to 8192 values

__global__ void __launch_bounds__(QR_THREADS) k_quant_rows(const GemvArgs a, uint8_t* __restrict__ bimg, float* __restrict__ inv_out) {
    extern __shared__ float xs[];                       // the row, K floats
    __shared__ float red[66];
    const int col = blockIdx.x, tid = threadIdx.x, K = a.K, n4 = K >> 2;
    pdl_launch_dependents();
    pdl_wait();
    if (col >= a.B) {                                   // unused columns multiply as zeros
        for (int i = tid; i < n4; i += blockDim.x) {
            const int k0 = 4 * i;
#pragma unroll
            for (int p = 0; p < TC_PLANES; ++p) *reinterpret_cast<uint2*>(bimg + bimg_off(p * TC_COLS + col, k0)) = make_uint2(0u, 0u);
            if ((k0 & 31) == 0) reinterpret_cast<float*>(bimg + bsum_off(k0 >> 5))[col] = 0.f;
        }
        if (tid == 0) inv_out[col] = 0.f;
        return;
    }
    const size_t row = (size_t)col * a.ldx;
    if (n4 <= (int)blockDim.x * QR_MAXV) {
        // the row lives in registers: every load of the chain is issued before the first use
        const float4 z4 = make_float4(0.f, 0.f, 0.f, 0.f), o4 = make_float4(1.f, 1.f, 1.f, 1.f);
        const float* ap = a.h_in && a.add_src ? a.add_src + row : nullptr;
        const bool post = ap && a.w_post, pre = a.h_in && a.w_pre;
        float4 v[QR_MAXV], va[QR_MAXV], vp[QR_MAXV], vw[QR_MAXV];
#pragma unroll
        for (int j = 0; j < QR_MAXV; ++j) {
            const int i = tid + j * (int)blockDim.x;
            const bool in = i < n4;
            v[j] = in ? reinterpret_cast<const float4*>((a.h_in ? a.h_in : a.x) + row)[i] : z4;
            va[j] = (in && ap) ? reinterpret_cast<const float4*>(ap)[i] : z4;
            vp[j] = (in && post) ? reinterpret_cast<const float4*>(a.w_post)[i] : o4;
            vw[j] = (in && pre) ? reinterpret_cast<const float4*>(a.w_pre)[i] : o4;
        }
        if (a.h_in) {
            float rms_a = 1.f;
            if (post) {
                float ss = 0.f;
#pragma unroll
                for (int j = 0; j < QR_MAXV; ++j) { ss = fmaf(va[j].x, va[j].x, ss); ss = fmaf(va[j].y, va[j].y, ss); ss = fmaf(va[j].z, va[j].z, ss); ss = fmaf(va[j].w, va[j].w, ss); }
                ss = block_sum(ss, red);
                rms_a = sqrtf(ss / (float)K + a.eps);
            }
            const float rcp_a = __frcp_rn(rms_a);
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < QR_MAXV; ++j) {
                if (ap) {
                    if (post) {
                        v[j].x += div_by(va[j].x, rms_a, rcp_a) * vp[j].x; v[j].y += div_by(va[j].y, rms_a, rcp_a) * vp[j].y;
                        v[j].z += div_by(va[j].z, rms_a, rcp_a) * vp[j].z; v[j].w += div_by(va[j].w, rms_a, rcp_a) * vp[j].w;
                    } else { v[j].x += va[j].x; v[j].y += va[j].y; v[j].z += va[j].z; v[j].w += va[j].w; }
                }
                ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
                const int i = tid + j * (int)blockDim.x;
                if (i < n4 && a.h_out) reinterpret_cast<float4*>(a.h_out + row)[i] = v[j];
            }
            if (pre) {
                ss = block_sum(ss, red);
                const float rms = sqrtf(ss / (float)K + a.eps), rcp = __frcp_rn(rms);
#pragma unroll
                for (int j = 0; j < QR_MAXV; ++j) {
                    v[j].x = div_by(v[j].x, rms, rcp) * vw[j].x; v[j].y = div_by(v[j].y, rms, rcp) * vw[j].y;
                    v[j].z = div_by(v[j].z, rms, rcp) * vw[j].z; v[j].w = div_by(v[j].w, rms, rcp) * vw[j].w;
                }
            }
        }
        float am = 0.f;
#pragma unroll
        for (int j = 0; j < QR_MAXV; ++j) am = fmaxf(am, fmaxf(fmaxf(fabsf(v[j].x), fabsf(v[j].y)), fmaxf(fabsf(v[j].z), fabsf(v[j].w))));
        am = block_max(am, red);
        float s, inv;
        pow2_scale(am, s, inv);
        if (tid == 0) inv_out[col] = inv;
#pragma unroll
        for (int j = 0; j < QR_MAXV; ++j) {
            const int i = tid + j * (int)blockDim.x;
            if (j * (int)blockDim.x < n4) put_planes(bimg, col, i, i < n4, v[j], s);     // warp-uniform: whole warps skip together only past the row's end
        }
        return;
    }
    float am = 0.f;
    if (a.h_in) {
        const float* hp = a.h_in + row;
        const float* ap = a.add_src ? a.add_src + row : nullptr;
        float rms_a = 1.f;
        if (ap && a.w_post) {
            float ss = 0.f;
            for (int i = tid; i < K; i += blockDim.x) ss = fmaf(ap[i], ap[i], ss);
            ss = block_sum(ss, red);
            rms_a = sqrtf(ss / (float)K + a.eps);
        }
        const float rcp_a = __frcp_rn(rms_a);
        float ss = 0.f;
        for (int i = tid; i < K; i += blockDim.x) {
            float h = hp[i];
            if (ap) h += a.w_post ? div_by(ap[i], rms_a, rcp_a) * a.w_post[i] : ap[i];
            if (a.h_out) a.h_out[row + i] = h;
            xs[i] = h;
            ss = fmaf(h, h, ss);
        }
        ss = block_sum(ss, red);
        if (a.w_pre) {
            const float rms = sqrtf(ss / (float)K + a.eps), rcp = __frcp_rn(rms);
            for (int i = tid; i < K; i += blockDim.x) xs[i] = div_by(xs[i], rms, rcp) * a.w_pre[i];
        }
        for (int i = tid; i < K; i += blockDim.x) am = fmaxf(am, fabsf(xs[i]));
    } else {
        for (int i = tid; i < K; i += blockDim.x) { const float v = a.x[row + i]; xs[i] = v; am = fmaxf(am, fabsf(v)); }
    }
    am = block_max(am, red);
    float s, inv;
    pow2_scale(am, s, inv);
    if (tid == 0) inv_out[col] = inv;
    for (int i0 = 0; i0 < n4; i0 += blockDim.x) {
        const int i = i0 + tid;
        const bool on = i < n4;
        put_planes(bimg, col, i, on, on ? reinterpret_cast<const float4*>(xs)[i] : make_float4(0.f, 0.f, 0.f, 0.f), s);
    }
}

// ---- tcgen05 primitives --------------------------------------------------------------------------
// Shared-memory matrix descriptor, K-major with the 128-byte swizzle (layout 2 at bit 61): start
// address and the distance between 8-row groups (1024 bytes), in 16-byte units, plus the descriptor
// version of this architecture (bit 46).  The 16 values of K of one instruction are 32 bytes of a
// row: the next instruction's descriptor starts 32 bytes further.
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: D = f32 (1 at bit 4), A = B = f16 (0 at bits 7 and 10), both
// operands K-major, N / 8 at bit 17, M / 16 at bit 24.
constexpr uint32_t TC_IDESC = (1u << 4) | ((uint32_t)(TC_N >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void tc_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(slot)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] = A * B (accumulate == 0) or D += A * B; one instruction covers 16 values of K
__device__ __forceinline__ void tc_mma_f16(uint32_t taddr, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(taddr), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// The mbarrier gets one arrival when all tensor-core operations issued so far by this thread are done.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&r)[32]) {
    // the registers hold the values only after tc_ld_wait(): nothing may touch them before
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]), "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15]), "=f"(r[16]), "=f"(r[17]), "=f"(r[18]), "=f"(r[19]), "=f"(r[20]), "=f"(r[21]), "=f"(r[22]), "=f"(r[23]), "=f"(r[24]), "=f"(r[25]), "=f"(r[26]), "=f"(r[27]), "=f"(r[28]), "=f"(r[29]), "=f"(r[30]), "=f"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Two nibbles-as-bytes (bytes `sel` picks from t) -> two fp16 values minus `off` (1024 + the zero point).
__device__ __forceinline__ uint32_t nib2_to_h2(uint32_t t, uint32_t sel, __half2 off) {
    const uint32_t v = __byte_perm(t, 0x64646464u, sel);       // { 0x64, nibble } per half = 1024 + nibble
    const __half2 h = __hsub2(*reinterpret_cast<const __half2*>(&v), off);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// Eight nibbles-as-bytes of two words -> eight consecutive fp16 values (one 16-byte core-matrix row).
__device__ __forceinline__ uint4 nib8_to_h8(uint32_t t0, uint32_t t1, __half2 off) {
    return make_uint4(nib2_to_h2(t0, 0x4140u, off), nib2_to_h2(t0, 0x4342u, off), nib2_to_h2(t1, 0x4140u, off), nib2_to_h2(t1, 0x4342u, off));
}

// ---- the GEMM ---------------------------------------------------------------------------------
// grid = tiles * S; CTA (tile, sp) covers chunks [sp * n_chunks / S, (sp + 1) * n_chunks / S).
// PAIR: a tile is 64 rows of w0 (gate) in TMEM lanes 0..63 and the same 64 rows of w1 (up) in
// lanes 64..127; otherwise 128 consecutive rows of w0.
template <int WT, bool PAIR>
__global__ void __launch_bounds__(TC_THREADS, 2) k_gemm_tc(const GemvArgs a, const uint8_t* __restrict__ bimg, const float* __restrict__ inv,
                                                    float* __restrict__ part, unsigned int* __restrict__ tickets, int S, int items) {
    extern __shared__ __align__(1024) uint8_t sm_raw[];
    uint8_t* sm = sm_raw + ((1024u - (smem_u32(sm_raw) & 1023u)) & 1023u);     // the swizzle needs images at multiples of 1024 bytes
    uint8_t* smA = sm;
    uint8_t* smB = sm + TC_A_CHUNK;
    __shared__ __align__(8) uint64_t bar_b[2], bar_m[2];
    __shared__ uint32_t s_tmem;
    __shared__ bool s_last;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int lane_row = tid & 127, chalf = tid >> 7;          // TMEM lane (row of the tile) and column half of this thread
    int tile = 0, ch0 = 0, ch1 = 0;                           // of the work item in hand (set per item below)
    const int units = a.K >> 5, n_chunks = (units + TC_CH - 1) / TC_CH;
    constexpr int TILE_ROWS = PAIR ? 64 : 128;
    // the weight row behind TMEM lane `l` of this tile
    auto row_of = [&](int l, const WeightRef*& w) -> int {
        if constexpr (PAIR) { w = (l >> 6) ? &a.w1 : &a.w0; return min(tile * 64 + (l & 63), a.N - 1); }
        else { w = &a.w0; return min(tile * 128 + l, a.N - 1); }
    };
    if (tid == 0) { mbar_init(&bar_b[0], 1); mbar_init(&bar_b[1], 1); mbar_init(&bar_m[0], 1); mbar_init(&bar_m[1], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) tc_alloc(&s_tmem, TC_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    const WeightRef* wmine = nullptr;
    int my_row = 0;
    float acc[TC_MYCOLS];
    uint32_t ph_b0 = 0, ph_b1 = 0, ph_m0 = 0, ph_m1 = 0;
    bool dead = false;
    const __half2 off = __float2half2_rn(WT == WT_Q4_0 ? 1032.f : 1024.f);     // Q4_0 values are q - 8

    // block j of the chunk into accumulator j & 1: two instructions of 16 values of K each
    auto issue = [&](int j, const uint8_t* smBc) {
        // block j = half (j & 1) of pair image j >> 1: its 32 values of K are bytes 64 * (j & 1) .. + 63 of every row
        const uint32_t po = (uint32_t)(j >> 1) * TC_PAIR_IMG + (uint32_t)(j & 1) * 64u;
        const uint32_t ab = smem_u32(smA) + po, bb = smem_u32(smBc) + po;
        const uint32_t d = tmem + (uint32_t)(j & 1) * TC_N;
        tc_fence_after();
        tc_mma_f16(d, tc_desc(ab), tc_desc(bb), TC_IDESC, 0u);
        tc_mma_f16(d, tc_desc(ab + 32u), tc_desc(bb + 32u), TC_IDESC, 1u);
        tc_commit(&bar_m[j & 1]);
    };

    // ---- main loop: chunks of TC_CH blocks; the next chunk's nibbles, scales (registers) and B image
    // (second shared-memory buffer) are requested while the current chunk is multiplied ----
    constexpr int NQ = TC_CH * 128 / TC_THREADS;            // 16-byte units per thread and chunk
    struct Raw { uint4 q[NQ]; uint4 h; unsigned short d[TC_CH]; };
    auto fetch = [&](int ch, Raw& r) {                      // global loads of chunk ch (weights only: no dependency on earlier kernels)
        const int c0 = ch * TC_CH, nb = min(TC_CH, units - c0);
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int idx = i * TC_THREADS + tid, rl = idx >> 2, u = idx & 3;
            const WeightRef* w;
            const int rr = row_of(rl, w);
            if constexpr (WT == WT_Q4_0) r.q[i] = ld_stream(w->q + (size_t)rr * units + c0 + min(u, nb - 1));
            else r.q[i] = ld_stream(w->q + ((size_t)rr * (units >> 3) + (ch >> 1)) * 9 + 1 + (ch & 1) * 4 + u);
        }
        if constexpr (WT == WT_Q4_0) {
#pragma unroll
            for (int j = 0; j < TC_CH; ++j) r.d[j] = __ldg(reinterpret_cast<const unsigned short*>(wmine->d) + (size_t)my_row * units + c0 + min(j, nb - 1));
        } else {
            r.h = __ldg(wmine->q + ((size_t)my_row * (units >> 3) + (ch >> 1)) * 9);
        }
    };
    auto fetch_b = [&](int ch) {                            // thread 0: bulk copy of chunk ch's B image into buffer (ch - ch0) & 1
        const int c0 = ch * TC_CH, nb = min(TC_CH, units - c0), st = (ch - ch0) & 1;
        mbar_expect_tx(&bar_b[st], (uint32_t)TC_B_CHUNK);
        bulk_g2s(smB + st * TC_B_CHUNK, bimg + (size_t)ch * TC_B_CHUNK, (uint32_t)TC_B_CHUNK, &bar_b[st]);
    };
    // Work items (tile, K split) are dealt round-robin to the CTAs of a grid that fills the GPU twice
    // over (two CTAs per SM); splits are cut finer than the grid so that the CTAs end together.
    Raw cur, nxt;
    bool first = true;
    pdl_launch_dependents();
    for (int item = (int)blockIdx.x; item < items; item += (int)gridDim.x) {
    {
        const int sp = item % S;
        tile = item / S;
        ch0 = (int)((long long)sp * n_chunks / S); ch1 = (int)((long long)(sp + 1) * n_chunks / S);
        my_row = row_of(lane_row, wmine);
    }
#pragma unroll
    for (int c = 0; c < TC_MYCOLS; ++c) acc[c] = 0.f;
    if (ch0 < ch1) fetch(ch0, cur);
    if (first) { pdl_wait(); first = false; }           // the B image comes from the kernel before this one; weights were requested above
    if (ch0 < ch1 && tid == 0) fetch_b(ch0);

    for (int ch = ch0; ch < ch1; ++ch) {
        const int c0 = ch * TC_CH, nb = min(TC_CH, units - c0), st = (ch - ch0) & 1;
        uint8_t* smBc = smB + st * TC_B_CHUNK;
        if (ch + 1 < ch1) {
            fetch(ch + 1, nxt);
            if (tid == 0) fetch_b(ch + 1);                  // its buffer was last read in chunk ch - 1, which ended with a barrier
        }
        // block scales of this thread's row: value = sa * q' + sb per weight (q' = q - 8 and sb = 0 for Q4_0)
        float sa[TC_CH], sb[TC_CH];
        if constexpr (WT == WT_Q4_0) {
#pragma unroll
            for (int j = 0; j < TC_CH; ++j) { sa[j] = __half2float(__ushort_as_half(cur.d[j])); sb[j] = 0.f; }
        } else {
#pragma unroll
            for (int gl = 0; gl < 2; ++gl) {
                float m0, m1;
                q4k_scales(cur.h, (ch & 1) * 2 + gl, sa[2 * gl], m0, sa[2 * gl + 1], m1);
                sb[2 * gl] = -m0; sb[2 * gl + 1] = -m1;
            }
        }
#pragma unroll
        for (int i = 0; i < NQ; ++i) {
            const int idx = i * TC_THREADS + tid, rl = idx >> 2, u = idx & 3;
            const uint4 q = cur.q[i];
            const uint32_t l0 = q.x & 0x0F0F0F0Fu, l1 = q.y & 0x0F0F0F0Fu, l2 = q.z & 0x0F0F0F0Fu, l3 = q.w & 0x0F0F0F0Fu;
            const uint32_t h0 = (q.x >> 4) & 0x0F0F0F0Fu, h1 = (q.y >> 4) & 0x0F0F0F0Fu, h2 = (q.z >> 4) & 0x0F0F0F0Fu, h3 = (q.w >> 4) & 0x0F0F0F0Fu;
            // row rl of a pair image; the 16-byte piece c (8 values of K) goes to piece c ^ (rl & 7)
            uint8_t* rowp = smA + (u >> 1) * TC_PAIR_IMG + (rl >> 3) * 1024 + (rl & 7) * 128;
            const int x7 = rl & 7;
            int c_lo, c_hi;                                     // first piece of the low / high nibbles' 16 values
            if constexpr (WT == WT_Q4_0) {
                // unit u = block u = half (u & 1) of pair u >> 1: low nibbles are its values 0..15, high nibbles 16..31
                c_lo = (u & 1) * 4; c_hi = c_lo + 2;
            } else {
                // units 2g, 2g+1 = bytes 0..15, 16..31 of group g = pair g: low nibbles sub-block 2g (first half
                // of the pair), high nibbles sub-block 2g+1 (second half)
                c_lo = (u & 1) * 2; c_hi = 4 + c_lo;
            }
            *reinterpret_cast<uint4*>(rowp + (((c_lo) ^ x7) << 4)) = nib8_to_h8(l0, l1, off);
            *reinterpret_cast<uint4*>(rowp + (((c_lo + 1) ^ x7) << 4)) = nib8_to_h8(l2, l3, off);
            *reinterpret_cast<uint4*>(rowp + (((c_hi) ^ x7) << 4)) = nib8_to_h8(h0, h1, off);
            *reinterpret_cast<uint4*>(rowp + (((c_hi + 1) ^ x7) << 4)) = nib8_to_h8(h2, h3, off);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        {
            uint32_t& ph = st ? ph_b1 : ph_b0;
            if (!dead && !mbar_wait(&bar_b[st], ph)) { dead = true; atomicOr(a.err, DEVERR_WAIT); }
            ph ^= 1u;
        }
        if (tid == 0) issue(0, smBc);
#pragma unroll
        for (int j = 0; j < TC_CH; ++j) {
            if (j < nb) {
                if (j + 1 < nb && tid == 0) issue(j + 1, smBc);    // runs while block j is read below
                uint32_t& ph = (j & 1) ? ph_m1 : ph_m0;
                if (!dead && !mbar_wait(&bar_m[j & 1], ph)) { dead = true; atomicOr(a.err, DEVERR_WAIT); }
                ph ^= 1u;
                tc_fence_after();
                const float* sx = reinterpret_cast<const float*>(smBc + TC_B_SUMS + j * (TC_COLS * 4));
                const float fa = sa[j], fb = sb[j];
                const uint32_t t0 = tlane + (uint32_t)(j & 1) * TC_N;
                {
                    float hi[32], lo[32];
                    tc_ld32(t0 + chalf * 32, hi);
                    tc_ld32(t0 + TC_COLS + chalf * 32, lo);
                    tc_ld_wait();
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float f = fmaf(hi[c], 2048.f, lo[c]);
                        if constexpr (WT == WT_Q4_0) acc[c] = fmaf(fa, f, acc[c]);
                        else acc[c] = fmaf(fa, f, fmaf(fb, sx[chalf * 32 + c], acc[c]));
                    }
                }
                tc_fence_before();
                __syncthreads();                        // this accumulator (and, after the last block, the images) may be overwritten
            }
        }
        cur = nxt;
    }

    // ---- epilogue ----
    const int r_out = PAIR ? (tid & 63) : lane_row;             // row of the tile this thread finishes
    const int row = tile * TILE_ROWS + r_out;
    auto finish = [&](int c, float v0, float v1) {              // column c: scale back, activation, store
        if (c < a.B && row < a.N) {
            const float sc = inv[c];
            float out = v0 * sc;
            if constexpr (PAIR) out = (a.epi == EPI_GEGLU ? gelu_tanh(out) : silu_clip(out)) * (v1 * sc);
            a.y[(size_t)c * a.ldy + row] = out;
        }
    };
    if (S == 1) {
        if constexpr (!PAIR) {
#pragma unroll
            for (int c = 0; c < TC_MYCOLS; ++c) finish(chalf * TC_MYCOLS + c, acc[c], 0.f);
        } else {
            // gate (lanes 0..63) and up (lanes 64..127) of a row meet through shared memory
            float* ex = reinterpret_cast<float*>(sm);           // [64 columns][128 lanes]; the images are no longer read
#pragma unroll
            for (int c = 0; c < TC_MYCOLS; ++c) ex[(chalf * TC_MYCOLS + c) * 128 + lane_row] = acc[c];
            __syncthreads();
            for (int c = tid >> 6; c < a.B; c += TC_THREADS / 64) finish(c, ex[c * 128 + r_out], ex[c * 128 + 64 + r_out]);
        }
    } else {
        // partial sums of this (tile, split): [64 columns][128 lanes]
        float* mine = part + (size_t)item * TC_COLS * 128;
#pragma unroll
        for (int c = 0; c < TC_MYCOLS; ++c) mine[(chalf * TC_MYCOLS + c) * 128 + lane_row] = acc[c];
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned int t = atomicAdd(&tickets[tile], 1u);
            s_last = t == (unsigned int)(S - 1);
            if (s_last) tickets[tile] = 0u;
        }
        __syncthreads();
        if (s_last) {
            // the last CTA of the tile adds the splits in order, 8 columns x 4 splits of loads in flight
            __threadfence();
            const float* base = part + (size_t)tile * S * TC_COLS * 128;
            constexpr int CG = 8;
            constexpr int GSTEP = TC_THREADS / TILE_ROWS;       // column groups worked on side by side
            for (int g8 = tid / TILE_ROWS; g8 * CG < a.B; g8 += GSTEP) {
                float v0[CG], v1[CG];
#pragma unroll
                for (int e = 0; e < CG; ++e) { v0[e] = 0.f; v1[e] = 0.f; }
                for (int s0 = 0; s0 < S; s0 += 4) {
                    float t0[4][CG], t1[4][CG];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float* p = base + ((size_t)min(s0 + i, S - 1) * TC_COLS + g8 * CG) * 128;
#pragma unroll
                        for (int e = 0; e < CG; ++e) {
                            t0[i][e] = __ldcg(p + e * 128 + r_out);
                            if constexpr (PAIR) t1[i][e] = __ldcg(p + e * 128 + 64 + r_out);
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if (s0 + i < S) {
#pragma unroll
                            for (int e = 0; e < CG; ++e) { v0[e] += t0[i][e]; if constexpr (PAIR) v1[e] += t1[i][e]; }
                        }
                    }
                }
#pragma unroll
                for (int e = 0; e < CG; ++e) finish(g8 * CG + e, v0[e], v1[e]);
            }
        }
    }
    __syncthreads();                                    // the images, s_last and the exchange buffer are free again
    }   // work items
    if (warp == 0) tc_dealloc(tmem, TC_TMEM_COLS);
}

// ---- host ----------------------------------------------------------------------------------------
bool gemm_tc_supports(int wtype, const GemvArgs& a) {
    if (g_tc_policy < 0) g_tc_policy = getenv("ADAM_B200_TC") ? atoi(getenv("ADAM_B200_TC")) : 1;
    if (g_tc_policy == 0 || !g_tc.ok) return false;
    if (a.B < TC_MIN_ROWS || a.B > TC_COLS) return false;
    if (a.epi != EPI_STORE && a.epi != EPI_GEGLU && a.epi != EPI_SWIGLU) return false;
    if (a.K <= 0 || a.K > TC_MAX_K || a.N < 16 || !a.y) return false;
    if (wtype == WT_Q4_0 ? (a.K % 32) != 0 : (a.K % 256) != 0) return false;
    if ((a.ldx & 3) || (!a.h_in && !a.x)) return false;
    const bool pair = a.epi != EPI_STORE;
    if (g_tc_policy == 1) {
        // The GEMV kernels pass over the weights once per 4 rows; this kernel passes once but has a fixed
        // cost of 10-15 us.  Measured cross-over: weights x passes of about 2e8 (Q4_0) / 1e8 (Q4_K) elements.
        const double work = (double)a.N * a.K * (pair ? 2 : 1) * ((a.B + 3) / 4);
        if (work < (wtype == WT_Q4_0 ? 2.0e8 : 1.0e8)) return false;
    }
    const int tiles = pair ? (a.N + 63) / 64 : (a.N + 127) / 128;
    return tiles <= TC_MAX_CTAS && tiles <= TC_MAX_TILES && (size_t)a.K * 4 <= 160 * 1024;
}

int launch_gemm_tc(int wtype, const GemvArgs& a_in, cudaStream_t stream) {
    GemvArgs a = a_in;
    a.err = g.dev_err;
    const bool pair = a.epi != EPI_STORE;
    const int tiles = pair ? (a.N + 63) / 64 : (a.N + 127) / 128;
    const int n_chunks = (a.K / 32 + TC_CH - 1) / TC_CH;
    // Splits per tile: the cheapest of 1..32 under a simple model (time in chunks: the items are dealt to
    // 2 CTAs per SM; every item costs its chunks plus about two chunks of fixed work, the last CTA of a
    // tile also reads every split's partial sums).
    const int slots = 2 * g.sm_count;
    int S = 1;
    {
        double best = 1e30;
        for (int c = 1; c <= 32 && c <= n_chunks; ++c) {
            const long long it = (long long)tiles * c;
            if (it > TC_MAX_CTAS) break;
            const double rounds = (double)((it + slots - 1) / slots);
            const double cost = rounds * ((double)((n_chunks + c - 1) / c) + 2.0) + (c > 1 ? 0.5 + 0.1 * c : 0.0);
            if (cost < best - 1e-9) { best = cost; S = c; }
        }
    }
    const int items = tiles * S;
    static bool attr_done = false;
    if (!attr_done) {
        cudaFuncSetAttribute(k_quant_rows, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_K, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_K, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
        attr_done = true;
    }
    launch_k(k_quant_rows, dim3(TC_COLS), dim3(QR_THREADS), (a.K >> 2) <= QR_THREADS * QR_MAXV ? (size_t)0 : (size_t)a.K * 4, stream, g.pdl, a, g_tc.bimg, g_tc.inv);
    count_launch();
    const dim3 grid((unsigned)(items < slots ? items : slots)), block(TC_THREADS);
    if (wtype == WT_Q4_0) {
        if (pair) launch_k(k_gemm_tc<WT_Q4_0, true>, grid, block, (size_t)TC_SMEM, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
        else launch_k(k_gemm_tc<WT_Q4_0, false>, grid, block, (size_t)TC_SMEM, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
    } else {
        if (pair) launch_k(k_gemm_tc<WT_Q4_K, true>, grid, block, (size_t)TC_SMEM, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
        else launch_k(k_gemm_tc<WT_Q4_K, false>, grid, block, (size_t)TC_SMEM, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
    }
    count_launch();
    ++g_tc_calls;
    return check_launch("gemm_tc");
}

}  // namespace ab

// Number of GEMMs enqueued on the tcgen05 path since the library was loaded (tests use it to
// see which kernel a call took).
extern "C" uint64_t adam_b200_tc_gemm_count(void) { return ab::g_tc_calls; }
// 0 = never use the tcgen05 GEMM, 1 = where it is expected to be faster (default), 2 = whenever the shape allows.
extern "C" int adam_b200_tc_gemm_policy(int policy) {
    if (policy < 0 || policy > 2) return ADAMAH_ERR_INVALID;
    ab::g_tc_policy = policy;
    return ADAMAH_OK;
}
