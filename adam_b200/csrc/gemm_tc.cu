// Dequant-fused GEMM  y[b][n] = sum_k W[n][k] x[b][k]  for 9..64 activation rows b (a prefill chunk
// or a large decode batch) on the 5th-generation tensor cores: tcgen05.mma with the accumulator in
// tensor memory (TMEM).  Same operator as the GEMV kernels (the reference's Q4 mat-vec shader
// adamah-MAIN/adamah/shaders/src/f32/map_matvec_t_xq4.comp and map_fused_gateup_t_xq4.comp run once
// per row by adamah.c:8606-8691).  Arithmetic: a row's activations become integers of up to 23 bits
// with one power-of-two scale per row, split into two signed parts that fp16 holds exactly
// (x = 2048 x_hi + x_lo); a weight is dequantised in fp32 (block scale and offset applied) and split
// into two fp16 terms (22 bits); the three significant cross products are accumulated over all of K in
// fp32 in TMEM and combined once per output.  Measured error ~5e-7 of max |y| (operator tolerance 1e-3).
//
// Two kernels:
//   k_quant_rows   one CTA per activation row: the optional input chain (residual add + RMS norms,
//                  as the GEMV prologue; the row stays in registers and all loads are issued before
//                  the first use), the row's scale, and the row's two fp16 planes written straight
//                  into the B-operand image in global memory: K-major with the 128-byte swizzle,
//                  two 32-wide K blocks per 128-byte operand row, 128 operand rows (row n = plane *
//                  64 + activation row) = 16 KB per block pair (behind each chunk of two pairs the
//                  4 x 64 per-row integer sums are kept as floats for callers that want them).
//   k_gemm_tc      256 threads, two CTAs per SM (256 TMEM columns and 97 KB of shared memory each), a
//                  grid that fills the GPU twice over and takes work items (tile of 128 weight rows
//                  x K split) round-robin; see the comment at the kernel.  K splits leave partial
//                  sums in a workspace; the last CTA of a tile (atomic ticket) adds them in split
//                  order and runs the epilogue (store, or GeGLU / SwiGLU over a tile of 64 gate
//                  rows + 64 up rows).
// Every wait (bulk copy, tensor-core completion) is bounded: when one runs out the kernel records
// DEVERR_WAIT, stops waiting, and still frees its tensor memory.  The shared-memory request keeps a
// third CTA off an SM, so a TMEM allocation never waits on a CTA that cannot run.
#include "gemm_tc.cuh"
#include "gemv_mma.cuh"

#include <cstdlib>

namespace ab {

constexpr int TC_PLANES = 2;
constexpr int TC_N = TC_PLANES * TC_COLS;                // 128 B-operand rows
constexpr int TC_CH = 4;                                 // K blocks per chunk of the B image (two pair images + the sums)
// Operand images, K-major with the 128-byte swizzle: a "pair" image holds two K blocks (64 fp16 = 128
// bytes per operand row) of 128 operand rows = 16 KB: 8-row groups of 1024 bytes, a row's 128 bytes
// contiguous, and the 16-byte piece c of row r stored at piece c ^ (r & 7).  Images start at
// multiples of 1024 bytes (the swizzle works on address bits).
constexpr int TC_PAIR_IMG = 128 * 128;                   // 16384
constexpr int TC_A_CHUNK = (TC_CH / 2) * TC_PAIR_IMG;    // 32768
constexpr int TC_B_SUMS = TC_A_CHUNK;                    // offset of the chunk's [4][64] row sums in the B chunk image
constexpr int TC_B_CHUNK = TC_A_CHUNK + TC_CH * TC_COLS * 4;        // 33792 = 33 * 1024
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

// ---- the GEMM ---------------------------------------------------------------------------------
// Weights enter the tensor core already scaled: w = 64 * (sa * q + sb) in fp32 (the factor keeps the low
// term of typical weights out of the fp16 subnormals; |sa * q + sb| must stay below 1000) (sa, sb the block's
// scale and offset: d and -8 d for Q4_0, d*sc and -dmin*m for Q4_K), split into two fp16 terms
// w_hi + w_lo (22 bits).  With the activations' planes x_hi, x_lo the product is
//   sum_k w x = 2048 * (sum w_hi x_hi + sum w_lo x_hi) + sum w_hi x_lo      (w_lo x_lo is below fp32 resolution)
// and all of a work item's K is accumulated in TMEM: D1 (128 columns) = w_hi x [x_hi | x_lo],
// D2 (64 columns) = w_lo x x_hi.  Nothing is read back per block.
//
// Per step of two K blocks (64 values of K, one 128-byte operand row): the threads expand one 16-byte
// unit of nibbles each into the two A images of buffer b (the unit was requested one step ahead), one
// thread waits for the step's B image (16 KB bulk copy, requested one step ahead into buffer b) and
// issues 4 x 2 tcgen05.mma (K 16 each; N 128 and N 64) and a commit that frees buffer b two steps later.
// grid = min(items, 2 per SM); item = (tile of 128 weight rows, K split) dealt round-robin.
// PAIR: a tile is 64 rows of w0 (gate) in TMEM lanes 0..63 and the same 64 rows of w1 (up) in lanes 64..127.
constexpr uint32_t TC_IDESC_N64 = (1u << 4) | ((uint32_t)(TC_COLS >> 3) << 17) | ((128u >> 4) << 24);
constexpr int TC_A_BUF = 2 * TC_PAIR_IMG;               // w_hi image + w_lo image of one step
constexpr int TC_SMEM2 = 2 * TC_A_BUF + 2 * TC_PAIR_IMG + 1024;     // 99328: two A buffers, two B buffers, alignment slack

// Four nibbles-as-bytes of t -> sa * q + sb (the callers pass scales times 64) as fp16 high and low terms (two packed pairs each).
__device__ __forceinline__ void nib4_split(uint32_t t, float sa, float sb, uint32_t (&hi)[2], uint32_t (&lo)[2]) {
    float w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // byte i of t into mantissa bits 16..23 of 2^7: the float 128 + q, exactly
        const float f = __uint_as_float(__byte_perm(t, 0x43000000u, 0x7054u | ((uint32_t)i << 8)));
        w[i] = fmaf(sa, f - 128.f, sb);
    }
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const __half2 h = __floats2half2_rn(w[2 * p], w[2 * p + 1]);
        const float2 hf = __half22float2(h);
        const __half2 l = __floats2half2_rn(w[2 * p] - hf.x, w[2 * p + 1] - hf.y);
        hi[p] = *reinterpret_cast<const uint32_t*>(&h);
        lo[p] = *reinterpret_cast<const uint32_t*>(&l);
    }
}

template <int WT, bool PAIR>
__global__ void __launch_bounds__(TC_THREADS, 2) k_gemm_tc(const GemvArgs a, const uint8_t* __restrict__ bimg, const float* __restrict__ inv,
                                                           float* __restrict__ part, unsigned int* __restrict__ tickets, int S, int items) {
    extern __shared__ __align__(1024) uint8_t sm_raw[];
    uint8_t* sm = sm_raw + ((1024u - (smem_u32(sm_raw) & 1023u)) & 1023u);     // the swizzle needs images at multiples of 1024 bytes
    uint8_t* smA = sm;                                  // [2 buffers][w_hi image, w_lo image]
    uint8_t* smB = sm + 2 * TC_A_BUF;                   // [2 buffers][pair image]
    __shared__ __align__(8) uint64_t bar_b[2], bar_free[2];
    __shared__ uint32_t s_tmem;
    __shared__ bool s_last;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int lane_row = tid & 127, chalf = tid >> 7;          // TMEM lane (row of the tile) and column half this thread reads back
    const int urow = tid >> 1, uu = tid & 1;                    // operand row and 16-byte unit (of the step's two) this thread expands
    const int units = a.K >> 5, n_steps = (units + 1) >> 1;
    constexpr int TILE_ROWS = PAIR ? 64 : 128;
    int tile = 0;
    auto row_of = [&](int l, const WeightRef*& w) -> int {      // the weight row behind TMEM lane l of this tile
        if constexpr (PAIR) { w = (l >> 6) ? &a.w1 : &a.w0; return min(tile * 64 + (l & 63), a.N - 1); }
        else { w = &a.w0; return min(tile * 128 + l, a.N - 1); }
    };
    if (tid == 0) { mbar_init(&bar_b[0], 1); mbar_init(&bar_b[1], 1); mbar_init(&bar_free[0], 1); mbar_init(&bar_free[1], 1); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) tc_alloc(&s_tmem, TC_TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem;
    const uint32_t tlane = tmem + ((uint32_t)((warp & 3) * 32) << 16);
    bool dead = false;
    auto wait_on = [&](uint64_t* bar, uint32_t parity) {
        if (!dead && !mbar_wait(bar, parity)) { dead = true; atomicOr(a.err, DEVERR_WAIT); }
    };

    struct Raw { uint4 q; uint4 h; unsigned short d; };
    const WeightRef* wu = nullptr;
    int r_u = 0;
    auto fetch = [&](int st, Raw& r) {                      // this thread's unit of step st (weights only: no dependency on earlier kernels)
        if constexpr (WT == WT_Q4_0) {
            const int blk = min(2 * st + uu, units - 1);
            r.q = ld_stream(wu->q + (size_t)r_u * units + blk);
            r.d = __ldg(reinterpret_cast<const unsigned short*>(wu->d) + (size_t)r_u * units + blk);
        } else {
            const uint4* sb = wu->q + ((size_t)r_u * (units >> 3) + (st >> 2)) * 9;
            r.h = __ldg(sb);
            r.q = ld_stream(sb + 1 + (st & 3) * 2 + uu);
        }
    };
    auto fetch_b = [&](int st, int b) {                     // thread 0: the step's B pair image into buffer b
        mbar_expect_tx(&bar_b[b], (uint32_t)TC_PAIR_IMG);
        bulk_g2s(smB + b * TC_PAIR_IMG, bimg + (size_t)(st >> 1) * TC_B_CHUNK + (size_t)(st & 1) * TC_PAIR_IMG, (uint32_t)TC_PAIR_IMG, &bar_b[b]);
    };

    Raw cur, nxt;
    bool first = true;
    uint32_t it = 0;                                        // steps done by this CTA: buffer = it & 1, use number of the buffer = it >> 1
    pdl_launch_dependents();
    for (int item = (int)blockIdx.x; item < items; item += (int)gridDim.x) {
        const int sp = item % S;
        tile = item / S;
        const int st0 = (int)((long long)sp * n_steps / S), st1 = (int)((long long)(sp + 1) * n_steps / S);
        r_u = row_of(urow, wu);
        if (st0 < st1) fetch(st0, cur);
        if (first) { pdl_wait(); first = false; }           // the B image comes from the kernel before this one; weights were requested above
        if (tid == 0 && st0 < st1) {
            if ((it >> 1) >= 1u) wait_on(&bar_free[it & 1u], ((it >> 1) - 1u) & 1u);
            fetch_b(st0, (int)(it & 1u));
        }
        for (int st = st0; st < st1; ++st, ++it) {
            const uint32_t b = it & 1u, n = it >> 1;
            if (st + 1 < st1) fetch(st + 1, nxt);
            // scales of the unit's low-nibble and high-nibble halves, times 64
            float sa0, sb0, sa1, sb1;
            int p_lo, p_hi;                                 // first 16-byte piece (8 values of K) of the two halves in the 128-byte row
            if constexpr (WT == WT_Q4_0) {
                // unit = block 2 st + uu = half uu of the row: low nibbles are its values 0..15, high nibbles 16..31
                const float d = (2 * st + uu < units) ? 64.f * __half2float(__ushort_as_half(cur.d)) : 0.f;
                sa0 = sa1 = d; sb0 = sb1 = -8.f * d;
                p_lo = uu * 4; p_hi = p_lo + 2;
            } else {
                // units 2g, 2g+1 = bytes 0..15, 16..31 of group g = this step: low nibbles sub-block 2g (first half
                // of the row), high nibbles sub-block 2g+1 (second half)
                float m0, m1;
                q4k_scales(cur.h, st & 3, sa0, m0, sa1, m1);
                sa0 *= 64.f; sa1 *= 64.f; sb0 = -64.f * m0; sb1 = -64.f * m1;
                p_lo = uu * 2; p_hi = 4 + p_lo;
            }
            if (n >= 1u) wait_on(&bar_free[b], (n - 1u) & 1u);  // the tensor core has finished with buffer b
            {
                const uint32_t l[4] = {cur.q.x & 0x0F0F0F0Fu, cur.q.y & 0x0F0F0F0Fu, cur.q.z & 0x0F0F0F0Fu, cur.q.w & 0x0F0F0F0Fu};
                const uint32_t h[4] = {(cur.q.x >> 4) & 0x0F0F0F0Fu, (cur.q.y >> 4) & 0x0F0F0F0Fu, (cur.q.z >> 4) & 0x0F0F0F0Fu, (cur.q.w >> 4) & 0x0F0F0F0Fu};
                uint8_t* rowp = smA + b * TC_A_BUF + (urow >> 3) * 1024 + (urow & 7) * 128;
                const int x7 = urow & 7;
#pragma unroll
                for (int pc = 0; pc < 2; ++pc) {            // 16-byte pieces: words 2 pc, 2 pc + 1 of each nibble half
                    uint32_t ha[2], la[2], hb[2], lb[2];
                    nib4_split(l[2 * pc], sa0, sb0, ha, la); nib4_split(l[2 * pc + 1], sa0, sb0, hb, lb);
                    *reinterpret_cast<uint4*>(rowp + (((p_lo + pc) ^ x7) << 4)) = make_uint4(ha[0], ha[1], hb[0], hb[1]);
                    *reinterpret_cast<uint4*>(rowp + TC_PAIR_IMG + (((p_lo + pc) ^ x7) << 4)) = make_uint4(la[0], la[1], lb[0], lb[1]);
                    nib4_split(h[2 * pc], sa1, sb1, ha, la); nib4_split(h[2 * pc + 1], sa1, sb1, hb, lb);
                    *reinterpret_cast<uint4*>(rowp + (((p_hi + pc) ^ x7) << 4)) = make_uint4(ha[0], ha[1], hb[0], hb[1]);
                    *reinterpret_cast<uint4*>(rowp + TC_PAIR_IMG + (((p_hi + pc) ^ x7) << 4)) = make_uint4(la[0], la[1], lb[0], lb[1]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncthreads();
            if (tid == 0) {
                if (st + 1 < st1) {                         // next step's B image into the other buffer (free once the step before this one is done)
                    const uint32_t b1 = (it + 1u) & 1u, n1 = (it + 1u) >> 1;
                    if (n1 >= 1u) wait_on(&bar_free[b1], (n1 - 1u) & 1u);
                    fetch_b(st + 1, (int)b1);
                }
                wait_on(&bar_b[b], n & 1u);
                tc_fence_after();
                const uint32_t ahi = smem_u32(smA + b * TC_A_BUF), alo = ahi + TC_PAIR_IMG, bb = smem_u32(smB + b * TC_PAIR_IMG);
#pragma unroll
                for (uint32_t t = 0; t < 4; ++t) {
                    const uint32_t accf = (st > st0 || t > 0) ? 1u : 0u;
                    tc_mma_f16(tmem, tc_desc(ahi + t * 32u), tc_desc(bb + t * 32u), TC_IDESC, accf);
                    tc_mma_f16(tmem + TC_N, tc_desc(alo + t * 32u), tc_desc(bb + t * 32u), TC_IDESC_N64, accf);
                }
                tc_commit(&bar_free[b]);
            }
            cur = nxt;
        }
        // ---- all of this item's K is in TMEM: read it back once ----
        float acc[TC_MYCOLS];
        if (st0 < st1) {
            const uint32_t last = it - 1u;
            wait_on(&bar_free[last & 1u], (last >> 1) & 1u);    // the last commit covers every instruction before it
            tc_fence_after();
            float hh[32], hl[32], lh[32];
            tc_ld32(tlane + chalf * 32, hh);                    // w_hi x x_hi
            tc_ld32(tlane + TC_COLS + chalf * 32, hl);          // w_hi x x_lo
            tc_ld32(tlane + TC_N + chalf * 32, lh);             // w_lo x x_hi
            tc_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[c] = fmaf(hh[c] + lh[c], 2048.f, hl[c]);
            tc_fence_before();
        } else {
#pragma unroll
            for (int c = 0; c < 32; ++c) acc[c] = 0.f;
        }
    // ---- epilogue ----
    const int r_out = PAIR ? (tid & 63) : lane_row;             // row of the tile this thread finishes
    const int row = tile * TILE_ROWS + r_out;
    auto finish = [&](int c, float v0, float v1) {              // column c: scale back, activation, store
        if (c < a.B && row < a.N) {
            const float sc = inv[c] * (1.f / 64.f);             // the weights went in times 64
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
    if (wtype != WT_Q4_0 && wtype != WT_Q4_K) return false;
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
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_0, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM2);
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM2);
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_K, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM2);
        cudaFuncSetAttribute(k_gemm_tc<WT_Q4_K, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM2);
        attr_done = true;
    }
    launch_k(k_quant_rows, dim3(TC_COLS), dim3(QR_THREADS), (a.K >> 2) <= QR_THREADS * QR_MAXV ? (size_t)0 : (size_t)a.K * 4, stream, g.pdl, a, g_tc.bimg, g_tc.inv);
    count_launch();
    const dim3 grid((unsigned)(items < slots ? items : slots)), block(TC_THREADS);
    if (wtype == WT_Q4_0) {
        if (pair) launch_k(k_gemm_tc<WT_Q4_0, true>, grid, block, (size_t)TC_SMEM2, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
        else launch_k(k_gemm_tc<WT_Q4_0, false>, grid, block, (size_t)TC_SMEM2, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
    } else {
        if (pair) launch_k(k_gemm_tc<WT_Q4_K, true>, grid, block, (size_t)TC_SMEM2, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
        else launch_k(k_gemm_tc<WT_Q4_K, false>, grid, block, (size_t)TC_SMEM2, stream, g.pdl, a, (const uint8_t*)g_tc.bimg, (const float*)g_tc.inv, g_tc.part, g_tc.tickets, S, items);
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
