// Row-tiled copies of Q4_0 and Q4_K tensors for the tensor-core GEMV (gemv_mma.cuh).
//
// A GGUF-block map is a flat element array and does not know tensor shapes, so the
// plane layout used by the generic kernels keeps rows apart (a row's blocks are
// contiguous).  The tensor-core GEMV wants 16 rows of the same block side by side, in
// the order its lanes consume them.  `adam_b200_tensor_tile` builds such a copy for one
// [rows, cols] tensor of a GGUF-block map and registers it under (map, element offset, rows,
// cols); operators that are later called on exactly that tensor use the copy.  The
// Q4_0 bytes are the same 18 per block (16 nibble bytes + fp16 scale), only their order
// changes, so block decode stays bit-identical; the Q4_K form is described at k_tile_q4_k (role of the reference's load-time
// re-layout into its Q4 map, adam/models/engine.py:1049-1056).
//
// Q4_0 tile pair = 16 rows x 2 blocks (64 weights per row) = 576 bytes:
//   bytes   0..511  one uint4 per lane (lane = 4*g + t, g = 0..7, t = 0..3):
//                   { block0: row g word t, row g+8 word t, block1: row g word t, row g+8 word t }
//                   where word t of a block is its nibble bytes 4t..4t+3
//   bytes 512..575  per g: 4 halves { d[g][b0], d[g+8][b0], d[g][b1], d[g+8][b1] }
// Tile pairs of a 16-row group are contiguous along K; groups follow each other.
#include "common.cuh"
#include "gemv.cuh"
#include "gemv_mma.cuh"

#include <vector>

namespace ab {

struct TiledEntry { uint32_t map_id; uint64_t elem_off; uint32_t rows, cols; void* dev; size_t bytes; };
static std::vector<TiledEntry> g_tiled;

const void* find_tiled(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols) {
    for (const TiledEntry& e : g_tiled)
        if (e.map_id == map_id && e.elem_off == elem_off && e.rows == rows && e.cols == cols) return e.dev;
    return nullptr;
}

// A tensor that starts at elem_off and spans rows*cols, possibly a leading slice of a
// registered one (e.g. a wider QKV view or a row prefix): same cols, offset equal,
// rows a multiple of 16 and not beyond the registered rows.
const void* find_tiled_prefix(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols) {
    for (const TiledEntry& e : g_tiled)
        if (e.map_id == map_id && e.elem_off == elem_off && e.cols == cols && rows <= e.rows && rows % 16 == 0) return e.dev;
    return nullptr;
}

void tiled_drop_map(uint32_t map_id) {
    for (size_t i = 0; i < g_tiled.size();) {
        if (g_tiled[i].map_id == map_id || map_id == 0xFFFFFFFFu) { cudaFree(g_tiled[i].dev); g_tiled.erase(g_tiled.begin() + i); }
        else ++i;
    }
}

__global__ void k_tile_q4_0(const uint4* __restrict__ qs, const __half* __restrict__ d, uint32_t rows, uint32_t blocks_per_row,
                            uint8_t* __restrict__ out) {
    // one warp per tile pair
    const uint64_t pair = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t pairs_per_group = blocks_per_row / 2;
    const uint64_t n_pairs = (uint64_t)(rows / 16) * pairs_per_group;
    if (pair >= n_pairs) return;
    const uint32_t rg = (uint32_t)(pair / pairs_per_group), bp = (uint32_t)(pair % pairs_per_group);
    const size_t r0 = (size_t)rg * 16 + g, r1 = r0 + 8;
    const uint32_t b0 = 2 * bp, b1 = b0 + 1;
    auto word = [&](size_t row, uint32_t blk) -> uint32_t {
        return reinterpret_cast<const uint32_t*>(qs + row * blocks_per_row + blk)[t];
    };
    uint4 v;
    v.x = word(r0, b0); v.y = word(r1, b0); v.z = word(r0, b1); v.w = word(r1, b1);
    uint8_t* tile = out + pair * 576;
    reinterpret_cast<uint4*>(tile)[lane] = v;
    if (t == 0) {
        __half* sc = reinterpret_cast<__half*>(tile + 512) + g * 4;
        sc[0] = d[r0 * blocks_per_row + b0]; sc[1] = d[r1 * blocks_per_row + b0];
        sc[2] = d[r0 * blocks_per_row + b1]; sc[3] = d[r1 * blocks_per_row + b1];
    }
}

// Q4_K: same nibble order per 32-weight block as above (byte i of word t: low nibble = weight
// 4t+i, high nibble = weight 16+4t+i of the block), built from the superblock's own pairing
// (byte j of a 64-weight group: low nibble = weight j, high nibble = weight 32+j).  A tile
// pair covers one 64-weight group = sub-blocks 2q and 2q+1 of a superblock:
//   bytes   0..511  as for Q4_0
//   bytes 512..575  per g: { blk0: sc[g], m[g], sc[g+8], m[g+8]; blk1: the same } 6-bit values as bytes
//   bytes 576..639  per g: 4 halves { d[g], dmin[g], d[g+8], dmin[g+8] } of the superblock
// so a pair is 640 bytes (576 in GGUF): the superblock header is repeated in its four pairs.
__device__ __forceinline__ void q4k_sc_m(const uint8_t* sc12, int j, uint32_t& sc, uint32_t& mn) {
    // 6-bit scale and min of sub-block j (unpack at adam/loaders/gguf.py:325-328)
    if (j < 4) { sc = sc12[j] & 63u; mn = sc12[j + 4] & 63u; }
    else { sc = (sc12[j + 4] & 0x0Fu) | ((sc12[j - 4] >> 6) << 4); mn = (sc12[j + 4] >> 4) | ((sc12[j] >> 6) << 4); }
}
__global__ void k_tile_q4_k(const uint8_t* __restrict__ blocks, uint32_t rows, uint32_t sb_per_row, uint8_t* __restrict__ out) {
    const uint64_t pair = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const uint32_t pairs_per_group = sb_per_row * 4;
    const uint64_t n_pairs = (uint64_t)(rows / 16) * pairs_per_group;
    if (pair >= n_pairs) return;
    const uint32_t rg = (uint32_t)(pair / pairs_per_group), bp = (uint32_t)(pair % pairs_per_group);
    const uint32_t sb = bp / 4, q = bp % 4;
    const size_t r0 = (size_t)rg * 16 + g, r1 = r0 + 8;
    const uint8_t* s0 = blocks + (r0 * sb_per_row + sb) * 144;
    const uint8_t* s1 = blocks + (r1 * sb_per_row + sb) * 144;
    auto words = [&](const uint8_t* sblk, uint32_t& lo, uint32_t& hi) {
        const uint32_t* qs = reinterpret_cast<const uint32_t*>(sblk + 16 + 32 * q);
        const uint32_t A = qs[t], B = qs[4 + t];                 // bytes 4t..4t+3 and 16+4t..16+4t+3 of the group
        lo = (A & 0x0F0F0F0Fu) | ((B & 0x0F0F0F0Fu) << 4);      // sub-block 2q
        hi = ((A >> 4) & 0x0F0F0F0Fu) | (B & 0xF0F0F0F0u);      // sub-block 2q+1
    };
    uint4 v;
    words(s0, v.x, v.z);
    words(s1, v.y, v.w);
    uint8_t* tile = out + pair * 640;
    reinterpret_cast<uint4*>(tile)[lane] = v;
    if (t < 2) {            // lane t writes block t's scale bytes
        uint32_t a, b, c, d2;
        q4k_sc_m(s0 + 4, 2 * q + t, a, b);
        q4k_sc_m(s1 + 4, 2 * q + t, c, d2);
        reinterpret_cast<uint32_t*>(tile + 512)[g * 2 + t] = a | (b << 8) | (c << 16) | (d2 << 24);
    } else if (t == 2) {
        uint2 h;
        h.x = *reinterpret_cast<const uint32_t*>(s0);            // d | dmin << 16
        h.y = *reinterpret_cast<const uint32_t*>(s1);
        reinterpret_cast<uint2*>(tile + 576)[g] = h;
    }
}

int tile_tensor(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols) {
    Map* m = get_map(map_id);
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    const bool q40 = m->dtype == ADAMAH_DTYPE_GGUF_Q4_0, q4k = m->dtype == ADAMAH_DTYPE_GGUF_Q4_K;
    if (!q40 && !q4k) return fail(ADAMAH_ERR_INVALID, "tensor_tile: map %u does not hold GGUF Q4_0 / Q4_K blocks", map_id);
    if (rows == 0 || cols == 0 || rows % 16 || cols % (q40 ? 64 : 256))
        return fail(ADAMAH_ERR_INVALID, "tensor_tile: need rows %% 16 == 0 and cols %% %d == 0", q40 ? 64 : 256);
    if (elem_off % (q40 ? 32 : 256) || elem_off + (uint64_t)rows * cols > m->n_elems) return fail(ADAMAH_ERR_INVALID, "tensor_tile: tensor lies beyond map %u", map_id);
    if (find_tiled(map_id, elem_off, rows, cols)) return ADAMAH_OK;
    const uint64_t n_pairs = (uint64_t)(rows / 16) * (cols / 64);
    const size_t bytes = (size_t)n_pairs * (q40 ? 576 : 640);
    void* dev = nullptr;
    if (cudaMalloc(&dev, bytes) != cudaSuccess) { cudaGetLastError(); return fail(ADAMAH_ERR_MEMORY, "tensor_tile: out of device memory (%zu bytes)", bytes); }
    const uint64_t threads = n_pairs * 32;
    if (q40)
        k_tile_q4_0<<<(unsigned)((threads + 255) / 256), 256, 0, g.stream>>>(m->q40_qs + elem_off / 32, m->q40_d + elem_off / 32, rows, cols / 32, (uint8_t*)dev);
    else
        k_tile_q4_k<<<(unsigned)((threads + 255) / 256), 256, 0, g.stream>>>((const uint8_t*)m->buf + elem_off / 256 * 144, rows, cols / 256, (uint8_t*)dev);
    count_launch();
    cudaStreamSynchronize(g.stream);
    int rc = check_launch("tensor_tile");
    if (rc) { cudaFree(dev); return rc; }
    g_tiled.push_back(TiledEntry{map_id, elem_off, rows, cols, dev, bytes});
    return ADAMAH_OK;
}

}  // namespace ab

using namespace ab;

extern "C" int adam_b200_tensor_tile(uint32_t map_wt, uint64_t elem_off, uint32_t rows, uint32_t cols) {
    if (!ready()) return ADAMAH_ERR_INVALID;
    return tile_tensor(map_wt, elem_off, rows, cols);
}
