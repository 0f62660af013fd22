// Row-tiled copies of Q4_0 tensors for the tensor-core GEMV (gemv_mma.cuh).
//
// A GGUF-block map is a flat element array and does not know tensor shapes, so the
// plane layout used by the generic kernels keeps rows apart (a row's blocks are
// contiguous).  The tensor-core GEMV wants 16 rows of the same block side by side, in
// the order its lanes consume them.  `adam_b200_tensor_tile` builds such a copy for one
// [rows, cols] tensor of a Q4_0 map and registers it under (map, element offset, rows,
// cols); operators that are later called on exactly that tensor use the copy.  The
// bytes are the same 18 per block (16 nibble bytes + fp16 scale), only their order
// changes, so block decode stays bit-identical (role of the reference's load-time
// re-layout into its Q4 map, adam/models/engine.py:1049-1056).
//
// Tile pair = 16 rows x 2 blocks (64 weights per row) = 576 bytes:
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

int tile_tensor(uint32_t map_id, uint64_t elem_off, uint32_t rows, uint32_t cols) {
    Map* m = get_map(map_id);
    if (!m) return ADAMAH_ERR_NOT_FOUND;
    if (m->dtype != ADAMAH_DTYPE_GGUF_Q4_0) return fail(ADAMAH_ERR_INVALID, "tensor_tile: map %u does not hold Q4_0 blocks", map_id);
    if (rows == 0 || cols == 0 || rows % 16 || cols % 64) return fail(ADAMAH_ERR_INVALID, "tensor_tile: need rows %% 16 == 0 and cols %% 64 == 0");
    if (elem_off % 32 || elem_off + (uint64_t)rows * cols > m->n_elems) return fail(ADAMAH_ERR_INVALID, "tensor_tile: tensor lies beyond map %u", map_id);
    if (find_tiled(map_id, elem_off, rows, cols)) return ADAMAH_OK;
    const size_t bytes = (size_t)rows * cols / 32 * 18;
    void* dev = nullptr;
    if (cudaMalloc(&dev, bytes) != cudaSuccess) { cudaGetLastError(); return fail(ADAMAH_ERR_MEMORY, "tensor_tile: out of device memory (%zu bytes)", bytes); }
    const uint64_t n_pairs = (uint64_t)(rows / 16) * (cols / 64);
    const uint64_t threads = n_pairs * 32;
    k_tile_q4_0<<<(unsigned)((threads + 255) / 256), 256, 0, g.stream>>>(m->q40_qs + elem_off / 32, m->q40_d + elem_off / 32, rows, cols / 32, (uint8_t*)dev);
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
