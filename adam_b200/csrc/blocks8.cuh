// GGUF Q8_0 and Q5_0 block storage: the types real Gemma GGUF files use for the token embedding
// (and tied LM head) next to Q4_0 / Q4_K matrices.  The reference widens both to an 8-bit map with
// per-32 (scale, zero) pairs at load (adam/models/engine.py:1118-1198) and reads it with the *_xq8
// operators (adamah-MAIN/adamah/adamah.c:9834, :10189; shaders map_matvec_t_xq8.comp,
// map_row_gather_xq8.comp).  Here the blocks stay as they are in the file, split into planes so that
// every device load is aligned:
//   Q8_0 (34 B / 32 weights): quant plane 32 B per block (int8), then fp16 scale plane.
//   Q5_0 (22 B / 32 weights): nibble plane 16 B per block (byte j = weight j low, weight j+16 high),
//                             then high-bit plane (uint32 per block, bit j = bit 4 of weight j),
//                             then fp16 scale plane.
// Values: Q8_0 w = d * q;  Q5_0 w = d * ((nibble | high << 4) - 16)   (adam/loaders/gguf.py:282-310).
#pragma once
#include "common.cuh"
#include "gemv.cuh"

namespace ab {

inline bool wt_is_b8(int wt) { return wt == WT_Q8_0 || wt == WT_Q5_0; }

// y[b][n] = sum_k W[n][k] x[b][k] for b < B (raw products, no epilogue); x rows 16-byte aligned.
int launch_gemv_b8(int wt, const WeightRef& w, const float* x, int ldx, float* y, int ldy, int N, int K, int B, cudaStream_t st);
// out[i] = decode(first_elem + i) [* scale, rounded separately], n a multiple of 32, first_elem too.
int launch_dequant_b8(int wt, const WeightRef& w, uint64_t n_elems, float* out, float scale, bool with_scale, cudaStream_t st);
// Raw file blocks (device pointer, 2-byte aligned) -> planes of the tensor at `w`.
int launch_repack_b8(int wt, const void* raw_dev, const WeightRef& w, uint64_t n_blocks, cudaStream_t st);
// The norm chain that the Q4 GEMVs fold into their prologue, as a kernel of its own (one CTA per row):
//   h' = h_in + (add_src ? (w_post ? rms(add_src) * w_post : add_src) : 0)  -> h_out
//   x  = w_pre ? rms(h') * w_pre : h'                                       -> x_out
int launch_chain_rows(const float* h_in, const float* add_src, const float* w_post, const float* w_pre, float* h_out, float* x_out,
                      int E, int rows, float eps, cudaStream_t st, bool pdl);
// Per row of logits [rows][V]: arg-max (ties to the lower index, NaN as -FLT_MAX) into tok / val, then, if
// `store_capped`, the logits are replaced by cap * tanh(logit / cap) (cap > 0).
int launch_argmax_rows(float* logits, int V, int rows, float cap, bool store_capped, int32_t* tok, float* val, float* tok_f32,
                       cudaStream_t st, bool pdl);


// ---- placing file blocks of any supported kind into a GGUF-block map (runtime.cu) ------------------------------
// ggml type id, the map dtype that stores it, weights and bytes per block.
struct BlockKind { uint32_t ggml_type, dtype, elems, bytes; const char* name; };
const BlockKind* block_kind(uint32_t ggml_type);                 // NULL if the type is not supported
int check_block_range(const Map* m, uint32_t id, const BlockKind* k, uint32_t ggml_type, uint64_t elem_off, uint64_t n_bytes);
// Enqueue the placement of n_bytes of file blocks that already lie on the device (2-byte aligned).
int place_blocks_from_device(Map* m, const BlockKind& k, uint64_t elem_off, const void* dev_src, uint64_t n_bytes);

}  // namespace ab
