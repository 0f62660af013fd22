/*
 * adam_b200.h -- C ABI of libadam_b200.so, a CUDA (sm_100a) backend for ADAM's
 * quantized decode path.
 *
 * Part 1 keeps the symbol names, argument order and status codes of the
 * reference's native backend (adamah-MAIN/adamah/adamah.c) for the operators on
 * the decode path, so the reference's ctypes binding
 * (adamah-MAIN/adamah/__init__.py:_setup_ctypes, :527-1103) resolves them
 * unchanged.  Every declaration cites the reference definition it replaces.
 *
 * Part 2 holds additive extensions (prefix adam_b200_ or a new map_ name): maps
 * that keep weights as native GGUF blocks, and a fused decoder that runs a whole
 * token as one CUDA graph.
 *
 * Conventions (same as the reference): one global context per process, calls
 * come from one thread; a "map" is a flat typed device array addressed by
 * element (pack) index; a "loc handle" is the id of a small device array of
 * uint32 element indices (or of raw float data); functions returning int give 0
 * on success and a negative ADAMAH_ERR_* code otherwise; host buffers are read
 * or written before the call returns and stay owned by the caller.
 * All pointers are host pointers unless a parameter says otherwise.
 */
#ifndef ADAM_B200_H
#define ADAM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes: adamah.c:23-28 --------------------------------------- */
#define ADAMAH_OK             0
#define ADAMAH_ERR_BACKEND   -1   /* reference name: ADAMAH_ERR_VULKAN */
#define ADAMAH_ERR_MEMORY    -2
#define ADAMAH_ERR_INVALID   -3
#define ADAMAH_ERR_NOT_FOUND -4

/* ---- map element types: adamah.c:2698-2824 (DTYPE_*) ---------------------- */
#define ADAMAH_DTYPE_F32       0
#define ADAMAH_DTYPE_Q4        3    /* nibbles, 8 per uint32, + f32 (scale,zero) per group */
#define ADAMAH_DTYPE_GGUF_Q4_0 16   /* extension: 18-byte GGUF blocks of 32 */
#define ADAMAH_DTYPE_GGUF_Q4_K 17   /* extension: 144-byte GGUF superblocks of 256 */
#define ADAMAH_DTYPE_GGUF_Q8_0 18   /* extension: 34-byte GGUF blocks of 32 (int8 codes) */
#define ADAMAH_DTYPE_GGUF_Q5_0 19   /* extension: 22-byte GGUF blocks of 32 (5-bit codes) */

/* ======================= Part 1: reference-compatible ====================== */

/* context: adamah.c:2503 adamah_init, :1975 adamah_init_ex, :2596, :1820 */
int      adamah_init(void);
int      adamah_init_ex(uint64_t hot_pool_bytes, uint64_t cold_pool_bytes);
void     adamah_shutdown(void);
void     adamah_sync(void);
void     adamah_synchronize(uint64_t ticket);          /* adamah.c: adamah_synchronize */
void     adamah_synchronize_all(void);

/* active dtype for map_init: adamah.c:4585, :4614 */
int      adamah_set_dtype(uint32_t dtype);
uint32_t adamah_get_dtype(void);

/* maps: adamah.c:2686 map_init, :2698 map_init_dtype, :2826 map_destroy, map_size */
int      map_init(uint32_t id, uint32_t word_size, uint32_t pack_size, uint32_t n_packs);
int      map_init_dtype(uint32_t id, uint32_t dtype, uint32_t pack_size, uint32_t n_packs, uint32_t group_size);
int      map_destroy(uint32_t id);
uint32_t map_size(uint32_t id);
uint32_t map_get_dtype(uint32_t id);
/* adamah.c:4621 -- per-group (scale, zero) of a Q4 map */
int      map_set_qparams(uint32_t id, const float* scales, const float* zeros, uint32_t n_groups);

/* host <-> map: adamah.c:3087, :2896, :3035, :3374 */
int      map_scatter(uint32_t id, const uint32_t* locs, const void* data, uint32_t n_locs);
int      map_scatter_contiguous(uint32_t id, uint32_t start_pack, const void* data, uint32_t n_locs);
int      map_scatter_q4_packed_contiguous(uint32_t id, uint32_t start_pack, const void* packed_u8, uint32_t n_locs);
int      map_gather(uint32_t id, const uint32_t* locs, void* out, uint32_t n_locs);

/* loc handles: adamah.c:3570 map_upload_dev (returns handle | ticket<<32, 0 on
 * failure; handle 0 creates, otherwise overwrites in place, same size), :3665 */
uint64_t map_upload_dev(uint32_t handle_or_0, const void* data, uint32_t n_bytes);
int      map_download_dev(uint32_t handle, void* out, uint32_t n_bytes);
/* adamah.c:3788, :3703 -- device-side gather into a new data handle / scatter from one */
uint64_t map_gather_dev(uint32_t id, uint32_t locs_handle, uint32_t n_locs);
uint64_t map_scatter_dev(uint32_t id, uint32_t locs_handle, uint32_t n_locs, uint32_t src_handle);

/* batching: adamah.c:1629, :1647 -- results are host-visible after batch_end */
void     batch_begin(void);
void     batch_end(void);

/* fusion scheduler: adamah.c:4670, :4677, :5653, :708, :718, :675, :691.
 * A CUDA stream already runs ops in program order, so these keep state and
 * counters only. */
void     adamah_fusion_enable(int enable);
int      adamah_fusion_is_enabled(void);
int      adamah_fusion_flush(void);
void     adamah_fusion_set_scheduler_mode(int mode);
int      adamah_fusion_get_scheduler_mode(void);
int      adamah_register_loc_span(uint32_t handle, uint32_t map_id, uint32_t start, uint32_t count);
int      adamah_register_row_base_span(uint32_t handle, uint32_t map_id, uint32_t start, uint32_t count,
                                       uint32_t stride, uint32_t row_size);
int      adamah_clear_loc_alias_meta(uint32_t handle);

/* counters: adamah.c:316, :321 (nine uint64 outputs, any may be NULL) */
void     adamah_stats_reset(void);
void     adamah_stats_get(uint64_t* dispatch_count, uint64_t* submit_count, uint64_t* barrier_count,
                          uint64_t* fusion_flush_count, uint64_t* descriptor_set_update_count,
                          uint64_t* descriptor_cache_hit_count, uint64_t* descriptor_cache_miss_count,
                          uint64_t* alias_conflict_count, uint64_t* scheduler_mode);

/* ---- operators on the decode path ---------------------------------------- */
/* adamah.c:7687, :8459, :7786 */
int map_rmsnorm_dev(uint32_t map, uint32_t src_h, uint32_t wt_h, uint32_t dst_h, uint32_t n_rows, uint32_t dim, float eps);
int map_rmsnorm_x_dev(uint32_t map_act, uint32_t map_wt, uint32_t src_h, uint32_t wt_h, uint32_t dst_h,
                      uint32_t n_rows, uint32_t dim, float eps);
int map_rmsnorm_add_dev(uint32_t map, uint32_t src_h, uint32_t wt_h, uint32_t resid_h, uint32_t dst_h,
                        uint32_t n_rows, uint32_t dim, float eps);
/* adamah.c:7879, :8586 */
int map_rope_dev(uint32_t map, uint32_t src_h, uint32_t dst_h, uint32_t n_tokens, uint32_t n_heads,
                 uint32_t head_dim, uint32_t pos_offset, float freq_base);
int map_qk_norm_rope_x_dev(uint32_t map_act, uint32_t map_wt, uint32_t qsrc_h, uint32_t qwt_h,
                           uint32_t ksrc_h, uint32_t kwt_h, uint32_t qkdst_h,
                           uint32_t q_rows, uint32_t q_dim, uint32_t k_rows, uint32_t k_dim,
                           uint32_t pos_offset, float freq_base);
/* adamah.c:8061 (and map_row_copy_dev) -- KV append */
int map_row_copy_dev(uint32_t map, uint32_t spec_h, uint32_t src_base_h, uint32_t n_copies, uint32_t row_size);
int map_row_copy_offset_dev(uint32_t map, uint32_t spec_h, uint32_t src_base_h, uint32_t dst_row_offset,
                            uint32_t n_copies, uint32_t row_size);
/* adamah.c:7894 -- C[M,N] = A[M,K] * B[N,K]^T, n_ops independent problems */
int map_matmul_t_dev(uint32_t map, uint32_t a_h, uint32_t b_h, uint32_t c_h,
                     uint32_t M, uint32_t K, uint32_t N, uint32_t n_ops);
/* adamah.c:8693 -- activations in map_act (f32), weights in map_wt (Q4 map or GGUF blocks) */
int map_matmul_t_xq4_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t c_h,
                         uint32_t M, uint32_t K, uint32_t N, uint32_t n_ops);
/* adamah.c:6768 */
int map_attn_softmax_value_dev(uint32_t map, uint32_t scores_h, uint32_t values_h, uint32_t out_h,
                               uint32_t n_ops, uint32_t row_size, uint32_t value_dim, float scale, float cap);
/* adamah.c:5923, :6029, :6398 */
int map_op1_dev(uint32_t map, uint32_t op, uint32_t src_h, uint32_t dst_h, uint32_t n);
int map_op2_dev(uint32_t map, uint32_t op, uint32_t a_h, uint32_t b_h, uint32_t dst_h, uint32_t n);
int map_broadcast_dev(uint32_t map, uint32_t op, uint32_t src_h, uint32_t scalar_h, uint32_t dst_h, uint32_t n);
/* adamah.c:6875, :7210, :9699 */
int map_argmax_dev(uint32_t map, uint32_t src_h, uint32_t dst_h, uint32_t n);
int map_resolve_idx_dev(uint32_t map, uint32_t base_h, uint32_t sel_h, uint32_t dst_h, uint32_t n);
/* Sampled-decoding tail (adamah.c:6978 map_topk_dev, :7095 map_topp_dev, :7286
 * map_sample_categorical_dev, :6787 map_repeat_penalty_dev): the k <= 64 largest values and their
 * indices (ties to the lower index), soft-max with temperature + nucleus cut over <= 64 sorted
 * candidates, inverse-CDF draw from a uniform number stored in the map, and the repeat penalty on
 * listed token ids (raw uint32 ids, not locs).  Indices travel as float32, like everything else. */
int map_topk_dev(uint32_t map, uint32_t src_h, uint32_t idx_dst_h, uint32_t val_dst_h, uint32_t n, uint32_t k);
int map_topp_dev(uint32_t map, uint32_t src_h, uint32_t dst_h, uint32_t n, float temperature, float top_p);
int map_sample_categorical_dev(uint32_t map, uint32_t idx_h, uint32_t prob_h, uint32_t rand_h, uint32_t dst_h, uint32_t n);
int map_repeat_penalty_dev(uint32_t map, uint32_t src_h, uint32_t token_ids_h, uint32_t n_ids, float penalty);
/* adamah.c:9727-9832: per group of rows_per_group rows the k (<= 64) largest W[n,:] . x after the repeat
 * penalty, (row as float32, value) at locs_idx_dst / locs_val_dst [group * k + r]; _dev uses 256 rows. */
int map_matvec_topk_t_xq4_ex_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t penalty_ids_h,
                                 uint32_t idx_dst_h, uint32_t val_dst_h, uint32_t K, uint32_t N, uint32_t k,
                                 uint32_t n_penalty, float repeat_penalty, uint32_t rows_per_group);
int map_matvec_topk_t_xq4_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t penalty_ids_h,
                              uint32_t idx_dst_h, uint32_t val_dst_h, uint32_t K, uint32_t N, uint32_t k,
                              uint32_t n_penalty, float repeat_penalty);
int map_matvec_argmax_t_xq4_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h,
                                uint32_t idx_tmp_h, uint32_t val_tmp_h, uint32_t dst_h,
                                uint32_t K, uint32_t N, uint32_t rows_per_group);

/* 8-bit weight operators: adamah.c:9834 (map_matmul_t_xq8_dev), :10189 (map_row_gather_xq8_dev).  The weight map is a
 * GGUF-block map of Q8_0 or Q5_0 blocks (ADAMAH_DTYPE_GGUF_Q8_0 / _Q5_0) instead of the reference's byte map with a
 * (scale, zero) pair per 32.  map_matmul_t_xq8_dev: C[M,N] = A[M,K] * W[N,K]^T.  map_row_gather_xq8_dev: the row
 * row_idx of length row_size starting at element src_base of the weight map, decoded and multiplied by scale, to
 * element dst_base of the activation map (bases and row index are immediates). */
int map_matmul_t_xq8_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h, uint32_t c_h,
                         uint32_t M, uint32_t K, uint32_t N, uint32_t n_ops);
int map_row_gather_xq8_dev(uint32_t map_act, uint32_t map_wt, uint32_t src_base, uint32_t dst_base,
                           uint32_t row_idx, uint32_t row_size, float scale);

/* decode plan: adamah.c:175-194 (struct), :10341, :10367, :10361 */
typedef struct AdamahDecodePlanOp {
    uint32_t kind, map_id, map_id2, op_code;
    uint32_t h0, h1, h2, h3, h4, h5;
    uint32_t u0, u1, u2, u3, u4, u5;
    float    f0, f1;
} AdamahDecodePlanOp;
#define ADAMAH_DECODE_RUNTIME_POS     0xFFFFFFFEu
#define ADAMAH_DECODE_RUNTIME_SEQ_LEN 0xFFFFFFFDu
int  adamah_register_decode_plan(uint32_t plan_id, const AdamahDecodePlanOp* ops, uint32_t n_ops);
int  adamah_decode_step(uint32_t plan_id, uint32_t pos, uint32_t seq_len);
void adamah_clear_decode_plan(uint32_t plan_id);
/* How a registered plan runs (extension).  From its second step on a plan is one CUDA graph in which the run-time
 * arguments stay symbolic (kernels read pos / seq_len from device words set by a one-thread kernel before each graph
 * launch).  out[0..5] = state (2 = graph, -1 = host-side substitution as in the reference, 0 / 1 = not recorded yet),
 * positions the graph is sized for, kernels in the graph, times recorded, steps run as a graph, steps run by host
 * substitution. */
int  adam_b200_decode_plan_info(uint32_t plan_id, uint32_t* out);

/* Symbols the reference binding resolves without a guard but which lie off the
 * decode path (generic tensor ops, untransposed 8-bit products).  They exist so the binding
 * loads, and return ADAMAH_ERR_INVALID.  adamah-MAIN/adamah/__init__.py:530-960. */
int map_op1(uint32_t, uint32_t, const uint32_t*, const uint32_t*, uint32_t);
int map_op2(uint32_t, uint32_t, const uint32_t*, const uint32_t*, const uint32_t*, uint32_t);
int map_matmul(uint32_t, const uint32_t*, const uint32_t*, const uint32_t*, uint32_t, uint32_t, uint32_t, uint32_t);
int map_softmax(uint32_t, const uint32_t*, const uint32_t*, uint32_t, uint32_t);
int map_layernorm(uint32_t, const uint32_t*, const uint32_t*, const uint32_t*, const uint32_t*, uint32_t, uint32_t, float);
int map_broadcast(uint32_t, uint32_t, const uint32_t*, const uint32_t*, const uint32_t*, uint32_t);
int map_reduce(uint32_t, uint32_t, const uint32_t*, const uint32_t*, uint32_t);
int map_matmul_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_softmax_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_softmax_abs_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_attn_softmax_abs_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, float, float);
int map_layernorm_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, float);
int map_reduce_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_fma_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_matmul_t_x_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_matmul_x_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_matmul_xq4_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);
int map_matmul_xq8_dev(uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t);

/* ============================ Part 2: extensions =========================== */

/* Human-readable text for the last failure of any call (never NULL). */
const char* adam_b200_last_error(void);
/* Device ordinal in use, SM count, and library build tag. */
int         adam_b200_device_info(int* device, int* sm_count, uint64_t* total_mem_bytes);
/* Number of kernel launches (graph nodes count individually) since the last
 * adamah_stats_reset; also reported as dispatch_count by adamah_stats_get. */
uint64_t    adam_b200_kernel_launches(void);

/* Reads and clears the device error word: bit 0 = a loc fell outside its map,
 * bit 1 = a bounded device-side wait ran out, bit 2 = token id out of range.
 * Kernels record these instead of faulting. */
uint32_t    adam_b200_device_error(void);
/* Free a loc handle (the reference evicts instead: adamah.c:1328 res_evict_one). */
int         adam_b200_handle_free(uint32_t handle);

/* CUDA-event timer around work on the context stream. */
int adam_b200_timer_begin(void);
int adam_b200_timer_end(float* ms);
/* Record the operator calls made between begin and end into a CUDA graph (no
 * host I/O in between), then replay it `times` times with one launch each.
 * CUDA counterpart of batching many dispatches into one command buffer
 * (adamah.c:1629-1721). */
int adam_b200_capture_begin(void);
int adam_b200_capture_end(uint32_t* graph_id);
int adam_b200_graph_launch(uint32_t graph_id, uint32_t times);
int adam_b200_graph_destroy(uint32_t graph_id);

/* Copy raw GGUF blocks (ggml_type 2 = Q4_0, 12 = Q4_K, 8 = Q8_0, 6 = Q5_0) into a GGUF-block map of the matching dtype at
 * element offset elem_off (a multiple of the block size).  `raw` may be a host
 * or a device pointer.  Replaces the reference's Python re-quantization at load
 * (adam/models/engine.py:974-1116); op signatures are unchanged -- weight handles
 * still carry element offsets. */
int map_upload_gguf_blocks(uint32_t map_wt, uint32_t ggml_type, uint64_t elem_off, const void* raw, uint64_t n_bytes);
/* The same placement with the blocks read from a file: n_bytes starting at file_offset of `path` (a tensor's
 * data inside a .gguf file) stream through two pinned 32 MB buffers, one cudaMemcpyAsync per chunk, the read of
 * the next chunk overlapping the copy of the current one.  Replaces adam/loaders/gguf.py:196-253
 * (load_tensor_raw / iter_tensor_chunks) + the upload loops of adam/models/engine.py:929-1116. */
int adam_b200_upload_gguf_file(uint32_t map_wt, uint32_t ggml_type, uint64_t elem_off, const char* path,
                               uint64_t file_offset, uint64_t n_bytes);
/* Build and register a row-tiled copy of the [rows, cols] Q4_0 tensor at elem_off of a
 * GGUF Q4_0 map (rows % 16 == 0, cols % 64 == 0).  Later GEMV / arg-max calls on exactly
 * that tensor run the tensor-core kernel on the copy; results stay within the same
 * tolerance.  Costs one extra copy of the tensor's bytes; freed with the map. */
int adam_b200_tensor_tile(uint32_t map_wt, uint64_t elem_off, uint32_t rows, uint32_t cols);
/* Decode n_elems weights starting at elem_off of a GGUF-block or Q4 map to
 * float32 (host pointer `out`); bit-exact w.r.t. adam/loaders/gguf.py:282-337. */
int map_dequant_gguf(uint32_t map_wt, uint64_t elem_off, float* out, uint64_t n_elems);
/* Quantize float32 rows (device pointer, n_elems multiple of 32) to raw Q4_0
 * blocks (device pointer) with the ggml rule; load-time helper for synthetic
 * models (role of adamah-MAIN/adamah/shaders/src/q4/map_scatter.comp). */
int adam_b200_quantize_q4_0_dev(const float* w_dev, uint64_t n_elems, void* raw_dev);

/* LM head + arg-max that allocates nothing (no counterpart in the reference, whose
 * callers always hand in their own partial buffers).  Same arguments and result as
 * map_matvec_argmax_t_xq4_dev, for callers that must not trigger cudaMalloc when they
 * call in (a serving loop that owns the card's memory through its own pool, a
 * latency-critical section that cannot afford the device-wide synchronisation an
 * allocation implies, a process already at its memory cap).  The partial-result
 * scratch is a fixed array inside the library image: about 32 KB of device memory on
 * every GPU on which the library is initialised, from adamah_init until the process exits.  Limit: N may not exceed
 * 4096 * rows_per_group rows (rows_per_group 0 -> 256, i.e. 1,048,576 rows); larger N
 * returns ADAMAH_ERR_INVALID.  All calls share that one array and it keeps the last
 * call's contents (the arrival counter is cleared before every launch): calls that
 * overlap on the GPU race, so issue them from one thread on the library's stream.  The
 * array's device address is looked up once per device by adamah_init (adam_b200_noalloc_prepare);
 * without that, by the first call of the entry point, which should then come before any
 * stream capture. */
int adam_b200_noalloc_prepare(void);
int map_matvec_argmax_t_xq4_static_dev(uint32_t map_act, uint32_t map_wt, uint32_t a_h, uint32_t b_h,
                                       uint32_t idx_tmp_h, uint32_t val_tmp_h, uint32_t dst_h,
                                       uint32_t K, uint32_t N, uint32_t rows_per_group);

/* Enqueue everything on a CUDA stream the caller owns (a cudaStream_t passed as an
 * integer; 0 = back to the library's own stream), so the caller's collectives or kernels on
 * that stream are ordered with the library's.  Synchronises the stream in use first. */
int adam_b200_set_stream(uint64_t stream);

/* ---- one-shot all-reduce over peer memory (tensor-parallel decode) -----------------
 * Sum of a small fp32 buffer over 2..8 ranks (one process per GPU of one node): every rank
 * stages its values in its own memory, raises a flag in every peer's memory and, once all
 * flags of the call are up (bounded wait: bit value 2 of adam_b200_device_error on expiry,
 * the kernel still ends), adds the peers' staged values in rank order.  ar_create returns
 * this rank's two 64-byte CUDA IPC handles; the caller gathers all ranks' (world x 128 bytes,
 * rank order), passes them to ar_open and synchronises the ranks once before the first
 * all-reduce.  All ranks issue the same sequence of calls with the same sizes.  No counterpart
 * in the reference (it has no multi-GPU path). */
int adam_b200_ar_create(uint32_t world, uint32_t rank, uint64_t max_bytes, uint32_t* id_out, void* handles_out);
int adam_b200_ar_open(uint32_t id, const void* all_handles);
int adam_b200_ar_allreduce(uint32_t id, uint64_t buf, uint32_t n_floats);     /* in place, on the library stream */
int adam_b200_ar_destroy(uint32_t id);
/* Bound of one all-reduce call's wait in microseconds (about 5 s by default; env ADAM_B200_AR_WAIT_US). */
int adam_b200_ar_set_wait_us(uint32_t id, uint64_t wait_us);
/* Clears the sticky "a wait ran out" word (every rank, followed by a host barrier); _timed_out reads it. */
int adam_b200_ar_reset(uint32_t id);
int adam_b200_ar_timed_out(uint32_t id);
/* Test set-up: connect communicators of this process (ids[q] plays rank q) by pointer instead of IPC. */
int adam_b200_ar_open_local(uint32_t id, const uint32_t* ids, uint32_t n);

/* ---- fused decoder ------------------------------------------------------------
 * Runs the reference engine's per-token loop (adam/models/engine.py:2971-3706
 * `_forward`, generate loop :3810-3944) for a batch of sequences as one CUDA
 * graph per token.  Weights stay in GGUF-block maps and norm weights in a
 * float32 map; the decoder keeps pointers into them.  Extensions over the
 * reference: batch > 1, paged fp16/fp32 KV cache, optional sliding-window mask. */
typedef struct adam_b200_decoder_desc {
    uint32_t n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab;
    uint32_t ffn_act;            /* 0 = GeGLU (gelu), 1 = SwiGLU (silu) */
    float    norm_eps, emb_scale, attn_softcap, final_softcap;
    float    attn_scale;         /* 0 -> 1/sqrt(head_dim) */
    uint32_t sliding_window;     /* tokens; used on non-global layers when flags bit 0 is set */
    uint32_t global_every;       /* layer L is global when (L+1) % global_every == 0; 0 = all global */
    uint32_t max_batch, kv_cap;
    uint32_t kv_dtype;           /* 0 = float32, 1 = float16 */
    uint32_t page_size;          /* tokens per KV page (0 -> 64) */
    uint32_t n_pages;            /* 0 -> max_batch * ceil(kv_cap / page_size) */
    uint32_t tp_rank, tp_size;   /* tensor-parallel shard (1 = whole model) */
    uint32_t flags;              /* bit 0: apply the sliding-window mask; bit 1: no row-tiled weight copies */
} adam_b200_decoder_desc;

int adam_b200_decoder_create(const adam_b200_decoder_desc* desc, uint32_t* id_out);
int adam_b200_decoder_destroy(uint32_t id);
/* kind: 0 attn_q, 1 attn_k, 2 attn_v, 3 attn_output, 4 ffn_gate, 5 ffn_up, 6 ffn_down,
 * 7 token_embd, 8 output (LM head; token_embd is used when unbound). */
int adam_b200_decoder_bind_matrix(uint32_t id, uint32_t layer, uint32_t kind, uint32_t map_wt, uint64_t elem_off,
                                  uint32_t rows, uint32_t cols);
/* kind: 0 attn_norm, 1 post_attention_norm, 2 ffn_norm, 3 post_ffw_norm, 4 attn_q_norm,
 * 5 attn_k_norm, 6 output_norm. */
int adam_b200_decoder_bind_norm(uint32_t id, uint32_t layer, uint32_t kind, uint32_t map_f32, uint64_t elem_off, uint32_t n);
/* cos/sin of the rotary angles, [n_pos][half] float32, which: 0 = local layers, 1 = global layers. */
int adam_b200_decoder_set_rope(uint32_t id, uint32_t which, const float* cos_t, const float* sin_t, uint32_t n_pos, uint32_t half);
/* Start `batch` sequences from position 0.  prompt_tokens holds the prompts back to
 * back; reserve[b] >= prompt_lens[b] tokens of KV pages are set aside per sequence. */
int adam_b200_decoder_begin(uint32_t id, uint32_t batch, const int32_t* prompt_tokens, const uint32_t* prompt_lens,
                            const uint32_t* reserve);
/* n_steps token steps.  flags: bit 0 LM head + arg-max, bit 1 also store logits,
 * bit 2 launch kernels directly (no graph replay). */
int adam_b200_decoder_step(uint32_t id, uint32_t n_steps, uint32_t flags);
/* Asynchronous read of the current token ids: tokens_async queues a copy into one of four pinned
 * slots behind the work issued so far; tokens_wait blocks only until that copy has landed, so the
 * caller can keep the next step queued while it inspects the last ids ([batch] values). */
int adam_b200_decoder_tokens_async(uint32_t id, uint32_t* slot_out);
int adam_b200_decoder_tokens_wait(uint32_t id, uint32_t slot, int32_t* out);
/* Replace the current token of every active sequence ([batch] host ids): for callers that sample on
 * the host from the logits of the last step (the reference's 'cpu' sampling mode, engine.py:3711-3729). */
int adam_b200_decoder_set_tokens(uint32_t id, const int32_t* tokens);
/* Continue the single active sequence with a new prompt whose first n_reuse tokens are already in
 * the cache (generate(reuse_prefix=..), adam/models/engine.py:3815-3833): positions restart at
 * n_reuse (which must not exceed the positions computed so far), pages are kept and extended. */
int adam_b200_decoder_continue(uint32_t id, const int32_t* prompt_tokens, uint32_t prompt_len, uint32_t reserve, uint32_t n_reuse);
/* Chunked prefill: consume the next n_tokens prompt tokens of every active sequence, up to 64
 * rows (sequences x tokens) per pass through the layers; same results as n_tokens steps without
 * the LM head.  Every sequence must still have n_tokens prompt tokens ahead.  The reference
 * consumes prompts token by token (adam/models/engine.py:3838-3847). */
int adam_b200_decoder_prefill(uint32_t id, uint32_t n_tokens);
/* The same step in parts, each enqueued directly on the stream, for callers that put their
 * own work between them (tensor parallelism).  Parts 2L / 2L+1 = attention half (embedding
 * for L = 0, QKV, attention, o-proj) / FFN half (gate+up, down) of layer L; then the LM head
 * (flags bit 0) and the position update.  After each layer part the projection buffer holds
 * this shard's partial sums.  No counterpart in the reference (it has no multi-GPU path). */
int adam_b200_decoder_n_parts(uint32_t id);                                   /* 2*n_layer + 2, or a negative status */
int adam_b200_decoder_step_part(uint32_t id, uint32_t part, uint32_t flags);
/* Number of matrix products enqueued so far on the tcgen05 (tensor memory) GEMM, which takes calls
 * with 9..64 activation rows; calls with fewer rows run on the GEMV kernels. */
uint64_t adam_b200_tc_gemm_count(void);
/* Which calls take it: 0 = none, 1 = those expected to be faster than the GEMV kernels (default; also the
 * initial value of environment variable ADAM_B200_TC), 2 = every call whose shape allows. */
int adam_b200_tc_gemm_policy(int policy);
/* One part of one prefill chunk of n_tokens (batch * n_tokens <= 64 rows) tokens per sequence: parts
 * 0 .. 2*n_layer-1 as above (the projection buffer then holds batch * n_tokens rows of partial
 * sums), part 2*n_layer advances the positions by n_tokens. */
int adam_b200_decoder_prefill_part(uint32_t id, uint32_t n_tokens, uint32_t part);
/* Diagnostics of the single-launch token kernel (one active sequence; no counterpart in the reference): runs
 * one token step with the LM head and returns every CTA's SM clock at 32 points: slots 0..9 phases of layer
 * (layer & 0xFFFF), 10..13 LM head, 16..22 inside product (layer >> 16) of that layer; out[cta * 32 + slot],
 * out holds 32 * 256 values. */
int adam_b200_decoder_token_trace(uint32_t id, uint32_t layer, long long* out, uint32_t* n_cta_out);
/* Diagnostics of the default one-sequence step (the CUDA graph of per-operation kernels; no counterpart in the
 * reference).  Only a library built with -DADAM_B200_STEP_TRACE (`python -m adam_b200.build --step-trace`) records
 * anything; the regular build returns ADAMAH_ERR_INVALID.  out == NULL arms the trace for `layer`; after some steps a
 * call with out (512 values) returns the stamps of the latest step in nanoseconds of the GPU's global timer:
 *   out[(p * 8 + cta) * 8 + slot], p = 0 QKV, 1 o-proj, 2 gate/up, 3 down, cta = 0..7, slots: 0 kernel start,
 *     1 prologue done (weight copies requested), 2 dependency wait over, 3 input staged, 4 products done;
 *   out[256 + cta * 8 + slot], attention CTAs 0..31, slots: 0 start, 1 cached rows requested, 2 wait over, 3 query /
 *     key rows normed and rotated, 4 positions done, 5 partial result stored, 6 ticket taken, 7 splits merged (last CTA). */
int adam_b200_decoder_step_trace(uint32_t id, uint32_t layer, long long* out, uint32_t n_words);
/* Test hook for the bounded device-side waits (no counterpart in the reference): launches one token step of the
 * single active sequence on the token kernel with its last CTA left out and every wait limited to wait_us
 * microseconds; the waits run out, the kernel records error bit 2 (adam_b200_device_error), sets the decoder's
 * sticky word and returns.  Later steps return at once until decoder_begin / decoder_continue. */
int adam_b200_decoder_test_wait_expiry(uint32_t id, uint32_t wait_us);
/* Sampling on the device (role of GenerationConfig + ADAMEngine._sample, adam/models/engine.py:24-29, :3711-3729):
 * steps with flag bit4 (16) replace the arg-max token by a draw -- repeat penalty on the last 64 history ids,
 * temperature, top_k (1..64), soft-max, nucleus top_p, counter-based generator keyed by (seed, sequence, position). */
int adam_b200_decoder_set_sampling(uint32_t id, uint32_t top_k, float top_p, float temperature, float repeat_penalty,
                                   uint32_t repeat_on_prompt, uint64_t seed);
/* Device address / size of a decoder buffer: 0 projection output [batch][n_embd] f32,
 * 1 current token ids [max_batch] i32, 2 their logit values [max_batch] f32, 3 positions. */
int adam_b200_decoder_buffer_ptr(uint32_t id, uint32_t which, uint64_t* ptr_out, uint64_t* bytes_out);
int adam_b200_decoder_read_state(uint32_t id, int32_t* pos_out, int32_t* cur_tok_out);   /* [max_batch] each, may be NULL */
int adam_b200_decoder_read_log(uint32_t id, uint32_t seq, uint32_t first_pos, uint32_t n, int32_t* out);
int adam_b200_decoder_read_logits(uint32_t id, uint32_t seq, float* out);                 /* [n_vocab] */
int adam_b200_decoder_read_buffer(uint32_t id, uint32_t what, uint32_t seq, float* out, uint32_t n);

#ifdef __cplusplus
}
#endif
#endif /* ADAM_B200_H */
