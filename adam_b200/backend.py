"""The backend object: same method names, argument meaning and error behaviour as
the reference's ``Adamah`` class (adamah-MAIN/adamah/__init__.py:478-2900) for
the operators on the decode path.  Every method is one call into
``libadam_b200.so`` and raises ``RuntimeError("<fn> failed with code N: ...")`` on a
non-zero status, as the reference binding does (e.g. __init__.py:1816-1817).
"""
from __future__ import annotations

import contextlib
import ctypes
import os
from typing import Dict, Optional

import numpy as np

from . import _lib
from ._lib import DecodePlanOp  # noqa: F401  (re-exported)
from . import constants as C

_SCHED_NAMES = {0: "legacy", 1: "alias_safe", 2: "level_batched"}


def _unpack(v: int):
    """``handle | ticket << 32`` -> (handle, ticket) (__init__.py:150-153)."""
    return int(v & 0xFFFFFFFF), int(v >> 32)


class Adamah:
    def __init__(self, lib_path: Optional[str] = None, cache_mb: Optional[int] = None, cold_cache_mb: Optional[int] = None):
        self._lib = _lib.load()
        rc = self._lib.adamah_init_ex(int(cache_mb or 0) << 20, int(cold_cache_mb or 0) << 20)
        if rc != 0:
            raise RuntimeError(f"adamah_init failed with code {rc}: {_lib.last_error()}")
        self._maps: Dict[int, tuple] = {}
        self._active_dtype = C.DTYPE_F32
        self._group_size = 32
        self._metrics = {"scatter_calls": 0, "gather_calls": 0, "total_bytes_cpu_to_gpu": 0, "total_bytes_gpu_to_cpu": 0}
        self._closed = False
        # feature flags consulted with getattr(gpu, '_has_x', False) (engine.py:1865-1973)
        self._has_dtype = True
        self._has_native_stats = True
        self._has_decode_plan = True
        self._has_map_scatter_contiguous = True
        self._has_map_scatter_q4_packed_contiguous = True
        self._has_map_matvec_argmax_t_xq4_dev = True
        self._has_map_matvec_topk_t_xq4_dev = True
        self._has_map_matvec_topk_t_xq4_ex_dev = True
        self._has_map_resolve_idx_dev = True
        self._has_map_sample_categorical_dev = True
        self._has_map_repeat_penalty_dev = True
        self._has_map_upload_gguf_blocks = True
        self._has_decoder = True
        self._is_integrated_gpu = False
        dev, sms, mem = ctypes.c_int(), ctypes.c_int(), ctypes.c_uint64()
        self._lib.adam_b200_device_info(ctypes.byref(dev), ctypes.byref(sms), ctypes.byref(mem))
        self.device_index, self.sm_count, self.total_mem = dev.value, sms.value, mem.value

    # ---- helpers -------------------------------------------------------------
    def _check(self, rc: int, name: str):
        if rc != 0:
            raise RuntimeError(f"{name} failed with code {rc}: {_lib.last_error()}")

    @staticmethod
    def _ptr(a: np.ndarray):
        return a.ctypes.data_as(ctypes.c_void_p)

    # ---- dtype / maps ----------------------------------------------------------
    def set_dtype(self, dtype: int, group_size: int = 128):
        rc = self._lib.adamah_set_dtype(dtype)
        if rc != 0:
            raise RuntimeError(f"Failed to set dtype {dtype} (code {rc}): {_lib.last_error()}")
        self._active_dtype = dtype
        self._group_size = group_size

    def get_dtype(self) -> int:
        return int(self._lib.adamah_get_dtype())

    def map_create_typed(self, map_id: int, dtype: int, pack_size: int, n_packs: int, group_size: int = 128):
        rc = self._lib.map_init_dtype(map_id, dtype, pack_size, n_packs, group_size)
        if rc != 0:
            raise RuntimeError(f"map_init_dtype({dtype}) failed: {rc}: {_lib.last_error()}")
        self._maps[map_id] = (4 if dtype == C.DTYPE_F32 else 1, pack_size, n_packs, dtype)

    def map_create(self, map_id: int, pack_size: int = 0, n_packs: int = 0, word_size: int = 0, **kw):
        self.map_create_typed(map_id, self._active_dtype, pack_size, n_packs, self._group_size)

    def map_init(self, map_id: int, word_size: int, pack_size: int, n_packs: int):
        return self.map_create(map_id, pack_size=pack_size, n_packs=n_packs, word_size=word_size)

    def map_destroy(self, map_id: int):
        self._check(self._lib.map_destroy(map_id), "map_destroy")
        self._maps.pop(map_id, None)

    def map_size(self, map_id: int) -> int:
        return int(self._lib.map_size(map_id))

    def set_qparams(self, map_id: int, scales: np.ndarray, zero_points: np.ndarray):
        s = np.ascontiguousarray(scales, dtype=np.float32)
        z = np.ascontiguousarray(zero_points, dtype=np.float32)
        self._check(self._lib.map_set_qparams(map_id, self._ptr(s), self._ptr(z), len(s)), "map_set_qparams")

    # ---- host <-> map ----------------------------------------------------------
    @staticmethod
    def _words(data) -> np.ndarray:
        a = np.ascontiguousarray(data)
        if a.dtype.itemsize != 4:
            a = a.astype(np.float32)
        return a

    def scatter(self, map_id: int, locs: np.ndarray, data: np.ndarray) -> int:
        locs = np.ascontiguousarray(locs, dtype=np.uint32)
        a = self._words(data)
        self._metrics["scatter_calls"] += 1
        self._metrics["total_bytes_cpu_to_gpu"] += a.nbytes
        self._check(self._lib.map_scatter(map_id, self._ptr(locs), self._ptr(a), len(locs)), "map_scatter")
        return 0

    map_scatter = scatter

    def scatter_contiguous(self, map_id: int, start_pack: int, data: np.ndarray, n_locs: Optional[int] = None) -> int:
        a = self._words(data)
        if n_locs is None:
            n_locs = int(a.size)
        self._metrics["scatter_calls"] += 1
        self._metrics["total_bytes_cpu_to_gpu"] += a.nbytes
        self._check(self._lib.map_scatter_contiguous(map_id, start_pack, self._ptr(a), n_locs), "map_scatter_contiguous")
        return 0

    map_scatter_contiguous = scatter_contiguous

    def scatter_q4_packed_contiguous(self, map_id: int, start_pack: int, packed_u8: np.ndarray, n_locs: Optional[int] = None) -> int:
        a = np.ascontiguousarray(packed_u8, dtype=np.uint8)
        if n_locs is None:
            n_locs = int(a.size) * 2
        self._metrics["scatter_calls"] += 1
        self._metrics["total_bytes_cpu_to_gpu"] += a.nbytes
        self._check(self._lib.map_scatter_q4_packed_contiguous(map_id, start_pack, self._ptr(a), n_locs),
                    "map_scatter_q4_packed_contiguous")
        return 0

    map_scatter_q4_packed_contiguous = scatter_q4_packed_contiguous

    def gather(self, map_id: int, locs: np.ndarray, n_packs: Optional[int] = None, n_locs: Optional[int] = None) -> np.ndarray:
        """Raw 32-bit words (view as float32), like the reference (__init__.py:1347-1360)."""
        locs = np.ascontiguousarray(locs, dtype=np.uint32)
        n = n_locs if n_locs is not None else (n_packs if n_packs is not None else len(locs))
        pack = self._maps.get(map_id, (4, 1, 0, 0))[1]
        out = np.empty(n * pack, dtype=np.uint32)
        self._metrics["gather_calls"] += 1
        self._check(self._lib.map_gather(map_id, self._ptr(locs), self._ptr(out), n), "map_gather")
        self._metrics["total_bytes_gpu_to_cpu"] += out.nbytes
        return out

    map_gather = gather

    def upload_dev(self, data, handle: int = 0):
        """Host array -> device loc handle; returns (handle, ticket)."""
        a = np.ascontiguousarray(data)
        packed = int(self._lib.map_upload_dev(handle, self._ptr(a), a.nbytes))
        if packed == 0:
            raise RuntimeError(f"map_upload_dev failed: {_lib.last_error()}")
        return _unpack(packed)

    def download_dev(self, handle: int, n_elems: int, dtype=np.float32):
        out = np.empty(n_elems, dtype=dtype)
        self._check(self._lib.map_download_dev(handle, self._ptr(out), out.nbytes), "map_download_dev")
        return out

    def free_handle(self, handle: int):
        self._check(self._lib.adam_b200_handle_free(handle), "adam_b200_handle_free")

    def map_gather_dev(self, map_id: int, locs_handle: int, n_locs: int):
        if map_id not in self._maps:
            raise ValueError(f"Map {map_id} not initialized")
        pack = self._maps[map_id][1]
        packed = int(self._lib.map_gather_dev(map_id, locs_handle, n_locs))
        if packed == 0:
            raise RuntimeError(f"map_gather_dev failed: {_lib.last_error()}")
        h, t = _unpack(packed)
        return h, t, n_locs * pack, np.float32

    def map_scatter_dev(self, map_id: int, locs_handle: int, n_locs: int, src_handle: int):
        if map_id not in self._maps:
            raise ValueError(f"Map {map_id} not initialized")
        t = int(self._lib.map_scatter_dev(map_id, locs_handle, n_locs, src_handle))
        if t == 0:
            raise RuntimeError(f"map_scatter_dev failed: {_lib.last_error()}")
        return t

    def synchronize(self, ticket: int):
        self._lib.adamah_synchronize(ticket)

    def synchronize_all(self):
        self._lib.adamah_synchronize_all()

    def sync(self):
        self._lib.adamah_sync()

    # ---- operators ---------------------------------------------------------------
    def map_op1_dev(self, map_id, op, locs_in_handle, locs_out_handle, n):
        self._check(self._lib.map_op1_dev(map_id, op, locs_in_handle, locs_out_handle, n), "map_op1_dev")

    def map_op2_dev(self, map_id, op, locs_a_handle, locs_b_handle, locs_out_handle, n):
        self._check(self._lib.map_op2_dev(map_id, op, locs_a_handle, locs_b_handle, locs_out_handle, n), "map_op2_dev")

    def map_broadcast_dev(self, map_id, op, locs_src_handle, locs_scalar_handle, locs_dst_handle, n):
        self._check(self._lib.map_broadcast_dev(map_id, op, locs_src_handle, locs_scalar_handle, locs_dst_handle, n), "map_broadcast_dev")

    def map_rmsnorm_dev(self, map_id, locs_src_handle, locs_wt_handle, locs_dst_handle, n_rows, dim, eps=1e-5):
        self._check(self._lib.map_rmsnorm_dev(map_id, locs_src_handle, locs_wt_handle, locs_dst_handle, n_rows, dim, eps), "map_rmsnorm_dev")

    def map_rmsnorm_x_dev(self, map_act, map_wt, locs_src_handle, locs_wt_handle, locs_dst_handle, n_rows, dim, eps=1e-5):
        self._check(self._lib.map_rmsnorm_x_dev(map_act, map_wt, locs_src_handle, locs_wt_handle, locs_dst_handle, n_rows, dim, eps),
                    "map_rmsnorm_x_dev")

    def map_rmsnorm_add_dev(self, map_id, locs_src_handle, locs_wt_handle, locs_resid_handle, locs_dst_handle, n_rows, dim, eps=1e-5):
        self._check(self._lib.map_rmsnorm_add_dev(map_id, locs_src_handle, locs_wt_handle, locs_resid_handle, locs_dst_handle,
                                                  n_rows, dim, eps), "map_rmsnorm_add_dev")

    def map_rope_dev(self, map_id, locs_src_handle, locs_dst_handle, n_tokens, n_heads, head_dim, pos_offset=0, freq_base=10000.0):
        self._check(self._lib.map_rope_dev(map_id, locs_src_handle, locs_dst_handle, n_tokens, n_heads, head_dim, pos_offset, freq_base),
                    "map_rope_dev")

    def map_qk_norm_rope_x_dev(self, map_act_id, map_wt_id, locs_q_src_handle, locs_q_wt_handle, locs_k_src_handle, locs_k_wt_handle,
                               locs_qk_dst_handle, q_rows, q_dim, k_rows, k_dim, pos_offset=0, freq_base=10000.0):
        self._check(self._lib.map_qk_norm_rope_x_dev(map_act_id, map_wt_id, locs_q_src_handle, locs_q_wt_handle, locs_k_src_handle,
                                                     locs_k_wt_handle, locs_qk_dst_handle, q_rows, q_dim, k_rows, k_dim,
                                                     pos_offset, freq_base), "map_qk_norm_rope_x_dev")

    def map_row_copy_dev(self, map_id, copy_spec_handle, src_base_handle, n_copies, row_size):
        self._check(self._lib.map_row_copy_dev(map_id, copy_spec_handle, src_base_handle, n_copies, row_size), "map_row_copy_dev")

    def map_row_copy_offset_dev(self, map_id, copy_spec_handle, src_base_handle, dst_row_offset, n_copies, row_size):
        self._check(self._lib.map_row_copy_offset_dev(map_id, copy_spec_handle, src_base_handle, dst_row_offset, n_copies, row_size),
                    "map_row_copy_offset_dev")

    def map_matmul_t_dev(self, map_id, locs_a_handle, locs_b_handle, locs_c_handle, M, K, N, n_ops=1):
        self._check(self._lib.map_matmul_t_dev(map_id, locs_a_handle, locs_b_handle, locs_c_handle, M, K, N, n_ops), "map_matmul_t_dev")

    def map_matmul_t_xq4_dev(self, map_act, map_wt, locs_a_handle, locs_b_handle, locs_c_handle, M, K, N, n_ops=1):
        self._check(self._lib.map_matmul_t_xq4_dev(map_act, map_wt, locs_a_handle, locs_b_handle, locs_c_handle, M, K, N, n_ops),
                    "map_matmul_t_xq4_dev")

    def map_matmul_t_xq8_dev(self, map_act, map_wt, locs_a_handle, locs_b_handle, locs_c_handle, M, K, N, n_ops=1):
        """C = A @ B^T with B in a GGUF Q8_0 / Q5_0 block map (adamah-MAIN/adamah/__init__.py map_matmul_t_xq8_dev)."""
        self._check(self._lib.map_matmul_t_xq8_dev(map_act, map_wt, locs_a_handle, locs_b_handle, locs_c_handle, M, K, N, n_ops),
                    "map_matmul_t_xq8_dev")

    def map_row_gather_xq8_dev(self, map_act, map_wt, src_base, dst_base, row_idx, row_size, scale=1.0):
        """One decoded row of a Q8_0 / Q5_0 block map, times ``scale``, into the float32 map
        (adamah-MAIN/adamah/__init__.py:1786-1798)."""
        self._check(self._lib.map_row_gather_xq8_dev(map_act, map_wt, src_base, dst_base, row_idx, row_size, float(scale)),
                    "map_row_gather_xq8_dev")

    def map_attn_softmax_value_dev(self, map_id, locs_scores_handle, locs_values_handle, locs_out_handle, n_ops, row_size, value_dim,
                                   scale=1.0, cap=0.0):
        self._check(self._lib.map_attn_softmax_value_dev(map_id, locs_scores_handle, locs_values_handle, locs_out_handle, n_ops,
                                                         row_size, value_dim, scale, cap), "map_attn_softmax_value_dev")

    def map_argmax_dev(self, map_id, locs_src_handle, locs_dst_handle, n):
        self._check(self._lib.map_argmax_dev(map_id, locs_src_handle, locs_dst_handle, n), "map_argmax_dev")

    def map_resolve_idx_dev(self, map_id, base_locs_handle, locs_sel_handle, locs_dst_handle, n):
        self._check(self._lib.map_resolve_idx_dev(map_id, base_locs_handle, locs_sel_handle, locs_dst_handle, n), "map_resolve_idx_dev")

    def map_matvec_topk_t_xq4_dev(self, map_act_id, map_wt_id, locs_a_handle, locs_b_handle, penalty_ids_handle, locs_idx_dst_handle,
                                  locs_val_dst_handle, K, N, k, n_penalty, repeat_penalty):
        """adamah-MAIN/adamah/__init__.py `map_matvec_topk_t_xq4_dev` (adamah.c:9823)."""
        self._check(self._lib.map_matvec_topk_t_xq4_dev(map_act_id, map_wt_id, locs_a_handle, locs_b_handle, penalty_ids_handle,
                                                        locs_idx_dst_handle, locs_val_dst_handle, K, N, k, n_penalty, float(repeat_penalty)),
                    "map_matvec_topk_t_xq4_dev")

    def map_matvec_topk_t_xq4_ex_dev(self, map_act_id, map_wt_id, locs_a_handle, locs_b_handle, penalty_ids_handle, locs_idx_dst_handle,
                                     locs_val_dst_handle, K, N, k, n_penalty, repeat_penalty, rows_per_group):
        self._check(self._lib.map_matvec_topk_t_xq4_ex_dev(map_act_id, map_wt_id, locs_a_handle, locs_b_handle, penalty_ids_handle,
                                                           locs_idx_dst_handle, locs_val_dst_handle, K, N, k, n_penalty, float(repeat_penalty),
                                                           rows_per_group), "map_matvec_topk_t_xq4_ex_dev")

    def map_topk_dev(self, map_id, locs_src_handle, locs_idx_dst_handle, locs_val_dst_handle, n, k):
        self._check(self._lib.map_topk_dev(map_id, locs_src_handle, locs_idx_dst_handle, locs_val_dst_handle, n, k), "map_topk_dev")

    def map_topp_dev(self, map_id, locs_src_handle, locs_dst_handle, n, temperature, top_p):
        self._check(self._lib.map_topp_dev(map_id, locs_src_handle, locs_dst_handle, n, float(temperature), float(top_p)), "map_topp_dev")

    def map_sample_categorical_dev(self, map_id, locs_idx_handle, locs_prob_handle, rand_loc_handle, dst_loc_handle, n):
        self._check(self._lib.map_sample_categorical_dev(map_id, locs_idx_handle, locs_prob_handle, rand_loc_handle, dst_loc_handle, n),
                    "map_sample_categorical_dev")

    def map_repeat_penalty_dev(self, map_id, locs_src_handle, token_ids_handle, n_ids, penalty):
        self._check(self._lib.map_repeat_penalty_dev(map_id, locs_src_handle, token_ids_handle, n_ids, float(penalty)), "map_repeat_penalty_dev")

    def map_matvec_argmax_t_xq4_dev(self, map_act, map_wt, locs_a_handle, locs_b_handle, locs_idx_tmp_handle, locs_val_tmp_handle,
                                    locs_dst_handle, K, N, rows_per_group=256):
        self._check(self._lib.map_matvec_argmax_t_xq4_dev(map_act, map_wt, locs_a_handle, locs_b_handle, locs_idx_tmp_handle,
                                                          locs_val_tmp_handle, locs_dst_handle, K, N, rows_per_group),
                    "map_matvec_argmax_t_xq4_dev")

    def map_matvec_argmax_t_xq4_static_dev(self, map_act, map_wt, locs_a_handle, locs_b_handle, locs_idx_tmp_handle,
                                           locs_val_tmp_handle, locs_dst_handle, K, N, rows_per_group=256):
        """``map_matvec_argmax_t_xq4_dev`` for callers that must not allocate device memory
        during the call (their own memory pool owns the card, or an allocation's implicit
        device-wide sync is unacceptable where they call from).  Scratch is a fixed ~32 KB
        array in the library; N is limited to 4096 * rows_per_group rows, larger N raises.
        Calls share that array, so do not overlap them; make the first call on a device
        before any stream capture (it resolves the array's address)."""
        self._check(self._lib.map_matvec_argmax_t_xq4_static_dev(map_act, map_wt, locs_a_handle, locs_b_handle, locs_idx_tmp_handle,
                                                                 locs_val_tmp_handle, locs_dst_handle, K, N, rows_per_group),
                    "map_matvec_argmax_t_xq4_static_dev")

    # ---- batching / fusion / stats -------------------------------------------------
    def batch_begin(self):
        self._lib.batch_begin()

    def batch_end(self):
        self._lib.batch_end()

    @contextlib.contextmanager
    def batch(self):
        self.batch_begin()
        try:
            yield
        finally:
            self.batch_end()

    def fusion_enable(self, enable: bool):
        self._lib.adamah_fusion_enable(1 if enable else 0)

    def fusion_is_enabled(self) -> bool:
        return bool(self._lib.adamah_fusion_is_enabled())

    def fusion_flush(self):
        self._check(self._lib.adamah_fusion_flush(), "adamah_fusion_flush")

    def fusion_set_scheduler_mode(self, mode):
        if isinstance(mode, str):
            inv = {v: k for k, v in _SCHED_NAMES.items()}
            if mode not in inv:
                raise ValueError(f"unknown scheduler mode {mode!r}")
            mode = inv[mode]
        self._lib.adamah_fusion_set_scheduler_mode(int(mode))

    def fusion_get_scheduler_mode(self) -> str:
        return _SCHED_NAMES.get(int(self._lib.adamah_fusion_get_scheduler_mode()), "unknown")

    @contextlib.contextmanager
    def fusion_disabled(self):
        was = self.fusion_is_enabled()
        if was:
            self.fusion_enable(False)
        try:
            yield
        finally:
            if was:
                self.fusion_enable(True)

    def register_loc_span(self, handle: int, map_id: int, start: int, count: int):
        self._check(self._lib.adamah_register_loc_span(handle, map_id, start, count), "adamah_register_loc_span")

    def register_row_base_span(self, handle: int, map_id: int, start: int, count: int, stride: int, row_size: int):
        self._check(self._lib.adamah_register_row_base_span(handle, map_id, start, count, stride, row_size), "adamah_register_row_base_span")

    def clear_loc_alias_meta(self, handle: int):
        self._lib.adamah_clear_loc_alias_meta(handle)

    def reset_native_stats(self):
        self._lib.adamah_stats_reset()

    def get_native_stats(self) -> Dict[str, int]:
        v = [ctypes.c_uint64(0) for _ in range(9)]
        self._lib.adamah_stats_get(*[ctypes.byref(x) for x in v])
        keys = ["dispatch_count", "submit_count", "barrier_count", "fusion_flush_count", "descriptor_set_update_count",
                "descriptor_cache_hit_count", "descriptor_cache_miss_count", "alias_conflict_count", "scheduler_mode"]
        out = {k: int(x.value) for k, x in zip(keys, v)}
        out["scheduler_mode_name"] = _SCHED_NAMES.get(out["scheduler_mode"], "unknown")
        return out

    def kernel_launches(self) -> int:
        return int(self._lib.adam_b200_kernel_launches())

    def tc_gemm_count(self) -> int:
        """Matrix products enqueued so far on the tcgen05 GEMM (calls with 9..64 activation rows)."""
        return int(self._lib.adam_b200_tc_gemm_count())

    def tc_gemm_policy(self, policy: int):
        """0 = never take the tcgen05 GEMM, 1 = where it is expected to be faster (default), 2 = whenever the shape allows."""
        self._check(self._lib.adam_b200_tc_gemm_policy(int(policy)), "adam_b200_tc_gemm_policy")

    def device_error(self) -> int:
        """Reads and clears the device error word (0 = none)."""
        return int(self._lib.adam_b200_device_error())

    # ---- timers and captured graphs (extension) ----------------------------------------
    def timer_begin(self):
        self._check(self._lib.adam_b200_timer_begin(), "adam_b200_timer_begin")

    def timer_end(self) -> float:
        """Milliseconds of device time since ``timer_begin`` (CUDA events on the context stream)."""
        ms = ctypes.c_float(0)
        self._check(self._lib.adam_b200_timer_end(ctypes.byref(ms)), "adam_b200_timer_end")
        return float(ms.value)

    def capture_begin(self):
        self._check(self._lib.adam_b200_capture_begin(), "adam_b200_capture_begin")

    def capture_end(self) -> int:
        gid = ctypes.c_uint32(0)
        self._check(self._lib.adam_b200_capture_end(ctypes.byref(gid)), "adam_b200_capture_end")
        return int(gid.value)

    def set_stream(self, cuda_stream: int = 0):
        """Enqueue on a caller-owned CUDA stream (``torch.cuda.current_stream().cuda_stream``); 0 restores
        the library's own stream.  Lets collectives issued by the caller order with the library's kernels."""
        self._check(self._lib.adam_b200_set_stream(int(cuda_stream)), "adam_b200_set_stream")

    def graph_launch(self, graph_id: int, times: int = 1):
        self._check(self._lib.adam_b200_graph_launch(graph_id, times), "adam_b200_graph_launch")

    def graph_destroy(self, graph_id: int):
        self._check(self._lib.adam_b200_graph_destroy(graph_id), "adam_b200_graph_destroy")

    # ---- decode plan -----------------------------------------------------------------
    def register_decode_plan(self, plan_id: int, ops):
        arr = (DecodePlanOp * len(ops))(*ops)
        self._check(self._lib.adamah_register_decode_plan(plan_id, arr, len(ops)), "adamah_register_decode_plan")

    def clear_decode_plan(self, plan_id: int):
        self._lib.adamah_clear_decode_plan(plan_id)

    def decode_step(self, plan_id: int, pos: int, seq_len: int):
        self._check(self._lib.adamah_decode_step(plan_id, pos, seq_len), "adamah_decode_step")

    def decode_plan_info(self, plan_id: int) -> dict:
        """How a registered plan runs: as one CUDA graph with device-side pos / seq_len, or by host substitution."""
        out = (ctypes.c_uint32 * 6)()
        self._check(self._lib.adam_b200_decode_plan_info(plan_id, out), "adam_b200_decode_plan_info")
        state = ctypes.c_int32(out[0]).value
        return dict(state=state, runs_as_graph=state == 2, cap=int(out[1]), graph_kernels=int(out[2]), recordings=int(out[3]),
                    graph_steps=int(out[4]), host_steps=int(out[5]))

    # ---- GGUF-block maps (extension) ---------------------------------------------------
    def upload_gguf_blocks(self, map_id: int, ggml_type: int, elem_off: int, raw, n_bytes: Optional[int] = None):
        """Raw GGUF blocks (numpy uint8 array, or a device pointer given as int
        together with ``n_bytes``) into a GGUF-block map at element ``elem_off``."""
        if isinstance(raw, int):
            ptr, nb = ctypes.c_void_p(raw), int(n_bytes)
        else:
            a = np.ascontiguousarray(raw, dtype=np.uint8)
            ptr, nb = self._ptr(a), a.nbytes
        self._check(self._lib.map_upload_gguf_blocks(map_id, ggml_type, elem_off, ptr, nb), "map_upload_gguf_blocks")

    def upload_gguf_file(self, map_id: int, ggml_type: int, elem_off: int, path: str, file_offset: int, n_bytes: int):
        """Blocks of one tensor straight from a .gguf file (``n_bytes`` at ``file_offset``) into a GGUF-block map."""
        self._check(self._lib.adam_b200_upload_gguf_file(map_id, ggml_type, elem_off, os.fsencode(path), file_offset, n_bytes),
                    "adam_b200_upload_gguf_file")

    def tile_tensor(self, map_id: int, elem_off: int, rows: int, cols: int):
        """Register a row-tiled copy of a Q4_0 tensor so GEMVs on it use the tensor-core kernel."""
        self._check(self._lib.adam_b200_tensor_tile(map_id, elem_off, rows, cols), "adam_b200_tensor_tile")

    def dequant_gguf(self, map_id: int, elem_off: int, n_elems: int) -> np.ndarray:
        out = np.empty(n_elems, np.float32)
        self._check(self._lib.map_dequant_gguf(map_id, elem_off, self._ptr(out), n_elems), "map_dequant_gguf")
        return out

    def quantize_q4_0_dev(self, w_dev_ptr: int, n_elems: int, raw_dev_ptr: int):
        self._check(self._lib.adam_b200_quantize_q4_0_dev(ctypes.c_void_p(w_dev_ptr), n_elems, ctypes.c_void_p(raw_dev_ptr)),
                    "adam_b200_quantize_q4_0_dev")

    # ---- lifetime ---------------------------------------------------------------------
    def shutdown(self):
        if not self._closed:
            self._closed = True
            self._lib.adamah_shutdown()

    def __repr__(self):
        return f"<adam_b200.Adamah cuda:{self.device_index} sms={self.sm_count} maps={sorted(self._maps)}>"


def init(cache_mb: Optional[int] = None, cold_cache_mb: Optional[int] = None) -> Adamah:
    """Mirrors ``adamah.init`` (adamah-MAIN/adamah/__init__.py:2926)."""
    return Adamah(cache_mb=cache_mb, cold_cache_mb=cold_cache_mb)
