"""Loads ``libadam_b200.so`` and declares the ctypes signatures of its C ABI
(``include/adam_b200.h``).  There is no fallback: if the library is missing it is
built with nvcc, and if that fails the import error is raised to the caller."""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_uint32, c_uint64, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libadam_b200.so")

u32, u64, f32 = c_uint32, c_uint64, c_float
_lib = None


class DecodePlanOp(ctypes.Structure):
    """Same layout as the reference's ``AdamahDecodePlanOp``
    (adamah-MAIN/adamah/adamah.c:175-194; binding __init__.py:375-398)."""
    _fields_ = [("kind", u32), ("map_id", u32), ("map_id2", u32), ("op_code", u32),
                ("h0", u32), ("h1", u32), ("h2", u32), ("h3", u32), ("h4", u32), ("h5", u32),
                ("u0", u32), ("u1", u32), ("u2", u32), ("u3", u32), ("u4", u32), ("u5", u32),
                ("f0", f32), ("f1", f32)]


class DecoderDesc(ctypes.Structure):
    """``adam_b200_decoder_desc`` of include/adam_b200.h."""
    _fields_ = [("n_layer", u32), ("n_embd", u32), ("n_head", u32), ("n_head_kv", u32), ("head_dim", u32),
                ("n_ff", u32), ("n_vocab", u32), ("ffn_act", u32),
                ("norm_eps", f32), ("emb_scale", f32), ("attn_softcap", f32), ("final_softcap", f32), ("attn_scale", f32),
                ("sliding_window", u32), ("global_every", u32),
                ("max_batch", u32), ("kv_cap", u32), ("kv_dtype", u32), ("page_size", u32), ("n_pages", u32),
                ("tp_rank", u32), ("tp_size", u32), ("flags", u32)]


# name -> (restype, argtypes); the part-1 entries follow adamah.c's signatures
_SIGS = {
    "adamah_init": (c_int, []),
    "adamah_init_ex": (c_int, [u64, u64]),
    "adamah_shutdown": (None, []),
    "adamah_sync": (None, []),
    "adamah_synchronize": (None, [u64]),
    "adamah_synchronize_all": (None, []),
    "adamah_set_dtype": (c_int, [u32]),
    "adamah_get_dtype": (u32, []),
    "map_init": (c_int, [u32, u32, u32, u32]),
    "map_init_dtype": (c_int, [u32, u32, u32, u32, u32]),
    "map_destroy": (c_int, [u32]),
    "map_size": (u32, [u32]),
    "map_get_dtype": (u32, [u32]),
    "map_set_qparams": (c_int, [u32, c_void_p, c_void_p, u32]),
    "map_scatter": (c_int, [u32, c_void_p, c_void_p, u32]),
    "map_scatter_contiguous": (c_int, [u32, u32, c_void_p, u32]),
    "map_scatter_q4_packed_contiguous": (c_int, [u32, u32, c_void_p, u32]),
    "map_gather": (c_int, [u32, c_void_p, c_void_p, u32]),
    "map_upload_dev": (u64, [u32, c_void_p, u32]),
    "map_download_dev": (c_int, [u32, c_void_p, u32]),
    "map_gather_dev": (u64, [u32, u32, u32]),
    "map_scatter_dev": (u64, [u32, u32, u32, u32]),
    "batch_begin": (None, []),
    "batch_end": (None, []),
    "adamah_fusion_enable": (None, [c_int]),
    "adamah_fusion_is_enabled": (c_int, []),
    "adamah_fusion_flush": (c_int, []),
    "adamah_fusion_set_scheduler_mode": (None, [c_int]),
    "adamah_fusion_get_scheduler_mode": (c_int, []),
    "adamah_register_loc_span": (c_int, [u32, u32, u32, u32]),
    "adamah_register_row_base_span": (c_int, [u32, u32, u32, u32, u32, u32]),
    "adamah_clear_loc_alias_meta": (c_int, [u32]),
    "adamah_stats_reset": (None, []),
    "adamah_stats_get": (None, [POINTER(u64)] * 9),
    "map_rmsnorm_dev": (c_int, [u32, u32, u32, u32, u32, u32, f32]),
    "map_rmsnorm_x_dev": (c_int, [u32, u32, u32, u32, u32, u32, u32, f32]),
    "map_rmsnorm_add_dev": (c_int, [u32, u32, u32, u32, u32, u32, u32, f32]),
    "map_rope_dev": (c_int, [u32, u32, u32, u32, u32, u32, u32, f32]),
    "map_qk_norm_rope_x_dev": (c_int, [u32] * 12 + [f32]),
    "map_row_copy_dev": (c_int, [u32, u32, u32, u32, u32]),
    "map_row_copy_offset_dev": (c_int, [u32, u32, u32, u32, u32, u32]),
    "map_matmul_t_dev": (c_int, [u32] * 8),
    "map_matmul_t_xq4_dev": (c_int, [u32] * 9),
    "map_attn_softmax_value_dev": (c_int, [u32] * 7 + [f32, f32]),
    "map_op1_dev": (c_int, [u32] * 5),
    "map_op2_dev": (c_int, [u32] * 6),
    "map_broadcast_dev": (c_int, [u32] * 6),
    "map_argmax_dev": (c_int, [u32] * 4),
    "map_resolve_idx_dev": (c_int, [u32] * 5),
    "map_topk_dev": (c_int, [u32] * 6),
    "map_topp_dev": (c_int, [u32] * 4 + [ctypes.c_float, ctypes.c_float]),
    "map_sample_categorical_dev": (c_int, [u32] * 6),
    "map_repeat_penalty_dev": (c_int, [u32] * 4 + [ctypes.c_float]),
    "map_matvec_argmax_t_xq4_dev": (c_int, [u32] * 10),
    "map_matvec_argmax_t_xq4_static_dev": (c_int, [u32] * 10),
    "adamah_register_decode_plan": (c_int, [u32, POINTER(DecodePlanOp), u32]),
    "adamah_decode_step": (c_int, [u32, u32, u32]),
    "adamah_clear_decode_plan": (None, [u32]),
    # extensions
    "adam_b200_last_error": (c_char_p, []),
    "adam_b200_device_info": (c_int, [POINTER(c_int), POINTER(c_int), POINTER(u64)]),
    "adam_b200_kernel_launches": (u64, []),
    "adam_b200_device_error": (u32, []),
    "adam_b200_handle_free": (c_int, [u32]),
    "adam_b200_timer_begin": (c_int, []),
    "adam_b200_timer_end": (c_int, [POINTER(c_float)]),
    "adam_b200_capture_begin": (c_int, []),
    "adam_b200_capture_end": (c_int, [POINTER(u32)]),
    "adam_b200_graph_launch": (c_int, [u32, u32]),
    "adam_b200_graph_destroy": (c_int, [u32]),
    "adam_b200_decoder_create": (c_int, [POINTER(DecoderDesc), POINTER(u32)]),
    "adam_b200_decoder_destroy": (c_int, [u32]),
    "adam_b200_decoder_bind_matrix": (c_int, [u32, u32, u32, u32, u64, u32, u32]),
    "adam_b200_decoder_bind_norm": (c_int, [u32, u32, u32, u32, u64, u32]),
    "adam_b200_decoder_set_rope": (c_int, [u32, u32, c_void_p, c_void_p, u32, u32]),
    "adam_b200_decoder_begin": (c_int, [u32, u32, c_void_p, c_void_p, c_void_p]),
    "adam_b200_decoder_step": (c_int, [u32, u32, u32]),
    "adam_b200_decoder_prefill": (c_int, [u32, u32]),
    "adam_b200_decoder_set_tokens": (c_int, [u32, c_void_p]),
    "adam_b200_decoder_tokens_async": (c_int, [u32, POINTER(u32)]),
    "adam_b200_decoder_tokens_wait": (c_int, [u32, u32, c_void_p]),
    "adam_b200_decoder_continue": (c_int, [u32, c_void_p, u32, u32, u32]),
    "adam_b200_tc_gemm_count": (ctypes.c_uint64, []),
    "adam_b200_tc_gemm_policy": (c_int, [c_int]),
    "adam_b200_decoder_n_parts": (c_int, [u32]),
    "adam_b200_decoder_prefill_part": (c_int, [u32, u32, u32]),
    "adam_b200_decoder_step_part": (c_int, [u32, u32, u32]),
    "adam_b200_decoder_buffer_ptr": (c_int, [u32, u32, POINTER(u64), POINTER(u64)]),
    "adam_b200_set_stream": (c_int, [u64]),
    "adam_b200_ar_create": (c_int, [u32, u32, u64, POINTER(u32), c_void_p]),
    "adam_b200_ar_open": (c_int, [u32, c_void_p]),
    "adam_b200_ar_allreduce": (c_int, [u32, u64, u32]),
    "adam_b200_ar_destroy": (c_int, [u32]),
    "adam_b200_noalloc_prepare": (c_int, []),
    "adam_b200_ar_set_wait_us": (c_int, [u32, u64]),
    "adam_b200_ar_reset": (c_int, [u32]),
    "adam_b200_ar_timed_out": (c_int, [u32]),
    "adam_b200_ar_open_local": (c_int, [u32, c_void_p, u32]),
    "adam_b200_decoder_read_state": (c_int, [u32, c_void_p, c_void_p]),
    "adam_b200_decoder_read_log": (c_int, [u32, u32, u32, u32, c_void_p]),
    "adam_b200_decoder_read_logits": (c_int, [u32, u32, c_void_p]),
    "adam_b200_decoder_read_buffer": (c_int, [u32, u32, u32, c_void_p, u32]),
    "adam_b200_decoder_token_trace": (c_int, [u32, u32, c_void_p, c_void_p]),
    "adam_b200_decoder_step_trace": (c_int, [u32, u32, c_void_p, u32]),
    "adam_b200_decoder_test_wait_expiry": (c_int, [u32, u32]),
    "adam_b200_decoder_set_sampling": (c_int, [u32, u32, f32, f32, f32, u32, u64]),
    "map_matvec_topk_t_xq4_ex_dev": (c_int, [u32, u32, u32, u32, u32, u32, u32, u32, u32, u32, u32, f32, u32]),
    "map_matvec_topk_t_xq4_dev": (c_int, [u32, u32, u32, u32, u32, u32, u32, u32, u32, u32, u32, f32]),
    "map_matmul_t_xq8_dev": (c_int, [u32, u32, u32, u32, u32, u32, u32, u32, u32]),
    "map_row_gather_xq8_dev": (c_int, [u32, u32, u32, u32, u32, u32, f32]),
    "map_upload_gguf_blocks": (c_int, [u32, u32, u64, c_void_p, u64]),
    "adam_b200_decode_plan_info": (c_int, [u32, POINTER(u32)]),
    "adam_b200_upload_gguf_file": (c_int, [u32, u32, u64, ctypes.c_char_p, u64, u64]),
    "map_dequant_gguf": (c_int, [u32, u64, c_void_p, u64]),
    "adam_b200_tensor_tile": (c_int, [u32, u64, u32, u32]),
    "adam_b200_quantize_q4_0_dev": (c_int, [c_void_p, u64, c_void_p]),
}

# Symbols that exist only so the reference's own binding loads; they return -3.
OFF_PATH_SYMBOLS = [
    "map_op1", "map_op2", "map_matmul", "map_softmax", "map_layernorm", "map_broadcast", "map_reduce",
    "map_matmul_dev", "map_softmax_dev", "map_softmax_abs_dev", "map_attn_softmax_abs_dev", "map_layernorm_dev",
    "map_reduce_dev", "map_fma_dev", "map_matmul_t_x_dev", "map_matmul_x_dev",
    "map_matmul_xq4_dev", "map_matmul_xq8_dev",
]


def declared_symbols():
    """Every function ``include/adam_b200.h`` declares."""
    return list(_SIGS) + OFF_PATH_SYMBOLS


def register_signatures(extra: dict):
    _SIGS.update(extra)
    if _lib is not None:
        _apply(_lib, extra)


def _apply(lib, sigs):
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)          # AttributeError = the library is out of date: fail loudly
        fn.restype = res
        fn.argtypes = args


def load(build_if_missing: bool = True):
    """Return the loaded library (cached)."""
    global _lib
    if _lib is not None:
        return _lib
    path = os.environ.get("ADAM_B200_LIB_PATH", LIB_PATH)
    if not os.path.exists(path):
        if not build_if_missing:
            raise OSError(f"{path} not found; run `python -m adam_b200.build`")
        from .build import build
        path = build()
    lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
    _apply(lib, _SIGS)
    _lib = lib
    return lib


def last_error() -> str:
    return load().adam_b200_last_error().decode("utf-8", "replace")
