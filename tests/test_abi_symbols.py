"""The C-ABI library loads and exports every symbol include/adam_b200.h declares
(no compute; runs without a GPU)."""
import ctypes
import os
import re

import pytest

from adam_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    src = open(os.path.join(ROOT, "include", "adam_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    src = re.sub(r"typedef struct.*?}\s*\w+;", "", src, flags=re.S)
    names = re.findall(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b([a-z_][a-z0-9_]*)\s*\(", src, flags=re.M)
    return sorted(set(n for n in names if n not in ("defined",)))


@pytest.fixture(scope="module")
def lib():
    from adam_b200.build import build
    return ctypes.CDLL(build())


def test_header_lists_functions():
    names = _header_functions()
    assert "map_matmul_t_xq4_dev" in names and "adamah_init" in names and len(names) > 70


def test_every_declared_symbol_is_exported(lib):
    missing = [n for n in _header_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in include/adam_b200.h but not exported: {missing}"


def test_binding_table_matches_header(lib):
    declared = set(_header_functions())
    bound = set(_lib.declared_symbols())
    assert declared <= bound | {"adam_b200_device_error", "adam_b200_handle_free"} or not (declared - bound), declared - bound
    for n in bound:
        assert hasattr(lib, n), n


def test_reference_binding_unguarded_symbols_present(lib):
    """The 55 symbols the reference's ctypes binding resolves without a guard
    (adamah-MAIN/adamah/__init__.py:530-960)."""
    names = """adamah_init adamah_shutdown adamah_sync adamah_synchronize adamah_synchronize_all adamah_fusion_enable
    adamah_fusion_is_enabled adamah_fusion_flush batch_begin batch_end map_init map_destroy map_size map_scatter map_gather
    map_upload_dev map_download_dev map_gather_dev map_scatter_dev map_op1 map_op2 map_matmul map_softmax map_layernorm
    map_broadcast map_reduce map_op1_dev map_op2_dev map_matmul_dev map_softmax_dev map_softmax_abs_dev
    map_attn_softmax_abs_dev map_attn_softmax_value_dev map_layernorm_dev map_broadcast_dev map_reduce_dev map_argmax_dev
    map_topk_dev map_topp_dev map_rmsnorm_dev map_rmsnorm_add_dev map_rmsnorm_x_dev map_rope_dev map_qk_norm_rope_x_dev
    map_matmul_t_dev map_row_copy_dev map_row_copy_offset_dev map_fma_dev map_matmul_t_x_dev map_matmul_x_dev
    map_matmul_t_xq4_dev map_matmul_xq4_dev map_matmul_t_xq8_dev map_matmul_xq8_dev map_row_gather_xq8_dev""".split()
    assert len(names) == 55
    assert not [n for n in names if not hasattr(lib, n)]


def test_calls_before_init_fail_cleanly(lib):
    lib.map_init.restype = ctypes.c_int
    assert lib.map_init(0, 4, 1, 16) == -3          # ADAMAH_ERR_INVALID: backend not initialised
    lib.adam_b200_last_error.restype = ctypes.c_char_p
    assert b"not initialised" in lib.adam_b200_last_error()
