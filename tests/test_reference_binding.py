"""The reference's OWN ctypes binding (adamah-MAIN/adamah/__init__.py) over libadam_b200.so, selected the way a user
of the reference would select it: the ADAMAH_LIB_PATH variable (__init__.py:156-161).  CPU only; needs a checkout of the
reference beside the repository (ADAM_REFERENCE_DIR, default /root/reference) and is skipped without one."""
import ctypes
import importlib.util
import os
import sys

import pytest

from adam_b200 import _lib

REFERENCE = os.environ.get("ADAM_REFERENCE_DIR", "/root/reference")
BINDING = os.path.join(REFERENCE, "adamah-MAIN", "adamah", "__init__.py")

pytestmark = pytest.mark.skipif(not os.path.isfile(BINDING), reason="no checkout of the reference")


@pytest.fixture(scope="module")
def ref_adamah():
    _lib.load()                                     # builds the library if it is missing
    old = os.environ.get("ADAMAH_LIB_PATH")
    os.environ["ADAMAH_LIB_PATH"] = _lib.LIB_PATH
    spec = importlib.util.spec_from_file_location("ref_adamah_binding", BINDING, submodule_search_locations=[os.path.dirname(BINDING)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_adamah_binding"] = mod
    spec.loader.exec_module(mod)
    yield mod
    sys.modules.pop("ref_adamah_binding", None)
    if old is None:
        os.environ.pop("ADAMAH_LIB_PATH", None)
    else:
        os.environ["ADAMAH_LIB_PATH"] = old


def test_binding_resolves_this_library(ref_adamah):
    assert ref_adamah._resolve_lib_path() == _lib.LIB_PATH


def test_setup_ctypes_finds_every_symbol_it_needs(ref_adamah):
    """``_setup_ctypes`` sets argument types on every entry point the binding uses; a missing unguarded symbol raises
    AttributeError, a missing optional one clears its ``_has_*`` flag."""
    gpu = ref_adamah.Adamah.__new__(ref_adamah.Adamah)
    gpu._lib = ctypes.CDLL(ref_adamah._resolve_lib_path())
    gpu._setup_ctypes()
    flags = {k: v for k, v in vars(gpu).items() if k.startswith("_has_")}
    # the optional entry points of the decode path are all present
    for name in ("_has_map_matvec_argmax_t_xq4_dev", "_has_map_matvec_topk_t_xq4_dev", "_has_map_matvec_topk_t_xq4_ex_dev",
                 "_has_map_resolve_idx_dev", "_has_map_sample_categorical_dev", "_has_map_repeat_penalty_dev", "_has_decode_plan",
                 "_has_native_stats"):
        if name in flags:
            assert flags[name], name
    assert any(flags.values())
    # constants the two bindings share
    import adam_b200 as A
    for name in ("DTYPE_F32", "DTYPE_Q4", "DTYPE_Q8", "OP_ADD", "OP_GEGLU", "OP_TANH", "BROADCAST_MUL", "BROADCAST_DIV", "DECODE_RUNTIME_POS",
                 "DECODE_RUNTIME_SEQ_LEN", "DECODE_OP_MATMUL_T_XQ4", "DECODE_OP_ROW_COPY_OFFSET", "DECODE_OP_ATTN_SOFTMAX_VALUE"):
        if hasattr(ref_adamah, name):
            assert getattr(ref_adamah, name) == getattr(A, name), name
    # the plan record has the layout the library reads
    if hasattr(ref_adamah, "DecodePlanOp"):
        assert ctypes.sizeof(ref_adamah.DecodePlanOp) == ctypes.sizeof(A.DecodePlanOp)
        assert [f[0] for f in ref_adamah.DecodePlanOp._fields_] == [f[0] for f in A.DecodePlanOp._fields_]


def test_init_without_a_gpu_raises_like_the_reference(ref_adamah):
    """On a machine without a CUDA device the binding's constructor gets a non-zero status from adamah_init and raises."""
    try:
        import torch
        if torch.cuda.is_available():
            pytest.skip("a CUDA device is present")
    except ImportError:
        pass
    with pytest.raises(RuntimeError, match="adamah_init failed"):
        ref_adamah.Adamah()
