"""adam_b200: a B200-native (sm_100a) backend for ADAM's quantized decode path.

The package mirrors the operator surface of the reference's ``adamah`` backend
module (adamah-MAIN/adamah/__init__.py): ``init()`` returns a backend object with
the same ``map_*`` / ``batch_*`` / ``fusion_*`` methods, and the module exposes
the same ``DTYPE_*`` / ``OP_*`` constants, so it can be handed to a model engine
as ``(gpu, A)``.  All compute runs in hand-written CUDA kernels behind a C ABI
(``libadam_b200.so``); there is no CPU fallback.
"""
from .config import GenerationConfig, ModelConfig  # noqa: F401
from .constants import *  # noqa: F401,F403


def init(*args, **kwargs):
    """Create the backend object (loads ``libadam_b200.so``; raises if the
    library or a CUDA device is missing).  Mirrors ``adamah.init``
    (adamah-MAIN/adamah/__init__.py:2926)."""
    from .backend import init as _init
    return _init(*args, **kwargs)


def __getattr__(name):
    if name in ("Adamah", "DecodePlanOp"):
        from . import backend
        return getattr(backend, name)
    if name == "ADAMEngine":
        from .engine import ADAMEngine
        return ADAMEngine
    raise AttributeError(name)
