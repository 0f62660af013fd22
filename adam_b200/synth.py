"""Seeded synthetic models: random-init weights quantized to GGUF blocks.

No model file, tokenizer or dataset is involved: every benchmark configuration
uses seeded N(0, 0.02) weights, then Q4_0 / Q4_K quantization, and random token
ids.  Tensor names follow the GGUF names the reference engine looks up
(adam/models/engine.py:2895-2921).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Union

import numpy as np

from . import gguf_blocks as gb
from .config import ModelConfig


@dataclass
class QTensor:
    """A 2-D weight kept as raw GGUF blocks, row-major ``[rows, cols]``."""
    ggml_type: int
    rows: int
    cols: int
    raw: np.ndarray            # uint8, rows * cols/block * block_bytes
    file: Optional[tuple] = None   # (path, byte offset) when the blocks still lie in a GGUF file (raw is a view of its mapping)

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def nbytes(self) -> int:
        return int(self.raw.size)


Tensor = Union[QTensor, np.ndarray]

LAYER_MATS = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")
LAYER_NORMS = ("attn_norm", "post_attention_norm", "ffn_norm", "post_ffw_norm")


def mat_shapes(cfg: ModelConfig) -> Dict[str, tuple]:
    q_dim = cfg.n_head * cfg.head_dim
    k_dim = cfg.n_head_kv * cfg.head_dim_kv
    return {
        "attn_q": (q_dim, cfg.n_embd), "attn_k": (k_dim, cfg.n_embd), "attn_v": (k_dim, cfg.n_embd),
        "attn_output": (cfg.n_embd, q_dim),
        "ffn_gate": (cfg.n_ff, cfg.n_embd), "ffn_up": (cfg.n_ff, cfg.n_embd),
        "ffn_down": (cfg.n_embd, cfg.n_ff),
    }


_QUANT_CHUNK_ROWS = 4096


def _quantize(w: np.ndarray, ggml_type: int) -> QTensor:
    """Encode a matrix; large ones in row chunks on a thread pool (the encoders are
    row-independent numpy code that releases the GIL, so the bytes do not depend on the split)."""
    enc = {gb.GGML_TYPE_Q4_0: gb.quantize_q4_0, gb.GGML_TYPE_Q4_K: gb.quantize_q4_k,
           gb.GGML_TYPE_Q8_0: gb.quantize_q8_0, gb.GGML_TYPE_Q5_0: gb.quantize_q5_0}[ggml_type]
    rows = w.shape[0]
    if rows <= _QUANT_CHUNK_ROWS:
        raw = enc(w)
    else:
        import os
        from concurrent.futures import ThreadPoolExecutor
        cuts = list(range(0, rows, _QUANT_CHUNK_ROWS)) + [rows]
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
            parts = list(ex.map(lambda i: enc(w[cuts[i]:cuts[i + 1]]), range(len(cuts) - 1)))
        raw = np.concatenate(parts, axis=0)
    return QTensor(ggml_type, w.shape[0], w.shape[1], np.ascontiguousarray(raw).reshape(-1))


def build_model(cfg: ModelConfig, ggml_type: int = gb.GGML_TYPE_Q4_0, seed: int = 0,
                tied: bool = True, norm_noise: float = 0.1, qk_norm: bool = True,
                post_norms: bool = True, embd_type: Optional[int] = None) -> Dict[str, Tensor]:
    """Random-init model on the host: N(0, 0.02) matrices quantized to
    ``ggml_type``, norm weights ``1 + norm_noise * N(0,1)``.  ``embd_type`` stores
    token_embd (and output.weight) in another block type, as real files do (Q8_0, Q5_0)."""
    rng = np.random.default_rng(seed)

    def mat(rows, cols, kind=None):
        w = rng.standard_normal((rows, cols), dtype=np.float32) * np.float32(0.02)
        return _quantize(w, ggml_type if kind is None else kind)

    def norm(n):
        return (np.float32(1) + np.float32(norm_noise) * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)

    t: Dict[str, Tensor] = {}
    t["token_embd.weight"] = mat(cfg.n_vocab, cfg.n_embd, embd_type)
    if not tied:
        t["output.weight"] = mat(cfg.n_vocab, cfg.n_embd, embd_type)
    t["output_norm.weight"] = norm(cfg.n_embd)
    shapes = mat_shapes(cfg)
    for L in range(cfg.n_layer):
        p = f"blk.{L}"
        for n in LAYER_NORMS:
            if n.startswith("post_") and not post_norms:
                continue
            t[f"{p}.{n}.weight"] = norm(cfg.n_embd)
        if qk_norm:
            t[f"{p}.attn_q_norm.weight"] = norm(cfg.head_dim)
            t[f"{p}.attn_k_norm.weight"] = norm(cfg.head_dim_kv)
        for n in LAYER_MATS:
            t[f"{p}.{n}.weight"] = mat(*shapes[n])
    return t


def build_model_cuda(gpu, cfg: ModelConfig, seed: int = 0, tied: bool = True, norm_noise: float = 0.1) -> Dict[str, Tensor]:
    """The same kind of model as ``build_model`` (Q4_0 only), generated on the GPU so
    that billion-weight shapes take seconds: seeded N(0, 0.02) matrices from torch's
    CUDA generator, quantized to raw Q4_0 blocks by the library's ggml-rule kernel.
    ``QTensor.raw`` is then a CUDA uint8 tensor (device memory), which the engine
    uploads without a host round trip.  torch is used for device memory and random
    numbers only."""
    import torch

    dev = torch.device("cuda", gpu.device_index)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    rng = np.random.default_rng(seed)

    def mat(rows, cols):
        w = torch.randn((rows, cols), generator=gen, device=dev, dtype=torch.float32) * 0.02
        raw = torch.empty(rows * cols // gb.Q4_0_BLOCK * gb.Q4_0_BYTES, dtype=torch.uint8, device=dev)
        torch.cuda.synchronize(dev)
        gpu.quantize_q4_0_dev(w.data_ptr(), rows * cols, raw.data_ptr())
        del w
        return QTensor(gb.GGML_TYPE_Q4_0, rows, cols, raw)

    def norm(n):
        return (np.float32(1) + np.float32(norm_noise) * rng.standard_normal(n, dtype=np.float32)).astype(np.float32)

    t: Dict[str, Tensor] = {}
    t["token_embd.weight"] = mat(cfg.n_vocab, cfg.n_embd)
    if not tied:
        t["output.weight"] = mat(cfg.n_vocab, cfg.n_embd)
    t["output_norm.weight"] = norm(cfg.n_embd)
    shapes = mat_shapes(cfg)
    for L in range(cfg.n_layer):
        p = f"blk.{L}"
        for n in LAYER_NORMS:
            t[f"{p}.{n}.weight"] = norm(cfg.n_embd)
        t[f"{p}.attn_q_norm.weight"] = norm(cfg.head_dim)
        t[f"{p}.attn_k_norm.weight"] = norm(cfg.head_dim_kv)
        for n in LAYER_MATS:
            t[f"{p}.{n}.weight"] = mat(*shapes[n])
    return t


def raw_to_host(t: "QTensor") -> np.ndarray:
    """Raw GGUF bytes of a tensor as a numpy array, wherever they live."""
    if isinstance(t.raw, np.ndarray):
        return t.raw
    return t.raw.cpu().numpy()


def model_weight_elems(cfg: ModelConfig, tied: bool = True) -> int:
    """Number of quantized weights one decoded token reads."""
    per_layer = sum(r * c for r, c in mat_shapes(cfg).values())
    return cfg.n_layer * per_layer + cfg.n_vocab * cfg.n_embd


def random_prompt(n_vocab: int, n: int, seed: int = 1) -> np.ndarray:
    return np.random.default_rng(seed).integers(0, n_vocab, size=n, dtype=np.int64).astype(np.int32)
