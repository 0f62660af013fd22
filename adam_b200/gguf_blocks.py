"""Host-side encoders and synthetic generators for GGUF Q4_0 / Q4_K / Q8_0 / Q5_0 blocks.

These build *inputs* (model files in memory): they are load-time host logic, not
part of the decode path, and they never decode blocks — decoding happens only in
the CUDA kernels.  Formats follow the GGUF block layouts the reference loader
reads (adam/loaders/gguf.py:24-33 QUANT_INFO, :290-299 Q4_0, :312-337 Q4_K,
:282-288 Q8_0, :301-310 Q5_0).
"""
from __future__ import annotations

import numpy as np

GGML_TYPE_F32 = 0
GGML_TYPE_Q4_0 = 2
GGML_TYPE_Q5_0 = 6
GGML_TYPE_Q8_0 = 8
GGML_TYPE_Q4_K = 12

Q4_0_BLOCK, Q4_0_BYTES = 32, 18
Q4_K_BLOCK, Q4_K_BYTES = 256, 144
Q8_0_BLOCK, Q8_0_BYTES = 32, 34
Q5_0_BLOCK, Q5_0_BYTES = 32, 22


def block_geometry(ggml_type: int) -> tuple[int, int]:
    """(elements per block, bytes per block) for a supported block type."""
    if ggml_type == GGML_TYPE_Q4_0:
        return Q4_0_BLOCK, Q4_0_BYTES
    if ggml_type == GGML_TYPE_Q4_K:
        return Q4_K_BLOCK, Q4_K_BYTES
    if ggml_type == GGML_TYPE_Q8_0:
        return Q8_0_BLOCK, Q8_0_BYTES
    if ggml_type == GGML_TYPE_Q5_0:
        return Q5_0_BLOCK, Q5_0_BYTES
    raise ValueError(f"unsupported ggml type {ggml_type}")


def gguf_nbytes(ggml_type: int, n_elems: int) -> int:
    be, bb = block_geometry(ggml_type)
    if n_elems % be:
        raise ValueError("element count is not a whole number of blocks")
    return n_elems // be * bb


def quantize_q4_0(w: np.ndarray) -> np.ndarray:
    """float32 ``[..., K]`` -> Q4_0 raw bytes ``[..., K/32*18]``.

    The published ggml/gguf-py Q4_0 rule, which the reference reaches through
    the PyPI ``gguf`` package (adam/loaders/gguf.py:16-17): per block of 32 take
    the element of largest magnitude (first one on ties) *with its sign*,
    ``d = that / -8``; codes are ``trunc(x * (1/d) + 8.5)`` clipped to 0..15;
    ``d`` is stored as fp16; byte j packs code j (low nibble) and code j+16
    (high nibble).  All arithmetic in float32.
    """
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.shape[-1] % Q4_0_BLOCK:
        raise ValueError("last dimension must be a multiple of 32")
    lead = w.shape[:-1]
    b = w.reshape(-1, Q4_0_BLOCK)
    imax = np.abs(b).argmax(axis=-1)[:, None]
    vmax = np.take_along_axis(b, imax, axis=-1)
    d = vmax / np.float32(-8)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1) / d).astype(np.float32)
    q = np.trunc(b * inv + np.float32(8.5)).astype(np.float32)
    q = np.clip(q, 0, 15).astype(np.uint8)
    packed = q[:, :16] | (q[:, 16:] << np.uint8(4))
    d16 = d.astype(np.float16).view(np.uint8).reshape(-1, 2)
    out = np.concatenate([d16, packed], axis=1)
    return out.reshape(lead + (w.shape[-1] // Q4_0_BLOCK * Q4_0_BYTES,))


def _round_half_away(x: np.ndarray) -> np.ndarray:
    """C ``roundf``: halves go away from zero (numpy's ``rint`` sends them to even)."""
    a = np.abs(x)
    f = np.floor(a)
    return np.sign(x) * (f + np.floor(np.float32(2) * (a - f)))


def quantize_q8_0(w: np.ndarray) -> np.ndarray:
    """float32 ``[..., K]`` -> Q8_0 raw bytes ``[..., K/32*34]``.

    The published ggml/gguf-py Q8_0 rule: per block of 32, ``d = max|x| / 127``,
    codes ``roundf(x * (1/d))`` (0 when d is 0) as int8, ``d`` stored as fp16.
    All arithmetic in float32."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.shape[-1] % Q8_0_BLOCK:
        raise ValueError("last dimension must be a multiple of 32")
    lead = w.shape[:-1]
    b = w.reshape(-1, Q8_0_BLOCK)
    d = np.abs(b).max(axis=-1, keepdims=True) / np.float32(127)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1) / d).astype(np.float32)
    q = _round_half_away(b * inv).astype(np.int8)
    out = np.concatenate([d.astype(np.float16).view(np.uint8).reshape(-1, 2), q.view(np.uint8)], axis=1)
    return out.reshape(lead + (w.shape[-1] // Q8_0_BLOCK * Q8_0_BYTES,))


def quantize_q5_0(w: np.ndarray) -> np.ndarray:
    """float32 ``[..., K]`` -> Q5_0 raw bytes ``[..., K/32*22]``.

    The published ggml/gguf-py Q5_0 rule: per block of 32 take the element of largest
    magnitude (first on ties) with its sign, ``d = that / -16``; codes are
    ``trunc(x * (1/d) + 16.5)`` clipped to 0..31; byte j packs the low four bits of
    code j (low nibble) and of code j+16 (high nibble); bit j of the little-endian
    uint32 ``qh`` is bit 4 of code j; ``d`` stored as fp16."""
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.shape[-1] % Q5_0_BLOCK:
        raise ValueError("last dimension must be a multiple of 32")
    lead = w.shape[:-1]
    b = w.reshape(-1, Q5_0_BLOCK)
    imax = np.abs(b).argmax(axis=-1)[:, None]
    vmax = np.take_along_axis(b, imax, axis=-1)
    d = vmax / np.float32(-16)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1) / d).astype(np.float32)
    q = np.clip(np.trunc(b * inv + np.float32(16.5)), 0, 31).astype(np.uint8)
    ql = (q[:, :16] & 0x0F) | ((q[:, 16:] & 0x0F) << np.uint8(4))
    qh = (((q >> 4) & 1).astype(np.uint32) << np.arange(32, dtype=np.uint32)[None, :]).sum(axis=1, dtype=np.uint32)
    out = np.concatenate([d.astype(np.float16).view(np.uint8).reshape(-1, 2), qh.astype("<u4").view(np.uint8).reshape(-1, 4), ql], axis=1)
    return out.reshape(lead + (w.shape[-1] // Q5_0_BLOCK * Q5_0_BYTES,))


def pack_q4_k_scales(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Pack ``[nb,8]`` 6-bit scales and mins into the 12-byte Q4_K field (the
    inverse of the unpack at adam/loaders/gguf.py:325-328)."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    rs = np.empty(sc.shape[:-1] + (12,), np.uint8)
    rs[..., 0:4] = (sc[..., 0:4] & 0x3F) | ((sc[..., 4:8] >> 4) << 6)
    rs[..., 4:8] = (mn[..., 0:4] & 0x3F) | ((mn[..., 4:8] >> 4) << 6)
    rs[..., 8:12] = (sc[..., 4:8] & 0x0F) | ((mn[..., 4:8] & 0x0F) << 4)
    return rs


def quantize_q4_k(w: np.ndarray) -> np.ndarray:
    """float32 ``[..., K]`` -> Q4_K raw bytes ``[..., K/256*144]``.

    A simple min/max encoder of this project's own (the reference has none and
    ``gguf.quantize`` does not implement Q4_K): per sub-block of 32 an affine
    range ``[-m, 15*s - m]`` with ``m >= 0``, then the 8 ``s`` and 8 ``m`` of a
    superblock are quantized to 6 bits against fp16 ``d`` and ``dmin``.  Parity is
    defined on the *decoded* blocks, so any valid encoder serves.
    """
    w = np.ascontiguousarray(w, dtype=np.float32)
    if w.shape[-1] % Q4_K_BLOCK:
        raise ValueError("last dimension must be a multiple of 256")
    lead = w.shape[:-1]
    x = w.reshape(-1, 8, 32)
    nb = x.shape[0]
    lo = np.minimum(x.min(axis=-1), 0)
    hi = np.maximum(x.max(axis=-1), 0)
    m_f = -lo
    s_f = (hi - lo) / np.float32(15)
    d = (s_f.max(axis=-1) / np.float32(63)).astype(np.float16)
    dm = (m_f.max(axis=-1) / np.float32(63)).astype(np.float16)
    d32 = d.astype(np.float32)[:, None]
    dm32 = dm.astype(np.float32)[:, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(d32 > 0, np.rint(s_f / d32), 0)
        mn = np.where(dm32 > 0, np.rint(m_f / dm32), 0)
    sc = np.clip(sc, 0, 63).astype(np.uint8)
    mn = np.clip(mn, 0, 63).astype(np.uint8)
    eff_s = (d32 * sc.astype(np.float32))[:, :, None]
    eff_m = (dm32 * mn.astype(np.float32))[:, :, None]
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(eff_s > 0, np.rint((x + eff_m) / eff_s), 0)
    q = np.clip(q, 0, 15).astype(np.uint8)                    # [nb,8,32]
    qg = q.reshape(nb, 4, 2, 32)
    packed = (qg[:, :, 0, :] | (qg[:, :, 1, :] << np.uint8(4))).reshape(nb, 128)
    out = np.empty((nb, Q4_K_BYTES), np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dm.view(np.uint8).reshape(nb, 2)
    out[:, 4:16] = pack_q4_k_scales(sc, mn)
    out[:, 16:] = packed
    return out.reshape(lead + (w.shape[-1] // Q4_K_BLOCK * Q4_K_BYTES,))


def random_q4_0_blocks(rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """Seeded synthetic Q4_0 matrix: per block ``d = fp16(|N(0,0.02)|/8)`` and 16
    uniform random bytes (nibbles uniform 0..15).  Returns ``[rows, cols/32*18]``."""
    nb = rows * cols // Q4_0_BLOCK
    d = (np.abs(rng.standard_normal(nb, dtype=np.float32)) * np.float32(0.02) / np.float32(8)).astype(np.float16)
    qs = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    out = np.empty((nb, Q4_0_BYTES), np.uint8)
    out[:, :2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:] = qs
    return out.reshape(rows, cols // Q4_0_BLOCK * Q4_0_BYTES)


def random_q4_k_blocks(rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """Seeded synthetic Q4_K matrix: ``d, dmin = fp16(|N(0,0.02)|/8)``, 12 uniform
    scale bytes (6-bit fields uniform 0..63) and 128 uniform quant bytes per
    superblock.  Returns ``[rows, cols/256*144]``."""
    nb = rows * cols // Q4_K_BLOCK
    dd = (np.abs(rng.standard_normal((nb, 2), dtype=np.float32)) * np.float32(0.02) / np.float32(8)).astype(np.float16)
    out = np.empty((nb, Q4_K_BYTES), np.uint8)
    out[:, 0:4] = dd.view(np.uint8).reshape(nb, 4)
    out[:, 4:] = rng.integers(0, 256, size=(nb, 140), dtype=np.uint8)
    return out.reshape(rows, cols // Q4_K_BLOCK * Q4_K_BYTES)


def random_q8_0_blocks(rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """Seeded synthetic Q8_0 matrix: per block ``d = fp16(|N(0,0.02)|/127)`` and 32 uniform
    random bytes (codes uniform -128..127).  Returns ``[rows, cols/32*34]``."""
    nb = rows * cols // Q8_0_BLOCK
    d = (np.abs(rng.standard_normal(nb, dtype=np.float32)) * np.float32(0.02) / np.float32(127)).astype(np.float16)
    out = np.empty((nb, Q8_0_BYTES), np.uint8)
    out[:, :2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:] = rng.integers(0, 256, size=(nb, 32), dtype=np.uint8)
    return out.reshape(rows, cols // Q8_0_BLOCK * Q8_0_BYTES)


def random_q5_0_blocks(rng: np.random.Generator, rows: int, cols: int) -> np.ndarray:
    """Seeded synthetic Q5_0 matrix: per block ``d = fp16(+-|N(0,0.02)|/16)`` (either sign, as
    the encoder produces), 4 uniform high-bit bytes and 16 uniform nibble bytes.
    Returns ``[rows, cols/32*22]``."""
    nb = rows * cols // Q5_0_BLOCK
    d = (rng.standard_normal(nb, dtype=np.float32) * np.float32(0.02) / np.float32(16)).astype(np.float16)
    out = np.empty((nb, Q5_0_BYTES), np.uint8)
    out[:, :2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:] = rng.integers(0, 256, size=(nb, 20), dtype=np.uint8)
    return out.reshape(rows, cols // Q5_0_BLOCK * Q5_0_BYTES)
