"""Numpy decoders for the weight storage formats on the decode path (oracle).

Test infrastructure: see ``oracle/__init__.py`` for who may import this.

Every function cites the reference code it restates.  All arithmetic is float32
with one rounding per operation, in the same order as the reference, so the
results are bit-identical to the reference loader (checked against committed
fixtures made by running the reference itself).
"""
from __future__ import annotations

import numpy as np

Q4_0_BLOCK = 32
Q4_0_BYTES = 18
Q4_K_BLOCK = 256
Q4_K_BYTES = 144
Q8_0_BLOCK = 32
Q8_0_BYTES = 34
Q5_0_BLOCK = 32
Q5_0_BYTES = 22


def _as_u8(raw) -> np.ndarray:
    a = np.frombuffer(raw, dtype=np.uint8) if isinstance(raw, (bytes, bytearray, memoryview)) else np.asarray(raw)
    if a.dtype != np.uint8:
        raise TypeError("raw GGUF blocks must be uint8")
    return a.reshape(-1)


def dequant_q4_0(raw, n_elems: int | None = None) -> np.ndarray:
    """GGUF Q4_0 -> float32, flat, logical order.

    Restates ``GGUFLoader._dq4_0`` (adam/loaders/gguf.py:290-299): an 18-byte
    block is an fp16 scale ``d`` followed by 16 bytes; element ``j`` (j<16) is
    ``(low nibble of byte j - 8) * d`` and element ``j+16`` is
    ``(high nibble of byte j - 8) * d``.  The subtraction is exact in float32
    and the product is rounded once.
    """
    a = _as_u8(raw)
    if a.size % Q4_0_BYTES:
        raise ValueError("Q4_0 byte count must be a multiple of 18")
    blk = a.reshape(-1, Q4_0_BYTES)
    d = blk[:, :2].copy().view(np.float16).astype(np.float32)          # [nb,1]
    qs = blk[:, 2:]
    lo = (qs & 0x0F).astype(np.float32) - np.float32(8)
    hi = ((qs >> 4) & 0x0F).astype(np.float32) - np.float32(8)
    out = np.concatenate([lo * d, hi * d], axis=1).reshape(-1)
    if n_elems is not None:
        if n_elems != out.size:
            raise ValueError("n_elems does not match the block count")
    return out


def unpack_q4_k_scales(scales12: np.ndarray):
    """6-bit sub-block scales and mins of Q4_K superblocks.

    Restates the unpack loop at adam/loaders/gguf.py:325-328.  ``scales12`` is
    ``[nb,12]`` uint8; returns two ``[nb,8]`` uint8 arrays (scale, min).
    """
    rs = scales12.astype(np.uint8)
    sc = np.empty(rs.shape[:-1] + (8,), np.uint8)
    mn = np.empty_like(sc)
    sc[..., :4] = rs[..., 0:4] & 0x3F
    mn[..., :4] = rs[..., 4:8] & 0x3F
    sc[..., 4:] = (rs[..., 8:12] & 0x0F) | ((rs[..., 0:4] >> 6) << 4)
    mn[..., 4:] = (rs[..., 8:12] >> 4) | ((rs[..., 4:8] >> 6) << 4)
    return sc, mn


def dequant_q4_k(raw, n_elems: int | None = None) -> np.ndarray:
    """GGUF Q4_K -> float32, flat, logical order.

    Restates ``GGUFLoader._dq4k`` (adam/loaders/gguf.py:312-337).  A 144-byte
    superblock holds fp16 ``d``, fp16 ``dmin``, 12 bytes of packed 6-bit
    scales/mins and 128 quant bytes.  For group g (0..3) the 32 bytes
    ``qs[32g:32g+32]`` give elements ``64g..64g+31`` from their low nibbles with
    ``(d*sc[2g], dmin*m[2g])`` and elements ``64g+32..64g+63`` from their high
    nibbles with ``(d*sc[2g+1], dmin*m[2g+1])``; value = ``q*(d*sc) - dmin*m``
    with every product and the difference rounded to float32 separately.
    """
    a = _as_u8(raw)
    if a.size % Q4_K_BYTES:
        raise ValueError("Q4_K byte count must be a multiple of 144")
    blk = a.reshape(-1, Q4_K_BYTES)
    nb = blk.shape[0]
    d = blk[:, 0:2].copy().view(np.float16).astype(np.float32)          # [nb,1]
    dm = blk[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc6, mn6 = unpack_q4_k_scales(blk[:, 4:16])
    sc = d * sc6.astype(np.float32)                                     # [nb,8]  d*s2
    mn = dm * mn6.astype(np.float32)                                    # [nb,8]  dm*m2
    qs = blk[:, 16:].reshape(nb, 4, 32)
    lo = (qs & 0x0F).astype(np.float32)
    hi = ((qs >> 4) & 0x0F).astype(np.float32)
    out = np.empty((nb, 4, 2, 32), np.float32)
    out[:, :, 0, :] = lo * sc[:, 0::2, None] - mn[:, 0::2, None]
    out[:, :, 1, :] = hi * sc[:, 1::2, None] - mn[:, 1::2, None]
    out = out.reshape(-1)
    if n_elems is not None and n_elems != out.size:
        raise ValueError("n_elems does not match the block count")
    return out


def dequant_q8_0(raw, n_elems: int | None = None) -> np.ndarray:
    """GGUF Q8_0 -> float32, flat, logical order.

    Restates ``GGUFLoader._dq8`` (adam/loaders/gguf.py:282-288): a 34-byte block
    is an fp16 scale ``d`` followed by 32 int8 codes; element ``j`` is
    ``float32(q_j) * float32(d)`` (exact in float32: 8 + 11 significant bits).
    """
    a = _as_u8(raw)
    if a.size % Q8_0_BYTES:
        raise ValueError("Q8_0 byte count must be a multiple of 34")
    blk = a.reshape(-1, Q8_0_BYTES)
    d = blk[:, :2].copy().view(np.float16).astype(np.float32)          # [nb,1]
    q = blk[:, 2:].view(np.int8).astype(np.float32)
    out = (q * d).reshape(-1)
    if n_elems is not None and n_elems != out.size:
        raise ValueError("n_elems does not match the block count")
    return out


def dequant_q5_0(raw, n_elems: int | None = None) -> np.ndarray:
    """GGUF Q5_0 -> float32, flat, logical order.

    Restates ``GGUFLoader._dq5_0`` (adam/loaders/gguf.py:301-310): a 22-byte
    block is an fp16 scale ``d``, a little-endian uint32 ``qh`` and 16 nibble
    bytes; element ``j`` has the low nibble of byte ``j`` (j < 16) or the high
    nibble of byte ``j-16`` as its low four bits and bit ``j`` of ``qh`` as bit 4;
    value = ``d * (code - 16)`` (exact in float32).
    """
    a = _as_u8(raw)
    if a.size % Q5_0_BYTES:
        raise ValueError("Q5_0 byte count must be a multiple of 22")
    blk = a.reshape(-1, Q5_0_BYTES)
    d = blk[:, :2].copy().view(np.float16).astype(np.float32)          # [nb,1]
    qh = blk[:, 2:6].copy().view("<u4")                                 # [nb,1]
    ql = blk[:, 6:]
    lo = np.concatenate([ql & 0x0F, (ql >> 4) & 0x0F], axis=1).astype(np.int32)
    hi = ((qh >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.int32)
    out = (d * ((lo | (hi << 4)) - 16).astype(np.float32)).reshape(-1)
    if n_elems is not None and n_elems != out.size:
        raise ValueError("n_elems does not match the block count")
    return out


def dequant(raw, ggml_type: int, rows: int, cols: int) -> np.ndarray:
    """Decode a ``[rows, cols]`` tensor stored as GGUF blocks (type 2, 12, 8 or 6)."""
    if ggml_type == 2:
        return dequant_q4_0(raw, rows * cols).reshape(rows, cols)
    if ggml_type == 12:
        return dequant_q4_k(raw, rows * cols).reshape(rows, cols)
    if ggml_type == 8:
        return dequant_q8_0(raw, rows * cols).reshape(rows, cols)
    if ggml_type == 6:
        return dequant_q5_0(raw, rows * cols).reshape(rows, cols)
    raise ValueError(f"unsupported ggml type {ggml_type}")


# ---------------------------------------------------------------------------
# The reference backend's own "Q4 map" storage (nibbles + per-group scale/zero)
# ---------------------------------------------------------------------------

def q4map_quantize(values: np.ndarray, scales: np.ndarray, zeros: np.ndarray, group_size: int = 32) -> np.ndarray:
    """Nibble codes the reference backend stores when float32 values are
    scattered into a Q4 map: ``q = clamp(round((v - zero)/max(scale,1e-10)), 0, 15)``
    (adamah-MAIN/adamah/shaders/src/q4/map_scatter.comp; CPU model in
    tests/test_q4_roundtrip.py:47-63).  Ties round to even, as ``np.round`` does
    in that CPU model (GLSL leaves the direction of a tie to the driver).
    """
    v = np.asarray(values, np.float32).reshape(-1)
    g = np.arange(v.size) // group_size
    s = np.maximum(np.asarray(scales, np.float32)[g], np.float32(1e-10))
    z = np.asarray(zeros, np.float32)[g]
    qf = (v - z) / s
    q = np.clip(np.round(qf), np.float32(0), np.float32(15))
    return q.astype(np.uint8)


def q4map_dequantize(codes: np.ndarray, scales: np.ndarray, zeros: np.ndarray, group_size: int = 32) -> np.ndarray:
    """``value = code*scale + zero`` per element (shader ``load_q4``,
    adamah-MAIN/adamah/shaders/src/f32/map_matvec_t_xq4.comp:49-55; CPU model in
    tests/test_q4_roundtrip.py:47-63)."""
    c = np.asarray(codes).reshape(-1).astype(np.float32)
    g = np.arange(c.size) // group_size
    return c * np.asarray(scales, np.float32)[g] + np.asarray(zeros, np.float32)[g]


def q4k_to_q4map_params(raw) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Lossless mapping of Q4_K superblocks to Q4-map storage, as the reference
    engine does at load (adam/models/engine.py:1022-1065): per group of 32,
    ``scale = d*sc`` and ``zero = -(dmin*m)``, nibble codes in logical order.
    Returns (codes uint8 [n], scales f32 [n/32], zeros f32 [n/32]).
    """
    a = _as_u8(raw).reshape(-1, Q4_K_BYTES)
    nb = a.shape[0]
    d = a[:, 0:2].copy().view(np.float16).astype(np.float32)
    dm = a[:, 2:4].copy().view(np.float16).astype(np.float32)
    sc6, mn6 = unpack_q4_k_scales(a[:, 4:16])
    scales = (d * sc6.astype(np.float32)).reshape(-1)
    zeros = (-(dm * mn6.astype(np.float32))).reshape(-1)
    qs = a[:, 16:].reshape(nb, 4, 32)
    codes = np.stack([qs & 0x0F, (qs >> 4) & 0x0F], axis=2).reshape(-1).astype(np.uint8)
    return codes, scales, zeros
