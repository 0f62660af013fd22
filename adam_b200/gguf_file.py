"""GGUF file reader with the surface of the reference's ``GGUFLoader``
(adam/loaders/gguf.py:44-370): ``GGUFLoader(path).load()``, ``metadata``, ``tensor_infos``,
``tensor_info_by_name``, ``tensor_types``, ``tensor_shapes``, ``get_tensor_info``,
``estimate_raw_bytes`` / ``estimate_f32_bytes``, ``load_tensor_raw``, ``load_tensor_f32``,
``iter_tensor_chunks`` and the tokenizer getters.

What differs, by design: nothing is read at ``load()`` beyond the header, the key/value table
and the tensor table; tensor data stays in the file (a read-only memory map serves
``load_tensor_raw``), and quantized tensors are never decoded on the host -- their blocks go
from the file to the GPU as they are (``ADAMEngine.from_gguf`` /
``adam_b200_upload_gguf_file``) and are decoded there.  ``load_tensor_f32`` therefore serves
only the unquantized types (F32, F16, BF16: the norm vectors).
"""
from __future__ import annotations

import mmap
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np

from .config import ModelConfig
from .synth import QTensor

GGUF_MAGIC = 0x46554747
GGML_TYPE_F32 = 0; GGML_TYPE_F16 = 1; GGML_TYPE_Q4_0 = 2; GGML_TYPE_Q5_0 = 6
GGML_TYPE_Q8_0 = 8; GGML_TYPE_Q4_K = 12; GGML_TYPE_Q6_K = 14; GGML_TYPE_BF16 = 30

# (bytes per block, elements per block) of every type the reader can size (adam/loaders/gguf.py:24-33)
QUANT_INFO = {
    GGML_TYPE_F32: (4, 1), GGML_TYPE_F16: (2, 1), GGML_TYPE_BF16: (2, 1),
    GGML_TYPE_Q8_0: (34, 32), GGML_TYPE_Q4_0: (18, 32), GGML_TYPE_Q5_0: (22, 32),
    GGML_TYPE_Q4_K: (144, 256), GGML_TYPE_Q6_K: (210, 256),
}
# block types the device kernels read
DEVICE_BLOCK_TYPES = (GGML_TYPE_Q4_0, GGML_TYPE_Q4_K, GGML_TYPE_Q8_0, GGML_TYPE_Q5_0)

# key/value scalar encodings (GGUF value types 0..7, 10..12)
_SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}
_NP_SCALAR = {0: "<u1", 1: "<i1", 2: "<u2", 3: "<i2", 4: "<u4", 5: "<i4", 6: "<f4", 10: "<u8", 11: "<i8", 12: "<f8"}


@dataclass
class TensorInfo:
    """One row of the tensor table: ``shape`` in GGUF order (fastest dimension first), ggml type, byte
    offset from the start of the data section (adam/loaders/gguf.py:40-42)."""
    name: str
    shape: Tuple[int, ...]
    dtype: int
    offset: int


class _Cursor:
    """Sequential little-endian reads from a buffer."""

    def __init__(self, buf, pos: int = 0):
        self.buf, self.pos = buf, pos

    def unpack(self, fmt: str):
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += struct.calcsize(fmt)
        return v

    def string(self) -> str:
        n = self.unpack("<Q")
        s = bytes(self.buf[self.pos:self.pos + n]).decode("utf-8")
        self.pos += n
        return s

    def value(self, t: int):
        if t in _SCALAR:
            v = self.unpack(_SCALAR[t])
            return bool(v) if t == 7 else v
        if t == 8:
            return self.string()
        if t == 9:
            et, n = self.unpack("<I"), self.unpack("<Q")
            if et in _NP_SCALAR:                       # numeric arrays (token scores, types) in one slice
                a = np.frombuffer(self.buf, dtype=_NP_SCALAR[et], count=n, offset=self.pos)
                self.pos += a.nbytes
                return a.tolist()
            return [self.value(et) for _ in range(n)]
        raise ValueError(f"Unknown type {t}")


class GGUFLoader:
    def __init__(self, path: str, keep_tensors: bool = False, keep_raw_blocks: bool = False):
        """``keep_tensors`` / ``keep_raw_blocks`` are accepted for signature compatibility; data always stays in
        the file until it is asked for."""
        self.path = Path(path)
        self.keep_tensors = bool(keep_tensors)
        self.keep_raw_blocks = bool(keep_raw_blocks)
        self.metadata: Dict = {}
        self.tensor_infos: List[TensorInfo] = []
        self.tensor_info_by_name: Dict[str, TensorInfo] = {}
        self.tensor_types: Dict[str, int] = {}
        self.tensor_shapes: Dict[str, Tuple] = {}
        self.version = 0
        self.n_tensors = 0
        self.n_kv = 0
        self._data_offset = 0
        self._map = None

    # ---- parsing (adam/loaders/gguf.py:58-133) ------------------------------------------------
    def load(self, verbose: bool = False):
        with open(self.path, "rb") as f:
            self._map = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        c = _Cursor(self._map)
        magic = c.unpack("<I")
        if magic != GGUF_MAGIC:
            raise ValueError(f"Bad magic {magic:#x}")
        self.version = c.unpack("<I")
        self.n_tensors = c.unpack("<Q")
        self.n_kv = c.unpack("<Q")
        for _ in range(self.n_kv):
            key = c.string()
            self.metadata[key] = c.value(c.unpack("<I"))
        for _ in range(self.n_tensors):
            name = c.string()
            nd = c.unpack("<I")
            shape = tuple(c.unpack("<Q") for _ in range(nd))
            dtype = c.unpack("<I")
            ti = TensorInfo(name, shape, dtype, c.unpack("<Q"))
            self.tensor_infos.append(ti)
            self.tensor_info_by_name[name] = ti
            self.tensor_types[name] = dtype
            self.tensor_shapes[name] = shape[::-1]           # logical row-major order: [out, in]
        align = self.metadata.get("general.alignment", 32)
        self._data_offset = (c.pos + align - 1) // align * align
        for ti in self.tensor_infos:
            if ti.dtype in QUANT_INFO and self._data_offset + ti.offset + self._tensor_raw_size(ti) > len(self._map):
                raise ValueError(f"tensor {ti.name} extends past the end of {self.path.name}")
        if verbose:
            print(f"[GGUF] v{self.version}, {self.n_tensors} tensors, {self.n_kv} KV, data at byte {self._data_offset}")
        return self

    def close(self):
        if self._map is not None:
            self._map.close()
            self._map = None

    # ---- sizes (adam/loaders/gguf.py:174-194) ---------------------------------------------------
    def _tensor_numel(self, ti: TensorInfo) -> int:
        ne = 1
        for s in ti.shape:
            ne *= s
        return ne

    def _tensor_raw_size(self, ti: TensorInfo) -> int:
        if ti.dtype not in QUANT_INFO:
            raise NotImplementedError(f"Unsupported type {ti.dtype} for {ti.name}")
        bpb, epb = QUANT_INFO[ti.dtype]
        return (self._tensor_numel(ti) // epb) * bpb

    def get_tensor_info(self, name: str) -> TensorInfo:
        return self.tensor_info_by_name[name]

    def estimate_raw_bytes(self) -> int:
        return sum(self._tensor_raw_size(ti) for ti in self.tensor_infos)

    def estimate_f32_bytes(self) -> int:
        return sum(self._tensor_numel(ti) * 4 for ti in self.tensor_infos)

    def tensor_file_range(self, name: str) -> Tuple[int, int]:
        """(absolute byte offset in the file, byte count) of a tensor's data."""
        ti = self.get_tensor_info(name)
        return self._data_offset + ti.offset, self._tensor_raw_size(ti)

    # ---- data (adam/loaders/gguf.py:196-253) ----------------------------------------------------
    def load_tensor_raw(self, name: str) -> np.ndarray:
        """The tensor's bytes as a read-only uint8 view of the memory-mapped file (no copy)."""
        off, n = self.tensor_file_range(name)
        return np.frombuffer(self._map, dtype=np.uint8, count=n, offset=off)

    def load_tensor_f32(self, name: str) -> np.ndarray:
        ti = self.get_tensor_info(name)
        raw = self.load_tensor_raw(name)
        if ti.dtype == GGML_TYPE_F32:
            return raw.view("<f4").astype(np.float32)
        if ti.dtype == GGML_TYPE_F16:
            return raw.view("<f2").astype(np.float32)
        if ti.dtype == GGML_TYPE_BF16:
            return (raw.view("<u2").astype(np.uint32) << 16).view(np.float32)
        raise NotImplementedError(f"{name}: quantized blocks are decoded on the device (map_dequant_gguf), not on the host")

    def iter_tensor_chunks(self, name: str, max_chunk_mb: int = 32, include_raw: bool = True, include_f32: bool = False):
        """Yield ``(elem_off, n_elems, raw, None)`` over whole blocks, ``max_chunk_mb`` of raw bytes at a time
        (the reference's tuple layout; the float32 member is always None for quantized tensors)."""
        ti = self.get_tensor_info(name)
        ne = self._tensor_numel(ti)
        if ne <= 0:
            return
        if include_f32 and ti.dtype in DEVICE_BLOCK_TYPES + (GGML_TYPE_Q6_K,):
            raise NotImplementedError(f"{name}: quantized blocks are decoded on the device, not on the host")
        bpb, epb = QUANT_INFO[ti.dtype]
        raw = self.load_tensor_raw(name)
        chunk_elems = min(ne, max(epb, (max(1, int(max_chunk_mb)) * 1024 * 1024 // bpb) * epb))
        for elem_off in range(0, ne, chunk_elems):
            take = min(chunk_elems, ne - elem_off)
            part = raw[elem_off // epb * bpb:(elem_off + take) // epb * bpb]
            yield elem_off, take, (part if include_raw else None), (self.load_tensor_f32(name)[elem_off:elem_off + take] if include_f32 else None)

    # ---- tokenizer keys (adam/loaders/gguf.py:367-370) -------------------------------------------
    def get_tokenizer_vocab(self): return self.metadata.get("tokenizer.ggml.tokens")
    def get_tokenizer_scores(self): return self.metadata.get("tokenizer.ggml.scores")
    def get_bos_token_id(self): return self.metadata.get("tokenizer.ggml.bos_token_id", 2)
    def get_eos_token_id(self): return self.metadata.get("tokenizer.ggml.eos_token_id", 1)

    # ---- what the engine needs -----------------------------------------------------------------
    def model_config(self, verbose: bool = False) -> ModelConfig:
        """``ModelConfig.from_gguf_metadata`` followed by the shape-based corrections the reference engine
        applies after loading (adam/models/engine.py:56-111, :477-500)."""
        return ModelConfig.from_gguf_metadata(self.metadata, verbose=verbose).detect_dims(self.tensor_shapes)

    def model_tensors(self) -> Dict[str, object]:
        """The tensor dictionary ``ADAMEngine`` takes: matrices as ``QTensor`` whose blocks are still in the file
        (``raw`` is a view of the mapping, ``file`` = (path, offset) for the streamed upload), vectors as float32."""
        out: Dict[str, object] = {}
        for ti in self.tensor_infos:
            shape = self.tensor_shapes[ti.name]
            if ti.dtype in DEVICE_BLOCK_TYPES and len(shape) == 2:
                off, _ = self.tensor_file_range(ti.name)
                out[ti.name] = QTensor(ti.dtype, int(shape[0]), int(shape[1]), self.load_tensor_raw(ti.name), file=(str(self.path), off))
            elif ti.dtype in (GGML_TYPE_F32, GGML_TYPE_F16, GGML_TYPE_BF16):
                out[ti.name] = self.load_tensor_f32(ti.name).reshape(shape)
            else:
                raise NotImplementedError(f"{ti.name}: ggml type {ti.dtype} has no device kernels here (supported blocks: Q4_0, Q4_K, Q8_0, Q5_0)")
        return out
