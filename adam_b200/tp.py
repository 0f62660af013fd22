"""Tensor-parallel decode: one process per GPU, NCCL all-reduce of the projection partial sums.

Sharding (the usual Megatron split, applied to the decode path of the 27B shape):

* q, k, v by whole heads and gate/up by rows of ``n_ff`` (column-parallel): every rank runs
  attention for its own heads and GeGLU for its own slice of the FFN with no communication;
* o-proj and down-proj along K (row-parallel): each rank produces a partial ``[batch, n_embd]``
  sum, one all-reduce each, i.e. two per layer;
* the LM head by vocabulary rows: each rank finds the arg-max of its rows, the ``(value, id)``
  pairs are all-gathered and the best one (ties to the lower id) becomes every rank's next token;
* norm weights and the embedding table are replicated.

K shards must be whole GGUF blocks (32 weights for Q4_0, 256 for Q4_K), so ``n_ff`` is split in
block units and may be uneven across ranks; heads must divide evenly.

The reference has no multi-GPU path; parity is defined against the oracle decoder summing the
shard partials in rank order (``OracleDecoder(tp_size=..)``).

The step runs as the decoder's parts (``adam_b200_decoder_step_part``) on torch's current stream
with ``torch.distributed`` collectives between them; after a warm-up the whole step, collectives
included, is captured into one CUDA graph and replayed.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Sequence, Tuple

import numpy as np

from . import gguf_blocks as gb
from .engine import ADAMEngine, STEP_LM, STEP_LOGITS
from .replicas import shard_sequences
from .synth import QTensor

PREFILL_ROWS = 64      # (sequence, position) rows of one prefill pass; the library's buffers hold max(max_batch, 64)


@dataclasses.dataclass
class ShardPlan:
    rank: int
    world: int
    heads: range          # query heads of this rank
    kv_heads: range
    ff: range             # rows of gate/up = K range of down
    vocab: range          # LM-head rows
    ff_bounds: Tuple[int, ...]   # K boundaries of down-proj over all ranks (len world + 1)


def block_elems(ggml_type: int) -> int:
    return 32 if ggml_type == gb.GGML_TYPE_Q4_0 else 256


def block_bytes(ggml_type: int) -> int:
    return 18 if ggml_type == gb.GGML_TYPE_Q4_0 else 144


def shard_plan(cfg, rank: int, world: int, ggml_type: int) -> ShardPlan:
    if cfg.n_head % world or cfg.n_head_kv % world:
        raise ValueError(f"{cfg.n_head} query / {cfg.n_head_kv} kv heads do not split over {world} ranks")
    be = block_elems(ggml_type)
    if (cfg.n_head // world) * cfg.head_dim % be:
        raise ValueError("a rank's heads must cover whole weight blocks of the o-proj K dimension")
    if cfg.n_ff % be:
        raise ValueError("n_ff must be a multiple of the weight block size")
    hq, hk = cfg.n_head // world, cfg.n_head_kv // world

    def scaled(r: range, unit: int) -> range:
        return range(r.start * unit, r.stop * unit)

    ff_units = cfg.n_ff // be
    bounds = tuple(shard_sequences(ff_units, r, world).start * be for r in range(world)) + (cfg.n_ff,)
    v_unit = 16
    if cfg.n_vocab % v_unit:
        v_unit = 1
    return ShardPlan(rank, world, range(rank * hq, (rank + 1) * hq), range(rank * hk, (rank + 1) * hk),
                     scaled(shard_sequences(ff_units, rank, world), be),
                     scaled(shard_sequences(cfg.n_vocab // v_unit, rank, world), v_unit), bounds)


def _rows(t: QTensor, r: range) -> QTensor:
    bpr = t.cols // block_elems(t.ggml_type) * block_bytes(t.ggml_type)
    raw = t.raw.reshape(t.rows, bpr)[r.start:r.stop]
    raw = raw.contiguous().reshape(-1) if hasattr(raw, "contiguous") else np.ascontiguousarray(raw).reshape(-1)
    return QTensor(t.ggml_type, len(r), t.cols, raw)


def _cols(t: QTensor, r: range) -> QTensor:
    be, bb = block_elems(t.ggml_type), block_bytes(t.ggml_type)
    if r.start % be or r.stop % be:
        raise ValueError("K shards must be whole weight blocks")
    raw = t.raw.reshape(t.rows, t.cols // be, bb)[:, r.start // be:r.stop // be]
    raw = raw.contiguous().reshape(-1) if hasattr(raw, "contiguous") else np.ascontiguousarray(raw).reshape(-1)
    return QTensor(t.ggml_type, t.rows, len(r), raw)


def local_config(cfg, plan: ShardPlan):
    """The configuration one rank's decoder is created with: its own heads, FFN rows and LM-head rows."""
    return dataclasses.replace(cfg, n_head=len(plan.heads), n_head_kv=len(plan.kv_heads), n_ff=len(plan.ff),
                               n_vocab=len(plan.vocab))


def shard_tensors(cfg, tensors: Dict[str, object], plan: ShardPlan):
    """This rank's configuration and tensors.  The local ``n_vocab`` is the LM-head shard; the
    embedding table stays whole (``token_embd.weight``) and the shard is ``output.weight``."""
    hd = cfg.head_dim
    q_rows = range(plan.heads.start * hd, plan.heads.stop * hd)
    k_rows = range(plan.kv_heads.start * hd, plan.kv_heads.stop * hd)
    local = local_config(cfg, plan)
    out: Dict[str, object] = {}
    lm = tensors["output.weight"] if "output.weight" in tensors else tensors["token_embd.weight"]
    for name, t in tensors.items():
        if not isinstance(t, QTensor):
            out[name] = t
        elif name == "token_embd.weight":
            out[name] = t
        elif name == "output.weight":
            continue
        elif name.endswith(("attn_q.weight",)):
            out[name] = _rows(t, q_rows)
        elif name.endswith(("attn_k.weight", "attn_v.weight")):
            out[name] = _rows(t, k_rows)
        elif name.endswith("attn_output.weight"):
            out[name] = _cols(t, q_rows)
        elif name.endswith(("ffn_gate.weight", "ffn_up.weight")):
            out[name] = _rows(t, plan.ff)
        elif name.endswith("ffn_down.weight"):
            out[name] = _cols(t, plan.ff)
        else:
            raise KeyError(f"do not know how to shard {name}")
    out["output.weight"] = _rows(lm, plan.vocab)
    return local, out


def merge_argmax_pairs(vals, ids):
    """Winner over ranks of per-rank ``(max logit, global id)`` pairs, ``[world, batch]`` torch tensors:
    the largest value wins, equal values go to the lower id (the single-GPU arg-max rule)."""
    import torch
    best = vals.max(dim=0).values
    cand = torch.where(vals == best.unsqueeze(0), ids, torch.full_like(ids, 2 ** 31 - 1))
    return cand.min(dim=0).values


class _DeviceArray:
    """Just enough of the CUDA array interface for ``torch.as_tensor`` to alias library memory."""

    def __init__(self, ptr: int, n: int, typestr: str):
        self.__cuda_array_interface__ = {"shape": (int(n),), "typestr": typestr, "data": (int(ptr), False), "version": 2}


class ADAMEngineTP(ADAMEngine):
    """``ADAMEngine`` over this rank's shard; ``step`` adds the collectives.  Needs an initialised
    ``torch.distributed`` process group (NCCL) and the library on this rank's GPU."""

    def __init__(self, gpu, cfg, tensors, rank: int, world: int, group=None, use_graph: bool = True,
                 presharded: bool = False, collectives: bool = True, allreduce: str = "p2p", **kw):
        """``cfg`` is the whole model's configuration.  ``tensors`` is the whole model (each rank
        keeps its slice) or, with ``presharded``, already this rank's tensors as ``shard_tensors``
        would return them (``token_embd.weight`` whole, ``output.weight`` = the vocabulary shard)."""
        import torch
        ggml_type = next(t.ggml_type for t in tensors.values() if isinstance(t, QTensor))
        self.plan = shard_plan(cfg, rank, world, ggml_type)
        self.full_cfg = cfg
        if presharded:
            local_cfg = local_config(cfg, self.plan)
            local_t = tensors
        else:
            local_cfg, local_t = shard_tensors(cfg, tensors, self.plan)
        self._group = group
        self._world = world
        self._collectives = collectives and world > 1      # False: time one shard's kernels alone (results are partial sums)
        self._use_graph = use_graph
        self._graphs: Dict[tuple, object] = {}
        self._eager_steps: Dict[tuple, int] = {}
        self._torch = torch
        # the library enqueues on this torch stream from here on, so the collectives order with its kernels
        self._stream = torch.cuda.Stream(device=gpu.device_index)
        gpu.set_stream(self._stream.cuda_stream)
        super().__init__(gpu, local_cfg, local_t, tp_rank=rank, tp_size=world, **kw)
        self._n_parts = int(self._lib.adam_b200_decoder_n_parts(self._dec))
        self._ar = None
        self._rows_cap = max(self._max_batch, PREFILL_ROWS)     # rows of the activation buffers (a prefill chunk fills them)
        if self._collectives and allreduce == "p2p":
            self._ar = self._open_peer_allreduce(cfg.n_embd * self._rows_cap * 4)
        dev = f"cuda:{gpu.device_index}"
        mb = self._max_batch
        self._proj = torch.as_tensor(_DeviceArray(self._buf(0), self._rows_cap * cfg.n_embd, "<f4"), device=dev).view(self._rows_cap, cfg.n_embd)
        self._tok = torch.as_tensor(_DeviceArray(self._buf(1), mb, "<i4"), device=dev)
        self._val = torch.as_tensor(_DeviceArray(self._buf(2), mb, "<f4"), device=dev)

    def _buf(self, which: int) -> int:
        import ctypes
        p, n = ctypes.c_uint64(0), ctypes.c_uint64(0)
        self._check(self._lib.adam_b200_decoder_buffer_ptr(self._dec, which, ctypes.byref(p), ctypes.byref(n)), "adam_b200_decoder_buffer_ptr")
        return int(p.value)

    def _open_peer_allreduce(self, max_bytes: int):
        """The library's one-shot all-reduce over peer memory: exchange the CUDA IPC handles of every
        rank's staging area and flags, map them, and line the ranks up once before first use.
        Returns the communicator id, or None when peer mapping is not possible (NCCL is used then)."""
        import ctypes
        import torch.distributed as dist
        cid = ctypes.c_uint32(0)
        mine = ctypes.create_string_buffer(128)
        rc = self._lib.adam_b200_ar_create(self._world, self.plan.rank, max_bytes, ctypes.byref(cid), mine)
        handles = [None] * self._world
        dist.all_gather_object(handles, bytes(mine.raw) if rc == 0 else None, group=self._group)
        ok = rc == 0 and all(h is not None for h in handles)
        if ok:
            blob = ctypes.create_string_buffer(b"".join(handles), 128 * self._world)
            ok = self._lib.adam_b200_ar_open(int(cid.value), blob) == 0
        flags = [None] * self._world
        dist.all_gather_object(flags, bool(ok), group=self._group)          # also the barrier before first use
        if all(flags):
            return int(cid.value)
        if rc == 0:
            self._lib.adam_b200_ar_destroy(int(cid.value))
        return None

    def _one_step(self, flags: int):
        """All parts of one token step with the collectives between them, on the current stream."""
        import torch.distributed as dist
        torch = self._torch
        B, L2, W = self._batch, 2 * self.cfg.n_layer, self._world
        for part in range(self._n_parts):
            self._check(self._lib.adam_b200_decoder_step_part(self._dec, part, flags), "adam_b200_decoder_step_part")
            if not self._collectives:
                continue
            if part < L2:
                self._reduce_proj(B)
            elif part == L2 and (flags & STEP_LM):
                # (value, global id) of every rank's best row; the best value wins, ties go to the lower id
                gid = self._tok[:B] + self.plan.vocab.start
                vals = torch.empty(W * B, dtype=torch.float32, device=gid.device)
                ids = torch.empty(W * B, dtype=torch.int32, device=gid.device)
                dist.all_gather_into_tensor(vals, self._val[:B].contiguous(), group=self._group)
                dist.all_gather_into_tensor(ids, gid.contiguous(), group=self._group)
                self._tok[:B].copy_(merge_argmax_pairs(vals.view(W, B), ids.view(W, B)))

    def _select_sampling_mode(self, config) -> str:
        """Greedy decoding stays on the devices (per-shard arg-max + merge); the device-side sampling step works on one
        GPU's full logits, so every other rule samples on the host from the gathered logits."""
        return "gpu_matvec_argmax" if config.is_greedy() and config.repeat_penalty == 1.0 else "cpu"

    def step(self, n_steps: int = 1, lm_head: bool = True, logits: bool = False, direct: bool = False, chain: bool = False,
             sample: bool = False):
        if sample:
            raise ValueError("device-side sampling is not available with tensor parallelism")
        torch = self._torch
        flags = (STEP_LM if lm_head else 0) | (STEP_LOGITS if logits else 0)
        key = (flags, self._batch)
        with torch.cuda.stream(self._stream):
            for _ in range(n_steps):
                if self._use_graph and not direct and key in self._graphs:
                    self._graphs[key].replay()
                    continue
                self._one_step(flags)
                n = self._eager_steps.get(key, 0) + 1
                self._eager_steps[key] = n
                if self._use_graph and not direct and n == 2:
                    # after two eager steps of a kind the step is recorded once (recording does not run
                    # it), collectives included, and replayed from then on
                    self._stream.synchronize()
                    gr = torch.cuda.CUDAGraph()
                    self.gpu.batch_begin()              # no per-call synchronisation inside the recording
                    try:
                        with torch.cuda.graph(gr, stream=self._stream):
                            self._one_step(flags)
                    finally:
                        self.gpu.batch_end()
                    self._graphs[key] = gr

    def _reduce_proj(self, rows: int):
        if self._ar is not None:
            self._check(self._lib.adam_b200_ar_allreduce(self._ar, self._proj.data_ptr(), rows * self.full_cfg.n_embd), "adam_b200_ar_allreduce")
        else:
            import torch.distributed as dist
            dist.all_reduce(self._proj[:rows], group=self._group)

    def prefill(self, n_tokens: int, chunked: bool = True):
        """Consumes ``n_tokens`` prompt positions of every sequence without the LM head, in chunks of
        up to 64 (sequence, position) rows per pass over this rank's weights, the partial sums of the
        o- and down-projections (one row per chunk row) all-reduced after each half layer."""
        if n_tokens <= 0:
            return
        if not chunked:
            self.step(n_tokens, lm_head=False)
            return
        t_max = max(1, self._rows_cap // self._batch)
        L2 = 2 * self.cfg.n_layer
        with self._torch.cuda.stream(self._stream):
            left = n_tokens
            while left > 0:
                T = min(t_max, left)
                for part in range(L2 + 1):
                    self._check(self._lib.adam_b200_decoder_prefill_part(self._dec, T, part), "adam_b200_decoder_prefill_part")
                    if self._collectives and part < L2:
                        self._reduce_proj(self._batch * T)
                left -= T

    def begin(self, prompts, reserve):
        super().begin(prompts, reserve)
        self._graphs = {k: g for k, g in self._graphs.items() if k[1] == self._batch}

    def close(self):
        self._graphs.clear()
        if self._ar is not None:
            self._lib.adam_b200_ar_destroy(self._ar)
            self._ar = None
        super().close()
        self.gpu.set_stream(0)
