"""Model engine with the surface of the reference's ``ADAMEngine``
(adam/models/engine.py:114-3964): ``ADAMEngine(gpu, cfg, tensors, adamah_mod=A,
**kw)``, ``generate(token_ids, GenerationConfig, stream=..., **kw) -> (tokens,
stats)``, ``reset()``.  All device work goes through the backend object's C ABI.

What differs from the reference engine, by design:

* weights arrive as raw GGUF Q4_0 / Q4_K blocks and are uploaded as they are
  (``map_upload_gguf_blocks``), instead of being re-quantized into the Q4 map with
  per-group Python loops (engine.py:974-1116);
* the per-token loop of ~400 backend calls (engine.py:2971-3706) is one fused
  decoder step replayed from a CUDA graph, positions and sampled ids stay on the
  device, and the prompt is consumed without host work between tokens;
* extensions: several independent sequences per step (``generate_batch``), fp16
  paged KV cache, optional sliding-window mask.

Sampling modes (engine.py:3760-3805): ``gpu_matvec_argmax`` (greedy, fused LM head + arg-max),
``gpu_fused_topk`` (repeat penalty, top-k <= 64, nucleus and the draw on the device: 4 bytes come
back per token) and ``cpu`` (logits read back, the reference's host rule) for anything else.
"""
from __future__ import annotations

import ctypes
import math
import os
import time
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _lib
from . import constants as C
from .config import GenerationConfig, ModelConfig
from .synth import LAYER_MATS, QTensor

_MAT_KIND = {"attn_q": 0, "attn_k": 1, "attn_v": 2, "attn_output": 3, "ffn_gate": 4, "ffn_up": 5, "ffn_down": 6}
_NORM_KIND = {"attn_norm": 0, "post_attention_norm": 1, "ffn_norm": 2, "post_ffw_norm": 3, "attn_q_norm": 4, "attn_k_norm": 5}
_KIND_EMBD, _KIND_OUTPUT, _KIND_OUTPUT_NORM = 7, 8, 6

STEP_LM, STEP_LOGITS, STEP_DIRECT, STEP_CHAIN, STEP_SAMPLE = 1, 2, 4, 8, 16
SAMPLE_TOPK_MAX = 64           # candidates the device-side sampling step keeps (the reference's SAMPLE_TOPK_MAX)


def rope_tables(n_pos: int, head_dim: int, freq_base: float):
    """cos/sin of the rotary angles for positions 0..n_pos-1, formed exactly as the
    reference's numpy decoder forms them (tests/diagnostics/diag_inference.py:948-954):
    float32 inverse frequencies, float32 angle = float32(pos) * freq, float32 cos/sin."""
    half = head_dim // 2
    freqs = np.float32(1.0) / (freq_base ** (np.arange(0, half, dtype=np.float32) * np.float32(2.0) / head_dim))
    theta = np.arange(n_pos, dtype=np.float32)[:, None] * freqs[None, :]
    return np.ascontiguousarray(np.cos(theta).astype(np.float32)), np.ascontiguousarray(np.sin(theta).astype(np.float32))


class ADAMEngine:
    WS_MAP = 0                       # float32 map: norm weights (the reference's workspace map id)
    FIRST_WT_MAP = 1                 # GGUF-block maps start here (the reference's Q4 map id)

    def __init__(self, gpu, cfg: ModelConfig, tensors: Dict[str, object], adamah_mod=None, kv_cap: int = 1024,
                 max_batch: int = 1, kv_dtype: str = "f16", window: bool = False, page_size: int = 64,
                 n_pages: int = 0, verbose: bool = False, tile: bool = True, tp_rank: int = 0, tp_size: int = 1,
                 single_launch: Optional[bool] = None, **kw):
        self.gpu = gpu
        # One-sequence steps can run as ONE kernel launch per token (the persistent token kernel) or as a CUDA graph of
        # the per-operation kernels.  The graph is the default: at the Gemma-3-1B shape it is a few percent faster
        # (0.69 against 0.73 ms per token); ``single_launch=True`` or ADAM_B200_SINGLE_LAUNCH=1 selects the other.
        self.single_launch = bool(int(os.environ.get("ADAM_B200_SINGLE_LAUNCH", "0"))) if single_launch is None else bool(single_launch)
        self.A = adamah_mod if adamah_mod is not None else C
        self.cfg = cfg
        self.tensors = tensors
        self._kv_cap = int(kv_cap)
        self._max_batch = int(max_batch)
        self._lib = gpu._lib
        self.timing: Dict[str, float] = {}
        self.ws_map_id = self.WS_MAP
        if not getattr(gpu, "_has_decoder", False):
            raise RuntimeError("backend has no fused decoder (libadam_b200.so is out of date)")
        if cfg.head_dim != cfg.head_dim_kv:
            raise ValueError("head_dim and head_dim_kv must match")
        self._tied = "output.weight" not in tensors
        self._upload_all(verbose)
        desc = _lib.DecoderDesc(
            n_layer=cfg.n_layer, n_embd=cfg.n_embd, n_head=cfg.n_head, n_head_kv=cfg.n_head_kv, head_dim=cfg.head_dim,
            n_ff=cfg.n_ff, n_vocab=cfg.n_vocab, ffn_act=0 if cfg.ffn_act == "gelu" else 1,
            norm_eps=cfg.norm_eps, emb_scale=cfg.emb_scale, attn_softcap=cfg.attn_softcap, final_softcap=cfg.final_softcap,
            attn_scale=float(np.float32(1.0 / np.sqrt(cfg.head_dim))),
            sliding_window=cfg.sliding_window, global_every=6 if cfg.arch == "gemma3" else 0,
            max_batch=self._max_batch, kv_cap=self._kv_cap, kv_dtype={"f32": 0, "f16": 1}[kv_dtype], page_size=page_size,
            n_pages=n_pages, tp_rank=tp_rank, tp_size=tp_size, flags=(1 if window else 0) | (0 if tile else 2))
        did = ctypes.c_uint32(0)
        self._check(self._lib.adam_b200_decoder_create(ctypes.byref(desc), ctypes.byref(did)), "adam_b200_decoder_create")
        self._dec = int(did.value)
        self._bind_all()
        for which, base in ((0, cfg.rope_base_local), (1, cfg.rope_base_global)):
            cos_t, sin_t = rope_tables(self._kv_cap, cfg.head_dim, base)
            self._check(self._lib.adam_b200_decoder_set_rope(self._dec, which, cos_t.ctypes.data, sin_t.ctypes.data,
                                                             self._kv_cap, cfg.head_dim // 2), "adam_b200_decoder_set_rope")
        self._closed = False

    @classmethod
    def from_gguf(cls, gpu, path: str, verbose: bool = False, **kw) -> "ADAMEngine":
        """Engine over a .gguf file (role of adam/models/engine.py:118-170 with a streaming ``GGUFLoader``): the
        header, key/value table and tensor table are parsed on the host, the configuration comes from the
        metadata and the tensor shapes, and every matrix goes from the file to the GPU as raw blocks through
        pinned staging (``adam_b200_upload_gguf_file``) -- no host-side decode or re-quantization."""
        from .gguf_file import GGUFLoader
        loader = GGUFLoader(path).load(verbose=verbose)
        try:
            cfg = loader.model_config(verbose=verbose)
            kw.setdefault("kv_cap", min(int(cfg.n_ctx), 4096))
            eng = cls(gpu, cfg, loader.model_tensors(), verbose=verbose, **kw)
            eng.tensors = {}                 # views of the file mapping: not needed once the blocks are on the device
            eng.metadata = loader.metadata
        finally:
            loader.close()
        return eng

    # ---- helpers ---------------------------------------------------------------------
    def _check(self, rc: int, name: str):
        if rc != 0:
            raise RuntimeError(f"{name} failed with code {rc}: {_lib.last_error()}")

    def _upload_all(self, verbose: bool):
        """Weight layout (role of ``_build_layout`` / ``_upload_all``,
        engine.py:518, :929): one GGUF-block map per layer holding q,k,v back to back
        (so QKV is one GEMV), then o, gate, up, down; one map for token_embd (+ output);
        norm weights in the float32 map."""
        c, g = self.cfg, self.gpu
        t0 = time.perf_counter()
        self._mat_loc: Dict[str, tuple] = {}
        self._norm_loc: Dict[str, tuple] = {}
        layer_types = {t.ggml_type for n, t in self.tensors.items() if isinstance(t, QTensor) and n.startswith("blk.")}
        if len(layer_types) != 1 or not layer_types <= {C.GGML_TYPE_Q4_0, C.GGML_TYPE_Q4_K}:
            raise ValueError("the layers' matrices must share one block type, Q4_0 or Q4_K")
        self._ggml_type = layer_types.pop()
        next_map = self.FIRST_WT_MAP

        def put(map_id, names):
            """One GGUF-block map holding the named tensors back to back (they share a block type)."""
            kinds = {self.tensors[n].ggml_type for n in names}
            if len(kinds) != 1 or next(iter(kinds)) not in C.GGUF_MAP_DTYPE:
                raise ValueError(f"tensors {names} must share one supported block type (Q4_0, Q4_K, Q8_0, Q5_0)")
            total = sum(self.tensors[n].rows * self.tensors[n].cols for n in names)
            g.map_create_typed(map_id, C.GGUF_MAP_DTYPE[next(iter(kinds))], 1, total)
            off = 0
            for n in names:
                t = self.tensors[n]
                if hasattr(t.raw, "data_ptr"):          # CUDA tensor: blocks already on the device
                    g.upload_gguf_blocks(map_id, t.ggml_type, off, int(t.raw.data_ptr()), int(t.raw.numel()))
                elif getattr(t, "file", None) is not None:   # blocks still in a GGUF file: streamed through pinned staging
                    g.upload_gguf_file(map_id, t.ggml_type, off, t.file[0], t.file[1], t.nbytes)
                else:
                    g.upload_gguf_blocks(map_id, t.ggml_type, off, t.raw)
                self._mat_loc[n] = (map_id, off, t.rows, t.cols)
                off += t.rows * t.cols

        # token_embd (Q8_0 / Q5_0 in many real files) and output.weight share a map only when their types agree
        head = ["token_embd.weight"] + ([] if self._tied else ["output.weight"])
        if len({self.tensors[n].ggml_type for n in head}) == 1:
            put(next_map, head)
            next_map += 1
        else:
            for n in head:
                put(next_map, [n])
                next_map += 1
        for L in range(c.n_layer):
            put(next_map, [f"blk.{L}.{m}.weight" for m in LAYER_MATS])
            next_map += 1
        self._n_wt_maps = next_map - self.FIRST_WT_MAP
        norms = [(n, t) for n, t in self.tensors.items() if isinstance(t, np.ndarray)]
        total = sum(int(t.size) for _, t in norms)
        g.map_create_typed(self.WS_MAP, C.DTYPE_F32, 1, max(total, 16))
        off = 0
        for n, t in norms:
            g.scatter_contiguous(self.WS_MAP, off, np.ascontiguousarray(t, np.float32).reshape(-1))
            self._norm_loc[n] = (self.WS_MAP, off, int(t.size))
            off += int(t.size)
        if verbose:
            print(f"[GPU] uploaded {len(self._mat_loc)} matrices, {len(norms)} norm vectors in {time.perf_counter() - t0:.2f}s")

    def _bind_all(self):
        c, lib, d = self.cfg, self._lib, self._dec
        m = self._mat_loc["token_embd.weight"]
        self._check(lib.adam_b200_decoder_bind_matrix(d, 0, _KIND_EMBD, m[0], m[1], m[2], m[3]), "bind token_embd")
        if not self._tied:
            m = self._mat_loc["output.weight"]
            self._check(lib.adam_b200_decoder_bind_matrix(d, 0, _KIND_OUTPUT, m[0], m[1], m[2], m[3]), "bind output")
        n = self._norm_loc["output_norm.weight"]
        self._check(lib.adam_b200_decoder_bind_norm(d, 0, _KIND_OUTPUT_NORM, n[0], n[1], n[2]), "bind output_norm")
        for L in range(c.n_layer):
            for name, kind in _MAT_KIND.items():
                m = self._mat_loc[f"blk.{L}.{name}.weight"]
                self._check(lib.adam_b200_decoder_bind_matrix(d, L, kind, m[0], m[1], m[2], m[3]), f"bind blk.{L}.{name}")
            for name, kind in _NORM_KIND.items():
                key = f"blk.{L}.{name}.weight"
                if key in self._norm_loc:
                    n = self._norm_loc[key]
                    self._check(lib.adam_b200_decoder_bind_norm(d, L, kind, n[0], n[1], n[2]), f"bind {key}")

    # ---- low-level stepping ------------------------------------------------------------
    def begin(self, prompts: Sequence[Sequence[int]], reserve: Sequence[int]):
        """Start ``len(prompts)`` sequences at position 0 (host prompts are copied to the device here)."""
        lens = np.array([len(p) for p in prompts], np.uint32)
        flat = np.ascontiguousarray(np.concatenate([np.asarray(p, np.int32) for p in prompts]), np.int32)
        res = np.asarray(reserve, np.uint32)
        self._check(self._lib.adam_b200_decoder_begin(self._dec, len(prompts), flat.ctypes.data, lens.ctypes.data, res.ctypes.data),
                    "adam_b200_decoder_begin")
        self._batch = len(prompts)
        self._h2d_bytes = flat.nbytes + lens.nbytes + res.nbytes

    def step(self, n_steps: int = 1, lm_head: bool = True, logits: bool = False, direct: bool = False, chain: Optional[bool] = None,
             sample: bool = False):
        """``chain=True`` runs the chain of per-operation kernels, ``chain=False`` the single-launch token kernel where the
        model is eligible for it; by default the engine's ``single_launch`` setting decides;
        ``sample=True`` draws the token on the device with the rule given to ``set_sampling``."""
        if chain is None:
            chain = not self.single_launch
        flags = ((STEP_LM if lm_head else 0) | (STEP_LOGITS if logits else 0) | (STEP_DIRECT if direct else 0) | (STEP_CHAIN if chain else 0)
                 | (STEP_SAMPLE if sample else 0))
        self._check(self._lib.adam_b200_decoder_step(self._dec, n_steps, flags), "adam_b200_decoder_step")

    def set_sampling(self, top_k: int, top_p: float, temperature: float, repeat_penalty: float, repeat_on_prompt: bool, seed: int):
        self._check(self._lib.adam_b200_decoder_set_sampling(self._dec, int(top_k), float(top_p), float(temperature), float(repeat_penalty),
                                                             1 if repeat_on_prompt else 0, int(seed) & 0xFFFFFFFFFFFFFFFF),
                    "adam_b200_decoder_set_sampling")

    def prefill(self, n_tokens: int):
        """Consume the next ``n_tokens`` prompt tokens of every sequence, many positions per pass
        (same results as ``step(n_tokens, lm_head=False)``)."""
        if n_tokens > 0:
            self._check(self._lib.adam_b200_decoder_prefill(self._dec, int(n_tokens)), "adam_b200_decoder_prefill")

    def read_state(self):
        pos = np.empty(self._max_batch, np.int32)
        tok = np.empty(self._max_batch, np.int32)
        self._check(self._lib.adam_b200_decoder_read_state(self._dec, pos.ctypes.data, tok.ctypes.data), "adam_b200_decoder_read_state")
        return pos, tok

    def read_log(self, seq: int, first_pos: int, n: int) -> np.ndarray:
        out = np.empty(n, np.int32)
        self._check(self._lib.adam_b200_decoder_read_log(self._dec, seq, first_pos, n, out.ctypes.data), "adam_b200_decoder_read_log")
        return out

    def read_logits(self, seq: int = 0) -> np.ndarray:
        out = np.empty(self.cfg.n_vocab, np.float32)
        self._check(self._lib.adam_b200_decoder_read_logits(self._dec, seq, out.ctypes.data), "adam_b200_decoder_read_logits")
        return out

    def read_buffer(self, what: int, n: int, seq: int = 0) -> np.ndarray:
        out = np.empty(n, np.float32)
        self._check(self._lib.adam_b200_decoder_read_buffer(self._dec, what, seq, out.ctypes.data, n), "adam_b200_decoder_read_buffer")
        return out

    def token_trace(self, layer: int = 1, phase: int = 2) -> np.ndarray:
        """One token step on the single-launch token kernel with per-phase SM clock stamps: ``[n_cta, 32]``
        (slots 0..9 = phases of ``layer``, 10..13 = LM head, 16..22 = inside product ``phase`` of that layer;
        diagnostics)."""
        out = np.zeros((256, 32), np.int64)
        n = ctypes.c_uint32(0)
        self._check(self._lib.adam_b200_decoder_token_trace(self._dec, int(layer) | (int(phase) << 16), out.ctypes.data, ctypes.byref(n)), "adam_b200_decoder_token_trace")
        return out[:int(n.value)]

    def step_trace(self, layer: Optional[int] = None):
        """Diagnostics build only (``python -m adam_b200.build --step-trace``).  ``step_trace(layer)`` arms the trace
        for one layer of the default one-sequence step; ``step_trace()`` returns the stamps of the latest step in
        nanoseconds: ``(products[4, 8, 8], attention[32, 8])`` (slot meanings: ``adam_b200_decoder_step_trace``)."""
        if layer is not None:
            self._check(self._lib.adam_b200_decoder_step_trace(self._dec, int(layer), None, 0), "adam_b200_decoder_step_trace")
            return None
        out = np.zeros(512, np.int64)
        self._check(self._lib.adam_b200_decoder_step_trace(self._dec, 0, out.ctypes.data, 512), "adam_b200_decoder_step_trace")
        return out[:256].reshape(4, 8, 8), out[256:512].reshape(32, 8)

    def logits_trace(self, tokens: Sequence[int], direct: bool = True) -> np.ndarray:
        """Teacher-forced pass over ``tokens``: the soft-capped logits after every
        position, ``[len(tokens), n_vocab]`` (for parity checks)."""
        self.begin([tokens], [len(tokens)])
        out = np.empty((len(tokens), self.cfg.n_vocab), np.float32)
        for i in range(len(tokens)):
            self.step(1, lm_head=True, logits=True, direct=direct)
            out[i] = self.read_logits(0)
        return out

    # ---- generate ----------------------------------------------------------------------
    def _select_sampling_mode(self, config: GenerationConfig) -> str:
        """'gpu_matvec_argmax' (fused LM head + arg-max, ids stay on the device) for greedy decoding without
        a repeat penalty -- the reference refuses that mode when a penalty is set
        (engine.py:1876-1881) -- else 'cpu': logits are read back and sampled on the host
        (engine.py:3760-3805)."""
        if config.is_greedy() and config.repeat_penalty == 1.0:
            return "gpu_matvec_argmax"
        # LM head + top-k with repeat penalty + nucleus + draw, all on the device (the reference's
        # 'gpu_fused_topk', engine.py:3403-3512): for up to SAMPLE_TOPK_MAX candidates
        if config.is_greedy() or 0 < config.top_k <= SAMPLE_TOPK_MAX:
            return "gpu_fused_topk"
        return "cpu"

    @staticmethod
    def _sample(logits: np.ndarray, cfg: GenerationConfig, prev, rng) -> int:
        """Host-side sampling, the reference's rule (engine.py:3711-3729): repeat penalty on the last 64
        history ids, temperature, top-k mask, soft-max, nucleus cut, categorical draw."""
        logits = logits.astype(np.float32).copy()
        if cfg.repeat_penalty != 1.0 and prev:
            for t in set(prev[-64:]):
                if t < len(logits):
                    logits[t] = logits[t] / cfg.repeat_penalty if logits[t] > 0 else logits[t] * cfg.repeat_penalty
        if cfg.temperature <= 0:
            return int(np.argmax(logits))
        logits /= np.float32(cfg.temperature)
        if cfg.top_k > 0:
            tk = min(cfg.top_k, len(logits))
            ti = np.argpartition(logits, -tk)[-tk:]
            m = np.full_like(logits, -np.inf)
            m[ti] = logits[ti]
            logits = m
        p = np.exp(logits - np.max(logits))
        p /= p.sum()
        if cfg.top_p < 1.0:
            si = np.argsort(p)[::-1]
            cs = np.cumsum(p[si])
            co = int(np.searchsorted(cs, cfg.top_p)) + 1
            m = np.zeros_like(p)
            m[si[:co]] = p[si[:co]]
            p = m / m.sum()
        return int(rng.choice(len(p), p=p.astype(np.float64) / float(p.astype(np.float64).sum())))

    def set_tokens(self, tokens: Sequence[int]):
        arr = np.ascontiguousarray(np.asarray(tokens, np.int32))
        self._check(self._lib.adam_b200_decoder_set_tokens(self._dec, arr.ctypes.data), "adam_b200_decoder_set_tokens")

    def continue_with(self, prompt: Sequence[int], reserve: int, n_reuse: int):
        """Keep the active sequence's cache and restart at position ``n_reuse`` with a new prompt whose first
        ``n_reuse`` tokens are the cached ones."""
        arr = np.ascontiguousarray(np.asarray(prompt, np.int32))
        self._check(self._lib.adam_b200_decoder_continue(self._dec, arr.ctypes.data, len(arr), int(reserve), int(n_reuse)),
                    "adam_b200_decoder_continue")
        self._batch = 1
        self._h2d_bytes = arr.nbytes

    def generate_batch(self, prompts: Sequence[Sequence[int]], config: Optional[GenerationConfig] = None, sync_every: int = 1,
                       reuse_prefix: int = 0):
        """Greedy generation for independent sequences (one step advances all of them).
        Returns (list of token lists, stats).  The host reads every step's ids (as the reference does,
        engine.py:1979) but asynchronously: up to ``sync_every`` (1..3) later steps are already queued
        while it looks at them, so a sequence may run that many steps past its EOS before the loop stops."""
        config = config or GenerationConfig(top_k=1, repeat_penalty=1.0)
        mode = self._select_sampling_mode(config)
        if len(prompts) == 0 or len(prompts) > self._max_batch:
            raise ValueError(f"need 1..{self._max_batch} prompts")
        lens = [len(p) for p in prompts]
        for n in lens:
            total_needed = n + config.max_tokens
            if n == 0:
                raise ValueError("empty prompt")
            if total_needed > self._kv_cap:
                raise RuntimeError(f"KV cache too small: need {total_needed} tokens but kv_cap={self._kv_cap}. "
                                   f"Reinitialize with kv_cap>={total_needed}.")
        g = self.gpu
        g.reset_native_stats()
        tp = time.perf_counter()
        # all sequences step together, so each needs room up to the longest one's end
        max_len, min_len = max(lens), min(lens)
        # reuse_prefix (one sequence): the first tokens' keys and values are still cached from the previous call
        reuse = int(reuse_prefix or 0)
        if reuse >= min_len or len(prompts) != 1:
            reuse = 0
        if reuse:
            self.continue_with(prompts[0], max_len + config.max_tokens, reuse)
        else:
            self.begin(prompts, [max_len + config.max_tokens] * len(prompts))
        # prefill: every sequence consumes its own prompt; shorter ones start decoding earlier
        with g.batch():
            if min_len - 1 > reuse:
                self.prefill(min_len - 1 - reuse)
        t_pre = time.perf_counter() - tp
        td = time.perf_counter()
        n_steps = (max_len - min_len) + config.max_tokens          # steps that run the LM head
        eos = set(int(e) for e in config.eos_token_ids)
        steps_done = 0
        d2h = 0
        sampled: List[List[int]] = [[] for _ in prompts]
        if mode == "cpu":
            # one step at a time: read the logits of every sequence that is past its prompt, draw its token on
            # the host and hand it back as the next step's input
            rng = np.random.default_rng(config.seed)
            finished = [False] * len(prompts)
            while steps_done < n_steps and not all(finished):
                with g.batch():
                    self.step(1, lm_head=True, logits=True)
                new_pos = min_len + steps_done              # position of the token this step produced
                steps_done += 1
                toks = np.zeros(len(prompts), np.int32)
                for b, n in enumerate(lens):
                    if finished[b] or new_pos < n:
                        continue
                    lg = self.read_logits(b)
                    d2h += lg.nbytes
                    hist = (list(prompts[b]) if config.repeat_on_prompt else []) + sampled[b]
                    t = self._sample(lg, config, hist, rng)
                    if t in eos:
                        finished[b] = True
                        continue
                    sampled[b].append(t)
                    toks[b] = t
                    if len(sampled[b]) >= config.max_tokens:
                        finished[b] = True
                self.set_tokens(toks)
        if mode != "cpu":
            # Greedy: the sampled id feeds the next step on the device, so the host only watches for EOS.  The
            # ids of a step are fetched asynchronously while up to ``sync_every`` later steps are already queued.
            import collections
            import ctypes as _ct
            finished = [False] * len(prompts)
            pending = collections.deque()
            buf = np.zeros(self._max_batch, np.int32)

            def consume(step_no, slot):
                nonlocal d2h
                self._check(self._lib.adam_b200_decoder_tokens_wait(self._dec, slot, buf.ctypes.data), "adam_b200_decoder_tokens_wait")
                d2h += 4 * len(prompts)
                for b, n in enumerate(lens):
                    if finished[b] or min_len + step_no < n:          # still inside its prompt
                        continue
                    t = int(buf[b])
                    if t in eos:
                        finished[b] = True
                        continue
                    sampled[b].append(t)
                    if len(sampled[b]) >= config.max_tokens:
                        finished[b] = True

            depth = max(1, int(sync_every))
            fused = mode == "gpu_fused_topk"
            if fused:
                seed = config.seed if config.seed is not None else int.from_bytes(__import__("os").urandom(8), "little")
                greedy = config.is_greedy()
                self.set_sampling(1 if greedy else config.top_k, config.top_p, 0.0 if greedy else config.temperature,
                                  config.repeat_penalty, config.repeat_on_prompt, seed)
            with g.batch():
                while steps_done < n_steps and not all(finished):
                    self.step(1, lm_head=True, sample=fused)
                    slot = _ct.c_uint32(0)
                    self._check(self._lib.adam_b200_decoder_tokens_async(self._dec, _ct.byref(slot)), "adam_b200_decoder_tokens_async")
                    pending.append((steps_done, int(slot.value)))
                    steps_done += 1
                    if len(pending) > min(depth, 3):
                        consume(*pending.popleft())
                while pending:
                    consume(*pending.popleft())
        t_dec = time.perf_counter() - td
        # Kernels record trouble (a position past the reserved pages, a bounded wait that ran out, a
        # token id outside the vocabulary) in a device word instead of faulting: tokens produced
        # after that are not trustworthy, so say so rather than return them.
        err = g.device_error()
        if err:
            raise RuntimeError(f"device error word {err:#x} after generation (1 = index outside its buffer, "
                               f"2 = a bounded device-side wait ran out, 4 = token id outside the vocabulary)")
        outs: List[List[int]] = []
        for b, n in enumerate(lens):
            outs.append(sampled[b])
        ng = sum(len(o) for o in outs)
        stats = {
            "n_prompt": sum(lens), "n_prompt_total": sum(lens), "n_prompt_reused": reuse, "n_prompt_prefilled": sum(lens) - reuse,
            "n_gen": ng, "prefill_s": t_pre, "decode_s": t_dec, "total_s": time.perf_counter() - tp,
            "prefill_tps": (sum(lens) - len(lens)) / t_pre if t_pre > 0 else 0.0,
            "decode_tps": ng / t_dec if t_dec > 0 else 0.0,
            "avg_ms": 1000.0 * t_dec / max(1, steps_done), "sampling_mode": mode, "batch": len(prompts),
            "h2d_bytes": self._h2d_bytes, "d2h_bytes": d2h, "timing": dict(self.timing),
            "native_stats": g.get_native_stats(), "trace_summary": {}, "trace_steps": [],
        }
        return outs, stats

    def generate(self, token_ids, config: Optional[GenerationConfig] = None, stream: bool = False, **kw):
        """Single sequence; same return shape as the reference: (tokens, stats dict)
        (engine.py:3810-3944).  Stops at the first id in ``config.eos_token_ids``."""
        outs, stats = self.generate_batch([list(token_ids)], config, sync_every=int(kw.get("sync_every", 1)),
                                          reuse_prefix=int(kw.get("reuse_prefix", 0) or 0))
        return outs[0], stats

    def reset(self):
        """Kept for interface parity (engine.py:3946): sequences restart in ``begin``."""
        self.timing = {}

    def close(self):
        if not self._closed:
            self._closed = True
            self._lib.adam_b200_decoder_destroy(self._dec)
            for mid in range(self.FIRST_WT_MAP, self.FIRST_WT_MAP + self._n_wt_maps):
                self.gpu.map_destroy(mid)
