"""Numpy restatement of the reference's CPU decoder (oracle).

Test infrastructure: see ``oracle/__init__.py`` for who may import this.

Follows ``forward_cpu`` and its helpers in
tests/diagnostics/diag_inference.py:934-1037 operation by operation, in float32,
on weights already decoded to float32 (the reference pre-decodes them at
:966-969).  With the default flags it reproduces the greedy token ids of the
unmodified reference (pinned by the fixtures under ``tests/golden/``).

Flagged extensions, none of which exists in the reference (parity unpinned):
``window=True`` applies the sliding-window mask on non-global layers;
``kv_dtype=np.float16`` rounds K and V to fp16 when they are stored;
``tp_size>1`` sums the row-sharded projections (o, down) as per-rank partial
sums added in rank order, as a tensor-parallel run does.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np

from . import q4_blocks


def rms_norm(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """``(x / sqrt(mean(x^2) + eps)) * w`` -- diag_inference.py:938-939."""
    rms = np.sqrt(np.mean(x ** 2) + eps)
    return (x / rms) * w


def gelu_tanh(x: np.ndarray) -> np.ndarray:
    """diag_inference.py:941-943."""
    return np.float32(0.5) * x * (np.float32(1.0) + np.tanh(
        np.float32(np.sqrt(2.0 / np.pi)) * (x + np.float32(0.044715) * x ** 3)))


def silu(x: np.ndarray) -> np.ndarray:
    """diag_inference.py:945-946."""
    return x * (np.float32(1.0) / (np.float32(1.0) + np.exp(-x.clip(-80, 80))))


def rope_angles(pos: int, head_dim: int, freq_base: float):
    """cos/sin of the rotation angles for one position, computed exactly as
    diag_inference.py:948-954 does (float32 throughout)."""
    half = head_dim // 2
    freqs = np.float32(1.0) / (freq_base ** (
        np.arange(0, half, dtype=np.float32) * np.float32(2.0) / head_dim))
    theta = np.float32(pos) * freqs
    return np.cos(theta).astype(np.float32), np.sin(theta).astype(np.float32)


def rope_half(x: np.ndarray, pos: int, freq_base: float) -> np.ndarray:
    """Half-split RoPE on rows of ``x`` -- diag_inference.py:948-956."""
    n, d = x.shape
    half = d // 2
    c_t, s_t = rope_angles(pos, d, freq_base)
    x0, x1 = x[:, :half], x[:, half:]
    return np.concatenate([x0 * c_t - x1 * s_t, x0 * s_t + x1 * c_t], axis=1)


def attention_head(q_h, K_h, V_h, scale, softcap):
    """One query head over its cached keys/values -- diag_inference.py:1003-1012."""
    sc = q_h @ K_h.T * scale
    if softcap > 0:
        cap = np.float32(softcap)
        sc = np.tanh(sc / cap) * cap
    sc -= sc.max()
    w_ = np.exp(sc)
    w_ /= w_.sum()
    return w_ @ V_h


def dequant_model(tensors) -> Dict[str, np.ndarray]:
    """Decode every quantized tensor of a synthetic model to float32."""
    out = {}
    for name, t in tensors.items():
        if isinstance(t, np.ndarray):
            out[name] = t.astype(np.float32)
        else:
            out[name] = q4_blocks.dequant(t.raw, t.ggml_type, t.rows, t.cols)
    return out


class OracleDecoder:
    """Single-sequence greedy decoder on float32 weights."""

    def __init__(self, cfg, tensors_f32: Dict[str, np.ndarray], kv_cap: int,
                 window: bool = False, kv_dtype=np.float32, tp_size: int = 1, tp_ff_bounds=None):
        self.c = cfg
        self.t = tensors_f32
        self.kv_cap = kv_cap
        self.window = window
        self.kv_dtype = np.dtype(kv_dtype)
        self.tp = tp_size
        # K boundaries of the down-projection shards (len tp_size + 1); equal shards when None
        self.tp_ff_bounds = None if tp_ff_bounds is None else [int(b) for b in tp_ff_bounds]
        c = cfg
        # diag_inference.py:958-961
        self.k_cache = np.zeros((c.n_layer, c.n_head_kv, kv_cap, c.head_dim_kv), np.float32)
        self.v_cache = np.zeros((c.n_layer, c.n_head_kv, kv_cap, c.head_dim_kv), np.float32)
        self.trace: Optional[dict] = None

    def reset(self):
        self.k_cache[:] = 0
        self.v_cache[:] = 0

    def _row_sharded(self, x: np.ndarray, W: np.ndarray, bounds=None) -> np.ndarray:
        """``x @ W.T`` ; with tp_size>1 the K dimension is split into contiguous
        shards (equal ones unless ``bounds`` gives the boundaries) whose partial
        products are added in rank order."""
        if self.tp == 1:
            return x @ W.T
        K = x.shape[0]
        if bounds is None:
            step = K // self.tp
            bounds = [r * step for r in range(self.tp)] + [K]
        acc = None
        for r in range(self.tp):
            a, b = bounds[r], bounds[r + 1]
            part = x[a:b] @ W[:, a:b].T
            acc = part if acc is None else acc + part
        return acc

    def forward(self, tok_id: int, pos: int, want_logits: bool = True):
        c = self.c
        T = self.t
        eps = c.norm_eps
        gs = max(1, c.n_head // c.n_head_kv)
        seq_len = pos + 1
        tr = self.trace
        # diag_inference.py:975-977
        hidden = T["token_embd.weight"][tok_id].copy()
        if c.emb_scale != 1.0:
            hidden *= np.float32(c.emb_scale)
        if tr is not None:
            tr["embed"] = hidden.copy()
        for L in range(c.n_layer):
            p = f"blk.{L}"
            gl = c.is_global(L)
            freq = c.rope_base_global if gl else c.rope_base_local
            normed = rms_norm(hidden, T[f"{p}.attn_norm.weight"], eps)
            q = (normed @ T[f"{p}.attn_q.weight"].T).reshape(c.n_head, c.head_dim)
            k = (normed @ T[f"{p}.attn_k.weight"].T).reshape(c.n_head_kv, c.head_dim_kv)
            v = (normed @ T[f"{p}.attn_v.weight"].T).reshape(c.n_head_kv, c.head_dim_kv)
            qnn = f"{p}.attn_q_norm.weight"
            if qnn in T:
                qnw = T[qnn]
                knw = T[f"{p}.attn_k_norm.weight"]
                for i in range(c.n_head):
                    q[i] = rms_norm(q[i], qnw, eps)
                for i in range(c.n_head_kv):
                    k[i] = rms_norm(k[i], knw, eps)
            q = rope_half(q, pos, freq)
            k = rope_half(k, pos, freq)
            if self.kv_dtype != np.float32:           # extension: low-precision KV
                k = k.astype(self.kv_dtype).astype(np.float32)
                v = v.astype(self.kv_dtype).astype(np.float32)
            self.k_cache[L, :, pos, :] = k
            self.v_cache[L, :, pos, :] = v
            start = 0
            if self.window and not gl and c.sliding_window > 0:   # extension
                start = max(0, seq_len - c.sliding_window)
            scale = np.float32(1.0 / np.sqrt(c.head_dim))
            attn_out = np.zeros((c.n_head, c.head_dim_kv), np.float32)
            for h in range(c.n_head):
                kv_h = h // gs
                attn_out[h] = attention_head(q[h], self.k_cache[L, kv_h, start:seq_len, :],
                                             self.v_cache[L, kv_h, start:seq_len, :],
                                             scale, c.attn_softcap)
            o_proj = self._row_sharded(attn_out.reshape(-1), T[f"{p}.attn_output.weight"])
            pan = f"{p}.post_attention_norm.weight"
            if pan in T:
                o_proj = rms_norm(o_proj, T[pan], eps)
            hidden = hidden + o_proj
            normed2 = rms_norm(hidden, T[f"{p}.ffn_norm.weight"], eps)
            gate = normed2 @ T[f"{p}.ffn_gate.weight"].T
            up = normed2 @ T[f"{p}.ffn_up.weight"].T
            gate = gelu_tanh(gate) if c.ffn_act == "gelu" else silu(gate)
            ffn = self._row_sharded(gate * up, T[f"{p}.ffn_down.weight"], self.tp_ff_bounds)
            pfn = f"{p}.post_ffw_norm.weight"
            if pfn in T:
                ffn = rms_norm(ffn, T[pfn], eps)
            hidden = hidden + ffn
            if tr is not None:
                tr[f"hidden.{L}"] = hidden.copy()
                if L == 0:
                    tr["q0"] = q.copy(); tr["k0"] = k.copy(); tr["v0"] = v.copy()
                    tr["attn0"] = attn_out.copy()
        if not want_logits:
            return None
        normed_final = rms_norm(hidden, T["output_norm.weight"], eps)
        if tr is not None:
            tr["final_norm"] = normed_final.copy()
        if "output.weight" in T:                      # diag_inference.py:1029-1033
            logits = normed_final @ T["output.weight"].T
        else:
            logits = T["token_embd.weight"] @ normed_final
        if c.final_softcap > 0:
            cap = np.float32(c.final_softcap)
            logits = np.tanh(logits / cap) * cap
        return logits

    def generate(self, prompt: Sequence[int], n_tokens: int, eos_ids: Sequence[int] = (),
                 keep_logits: bool = False):
        """Token-by-token prefill then greedy decode -- diag_inference.py:1045-1061.
        Returns (token ids, list of the logits each id was picked from)."""
        self.reset()
        logits = None
        for i, t in enumerate(prompt):
            logits = self.forward(int(t), i, want_logits=(i == len(prompt) - 1))
        out: List[int] = []
        all_logits = []
        pos = len(prompt)
        for _ in range(n_tokens):
            nt = int(np.argmax(logits))
            if nt in eos_ids:
                break
            out.append(nt)
            if keep_logits:
                all_logits.append(logits.copy())
            logits = self.forward(nt, pos)
            pos += 1
        return out, all_logits
