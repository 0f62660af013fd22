"""Model and generation configuration, field-compatible with the reference
engine's ``ModelConfig`` / ``GenerationConfig`` (adam/models/engine.py:24-111),
plus the named shapes used by the benchmark configurations."""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Optional


@dataclass
class GenerationConfig:
    """Same fields and defaults as adam/models/engine.py:24-29.  Greedy decoding
    (``top_k == 1`` or ``temperature == 0``) stays on the device; anything else
    is sampled on the host from the logits."""
    max_tokens: int = 128
    temperature: float = 0.8
    top_k: int = 40
    top_p: float = 0.95
    repeat_penalty: float = 1.1
    seed: Optional[int] = None
    repeat_on_prompt: bool = False
    eos_token_ids: tuple = (1,)

    def is_greedy(self) -> bool:
        return self.top_k == 1 or self.temperature <= 0.0


@dataclass
class ModelConfig:
    """Same fields as adam/models/engine.py:31-50."""
    arch: str = "llama"
    n_vocab: int = 32000
    n_ctx: int = 4096
    n_embd: int = 4096
    n_head: int = 32
    n_head_kv: int = 32
    n_layer: int = 32
    n_ff: int = 11008
    head_dim: int = 128
    head_dim_kv: int = 128
    norm_eps: float = 1e-6
    rope_base_global: float = 10000.0
    rope_base_local: float = 10000.0
    sliding_window: int = 0
    chat_template: Optional[str] = None
    ffn_act: str = "silu"
    emb_scale: float = 1.0
    attn_softcap: float = 0.0
    final_softcap: float = 0.0

    # ggml feed_forward.activation_type codes and the architectures whose gate is GELU (adam/models/engine.py:46-50)
    _GGML_ACT = {8: "gelu", 9: "gelu", 10: "silu", 6: "relu"}
    _GELU_ARCHS = frozenset({"gemma", "gemma2", "gemma3", "gpt2", "gptj", "gptneox", "falcon", "starcoder", "starcoder2", "refact"})

    @classmethod
    def from_gguf_metadata(cls, metadata: dict, verbose: bool = False) -> "ModelConfig":
        """Configuration from a GGUF key/value table, key for key as the reference reads it
        (adam/models/engine.py:56-111): ``<arch>.<key>`` first, then the bare key, then the
        default; Gemma-3 defaults for the sliding window (512), rotary bases (1e6, local =
        global unless ``rope.local_freq_base`` is present) and soft caps (50 / 30 when the file
        omits them).  ``head_dim`` here is ``n_embd // n_head``; ``detect_dims`` corrects it
        from the tensor shapes, as the reference engine does after loading."""
        arch = metadata.get("general.architecture", "llama")
        c = cls(arch=arch)

        def g(key, default):
            return metadata.get(f"{arch}.{key}", metadata.get(key, default))

        c.n_ctx = g("context_length", 4096)
        c.n_layer = g("block_count", 32)
        c.n_embd = g("embedding_length", 4096)
        c.n_ff = g("feed_forward_length", c.n_embd * 4)
        c.n_head = g("attention.head_count", 32)
        c.n_head_kv = g("attention.head_count_kv", c.n_head)
        c.norm_eps = g("attention.layer_norm_rms_epsilon", 1e-6)
        c.n_vocab = g("vocab_size", metadata.get("tokenizer.ggml.tokens", [None]))
        if isinstance(c.n_vocab, list):
            c.n_vocab = len(c.n_vocab)
        c.chat_template = metadata.get("tokenizer.chat_template")
        c.head_dim = c.n_embd // c.n_head if c.n_head > 0 else 128
        c.head_dim_kv = c.n_embd // c.n_head_kv if c.n_head_kv > 0 else c.head_dim
        if arch == "gemma3":
            c.sliding_window = g("attention.sliding_window", 512)
            c.rope_base_global = g("rope.freq_base", 1e6)
            c.rope_base_local = g("rope.local_freq_base", c.rope_base_global)
        else:
            c.sliding_window = g("attention.sliding_window", 0)
            c.rope_base_global = g("rope.freq_base", 10000.0)
            c.rope_base_local = c.rope_base_global
        act = g("feed_forward.activation_type", None)
        c.ffn_act = cls._GGML_ACT.get(act, "silu") if act is not None else ("gelu" if arch in cls._GELU_ARCHS else "silu")
        c.emb_scale = math.sqrt(c.n_embd) if arch.startswith("gemma") else 1.0
        c.attn_softcap = float(g("attention.logit_softcapping", 0.0))
        c.final_softcap = float(g("logit_softcapping", 0.0))
        if arch == "gemma3":
            c.attn_softcap = c.attn_softcap or 50.0
            c.final_softcap = c.final_softcap or 30.0
        if verbose:
            print(f"[CFG] {metadata.get('general.name', arch)} ({arch}): L={c.n_layer} E={c.n_embd} H={c.n_head} KV={c.n_head_kv} "
                  f"FF={c.n_ff} V={c.n_vocab} act={c.ffn_act} emb_scale={c.emb_scale:.2f}")
        return c

    def detect_dims(self, tensor_shapes: dict) -> "ModelConfig":
        """Head sizes, vocabulary, width and FFN width from the tensor shapes (``[out, in]`` order), which
        win over the metadata (role of ``_detect_dims``, adam/models/engine.py:477-500: Gemma-3 heads are
        wider than ``n_embd / n_head``)."""
        for name, sh in tensor_shapes.items():
            if "attn_q.weight" in name and len(sh) == 2:
                self.head_dim = (sh[1] if sh[0] == self.n_embd else sh[0]) // self.n_head
                break
        for name, sh in tensor_shapes.items():
            if "attn_k.weight" in name and len(sh) == 2:
                self.head_dim_kv = (sh[1] if sh[0] == self.n_embd else sh[0]) // self.n_head_kv
                break
        if "token_embd.weight" in tensor_shapes:
            sh = tensor_shapes["token_embd.weight"]
            self.n_vocab, self.n_embd = max(sh), min(sh)
        for name, sh in tensor_shapes.items():
            if "ffn_gate.weight" in name and len(sh) == 2:
                self.n_ff = max(sh) if min(sh) == self.n_embd else min(sh)
                break
        return self

    def is_global(self, L: int) -> bool:
        """Gemma-3 interleaves 5 local layers with 1 global one
        (adam/models/engine.py:52-54); every other arch is all-global."""
        if self.arch == "gemma3":
            return (L + 1) % 6 == 0
        return True

    def rope_base(self, L: int) -> float:
        return self.rope_base_global if self.is_global(L) else self.rope_base_local


def gemma3_shape(n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab,
                 sliding_window, n_ctx=4096) -> ModelConfig:
    """Gemma-3 constants the reference hard-codes or derives
    (adam/models/engine.py:75-78, :93, :100-102)."""
    return ModelConfig(
        arch="gemma3", n_vocab=n_vocab, n_ctx=n_ctx, n_embd=n_embd, n_head=n_head,
        n_head_kv=n_head_kv, n_layer=n_layer, n_ff=n_ff, head_dim=head_dim,
        head_dim_kv=head_dim, norm_eps=1e-6, rope_base_global=1e6, rope_base_local=1e4,
        sliding_window=sliding_window, ffn_act="gelu", emb_scale=math.sqrt(n_embd),
        attn_softcap=50.0, final_softcap=30.0)


def gemma3_1b() -> ModelConfig:
    return gemma3_shape(26, 1152, 4, 1, 256, 6912, 262144, 512)


def gemma3_27b() -> ModelConfig:
    return gemma3_shape(62, 5376, 32, 16, 128, 21504, 262144, 1024)


def tiny_gemma3(n_layer=3, n_embd=256, n_head=4, n_head_kv=1, head_dim=64, n_ff=512,
                n_vocab=1024, sliding_window=0) -> ModelConfig:
    """A small Gemma-3-shaped configuration for parity tests."""
    return gemma3_shape(n_layer, n_embd, n_head, n_head_kv, head_dim, n_ff, n_vocab, sliding_window)


def with_layers(cfg: ModelConfig, n_layer: int) -> ModelConfig:
    return replace(cfg, n_layer=n_layer)
