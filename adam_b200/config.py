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
