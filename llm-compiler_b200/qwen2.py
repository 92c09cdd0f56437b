"""Qwen2 configuration and seeded synthetic weights for the serving engine.

Mirrors the fixture side of the reference (Qwen2CompatConfig, qwen2.py:14-47, and the
parameter layout of StatefulQwen2ForCausalLM, qwen2.py:392-478): same field names, same
state_dict names, same parameter order, so that seeded weights made here are the ones the
reference model holds after `torch.manual_seed(seed)` + `normal_(0, 0.02)` over
`model.parameters()`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterator, Tuple

import torch


@dataclass(frozen=True)
class Qwen2Config:
    hidden_size: int = 64
    intermediate_size: int = 128
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 2
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 32768
    vocab_size: int = 32000
    tie_word_embeddings: bool = False
    head_dim_override: int = 0

    def __post_init__(self) -> None:
        if self.head_dim_override == 0 and self.hidden_size % self.num_heads:
            raise ValueError("hidden_size must be divisible by num_heads")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        if self.num_layers <= 0 or self.vocab_size <= 0 or self.rope_theta <= 0:
            raise ValueError("num_layers, vocab_size and rope_theta must be positive")
        if self.head_dim % 2:
            raise ValueError("Qwen2 RoPE needs an even head_dim")

    @property
    def head_dim(self) -> int:
        return self.head_dim_override or self.hidden_size // self.num_heads

    @property
    def groups(self) -> int:
        return self.num_heads // self.num_kv_heads

    @property
    def q_size(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_kv_heads * self.head_dim


# The configurations the benchmarks and parity tests name.
TINY_FP32 = Qwen2Config(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4,
                        num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=1024,
                        tie_word_embeddings=True)
QWEN2_0_5B = Qwen2Config(hidden_size=896, intermediate_size=4864, num_layers=24, num_heads=14,
                         num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=151936,
                         tie_word_embeddings=True)
QWEN2_7B = Qwen2Config(hidden_size=3584, intermediate_size=18944, num_layers=28, num_heads=28,
                       num_kv_heads=4, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=152064,
                       tie_word_embeddings=False)


def parameter_shapes(config: Qwen2Config) -> Iterator[Tuple[str, Tuple[int, ...]]]:
    """(state_dict name, shape) in `model.parameters()` order of the reference model."""

    h, i = config.hidden_size, config.intermediate_size
    yield "embed_tokens.weight", (config.vocab_size, h)
    for layer in range(config.num_layers):
        p = f"decoder.layers.{layer}."
        yield p + "self_attn.q_proj.weight", (config.q_size, h)
        yield p + "self_attn.q_proj.bias", (config.q_size,)
        yield p + "self_attn.k_proj.weight", (config.kv_size, h)
        yield p + "self_attn.k_proj.bias", (config.kv_size,)
        yield p + "self_attn.v_proj.weight", (config.kv_size, h)
        yield p + "self_attn.v_proj.bias", (config.kv_size,)
        yield p + "self_attn.o_proj.weight", (h, config.q_size)
        yield p + "mlp.gate_proj.weight", (i, h)
        yield p + "mlp.up_proj.weight", (i, h)
        yield p + "mlp.down_proj.weight", (h, i)
        yield p + "input_layernorm.weight", (h,)
        yield p + "post_attention_layernorm.weight", (h,)
    yield "decoder.norm.weight", (h,)
    if not config.tie_word_embeddings:
        yield "lm_head.weight", (config.vocab_size, h)


def parameter_count(config: Qwen2Config) -> int:
    total = 0
    for _, shape in parameter_shapes(config):
        count = 1
        for extent in shape:
            count *= extent
        total += count
    return total


def make_weights(config: Qwen2Config, *, seed: int = 0, dtype: torch.dtype = torch.float32,
                 device: str | torch.device = "cpu", std: float = 0.02,
                 reproducible: bool = True) -> Dict[str, torch.Tensor]:
    """Random N(0, std) weights.

    reproducible=True draws every parameter on the CPU in fp32 from one generator seeded
    with `seed`, in parameter order, then casts and moves it: bit-identical to seeding the
    reference model. reproducible=False draws directly on `device` (large benchmark models).
    """

    weights: Dict[str, torch.Tensor] = {}
    if reproducible:
        generator = torch.Generator(device="cpu").manual_seed(seed)
        for name, shape in parameter_shapes(config):
            value = torch.empty(shape, dtype=torch.float32).normal_(0.0, std, generator=generator)
            weights[name] = value.to(dtype).to(device)
    else:
        generator = torch.Generator(device=device).manual_seed(seed)
        for name, shape in parameter_shapes(config):
            value = torch.empty(shape, dtype=torch.float32, device=device)
            value.normal_(0.0, std, generator=generator)
            weights[name] = value.to(dtype)
    if config.tie_word_embeddings:
        weights["lm_head.weight"] = weights["embed_tokens.weight"]
    return weights


def inverse_frequency(config: Qwen2Config, device: str | torch.device = "cpu") -> torch.Tensor:
    """fp32 RoPE inverse frequencies (qwen2.py:112-127), computed on the host: constants."""

    dimensions = torch.arange(0, config.head_dim, 2, dtype=torch.float32)
    return (1.0 / (config.rope_theta ** (dimensions / config.head_dim))).to(device)


def make_prompt_ids(config: Qwen2Config, batch: int, tokens: int, *, seed: int = 0) -> torch.Tensor:
    """Uniform token ids from a seeded CPU generator (make_qwen2_prefill_inputs, qwen2.py:552-559)."""

    generator = torch.Generator(device="cpu").manual_seed(seed)
    return torch.randint(0, config.vocab_size, (batch, tokens), generator=generator,
                         dtype=torch.int64)
