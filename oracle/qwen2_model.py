"""CPU oracle of the stateful Qwen2 prefill -> decode path -- TEST INFRASTRUCTURE.

Restates, with the per-operator functions of oracle/serve_ops.py, the op sequence the
reference's CPU executor runs for the optimised ServeIR of StatefulQwen2ForCausalLM
(model: src/stateful_llm_compiler/qwen2.py:152-478; per-layer op order after KV
bufferisation: passes/kv_bufferize.py:175-200; prefill KV state: passes/prefill_kv.py:95-96):

  prefill:  embedding -> cos/sin -> L x [rms_norm, q/k/v linear, rope, prefill_attention,
            o linear, add, rms_norm, gate/up linear, silu*mul, down linear, add]
            -> rms_norm -> lm_head (all positions) -> kv.init -> L x kv.prefill_store
  decode:   embedding -> cos/sin -> L x [rms_norm, q/k/v linear, rope, kv.length, kv.store,
            kv.advance, decode_attention, o linear, add, rms_norm, MLP, add]
            -> rms_norm -> lm_head

Pinned by tests/test_oracle.py against tests/golden/qwen2_tiny_fp32.pt, which holds the
logits the reference's own ReferenceExecutor produced for the same seeded weights and ids.
Only tests/, smoke() and bench.py's CPU-baseline legs may import this module.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from . import serve_ops as ops


@dataclass
class OracleKVState:
    """PreallocatedKVCacheState (execution.py:98-131): B x C x Hkv x D buffers + int64 lengths."""

    keys: List[torch.Tensor]
    values: List[torch.Tensor]
    lengths: List[torch.Tensor]
    capacity: int


def _layer_names(index: int) -> str:
    return f"decoder.layers.{index}."


def _attention_inputs(config, weights, prefix, hidden, batch, tokens):
    q = ops.linear(hidden, weights[prefix + "self_attn.q_proj.weight"],
                   weights[prefix + "self_attn.q_proj.bias"])
    k = ops.linear(hidden, weights[prefix + "self_attn.k_proj.weight"],
                   weights[prefix + "self_attn.k_proj.bias"])
    v = ops.linear(hidden, weights[prefix + "self_attn.v_proj.weight"],
                   weights[prefix + "self_attn.v_proj.bias"])
    q = q.view(batch, tokens, config.num_heads, config.head_dim).transpose(1, 2)
    k = k.view(batch, tokens, config.num_kv_heads, config.head_dim).transpose(1, 2)
    v = v.view(batch, tokens, config.num_kv_heads, config.head_dim).transpose(1, 2)
    return q, k, v


def _mlp(weights, prefix, hidden):
    gate = ops.linear(hidden, weights[prefix + "mlp.gate_proj.weight"])
    up = ops.linear(hidden, weights[prefix + "mlp.up_proj.weight"])
    return ops.linear(ops.swiglu(gate, up), weights[prefix + "mlp.down_proj.weight"])


def _norm(config, weights, name, tensor):
    # Qwen2's RMSNorm rounds to the input dtype before the weight product (model.py:44-51)
    return ops.rms_norm(tensor, weights[name], config.rms_norm_eps, round_before_weight=True)


def prefill(config, weights: Dict[str, torch.Tensor], input_ids: torch.Tensor, *, capacity: int,
            attention_mask: torch.Tensor | None = None):
    """StatefulQwen2ForCausalLM.prefill (qwen2.py:405-424) + MaterializePrefillKVState."""

    batch, tokens = input_ids.shape
    dtype = weights["embed_tokens.weight"].dtype
    if attention_mask is None:
        attention_mask = ops.causal_mask(batch, tokens)
    position_ids = torch.arange(tokens, dtype=torch.int64).view(1, -1).expand(batch, -1)
    inv_freq = ops.rope_inverse_frequency(config.head_dim, config.rope_theta)
    cosine, sine = ops.rope_table(position_ids, inv_freq, dtype)
    scale = config.head_dim ** -0.5
    hidden = ops.embedding(weights["embed_tokens.weight"], input_ids)
    layer_kv = []
    for index in range(config.num_layers):
        prefix = _layer_names(index)
        normed = _norm(config, weights, prefix + "input_layernorm.weight", hidden)
        q, k, v = _attention_inputs(config, weights, prefix, normed, batch, tokens)
        q, k = ops.rope(q, k, cosine, sine)
        layer_kv.append((k, v))
        context = ops.prefill_attention(q, k, v, attention_mask, groups=config.groups, scale=scale)
        context = context.transpose(1, 2).contiguous().reshape(batch, tokens, config.q_size)
        hidden = ops.residual_add(
            hidden, ops.linear(context, weights[prefix + "self_attn.o_proj.weight"]))
        normed = _norm(config, weights, prefix + "post_attention_layernorm.weight", hidden)
        hidden = ops.residual_add(hidden, _mlp(weights, prefix, normed))
    hidden = _norm(config, weights, "decoder.norm.weight", hidden)
    logits = ops.linear(hidden, weights["lm_head.weight"])
    state = OracleKVState([], [], [], capacity)
    for k, v in layer_kv:  # kv.init + kv.prefill_store (execution.py:133-162, 405-419)
        key_buffer = torch.zeros(batch, capacity, config.num_kv_heads, config.head_dim, dtype=dtype)
        value_buffer = torch.zeros_like(key_buffer)
        zeros = torch.zeros(batch, dtype=torch.int64)
        ops.kv_store(key_buffer, value_buffer, k, v, zeros)
        state.keys.append(key_buffer)
        state.values.append(value_buffer)
        state.lengths.append(ops.kv_advance(zeros, tokens, capacity))
    return logits, state


def decode(config, weights: Dict[str, torch.Tensor], input_ids: torch.Tensor,
           state: OracleKVState, *, position_ids: torch.Tensor | None = None,
           attention_mask: torch.Tensor | None = None):
    """One stateful decode step on B x 1 token ids (qwen2.py:438-452 after bufferisation).
    Mutates the KV buffers in place and replaces the per-slot lengths."""

    batch = input_ids.shape[0]
    dtype = weights["embed_tokens.weight"].dtype
    if position_ids is None:
        position_ids = state.lengths[0].view(batch, 1).clone()
    if attention_mask is None:
        # callers pass zeros[B,1,1,L+1] (validate_qwen2_checkpoint.py:365-396); any length
        # between max(lengths)+1 and the capacity is equivalent
        attention_mask = torch.zeros(batch, 1, 1, int(state.lengths[0].max()) + 1)
    inv_freq = ops.rope_inverse_frequency(config.head_dim, config.rope_theta)
    cosine, sine = ops.rope_table(position_ids, inv_freq, dtype)
    scale = config.head_dim ** -0.5
    hidden = ops.embedding(weights["embed_tokens.weight"], input_ids)
    for index in range(config.num_layers):
        prefix = _layer_names(index)
        normed = _norm(config, weights, prefix + "input_layernorm.weight", hidden)
        q, k, v = _attention_inputs(config, weights, prefix, normed, batch, 1)
        q, k = ops.rope(q, k, cosine, sine)
        positions = state.lengths[index]                                   # kv.length
        ops.kv_store(state.keys[index], state.values[index], k, v, positions)  # kv.store
        state.lengths[index] = ops.kv_advance(positions, 1, state.capacity)    # kv.advance
        context = ops.decode_attention(q, state.keys[index], state.values[index],
                                       state.lengths[index], attention_mask,
                                       groups=config.groups, scale=scale)
        context = context.transpose(1, 2).reshape(batch, 1, config.q_size)
        hidden = ops.residual_add(
            hidden, ops.linear(context, weights[prefix + "self_attn.o_proj.weight"]))
        normed = _norm(config, weights, prefix + "post_attention_layernorm.weight", hidden)
        hidden = ops.residual_add(hidden, _mlp(weights, prefix, normed))
    hidden = _norm(config, weights, "decoder.norm.weight", hidden)
    return ops.linear(hidden, weights["lm_head.weight"])


def greedy_generate(config, weights, prompt_ids: torch.Tensor, steps: int, *, capacity: int):
    """Prefill, then `steps` greedy decode steps feeding argmax tokens back. Returns
    (tokens B x (steps+1), list of per-step logits B x V, final state)."""

    logits, state = prefill(config, weights, prompt_ids, capacity=capacity)
    step_logits = [logits[:, -1]]
    tokens = [step_logits[0].argmax(dim=-1)]
    for _ in range(steps):
        out = decode(config, weights, tokens[-1].view(-1, 1), state)
        step_logits.append(out[:, 0])
        tokens.append(step_logits[-1].argmax(dim=-1))
    return torch.stack(tokens, dim=1), step_logits, state
