"""Qwen2 serving engine: stateful prefill -> greedy decode on the sm_100a kernels, with the
decode step captured in a CUDA graph over fixed KV / length / token buffer addresses.

This is the fused form of the per-layer KernelIR sequence the reference interprets op by
op (backends/triton_executor.py:69-130): per decode layer

    rms_norm -> linear(q|k|v fused, +bias) -> rope + kv.store (one launch)
             -> decode_attention -> linear(o) + residual (epilogue)
    rms_norm -> linear(gate|up interleaved) + SwiGLU (epilogue) -> linear(down) + residual

and, for bf16 in the fast numerical mode at decode batch sizes, the chain form of the same
sequence: the small projections leave fp32 split-K partials and the next operator reduces
them on load (bias + rope + kv.store after q|k|v; residual + rms_norm after o and down),
8 launches per layer, launched with programmatic dependent launch so that each kernel's
set-up and weight loads overlap its predecessor.

Every rounding point of the reference graph is kept (each linear result is rounded to the
model dtype before its bias-free residual add, SwiGLU rounds silu(gate) then the product),
so the fusions change launch counts, not numerics. One replica lives on one GPU; batch
partitioning across GPUs is in serving.py.
"""

from __future__ import annotations

import math
import os
from typing import Dict, Optional

import torch

from . import kernels
from .kv_state import ExecutionError, PagedKVCacheState, PreallocatedKVCacheState
from .qwen2 import Qwen2Config, inverse_frequency


class Qwen2Engine:
    def __init__(self, config: Qwen2Config, weights: Dict[str, torch.Tensor], *, batch: int,
                 capacity: int, numerical_mode: str = "fast",
                 device: Optional[torch.device] = None, kv_layout: str = "contiguous",
                 block_size: int = 128, num_blocks: Optional[int] = None) -> None:
        """kv_layout "paged": K / V live in block pools of `num_blocks` blocks of `block_size`
        tokens per layer (default: as many as the contiguous layout would hold) behind one block
        table; `capacity` is then the longest context one sequence may reach. Blocks are handed
        out on the host, ahead of the steps that need them."""

        if numerical_mode not in ("fast", "pytorch_compatible"):
            raise ValueError(f"unknown numerical mode {numerical_mode!r}")
        if kv_layout not in ("contiguous", "paged"):
            raise ValueError(f"unknown KV layout {kv_layout!r}")
        self.config = config
        self.batch = batch
        self.capacity = capacity
        self.mode = numerical_mode
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.dtype = weights["embed_tokens.weight"].dtype
        self.scale = config.head_dim ** -0.5
        # the five-launch decode layer (RMSNorm folded into q|k|v and gate|up, cluster split-K
        # o / down with the residual inside): bf16, fast mode, up to 128 rows while the layer's
        # largest matrix, gate|up, keeps its launch a chain of latencies, 64 rows for large models
        # (kernels.decode_chain_rows; B200_CHAIN_ROWS overrides). B200_DECODE_CHAIN=partials keeps
        # the seven-launch layer with reduce consumers.
        gate_up_bytes = 2 * config.intermediate_size * config.hidden_size * 2
        chain_rows = int(os.environ.get("B200_CHAIN_ROWS", "0")) or kernels.decode_chain_rows(gate_up_bytes)
        self.folded_norms = (self.dtype == torch.bfloat16 and numerical_mode == "fast" and
                             batch <= chain_rows and
                             config.hidden_size % 8 == 0 and
                             os.environ.get("B200_DECODE_CHAIN", "folded") != "partials")
        # the o projection leaves the row sums of squares that the gate|up projection's folded
        # RMSNorm needs (B200_NORM_SQUARES=own: gate|up squares its input rows itself)
        self.producer_squares = os.environ.get("B200_NORM_SQUARES", "producer") != "own"
        self._pack_weights(weights)
        self.inv_freq = inverse_frequency(config, self.device)

        layers = config.num_layers
        self.paged = kv_layout == "paged"
        # length arena rows: [0, L) per-slot lengths, L = positions, L + 1 = attention lengths
        if self.paged:
            if self.dtype != torch.bfloat16:
                raise ValueError("the paged KV layout holds bf16")
            blocks = num_blocks if num_blocks is not None else batch * -(-capacity // block_size)
            self.state = PagedKVCacheState.allocate_paged(
                num_layers=layers, batch=batch, max_tokens=capacity, block_size=block_size,
                num_blocks=blocks, kv_heads=config.num_kv_heads, head_dim=config.head_dim,
                dtype=self.dtype, device=self.device, extra_length_rows=2)
            self.capacity = capacity = self.state.capacity  # whole blocks
        else:
            self.state = PreallocatedKVCacheState.allocate(
                num_layers=layers, batch=batch, capacity=capacity, kv_heads=config.num_kv_heads,
                head_dim=config.head_dim, dtype=self.dtype, device=self.device, extra_length_rows=2)
        # host mirror of the context lengths: which blocks the next steps need (paged layout)
        self._host_lengths = [0] * batch
        self._block_slack = 0  # steps every sequence can still take inside its reserved blocks
        arena = self.state._length_arena
        self.positions = arena[layers]
        self.attention_lengths = arena[layers + 1]
        self.input_ids = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.next_ids = torch.zeros(batch, dtype=torch.int64, device=self.device)
        self.logits: Optional[torch.Tensor] = None
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._step_graph: Optional[torch.cuda.CUDAGraph] = None  # the same step between its two host copies
        self._host_ids = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self._host_tokens = torch.zeros(batch, dtype=torch.int64).pin_memory()
        self.max_length_hint = 0  # host-known upper bound of the context (0 = capacity)
        # programmatic dependent launch of the chain (B200_PROGRAMMATIC_LAUNCH=0 turns it off)
        self.programmatic_launch = os.environ.get("B200_PROGRAMMATIC_LAUNCH", "1") != "0"
        # q|k|v reduction + RoPE + KV store inside the attention kernel (B200_FUSED_QKV_ATTENTION=0
        # keeps them a launch of their own)
        self.fused_qkv_attention = os.environ.get("B200_FUSED_QKV_ATTENTION", "1") != "0"
        self.split_tokens = 0
        self.kernels_per_step = 0
        # longest-first service order of decode attention (ragged batches with more
        # (sequence, KV head) pairs than the GPU holds at once): one buffer, rewritten in place
        # by load_context, so that a captured step keeps reading the current order
        self.sequence_order: Optional[torch.Tensor] = None
        if self.dtype == torch.bfloat16:
            self.sequence_order = torch.arange(batch, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------------ weights ----
    def _pack_weights(self, weights: Dict[str, torch.Tensor]) -> None:
        cfg = self.config
        for name, tensor in weights.items():
            if not tensor.is_cuda:
                raise ValueError(f"weight {name} is not on a CUDA device")
        self.embed = weights["embed_tokens.weight"]
        self.lm_head = weights["lm_head.weight"]
        self.final_norm = weights["decoder.norm.weight"]
        # the final RMSNorm folded into the LM head as well (a second copy of that matrix)
        self.lm_head_folded = kernels.b200_scale_columns(self.lm_head, self.final_norm) \
            if self.folded_norms else None
        self.layers = []
        for index in range(cfg.num_layers):
            p = f"decoder.layers.{index}."
            qkv_w = torch.cat([weights[p + "self_attn.q_proj.weight"],
                               weights[p + "self_attn.k_proj.weight"],
                               weights[p + "self_attn.v_proj.weight"]], dim=0).contiguous()
            qkv_b = torch.cat([weights[p + "self_attn.q_proj.bias"],
                               weights[p + "self_attn.k_proj.bias"],
                               weights[p + "self_attn.v_proj.bias"]], dim=0).contiguous()
            gate_up = kernels.interleave_gate_up(weights[p + "mlp.gate_proj.weight"],
                                                 weights[p + "mlp.up_proj.weight"])
            layer = {
                "input_norm": weights[p + "input_layernorm.weight"],
                "post_norm": weights[p + "post_attention_layernorm.weight"],
                "qkv_w": qkv_w, "qkv_b": qkv_b,
                "o_w": weights[p + "self_attn.o_proj.weight"],
                "gate_up_w": gate_up,
                "down_w": weights[p + "mlp.down_proj.weight"],
            }
            if self.folded_norms:
                # the norm weights multiplied into the columns of the projections behind them
                layer["qkv_w_folded"] = kernels.b200_scale_columns(qkv_w, layer["input_norm"])
                layer["gate_up_w_folded"] = kernels.b200_scale_columns(gate_up, layer["post_norm"])
            self.layers.append(layer)

    # ------------------------------------------------------------------ prefill ----
    def prefill(self, input_ids: torch.Tensor, *, all_logits: bool = False) -> torch.Tensor:
        """Stateful prefill of a B x T prompt from an empty state. Returns logits for the last
        position (B x V) or, with all_logits=True, for every position (B x T x V) as the
        reference graph does (qwen2.py:418-424). Also primes the greedy next token."""

        cfg = self.config
        if input_ids.shape[0] != self.batch or input_ids.ndim != 2:
            raise ValueError("prompt must be batch x tokens")
        batch, tokens = input_ids.shape
        if tokens > self.capacity:
            raise ExecutionError(f"prompt of {tokens} tokens exceeds capacity {self.capacity}")
        ids = input_ids.to(self.device)
        if self.sequence_order is not None:  # every sequence holds the same number of tokens
            self.sequence_order.copy_(torch.arange(batch, dtype=torch.int32, device=self.device))
        self.state._length_arena.zero_()
        if self.paged:
            for sequence in range(batch):
                self.state.release(sequence)
            self._host_lengths = [tokens] * batch
            self._block_slack = 0
            self._reserve_blocks()
        position_ids = torch.arange(tokens, dtype=torch.int64, device=self.device).repeat(batch, 1)
        x = kernels.b200_embedding(self.embed, ids)
        cosine, sine = kernels.b200_rope_table(position_ids, self.inv_freq, self.dtype)
        zeros = self.positions  # all zero right now
        q_size, kv_size = cfg.q_size, cfg.kv_size
        for index, layer in enumerate(self.layers):
            h = kernels.b200_rms_norm(x, layer["input_norm"], epsilon=cfg.rms_norm_eps,
                                      round_before_weight=True, numerical_mode=self.mode)
            qkv = kernels.b200_linear(h, layer["qkv_w"], layer["qkv_b"])
            q = qkv[..., :q_size].view(batch, tokens, cfg.num_heads, cfg.head_dim).transpose(1, 2)
            k = qkv[..., q_size:q_size + kv_size].view(batch, tokens, cfg.num_kv_heads,
                                                       cfg.head_dim).transpose(1, 2)
            v = qkv[..., q_size + kv_size:].view(batch, tokens, cfg.num_kv_heads,
                                                 cfg.head_dim).transpose(1, 2)
            q, k = kernels.b200_rope(q, k, cosine, sine)
            if self.paged:
                kernels.b200_paged_kv_store(self.state.keys[index], self.state.values[index],
                                            self.state.block_table, k, v, zeros)
            else:
                kernels.b200_kv_store(self.state.keys[index], self.state.values[index], k, v, zeros)
            attn = kernels.b200_prefill_attention(q, k, v, None, scale=self.scale, causal=True,
                                                  numerical_mode=self.mode)
            attn = attn.transpose(1, 2).reshape(batch, tokens, q_size)  # a view: memory is B,T,H,D
            x = kernels.b200_linear(attn, layer["o_w"], residual=x, epilogue="residual")
            h = kernels.b200_rms_norm(x, layer["post_norm"], epsilon=cfg.rms_norm_eps,
                                      round_before_weight=True, numerical_mode=self.mode)
            a = kernels.b200_linear(h, layer["gate_up_w"], epilogue="swiglu")
            x = kernels.b200_linear(a, layer["down_w"], residual=x, epilogue="residual")
        if all_logits:
            h = kernels.b200_rms_norm(x, self.final_norm, epsilon=cfg.rms_norm_eps,
                                      round_before_weight=True, numerical_mode=self.mode)
            logits = kernels.b200_linear(h, self.lm_head)
            last = logits[:, -1]
        else:
            h = kernels.b200_rms_norm(x[:, -1], self.final_norm, epsilon=cfg.rms_norm_eps,
                                      round_before_weight=True, numerical_mode=self.mode)
            logits = kernels.b200_linear(h, self.lm_head)
            last = logits
        kernels.b200_argmax(last, self.next_ids)
        self.input_ids.copy_(self.next_ids)
        kernels.b200_advance_lengths(self.state._length_arena, tokens, self.capacity)
        # attention lengths run one ahead of the positions: they include the token being decoded
        kernels.b200_advance_lengths(self.attention_lengths, 1, self.capacity + 1)
        self.logits = last
        return logits

    def load_context(self, lengths: torch.Tensor, *, next_ids: Optional[torch.Tensor] = None) -> None:
        """Benchmark entry: declares that the KV buffers already hold `lengths[b]` tokens per
        sequence (filled by the caller) and sets the next input token ids."""

        lengths = lengths.to(device=self.device, dtype=torch.int64)
        layers = self.config.num_layers
        self.state._length_arena[:layers + 1].copy_(lengths.unsqueeze(0).expand(layers + 1, -1))
        self.attention_lengths.copy_(lengths + 1)
        if next_ids is not None:
            self.input_ids.copy_(next_ids.to(self.device))
        self._host_lengths = [int(n) for n in lengths.tolist()]
        self._block_slack = 0
        self._reserve_blocks()
        if self.sequence_order is not None and os.environ.get("B200_SEQUENCE_ORDER", "longest") != "grid":
            self.sequence_order.copy_(kernels.sequence_order_of(lengths))

    def _reserve_blocks(self) -> None:
        """Paged layout: every sequence owns the blocks for its context plus at least one more
        token before a step is launched; done a block ahead, so the host touches the table once
        per block_size steps (the table's address is fixed: a captured graph sees the update)."""

        if not self.paged or self._block_slack > 0:
            return
        size = self.state.block_size
        self.state.reserve([min(n + size, self.capacity) for n in self._host_lengths])
        self._block_slack = min(min(-(-(n + size) // size) * size, self.capacity) - n
                                for n in self._host_lengths)

    def sync_host_lengths(self) -> None:
        """Re-reads the context lengths from the device (one synchronising copy): for callers
        that set the length vectors themselves."""

        self._host_lengths = [int(n) for n in self.positions.tolist()]
        self._block_slack = 0
        self._reserve_blocks()

    def _count_step(self) -> None:
        if self.paged:
            self._host_lengths = [n + 1 for n in self._host_lengths]
            self._block_slack -= 1

    # ------------------------------------------------------------------- decode ----
    @property
    def chained(self) -> bool:
        """Whether a decode step runs the launch chain (fast bf16, up to 128 sequences)."""
        # (the paged layout has the folded five-launch chain and the separate kernels)
        return self.dtype == torch.bfloat16 and self.mode == "fast" and self.batch <= 128 and \
            (not self.paged or self.folded_norms)

    @property
    def attention_is_fused(self) -> bool:
        """Whether the step's attention launches are the fused form (q|k|v reduction, RoPE and
        KV store inside), which serves a CTA's tokens with 16 warps at head_dim 64."""
        return self.chained and self.fused_qkv_attention

    def _decode_step(self) -> None:
        if self.chained:
            self._decode_step_chain()
        else:
            self._decode_step_separate()

    def _decode_step_chain(self) -> None:
        """Fast bf16 decode step: every small projection is a split-K partial-sum producer on
        the tcgen05 kernel and the reduction rides in the next operator (bias + RoPE + KV store
        after q|k|v; residual + RMSNorm after o and down; with folded norms and cluster split-K
        five launches per layer, otherwise seven)."""

        # The weights are written once, when the engine is built. Lengths move at the end of a
        # step (advance_lengths, a fully serialised launch) and the only KV row a step writes
        # before its attention is the newest one, so both promises of the launch mode hold.
        with kernels.launch_mode(programmatic=self.programmatic_launch,
                                 constant_weights=self.programmatic_launch,
                                 stable_kv_prefix=self.programmatic_launch):
            self._chain_launches()

    def _folded_chain_launches(self) -> None:
        """Five launches per layer: q|k|v partials of the un-normalised x against the
        norm-folded weight -> attention (reduces q|k|v, applies the row's RMS factor, bias, RoPE,
        KV store) -> o projection (cluster split-K, + residual) -> gate|up + SwiGLU on the
        un-normalised x with the folded weight -> down projection (cluster split-K, + residual)."""

        cfg = self.config
        batch = self.batch
        eps = cfg.rms_norm_eps
        before = kernels.launch_count(self.device)
        x = kernels.b200_embedding(self.embed, self.input_ids)
        cosine, sine = kernels.b200_rope_table(self.positions.view(batch, 1), self.inv_freq,
                                               self.dtype)
        for index, layer in enumerate(self.layers):
            partials, squares = kernels.b200_linear_partial(x, layer["qkv_w_folded"],
                                                            row_squares=True)
            common = dict(q_heads=cfg.num_heads, scale=self.scale, split_tokens=self.split_tokens,
                          max_length_hint=self.max_length_hint, norm_row_squares=squares,
                          norm_hidden=cfg.hidden_size, norm_epsilon=eps,
                          sequence_order=self.sequence_order)
            if self.paged:
                attn = kernels.b200_paged_qkv_decode_attention(
                    partials, layer["qkv_b"], cosine, sine, self.state.keys[index],
                    self.state.values[index], self.state.block_table, self.attention_lengths, **common)
            else:
                attn = kernels.b200_qkv_decode_attention(
                    partials, layer["qkv_b"], cosine, sine, self.state.keys[index],
                    self.state.values[index], self.attention_lengths, **common)
            x = kernels.b200_linear_splitk_residual(attn.view(batch, cfg.q_size), layer["o_w"], x,
                                                    row_squares=self.producer_squares)
            x, x_squares = x if self.producer_squares else (x, None)
            a = kernels.b200_linear_rms_input(x, layer["gate_up_w_folded"], epsilon=eps,
                                              epilogue="swiglu", row_squares=x_squares)
            last = self.producer_squares and index + 1 == len(self.layers)
            x = kernels.b200_linear_splitk_residual(a, layer["down_w"], x, row_squares=last)
            x, x_squares = x if last else (x, None)  # (only the LM head's norm takes them)
        self.logits = kernels.b200_linear_rms_input(x, self.lm_head_folded, epsilon=eps,
                                                    row_squares=x_squares)
        kernels.b200_argmax(self.logits, self.next_ids)
        kernels.b200_advance_lengths(self.state._length_arena, 1, self.capacity + 1)
        self.kernels_per_step = kernels.launch_count(self.device) - before

    def _chain_launches(self) -> None:
        if self.folded_norms:
            return self._folded_chain_launches()
        cfg = self.config
        batch = self.batch
        before = kernels.launch_count(self.device)
        x = kernels.b200_embedding(self.embed, self.input_ids)
        cosine, sine = kernels.b200_rope_table(self.positions.view(batch, 1), self.inv_freq,
                                               self.dtype)
        h = kernels.b200_rms_norm(x, self.layers[0]["input_norm"], epsilon=cfg.rms_norm_eps,
                                  round_before_weight=True, numerical_mode=self.mode)
        for index, layer in enumerate(self.layers):
            partials = kernels.b200_linear_partial(h, layer["qkv_w"])
            if self.fused_qkv_attention:
                attn = kernels.b200_qkv_decode_attention(
                    partials, layer["qkv_b"], cosine, sine, self.state.keys[index],
                    self.state.values[index], self.attention_lengths, q_heads=cfg.num_heads,
                    scale=self.scale, split_tokens=self.split_tokens,
                    max_length_hint=self.max_length_hint, sequence_order=self.sequence_order)
            else:
                q = kernels.b200_reduce_rope_kv_store(
                    partials, layer["qkv_b"], cosine, sine, self.state.keys[index],
                    self.state.values[index], self.positions, q_heads=cfg.num_heads)
                attn = kernels.b200_decode_attention(
                    q, self.state.keys[index], self.state.values[index], self.attention_lengths,
                    None, scale=self.scale, numerical_mode=self.mode,
                    split_tokens=self.split_tokens, max_length_hint=self.max_length_hint)
            partials = kernels.b200_linear_partial(attn.view(batch, cfg.q_size), layer["o_w"])
            x, h = kernels.b200_reduce_residual_rms_norm(partials, x, layer["post_norm"],
                                                         epsilon=cfg.rms_norm_eps)
            a = kernels.b200_linear(h, layer["gate_up_w"], epilogue="swiglu")
            partials = kernels.b200_linear_partial(a, layer["down_w"])
            next_norm = self.layers[index + 1]["input_norm"] if index + 1 < len(self.layers) \
                else self.final_norm
            x, h = kernels.b200_reduce_residual_rms_norm(partials, x, next_norm,
                                                         epsilon=cfg.rms_norm_eps)
        self.logits = kernels.b200_linear(h, self.lm_head)
        kernels.b200_argmax(self.logits, self.next_ids)
        kernels.b200_advance_lengths(self.state._length_arena, 1, self.capacity + 1)
        self.kernels_per_step = kernels.launch_count(self.device) - before

    def _decode_step_separate(self) -> None:
        cfg = self.config
        batch = self.batch
        before = kernels.launch_count(self.device)
        x = kernels.b200_embedding(self.embed, self.input_ids)
        cosine, sine = kernels.b200_rope_table(self.positions.view(batch, 1), self.inv_freq,
                                               self.dtype)
        q_size, kv_size = cfg.q_size, cfg.kv_size
        for index, layer in enumerate(self.layers):
            h = kernels.b200_rms_norm(x, layer["input_norm"], epsilon=cfg.rms_norm_eps,
                                      round_before_weight=True, numerical_mode=self.mode)
            qkv = kernels.b200_linear(h, layer["qkv_w"], layer["qkv_b"])
            q = qkv[:, :q_size].view(batch, cfg.num_heads, cfg.head_dim)
            k = qkv[:, q_size:q_size + kv_size].view(batch, cfg.num_kv_heads, cfg.head_dim)
            v = qkv[:, q_size + kv_size:].view(batch, cfg.num_kv_heads, cfg.head_dim)
            if self.paged:
                q, k = kernels.b200_rope(q.unsqueeze(2), k.unsqueeze(2), cosine, sine)
                kernels.b200_paged_kv_store(self.state.keys[index], self.state.values[index],
                                            self.state.block_table, k, v.unsqueeze(2), self.positions)
                attn = kernels.b200_paged_decode_attention(
                    q, self.state.keys[index], self.state.values[index], self.state.block_table,
                    self.attention_lengths, None, scale=self.scale, numerical_mode=self.mode,
                    split_tokens=self.split_tokens, max_length_hint=self.max_length_hint)
            else:
                q = kernels.b200_rope_kv_store(q, k, v, cosine, sine, self.state.keys[index],
                                               self.state.values[index], self.positions)
                attn = kernels.b200_decode_attention(
                    q, self.state.keys[index], self.state.values[index], self.attention_lengths,
                    None, scale=self.scale, numerical_mode=self.mode,
                    split_tokens=self.split_tokens, max_length_hint=self.max_length_hint,
                    sequence_order=self.sequence_order)
            # o and down have few N tiles: at up to 256 bf16 rows they run as cluster split-K
            # projections that add the residual themselves (same rounding points)
            splitk = self.dtype == torch.bfloat16 and batch <= 256 and cfg.hidden_size % 4 == 0
            if splitk:
                x = kernels.b200_linear_splitk_residual(attn.view(batch, q_size), layer["o_w"], x)
            else:
                x = kernels.b200_linear(attn.view(batch, q_size), layer["o_w"], residual=x,
                                        epilogue="residual")
            h = kernels.b200_rms_norm(x, layer["post_norm"], epsilon=cfg.rms_norm_eps,
                                      round_before_weight=True, numerical_mode=self.mode)
            a = kernels.b200_linear(h, layer["gate_up_w"], epilogue="swiglu")
            if splitk:
                x = kernels.b200_linear_splitk_residual(a, layer["down_w"], x)
            else:
                x = kernels.b200_linear(a, layer["down_w"], residual=x, epilogue="residual")
        h = kernels.b200_rms_norm(x, self.final_norm, epsilon=cfg.rms_norm_eps,
                                  round_before_weight=True, numerical_mode=self.mode)
        self.logits = kernels.b200_linear(h, self.lm_head)
        kernels.b200_argmax(self.logits, self.next_ids)
        # all slot lengths, the positions row and the attention-length row move together
        kernels.b200_advance_lengths(self.state._length_arena, 1, self.capacity + 1)
        self.kernels_per_step = kernels.launch_count(self.device) - before

    def use_dispatch_profile(self, cost_model, context_bound: int):
        """Takes the decode-attention split size for this engine's batch and a context of up to
        `context_bound` tokens from a measured profile (dispatch_plan.DispatchCostModel). Call
        before capture(): the split is baked into the captured launches. Returns the decision."""

        from .dispatch_plan import resolve_dispatch_plan, split_tokens_of

        cfg = self.config
        batches = sorted({dict(e.key)["batch"] for e in cost_model.entries
                          if e.op == "decode_attention"})
        if not batches:
            return resolve_dispatch_plan(None, context_bound)
        nearest = min(batches, key=lambda b: abs(math.log(b / self.batch)))
        plan = cost_model.plan_attribute("decode_attention", batch=nearest, q_heads=cfg.num_heads,
                                         kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim,
                                         dtype=str(self.dtype))
        decision = resolve_dispatch_plan(plan, context_bound)
        self.split_tokens = split_tokens_of(decision.variant)
        return decision

    def capture(self) -> None:
        """Captures one decode step in a CUDA graph. A warm-up step runs first so that every
        workspace exists; lengths, positions and ids are restored afterwards (the KV row the
        warm-up wrote lies beyond the valid length and is overwritten by the real step)."""

        self._reserve_blocks()
        saved_lengths = self.state._length_arena.clone()
        saved_ids = self.input_ids.clone()
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            self._decode_step()
            self.state._length_arena.copy_(saved_lengths)
            self.input_ids.copy_(saved_ids)
        torch.cuda.current_stream(self.device).wait_stream(stream)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._decode_step()
        self._graph = graph
        self._graph_logits = self.logits  # each graph writes the logits into a buffer of its own
        # step(): the copy of the ids from pinned host memory, the step and the copy of the tokens
        # back as one graph launch instead of three submissions
        step_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(step_graph):
            self.input_ids.copy_(self._host_ids, non_blocking=True)
            self._decode_step()
            self._host_tokens.copy_(self.next_ids, non_blocking=True)
        self._step_graph = step_graph
        self._step_logits = self.logits
        self.logits = self._graph_logits
        kernels.runtime(self.device).status.zero_()

    def decode_step(self, *, feed_back: bool = True) -> torch.Tensor:
        """One decode step for the whole batch on device-resident inputs. Returns the device
        tensor of greedy tokens; with feed_back they become the next step's input ids."""

        self._reserve_blocks()
        if self._graph is not None:
            self._graph.replay()
            self.logits = self._graph_logits
        else:
            self._decode_step()
        self._count_step()
        if feed_back:
            self.input_ids.copy_(self.next_ids, non_blocking=True)
        return self.next_ids

    def step(self, host_ids: torch.Tensor) -> torch.Tensor:
        """The call a serving loop makes: host token ids in, host greedy tokens out. Copies
        the ids from pinned host memory, runs one decode step, copies the tokens back and
        waits for them."""

        self._host_ids.copy_(host_ids)
        if self._step_graph is not None:
            self._reserve_blocks()
            self._step_graph.replay()
            self.logits = self._step_logits
            self._count_step()
        else:
            self.input_ids.copy_(self._host_ids, non_blocking=True)
            self.decode_step(feed_back=False)
            self._host_tokens.copy_(self.next_ids, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return self._host_tokens

    def generate(self, prompt_ids: torch.Tensor, steps: int, *, use_graph: bool = True) -> torch.Tensor:
        """Greedy generation: prefill then `steps` decode steps. Returns B x (steps + 1) token
        ids (the token sampled from the prompt first)."""

        self.prefill(prompt_ids)
        history = torch.empty((steps + 1, self.batch), dtype=torch.int64, device=self.device)
        history[0].copy_(self.next_ids)
        if use_graph and self._graph is None and steps > 0:
            self.capture()
        for index in range(steps):
            self.decode_step()
            history[index + 1].copy_(self.next_ids)
        self.state.check()
        return history.transpose(0, 1).contiguous()
