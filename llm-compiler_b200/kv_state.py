"""Preallocated multi-slot KV runtime state: the state ABI of the KernelIR backend.

Same object shape as the reference's PreallocatedKVCacheState (execution.py:98-475):
`keys[i]` / `values[i]` are B x C x Hkv x D buffers per layer slot, `lengths[i]` an int64
[B] vector per slot, plus `capacity` and a `generation` counter. Differences, all forced
by CUDA-graph replay over fixed addresses:

 - all slots are views of one arena (`[L, B, C, Hkv, D]` for K, one for V, `[L, B]` for the
   lengths), so 180 GB of HBM is carved once and never reallocated;
 - `advance` updates the slot's length vector in place with a kernel and returns a new
   state object that shares the tensors (generation + 1), instead of allocating
   `positions + delta`; a caller must not keep reading an old state's lengths;
 - capacity overflow never asserts on the device (execution.py:1283-1293 does): the
   kernels skip/clamp and raise a status bit that `check()` turns into ExecutionError.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional, Sequence, Tuple

import torch

from . import kernels


class ExecutionError(RuntimeError):
    pass


@dataclass(frozen=True)
class PreallocatedKVCacheState:
    keys: Tuple[torch.Tensor, ...]
    values: Tuple[torch.Tensor, ...]
    lengths: Tuple[torch.Tensor, ...]
    capacity: int
    generation: int = 0

    def __post_init__(self) -> None:
        if self.capacity <= 0:
            raise ExecutionError("KV capacity must be positive")
        if not self.keys or len(self.keys) != len(self.values) or \
                len(self.keys) != len(self.lengths):
            raise ExecutionError("K, V and length slot counts must agree and be non-zero")
        for key, value, lengths in zip(self.keys, self.values, self.lengths):
            if key.shape != value.shape or key.ndim != 4:
                raise ExecutionError("KV buffers must be B x C x H x D tensors of one shape")
            if key.shape[1] != self.capacity:
                raise ExecutionError("the second KV buffer dimension must equal the capacity")
            if lengths.shape != (key.shape[0],) or lengths.dtype != torch.int64:
                raise ExecutionError("KV lengths must be one int64 vector per slot")

    # ---- construction ------------------------------------------------------------
    @classmethod
    def allocate(cls, *, num_layers: int, batch: int, capacity: int, kv_heads: int,
                 head_dim: int, dtype: torch.dtype, device: torch.device | str,
                 extra_length_rows: int = 0) -> "PreallocatedKVCacheState":
        """One zeroed arena for all slots. `extra_length_rows` appends rows to the length
        arena that the serving engine uses for its position / attention-length vectors, so a
        single kernel advances everything."""

        if num_layers <= 0 or batch <= 0 or capacity <= 0:
            raise ExecutionError("KV init needs positive layer count, batch and capacity")
        key_arena = torch.zeros((num_layers, batch, capacity, kv_heads, head_dim), dtype=dtype,
                                device=device)
        value_arena = torch.zeros_like(key_arena)
        length_arena = torch.zeros((num_layers + extra_length_rows, batch), dtype=torch.int64,
                                   device=device)
        state = cls(tuple(key_arena[i] for i in range(num_layers)),
                    tuple(value_arena[i] for i in range(num_layers)),
                    tuple(length_arena[i] for i in range(num_layers)), capacity)
        object.__setattr__(state, "_length_arena", length_arena)
        object.__setattr__(state, "_key_arena", key_arena)
        object.__setattr__(state, "_value_arena", value_arena)
        return state

    @classmethod
    def empty_from_key_template(cls, key: torch.Tensor, *, num_layers: int,
                                capacity: int) -> "PreallocatedKVCacheState":
        """runtime.kv.init (execution.py:133-162): empty slots shaped after a B x H x T x D key."""

        if key.ndim != 4 or num_layers <= 0 or capacity <= 0:
            raise ExecutionError("KV init got an illegal template, layer count or capacity")
        batch, heads, _, head_dim = key.shape
        return cls.allocate(num_layers=num_layers, batch=batch, capacity=capacity,
                            kv_heads=heads, head_dim=head_dim, dtype=key.dtype,
                            device=key.device)

    @classmethod
    def from_layer_tensors(cls, past_key_values: Sequence[Tuple[torch.Tensor, torch.Tensor]], *,
                           capacity: int) -> "PreallocatedKVCacheState":
        """Copies logical B x H x S x D caches into preallocated slots (execution.py:203-259)."""

        if not past_key_values:
            raise ExecutionError("a multi-layer KV cache needs at least one slot")
        key0 = past_key_values[0][0]
        batch, heads, sequence, head_dim = key0.shape
        if sequence > capacity:
            raise ExecutionError(f"initial KV length {sequence} exceeds capacity {capacity}")
        state = cls.allocate(num_layers=len(past_key_values), batch=batch, capacity=capacity,
                             kv_heads=heads, head_dim=head_dim, dtype=key0.dtype,
                             device=key0.device)
        zeros = torch.zeros(batch, dtype=torch.int64, device=key0.device)
        for slot, (key, value) in enumerate(past_key_values):
            if key.shape != key0.shape or value.shape != key0.shape:
                raise ExecutionError("all slots must share one KV shape")
            kernels.b200_kv_store(state.keys[slot], state.values[slot], key, value, zeros)
        state._length_arena[:len(past_key_values)].fill_(sequence)
        return state

    def _derive(self, generation: int) -> "PreallocatedKVCacheState":
        state = PreallocatedKVCacheState(self.keys, self.values, self.lengths, self.capacity,
                                         generation)
        for name in ("_length_arena", "_key_arena", "_value_arena"):
            if hasattr(self, name):
                object.__setattr__(state, name, getattr(self, name))
        return state

    # ---- accessors -----------------------------------------------------------------
    def _slot(self, slot: int):
        if slot < 0 or slot >= len(self.keys):
            raise ExecutionError(f"KV buffer has no slot {slot}")
        return self.keys[slot], self.values[slot], self.lengths[slot]

    def positions(self, slot: int) -> torch.Tensor:
        return self._slot(slot)[2]

    def read(self, slot: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Logical B x H x S x D views (execution.py:267-279); synchronises on lengths.max()."""

        key, value, lengths = self._slot(slot)
        used = int(lengths.max().item())
        return key[:, :used].transpose(1, 2), value[:, :used].transpose(1, 2)

    # ---- operations ------------------------------------------------------------------
    def store(self, slot: int, key: torch.Tensor, value: torch.Tensor, positions: torch.Tensor, *,
              writer: Optional[Callable] = None) -> "PreallocatedKVCacheState":
        """serve.kv.store (execution.py:371-403): writes in place, returns the same state."""

        buffer_key, buffer_value, _ = self._slot(slot)
        if key.shape != value.shape or key.ndim != 4:
            raise ExecutionError("KV store needs K and V of one B x H x T x D shape")
        batch, heads, tokens, head_dim = key.shape
        if batch != buffer_key.shape[0] or heads != buffer_key.shape[2] or \
                head_dim != buffer_key.shape[3]:
            raise ExecutionError("KV store batch, heads or head_dim mismatch")
        if positions.shape != (batch,) or positions.dtype != torch.int64:
            raise ExecutionError("KV store positions must be a one-dimensional int64 batch tensor")
        if positions.device != key.device:
            raise ExecutionError("KV store positions and K/V must live on one device")
        if tokens > self.capacity:
            raise ExecutionError(f"KV store exceeds capacity {self.capacity}")
        (writer or kernels.b200_kv_store)(buffer_key, buffer_value, key, value, positions)
        return self

    def advance(self, slot: int, *, delta: int) -> "PreallocatedKVCacheState":
        """runtime.kv.advance (execution.py:421-443), in place on the slot's length vector."""

        if delta <= 0:
            raise ExecutionError("KV advance delta must be positive")
        _, _, lengths = self._slot(slot)
        kernels.b200_advance_lengths(lengths, delta, self.capacity)
        return self._derive(self.generation + 1)

    def advance_all(self, *, delta: int, slots: Optional[int] = None) -> "PreallocatedKVCacheState":
        """runtime.kv.advance of the first `slots` layer slots (default: all) at once: one launch
        over the length arena when the state owns one, else one per slot. generation grows by
        the number of slots, as if each had been advanced on its own (execution.py:421-443)."""

        count = len(self.keys) if slots is None else int(slots)
        if delta <= 0 or count <= 0 or count > len(self.keys):
            raise ExecutionError("KV advance needs a positive delta and a valid slot count")
        arena = getattr(self, "_length_arena", None)
        if arena is not None:
            kernels.b200_advance_lengths(arena[:count], delta, self.capacity)
        else:
            for slot in range(count):
                kernels.b200_advance_lengths(self.lengths[slot], delta, self.capacity)
        return self._derive(self.generation + count)

    def prefill_store(self, slot: int, key: torch.Tensor, value: torch.Tensor, *,
                      writer: Optional[Callable] = None) -> "PreallocatedKVCacheState":
        """serve.kv.prefill_store (execution.py:405-419): store at the slot's positions (an
        empty slot: zeros) then advance by T. The reference's host check that the slot is
        empty costs a device synchronisation per layer and is left to `check()`."""

        self.store(slot, key, value, self.positions(slot), writer=writer)
        return self.advance(slot, delta=key.shape[2])

    def decode_attention(self, slot: int, query: torch.Tensor, attention_mask: torch.Tensor, *,
                         groups: int, scale: float, runner: Optional[Callable] = None,
                         **options) -> torch.Tensor:
        """serve.decode_attention on the physical buffers (execution.py:281-369)."""

        key_buffer, value_buffer, lengths = self._slot(slot)
        if query.ndim != 4 or query.shape[2] != 1:
            raise ExecutionError("decode attention query must be B x H x 1 x D")
        if attention_mask is not None:
            if attention_mask.ndim != 4 or attention_mask.shape[2] != 1:
                raise ExecutionError("decode attention mask must be B x 1 x 1 x S")
            if attention_mask.shape[0] != query.shape[0]:
                raise ExecutionError("decode attention batch mismatch")
            if attention_mask.shape[-1] > self.capacity:
                raise ExecutionError("decode attention mask is longer than the KV capacity")
        if query.shape[0] != key_buffer.shape[0] or query.shape[3] != key_buffer.shape[3]:
            raise ExecutionError("decode attention batch or head_dim does not match the KV buffer")
        if groups <= 0 or query.shape[1] != key_buffer.shape[2] * groups:
            raise ExecutionError("decode attention GQA groups mismatch")
        run = runner or kernels.b200_decode_attention
        return run(query, key_buffer, value_buffer, lengths, attention_mask, scale=scale,
                   **options)

    def check(self) -> None:
        """Step-boundary host check of the device status word; raises ExecutionError."""

        try:
            kernels.runtime(self.keys[0].device).check_status()
        except kernels.KernelStatusError as error:
            raise ExecutionError(str(error)) from error


class PagedKVCacheState(PreallocatedKVCacheState):
    """The same state ABI over paged storage (layout "paged": the reference's listed future work,
    README.md:295, docs/kv-bufferization.md:319-323): per layer slot `keys[i]` / `values[i]` are
    block POOLS [blocks, block_size, Hkv, D] and one int32 block table [B, max_blocks] shared by
    all slots maps token t of sequence b to row t % block_size of block table[b, t // block_size].
    `capacity` is the logical capacity max_blocks * block_size; lengths, advance, generation and
    the status word work as in the contiguous state, and store / decode_attention keep their
    signatures, so a KernelIR executor drives either layout through the same calls.

    Blocks are handed out by `reserve(tokens_per_sequence)` on the host between steps (a free
    list; a sequence only holds the blocks its length needs, so sequences of very different
    lengths share one pool instead of each owning a slot sized for the longest)."""

    def __post_init__(self) -> None:  # the contiguous layout's shape checks do not apply
        if self.capacity <= 0 or not self.keys or len(self.keys) != len(self.values) or \
                len(self.keys) != len(self.lengths):
            raise ExecutionError("K, V and length slot counts must agree and be non-zero")

    @classmethod
    def allocate_paged(cls, *, num_layers: int, batch: int, max_tokens: int, block_size: int,
                       num_blocks: int, kv_heads: int, head_dim: int, dtype: torch.dtype,
                       device: torch.device | str, extra_length_rows: int = 0) -> "PagedKVCacheState":
        if block_size <= 0 or block_size % 32 != 0:
            raise ExecutionError("the block size must be a positive multiple of 32 tokens")
        max_blocks = -(-max_tokens // block_size)
        key_pool = torch.zeros((num_layers, num_blocks, block_size, kv_heads, head_dim), dtype=dtype,
                               device=device)
        value_pool = torch.zeros_like(key_pool)
        # (extra rows: an engine's own length vectors, advanced by the same launch as the slots')
        length_arena = torch.zeros((num_layers + extra_length_rows, batch), dtype=torch.int64,
                                   device=device)
        state = cls(tuple(key_pool[i] for i in range(num_layers)),
                    tuple(value_pool[i] for i in range(num_layers)),
                    tuple(length_arena[i] for i in range(num_layers)), max_blocks * block_size)
        object.__setattr__(state, "_length_arena", length_arena)
        object.__setattr__(state, "block_size", block_size)
        # unassigned entries point at -1: a store through one raises a status bit instead of writing
        object.__setattr__(state, "block_table",
                           torch.full((batch, max_blocks), -1, dtype=torch.int32, device=device))
        object.__setattr__(state, "_host_table", [[] for _ in range(batch)])
        object.__setattr__(state, "_free", list(range(num_blocks - 1, -1, -1)))
        return state

    def _derive(self, generation: int) -> "PagedKVCacheState":
        state = PagedKVCacheState(self.keys, self.values, self.lengths, self.capacity, generation)
        for name in ("_length_arena", "block_size", "block_table", "_host_table", "_free"):
            object.__setattr__(state, name, getattr(self, name))
        return state

    def reserve(self, tokens_per_sequence: Sequence[int], *, order: Optional[Sequence[int]] = None) -> None:
        """Makes sure sequence b owns blocks for tokens_per_sequence[b] tokens (host-side, between
        steps). `order`: the pool blocks to hand out first (tests use a shuffled order to prove
        that nothing assumes contiguity)."""

        if order is not None:
            taken = {block for row in self._host_table for block in row}
            self._free[:] = [block for block in reversed(list(order)) if block not in taken]
        changed = False
        for b, tokens in enumerate(tokens_per_sequence):
            need = -(-int(tokens) // self.block_size)
            if need > self.block_table.shape[1]:
                raise ExecutionError(f"sequence {b} needs {tokens} tokens, beyond the paged capacity "
                                     f"{self.capacity}")
            while len(self._host_table[b]) < need:
                if not self._free:
                    raise ExecutionError("the KV block pool is exhausted")
                self._host_table[b].append(self._free.pop())
                changed = True
        if changed:
            host = torch.full(tuple(self.block_table.shape), -1, dtype=torch.int32)
            for b, row in enumerate(self._host_table):
                host[b, :len(row)] = torch.tensor(row, dtype=torch.int32)
            self.block_table.copy_(host)

    def release(self, sequence: int) -> None:
        """Returns a finished sequence's blocks to the pool and empties its lengths."""

        self._free.extend(reversed(self._host_table[sequence]))
        self._host_table[sequence] = []
        self.block_table[sequence].fill_(-1)
        self._length_arena[:, sequence].zero_()

    def blocks_in_use(self) -> int:
        return sum(len(row) for row in self._host_table)

    def read(self, slot: int) -> Tuple[torch.Tensor, torch.Tensor]:
        raise ExecutionError("a paged KV state has no contiguous logical view; gather through block_table")

    def gather(self, slot: int, sequence: int, tokens: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """The first `tokens` K and V rows of one sequence as dense T x H x D tensors (a host-driven
        debugging / test helper: index_select on the pools)."""

        blocks = torch.tensor(self._host_table[sequence], dtype=torch.int64, device=self.keys[slot].device)
        keys = self.keys[slot].index_select(0, blocks).flatten(0, 1)[:tokens]
        values = self.values[slot].index_select(0, blocks).flatten(0, 1)[:tokens]
        return keys, values

    def store(self, slot: int, key: torch.Tensor, value: torch.Tensor, positions: torch.Tensor, *,
              writer: Optional[Callable] = None) -> "PagedKVCacheState":
        pool_key, pool_value, _ = self._slot(slot)
        if key.shape != value.shape or key.ndim != 4:
            raise ExecutionError("KV store needs K and V of one B x H x T x D shape")
        if key.shape[0] != self.block_table.shape[0] or key.shape[1] != pool_key.shape[2] or \
                key.shape[3] != pool_key.shape[3]:
            raise ExecutionError("KV store batch, heads or head_dim mismatch")
        if positions.shape != (key.shape[0],) or positions.dtype != torch.int64:
            raise ExecutionError("KV store positions must be a one-dimensional int64 batch tensor")
        if key.shape[2] > self.capacity:
            raise ExecutionError(f"KV store exceeds capacity {self.capacity}")
        if writer is not None:
            writer(pool_key, pool_value, self.block_table, key, value, positions)
        else:
            kernels.b200_paged_kv_store(pool_key, pool_value, self.block_table, key, value, positions)
        return self

    def decode_attention(self, slot: int, query: torch.Tensor, attention_mask: torch.Tensor, *,
                         groups: int, scale: float, runner: Optional[Callable] = None,
                         **options) -> torch.Tensor:
        pool_key, pool_value, lengths = self._slot(slot)
        if query.ndim != 4 or query.shape[2] != 1:
            raise ExecutionError("decode attention query must be B x H x 1 x D")
        if attention_mask is not None and (attention_mask.ndim != 4 or attention_mask.shape[2] != 1 or
                                           attention_mask.shape[-1] > self.capacity):
            raise ExecutionError("decode attention mask must be B x 1 x 1 x S with S <= capacity")
        if groups <= 0 or query.shape[1] != pool_key.shape[2] * groups or \
                query.shape[3] != pool_key.shape[3]:
            raise ExecutionError("decode attention GQA groups or head_dim mismatch")
        if options.get("split_tokens") is None:  # (None = "the packaged plan": built-in here)
            options.pop("split_tokens", None)
        run = runner or kernels.b200_paged_decode_attention
        return run(query, pool_key, pool_value, self.block_table, lengths, attention_mask, scale=scale,
                   **options)
