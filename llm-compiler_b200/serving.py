"""Batch-partitioned replica serving across the GPUs of one box.

Sequences are independent units (own KV slot, length, position and mask row), so the
global batch is cut into contiguous slices, one process per GPU, each holding a full
weight replica, its own KV arena and its own CUDA graph. No kernel reads another GPU's
memory. The only exchange is an all-gather of the sampled token ids (int64, <= 4 KiB per
step at a global batch of 512), done with torch.distributed (NCCL on GPUs, Gloo in the CPU
tests) into a preallocated buffer. The reference has no distributed code at all; this is
the data-parallel layer the B200 deployment adds.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class BatchSlice:
    rank: int
    world_size: int
    start: int
    stop: int

    @property
    def size(self) -> int:
        return self.stop - self.start


def partition_batch(global_batch: int, world_size: int, rank: int) -> BatchSlice:
    """Contiguous slice of the global batch for `rank`; the remainder goes to the first ranks."""

    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("rank must lie in [0, world_size)")
    if global_batch < world_size:
        raise ValueError("every rank needs at least one sequence")
    base, extra = divmod(global_batch, world_size)
    start = rank * base + min(rank, extra)
    return BatchSlice(rank, world_size, start, start + base + (1 if rank < extra else 0))


def balanced_assignment(lengths: List[int], world_size: int) -> List[List[int]]:
    """Assigns sequences to ranks so that every rank gets the same number of sequences
    (+-1) and a near-equal sum of context lengths: sort by length, deal in a snake order.
    Decode time per rank is proportional to the KV bytes it streams, so balancing the
    length sums balances the step time across replicas."""

    order = sorted(range(len(lengths)), key=lambda i: -lengths[i])
    buckets: List[List[int]] = [[] for _ in range(world_size)]
    for position, index in enumerate(order):
        lap, offset = divmod(position, world_size)
        rank = offset if lap % 2 == 0 else world_size - 1 - offset
        buckets[rank].append(index)
    return buckets


class TokenGather:
    """All-gather of per-rank token ids into one preallocated [global_batch] int64 buffer."""

    def __init__(self, global_batch: int, *, device: torch.device | str,
                 group: Optional[dist.ProcessGroup] = None) -> None:
        self.group = group
        self.world_size = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.slices = [partition_batch(global_batch, self.world_size, r)
                       for r in range(self.world_size)]
        self.local = self.slices[self.rank]
        self.uniform = len({s.size for s in self.slices}) == 1
        self.width = max(s.size for s in self.slices)
        self.padded = torch.zeros(self.world_size * self.width, dtype=torch.int64, device=device)
        self.send = torch.zeros(self.width, dtype=torch.int64, device=device)
        self.output = torch.zeros(global_batch, dtype=torch.int64, device=device)

    def gather(self, local_tokens: torch.Tensor) -> torch.Tensor:
        if local_tokens.shape != (self.local.size,):
            raise ValueError("local token vector does not match this rank's batch slice")
        if self.world_size == 1:
            self.output.copy_(local_tokens)
            return self.output
        self.send[:self.local.size].copy_(local_tokens)
        dist.all_gather_into_tensor(self.padded, self.send, group=self.group)
        if self.uniform:
            self.output.copy_(self.padded)
        else:
            for piece in self.slices:
                begin = piece.rank * self.width
                self.output[piece.start:piece.stop].copy_(self.padded[begin:begin + piece.size])
        return self.output


class ReplicaServer:
    """One rank of the batch-partitioned deployment: a local engine plus the token gather."""

    def __init__(self, engine, global_batch: int, *, group: Optional[dist.ProcessGroup] = None,
                 device: torch.device | str | None = None) -> None:
        self.engine = engine
        device = device if device is not None else engine.device
        self.tokens = TokenGather(global_batch, device=device, group=group)
        if engine.batch != self.tokens.local.size:
            raise ValueError("engine batch does not match this rank's slice of the global batch")

    @property
    def local_slice(self) -> BatchSlice:
        return self.tokens.local

    def decode_step(self, *, gather: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        local = self.engine.decode_step()
        return local, (self.tokens.gather(local) if gather else None)
