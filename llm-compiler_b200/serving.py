"""Batch-partitioned replica serving across the GPUs of one box.

Sequences are independent units (own KV slot, length, position and mask row), so the
global batch is cut into contiguous slices, one process per GPU, each holding a full
weight replica, its own KV arena and its own CUDA graph. No kernel reads another GPU's
memory. The only exchange is an all-gather of the sampled token ids (int64, <= 4 KiB per
step at a global batch of 512), done with torch.distributed (NCCL on GPUs, Gloo in the CPU
tests) into a preallocated buffer. The reference has no distributed code at all; this is
the data-parallel layer the B200 deployment adds.


Failure detection is host-side and happens between steps (`FailureMonitor`): every rank
publishes a heartbeat (the step it is about to run) in the process group's store; before a
collective a rank checks that nobody has reported a failure and that every peer has reached the
same step, and gives up with ExecutionError after a timeout instead of entering a collective
that a lost rank would never join. A rank whose engine raises reports that before re-raising.
No GPU fault is ever provoked or relied on; kernels and collectives in flight are never
abandoned (a rank leaves only between steps).
"""

from __future__ import annotations

import time
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from .kv_state import ExecutionError


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


class ReplicaFailure(ExecutionError):
    """A peer replica reported a failure or stopped answering between steps."""


class FailureMonitor:
    """Host-side liveness protocol over a torch.distributed store (TCPStore / FileStore / the
    process group's own): heartbeats and failure reports are keys, nothing touches a GPU.

    beat(step)          publish "this rank is about to run `step`"
    report(reason)      publish a failure (first report wins) -- call before raising
    check(step)         raise ReplicaFailure if a failure was reported, or if some peer has not
                        published a heartbeat >= step within `timeout_s`
    """

    def __init__(self, store, rank: int, world_size: int, *, timeout_s: float = 10.0,
                 poll_s: float = 0.002, prefix: str = "b200/serving") -> None:
        self.store, self.rank, self.world_size = store, rank, world_size
        self.timeout_s, self.poll_s, self.prefix = timeout_s, poll_s, prefix
        self._seen = [-1] * world_size  # last step each peer was known to have reached

    def _key(self, name: str) -> str:
        return f"{self.prefix}/{name}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(f"heartbeat/{self.rank}"), str(int(step)))
        self._seen[self.rank] = int(step)

    def report(self, reason: str) -> None:
        if not self.store.check([self._key("failed")]):
            self.store.set(self._key("failed"), f"{self.rank}:{reason}")

    def failure(self) -> Optional[str]:
        if self.store.check([self._key("failed")]):
            return self.store.get(self._key("failed")).decode()
        return None

    def check(self, step: int) -> None:
        deadline = time.monotonic() + self.timeout_s
        while True:
            failed = self.failure()
            if failed is not None:
                rank, _, reason = failed.partition(":")
                raise ReplicaFailure(f"replica {rank} reported a failure before step {step}: {reason}")
            behind = []
            for peer in range(self.world_size):
                if self._seen[peer] >= step:
                    continue
                key = self._key(f"heartbeat/{peer}")
                if self.store.check([key]):
                    self._seen[peer] = int(self.store.get(key).decode())
                if self._seen[peer] < step:
                    behind.append(peer)
            if not behind:
                return
            if time.monotonic() >= deadline:
                raise ReplicaFailure(
                    f"replicas {behind} did not reach step {step} within {self.timeout_s} s "
                    f"(last seen at steps {[self._seen[p] for p in behind]})")
            time.sleep(self.poll_s)


class ReplicaServer:
    """One rank of the batch-partitioned deployment: a local engine plus the token gather and,
    when there are several ranks, the failure monitor: every `check_every` steps (and at step 0)
    the rank publishes its heartbeat and checks its peers before entering the collective."""

    def __init__(self, engine, global_batch: int, *, group: Optional[dist.ProcessGroup] = None,
                 device: torch.device | str | None = None, store=None, check_every: int = 32,
                 failure_timeout_s: float = 10.0) -> None:
        self.engine = engine
        device = device if device is not None else engine.device
        self.tokens = TokenGather(global_batch, device=device, group=group)
        if engine.batch != self.tokens.local.size:
            raise ValueError("engine batch does not match this rank's slice of the global batch")
        self.step_index = 0
        self.check_every = max(1, int(check_every))
        self.monitor: Optional[FailureMonitor] = None
        if self.tokens.world_size > 1:
            if store is None:
                store = dist.distributed_c10d._get_default_store()
            self.monitor = FailureMonitor(store, self.tokens.rank, self.tokens.world_size,
                                          timeout_s=failure_timeout_s)

    @property
    def local_slice(self) -> BatchSlice:
        return self.tokens.local

    def _guard(self) -> None:
        """After this rank's own step has been issued and before the step's collective: every
        replica must have got as far (a replica that failed in its step never publishes this
        heartbeat, it publishes a failure). With check_every > 1 a failure inside an unchecked
        step surfaces as the process group's own collective timeout instead."""
        if self.monitor is not None and self.step_index % self.check_every == 0:
            self.monitor.beat(self.step_index)
            self.monitor.check(self.step_index)

    def local_step(self) -> torch.Tensor:
        """The engine's decode step; a failure is reported to the other replicas before it is
        re-raised, so that they do not enter a collective this rank will never join."""
        try:
            return self.engine.decode_step()
        except Exception as error:
            if self.monitor is not None:
                self.monitor.report(f"{type(error).__name__}: {error}")
            raise

    def decode_step(self, *, gather: bool = True) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        local = self.local_step()
        if gather:
            self._guard()
        self.step_index += 1
        return local, (self.tokens.gather(local) if gather else None)

    def gather_async(self, local_tokens: torch.Tensor):
        """The all-gather of this step's tokens as an asynchronous work item (None with one
        rank); the gathered ids are in `self.tokens.padded` once it has been waited for."""
        self._guard()
        self.step_index += 1
        if self.tokens.world_size == 1:
            return None
        self.tokens.send[:self.tokens.local.size].copy_(local_tokens)
        return dist.all_gather_into_tensor(self.tokens.padded, self.tokens.send,
                                           group=self.tokens.group, async_op=True)

    def gather_host(self, local_tokens: torch.Tensor) -> torch.Tensor:
        """Blocking gather for a host-driven loop: returns the global token vector."""
        self._guard()
        self.step_index += 1
        return self.tokens.gather(local_tokens)
