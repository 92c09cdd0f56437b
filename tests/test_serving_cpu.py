"""Host-side logic of the batch-partitioned deployment, run as two Gloo ranks on CPU:
batch slicing, the token all-gather into a preallocated buffer, lock-step decoding of
replicas over a fake engine, and a rank that fails between steps (raised on the host;
the survivor learns of it through the store before its next collective)."""

import multiprocessing as mp
import os
import socket

import pytest
import torch
import torch.distributed as dist

from llm_compiler_b200.serving import (ReplicaFailure, ReplicaServer, TokenGather,
                                       balanced_assignment, partition_batch)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_partition_covers_the_batch_without_overlap():
    for batch, world in [(512, 8), (64, 1), (10, 4), (7, 7), (513, 8)]:
        slices = [partition_batch(batch, world, r) for r in range(world)]
        assert slices[0].start == 0 and slices[-1].stop == batch
        assert all(a.stop == b.start for a, b in zip(slices, slices[1:]))
        assert max(s.size for s in slices) - min(s.size for s in slices) <= 1
    with pytest.raises(ValueError):
        partition_batch(3, 4, 0)
    with pytest.raises(ValueError):
        partition_batch(8, 4, 4)


def test_balanced_assignment_evens_out_context_lengths():
    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(1024, 8193, (512,), generator=g).tolist()
    buckets = balanced_assignment(lengths, 8)
    assert sorted(i for b in buckets for i in b) == list(range(512))
    sums = [sum(lengths[i] for i in b) for b in buckets]
    assert all(len(b) == 64 for b in buckets)
    assert (max(sums) - min(sums)) / (sum(sums) / 8) < 0.01


class FakeEngine:
    """Stands in for Qwen2Engine on CPU: next token = (id * 3 + position) mod 1000."""

    def __init__(self, ids):
        self.batch = ids.shape[0]
        self.device = torch.device("cpu")
        self.ids = ids.clone()
        self.position = 0

    def decode_step(self):
        if getattr(self, "fail_at", None) == self.position:
            raise RuntimeError("injected host-side failure")
        self.ids = (self.ids * 3 + self.position) % 1000
        self.position += 1
        return self.ids


def _worker(rank, world, port, global_batch, fail_rank, queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        all_ids = torch.arange(global_batch, dtype=torch.int64) * 7 % 1000
        piece = partition_batch(global_batch, world, rank)
        engine = FakeEngine(all_ids[piece.start:piece.stop])
        if fail_rank == rank:
            engine.fail_at = 2
        if fail_rank == "silent" and rank == 1:
            engine.vanish_at = 2
        # the product's own failure protocol (serving.FailureMonitor inside ReplicaServer): a
        # rank whose engine raises reports it on the host before leaving; the others check
        # before their next collective and stop cleanly; a rank that just stops answering is
        # found by the heartbeat timeout
        server = ReplicaServer(engine, global_batch, check_every=1, failure_timeout_s=3.0)
        reference = FakeEngine(all_ids)
        gathered = []
        for step in range(4):
            if getattr(engine, "vanish_at", None) == step:
                queue.put((rank, "vanished", step))  # leaves between steps without a word
                return
            _, full = server.decode_step()
            expected = reference.decode_step()
            assert torch.equal(full, expected), (rank, step)
            gathered.append(full.clone())
        queue.put((rank, "ok", len(gathered)))
    except ReplicaFailure as error:
        queue.put((rank, "stopped", str(error)))
    except RuntimeError as error:
        queue.put((rank, "raised", str(error)))
    finally:
        dist.destroy_process_group()


def _run(world, global_batch, fail_rank=None):
    context = mp.get_context("spawn")
    queue = context.Queue()
    port = free_port()
    procs = [context.Process(target=_worker, args=(r, world, port, global_batch, fail_rank, queue))
             for r in range(world)]
    for p in procs:
        p.start()
    results = [queue.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    return sorted(results)


@pytest.mark.parametrize("global_batch", [8, 7])
def test_two_ranks_gather_tokens_in_lock_step(global_batch):
    results = _run(2, global_batch)
    assert results == [(0, "ok", 4), (1, "ok", 4)]


def test_rank_failure_between_steps_is_seen_on_the_host():
    results = _run(2, 8, fail_rank=1)
    assert results[0][:2] == (0, "stopped") and "replica 1 reported a failure" in results[0][2]
    assert "injected host-side failure" in results[0][2]
    assert results[1][:2] == (1, "raised")


def test_rank_that_stops_answering_is_found_by_the_heartbeat_timeout():
    results = _run(2, 8, fail_rank="silent")
    assert results[0][:2] == (0, "stopped") and "did not reach step 2" in results[0][2]
    assert results[1] == (1, "vanished", 2)


def test_failure_monitor_on_a_plain_store():
    """The protocol itself, on an in-process HashStore: no process group needed."""
    from llm_compiler_b200.serving import FailureMonitor

    store = dist.HashStore()
    a = FailureMonitor(store, 0, 2, timeout_s=0.2)
    b = FailureMonitor(store, 1, 2, timeout_s=0.2)
    a.beat(0)
    with pytest.raises(ReplicaFailure, match=r"replicas \[1\] did not reach step 0"):
        a.check(0)
    b.beat(0)
    a.check(0)
    b.check(0)
    b.beat(5)
    a.beat(3)
    a.check(3)  # a peer that is ahead is fine
    b.report("out of memory")
    a.report("second report loses")
    with pytest.raises(ReplicaFailure, match="replica 1 reported a failure before step 4: out of memory"):
        a.check(4)


def test_single_process_gather_is_a_copy():
    gather = TokenGather(5, device="cpu")
    tokens = torch.arange(5)
    assert torch.equal(gather.gather(tokens), tokens)
    with pytest.raises(ValueError):
        gather.gather(torch.arange(4))
