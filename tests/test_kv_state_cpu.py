"""Host-side logic of the KV states that needs no GPU: the paged state's block allocator (free
list, block table, exhaustion, capacity) and the argument checks that run before any launch."""

import pytest
import torch

from llm_compiler_b200.kv_state import ExecutionError, PagedKVCacheState, PreallocatedKVCacheState


def paged(batch=4, max_tokens=2048, block_size=128, num_blocks=32, layers=2, extra=0):
    return PagedKVCacheState.allocate_paged(
        num_layers=layers, batch=batch, max_tokens=max_tokens, block_size=block_size,
        num_blocks=num_blocks, kv_heads=2, head_dim=64, dtype=torch.bfloat16, device="cpu",
        extra_length_rows=extra)


def test_blocks_are_handed_out_on_demand_and_returned():
    state = paged()
    assert state.capacity == 2048 and state.block_table.shape == (4, 16)
    assert torch.all(state.block_table == -1) and state.blocks_in_use() == 0
    state.reserve([2000, 100, 64, 1500])
    assert state.blocks_in_use() == 16 + 1 + 1 + 12
    table = state.block_table
    used = table[table >= 0]
    assert used.numel() == 30 and used.unique().numel() == 30  # no block handed out twice
    assert torch.all(table[1, 1:] == -1) and torch.all(table[0] >= 0)
    state.reserve([2000, 100, 64, 1500])  # nothing new is needed: the table stays as it is
    assert torch.equal(state.block_table, table) and state.blocks_in_use() == 30
    with pytest.raises(ExecutionError, match="exhausted"):
        state.reserve([2000, 700, 64, 1500])  # 5 more blocks, 2 left
    state.release(0)
    assert state.blocks_in_use() <= 16 and torch.all(state.block_table[0] == -1)
    state.reserve([0, 2048, 64, 1500])  # the returned blocks serve sequence 1 now
    assert state.blocks_in_use() == 16 + 1 + 12
    with pytest.raises(ExecutionError, match="beyond the paged capacity"):
        state.reserve([4096, 0, 0, 0])


def test_a_requested_block_order_is_followed():
    state = paged(batch=2, max_tokens=512, num_blocks=8)
    state.reserve([256, 384], order=[5, 2, 7, 0, 3, 1, 6, 4])
    assert state.block_table[0, :2].tolist() == [5, 2] and state.block_table[1, :3].tolist() == [7, 0, 3]


def test_block_size_must_be_a_multiple_of_the_copy_step():
    with pytest.raises(ExecutionError, match="multiple of 32"):
        paged(block_size=48)


def test_extra_length_rows_share_the_arena():
    state = paged(layers=3, extra=2)
    assert state._length_arena.shape == (5, 4) and len(state.lengths) == 3
    state._length_arena[3].fill_(7)  # an engine's own row: not a slot
    assert all(int(l.sum()) == 0 for l in state.lengths)


def test_a_paged_state_has_no_contiguous_view():
    state = paged()
    with pytest.raises(ExecutionError, match="no contiguous logical view"):
        state.read(0)


def test_contiguous_state_checks_its_slots_before_any_launch():
    keys = tuple(torch.zeros(2, 64, 2, 16) for _ in range(2))
    lengths = tuple(torch.zeros(2, dtype=torch.int64) for _ in range(2))
    state = PreallocatedKVCacheState(keys, keys, lengths, 64)
    with pytest.raises(ExecutionError):
        state._slot(2)
    with pytest.raises(ExecutionError):
        PreallocatedKVCacheState(keys, keys[:1], lengths, 64)


def test_decode_chain_rows_and_service_order_helpers():
    from llm_compiler_b200 import kernels

    assert kernels.decode_chain_rows(torch.empty(9728, 896, dtype=torch.bfloat16)) == 128  # 17 MB
    assert kernels.decode_chain_rows(torch.empty(37888, 3584, dtype=torch.bfloat16, device="meta")) == 64
    assert kernels.decode_chain_rows(32 << 20) == 128 and kernels.decode_chain_rows((32 << 20) + 1) == 64
    lengths = torch.tensor([5, 900, 17, 900, 3])
    order = kernels.sequence_order_of(lengths)
    assert order.dtype == torch.int32 and order.tolist() == [1, 3, 2, 0, 4]  # longest first, stable
