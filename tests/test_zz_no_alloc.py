"""The decode-attention entry point that allocates nothing, called through the C ABI.

Who needs it: callers that cannot let a call reach cudaMalloc (or torch's caching
allocator) -- a step under CUDA-graph capture, a serving loop with a memory budget frozen at
start-up, a plugin that only owns the arena its host framework gave it. For them the
split-KV scratch is a fixed 8 MiB array inside the library instead of a workspace buffer.

The test runs two calls in a row (the array keeps the first call's contents, so the second
call proves the counters are cleared and stale partials are not picked up) and compares each
with the workspace entry point on the same inputs, bit for bit: both entry points run the same
kernel with the same split plan, only the scratch location differs, so any difference at all
would be a stale partial or a counter slip. The first case is also checked against the CPU
oracle within the bf16 tolerance of the other attention tests (2e-2). Different shapes are used
for the two calls on purpose. It also checks that an oversized request is refused, not truncated. The
file is named so that pytest collects it last: a failure here cannot hide any other test.
"""

import pytest
import torch

from oracle import serve_ops
import llm_compiler_b200 as b200
from llm_compiler_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


def allocation_events():
    """How many blocks torch's CUDA allocator has handed out so far (a monotonic counter)."""
    return torch.cuda.memory_stats().get("allocation.all.allocated", 0)


def make_case(seed, batch, capacity, lengths):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, 1, 14, 64, generator=g).bfloat16().transpose(1, 2).cuda()
    k = torch.randn(batch, capacity, 2, 64, generator=g).bfloat16().cuda()
    v = torch.randn(batch, capacity, 2, 64, generator=g).bfloat16().cuda()
    return q, k, v, torch.tensor(lengths, device="cuda")


def test_no_alloc_entry_point_matches_workspace_entry_point_twice_in_a_row():
    assert _lib.load().b200_decode_attention_static_scratch_bytes() == 8 << 20
    cases = [
        # several splits per sequence, ragged lengths (one sequence shorter than a split)
        (make_case(1, 5, 1500, [1500, 700, 64, 1, 1333]), 256),
        # other shape, other split count: must not see the first call's partials or counters
        (make_case(2, 3, 900, [900, 10, 450]), 128),
    ]
    kernels.runtime()  # the per-GPU status word exists before allocations are counted
    for index, ((q, k, v, lengths), split) in enumerate(cases):
        expected = b200.b200_decode_attention(q, k, v, lengths, None, scale=0.125,
                                              split_tokens=split)
        output = torch.full_like(expected, float("nan"))
        before = allocation_events()
        result = b200.b200_decode_attention_no_alloc(q, k, v, lengths, None, output, scale=0.125,
                                                     split_tokens=split)
        assert allocation_events() == before  # the call made no request to torch's allocator
        assert result.data_ptr() == output.data_ptr()
        # same kernel, same split plan: only the scratch location differs
        assert torch.equal(output, expected)
        assert not torch.isnan(output).any()
        if index == 0:
            mask = torch.zeros(q.shape[0], 1, 1, k.shape[1])
            reference = serve_ops.decode_attention(q.cpu(), k.cpu(), v.cpu(), lengths.cpu(), mask,
                                                   groups=7, scale=0.125)
            torch.testing.assert_close(output.float().cpu(), reference.float(), rtol=0, atol=2e-2)
    kernels.runtime().check_status()


def test_no_alloc_entry_point_with_mask_and_single_split():
    q, k, v, lengths = make_case(3, 2, 300, [300, 120])
    mask = torch.zeros(2, 1, 1, 300, device="cuda")
    mask[:, :, :, ::5] = float("-inf")
    for split in (64, 4096):  # many splits; one split (no scratch used at all)
        expected = b200.b200_decode_attention(q, k, v, lengths, mask, scale=0.125,
                                              split_tokens=split)
        output = torch.empty_like(expected)
        b200.b200_decode_attention_no_alloc(q, k, v, lengths, mask, output, scale=0.125,
                                            split_tokens=split)
        assert torch.equal(output, expected)


def test_no_alloc_entry_point_refuses_what_does_not_fit():
    # 256 sequences x 14 heads x 64 splits x 66 floats = 60 MB of partials: far beyond 8 MiB
    q, k, v, lengths = make_case(4, 256, 2048, [2048] * 256)
    output = torch.empty(256, 14, 1, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="do not fit"):
        b200.b200_decode_attention_no_alloc(q, k, v, lengths, None, output, scale=0.125,
                                            split_tokens=32)
    # with a split that fits, the same inputs go through
    b200.b200_decode_attention_no_alloc(q, k, v, lengths, None, output, scale=0.125,
                                        split_tokens=1024)
    expected = b200.b200_decode_attention(q, k, v, lengths, None, scale=0.125, split_tokens=1024)
    assert torch.equal(output, expected)
    kernels.runtime().check_status()
