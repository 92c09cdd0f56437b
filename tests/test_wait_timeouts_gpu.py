"""The give-up paths of the bounded in-kernel waits, one kernel family at a time.

No GPU is faulted, trapped or hung: the library's debug switch makes the copy-issuing threads of
the TMA / tcgen05 kernels issue nothing (so no copy is in flight) and shortens the poll limit of
every mbarrier wait, so each wait runs out at once. The kernel must then raise
B200_STATUS_WAIT_TIMEOUT, free its tensor memory and return; the very next call, with the
defaults restored, must work and be correct (which it could not if tensor memory had leaked or a
barrier had been left armed)."""

import contextlib

import pytest
import torch

from oracle import serve_ops
import llm_compiler_b200 as b200
from llm_compiler_b200 import _lib, kernels

pytestmark = pytest.mark.gpu


@contextlib.contextmanager
def waits_that_run_out():
    library = _lib.load()
    previous = library.b200_debug_set_waits(2000, 1)
    assert previous > 0
    try:
        yield
    finally:
        library.b200_debug_set_waits(previous, 0)
        torch.cuda.synchronize()


def expect_timeout():
    with pytest.raises(kernels.KernelStatusError, match="bounded in-kernel wait gave up"):
        kernels.runtime().check_status()
    kernels.runtime().check_status()  # cleared


def close(actual, expected, tol=2e-2):
    scale = max(1.0, float(expected.float().abs().max()))
    assert float((actual.float().cpu() - expected.float()).abs().max()) <= tol * scale


@pytest.mark.parametrize("rows", [64, 2048])
def test_linear_tcgen05_wait_timeout_then_recovery(rows):
    g = torch.Generator().manual_seed(rows)
    x = torch.randn(rows, 896, generator=g).bfloat16()
    w = (torch.randn(9728, 896, generator=g) * 0.03).bfloat16()
    for _ in range(3):  # repeated give-ups must not exhaust tensor memory either
        with waits_that_run_out():
            kernels.b200_linear(x.cuda(), w.cuda())
        expect_timeout()
    close(kernels.b200_linear(x.cuda(), w.cuda()), serve_ops.linear(x, w))
    kernels.runtime().check_status()


def test_cluster_split_k_and_partial_wait_timeout_then_recovery():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 4864, generator=g).bfloat16()
    w = (torch.randn(896, 4864, generator=g) * 0.02).bfloat16()
    residual = torch.randn(64, 896, generator=g).bfloat16()
    with waits_that_run_out():
        kernels.b200_linear_splitk_residual(x.cuda(), w.cuda(), residual.cuda())
        kernels.b200_linear_partial(x.cuda(), w.cuda())
    expect_timeout()
    out = kernels.b200_linear_splitk_residual(x.cuda(), w.cuda(), residual.cuda())
    close(out, serve_ops.residual_add(residual, serve_ops.linear(x, w)))
    kernels.runtime().check_status()


def test_prefill_attention_tcgen05_wait_timeout_then_recovery():
    g = torch.Generator().manual_seed(6)
    q = torch.randn(2, 300, 14, 64, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(2, 300, 2, 64, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(2, 300, 2, 64, generator=g).bfloat16().transpose(1, 2)
    mask = serve_ops.causal_mask(2, 300)
    with waits_that_run_out():
        b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), None, scale=0.125, causal=True)
        b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), mask.cuda(), scale=0.125)
    expect_timeout()
    ref = serve_ops.prefill_attention(q, k, v, mask, groups=7, scale=0.125)
    close(b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), None, scale=0.125, causal=True), ref)
    close(b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), mask.cuda(), scale=0.125), ref)
    kernels.runtime().check_status()


def test_decode_attention_wait_timeout_then_recovery():
    g = torch.Generator().manual_seed(7)
    q = torch.randn(4, 1, 14, 64, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(4, 1024, 2, 64, generator=g).bfloat16()
    v = torch.randn(4, 1024, 2, 64, generator=g).bfloat16()
    lengths = torch.tensor([1024, 300, 64, 777])
    with waits_that_run_out():
        b200.b200_decode_attention(q.cuda(), k.cuda(), v.cuda(), lengths.cuda(), None, scale=0.125,
                                   split_tokens=256)
    expect_timeout()
    ref = serve_ops.decode_attention(q, k, v, lengths, torch.zeros(4, 1, 1, 1024), groups=7, scale=0.125)
    close(b200.b200_decode_attention(q.cuda(), k.cuda(), v.cuda(), lengths.cuda(), None, scale=0.125,
                                     split_tokens=256), ref)
    kernels.runtime().check_status()
