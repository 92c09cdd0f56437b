"""Parity of every CUDA kernel, called through the C ABI, against the reference.

Three layers of evidence per operator:
  1. the committed golden outputs of the reference's own CPU executor (tests/golden/ops.pt)
     on the seeded inputs of tests/golden/cases.py;
  2. the CPU oracle (oracle/serve_ops.py, itself pinned to those goldens) on further seeded
     inputs: ragged lengths, length 0 and length == capacity, odd sizes, strided operands;
  3. size-independent properties at the benchmark's full shapes (store -> read-back round
     trip, invariance of decode attention to the number of KV splits).

Tolerances: KV store, RoPE and pytorch_compatible RMSNorm are bit-exact; fp32 kernels
3e-5; bf16 attention / GEMM 2e-2 (max abs and relative to the output scale).
"""

import pytest
import torch

import cases
from oracle import serve_ops
import llm_compiler_b200 as b200
from llm_compiler_b200 import kernels

pytestmark = pytest.mark.gpu

BF16_TOL = 2e-2
F32_TOL = 3e-5


def dev(x):
    return x.cuda() if isinstance(x, torch.Tensor) else x


def exact(actual, expected):
    torch.testing.assert_close(actual.cpu(), expected, rtol=0, atol=0, equal_nan=True)


def close(actual, expected, tol):
    actual = actual.float().cpu()
    expected = expected.float()
    assert actual.shape == expected.shape
    assert torch.equal(torch.isnan(actual), torch.isnan(expected))
    scale = max(1.0, float(expected.nan_to_num().abs().max()))
    diff = (actual - expected).nan_to_num().abs().max().item()
    assert diff <= tol * scale, f"max abs diff {diff} > {tol} * {scale}"


def tol_for(dtype):
    return F32_TOL if dtype == torch.float32 else BF16_TOL


# ------------------------------------------------------------------------ KV store ----
@pytest.mark.parametrize("name", list(cases.KV_STORE))
def test_kv_store_golden(name, golden_ops):
    x = cases.kv_store_inputs(name)
    kbuf, vbuf = dev(x["key_buffer"]), dev(x["value_buffer"])
    b200.b200_kv_store(kbuf, vbuf, dev(x["key"]), dev(x["value"]), dev(x["positions"]))
    exact(kbuf, golden_ops[name]["key_out"])
    exact(vbuf, golden_ops[name]["value_out"])
    kernels.runtime().check_status()


def test_kv_store_ragged_edges():
    g = torch.Generator().manual_seed(3)
    b, c, h, d, t = 5, 33, 2, 64, 4
    kbuf = torch.randn(b, c, h, d, generator=g).bfloat16()
    vbuf = torch.randn(b, c, h, d, generator=g).bfloat16()
    key = torch.randn(b, t, h, d, generator=g).bfloat16().transpose(1, 2)
    value = torch.randn(b, h, t, d, generator=g).bfloat16()  # contiguous B,H,T,D
    positions = torch.tensor([0, c - t, 7, 1, 20])  # first row, last legal row, ragged
    k_ref, v_ref = kbuf.clone(), vbuf.clone()
    serve_ops.kv_store(k_ref, v_ref, key, value, positions)
    k_dev, v_dev = kbuf.cuda(), vbuf.cuda()
    b200.b200_kv_store(k_dev, v_dev, key.cuda(), value.cuda(), positions.cuda())
    exact(k_dev, k_ref)
    exact(v_dev, v_ref)
    kernels.runtime().check_status()


def test_kv_store_overflow_sets_status_and_skips():
    kbuf = torch.zeros(2, 8, 2, 64, dtype=torch.bfloat16, device="cuda")
    vbuf = torch.zeros_like(kbuf)
    key = torch.ones(2, 2, 3, 64, dtype=torch.bfloat16, device="cuda")
    positions = torch.tensor([6, 1], device="cuda")  # row 0: tokens 6, 7 fit, 8 does not
    b200.b200_kv_store(kbuf, vbuf, key, key, positions)
    with pytest.raises(b200.KernelStatusError):
        kernels.runtime().check_status()
    assert kbuf[0, 6:8].eq(1).all() and kbuf[1, 1:4].eq(1).all()
    assert kbuf[0, :6].eq(0).all() and kbuf[1, 4:].eq(0).all()
    kernels.runtime().check_status()  # cleared


def test_kv_store_round_trip_full_size():
    """Benchmark shape (batch 16 x 4096 tokens into capacity 8192): store then read back."""
    b, c, h, d, t = 16, 8192, 2, 64, 4096
    g = torch.Generator(device="cuda").manual_seed(1)
    kbuf = torch.zeros(b, c, h, d, dtype=torch.bfloat16, device="cuda")
    vbuf = torch.zeros_like(kbuf)
    key = torch.randn(b, t, h, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
    value = torch.randn(b, t, h, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
    positions = torch.zeros(b, dtype=torch.int64, device="cuda")
    b200.b200_kv_store(kbuf, vbuf, key, value, positions)
    assert torch.equal(kbuf[:, :t].transpose(1, 2), key)
    assert torch.equal(vbuf[:, :t].transpose(1, 2), value)
    assert kbuf[:, t:].eq(0).all()
    # one decode append at position T (config 3 of the benchmark plan)
    positions.fill_(t)
    step = torch.randn(b, 1, h, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
    b200.b200_kv_store(kbuf, vbuf, step, step, positions)
    assert torch.equal(kbuf[:, t], step[:, :, 0]) and torch.equal(kbuf[:, :t].transpose(1, 2), key)
    kernels.runtime().check_status()


# ---------------------------------------------------------------------------- RoPE ----
@pytest.mark.parametrize("name", list(cases.ROPE))
def test_rope_golden_bit_exact(name, golden_ops):
    x = cases.rope_inputs(name)
    gold = golden_ops[name]
    q, k = b200.b200_rope(dev(x["query"]), dev(x["key"]), dev(gold["cosine"]), dev(gold["sine"]))
    assert q.is_contiguous() and k.is_contiguous()
    exact(q, gold["query_out"])
    exact(k, gold["key_out"])


def test_rope_unaligned_head_dim_uses_scalar_path():
    g = torch.Generator().manual_seed(4)
    q = torch.randn(2, 3, 5, 12, generator=g).bfloat16()
    k = torch.randn(2, 1, 5, 12, generator=g).bfloat16()
    cos = torch.randn(2, 5, 12, generator=g).bfloat16()
    sin = torch.randn(2, 5, 12, generator=g).bfloat16()
    q_ref, k_ref = serve_ops.rope(q, k, cos, sin)
    q_out, k_out = b200.b200_rope(q.cuda(), k.cuda(), cos.cuda(), sin.cuda())
    exact(q_out, q_ref)
    exact(k_out, k_ref)


@pytest.mark.parametrize("name", ["rope_bf16_decode", "rope_f32"])
def test_rope_kv_store_fusion_matches_separate_ops(name, golden_ops):
    x = cases.rope_inputs(name)
    gold = golden_ops[name]
    b, hkv, d = x["key"].shape[0], x["kv_heads"], x["head_dim"]
    dtype = x["query"].dtype
    capacity = 16
    g = torch.Generator().manual_seed(8)
    value = torch.randn(b, hkv, 1, d, generator=g).to(dtype)
    positions = torch.arange(b, dtype=torch.int64) % capacity
    kbuf = torch.zeros(b, capacity, hkv, d, dtype=dtype)
    vbuf = torch.zeros_like(kbuf)
    serve_ops.kv_store(kbuf, vbuf, gold["key_out"], value, positions)
    k_dev, v_dev = torch.zeros_like(kbuf).cuda(), torch.zeros_like(vbuf).cuda()
    q_out = b200.b200_rope_kv_store(dev(x["query"]), dev(x["key"]), value.cuda(),
                                    dev(gold["cosine"]), dev(gold["sine"]), k_dev, v_dev,
                                    positions.cuda())
    exact(q_out, gold["query_out"])
    exact(k_dev, kbuf)
    exact(v_dev, vbuf)


@pytest.mark.parametrize("name", list(cases.ROPE_TABLE))
def test_rope_table(name, golden_ops):
    x = cases.rope_table_inputs(name)
    inv_freq = serve_ops.rope_inverse_frequency(x["head_dim"], x["theta"])
    cos, sin = b200.b200_rope_table(dev(x["position_ids"]), inv_freq.cuda(), x["dtype"])
    for actual, expected in ((cos, golden_ops[name]["cosine"]), (sin, golden_ops[name]["sine"])):
        actual = actual.cpu()
        if x["dtype"] == torch.float32:
            torch.testing.assert_close(actual, expected, rtol=0, atol=2e-7)
        else:
            # cos/sin come from different libms (device vs host): after bf16 rounding a value
            # may land on the neighbouring bf16 in rare ties; never further
            differing = (actual != expected).float().mean().item()
            assert differing <= 0.01, f"{differing:.4f} of the table differs"
            torch.testing.assert_close(actual.float(), expected.float(), rtol=0, atol=2 ** -8)


# ------------------------------------------------------------------------- RMSNorm ----
@pytest.mark.parametrize("name", list(cases.RMS_NORM))
def test_rms_norm_pytorch_compatible_bit_exact(name, golden_ops):
    x = cases.rms_norm_inputs(name)
    out = b200.b200_rms_norm(dev(x["input"]), dev(x["weight"]), epsilon=x["epsilon"],
                             round_before_weight=x["round_before_weight"],
                             numerical_mode="pytorch_compatible")
    exact(out, golden_ops[name]["output"])


@pytest.mark.parametrize("name", list(cases.RMS_NORM))
def test_rms_norm_fast(name, golden_ops):
    x = cases.rms_norm_inputs(name)
    out = b200.b200_rms_norm(dev(x["input"]), dev(x["weight"]), epsilon=x["epsilon"],
                             round_before_weight=x["round_before_weight"], numerical_mode="fast")
    close(out, golden_ops[name]["output"], tol_for(x["input"].dtype))


def test_rms_norm_3d_and_strided_rows():
    g = torch.Generator().manual_seed(12)
    x = torch.randn(4, 3, 896, generator=g).bfloat16()
    w = torch.randn(896, generator=g).bfloat16()
    ref = serve_ops.rms_norm(x, w, 1e-6, round_before_weight=True)
    exact(b200.b200_rms_norm(x.cuda(), w.cuda(), epsilon=1e-6, round_before_weight=True,
                             numerical_mode="pytorch_compatible"), ref)
    wide = torch.randn(6, 2048, generator=g).bfloat16()
    view = wide[:, :896]
    ref = serve_ops.rms_norm(view, w, 1e-6, round_before_weight=True)
    for mode in ("pytorch_compatible", "fast"):
        out = b200.b200_rms_norm(wide.cuda()[:, :896], w.cuda(), epsilon=1e-6,
                                 round_before_weight=True, numerical_mode=mode)
        (exact if mode == "pytorch_compatible" else lambda a, e: close(a, e, BF16_TOL))(out, ref)


# ---------------------------------------------------------------- decode attention ----
@pytest.fixture(params=["tma", "cp.async"])
def decode_loads(request, monkeypatch):
    """Both ways of filling the shared-memory ring: tensor-map box copies and 16-byte cp.async."""
    monkeypatch.setenv("B200_DECODE_ATTENTION_LOADS", request.param)
    return request.param


@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
@pytest.mark.parametrize("name", list(cases.DECODE_ATTENTION))
def test_decode_attention_golden(name, mode, golden_ops, decode_loads):
    x = cases.decode_attention_inputs(name)
    out = b200.b200_decode_attention(dev(x["query"]), dev(x["key_buffer"]), dev(x["value_buffer"]),
                                     dev(x["lengths"]), dev(x["mask"]), scale=x["scale"],
                                     numerical_mode=mode)
    assert out.shape == golden_ops[name]["output"].shape
    close(out, golden_ops[name]["output"], tol_for(x["query"].dtype))
    kernels.runtime().check_status()


@pytest.mark.parametrize("split_tokens", [0, 16, 64, 256, 4096])
def test_decode_attention_splits_ragged_and_masked(split_tokens, decode_loads):
    """Ragged lengths incl. 0 (NaN row, as the oracle), 1 and == capacity; a mask with -inf
    holes; every split size must agree with the oracle."""
    g = torch.Generator().manual_seed(21)
    b, c, hq, hkv, d = 6, 777, 14, 2, 64
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16().transpose(1, 2)
    kbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    vbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    lengths = torch.tensor([0, 1, 16, 17, 500, c])
    mask = torch.zeros(b, 1, 1, c)
    mask[:, :, :, 3::7] = float("-inf")
    mask[4, :, :, :64] = float("-inf")  # a fully masked first tile
    mask[1, :, :, 0] = 0.0
    ref = serve_ops.decode_attention(q, kbuf, vbuf, lengths, mask, groups=hq // hkv, scale=0.125)
    out = b200.b200_decode_attention(q.cuda(), kbuf.cuda(), vbuf.cuda(), lengths.cuda(),
                                     mask.cuda(), scale=0.125, split_tokens=split_tokens)
    assert torch.isnan(out[0]).all()
    close(out, ref, BF16_TOL)
    kernels.runtime().check_status()


def test_decode_attention_no_mask_and_bf16_mask(decode_loads):
    x = cases.decode_attention_inputs("decode_attention_bf16_long")
    ref = serve_ops.decode_attention(x["query"], x["key_buffer"], x["value_buffer"], x["lengths"],
                                     x["mask"], groups=x["groups"], scale=x["scale"])
    args = [dev(x[k]) for k in ("query", "key_buffer", "value_buffer", "lengths")]
    close(b200.b200_decode_attention(*args, None, scale=x["scale"]), ref, BF16_TOL)
    close(b200.b200_decode_attention(*args, dev(x["mask"].bfloat16()), scale=x["scale"]), ref,
          BF16_TOL)
    short = x["mask"][..., :1200].contiguous()
    close(b200.b200_decode_attention(*args, dev(short), scale=x["scale"], max_length_hint=1200),
          ref, BF16_TOL)


def test_decode_attention_ignores_rows_beyond_the_length(decode_loads):
    """Rows past lengths[b] may hold anything, NaN included: they must not reach the output."""
    g = torch.Generator().manual_seed(17)
    b, c, hq, hkv, d = 4, 400, 14, 2, 64
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16().transpose(1, 2)
    kbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    vbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    lengths = torch.tensor([399, 33, 250, 64])
    ref = serve_ops.decode_attention(q, kbuf, vbuf, lengths, torch.zeros(b, 1, 1, c), groups=7,
                                     scale=0.125)
    for row, n in enumerate(lengths.tolist()):
        kbuf[row, n:] = float("nan")
        vbuf[row, n:] = float("inf")
    for split in (0, 64, 128):
        out = b200.b200_decode_attention(q.cuda(), kbuf.cuda(), vbuf.cuda(), lengths.cuda(), None,
                                         scale=0.125, split_tokens=split)
        close(out, ref, BF16_TOL)
    kernels.runtime().check_status()


def test_decode_attention_length_over_mask_sets_status():
    x = cases.decode_attention_inputs("decode_attention_bf16")
    mask = x["mask"][..., :200].contiguous()  # lengths are [1, 130, 300]
    b200.b200_decode_attention(dev(x["query"]), dev(x["key_buffer"]), dev(x["value_buffer"]),
                               dev(x["lengths"]), dev(mask), scale=x["scale"])
    with pytest.raises(b200.KernelStatusError):
        kernels.runtime().check_status()


def test_decode_attention_qwen2_7b_shape(decode_loads):
    g = torch.Generator().manual_seed(31)
    b, c, hq, hkv, d = 3, 1500, 28, 4, 128
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16().transpose(1, 2)
    kbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    vbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    lengths = torch.tensor([1500, 1024, 333])
    mask = torch.zeros(b, 1, 1, c)
    ref = serve_ops.decode_attention(q, kbuf, vbuf, lengths, mask, groups=7, scale=d ** -0.5)
    for split in (0, 128):
        out = b200.b200_decode_attention(q.cuda(), kbuf.cuda(), vbuf.cuda(), lengths.cuda(),
                                         mask.cuda(), scale=d ** -0.5, split_tokens=split)
        close(out, ref, BF16_TOL)


@pytest.mark.parametrize("hq,hkv", [(24, 2), (40, 2), (16, 1), (9, 1)])
def test_decode_attention_wide_groups(hq, hkv, decode_loads):
    """More than 8 (and more than 16) query heads per KV head: both row halves of the
    tensor-core tile and several 16-row blocks per KV head."""
    g = torch.Generator().manual_seed(hq)
    b, c, d = 2, 210, 64
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16().transpose(1, 2)
    kbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    vbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    lengths = torch.tensor([210, 45])
    mask = torch.zeros(b, 1, 1, c)
    ref = serve_ops.decode_attention(q, kbuf, vbuf, lengths, mask, groups=hq // hkv, scale=0.125)
    for split in (0, 64):
        out = b200.b200_decode_attention(q.cuda(), kbuf.cuda(), vbuf.cuda(), lengths.cuda(),
                                         mask.cuda(), scale=0.125, split_tokens=split)
        close(out, ref, BF16_TOL)


def test_decode_attention_split_invariance_full_size(decode_loads):
    """Benchmark shape (batch 64, capacity 4608, lengths ~4096, 14/2 heads x 64): the result
    must not depend on how the KV range is split; one sequence is checked against the oracle."""
    b, c, hq, hkv, d = 64, 4608, 14, 2, 64
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(b, hq, 1, d, generator=g, device="cuda").bfloat16()
    kbuf = torch.randn(b, c, hkv, d, generator=g, device="cuda").bfloat16()
    vbuf = torch.randn(b, c, hkv, d, generator=g, device="cuda").bfloat16()
    lengths = torch.randint(64, 4097, (b,), generator=g, device="cuda")
    lengths[0] = 4096
    outs = [b200.b200_decode_attention(q, kbuf, vbuf, lengths, None, scale=0.125,
                                       split_tokens=s, max_length_hint=4096)
            for s in (0, 256, 1024, 8192)]
    for other in outs[1:]:
        close(other, outs[0].float().cpu(), 4e-3)
    ref = serve_ops.decode_attention(q[:1].cpu(), kbuf[:1].cpu(), vbuf[:1].cpu(),
                                     lengths[:1].cpu(), torch.zeros(1, 1, 1, c), groups=7,
                                     scale=0.125)
    close(outs[0][:1], ref, BF16_TOL)
    kernels.runtime().check_status()


@pytest.mark.parametrize("schedule", ["flat", "grid"])
@pytest.mark.parametrize("shape", ["one_long", "many_short", "large_batch"])
def test_decode_attention_schedules_on_skewed_lengths(shape, schedule, monkeypatch, decode_loads):
    """With split_tokens == 0 the kernel runs on a fixed (split, head, batch) grid, or, with
    B200_DECODE_ATTENTION_SCHEDULE=flat, cuts the work by chunks counted from lengths[] on the
    device. Skewed batches make one pair span many CTAs and one CTA span many pairs; a second
    call on the same workspace checks that the arrival counters were left at zero."""
    monkeypatch.setenv("B200_DECODE_ATTENTION_SCHEDULE", schedule)
    g = torch.Generator().manual_seed(len(shape))
    hq, hkv, d = 14, 2, 64
    if shape == "one_long":
        b, c = 5, 6000
        lengths = torch.tensor([6000, 0, 3, 129, 0])
    elif shape == "many_short":
        b, c = 40, 300
        lengths = torch.randint(0, 301, (b,), generator=g)
        lengths[7] = 300
    else:
        b, c = 300, 140  # more sequences than threads in a CTA
        lengths = torch.randint(1, 141, (b,), generator=g)
    q = torch.randn(b, 1, hq, d, generator=g).bfloat16().transpose(1, 2)
    kbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    vbuf = torch.randn(b, c, hkv, d, generator=g).bfloat16()
    ref = serve_ops.decode_attention(q, kbuf, vbuf, lengths, torch.zeros(b, 1, 1, c),
                                     groups=hq // hkv, scale=0.125)
    args = (q.cuda(), kbuf.cuda(), vbuf.cuda(), lengths.cuda(), None)
    for _ in range(2):
        out = b200.b200_decode_attention(*args, scale=0.125, split_tokens=0)
        empty = lengths == 0
        assert torch.isnan(out[empty.cuda()]).all()
        close(out[~empty.cuda()], ref[~empty], BF16_TOL)
    kernels.runtime().check_status()


# --------------------------------------------------------------- prefill attention ----
@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
@pytest.mark.parametrize("name", list(cases.PREFILL_ATTENTION))
def test_prefill_attention_golden(name, mode, golden_ops):
    x = cases.prefill_attention_inputs(name)
    gold = golden_ops[name]["output"]
    tol = tol_for(x["query"].dtype)
    out = b200.b200_prefill_attention(dev(x["query"]), dev(x["key"]), dev(x["value"]),
                                      dev(x["mask"]), scale=x["scale"], numerical_mode=mode)
    assert out.shape == gold.shape
    assert out.transpose(1, 2).is_contiguous()  # token-major memory
    close(out, gold, tol)
    if not x["zero_mask"]:
        causal = b200.b200_prefill_attention(dev(x["query"]), dev(x["key"]), dev(x["value"]),
                                             None, scale=x["scale"], causal=True,
                                             numerical_mode=mode)
        close(causal, gold, tol)


def test_prefill_attention_arbitrary_mask_and_broadcast_batch():
    g = torch.Generator().manual_seed(44)
    b, t, hq, hkv, d = 2, 150, 14, 2, 64
    q = torch.randn(b, t, hq, d, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(b, t, hkv, d, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(b, t, hkv, d, generator=g).bfloat16().transpose(1, 2)
    mask = torch.randn(1, 1, t, t, generator=g)  # soft additive mask, broadcast over batch
    mask[:, :, :, 5::9] = float("-inf")
    ref = serve_ops.prefill_attention(q, k, v, mask, groups=7, scale=0.125)
    out = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), mask.cuda(), scale=0.125)
    close(out, ref, BF16_TOL)


@pytest.mark.parametrize("tokens", [16, 128, 512])
def test_prefill_attention_config3_shapes(tokens):
    g = torch.Generator().manual_seed(tokens)
    b, hq, hkv, d = 4, 14, 2, 64
    q = torch.randn(b, tokens, hq, d, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(b, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(b, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    ref = serve_ops.prefill_attention(q, k, v, None, groups=7, scale=0.125, causal=True)
    out = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), None, scale=0.125, causal=True)
    close(out, ref, BF16_TOL)
    masked = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(),
                                         serve_ops.causal_mask(b, tokens).cuda(), scale=0.125)
    close(masked, ref, BF16_TOL)


@pytest.mark.parametrize("layout", ["token_major", "head_major"])
@pytest.mark.parametrize("batch,tokens,hq,hkv,d", [(2, 1, 14, 2, 64), (2, 127, 14, 2, 64),
                                                    (3, 129, 14, 2, 64), (1, 700, 4, 4, 64),
                                                    (2, 333, 28, 4, 128), (1, 1024, 8, 1, 128),
                                                    (2, 255, 14, 2, 64), (1, 257, 14, 2, 64),
                                                    (1, 385, 4, 2, 128), (2, 512, 2, 1, 64)])
def test_prefill_attention_tensor_memory_path(batch, tokens, hq, hkv, d, layout, monkeypatch):
    """Causal-proved bf16 calls in the fast mode run on tcgen05 (S and O tiles in tensor memory,
    TMA boxes of 128 tokens): token counts around and off the 128-row tile, one token, several
    key tiles, both head dims, inputs as views of [B, T, H, D] (what the graphs produce) and as
    plain [B, H, T, D]. The oracle and the warp-level kernel must both agree."""
    g = torch.Generator().manual_seed(tokens + d)
    if layout == "token_major":
        q = torch.randn(batch, tokens, hq, d, generator=g).bfloat16().transpose(1, 2)
        k = torch.randn(batch, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
        v = torch.randn(batch, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    else:
        q = torch.randn(batch, hq, tokens, d, generator=g).bfloat16()
        k = torch.randn(batch, hkv, tokens, d, generator=g).bfloat16()
        v = torch.randn(batch, hkv, tokens, d, generator=g).bfloat16()
    scale = d ** -0.5
    ref = serve_ops.prefill_attention(q, k, v, None, groups=hq // hkv, scale=scale, causal=True)
    out = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), None, scale=scale, causal=True)
    assert out.transpose(1, 2).is_contiguous()
    close(out, ref, BF16_TOL)
    monkeypatch.setenv("B200_PREFILL_ATTENTION_PATH", "mma.sync")
    warp_level = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), None, scale=scale,
                                             causal=True)
    close(out, warp_level.float().cpu(), 1e-2)
    kernels.runtime().check_status()


@pytest.mark.parametrize("d", [64, 128])
def test_prefill_attention_moves_its_reference_maximum(d):
    """The tcgen05 kernel keeps O in tensor memory against a lazy reference maximum and rescales
    it only when a key tile raises a row's maximum by more than 8 (log2 domain). Scores with a
    standard deviation of 8 and a drift upwards along the keys make that happen tile after tile."""
    g = torch.Generator().manual_seed(d)
    batch, tokens, hq, hkv = 2, 1100, 4, 2
    q = (torch.randn(batch, tokens, hq, d, generator=g) * 8.0).bfloat16().transpose(1, 2)
    k = torch.randn(batch, tokens, hkv, d, generator=g)
    k = (k + torch.linspace(0.0, 1.5, tokens)[None, :, None, None] * q.transpose(1, 2)[:, -1:, :hkv].float().sign()).bfloat16().transpose(1, 2)
    v = torch.randn(batch, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    scale = d ** -0.5
    # With scores this large the oracle's own bf16 rounding of the scores (an absolute error of
    # up to 0.25 at |s| = 40) moves probabilities by tens of per cent, so the yardstick here is
    # the exact attention of the same bf16 inputs in float64, which the kernel (fp32 scores,
    # bf16 probabilities) must match within the bf16 tolerance.
    q64, k64, v64 = (t.double().repeat_interleave(hq // t.shape[1], dim=1) for t in (q, k, v))
    scores = q64 @ k64.transpose(-1, -2) * scale
    scores = scores.masked_fill(torch.triu(torch.ones(tokens, tokens, dtype=torch.bool), diagonal=1), float("-inf"))
    exact = (torch.softmax(scores, dim=-1) @ v64).float()
    out = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), None, scale=scale, causal=True)
    assert torch.isfinite(out.float()).all()
    close(out, exact, BF16_TOL)
    kernels.runtime().check_status()


# -------------------------------------------------------------------------- linear ----
@pytest.mark.parametrize("name", list(cases.LINEAR))
def test_linear_golden(name, golden_ops):
    x = cases.linear_inputs(name)
    out = b200.b200_linear(dev(x["input"]), dev(x["weight"]), dev(x["bias"]))
    close(out, golden_ops[name]["output"], tol_for(x["input"].dtype))


@pytest.mark.parametrize("m,k,n", [(1, 896, 896), (16, 896, 1152), (64, 896, 9728), (64, 4864, 896),
                                   (33, 896, 130), (256, 896, 896), (500, 512, 330)])
def test_linear_shapes_and_epilogues(m, k, n):
    g = torch.Generator().manual_seed(m * 31 + n)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    bias = torch.randn(n, generator=g).bfloat16()
    res = torch.randn(m, n, generator=g).bfloat16()
    ref = serve_ops.linear(x, w, bias)
    close(b200.b200_linear(x.cuda(), w.cuda(), bias.cuda()), ref, BF16_TOL)
    close(b200.b200_linear(x.cuda(), w.cuda()), serve_ops.linear(x, w), BF16_TOL)
    ref_res = serve_ops.residual_add(res, serve_ops.linear(x, w))
    close(b200.b200_linear(x.cuda(), w.cuda(), residual=res.cuda(), epilogue="residual"), ref_res,
          BF16_TOL)
    if n % 2 == 0:
        gate_w, up_w = w[: n // 2], w[n // 2:]
        ref_mlp = serve_ops.swiglu(serve_ops.linear(x, gate_w), serve_ops.linear(x, up_w))
        packed = kernels.interleave_gate_up(gate_w.cuda(), up_w.cuda())
        close(b200.b200_linear(x.cuda(), packed, epilogue="swiglu"), ref_mlp, BF16_TOL)


@pytest.mark.parametrize("m,k,n", [(128, 64, 128), (256, 896, 896), (1000, 4864, 896),
                                   (2048, 896, 9728), (300, 896, 1152), (129, 200, 72),
                                   (1100, 200, 1000), (1536, 896, 1152), (1024, 896, 896)])
def test_linear_tcgen05_path_matches_the_oracle_and_the_warp_level_path(m, k, n, monkeypatch):
    """More than 64 rows run on tcgen05 / TMEM / TMA (from 1024 rows on the persistent kernel with
    two accumulators: 608 tiles on 148 CTAs, 256-, 224- and 192-column tiles, ragged M, N and K);
    the same call with B200_LINEAR_PATH=mma.sync runs the warp-level kernel. Both against the
    CPU oracle, all epilogues, full and ragged tiles in M, N and K."""
    g = torch.Generator().manual_seed(m + n)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    bias = torch.randn(n, generator=g).bfloat16()
    res = torch.randn(m, n, generator=g).bfloat16()
    ref = serve_ops.linear(x, w, bias)
    ref_res = serve_ops.residual_add(res, serve_ops.linear(x, w))
    ref_mlp = serve_ops.swiglu(serve_ops.linear(x, w[: n // 2]), serve_ops.linear(x, w[n // 2:]))
    xd, wd, bd, rd = x.cuda(), w.cuda(), bias.cuda(), res.cuda()
    packed = kernels.interleave_gate_up(wd[: n // 2], wd[n // 2:])
    outputs = {}
    for path in ("tcgen05", "mma.sync"):
        if path == "mma.sync":
            monkeypatch.setenv("B200_LINEAR_PATH", "mma.sync")
        outputs[path] = (b200.b200_linear(xd, wd, bd), b200.b200_linear(xd, wd, residual=rd, epilogue="residual"),
                         b200.b200_linear(xd, packed, epilogue="swiglu"))
        close(outputs[path][0], ref, BF16_TOL)
        close(outputs[path][1], ref_res, BF16_TOL)
        close(outputs[path][2], ref_mlp, BF16_TOL)
    kernels.runtime().check_status()
    # the two kernels round at the same points: they agree to an ulp of the output scale
    close(outputs["tcgen05"][0], outputs["mma.sync"][0].float().cpu(), 1e-2)
    if m >= 1024:  # one tile per CTA and the persistent kernel accumulate in the same order
        monkeypatch.delenv("B200_LINEAR_PATH")
        monkeypatch.setenv("B200_LINEAR_PERSISTENT", "0")
        single = (b200.b200_linear(xd, wd, bd), b200.b200_linear(xd, wd, residual=rd, epilogue="residual"),
                  b200.b200_linear(xd, packed, epilogue="swiglu"))
        for ours, theirs in zip(outputs["tcgen05"], single):
            assert torch.equal(ours, theirs)


@pytest.mark.parametrize("m,k,n", [(64, 896, 1152), (64, 896, 896), (64, 4864, 896), (3, 256, 512),
                                   (128, 896, 896), (17, 512, 260)])
def test_split_k_partial_producer_and_its_consumers(m, k, n):
    """b200_linear_partial + reduce_residual_rms_norm == linear -> add -> rms_norm of the oracle;
    the partial sums themselves add up to the fp32 product."""
    g = torch.Generator().manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * 0.05).bfloat16()
    res = torch.randn(m, n, generator=g).bfloat16()
    nw = (1 + 0.1 * torch.randn(n, generator=g)).bfloat16()
    partials = b200.kernels.b200_linear_partial(x.cuda(), w.cuda())
    assert partials.shape[0] == kernels.linear_partial_splits(m, k, n)
    exact_product = x.float() @ w.float().t()
    torch.testing.assert_close(partials.sum(0).cpu(), exact_product, rtol=1e-3, atol=1e-3)
    y = serve_ops.residual_add(res, serve_ops.linear(x, w))
    h = serve_ops.rms_norm(y, nw, 1e-6, round_before_weight=True)
    x_out, h_out = b200.kernels.b200_reduce_residual_rms_norm(partials, res.cuda(), nw.cuda(),
                                                              epsilon=1e-6)
    close(x_out, y, BF16_TOL)
    close(h_out, h, BF16_TOL)
    plain, none = b200.kernels.b200_reduce_residual_rms_norm(partials, None, None, epsilon=1e-6)
    assert none is None
    close(plain, serve_ops.linear(x, w), BF16_TOL)
    kernels.runtime().check_status()


def test_split_k_partials_feed_rope_and_kv_store():
    g = torch.Generator().manual_seed(99)
    b, hq, hkv, d, hidden, capacity = 5, 14, 2, 64, 896, 32
    width = (hq + 2 * hkv) * d
    x = torch.randn(b, hidden, generator=g).bfloat16()
    w = (torch.randn(width, hidden, generator=g) * 0.05).bfloat16()
    bias = torch.randn(width, generator=g).bfloat16()
    positions = torch.tensor([0, 31, 7, 7, 20])
    inv_freq = serve_ops.rope_inverse_frequency(d, 1e6)
    cos, sin = serve_ops.rope_table(positions.view(b, 1), inv_freq, torch.bfloat16)
    qkv = serve_ops.linear(x, w, bias)
    q = qkv[:, : hq * d].view(b, 1, hq, d).transpose(1, 2)
    k = qkv[:, hq * d: (hq + hkv) * d].view(b, 1, hkv, d).transpose(1, 2)
    v = qkv[:, (hq + hkv) * d:].view(b, 1, hkv, d).transpose(1, 2)
    q_ref, k_ref = serve_ops.rope(q, k, cos, sin)
    kbuf = torch.zeros(b, capacity, hkv, d, dtype=torch.bfloat16)
    vbuf = torch.zeros_like(kbuf)
    serve_ops.kv_store(kbuf, vbuf, k_ref, v, positions)
    k_dev, v_dev = torch.zeros_like(kbuf).cuda(), torch.zeros_like(vbuf).cuda()
    partials = b200.kernels.b200_linear_partial(x.cuda(), w.cuda())
    q_out = b200.kernels.b200_reduce_rope_kv_store(partials, bias.cuda(), cos.cuda(), sin.cuda(),
                                                   k_dev, v_dev, positions.cuda(), q_heads=hq)
    close(q_out, q_ref, BF16_TOL)
    close(k_dev, kbuf, BF16_TOL)
    close(v_dev, vbuf, BF16_TOL)
    assert k_dev[0, 1:].eq(0).all()  # only the addressed rows were written
    kernels.runtime().check_status()


@pytest.mark.parametrize("split_tokens", [0, 64, 4096])
@pytest.mark.parametrize("hq,hkv,d", [(14, 2, 64), (28, 4, 128), (24, 2, 64)])
def test_fused_qkv_rope_store_attention_equals_separate_launches(hq, hkv, d, split_tokens,
                                                                 decode_loads):
    """One launch (q|k|v partial reduction + bias + RoPE + KV store inside decode attention, the
    new token attending from registers) against the two launches it replaces and against the
    oracle. Lengths put the new token first in the buffer, on split boundaries (63/64/65) and
    at the end of the capacity; the KV rows it writes must be bit-equal, all others untouched."""
    g = torch.Generator().manual_seed(hq + d + split_tokens)
    hidden, capacity = 256, 300
    lengths = torch.tensor([1, 2, 64, 65, 129, 300, 257])
    b = lengths.numel()
    width = (hq + 2 * hkv) * d
    x = torch.randn(b, hidden, generator=g).bfloat16()
    w = (torch.randn(width, hidden, generator=g) * 0.08).bfloat16()
    bias = torch.randn(width, generator=g).bfloat16()
    positions = lengths - 1
    inv_freq = serve_ops.rope_inverse_frequency(d, 1e6)
    cos, sin = serve_ops.rope_table(positions.view(b, 1), inv_freq, torch.bfloat16)
    kbuf = torch.randn(b, capacity, hkv, d, generator=g).bfloat16()
    vbuf = torch.randn(b, capacity, hkv, d, generator=g).bfloat16()
    # oracle: projection -> rope -> store -> attention
    qkv = serve_ops.linear(x, w, bias)
    q = qkv[:, : hq * d].view(b, 1, hq, d).transpose(1, 2)
    k = qkv[:, hq * d: (hq + hkv) * d].view(b, 1, hkv, d).transpose(1, 2)
    v = qkv[:, (hq + hkv) * d:].view(b, 1, hkv, d).transpose(1, 2)
    q_ref, k_ref = serve_ops.rope(q, k, cos, sin)
    k_gold, v_gold = kbuf.clone(), vbuf.clone()
    serve_ops.kv_store(k_gold, v_gold, k_ref, v, positions)
    ref = serve_ops.decode_attention(q_ref, k_gold, v_gold, lengths, torch.zeros(b, 1, 1, capacity),
                                     groups=hq // hkv, scale=d ** -0.5)
    for row, n in enumerate(lengths.tolist()):  # on the device, rows at and past the new token hold poison
        kbuf[row, n - 1:] = float("nan")
        vbuf[row, n - 1:] = float("inf")
    partials = kernels.b200_linear_partial(x.cuda(), w.cuda())
    # the two launches
    k_two, v_two = kbuf.cuda(), vbuf.cuda()
    q_two = kernels.b200_reduce_rope_kv_store(partials, bias.cuda(), cos.cuda(), sin.cuda(), k_two,
                                              v_two, positions.cuda(), q_heads=hq)
    out_two = b200.b200_decode_attention(q_two, k_two, v_two, lengths.cuda(), None, scale=d ** -0.5,
                                         split_tokens=split_tokens)
    # the one launch
    k_one, v_one = kbuf.cuda(), vbuf.cuda()
    out_one = kernels.b200_qkv_decode_attention(partials, bias.cuda(), cos.cuda(), sin.cuda(), k_one,
                                                v_one, lengths.cuda(), q_heads=hq, scale=d ** -0.5,
                                                split_tokens=split_tokens)
    assert torch.equal(k_one.view(torch.int16), k_two.view(torch.int16))
    assert torch.equal(v_one.view(torch.int16), v_two.view(torch.int16))
    close(out_one, ref, BF16_TOL)
    close(out_one, out_two.float().cpu(), 1e-2)
    kernels.runtime().check_status()


def test_linear_f32_epilogues():
    g = torch.Generator().manual_seed(77)
    x = torch.randn(7, 256, generator=g)
    w = torch.randn(512, 256, generator=g) * 0.05
    res = torch.randn(7, 512, generator=g)
    close(b200.b200_linear(x.cuda(), w.cuda(), residual=res.cuda(), epilogue="residual"),
          res + serve_ops.linear(x, w), F32_TOL)
    packed = kernels.interleave_gate_up(w[:256].cuda(), w[256:].cuda())
    close(b200.b200_linear(x.cuda(), packed, epilogue="swiglu"),
          serve_ops.swiglu(serve_ops.linear(x, w[:256]), serve_ops.linear(x, w[256:])), F32_TOL)


def test_linear_repeated_split_k_calls_leave_counters_clean():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 4864, generator=g).bfloat16().cuda()
    w = (torch.randn(896, 4864, generator=g) * 0.02).bfloat16().cuda()
    first = b200.b200_linear(x, w)
    for _ in range(3):
        assert torch.equal(b200.b200_linear(x, w), first)  # deterministic split-K reduction


# ------------------------------------------------------- ops left to eager upstream ----
def test_embedding_swiglu_add_argmax_advance():
    g = torch.Generator().manual_seed(9)
    table = torch.randn(1000, 896, generator=g).bfloat16()
    ids = torch.randint(0, 1000, (3, 5), generator=g)
    exact(b200.b200_embedding(table.cuda(), ids.cuda()), serve_ops.embedding(table, ids))
    gate = torch.randn(5, 4864, generator=g).bfloat16()
    up = torch.randn(5, 4864, generator=g).bfloat16()
    close(b200.b200_swiglu(gate.cuda(), up.cuda()), serve_ops.swiglu(gate, up), 1e-2)
    a = torch.randn(3, 7, 896, generator=g).bfloat16()
    b = torch.randn(3, 7, 896, generator=g).bfloat16()
    exact(b200.b200_add(a.cuda(), b.cuda()), a + b)
    af, bf = torch.randn(33, generator=g), torch.randn(33, generator=g)
    exact(b200.b200_add(af.cuda(), bf.cuda()), af + bf)
    logits = torch.randn(6, 151936, generator=g).bfloat16()
    logits[2, 77] = 100.0
    logits[2, 5000] = 100.0  # tie: lowest index wins
    out = b200.b200_argmax(logits.cuda()).cpu()
    assert out[2] == 77
    assert torch.equal(logits.float().max(-1).values, logits.float().gather(1, out.view(-1, 1))[:, 0])
    lengths = torch.tensor([[1, 5], [7, 63]], device="cuda")
    b200.b200_advance_lengths(lengths, 1, 64)
    assert lengths.tolist() == [[2, 6], [8, 64]]
    kernels.runtime().check_status()
    b200.b200_advance_lengths(lengths, 1, 64)
    with pytest.raises(b200.KernelStatusError):
        kernels.runtime().check_status()
    strided = torch.randn(4, 6, 10, generator=g).bfloat16().cuda().transpose(0, 2)
    exact(b200.b200_contiguous(strided), strided.cpu().contiguous())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,vocab", [(64, 151936), (3, 40001), (5, 1000), (400, 33000)])
def test_argmax_matches_torch_with_ties_across_parts(rows, vocab, dtype):
    """Maxima anywhere in the row, ties far apart (lowest index wins), a maximum in the ragged
    tail; odd vocabulary sizes take the scalar path."""
    g = torch.Generator().manual_seed(rows + vocab)
    logits = torch.randn(rows, vocab, generator=g).to(dtype)
    span = -(-vocab // 8)
    for row in range(min(rows, 9)):
        position = min(vocab - 1, row * span + 17) if row < 8 else vocab - 1
        logits[row, position] = 50.0
    logits[0, vocab - 3] = 50.0  # tie with an earlier part: the lower index must win
    if rows > 1:
        logits[1, 3] = 50.0      # tie with a later part
    out = b200.b200_argmax(logits.cuda()).cpu()
    assert torch.equal(out, logits.float().argmax(-1))


def test_embedding_bad_id_sets_status():
    table = torch.ones(10, 64, dtype=torch.bfloat16, device="cuda")
    out = b200.b200_embedding(table, torch.tensor([1, 10, -1], device="cuda"))
    assert out[0].eq(1).all() and out[1:].eq(0).all()
    with pytest.raises(b200.KernelStatusError):
        kernels.runtime().check_status()


def test_wrappers_reject_cpu_tensors_and_bad_shapes():
    x = torch.zeros(2, 4, 1, 64)
    with pytest.raises(ValueError):
        b200.b200_rms_norm(x, torch.zeros(64), epsilon=1e-6)
    q = torch.zeros(2, 4, 1, 64, device="cuda", dtype=torch.bfloat16)
    kv = torch.zeros(2, 8, 3, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):  # 4 query heads over 3 KV heads
        b200.b200_decode_attention(q, kv, kv, torch.zeros(2, dtype=torch.int64, device="cuda"),
                                   None, scale=1.0)


@pytest.mark.parametrize("split_tokens", [0, 128])
def test_decode_attention_service_order_changes_nothing(split_tokens):
    """sequence_order only decides which sequence a group of CTAs serves: any permutation gives
    the bit-identical output (here longest first and a shuffle, with and without KV splits, on
    more (sequence, KV head) pairs than the GPU holds at once); an entry outside the batch
    skips its group and touches nothing else."""
    g = torch.Generator().manual_seed(31 + split_tokens)
    batch, capacity, hq, hkv, d = 200, 640, 14, 2, 64
    lengths = torch.randint(1, capacity + 1, (batch,), generator=g)
    q = torch.randn(batch, hq, 1, d, generator=g).bfloat16().cuda()
    k = torch.randn(batch, capacity, hkv, d, generator=g).bfloat16().cuda()
    v = torch.randn(batch, capacity, hkv, d, generator=g).bfloat16().cuda()
    device_lengths = lengths.cuda()
    plain = kernels.b200_decode_attention(q, k, v, device_lengths, None, scale=d ** -0.5,
                                          split_tokens=split_tokens)
    longest_first = kernels.sequence_order_of(device_lengths)
    assert longest_first.dtype == torch.int32 and sorted(longest_first.tolist()) == list(range(batch))
    assert lengths[longest_first.cpu().long()].diff().max().item() <= 0
    shuffled = torch.randperm(batch, generator=g).to(torch.int32).cuda()
    for order in (longest_first, shuffled):
        out = kernels.b200_decode_attention(q, k, v, device_lengths, None, scale=d ** -0.5,
                                            split_tokens=split_tokens, sequence_order=order)
        assert torch.equal(out, plain)
    ref = serve_ops.decode_attention(q.cpu()[:8], k.cpu()[:8], v.cpu()[:8], lengths[:8],
                                     torch.zeros(8, 1, 1, capacity), groups=hq // hkv, scale=d ** -0.5)
    close(plain[:8], ref, BF16_TOL)
    holed = longest_first.clone()
    holed[5] = batch + 3  # not a sequence: that group does nothing
    skipped = int(longest_first[5])
    marked = torch.full_like(plain, 7.0)
    kernels.b200_decode_attention(q, k, v, device_lengths, None, scale=d ** -0.5, split_tokens=split_tokens,
                                  sequence_order=holed, output=marked)
    keep = torch.ones(batch, dtype=torch.bool)
    keep[skipped] = False
    assert torch.equal(marked[keep.cuda()], plain[keep.cuda()])
    assert torch.all(marked[skipped] == 7.0)
    with pytest.raises(ValueError):
        kernels.b200_decode_attention(q, k, v, device_lengths, None, scale=d ** -0.5,
                                      sequence_order=longest_first.long())
    kernels.runtime().check_status()


# ------------------------------------------ five-launch decode layer: its three kernels ----
@pytest.mark.parametrize("m,k,n", [(64, 896, 896), (64, 4864, 896), (3, 256, 256), (1, 512, 256),
                                   (33, 3584, 3584), (128, 896, 896), (100, 4864, 896),
                                   (64, 18944, 3584), (7, 960, 1092), (256, 896, 896),
                                   (200, 4864, 896), (256, 3584, 3584)])
def test_linear_splitk_residual_matches_linear_then_add(m, k, n):
    """serve.linear + aten.add in one launch: the K slices of a tile are the CTAs of a
    thread-block cluster that add their accumulators through distributed shared memory.
    Against the oracle's r(r(x W^T) + residual); repeated calls are bit-identical (the slices
    are added in a fixed order)."""
    g = torch.Generator().manual_seed(m + k + n)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) * k ** -0.5).bfloat16()
    residual = torch.randn(m, n, generator=g).bfloat16()
    ref = serve_ops.residual_add(residual, serve_ops.linear(x, w))
    out = kernels.b200_linear_splitk_residual(x.cuda(), w.cuda(), residual.cuda())
    close(out, ref, BF16_TOL)
    again = kernels.b200_linear_splitk_residual(x.cuda(), w.cuda(), residual.cuda())
    assert torch.equal(out, again)
    # a strided input (rows of a wider matrix), as the attention output is handed over
    wide = torch.randn(m, k + 64, generator=g).bfloat16().cuda()
    view = wide[:, :k]
    ref = serve_ops.residual_add(residual, serve_ops.linear(view.cpu(), w))
    close(kernels.b200_linear_splitk_residual(view, w.cuda(), residual.cuda()), ref, BF16_TOL)
    kernels.runtime().check_status()


def test_scale_columns_is_the_rounded_product():
    g = torch.Generator().manual_seed(4)
    w = torch.randn(333, 896, generator=g).bfloat16()
    s = torch.randn(896, generator=g).bfloat16()
    exact(kernels.b200_scale_columns(w.cuda(), s.cuda()), (w.float() * s.float()).bfloat16())
    wf, sf = torch.randn(7, 40, generator=g), torch.randn(40, generator=g)
    exact(kernels.b200_scale_columns(wf.cuda(), sf.cuda()), wf * sf)


@pytest.mark.parametrize("epilogue", ["none", "swiglu"])
@pytest.mark.parametrize("m,k,n", [(64, 896, 9728), (4, 3584, 37888), (3, 256, 1024), (17, 896, 1152),
                                   (64, 896, 2304), (100, 896, 9728), (128, 896, 2304), (65, 3584, 4608)])
def test_linear_rms_input_matches_rms_norm_then_linear(m, k, n, epilogue):
    """serve.rms_norm folded into the projection behind it: un-normalised rows in, the norm
    weight pre-multiplied into the weight's columns, the row factor applied to the accumulator.
    Against the oracle's rms_norm (Qwen2 rounding order) -> linear (-> SwiGLU)."""
    g = torch.Generator().manual_seed(m + k + n)
    x = (torch.randn(m, k, generator=g) * 3.0).bfloat16()
    norm_w = (1.0 + 0.2 * torch.randn(k, generator=g)).bfloat16()
    w = (torch.randn(n, k, generator=g) * k ** -0.5).bfloat16()
    bias = torch.randn(n, generator=g).bfloat16() if epilogue == "none" else None
    h = serve_ops.rms_norm(x, norm_w, 1e-6, round_before_weight=True)
    y = serve_ops.linear(h, w, bias)
    folded = kernels.b200_scale_columns(w.cuda(), norm_w.cuda())
    if epilogue == "swiglu":
        ref = serve_ops.swiglu(y[:, 0::2], y[:, 1::2])  # rows of w alternate gate_j, up_j
    else:
        ref = y
    out = kernels.b200_linear_rms_input(x.cuda(), folded, None if bias is None else bias.cuda(),
                                        epsilon=1e-6, epilogue=epilogue)
    close(out, ref, BF16_TOL)
    kernels.runtime().check_status()


@pytest.mark.parametrize("m,k,n", [(64, 896, 896), (64, 4864, 896), (3, 256, 256), (33, 3584, 3584),
                                   (7, 960, 1092), (128, 896, 896), (256, 3584, 3584)])
def test_linear_splitk_residual_leaves_row_sums_of_squares(m, k, n):
    """With row_squares the cluster split-K projection also leaves sum(output_r^2) in slices
    (one per N tile and K slice): their sum over the slices is the sum of squares of the stored
    bf16 rows, the output itself is unchanged, and a shape that runs without a cluster says so
    by returning None."""
    g = torch.Generator().manual_seed(m * 3 + k + n)
    x = torch.randn(m, k, generator=g).bfloat16().cuda()
    w = (torch.randn(n, k, generator=g) * k ** -0.5).bfloat16().cuda()
    residual = torch.randn(m, n, generator=g).bfloat16().cuda()
    plain = kernels.b200_linear_splitk_residual(x, w, residual)
    out, squares = kernels.b200_linear_splitk_residual(x, w, residual, row_squares=True)
    assert torch.equal(out, plain)
    if squares is None:
        assert kernels._lib.load().b200_linear_splitk_slices(m, k, n) == 0
    else:
        assert squares.shape == (kernels._lib.load().b200_linear_splitk_slices(m, k, n), m)
        expected = out.double().pow(2).sum(dim=1)
        assert torch.allclose(squares.double().sum(dim=0), expected, rtol=1e-5, atol=1e-5)
        again = kernels.b200_linear_splitk_residual(x, w, residual, row_squares=True)[1]
        assert torch.equal(squares, again)
    kernels.runtime().check_status()


@pytest.mark.parametrize("epilogue", ["none", "swiglu"])
@pytest.mark.parametrize("m,k_in,hidden,n", [(64, 896, 896, 9728), (64, 4864, 896, 1152), (5, 256, 256, 1024),
                                             (33, 512, 1536, 2304), (128, 896, 896, 9728), (90, 4864, 896, 2304)])
def test_linear_rms_input_takes_the_producers_row_squares(m, k_in, hidden, n, epilogue):
    """The folded-RMSNorm projection fed with the row sums of squares that the projection before
    it left (o projection -> gate|up in a decode layer): same result as squaring the rows itself
    up to the order of an fp32 sum, and the oracle's rms_norm -> linear (-> SwiGLU)."""
    g = torch.Generator().manual_seed(m + k_in + hidden + n)
    a = torch.randn(m, k_in, generator=g).bfloat16()
    wo = (torch.randn(hidden, k_in, generator=g) * k_in ** -0.5).bfloat16()
    residual = (torch.randn(m, hidden, generator=g) * 2.0).bfloat16()
    norm_w = (1.0 + 0.2 * torch.randn(hidden, generator=g)).bfloat16()
    w = (torch.randn(n, hidden, generator=g) * hidden ** -0.5).bfloat16()
    x, squares = kernels.b200_linear_splitk_residual(a.cuda(), wo.cuda(), residual.cuda(), row_squares=True)
    folded = kernels.b200_scale_columns(w.cuda(), norm_w.cuda())
    own = kernels.b200_linear_rms_input(x, folded, epsilon=1e-6, epilogue=epilogue)
    if squares is None:
        pytest.skip("this shape runs without a cluster: no slices to hand over")
    fed = kernels.b200_linear_rms_input(x, folded, epsilon=1e-6, epilogue=epilogue, row_squares=squares)
    assert (fed.float() - own.float()).abs().max().item() <= 2.0 ** -7 * own.float().abs().max().item() + 1e-6
    y = serve_ops.linear(serve_ops.rms_norm(x.cpu(), norm_w, 1e-6, round_before_weight=True), w)
    ref = serve_ops.swiglu(y[:, 0::2], y[:, 1::2]) if epilogue == "swiglu" else y
    close(fed, ref, BF16_TOL)
    with pytest.raises(ValueError):  # slices for another row count
        kernels.b200_linear_rms_input(x, folded, epsilon=1e-6, row_squares=squares[:, :-1].contiguous())
    kernels.runtime().check_status()


@pytest.mark.parametrize("batch", [5, 100])
def test_fused_attention_applies_the_folded_norm(batch):
    """b200_qkv_decode_attention with norm_input: the q|k|v partials come from un-normalised
    rows and a norm-folded weight; the result and the stored K / V rows must match the oracle's
    rms_norm -> projection -> rope -> store -> attention. 100 rows: the 128-row tile of the
    partial producer, two rows of squares per idle-warp thread."""
    g = torch.Generator().manual_seed(77)
    hq, hkv, d, hidden, capacity = 14, 2, 64, 896, 200
    lengths = torch.tensor([1, 64, 65, 200, 131])
    if batch > lengths.numel():
        lengths = torch.cat([lengths, torch.randint(1, capacity + 1, (batch - lengths.numel(),), generator=g)])
    b = lengths.numel()
    width = (hq + 2 * hkv) * d
    x = (torch.randn(b, hidden, generator=g) * 2.0).bfloat16()
    norm_w = (1.0 + 0.2 * torch.randn(hidden, generator=g)).bfloat16()
    w = (torch.randn(width, hidden, generator=g) * 0.05).bfloat16()
    bias = torch.randn(width, generator=g).bfloat16()
    positions = lengths - 1
    cos, sin = serve_ops.rope_table(positions.view(b, 1), serve_ops.rope_inverse_frequency(d, 1e6),
                                    torch.bfloat16)
    kbuf = torch.randn(b, capacity, hkv, d, generator=g).bfloat16()
    vbuf = torch.randn(b, capacity, hkv, d, generator=g).bfloat16()
    qkv = serve_ops.linear(serve_ops.rms_norm(x, norm_w, 1e-6, round_before_weight=True), w, bias)
    q = qkv[:, : hq * d].view(b, 1, hq, d).transpose(1, 2)
    k = qkv[:, hq * d: (hq + hkv) * d].view(b, 1, hkv, d).transpose(1, 2)
    v = qkv[:, (hq + hkv) * d:].view(b, 1, hkv, d).transpose(1, 2)
    q_ref, k_ref = serve_ops.rope(q, k, cos, sin)
    k_gold, v_gold = kbuf.clone(), vbuf.clone()
    serve_ops.kv_store(k_gold, v_gold, k_ref, v, positions)
    ref = serve_ops.decode_attention(q_ref, k_gold, v_gold, lengths, torch.zeros(b, 1, 1, capacity),
                                     groups=hq // hkv, scale=d ** -0.5)
    folded = kernels.b200_scale_columns(w.cuda(), norm_w.cuda())
    x_dev = x.cuda()
    partials, squares = kernels.b200_linear_partial(x_dev, folded, row_squares=True)
    torch.testing.assert_close(squares.sum(0).cpu(), x.float().pow(2).sum(-1), rtol=1e-5, atol=0)
    k_dev, v_dev = kbuf.cuda(), vbuf.cuda()
    out = kernels.b200_qkv_decode_attention(partials, bias.cuda(), cos.cuda(), sin.cuda(), k_dev, v_dev,
                                            lengths.cuda(), q_heads=hq, scale=d ** -0.5,
                                            norm_row_squares=squares, norm_hidden=hidden,
                                            norm_epsilon=1e-6)
    close(out, ref, BF16_TOL)
    close(k_dev, k_gold, BF16_TOL)
    close(v_dev, v_gold, BF16_TOL)
    kernels.runtime().check_status()


# ------------------------------ prefill attention: the additive-mask contract on tcgen05 ----
def _mask_case(kind, batch, tokens, generator):
    """Additive fp32 masks B x 1 x T x T of the kinds serving meets."""
    index = torch.arange(tokens)
    future = index.view(1, -1) > index.view(-1, 1)
    mask = torch.zeros(batch, 1, tokens, tokens)
    if kind == "causal":
        mask.masked_fill_(future, float("-inf"))
    elif kind == "sliding_window":  # causal, and at most 200 keys back: -inf tiles at both ends
        mask.masked_fill_(future | (index.view(1, -1) < index.view(-1, 1) - 200), float("-inf"))
    elif kind == "padded":  # causal + the last keys of every second sequence are padding
        mask.masked_fill_(future, float("-inf"))
        for b in range(0, batch, 2):
            mask[b, :, :, tokens - tokens // 3:] = float("-inf")  # rows past that point: all keys masked
    elif kind == "soft":  # arbitrary finite biases everywhere, no structure
        mask = torch.randn(batch, 1, tokens, tokens, generator=generator)
    elif kind == "soft_causal":
        mask = (0.5 * torch.randn(batch, 1, tokens, tokens, generator=generator)).masked_fill(
            future, float("-inf"))
    elif kind == "empty_rows":  # causal; the last 50 query rows of sequence 0 see no key at all
        mask.masked_fill_(future, float("-inf"))
        mask[0, :, tokens - 50:, :] = float("-inf")
    elif kind == "zero":
        pass
    else:
        raise AssertionError(kind)
    return mask


@pytest.mark.parametrize("kind", ["causal", "sliding_window", "padded", "soft", "soft_causal", "zero",
                                  "empty_rows"])
@pytest.mark.parametrize("batch,tokens,hq,hkv,d", [(2, 300, 14, 2, 64), (1, 1100, 14, 2, 64),
                                                   (2, 257, 8, 4, 128), (3, 128, 4, 2, 64)])
def test_prefill_attention_masked_tensor_memory_path(kind, batch, tokens, hq, hkv, d, monkeypatch):
    """The reference's contract (any additive B x 1 x T x T mask) on the tcgen05 kernel with its
    mask-tile pre-pass, against the oracle and against the warp-level kernel; rows whose keys are
    all masked are NaN in both, as in the reference."""
    g = torch.Generator().manual_seed(tokens + d + len(kind))
    q = torch.randn(batch, tokens, hq, d, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(batch, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(batch, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    mask = _mask_case(kind, batch, tokens, g)
    ref = serve_ops.prefill_attention(q, k, v, mask, groups=hq // hkv, scale=d ** -0.5)
    out = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), mask.cuda(), scale=d ** -0.5)
    with kernels.kernel_variants(prefill_attention="mma.sync"):
        warp = b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), mask.cuda(), scale=d ** -0.5)
    if kind == "empty_rows":
        # Exactly the rows without a visible key are NaN (softmax over nothing, execution.py:733-739).
        # (The CPU matmul behind the oracle lets the NaN probabilities of row T - 50 leak into
        # the row before it, so that one row is left out of the comparison.)
        assert torch.isnan(ref[0, :, -50:]).all()
        for result in (out, warp):
            assert torch.isnan(result[0, :, -50:]).all()
            assert not torch.isnan(result[0, :, :tokens - 50]).any() and not torch.isnan(result[1:]).any()
            close(result[0, :, :tokens - 51], ref[0, :, :tokens - 51], BF16_TOL)
            if batch > 1:
                close(result[1:], ref[1:], BF16_TOL)
    else:
        close(out, ref, BF16_TOL)
        close(warp, ref, BF16_TOL)
    # one mask for every sequence (batch stride 0) is classified once
    if kind in ("causal", "sliding_window"):
        shared = mask[:1].cuda().expand(batch, 1, tokens, tokens)
        close(b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), shared, scale=d ** -0.5), ref,
              BF16_TOL)
    kernels.runtime().check_status()


def test_prefill_attention_masked_strided_mask_falls_back():
    """A mask whose rows are not 16-byte aligned cannot take the vector path: it still works."""
    g = torch.Generator().manual_seed(9)
    batch, tokens, hq, hkv, d = 1, 130, 4, 2, 64
    q = torch.randn(batch, tokens, hq, d, generator=g).bfloat16().transpose(1, 2)
    k = torch.randn(batch, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    v = torch.randn(batch, tokens, hkv, d, generator=g).bfloat16().transpose(1, 2)
    wide = torch.randn(batch, 1, tokens, tokens + 1, generator=g).cuda()
    mask = wide[..., 1:]  # row stride T + 1, first element off by 4 bytes
    ref = serve_ops.prefill_attention(q, k, v, mask.cpu(), groups=2, scale=0.125)
    close(b200.b200_prefill_attention(q.cuda(), k.cuda(), v.cuda(), mask, scale=0.125), ref, BF16_TOL)
