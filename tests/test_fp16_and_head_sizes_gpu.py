"""fp16 tensors and the head sizes 16 / 32 / 256 through the C ABI, against the CPU oracle.

The reference's Triton kernels accept fp16 next to bf16 and fp32
(backends/triton_linear.py:100-105) and any head size Triton can tile; no benchmark
configuration uses either. Here both run on the generic CUDA-core kernels (fp32 arithmetic,
the 16-bit type rounded where the reference rounds), so the bar is the reference's own fp16
tolerance band (tests/test_linear.py:165-180: 2e-3 ... 3e-2): 4e-3 of the output scale;
copies are bit-exact. The last block compares with the reference's own fp16 outputs
(tests/golden/ops_fp16.pt), to which the oracle is pinned bit for bit.
"""

import pytest
import torch

import cases
from oracle import serve_ops
import llm_compiler_b200 as b200
from llm_compiler_b200 import kernels

pytestmark = pytest.mark.gpu

F16_TOL = 4e-3
TOLERANCE = {torch.float16: F16_TOL, torch.bfloat16: 2e-2, torch.float32: 3e-5}


def close(actual, expected, tol):
    actual, expected = actual.float().cpu(), expected.float()
    assert actual.shape == expected.shape
    assert torch.equal(torch.isnan(actual), torch.isnan(expected))
    scale = max(1.0, float(expected.nan_to_num().abs().max()))
    diff = (actual - expected).nan_to_num().abs().max().item()
    assert diff <= tol * scale, f"max abs diff {diff} > {tol} * {scale}"


def exact(actual, expected):
    torch.testing.assert_close(actual.cpu(), expected, rtol=0, atol=0, equal_nan=True)


def half(*shape, generator, scale=1.0):
    return (torch.randn(*shape, generator=generator) * scale).half()


def test_fp16_kv_store_contiguous_and_paged_are_exact():
    g = torch.Generator().manual_seed(1)
    b, c, h, d, t = 3, 40, 2, 64, 5
    kbuf, vbuf = half(b, c, h, d, generator=g), half(b, c, h, d, generator=g)
    key = half(b, t, h, d, generator=g).transpose(1, 2)  # strided B x H x T x D view
    value = half(b, h, t, d, generator=g)
    positions = torch.tensor([0, 7, c - t])
    expected_k, expected_v = kbuf.clone(), vbuf.clone()
    serve_ops.kv_store(expected_k, expected_v, key, value, positions)
    k_dev, v_dev = kbuf.cuda(), vbuf.cuda()
    b200.b200_kv_store(k_dev, v_dev, key.cuda(), value.cuda(), positions.cuda())
    exact(k_dev, expected_k)
    exact(v_dev, expected_v)
    # the same rows through a block table: block_size 8, sequence s owns blocks 5s .. 5s+4
    block_size, blocks_each = 8, c // 8
    table = (torch.arange(b * blocks_each, dtype=torch.int32).view(b, blocks_each)).cuda()
    k_pool = torch.zeros(b * blocks_each, block_size, h, d, dtype=torch.float16, device="cuda")
    v_pool = torch.zeros_like(k_pool)
    kernels.b200_paged_kv_store(k_pool, v_pool, table, key.cuda(), value.cuda(), positions.cuda())
    for s in range(b):
        rows = slice(s * c + int(positions[s]), s * c + int(positions[s]) + t)
        exact(k_pool.view(-1, h, d)[rows], key[s].transpose(0, 1).contiguous())
        exact(v_pool.view(-1, h, d)[rows], value[s].transpose(0, 1).contiguous())
    kernels.runtime().check_status()


def test_fp16_rope_table_rope_and_the_decode_fusion():
    g = torch.Generator().manual_seed(2)
    b, hq, hkv, t, d = 2, 4, 2, 6, 64
    inv_freq = serve_ops.rope_inverse_frequency(d, 10000.0)
    positions = torch.arange(t).repeat(b, 1) + torch.tensor([[0], [11]])
    cos_ref, sin_ref = serve_ops.rope_table(positions, inv_freq, torch.float16)
    cos, sin = b200.b200_rope_table(positions.cuda(), inv_freq.cuda(), torch.float16)
    close(cos, cos_ref, 1e-3)
    close(sin, sin_ref, 1e-3)
    q, k = half(b, hq, t, d, generator=g), half(b, hkv, t, d, generator=g)
    q_ref, k_ref = serve_ops.rope(q, k, cos_ref, sin_ref)
    q_out, k_out = b200.b200_rope(q.cuda(), k.cuda(), cos_ref.cuda(), sin_ref.cuda())
    close(q_out, q_ref, 1e-3)
    close(k_out, k_ref, 1e-3)
    # one decode token: rope + KV store in one launch == the two operators
    q1, k1, v1 = q[:, :, :1].contiguous(), k[:, :, :1].contiguous(), half(b, hkv, 1, d, generator=g)
    cos1, sin1 = cos_ref[:, :1].contiguous(), sin_ref[:, :1].contiguous()
    q1_ref, k1_ref = b200.b200_rope(q1.cuda(), k1.cuda(), cos1.cuda(), sin1.cuda())
    slots = torch.tensor([3, 0])
    kbuf = torch.zeros(b, 8, hkv, d, dtype=torch.float16, device="cuda")
    vbuf = torch.zeros_like(kbuf)
    q1_out = b200.b200_rope_kv_store(q1.cuda(), k1.cuda(), v1.cuda(), cos1.cuda(), sin1.cuda(), kbuf,
                                     vbuf, slots.cuda())
    exact(q1_out, q1_ref.cpu())
    for s in range(b):
        exact(kbuf[s, int(slots[s])], k1_ref[s, :, 0].cpu())
        exact(vbuf[s, int(slots[s])], v1[s, :, 0])


@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
def test_fp16_rms_norm(mode):
    g = torch.Generator().manual_seed(3)
    x, w = half(5, 896, generator=g), half(896, generator=g)
    for round_before_weight in (False, True):
        ref = serve_ops.rms_norm(x, w, 1e-6, round_before_weight=round_before_weight)
        out = b200.b200_rms_norm(x.cuda(), w.cuda(), epsilon=1e-6, numerical_mode=mode,
                                 round_before_weight=round_before_weight)
        assert out.dtype == torch.float16
        close(out, ref, 2e-3)


@pytest.mark.parametrize("m,k,n", [(1, 256, 512), (37, 896, 1152), (130, 200, 96)])
def test_fp16_linear_and_its_epilogues(m, k, n):
    g = torch.Generator().manual_seed(m + k + n)
    x = half(m, k, generator=g)
    w, bias = half(n, k, generator=g, scale=0.05), half(n, generator=g)
    residual = half(m, n, generator=g)
    out = b200.b200_linear(x.cuda(), w.cuda(), bias.cuda())
    assert out.dtype == torch.float16
    close(out, serve_ops.linear(x, w, bias), F16_TOL)
    close(b200.b200_linear(x.cuda(), w.cuda()), serve_ops.linear(x, w), F16_TOL)
    close(b200.b200_linear(x.cuda(), w.cuda(), bias.cuda(), residual=residual.cuda(), epilogue="residual"),
          serve_ops.residual_add(serve_ops.linear(x, w, bias), residual), F16_TOL)
    packed = kernels.interleave_gate_up(w[: n // 2].cuda(), w[n // 2:].cuda())
    close(b200.b200_linear(x.cuda(), packed, epilogue="swiglu"),
          serve_ops.swiglu(serve_ops.linear(x, w[: n // 2]), serve_ops.linear(x, w[n // 2:])), F16_TOL)


def test_fp16_embedding_swiglu_add_cast_argmax():
    g = torch.Generator().manual_seed(5)
    table, ids = half(300, 256, generator=g), torch.randint(0, 300, (3, 4), generator=g)
    exact(b200.b200_embedding(table.cuda(), ids.cuda()), serve_ops.embedding(table, ids))
    gate, up = half(5, 512, generator=g), half(5, 512, generator=g)
    close(b200.b200_swiglu(gate.cuda(), up.cuda()), serve_ops.swiglu(gate, up), F16_TOL)
    exact(b200.b200_add(gate.cuda(), up.cuda()), gate + up)
    odd = half(33, generator=g)
    exact(b200.b200_add(odd.cuda(), odd.cuda()), odd + odd)  # scalar path
    wide = torch.randn(4, 6, 10, generator=g)
    exact(b200.b200_contiguous(wide.cuda().transpose(0, 2), torch.float16),
          wide.transpose(0, 2).contiguous().half())
    exact(b200.b200_contiguous(gate.cuda(), torch.float32), gate.float())
    logits = half(6, 40001, generator=g)
    logits[2, 77] = 100.0
    logits[2, 5000] = 100.0  # tie: lowest index wins
    exact(b200.b200_argmax(logits.cuda()), logits.float().argmax(-1))
    kernels.runtime().check_status()


@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
@pytest.mark.parametrize("d", [64, 128])
def test_fp16_decode_attention_ragged_and_masked(d, mode):
    g = torch.Generator().manual_seed(d)
    b, c, hq, hkv = 5, 300, 8, 2
    q = half(b, 1, hq, d, generator=g).transpose(1, 2)
    kbuf, vbuf = half(b, c, hkv, d, generator=g), half(b, c, hkv, d, generator=g)
    lengths = torch.tensor([0, 1, 17, 200, c])
    mask = torch.zeros(b, 1, 1, c)
    mask[:, :, :, 3::7] = float("-inf")
    mask[1, :, :, 0] = 0.0
    ref = serve_ops.decode_attention(q, kbuf, vbuf, lengths, mask, groups=hq // hkv, scale=d ** -0.5)
    args = (q.cuda(), kbuf.cuda(), vbuf.cuda(), lengths.cuda())
    out = b200.b200_decode_attention(*args, mask.cuda(), scale=d ** -0.5, numerical_mode=mode)
    assert out.dtype == torch.float16 and torch.isnan(out[0]).all()
    close(out, ref, F16_TOL)
    close(b200.b200_decode_attention(*args, mask.half().cuda(), scale=d ** -0.5), ref, F16_TOL)  # fp16 mask
    kernels.runtime().check_status()


@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
def test_fp16_prefill_attention_causal_and_masked(mode):
    g = torch.Generator().manual_seed(6)
    b, t, hq, hkv, d = 2, 70, 4, 2, 64
    q = half(b, t, hq, d, generator=g).transpose(1, 2)
    k = half(b, t, hkv, d, generator=g).transpose(1, 2)
    v = half(b, t, hkv, d, generator=g).transpose(1, 2)
    causal = serve_ops.causal_mask(b, t)
    ref = serve_ops.prefill_attention(q, k, v, causal, groups=2, scale=0.125)
    args = (q.cuda(), k.cuda(), v.cuda())
    close(b200.b200_prefill_attention(*args, causal.cuda(), scale=0.125, numerical_mode=mode), ref, F16_TOL)
    close(b200.b200_prefill_attention(*args, None, scale=0.125, causal=True, numerical_mode=mode), ref,
          F16_TOL)
    soft = torch.randn(1, 1, t, t, generator=g)  # additive, broadcast over the batch
    soft[:, :, :, 5::9] = float("-inf")
    close(b200.b200_prefill_attention(*args, soft.cuda(), scale=0.125, numerical_mode=mode),
          serve_ops.prefill_attention(q, k, v, soft, groups=2, scale=0.125), F16_TOL)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("d", [16, 32, 256])
def test_head_sizes_beside_64_and_128(d, dtype):
    """Decode and prefill attention at the head sizes the tensor-core kernels do not take."""
    g = torch.Generator().manual_seed(d)
    b, c, hq, hkv, t = 3, 90, 4, 2, 33
    tol = TOLERANCE[dtype]
    q = torch.randn(b, 1, hq, d, generator=g).to(dtype).transpose(1, 2)
    kbuf = torch.randn(b, c, hkv, d, generator=g).to(dtype)
    vbuf = torch.randn(b, c, hkv, d, generator=g).to(dtype)
    lengths = torch.tensor([1, 40, c])
    mask = torch.zeros(b, 1, 1, c)
    ref = serve_ops.decode_attention(q, kbuf, vbuf, lengths, mask, groups=2, scale=d ** -0.5)
    out = b200.b200_decode_attention(q.cuda(), kbuf.cuda(), vbuf.cuda(), lengths.cuda(), mask.cuda(),
                                     scale=d ** -0.5)
    close(out, ref, tol)
    qp = torch.randn(b, t, hq, d, generator=g).to(dtype).transpose(1, 2)
    kp = torch.randn(b, t, hkv, d, generator=g).to(dtype).transpose(1, 2)
    vp = torch.randn(b, t, hkv, d, generator=g).to(dtype).transpose(1, 2)
    ref = serve_ops.prefill_attention(qp, kp, vp, serve_ops.causal_mask(b, t), groups=2, scale=d ** -0.5)
    close(b200.b200_prefill_attention(qp.cuda(), kp.cuda(), vp.cuda(), None, scale=d ** -0.5, causal=True),
          ref, tol)
    close(b200.b200_prefill_attention(qp.cuda(), kp.cuda(), vp.cuda(), serve_ops.causal_mask(b, t).cuda(),
                                      scale=d ** -0.5), ref, tol)
    kernels.runtime().check_status()


# ------------------------------- the reference's own fp16 outputs (tests/golden/ops_fp16.pt) ----
@pytest.mark.parametrize("name", list(cases.KV_STORE_F16))
def test_fp16_kv_store_golden(name, golden_ops):
    x = cases.kv_store_inputs(name)
    kbuf, vbuf = x["key_buffer"].cuda(), x["value_buffer"].cuda()
    b200.b200_kv_store(kbuf, vbuf, x["key"].cuda(), x["value"].cuda(), x["positions"].cuda())
    exact(kbuf, golden_ops[name]["key_out"])
    exact(vbuf, golden_ops[name]["value_out"])


@pytest.mark.parametrize("name", list(cases.ROPE_F16))
def test_fp16_rope_golden(name, golden_ops):
    x, gold = cases.rope_inputs(name), golden_ops[name]
    q, k = b200.b200_rope(x["query"].cuda(), x["key"].cuda(), gold["cosine"].cuda(), gold["sine"].cuda())
    close(q, gold["query_out"], 1e-3)
    close(k, gold["key_out"], 1e-3)


@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
@pytest.mark.parametrize("name", list(cases.RMS_NORM_F16))
def test_fp16_rms_norm_golden(name, mode, golden_ops):
    x = cases.rms_norm_inputs(name)
    out = b200.b200_rms_norm(x["input"].cuda(), x["weight"].cuda(), epsilon=x["epsilon"],
                             round_before_weight=x["round_before_weight"], numerical_mode=mode)
    close(out, golden_ops[name]["output"], 2e-3)


@pytest.mark.parametrize("name", list(cases.DECODE_ATTENTION_F16))
def test_fp16_decode_attention_golden(name, golden_ops):
    x = cases.decode_attention_inputs(name)
    out = b200.b200_decode_attention(x["query"].cuda(), x["key_buffer"].cuda(), x["value_buffer"].cuda(),
                                     x["lengths"].cuda(), x["mask"].cuda(), scale=x["scale"])
    close(out, golden_ops[name]["output"], F16_TOL)


@pytest.mark.parametrize("name", list(cases.PREFILL_ATTENTION_F16))
def test_fp16_prefill_attention_golden(name, golden_ops):
    x = cases.prefill_attention_inputs(name)
    out = b200.b200_prefill_attention(x["query"].cuda(), x["key"].cuda(), x["value"].cuda(), x["mask"].cuda(),
                                      scale=x["scale"])
    close(out, golden_ops[name]["output"], F16_TOL)


@pytest.mark.parametrize("name", list(cases.LINEAR_F16))
def test_fp16_linear_golden(name, golden_ops):
    x = cases.linear_inputs(name)
    bias = x["bias"].cuda() if x["bias"] is not None else None
    close(b200.b200_linear(x["input"].cuda(), x["weight"].cuda(), bias), golden_ops[name]["output"], F16_TOL)


@pytest.mark.parametrize("name", list(cases.ROPE_TABLE_F16))
def test_fp16_rope_table_golden(name, golden_ops):
    x = cases.rope_table_inputs(name)
    inv_freq = serve_ops.rope_inverse_frequency(x["head_dim"], x["theta"])
    cos, sin = b200.b200_rope_table(x["position_ids"].cuda(), inv_freq.cuda(), torch.float16)
    close(cos, golden_ops[name]["cosine"], 1e-3)
    close(sin, golden_ops[name]["sine"], 1e-3)
