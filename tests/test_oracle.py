"""The CPU oracle against the reference's own outputs (tests/golden), atol = 0.

ops.pt, ops_fp16.pt and qwen2_tiny_*.pt were produced by the reference's ReferenceExecutor; every oracle
function must reproduce them exactly on the seeded inputs of tests/golden/cases.py.
"""

import numpy as np
import pytest
import torch

import cases
from oracle import qwen2_model, serve_ops
from llm_compiler_b200 import qwen2 as q2


def same(a, b):
    torch.testing.assert_close(a, b, rtol=0, atol=0, equal_nan=True)


@pytest.mark.parametrize("name", list(cases.KV_STORE) + list(cases.KV_STORE_F16))
def test_kv_store(name, golden_ops):
    x = cases.kv_store_inputs(name)
    kbuf, vbuf = x["key_buffer"].clone(), x["value_buffer"].clone()
    serve_ops.kv_store(kbuf, vbuf, x["key"], x["value"], x["positions"])
    same(kbuf, golden_ops[name]["key_out"])
    same(vbuf, golden_ops[name]["value_out"])


def test_kv_store_overflow_raises():
    x = cases.kv_store_inputs("kv_store_f32")
    with pytest.raises(ValueError):
        serve_ops.kv_store(x["key_buffer"], x["value_buffer"], x["key"], x["value"],
                           torch.tensor([1, 5, 16]))


@pytest.mark.parametrize("name", list(cases.ROPE) + list(cases.ROPE_F16))
def test_rope(name, golden_ops):
    x = cases.rope_inputs(name)
    inv_freq = serve_ops.rope_inverse_frequency(x["head_dim"], x["theta"])
    cos, sin = serve_ops.rope_table(x["position_ids"], inv_freq, x["query"].dtype)
    same(cos, golden_ops[name]["cosine"])
    same(sin, golden_ops[name]["sine"])
    q, k = serve_ops.rope(x["query"], x["key"], cos, sin)
    same(q, golden_ops[name]["query_out"])
    same(k, golden_ops[name]["key_out"])


@pytest.mark.parametrize("name", list(cases.ROPE_TABLE) + list(cases.ROPE_TABLE_F16))
def test_rope_table(name, golden_ops):
    x = cases.rope_table_inputs(name)
    inv_freq = serve_ops.rope_inverse_frequency(x["head_dim"], x["theta"])
    cos, sin = serve_ops.rope_table(x["position_ids"], inv_freq, x["dtype"])
    same(cos, golden_ops[name]["cosine"])
    same(sin, golden_ops[name]["sine"])


@pytest.mark.parametrize("name", list(cases.RMS_NORM) + list(cases.RMS_NORM_F16))
def test_rms_norm(name, golden_ops):
    x = cases.rms_norm_inputs(name)
    kwargs = dict(round_before_weight=x["round_before_weight"])
    same(serve_ops.rms_norm(x["input"], x["weight"], x["epsilon"], **kwargs),
         golden_ops[name]["output"])
    # the order-explicit restatement gives the same bits as the reference
    same(serve_ops.rms_norm_explicit(x["input"], x["weight"], x["epsilon"], **kwargs),
         golden_ops[name]["output"])


@pytest.mark.parametrize("count", [1, 7, 8, 31, 32, 33, 255, 256, 896, 1000, 2047, 3584, 8192,
                                   16384 + 40, 32767])
def test_float_sum_order(count):
    g = torch.Generator().manual_seed(count)
    row = torch.randn(count, generator=g).pow(2)
    assert np.float32(row.sum().item()) == serve_ops.float_sum_explicit(row.numpy())


@pytest.mark.parametrize("name", list(cases.DECODE_ATTENTION) + list(cases.DECODE_ATTENTION_F16))
def test_decode_attention(name, golden_ops):
    x = cases.decode_attention_inputs(name)
    out = serve_ops.decode_attention(x["query"], x["key_buffer"], x["value_buffer"], x["lengths"],
                                     x["mask"], groups=x["groups"], scale=x["scale"])
    same(out, golden_ops[name]["output"])


def test_decode_attention_empty_sequence_is_nan():
    x = cases.decode_attention_inputs("decode_attention_f32")
    lengths = torch.tensor([0, 3, 4])
    out = serve_ops.decode_attention(x["query"], x["key_buffer"], x["value_buffer"], lengths,
                                     x["mask"], groups=x["groups"], scale=x["scale"])
    assert torch.isnan(out[0]).all() and not torch.isnan(out[1:]).any()


@pytest.mark.parametrize("name", list(cases.PREFILL_ATTENTION) + list(cases.PREFILL_ATTENTION_F16))
def test_prefill_attention(name, golden_ops):
    x = cases.prefill_attention_inputs(name)
    out = serve_ops.prefill_attention(x["query"], x["key"], x["value"], x["mask"],
                                      groups=x["groups"], scale=x["scale"])
    same(out, golden_ops[name]["output"])
    if not x["zero_mask"]:
        # proven causality needs no mask and gives the same bits (execution.py:726-737)
        same(serve_ops.prefill_attention(x["query"], x["key"], x["value"], None,
                                         groups=x["groups"], scale=x["scale"], causal=True),
             golden_ops[name]["output"])


@pytest.mark.parametrize("name", list(cases.LINEAR) + list(cases.LINEAR_F16))
def test_linear(name, golden_ops):
    x = cases.linear_inputs(name)
    same(serve_ops.linear(x["input"], x["weight"], x["bias"]), golden_ops[name]["output"])


@pytest.mark.parametrize("tag", ["fp32", "bf16", "fp16"])
def test_qwen2_tiny_stateful_decode(tag, golden_tiny):
    """Config 1 of the benchmark plan: 2-layer Qwen2, batch 3, prompt 5, capacity 64, 4 greedy
    steps; the oracle model must match the reference executor's logits, tokens and KV state."""

    gold = golden_tiny[tag]
    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[tag]
    config = q2.Qwen2Config(**gold["config"])
    weights = q2.make_weights(config, seed=gold["seed"], dtype=dtype)
    same(q2.make_prompt_ids(config, gold["batch"], gold["prompt"], seed=0), gold["input_ids"])
    logits, state = qwen2_model.prefill(config, weights, gold["input_ids"],
                                        capacity=gold["capacity"])
    same(logits, gold["prefill_logits"])
    token = logits[:, -1].argmax(-1)
    same(token, gold["tokens"][:, 0])
    for step in range(gold["steps"]):
        out = qwen2_model.decode(config, weights, token.view(-1, 1), state)
        same(out[:, 0], gold["decode_logits"][step])
        token = out[:, 0].argmax(-1)
        same(token, gold["tokens"][:, step + 1])
    used = gold["prompt"] + gold["steps"]
    same(torch.stack(state.lengths, 0), gold["lengths"])
    same(torch.stack([k[:, :used] for k in state.keys], 0), gold["keys"])
    same(torch.stack([v[:, :used] for v in state.values], 0), gold["values"])
