"""Seeded inputs of the per-operator golden cases.

Shared by make_golden.py (which feeds them to the reference and stores only the OUTPUTS in
ops.pt) and by the tests (which regenerate the same inputs from the same seeds). Shapes and
seeds follow the reference's own GPU tests: tests/test_triton_backend.py:380-466 (decode
attention B=3, C=65, Hq=4, Hkv=2, D=16, lengths [7, 31, 65]; KV store B=3, C=16, H=2, D=8,
positions [1, 5, 9]), tests/test_prefill_attention.py:33-253 ((B, T) in {(1,2), (2,7), (1,33)},
the all-zero mask, the bf16 case B=2, Hq=14, Hkv=2, T=7, D=64 with seed 2026),
tests/test_rope.py:228-290, tests/test_triton_backend.py:78-93 (RMSNorm bf16 7 x 896) and
tests/test_linear.py:123-163.
"""

from __future__ import annotations

import torch

F32, BF16, F16 = torch.float32, torch.bfloat16, torch.float16


def _randn(generator, *shape, dtype=F32):
    return torch.randn(*shape, generator=generator, dtype=torch.float32).to(dtype)


def causal_mask(batch, tokens):
    future = torch.triu(torch.ones(tokens, tokens, dtype=torch.bool), diagonal=1)
    return torch.zeros(batch, 1, tokens, tokens).masked_fill(future, float("-inf"))


KV_STORE = {  # name: (B, C, H, D, T, dtype, positions)
    "kv_store_f32": (3, 16, 2, 8, 1, F32, [1, 5, 9]),
    "kv_store_bf16_strided": (2, 40, 2, 64, 5, BF16, [0, 33]),
    "kv_store_bf16_d128": (3, 24, 4, 128, 3, BF16, [21, 0, 7]),
}
ROPE = {  # name: (B, Hq, Hkv, T, D, dtype, seed, theta, first position)
    "rope_bf16": (2, 14, 2, 7, 64, BF16, 2026, 1e6, 3),
    "rope_bf16_decode": (5, 14, 2, 1, 64, BF16, 7, 1e6, 4095),
    "rope_bf16_d128": (2, 28, 4, 3, 128, BF16, 9, 1e6, 100),
    "rope_f32": (3, 4, 2, 1, 16, F32, 5, 1e4, 5),
}
RMS_NORM = {  # name: (rows, hidden, dtype, round_before_weight)
    "rms_norm_bf16_rbw": (7, 896, BF16, True),
    "rms_norm_bf16": (7, 896, BF16, False),
    "rms_norm_bf16_3584": (5, 3584, BF16, True),
    "rms_norm_bf16_rows64": (64, 896, BF16, True),
    "rms_norm_f32_rbw": (9, 256, F32, True),
    "rms_norm_f32_odd": (4, 1000, F32, False),
    "rms_norm_f32_long": (2, 20011, F32, True),
}
DECODE_ATTENTION = {  # name: (B, C, Hq, Hkv, D, dtype, lengths)
    "decode_attention_f32": (3, 65, 4, 2, 16, F32, [7, 31, 65]),
    "decode_attention_f32_d64": (3, 64, 4, 2, 64, F32, [6, 6, 6]),
    "decode_attention_bf16": (3, 300, 14, 2, 64, BF16, [1, 130, 300]),
    "decode_attention_bf16_long": (2, 1200, 14, 2, 64, BF16, [1200, 777]),
    "decode_attention_bf16_d128": (2, 260, 28, 4, 128, BF16, [260, 17]),
    "decode_attention_bf16_g2": (3, 96, 4, 2, 64, BF16, [96, 5, 40]),
}
PREFILL_ATTENTION = {  # name: (B, T, Hq, Hkv, D, dtype, zero mask)
    "prefill_attention_f32_1x2": (1, 2, 4, 2, 16, F32, False),
    "prefill_attention_f32_2x7": (2, 7, 4, 2, 16, F32, False),
    "prefill_attention_f32_1x33": (1, 33, 4, 2, 16, F32, False),
    "prefill_attention_f32_zero_mask": (2, 7, 4, 2, 16, F32, True),
    "prefill_attention_f32_d64": (3, 5, 4, 2, 64, F32, False),
    "prefill_attention_bf16": (2, 7, 14, 2, 64, BF16, False),
    "prefill_attention_bf16_130": (1, 130, 14, 2, 64, BF16, False),
    "prefill_attention_bf16_zero_mask": (2, 70, 14, 2, 64, BF16, True),
    "prefill_attention_bf16_d128": (1, 96, 8, 4, 128, BF16, False),
}
LINEAR = {  # name: (B, T, K, N, bias, dtype)
    "linear_f32": (2, 3, 64, 96, True, F32),
    "linear_f32_ragged": (1, 5, 100, 70, False, F32),
    "linear_bf16_bias": (2, 5, 896, 128, True, BF16),
    "linear_bf16": (1, 8, 512, 384, False, BF16),
    "linear_bf16_m64_splitk": (1, 64, 4864, 896, False, BF16),
    "linear_bf16_m200": (2, 100, 256, 200, True, BF16),
}
ROPE_TABLE = {  # name: (B, T, head_dim, theta, dtype, first position)
    "rope_table_bf16": (2, 9, 64, 1e6, BF16, 0),
    "rope_table_bf16_far": (4, 1, 64, 1e6, BF16, 4096),
    "rope_table_f32": (3, 1, 64, 1e4, F32, 5),
}

# fp16 cases (outputs in ops_fp16.pt): the reference's kernels take fp16 next to bf16
# (backends/triton_linear.py:100-105); same shapes and seeds as the bf16 cases above.
KV_STORE_F16 = {"kv_store_f16_strided": (2, 40, 2, 64, 5, F16, [0, 33])}
ROPE_F16 = {
    "rope_f16": (2, 14, 2, 7, 64, F16, 2026, 1e6, 3),
    "rope_f16_decode": (5, 14, 2, 1, 64, F16, 7, 1e6, 4095),
}
RMS_NORM_F16 = {
    "rms_norm_f16_rbw": (7, 896, F16, True),
    "rms_norm_f16": (7, 896, F16, False),
}
DECODE_ATTENTION_F16 = {
    "decode_attention_f16": (3, 300, 14, 2, 64, F16, [1, 130, 300]),
    "decode_attention_f16_d128": (2, 260, 28, 4, 128, F16, [260, 17]),
}
PREFILL_ATTENTION_F16 = {
    "prefill_attention_f16": (2, 7, 14, 2, 64, F16, False),
    "prefill_attention_f16_130": (1, 130, 14, 2, 64, F16, False),
    "prefill_attention_f16_zero_mask": (2, 70, 14, 2, 64, F16, True),
}
LINEAR_F16 = {
    "linear_f16_bias": (2, 5, 896, 128, True, F16),
    "linear_f16": (1, 8, 512, 384, False, F16),
}
ROPE_TABLE_F16 = {"rope_table_f16": (2, 9, 64, 1e6, F16, 0)}


def _case(table, table_f16, name):
    return table[name] if name in table else table_f16[name]


def kv_store_inputs(name):
    b, c, h, d, t, dtype, pos = _case(KV_STORE, KV_STORE_F16, name)
    g = torch.Generator().manual_seed(11 + c)
    return dict(key_buffer=_randn(g, b, c, h, d, dtype=dtype),
                value_buffer=_randn(g, b, c, h, d, dtype=dtype),
                key=_randn(g, b, t, h, d, dtype=dtype).transpose(1, 2),
                value=_randn(g, b, t, h, d, dtype=dtype).transpose(1, 2),
                positions=torch.tensor(pos, dtype=torch.int64))


def rope_inputs(name):
    b, hq, hkv, t, d, dtype, seed, theta, first = _case(ROPE, ROPE_F16, name)
    g = torch.Generator().manual_seed(seed)
    return dict(query=_randn(g, b, t, hq, d, dtype=dtype).transpose(1, 2),
                key=_randn(g, b, t, hkv, d, dtype=dtype).transpose(1, 2),
                position_ids=(torch.arange(t, dtype=torch.int64).view(1, -1).expand(b, -1) + first).contiguous(),
                theta=theta, head_dim=d, q_heads=hq, kv_heads=hkv)


def rms_norm_inputs(name):
    rows, hidden, dtype, rbw = _case(RMS_NORM, RMS_NORM_F16, name)
    g = torch.Generator().manual_seed(hidden + rows)
    return dict(input=_randn(g, rows, hidden, dtype=dtype),
                weight=(1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dtype),
                epsilon=1e-6, round_before_weight=rbw)


def decode_attention_inputs(name):
    b, c, hq, hkv, d, dtype, lens = _case(DECODE_ATTENTION, DECODE_ATTENTION_F16, name)
    g = torch.Generator().manual_seed(c * 7 + d)
    return dict(query=_randn(g, b, 1, hq, d, dtype=dtype).transpose(1, 2),
                key_buffer=_randn(g, b, c, hkv, d, dtype=dtype),
                value_buffer=_randn(g, b, c, hkv, d, dtype=dtype),
                lengths=torch.tensor(lens, dtype=torch.int64), mask=torch.zeros(b, 1, 1, c),
                groups=hq // hkv, scale=d ** -0.5)


def prefill_attention_inputs(name):
    b, t, hq, hkv, d, dtype, zero_mask = _case(PREFILL_ATTENTION, PREFILL_ATTENTION_F16, name)
    g = torch.Generator().manual_seed(2026 + t)
    return dict(query=_randn(g, b, t, hq, d, dtype=dtype).transpose(1, 2),
                key=_randn(g, b, t, hkv, d, dtype=dtype).transpose(1, 2),
                value=_randn(g, b, t, hkv, d, dtype=dtype).transpose(1, 2),
                mask=torch.zeros(b, 1, t, t) if zero_mask else causal_mask(b, t),
                groups=hq // hkv, scale=d ** -0.5, zero_mask=zero_mask)


def linear_inputs(name):
    b, t, k, n, bias, dtype = _case(LINEAR, LINEAR_F16, name)
    g = torch.Generator().manual_seed(k + n)
    return dict(input=_randn(g, b, t, k, dtype=dtype),
                weight=(0.05 * torch.randn(n, k, generator=g)).to(dtype),
                bias=(0.1 * torch.randn(n, generator=g)).to(dtype) if bias else None)


def rope_table_inputs(name):
    b, t, d, theta, dtype, first = _case(ROPE_TABLE, ROPE_TABLE_F16, name)
    return dict(position_ids=(torch.arange(t, dtype=torch.int64).view(1, -1).expand(b, -1) + first * (1 + torch.arange(b).view(-1, 1))).contiguous(),
                head_dim=d, theta=theta, dtype=dtype)
