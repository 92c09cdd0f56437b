"""Paged KV (block pools + block table): store and decode attention through the table against the
contiguous oracle on the same logical KV, a pool smaller than batch x capacity shared by
sequences of very different lengths, and the reference's decode graph run on a paged state."""

import json
from pathlib import Path

import pytest
import torch

from oracle import serve_ops
import llm_compiler_b200 as b200
from llm_compiler_b200 import kernel_ir as ir
from llm_compiler_b200 import kernels
from llm_compiler_b200 import qwen2 as q2
from llm_compiler_b200.engine import Qwen2Engine
from llm_compiler_b200.executor import B200Executor, bind_arguments
from llm_compiler_b200.kv_state import ExecutionError, PagedKVCacheState

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def close(actual, expected, tol=2e-2):
    actual, expected = actual.float().cpu(), expected.float()
    assert torch.equal(torch.isnan(actual), torch.isnan(expected))
    scale = max(1.0, float(expected.nan_to_num().abs().max()))
    assert float((actual - expected).nan_to_num().abs().max()) <= tol * scale


@pytest.mark.parametrize("hq,hkv,d", [(14, 2, 64), (28, 4, 128)])
@pytest.mark.parametrize("block_size", [32, 128])
@pytest.mark.parametrize("split_tokens", [0, 64, 512])
def test_paged_store_and_decode_attention_match_the_contiguous_oracle(hq, hkv, d, block_size, split_tokens):
    g = torch.Generator().manual_seed(hq + block_size + split_tokens)
    lengths = torch.tensor([1000, 1, 33, 640, 0, 257])
    batch, max_tokens = lengths.numel(), 1024
    state = PagedKVCacheState.allocate_paged(
        num_layers=1, batch=batch, max_tokens=max_tokens, block_size=block_size,
        num_blocks=batch * max_tokens // block_size, kv_heads=hkv, head_dim=d, dtype=torch.bfloat16,
        device="cuda")
    order = torch.randperm(batch * max_tokens // block_size, generator=g).tolist()  # scattered blocks
    state.reserve((lengths + 1).tolist(), order=order)
    keys = torch.randn(batch, max_tokens, hkv, d, generator=g).bfloat16()
    values = torch.randn(batch, max_tokens, hkv, d, generator=g).bfloat16()
    # the prompts in one store at position 0
    longest = int(lengths.max())
    zeros = torch.zeros(batch, dtype=torch.int64, device="cuda")
    state.reserve([longest + 1] * batch, order=order)  # every sequence may take the whole prompt store
    state.store(0, keys[:, :longest].transpose(1, 2).cuda(), values[:, :longest].transpose(1, 2).cuda(), zeros)
    state.lengths[0].copy_(lengths)
    for b in (0, 3, 5):
        got_k, got_v = state.gather(0, b, int(lengths[b]))
        assert torch.equal(got_k.cpu(), keys[b, :lengths[b]]) and torch.equal(got_v.cpu(), values[b, :lengths[b]])
    # one decode append at position lengths[b], then attention over lengths + 1
    new_k = torch.randn(batch, hkv, 1, d, generator=g).bfloat16()
    new_v = torch.randn(batch, hkv, 1, d, generator=g).bfloat16()
    state.store(0, new_k.cuda(), new_v.cuda(), state.positions(0))
    state = state.advance(0, delta=1)
    query = torch.randn(batch, 1, hq, d, generator=g).bfloat16().transpose(1, 2)
    mask = torch.zeros(batch, 1, 1, max_tokens)
    mask[:, :, :, 5::9] = float("-inf")
    out = state.decode_attention(0, query.cuda(), mask.cuda(), groups=hq // hkv, scale=d ** -0.5,
                                 split_tokens=split_tokens)
    ref_k, ref_v = keys.clone(), values.clone()
    serve_ops.kv_store(ref_k, ref_v, new_k, new_v, lengths)
    ref = serve_ops.decode_attention(query, ref_k, ref_v, lengths + 1, mask, groups=hq // hkv,
                                     scale=d ** -0.5)
    close(out, ref)
    none = state.decode_attention(0, query.cuda(), None, groups=hq // hkv, scale=d ** -0.5,
                                  split_tokens=split_tokens)
    ref_none = serve_ops.decode_attention(query, ref_k, ref_v, lengths + 1, torch.zeros_like(mask),
                                          groups=hq // hkv, scale=d ** -0.5)
    close(none, ref_none)
    state.check()


@pytest.mark.parametrize("hq,hkv,d", [(14, 2, 64), (28, 4, 128)])
@pytest.mark.parametrize("block_size", [32, 128])
def test_fused_qkv_attention_on_pools_equals_the_contiguous_launch(hq, hkv, d, block_size):
    """The decode layer's fused launch (q|k|v reduced from split-K partials, folded-RMSNorm factor,
    bias, RoPE, KV store, attention) through a block table: output and stored rows bit-equal to
    the same launch on contiguous buffers holding the same logical KV; a sequence whose next row
    has no block raises the overflow bit and writes nothing."""
    g = torch.Generator().manual_seed(hq * 7 + block_size)
    hidden, capacity = 256, 512
    lengths = torch.tensor([1, 64, 65, 200, 511, 131])  # attention lengths, the new token counted
    batch = lengths.numel()
    width = (hq + 2 * hkv) * d
    x = (torch.randn(batch, hidden, generator=g) * 2.0).bfloat16().cuda()
    norm_w = (1.0 + 0.2 * torch.randn(hidden, generator=g)).bfloat16().cuda()
    w = (torch.randn(width, hidden, generator=g) * 0.05).bfloat16().cuda()
    bias = torch.randn(width, generator=g).bfloat16().cuda()
    cos, sin = serve_ops.rope_table((lengths - 1).view(batch, 1), serve_ops.rope_inverse_frequency(d, 1e6),
                                    torch.bfloat16)
    kbuf = torch.randn(batch, capacity, hkv, d, generator=g).bfloat16().cuda()
    vbuf = torch.randn(batch, capacity, hkv, d, generator=g).bfloat16().cuda()
    state = PagedKVCacheState.allocate_paged(
        num_layers=1, batch=batch, max_tokens=capacity, block_size=block_size,
        num_blocks=batch * capacity // block_size, kv_heads=hkv, head_dim=d, dtype=torch.bfloat16,
        device="cuda")
    order = torch.randperm(batch * capacity // block_size, generator=g).tolist()
    state.reserve([capacity] * batch, order=order)
    state.store(0, kbuf.transpose(1, 2), vbuf.transpose(1, 2), torch.zeros(batch, dtype=torch.int64, device="cuda"))
    folded = kernels.b200_scale_columns(w, norm_w)
    partials, squares = kernels.b200_linear_partial(x, folded, row_squares=True)
    device_lengths = lengths.cuda()
    common = dict(q_heads=hq, scale=d ** -0.5, norm_row_squares=squares, norm_hidden=hidden, norm_epsilon=1e-6)
    flat = kernels.b200_qkv_decode_attention(partials, bias, cos.cuda(), sin.cuda(), kbuf, vbuf,
                                             device_lengths, **common)
    paged = kernels.b200_paged_qkv_decode_attention(partials, bias, cos.cuda(), sin.cuda(), state.keys[0],
                                                    state.values[0], state.block_table, device_lengths,
                                                    **common)
    assert torch.equal(paged, flat)
    # a service order only decides which CTAs take which sequence
    order = torch.tensor([4, 3, 5, 2, 1, 0], dtype=torch.int32, device="cuda")
    assert torch.equal(kernels.b200_qkv_decode_attention(partials, bias, cos.cuda(), sin.cuda(), kbuf, vbuf,
                                                         device_lengths, sequence_order=order, **common), flat)
    assert torch.equal(kernels.b200_paged_qkv_decode_attention(
        partials, bias, cos.cuda(), sin.cuda(), state.keys[0], state.values[0], state.block_table,
        device_lengths, sequence_order=order, **common), flat)
    for b in range(batch):
        got_k, got_v = state.gather(0, b, int(lengths[b]))
        assert torch.equal(got_k, kbuf[b, :lengths[b]]) and torch.equal(got_v, vbuf[b, :lengths[b]])
    kernels.runtime().check_status()
    # sequence 3 loses its blocks: its new row has nowhere to go
    state.release(3)
    before_k = state.keys[0].clone()
    kernels.b200_paged_qkv_decode_attention(partials, bias, cos.cuda(), sin.cuda(), state.keys[0],
                                            state.values[0], state.block_table, device_lengths, **common)
    with pytest.raises((ExecutionError, ValueError, RuntimeError)):
        kernels.runtime().check_status()
    rows_written = (state.keys[0] != before_k).flatten(2).any(dim=2).sum().item()
    assert rows_written == 0  # the other sequences rewrote identical rows, sequence 3 wrote none


def test_a_pool_smaller_than_batch_times_capacity_serves_ragged_sequences():
    """Four sequences of 2000 / 100 / 64 / 1500 tokens with a logical capacity of 2048: contiguous
    slots need 4 x 16 blocks of 128 tokens, the pool holds 32; a fifth long sequence does not fit
    until one is released."""
    lengths = [2000, 100, 64, 1500]
    state = PagedKVCacheState.allocate_paged(num_layers=2, batch=4, max_tokens=2048, block_size=128,
                                             num_blocks=32, kv_heads=2, head_dim=64,
                                             dtype=torch.bfloat16, device="cuda")
    state.reserve([n + 1 for n in lengths])
    assert state.blocks_in_use() == 16 + 1 + 1 + 12
    with pytest.raises(ExecutionError, match="exhausted"):
        state.reserve([2000, 2000, 64, 1500])
    state.release(0)
    assert state.blocks_in_use() == 16  # sequence 0's 16 blocks came back (sequence 1 kept the 2 it grabbed)
    with pytest.raises(ExecutionError, match="beyond the paged capacity"):
        state.reserve([4096, 100, 64, 1500])
    # a store through an unassigned table entry is refused with a status bit, nothing is written
    key = torch.ones(4, 2, 1, 64, dtype=torch.bfloat16, device="cuda")
    state.store(0, key, key, torch.tensor([0, 2000, 0, 0], device="cuda"))  # sequence 1 owns 1 block
    with pytest.raises(ExecutionError):
        state.check()


@pytest.mark.parametrize("batch,mode", [(4, "fast"), (64, "fast"), (70, "fast"), (4, "pytorch_compatible")])
def test_engine_on_the_paged_layout_equals_the_contiguous_engine(batch, mode):
    """Qwen2Engine(kv_layout="paged"): prefill stores through the block table, the decode step
    (the five-launch chain up to 64 sequences, the separate kernels beyond and in the compatible
    mode) reads and appends through it, blocks are handed out a block ahead of the captured
    graph's replays. 32-token blocks and 45 steps from a 50-token prompt: every sequence crosses
    a block boundary under graph replay. Logits and tokens bit-equal to the contiguous
    engine (same kernels, same arithmetic, another address map)."""
    config = q2.Qwen2Config(hidden_size=896, intermediate_size=4864, num_layers=3, num_heads=14,
                            num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=8192,
                            tie_word_embeddings=True)
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=9, dtype=torch.bfloat16).items()}
    prompt = q2.make_prompt_ids(config, batch, 50, seed=4)
    # 65 - 128 sequences: the contiguous engine runs its seven-launch chain, the paged one the
    # separate kernels (other summation orders): compared within the bf16 tolerance, teacher-forced
    exact = not (mode == "fast" and 64 < batch <= 128)
    runs = {}
    for layout in ("contiguous", "paged"):
        engine = Qwen2Engine(config, weights, batch=batch, capacity=128, numerical_mode=mode,
                             kv_layout=layout, block_size=32)
        engine.prefill(prompt)
        record = [engine.logits.clone()]
        forced = runs.get("contiguous")
        for step in range(45):
            if step == 1:
                engine.capture()  # the first step ran eagerly
            if forced is not None:
                engine.input_ids.copy_(forced[2 * step + 1])
            record.append(engine.input_ids.clone())
            engine.decode_step(feed_back=forced is None)
            record.append(engine.logits.clone())
        engine.state.check()
        runs[layout] = record
        if layout == "paged":
            assert engine.state.blocks_in_use() == batch * 3  # 95 tokens held: 3 of the 4 blocks a slot would pin
    for flat, paged in zip(runs["contiguous"], runs["paged"]):
        if exact or flat.dtype == torch.int64:
            assert torch.equal(flat, paged)
        else:
            scale = float(flat.float().abs().max())
            assert float((flat.float() - paged.float()).abs().max()) <= max(5e-2 * scale, 2e-3)


@pytest.mark.parametrize("chain", [True, False])
def test_reference_decode_graph_on_a_paged_state(chain, golden_tiny):
    """The reference-compiled bf16 decode graph, unchanged, driven over a PagedKVCacheState: the
    executor reaches the paged store / attention through the state object."""
    gold = golden_tiny["bf16"]
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0, dtype=torch.bfloat16).items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt, steps = gold["batch"], gold["prompt"], gold["steps"]
    state = PagedKVCacheState.allocate_paged(
        num_layers=config.num_layers, batch=batch, max_tokens=gold["capacity"], block_size=32,
        num_blocks=8, kv_heads=config.num_kv_heads, head_dim=config.head_dim, dtype=torch.bfloat16,
        device="cuda")
    state.reserve([prompt + steps] * batch, order=[5, 2, 7, 0, 3, 1, 6, 4])
    zeros = torch.zeros(batch, dtype=torch.int64, device="cuda")
    for layer in range(config.num_layers):  # the prompt's KV as the reference's prefill left it
        state.store(layer, gold["keys"][layer][:, :prompt].transpose(1, 2).cuda(),
                    gold["values"][layer][:, :prompt].transpose(1, 2).cuda(), zeros)
        state.lengths[layer].fill_(prompt)
    module = ir.module_from_json(json.loads((GOLDEN / "kernel_ir_tiny_bf16_decode_fast.json").read_text()))
    ir.lower_to_b200(module, zero_mask_arguments=("attention_mask",) if chain else ())
    executor = B200Executor()
    for step in range(steps):
        logits, state = executor.run(module, bind_arguments(module.functions[0], weights, {
            "input_ids": gold["tokens"][:, step].view(batch, 1).cuda(),
            "attention_mask": torch.zeros(batch, 1, 1, prompt + step + 1, device="cuda"),
            "position_ids": torch.full((batch, 1), prompt + step, device="cuda"),
            "kv_state": state, "inv_freq": inv_freq})).outputs
        assert isinstance(state, PagedKVCacheState)
        close(logits[:, 0], gold["decode_logits"][step])
    state.check()
    assert torch.equal(torch.stack(list(state.lengths), 0).cpu(), gold["lengths"])
    for layer in range(config.num_layers):
        for b in range(batch):
            got_k, got_v = state.gather(layer, b, prompt + steps)
            close(got_k, gold["keys"][layer][b, :prompt + steps])
            close(got_v, gold["values"][layer][b, :prompt + steps])
