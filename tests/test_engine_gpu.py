"""Whole-model parity of the serving engine (CUDA-graph decode) against the reference.

qwen2_tiny_{fp32,bf16,fp16}.pt hold what the reference's own ReferenceExecutor produced for the
2-layer stateful decode (batch 3, prompt 5, capacity 64, 4 greedy steps). Tolerances: fp32
graphs 1e-4 on logits; bf16 graphs 2e-2 (fp16: 1e-2) with greedy tokens equal (a token may differ only
where the reference's own top-2 logits are closer than the tolerance).
"""

import pytest
import torch

from oracle import qwen2_model
import llm_compiler_b200 as b200
from llm_compiler_b200 import qwen2 as q2
from llm_compiler_b200.engine import Qwen2Engine

pytestmark = pytest.mark.gpu


def cuda_weights(config, dtype, seed=0):
    return {k: v.cuda() for k, v in q2.make_weights(config, seed=seed, dtype=dtype).items()}


def assert_logits(actual, expected, tol):
    actual, expected = actual.float().cpu(), expected.float()
    scale = max(1e-3, float(expected.abs().max()))
    diff = float((actual - expected).abs().max())
    assert diff <= tol * max(1.0, scale) or diff <= tol * scale * 4, f"logit diff {diff} (scale {scale})"


def assert_tokens(actual, expected, expected_logits, tol):
    actual = actual.cpu()
    for row in range(expected.shape[0]):
        if actual[row] == expected[row]:
            continue
        top2 = expected_logits[row].float().topk(2).values
        assert float(top2[0] - top2[1]) <= tol, "greedy token differs beyond a near-tie"


@pytest.mark.parametrize("tag,mode", [("fp32", "fast"), ("fp32", "pytorch_compatible"),
                                      ("bf16", "fast"), ("bf16", "pytorch_compatible"),
                                      ("fp16", "fast"), ("fp16", "pytorch_compatible")])
def test_tiny_stateful_decode_matches_reference(tag, mode, golden_tiny):
    gold = golden_tiny[tag]
    dtype, tol = {"fp32": (torch.float32, 1e-4), "bf16": (torch.bfloat16, 2e-2),
                  "fp16": (torch.float16, 1e-2)}[tag]
    config = q2.Qwen2Config(**gold["config"])
    engine = Qwen2Engine(config, cuda_weights(config, dtype), batch=gold["batch"],
                         capacity=gold["capacity"], numerical_mode=mode)
    pointers = [k.data_ptr() for k in engine.state.keys]
    logits = engine.prefill(gold["input_ids"], all_logits=True)
    assert_logits(logits, gold["prefill_logits"], tol)
    assert_tokens(engine.next_ids, gold["tokens"][:, 0], gold["prefill_logits"][:, -1], tol)
    engine.capture()
    for step in range(gold["steps"]):
        engine.input_ids.copy_(gold["tokens"][:, step].cuda())  # teacher forcing
        engine.decode_step(feed_back=False)
        assert_logits(engine.logits, gold["decode_logits"][step], tol)
        assert_tokens(engine.next_ids, gold["tokens"][:, step + 1], gold["decode_logits"][step], tol)
    engine.state.check()
    used = gold["prompt"] + gold["steps"]
    lengths = torch.stack([l for l in engine.state.lengths], 0).cpu()
    assert torch.equal(lengths, gold["lengths"])
    keys = torch.stack([k[:, :used] for k in engine.state.keys], 0)
    values = torch.stack([v[:, :used] for v in engine.state.values], 0)
    assert_logits(keys, gold["keys"], tol)
    assert_logits(values, gold["values"], tol)
    assert pointers == [k.data_ptr() for k in engine.state.keys]  # fixed KV addresses


def test_greedy_generation_with_graph_equals_eager(golden_tiny):
    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    weights = cuda_weights(config, torch.float32)
    graph = Qwen2Engine(config, weights, batch=3, capacity=64)
    eager = Qwen2Engine(config, weights, batch=3, capacity=64)
    a = graph.generate(gold["input_ids"], 6, use_graph=True)
    b = eager.generate(gold["input_ids"], 6, use_graph=False)
    assert torch.equal(a, b)
    assert torch.equal(a[:, :5].cpu(), gold["tokens"])


def test_host_step_api_round_trip(golden_tiny):
    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    engine = Qwen2Engine(config, cuda_weights(config, torch.float32), batch=3, capacity=64)
    engine.prefill(gold["input_ids"])
    engine.capture()
    tokens = gold["tokens"][:, 0].clone()
    for step in range(gold["steps"]):
        tokens = engine.step(tokens).clone()
        assert torch.equal(tokens, gold["tokens"][:, step + 1])
        # step() replays a graph of its own (host copies included): engine.logits follows it
        assert_logits(engine.logits, gold["decode_logits"][step], 1e-4 if engine.dtype == torch.float32 else 2e-2)


def test_capacity_overflow_is_reported_not_trapped(golden_tiny):
    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    engine = Qwen2Engine(config, cuda_weights(config, torch.float32), batch=3, capacity=8)
    engine.prefill(gold["input_ids"])  # 5 tokens
    for _ in range(3):
        engine.decode_step()
    engine.state.check()  # 8 tokens: full, still fine
    engine.decode_step()
    with pytest.raises(b200.ExecutionError):
        engine.state.check()


def test_qwen2_0_5b_shaped_layers_match_oracle():
    """Qwen2-0.5B shapes (hidden 896, 14/2 heads x 64, SwiGLU 4864, biases, theta 1e6) with 2
    layers and a reduced vocabulary so that the CPU oracle finishes in seconds; bf16."""
    config = q2.Qwen2Config(hidden_size=896, intermediate_size=4864, num_layers=2, num_heads=14,
                            num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=4096,
                            tie_word_embeddings=True)
    weights = q2.make_weights(config, seed=3, dtype=torch.bfloat16)
    prompt = q2.make_prompt_ids(config, 4, 37, seed=1)
    ref_tokens, ref_logits, _ = qwen2_model.greedy_generate(config, weights, prompt, 3, capacity=64)
    engine = Qwen2Engine(config, {k: v.cuda() for k, v in weights.items()}, batch=4, capacity=64)
    engine.prefill(prompt)
    assert_logits(engine.logits, ref_logits[0], 2e-2)
    engine.capture()
    for step in range(3):
        engine.input_ids.copy_(ref_tokens[:, step].cuda())
        engine.decode_step(feed_back=False)
        assert_logits(engine.logits, ref_logits[step + 1], 2e-2)
        assert_tokens(engine.next_ids, ref_tokens[:, step + 1], ref_logits[step + 1], 2e-2)
    engine.state.check()


@pytest.mark.parametrize("batch", [4, 64])
def test_programmatic_launch_changes_nothing(batch):
    """The decode chain launched with programmatic dependent launch (kernels resident early,
    waiting on the device, weight tiles fetched before the wait) must give bit-identical
    logits to the fully serialised chain, eagerly and from the captured graph; a few repeats
    shake out ordering slips that only show under timing."""
    config = q2.Qwen2Config(hidden_size=896, intermediate_size=4864, num_layers=4, num_heads=14,
                            num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=8192,
                            tie_word_embeddings=True)
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=5, dtype=torch.bfloat16).items()}
    prompt = q2.make_prompt_ids(config, batch, 150, seed=2)
    logits = {}
    for programmatic in (False, True):
        engine = Qwen2Engine(config, weights, batch=batch, capacity=256)
        engine.programmatic_launch = programmatic
        engine.prefill(prompt)
        steps = [engine.decode_step().clone() for _ in range(2)]  # eager
        engine.capture()
        for _ in range(6):
            steps.append(engine.decode_step().clone())
            steps.append(engine.logits.clone())
        engine.state.check()
        logits[programmatic] = steps
    for serial, chained in zip(logits[False], logits[True]):
        assert torch.equal(serial, chained)


def test_qwen2_7b_shaped_layers_match_oracle():
    """Qwen2-7B shapes (hidden 3584, 28/4 heads x 128, SwiGLU 18944, untied LM head) with 2 layers
    and a reduced vocabulary: the decode chain (split-K partial producers, reduce consumers,
    fused q|k|v attention at head_dim 128, 80..256-column GEMM tiles) against the CPU oracle."""
    config = q2.Qwen2Config(hidden_size=3584, intermediate_size=18944, num_layers=2, num_heads=28,
                            num_kv_heads=4, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=4096,
                            tie_word_embeddings=False)
    weights = q2.make_weights(config, seed=11, dtype=torch.bfloat16)
    prompt = q2.make_prompt_ids(config, 3, 21, seed=4)
    ref_tokens, ref_logits, _ = qwen2_model.greedy_generate(config, weights, prompt, 2, capacity=32)
    engine = Qwen2Engine(config, {k: v.cuda() for k, v in weights.items()}, batch=3, capacity=32)
    engine.prefill(prompt)
    assert_logits(engine.logits, ref_logits[0], 2e-2)
    engine.capture()
    for step in range(2):
        engine.input_ids.copy_(ref_tokens[:, step].cuda())
        engine.decode_step(feed_back=False)
        assert_logits(engine.logits, ref_logits[step + 1], 2e-2)
        assert_tokens(engine.next_ids, ref_tokens[:, step + 1], ref_logits[step + 1], 2e-2)
    engine.state.check()


def test_captured_graph_survives_workspace_growth():
    """A captured step has its workspace addresses baked in. A second, larger engine on the same
    GPU outgrows the shared workspaces; the runtime must retire the old buffers instead of
    freeing them, so that replays of the first graph still match an eager step bit for bit."""
    config = q2.Qwen2Config(hidden_size=896, intermediate_size=4864, num_layers=2, num_heads=14,
                            num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=4096,
                            tie_word_embeddings=True)
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=9, dtype=torch.bfloat16).items()}
    prompt = q2.make_prompt_ids(config, 4, 300, seed=3)
    small = Qwen2Engine(config, weights, batch=4, capacity=2048)
    small.split_tokens = 256  # several KV splits: the attention scratch is in use
    small.prefill(prompt)
    small.capture()
    eager = Qwen2Engine(config, weights, batch=4, capacity=2048)
    eager.split_tokens = 256
    eager.prefill(prompt)
    large = Qwen2Engine(config, weights, batch=64, capacity=4096)
    large.split_tokens = 256
    large.prefill(q2.make_prompt_ids(config, 64, 700, seed=4))
    junk = []
    for step in range(4):
        large.decode_step()  # grows the workspaces, then keeps writing into the new ones
        junk.append(torch.full((1 << 20,), float(step), device="cuda"))  # takes freed blocks, if any
        assert torch.equal(small.decode_step(), eager.decode_step())
        assert torch.equal(small.logits, eager.logits)
    small.state.check()


@pytest.mark.parametrize("chain_rows", ["128", "64"])
def test_65_to_128_sequences_on_either_decode_layer(chain_rows, monkeypatch):
    """100 sequences: the five-launch layer on 128-row tiles (two rows of squares or slices per
    idle-warp thread), and with B200_CHAIN_ROWS=64 the seven-launch layer of split-K partial
    producers and reduce consumers; both against the CPU oracle, teacher-forced."""
    monkeypatch.setenv("B200_CHAIN_ROWS", chain_rows)
    config = q2.Qwen2Config(hidden_size=896, intermediate_size=4864, num_layers=2, num_heads=14,
                            num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048,
                            tie_word_embeddings=True)
    weights = q2.make_weights(config, seed=6, dtype=torch.bfloat16)
    prompt = q2.make_prompt_ids(config, 100, 9, seed=8)
    ref_tokens, ref_logits, _ = qwen2_model.greedy_generate(config, weights, prompt, 2, capacity=16)
    engine = Qwen2Engine(config, {k: v.cuda() for k, v in weights.items()}, batch=100, capacity=16)
    assert engine.folded_norms == (chain_rows == "128")
    engine.prefill(prompt)
    assert_logits(engine.logits, ref_logits[0], 2e-2)
    engine.capture()
    assert engine.kernels_per_step == (2 * 5 + 5 if chain_rows == "128" else 2 * 7 + 6)
    for step in range(2):
        engine.input_ids.copy_(ref_tokens[:, step].cuda())
        engine.decode_step(feed_back=False)
        assert_logits(engine.logits, ref_logits[step + 1], 2e-2)
        assert_tokens(engine.next_ids, ref_tokens[:, step + 1], ref_logits[step + 1], 2e-2)
    engine.state.check()


def test_batch_above_the_chain_limit_uses_plain_and_cluster_split_k_projections():
    """130 sequences: beyond the 128 rows of the partial-sum chain, the decode step runs one
    projection per launch, with o / down as cluster split-K projections over two row tiles."""
    config = q2.Qwen2Config(hidden_size=896, intermediate_size=4864, num_layers=2, num_heads=14,
                            num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=1e6, vocab_size=2048,
                            tie_word_embeddings=True)
    weights = q2.make_weights(config, seed=6, dtype=torch.bfloat16)
    prompt = q2.make_prompt_ids(config, 130, 9, seed=8)
    ref_tokens, ref_logits, _ = qwen2_model.greedy_generate(config, weights, prompt, 2, capacity=16)
    engine = Qwen2Engine(config, {k: v.cuda() for k, v in weights.items()}, batch=130, capacity=16)
    engine.prefill(prompt)
    assert_logits(engine.logits, ref_logits[0], 2e-2)
    engine.capture()
    for step in range(2):
        engine.input_ids.copy_(ref_tokens[:, step].cuda())
        engine.decode_step(feed_back=False)
        assert_logits(engine.logits, ref_logits[step + 1], 2e-2)
        assert_tokens(engine.next_ids, ref_tokens[:, step + 1], ref_logits[step + 1], 2e-2)
    engine.state.check()
