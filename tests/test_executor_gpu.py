"""The KernelIR executor on the reference's own graphs: the reference-compiled KernelIR of
the 2-layer stateful Qwen2 (golden JSON), finished by lower_to_b200, run op by op on the
B200 kernels, against the logits / tokens / KV state the reference's CPU executor produced
for the same seeded weights and ids (qwen2_tiny_fp32.pt)."""

import json
from pathlib import Path

import pytest
import torch

from llm_compiler_b200 import kernel_ir as ir
from llm_compiler_b200 import kernels
from llm_compiler_b200 import qwen2 as q2
from llm_compiler_b200.executor import B200Executor, bind_arguments
from llm_compiler_b200.kv_state import ExecutionError, PreallocatedKVCacheState

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def lowered(kind, mode, tag="fp32", **options):
    name = f"kernel_ir_tiny_{kind}_{mode}.json" if tag == "fp32" else \
        f"kernel_ir_tiny_{tag}_{kind}_{mode}.json"
    module = ir.module_from_json(json.loads((GOLDEN / name).read_text()))
    ir.lower_to_b200(module, **options)
    return module


def causal_mask(batch, tokens):
    future = torch.triu(torch.ones(tokens, tokens, dtype=torch.bool), diagonal=1)
    return torch.zeros(batch, 1, tokens, tokens).masked_fill(future, float("-inf")).cuda()


@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
@pytest.mark.parametrize("fuse", [True, False])
def test_prefill_then_decode_graphs_match_the_reference_executor(mode, fuse, golden_tiny):
    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0).items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt = gold["batch"], gold["prompt"]
    executor = B200Executor(strict=True)

    prefill = lowered("prefill", mode, fuse_epilogues=fuse)
    ids = gold["input_ids"].cuda()
    positions = torch.arange(prompt).repeat(batch, 1).cuda()
    result = executor.run(prefill, bind_arguments(prefill.functions[0], weights, {
        "input_ids": ids, "attention_mask": causal_mask(batch, prompt), "position_ids": positions,
        "inv_freq": inv_freq}))
    logits, state = result.outputs
    assert isinstance(state, PreallocatedKVCacheState) and state.capacity == gold["capacity"]
    torch.testing.assert_close(logits.cpu(), gold["prefill_logits"], rtol=1e-4, atol=1e-4)
    assert all(name.startswith(("kernel.b200.", "runtime.")) for name in result.executed_operations)
    assert state.generation == config.num_layers  # one advance per layer slot
    pointers = [k.data_ptr() for k in state.keys]

    decode = lowered("decode", mode, fuse_epilogues=fuse)
    token = logits[:, -1].argmax(-1)
    assert torch.equal(token.cpu(), gold["tokens"][:, 0])
    for step in range(gold["steps"]):
        length = prompt + step
        arguments = bind_arguments(decode.functions[0], weights, {
            "input_ids": gold["tokens"][:, step].view(batch, 1).cuda(),
            "attention_mask": torch.zeros(batch, 1, 1, length + 1, device="cuda"),
            "position_ids": torch.full((batch, 1), length, device="cuda"),
            "kv_state": state, "inv_freq": inv_freq})
        logits, state = executor.run(decode, arguments).outputs
        torch.testing.assert_close(logits[:, 0].cpu(), gold["decode_logits"][step], rtol=1e-4,
                                   atol=1e-4)
        assert torch.equal(logits[:, 0].argmax(-1).cpu(), gold["tokens"][:, step + 1])
    state.check()
    used = prompt + gold["steps"]
    assert torch.equal(torch.stack(list(state.lengths), 0).cpu(), gold["lengths"])
    torch.testing.assert_close(torch.stack([k[:, :used] for k in state.keys], 0).cpu(), gold["keys"],
                               rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(torch.stack([v[:, :used] for v in state.values], 0).cpu(),
                               gold["values"], rtol=1e-4, atol=1e-5)
    assert pointers == [k.data_ptr() for k in state.keys]  # prefill -> decode on the same buffers
    assert state.generation == config.num_layers * (1 + gold["steps"])
    assert len([e for e in executor.lowering_trace if "rows" in e]) == 5 * (1 + gold["steps"])
    # the caller's mask was classified on the device once and proved causal
    masks = [e for e in executor.lowering_trace if e.get("op") == "prefill_attention.mask"]
    assert len(masks) == config.num_layers and all(e["causal"] and e["proof"] == "classified"
                                                   for e in masks)


@pytest.mark.parametrize("tag,mode", [("fp32", "fast"), ("fp32", "pytorch_compatible"), ("bf16", "fast")])
def test_last_token_logits_prefill_matches_the_last_row_of_the_reference(tag, mode, golden_tiny):
    """lower_to_b200(last_token_logits=True): the prefill returns B x 1 x V logits equal to the
    last position of the reference executor's full logits, and the same KV state as the full
    graph (the cut sits behind the last decoder layer)."""
    gold = golden_tiny[tag]
    config = q2.Qwen2Config(**gold["config"])
    dtype = torch.float32 if tag == "fp32" else torch.bfloat16
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0, dtype=dtype).items()}
    batch, prompt = gold["batch"], gold["prompt"]
    inputs = {"input_ids": gold["input_ids"].cuda(), "attention_mask": causal_mask(batch, prompt),
              "position_ids": torch.arange(prompt).repeat(batch, 1).cuda(),
              "inv_freq": q2.inverse_frequency(config, "cuda")}
    outputs = {}
    for cut in (False, True):
        module = lowered("prefill", mode, tag, last_token_logits=cut)
        result = B200Executor(strict=True).run(module, bind_arguments(module.functions[0], weights, inputs))
        outputs[cut] = result.outputs
        assert ("runtime.view.last_token" in result.executed_operations) == cut
    logits, state = outputs[True]
    assert logits.shape == (batch, 1, config.vocab_size)
    reference = gold["prefill_logits"][:, -1:]
    if tag == "fp32":
        torch.testing.assert_close(logits.cpu(), reference, rtol=1e-4, atol=1e-4)
    else:
        scale = float(reference.float().abs().max())
        assert float((logits.float().cpu() - reference.float()).abs().max()) <= max(5e-2 * scale, 2e-2)
    if tag == "fp32":
        assert torch.equal(logits[:, 0].argmax(-1).cpu(), gold["tokens"][:, 0])
    full_state = outputs[False][1]
    for layer in range(config.num_layers):
        assert torch.equal(state.keys[layer][:, :prompt], full_state.keys[layer][:, :prompt])
        assert torch.equal(state.values[layer][:, :prompt], full_state.values[layer][:, :prompt])
        assert torch.equal(state.lengths[layer], full_state.lengths[layer])


@pytest.mark.parametrize("tag", ["fp32", "bf16"])
def test_prefill_graph_runs_under_cuda_graph_capture(tag, golden_tiny):
    """A whole prefill (state creation included) captured once and replayed on new token ids:
    logits and KV equal to the eager run of the same module on those ids. The mask is declared
    causal (a mask left to the executor is not classified under capture and takes the
    additive-mask kernel: also captured below)."""
    gold = golden_tiny[tag]
    config = q2.Qwen2Config(**gold["config"])
    dtype = torch.float32 if tag == "fp32" else torch.bfloat16
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0, dtype=dtype).items()}
    batch, prompt = gold["batch"], gold["prompt"]
    ids = gold["input_ids"].cuda().clone()
    inputs = {"input_ids": ids, "attention_mask": causal_mask(batch, prompt),
              "position_ids": torch.arange(prompt).repeat(batch, 1).cuda(),
              "inv_freq": q2.inverse_frequency(config, "cuda")}
    other = (gold["input_ids"].cuda() * 7 + 3) % config.vocab_size
    for options in ({"causal_mask_arguments": ("attention_mask",), "last_token_logits": True}, {}):
        module = lowered("prefill", "fast", tag, **options)
        executor = B200Executor(strict=True)
        arguments = bind_arguments(module.functions[0], weights, inputs)
        ids.copy_(other)
        eager_logits, eager_state = executor.run(module, arguments).outputs  # also sizes the workspaces
        eager_logits = eager_logits.clone()
        ids.copy_(gold["input_ids"].cuda())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            logits, state = executor.run(module, arguments).outputs
        ids.copy_(other)
        graph.replay()
        assert torch.equal(logits, eager_logits)
        for layer in range(config.num_layers):
            assert torch.equal(state.keys[layer], eager_state.keys[layer])
            assert torch.equal(state.lengths[layer], eager_state.lengths[layer])
        kernels.runtime().check_status()


def test_decode_graph_runs_under_cuda_graph_capture(golden_tiny):
    """The interpreter itself is capture-safe: one decode step captured and replayed."""
    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0).items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt = gold["batch"], gold["prompt"]
    executor = B200Executor()
    prefill = lowered("prefill", "fast")
    logits, state = executor.run(prefill, bind_arguments(prefill.functions[0], weights, {
        "input_ids": gold["input_ids"].cuda(), "attention_mask": causal_mask(batch, prompt),
        "position_ids": torch.arange(prompt).repeat(batch, 1).cuda(), "inv_freq": inv_freq})).outputs
    decode = lowered("decode", "fast")
    ids = torch.zeros(batch, 1, dtype=torch.int64, device="cuda")
    positions = torch.full((batch, 1), prompt, device="cuda")
    mask = torch.zeros(batch, 1, 1, gold["capacity"], device="cuda")  # fixed-capacity zero mask
    arguments = bind_arguments(decode.functions[0], weights, {
        "input_ids": ids, "attention_mask": mask, "position_ids": positions, "kv_state": state,
        "inv_freq": inv_freq})
    saved = [l.clone() for l in state.lengths]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        executor.run(decode, arguments)  # warm-up: sizes every workspace
    torch.cuda.current_stream().wait_stream(side)
    for length, value in zip(state.lengths, saved):
        length.copy_(value)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_logits, _ = executor.run(decode, arguments).outputs
    for length, value in zip(state.lengths, saved):
        length.copy_(value)
    for step in range(gold["steps"]):
        ids.copy_(gold["tokens"][:, step].view(batch, 1))
        positions.fill_(prompt + step)
        graph.replay()
        torch.testing.assert_close(out_logits[:, 0].cpu(), gold["decode_logits"][step], rtol=1e-4,
                                   atol=1e-4)
    state.check()


def test_executor_errors_mirror_the_reference(golden_tiny):
    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0).items()}
    decode = lowered("decode", "fast")
    executor = B200Executor()
    with pytest.raises(ExecutionError, match="arguments"):
        executor.run(decode, [])
    cpu_inputs = {"input_ids": torch.zeros(3, 1, dtype=torch.int64), "attention_mask": torch.zeros(3, 1, 1, 6),
                  "position_ids": torch.zeros(3, 1, dtype=torch.int64), "kv_state": None,
                  "inv_freq": q2.inverse_frequency(config, "cuda")}
    with pytest.raises(ExecutionError, match="CUDA"):
        executor.run(decode, bind_arguments(decode.functions[0], weights, cpu_inputs))


def test_dispatch_plans_are_resolved_per_call_and_recorded(golden_tiny):
    """The graphs with profile-guided plans attached (select_dispatch_plans): every planned op
    resolves its plan with the run-time rows / tokens / context bound, the decision lands in
    lowering_trace, and the results are those of the reference executor whatever variant the
    synthetic profile makes it pick."""
    from llm_compiler_b200.dispatch_plan import DispatchCostModel

    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0).items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt = gold["batch"], gold["prompt"]
    layout = {"q_heads": config.num_heads, "kv_heads": config.num_kv_heads,
              "head_dim": config.head_dim, "dtype": "fp32"}
    rows = [{"op": "decode_attention", "batch": 2, **layout, "length": 8,
             "variants_us": {"split:0": 5.0, "split:32": 4.0}},
            {"op": "decode_attention", "batch": 64, **layout, "length": 8,
             "variants_us": {"split:0": 5.0, "split:64": 9.0}},
            {"op": "prefill_attention", **layout, "tokens": 4, "variants_us": {"tcgen05": 9.0, "mma.sync": 7.0}}]
    for n in (config.hidden_size, config.intermediate_size, config.vocab_size,
              config.num_kv_heads * config.head_dim):
        for k in (config.hidden_size, config.intermediate_size):
            rows.append({"op": "linear", "k": k, "n": n, "dtype": "fp32", "m": 8,
                         "variants_us": {"tcgen05": 3.0, "mma.sync": 2.0}})
    model = DispatchCostModel.from_dict(rows)
    executor = B200Executor(strict=True)
    prefill = lowered("prefill", "fast")
    assert ir.select_dispatch_plans(prefill, model)["planned_operations"] > 0
    result = executor.run(prefill, bind_arguments(prefill.functions[0], weights, {
        "input_ids": gold["input_ids"].cuda(), "attention_mask": causal_mask(batch, prompt),
        "position_ids": torch.arange(prompt).repeat(batch, 1).cuda(), "inv_freq": inv_freq}))
    logits, state = result.outputs
    torch.testing.assert_close(logits.cpu(), gold["prefill_logits"], rtol=1e-4, atol=1e-4)
    decode = lowered("decode", "fast")
    assert ir.select_dispatch_plans(decode, model)["planned_operations"] > 0
    logits, state = executor.run(decode, bind_arguments(decode.functions[0], weights, {
        "input_ids": gold["tokens"][:, 0].view(batch, 1).cuda(),
        "attention_mask": torch.zeros(batch, 1, 1, prompt + 1, device="cuda"),
        "position_ids": torch.full((batch, 1), prompt, device="cuda"),
        "kv_state": state, "inv_freq": inv_freq})).outputs
    torch.testing.assert_close(logits[:, 0].cpu(), gold["decode_logits"][0], rtol=1e-4, atol=1e-4)
    planned = [entry for entry in executor.lowering_trace if "variant" in entry]
    by_op = {}
    for entry in planned:
        by_op.setdefault(entry["op"], []).append(entry)
    assert set(by_op) == {"linear", "prefill_attention", "decode_attention"}
    assert all(e["source"] == "profile" and e["variant"] == "mma.sync" for e in by_op["linear"])
    assert all(e["variant"] == "mma.sync" and e["value"] == prompt for e in by_op["prefill_attention"])
    # batch 3 is nearer to the batch-2 plan than to the batch-64 one on a log scale
    assert all(e["variant"] == "split:32" and e["value"] == prompt + 1 for e in by_op["decode_attention"])
    state.check()


@pytest.mark.parametrize("mode", ["fast", "pytorch_compatible"])
@pytest.mark.parametrize("fuse", [True, False])
@pytest.mark.parametrize("tag", ["bf16", "fp16"])
def test_16_bit_graphs_match_the_reference_executor(mode, fuse, tag, golden_tiny):
    """The reference-compiled bf16 (fp16) KernelIR of the 2-layer model through the drop-in path
    (lower_to_b200 + B200Executor) against what the reference's CPU executor produced for the
    same weights (qwen2_tiny_bf16.pt, qwen2_tiny_fp16.pt): real casts, the 16-bit RoPE table
    inside a graph, the residual epilogues, packed projections and both numerical modes. bf16
    runs on the tensor-core kernels, fp16 on the generic ones."""
    gold = golden_tiny[tag]
    dtype, tolerance = (torch.bfloat16, 2e-2) if tag == "bf16" else (torch.float16, 1e-2)
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0, dtype=dtype).items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt = gold["batch"], gold["prompt"]
    executor = B200Executor(strict=True)
    options = dict(fuse_epilogues=fuse, fuse_graph=fuse)

    def check(actual, expected):
        scale = max(1.0, float(expected.float().abs().max()))
        assert float((actual.float().cpu() - expected.float()).abs().max()) <= tolerance * scale

    prefill = lowered("prefill", mode, tag, **options)
    result = executor.run(prefill, bind_arguments(prefill.functions[0], weights, {
        "input_ids": gold["input_ids"].cuda(), "attention_mask": causal_mask(batch, prompt),
        "position_ids": torch.arange(prompt).repeat(batch, 1).cuda(), "inv_freq": inv_freq}))
    logits, state = result.outputs
    assert logits.dtype == dtype
    check(logits, gold["prefill_logits"])
    decode = lowered("decode", mode, tag, **options)
    for step in range(gold["steps"]):
        length = prompt + step
        logits, state = executor.run(decode, bind_arguments(decode.functions[0], weights, {
            "input_ids": gold["tokens"][:, step].view(batch, 1).cuda(),
            "attention_mask": torch.zeros(batch, 1, 1, length + 1, device="cuda"),
            "position_ids": torch.full((batch, 1), length, device="cuda"),
            "kv_state": state, "inv_freq": inv_freq})).outputs
        check(logits[:, 0], gold["decode_logits"][step])
        reference = gold["decode_logits"][step].float()
        picked = logits[:, 0].float().argmax(-1).cpu()
        for row in range(batch):
            if int(picked[row]) != int(gold["tokens"][row, step + 1]):
                top2 = reference[row].topk(2).values
                assert float(top2[0] - top2[1]) <= 2e-2
    state.check()
    used = prompt + gold["steps"]
    assert torch.equal(torch.stack(list(state.lengths), 0).cpu(), gold["lengths"])
    check(torch.stack([k[:, :used] for k in state.keys], 0), gold["keys"])
    check(torch.stack([v[:, :used] for v in state.values], 0), gold["values"])


def test_declared_and_classified_causal_masks_and_a_mask_that_is_not_causal(golden_tiny):
    """A caller-declared causal mask is never read (a NaN mask proves it); an undeclared one is
    classified on the device; a mask with one hole stays on the additive-mask kernel and gives
    the reference's answer for that mask."""
    from oracle import qwen2_model

    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    cpu_weights = q2.make_weights(config, seed=0)
    weights = {k: v.cuda() for k, v in cpu_weights.items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt = gold["batch"], gold["prompt"]
    inputs = {"input_ids": gold["input_ids"].cuda(),
              "position_ids": torch.arange(prompt).repeat(batch, 1).cuda(), "inv_freq": inv_freq}
    declared = lowered("prefill", "fast", causal_mask_arguments=("attention_mask",))
    executor = B200Executor()
    poisoned = torch.full((batch, 1, prompt, prompt), float("nan"), device="cuda")
    logits, _ = executor.run(declared, bind_arguments(declared.functions[0], weights, {
        **inputs, "attention_mask": poisoned})).outputs
    torch.testing.assert_close(logits.cpu(), gold["prefill_logits"], rtol=1e-4, atol=1e-4)
    assert all(e["proof"] == "declared:%attention_mask" for e in executor.lowering_trace
               if e.get("op") == "prefill_attention.mask")

    plain = lowered("prefill", "fast")
    holed = causal_mask(batch, prompt)
    holed[1, 0, 3, 1] = float("-inf")  # sequence 1: token 3 may not see token 1
    executor = B200Executor()
    logits, _ = executor.run(plain, bind_arguments(plain.functions[0], weights, {
        **inputs, "attention_mask": holed})).outputs
    assert not any(e["causal"] for e in executor.lowering_trace if e.get("op") == "prefill_attention.mask")
    expected, _ = qwen2_model.prefill(config, cpu_weights, gold["input_ids"], capacity=gold["capacity"],
                                      attention_mask=holed.cpu())
    torch.testing.assert_close(logits.cpu(), expected, rtol=1e-4, atol=1e-4)
    assert float((expected - gold["prefill_logits"]).abs().max()) > 1e-4  # the hole matters
    never = B200Executor(classify_masks=False)
    never.run(plain, bind_arguments(plain.functions[0], weights, {
        **inputs, "attention_mask": causal_mask(batch, prompt)}))
    assert not any(e["causal"] for e in never.lowering_trace if e.get("op") == "prefill_attention.mask")


def test_symbolic_dimensions_are_bound_and_guarded_at_run_time(golden_tiny):
    """The reference executor binds every symbolic dimension of the signature to its run-time
    extent and enforces the exporter's ranges (execution.py:1323-1347); so does this one."""
    gold = golden_tiny["fp32"]
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0).items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt = gold["batch"], gold["prompt"]
    prefill = lowered("prefill", "fast")
    executor = B200Executor()

    def arguments(batch, tokens, position_batch=None):
        return bind_arguments(prefill.functions[0], weights, {
            "input_ids": torch.zeros(batch, tokens, dtype=torch.int64, device="cuda"),
            "attention_mask": causal_mask(batch, tokens),
            "position_ids": torch.arange(tokens).repeat(position_batch or batch, 1).cuda(),
            "inv_freq": inv_freq})

    result = executor.run(prefill, arguments(batch, prompt))
    assert sorted(result.symbolic_dimensions.values()) == sorted([batch, prompt])
    with pytest.raises(ExecutionError, match="above the exporter's upper bound"):
        executor.run(prefill, arguments(9, prompt))  # exported with max_batch = 8
    with pytest.raises(ExecutionError, match="breaks the equality"):
        executor.run(prefill, arguments(batch, prompt, position_batch=batch - 1))


@pytest.mark.parametrize("chain_rows", [64, 0])
def test_bf16_decode_chain_through_the_executor(chain_rows, golden_tiny):
    """The reference-compiled bf16 decode graph with the decode chain fused (the caller declares
    the decode mask all zero): per layer the fused q|k|v attention op, the cluster split-K o and
    down projections and the folded-norm gate|up, one length update for all slots at the end.
    chain_rows = 0 makes the executor run the same fused ops as their unfused kernels (what it
    does beyond 64 rows). Both against the reference executor's logits, lengths and KV."""
    gold = golden_tiny["bf16"]
    config = q2.Qwen2Config(**gold["config"])
    weights = {k: v.cuda() for k, v in q2.make_weights(config, seed=0, dtype=torch.bfloat16).items()}
    inv_freq = q2.inverse_frequency(config, "cuda")
    batch, prompt = gold["batch"], gold["prompt"]
    executor = B200Executor(strict=True)
    executor.CHAIN_ROWS = chain_rows
    prefill = lowered("prefill", "fast", "bf16")
    logits, state = executor.run(prefill, bind_arguments(prefill.functions[0], weights, {
        "input_ids": gold["input_ids"].cuda(), "attention_mask": causal_mask(batch, prompt),
        "position_ids": torch.arange(prompt).repeat(batch, 1).cuda(), "inv_freq": inv_freq})).outputs
    decode = lowered("decode", "fast", "bf16", zero_mask_arguments=("attention_mask",))
    names = [op.name for op in decode.functions[0].block.operations]
    assert names.count("kernel.b200.qkv_decode_attention") == config.num_layers
    assert names.count("runtime.kv.advance_all") == 1 and "runtime.kv.advance" not in names
    generation = state.generation
    for step in range(gold["steps"]):
        length = prompt + step
        logits, state = executor.run(decode, bind_arguments(decode.functions[0], weights, {
            "input_ids": gold["tokens"][:, step].view(batch, 1).cuda(),
            "attention_mask": torch.zeros(batch, 1, 1, gold["capacity"], device="cuda"),
            "position_ids": torch.full((batch, 1), length, device="cuda"),
            "kv_state": state, "inv_freq": inv_freq})).outputs
        expected = gold["decode_logits"][step].float()
        scale = max(1.0, float(expected.abs().max()))
        assert float((logits[:, 0].float().cpu() - expected).abs().max()) <= 2e-2 * scale
    state.check()
    assert state.generation == generation + config.num_layers * gold["steps"]
    used = prompt + gold["steps"]
    assert torch.equal(torch.stack(list(state.lengths), 0).cpu(), gold["lengths"])
    keys = torch.stack([k[:, :used] for k in state.keys], 0).float().cpu()
    assert float((keys - gold["keys"].float()).abs().max()) <= 2e-2 * max(1.0, float(gold["keys"].abs().max()))
    fused = [e for e in executor.lowering_trace if e.get("op") == "qkv_decode_attention"]
    assert fused and all(e["fused"] == (chain_rows > 0) and e["length_offset"] == 1 for e in fused)
