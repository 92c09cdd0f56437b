"""The B200 lowering pass and coverage check on the reference's own KernelIR (golden JSON
written by tests/golden/make_golden.py) — host logic only, no GPU."""

import copy
import json
import os
import sys
from collections import Counter
from pathlib import Path

import pytest

from llm_compiler_b200 import fusion
from llm_compiler_b200 import kernel_ir as ir

GOLDEN = Path(__file__).resolve().parent / "golden"
KINDS = ["prefill", "decode"]
MODES = ["fast", "pytorch_compatible"]


def load(kind, mode):
    return ir.module_from_json(json.loads((GOLDEN / f"kernel_ir_tiny_{kind}_{mode}.json").read_text()))


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("mode", MODES)
def test_reference_kernel_ir_is_not_fully_lowered_but_b200_is(kind, mode):
    module = load(kind, mode)
    ir.verify_module(module)
    before = ir.analyze_lowering_coverage(module)
    # only the runtime.kv.* bookkeeping names are shared with the reference's dialect
    assert set(before.lowered_by_name) <= {"runtime.kv.init", "runtime.kv.length", "runtime.kv.advance"}
    assert before.unlowered_operations >= before.total_operations - 4
    with pytest.raises(ir.LoweringCoverageError):
        ir.require_full_lowering(module)
    report = ir.lower_to_b200(module)
    ir.verify_module(module)
    coverage = ir.require_full_lowering(module)
    assert coverage.is_complete and coverage.coverage == 1.0
    assert report.coverage == coverage
    names = Counter(op.name for op in module.functions[0].block.operations)
    assert not any(name.startswith(("aten.", "serve.", "kernel.triton.", "kernel.cuda.",
                                    "kernel.cublas.")) for name in names)
    # 2 layers: 5 RMSNorm, 1 RoPE table, 1 embedding; per layer ONE q|k|v projection over
    # packed weights (+ packed biases), o, ONE gate|up projection with the SwiGLU epilogue and
    # down; the LM head
    assert names["kernel.b200.rms_norm"] == 5
    assert names["kernel.b200.linear"] == 9
    assert names["kernel.b200.pack_rows"] == 4 and names["kernel.b200.interleave_rows"] == 2
    assert names["runtime.view.slice"] == 6
    assert names["kernel.b200.rope_table"] == 1
    assert names["kernel.b200.swiglu"] == 0
    assert names["kernel.b200.embedding"] == 1
    assert names["kernel.b200.add"] == 0  # all four residual adds became GEMM epilogues
    assert names.get("kernel.b200.cast", 0) == 0  # fp32 graph: every cast was an identity
    if kind == "decode":
        # rope + kv.length + kv_store of the new token: one launch per layer
        assert names["kernel.b200.rope_kv_store"] == 2 and names["kernel.b200.rope"] == 0
        assert names["kernel.b200.decode_attention"] == 2 and names["kernel.b200.kv_store"] == 0
        assert names["runtime.kv.length"] == 0 and names["runtime.kv.advance"] == 2
    else:
        assert names["kernel.b200.rope"] == 2
        assert names["kernel.b200.prefill_attention"] == 2
        assert names["kernel.b200.kv_prefill_store"] == 2 and names["runtime.kv.init"] == 1
    assert report.removed_casts + report.removed_dead >= 10


@pytest.mark.parametrize("kind", KINDS)
def test_without_graph_fusion_every_projection_stays_its_own_kernel(kind):
    module = load(kind, "fast")
    ir.lower_to_b200(module, fuse_graph=False)
    ir.verify_module(module)
    ir.require_full_lowering(module)
    names = Counter(op.name for op in module.functions[0].block.operations)
    assert names["kernel.b200.linear"] == 15 and names["kernel.b200.swiglu"] == 2
    assert names["kernel.b200.rope"] == 2 and names["kernel.b200.pack_rows"] == 0
    if kind == "decode":
        assert names["kernel.b200.kv_store"] == 2 and names["runtime.kv.length"] == 2


def load_gz(name):
    import gzip

    return ir.module_from_json(json.loads(gzip.open(GOLDEN / name).read()))


@pytest.mark.parametrize("kind,total", [("prefill", 738), ("decode", 760)])
def test_qwen2_0_5b_graphs_lower_fully(kind, total):
    """The reference's KernelIR of the real 24-layer architecture (bf16, vocabulary 151936): the
    graphs on which upstream reports 39 - 44 % coverage (docs/qwen2-0.5b-validation.md:96-118)
    and on which `--require-full-lowering` fails. Here every op gets a kernel or a host op."""
    module = load_gz(f"kernel_ir_qwen2_0_5b_{kind}_fast.json.gz")
    before = ir.analyze_lowering_coverage(module)
    assert before.total_operations == total
    assert before.coverage < 0.5
    options = dict(causal_mask_arguments=("attention_mask",), fuse_decode_chain=False)
    report = ir.lower_to_b200(module, **options)
    ir.verify_module(module)
    coverage = ir.require_full_lowering(module)
    assert coverage.is_complete
    names = Counter(op.name for op in module.functions[0].block.operations)
    layers = 24
    assert names["kernel.b200.linear"] == 4 * layers + 1
    assert names["kernel.b200.rms_norm"] == 2 * layers + 1
    assert names["kernel.b200.pack_rows"] == 2 * layers
    assert names["kernel.b200.interleave_rows"] == layers
    assert names["kernel.b200.embedding"] == 1 and names["kernel.b200.rope_table"] == 1
    assert names["kernel.b200.add"] == 0 and names["kernel.b200.swiglu"] == 0
    assert names.get("kernel.b200.cast", 0) == 0  # the only real casts are inside the RoPE table
    launches = sum(count for name, count in names.items() if name.startswith("kernel.b200.")) \
        - names["kernel.b200.pack_rows"] - names["kernel.b200.interleave_rows"]
    if kind == "decode":
        assert names["kernel.b200.rope_kv_store"] == layers
        assert names["kernel.b200.decode_attention"] == layers
        assert names["runtime.kv.advance"] == layers
        assert launches == 8 * layers + 4  # + embedding, rope table, final norm, LM head
        # with the decode chain and a caller-declared all-zero decode mask: five launches a layer
        chained = load_gz(f"kernel_ir_qwen2_0_5b_{kind}_fast.json.gz")
        chain_report = ir.lower_to_b200(chained, zero_mask_arguments=("attention_mask",))
        ir.verify_module(chained)
        ir.require_full_lowering(chained)
        chain = Counter(op.name for op in chained.functions[0].block.operations)
        assert chain["kernel.b200.qkv_decode_attention"] == layers  # partial GEMM + attention
        assert chain["kernel.b200.norm_linear"] == layers + 1        # gate|up and the LM head with their folded norms
        assert chain["kernel.b200.linear"] == 2 * layers             # o, down (+ residual)
        assert chain["kernel.b200.rms_norm"] == 0
        assert chain["runtime.kv.advance_all"] == 1 and chain["runtime.kv.advance"] == 0
        assert chain["kernel.b200.scale_columns"] == 2 * layers + 1  # (the tied LM head gets a folded copy)
        assert chain_report.lowered_rules["qkv+attention"] == layers
        fused = [op for op in chained.functions[0].block.operations
                 if op.name == "kernel.b200.qkv_decode_attention"]
        assert all(op.attributes["length_offset"] == 1 for op in fused)
        assert sorted(op.attributes["slot"] for op in fused) == list(range(layers))
        # without the declaration the mask is honoured: attention stays its own op
        kept = load_gz(f"kernel_ir_qwen2_0_5b_{kind}_fast.json.gz")
        ir.lower_to_b200(kept)
        kept_names = Counter(op.name for op in kept.functions[0].block.operations)
        assert kept_names["kernel.b200.qkv_decode_attention"] == 0
        assert kept_names["kernel.b200.decode_attention"] == layers
        assert kept_names["kernel.b200.norm_linear"] == 2 * layers + 1
    else:
        assert names["kernel.b200.prefill_attention"] == layers
        assert report.lowered_rules["causal_mask"] == layers
        assert all(op.attributes["causal"] is True and
                   op.attributes["causal_proof"] == "declared:%attention_mask"
                   for op in module.functions[0].block.operations
                   if op.name == "kernel.b200.prefill_attention")
    snapshot = json.dumps(ir.module_to_json(module), sort_keys=True)
    ir.lower_to_b200(module, **options)
    assert json.dumps(ir.module_to_json(module), sort_keys=True) == snapshot  # idempotent


@pytest.mark.parametrize("kind", KINDS)
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("tag", ["bf16", "fp16"])
def test_16_bit_tiny_graphs_lower_fully(kind, mode, tag):
    module = ir.module_from_json(json.loads(
        (GOLDEN / f"kernel_ir_tiny_{tag}_{kind}_{mode}.json").read_text()))
    ir.lower_to_b200(module)
    ir.verify_module(module)
    ir.require_full_lowering(module)
    names = Counter(op.name for op in module.functions[0].block.operations)
    assert names.get("kernel.b200.cast", 0) == 0 and names["kernel.b200.rope_table"] == 1
    for op in module.functions[0].block.operations:
        if op.name in ("kernel.b200.rms_norm", "kernel.b200.linear", "kernel.b200.norm_linear"):
            assert op.attributes["numerical_mode"] == mode
    # the RMSNorm is folded into the projection behind it in the fast mode of bf16 only (fp16
    # runs on the generic kernels, which have no folded form)
    assert (names["kernel.b200.norm_linear"] > 0) == (mode == "fast" and tag == "bf16")


@pytest.mark.parametrize("source", ["tiny_fp32", "tiny_bf16", "qwen2_0_5b"])
def test_last_token_logits_cut_the_prefill_in_front_of_the_final_norm(source):
    """lower_to_b200(last_token_logits=True): the hidden rows are cut to the last position in
    front of the final norm + LM head (a view op), the first result becomes B x 1 x V, every
    other op keeps its type; decode graphs (one token already) and a second application change
    nothing."""
    def fresh(kind):
        if source == "qwen2_0_5b":
            return load_gz(f"kernel_ir_qwen2_0_5b_{kind}_fast.json.gz")
        if source == "tiny_bf16":
            return ir.module_from_json(json.loads((GOLDEN / f"kernel_ir_tiny_bf16_{kind}_fast.json").read_text()))
        return load(kind, "fast")

    full, cut = fresh("prefill"), fresh("prefill")
    ir.lower_to_b200(full)
    report = ir.lower_to_b200(cut, last_token_logits=True)
    assert report.lowered_rules["last_token_logits"] == 1
    ir.verify_module(cut)
    ir.require_full_lowering(cut)
    names = Counter(op.name for op in cut.functions[0].block.operations)
    assert names["runtime.view.last_token"] == 1
    assert len(cut.functions[0].block.operations) == len(full.functions[0].block.operations) + 1
    dims = lambda value: fusion._split_dims(fusion._DIMS.match(str(value.type)).group(1))
    before, after = dims(full.functions[0].returns[0]), dims(cut.functions[0].returns[0])
    assert after[1] == "1" and after[0] == before[0] and after[2] == before[2] and before[1] != "1"
    view = next(op for op in cut.functions[0].block.operations if op.name == "runtime.view.last_token")
    consumer = next(op for op in cut.functions[0].block.operations
                    if any(operand is view.results[0] for operand in op.operands))
    assert consumer.name in ("kernel.b200.rms_norm", "kernel.b200.norm_linear")
    again = ir.lower_to_b200(cut, last_token_logits=True)
    assert "last_token_logits" not in again.lowered_rules
    decode = fresh("decode")
    assert "last_token_logits" not in ir.lower_to_b200(decode, last_token_logits=True).lowered_rules


def test_only_declared_masks_are_marked_causal():
    module = load("prefill", "fast")
    report = ir.lower_to_b200(module)
    assert "causal_mask" not in report.lowered_rules
    assert all(op.attributes.get("causal") == "mask" for op in module.functions[0].block.operations
               if op.name == "kernel.b200.prefill_attention")
    report = ir.lower_to_b200(module, causal_mask_arguments=("position_ids",))  # not the mask
    assert "causal_mask" not in report.lowered_rules


@pytest.mark.parametrize("mode", MODES)
def test_numerical_mode_is_carried_onto_every_kernel(mode):
    module = load("decode", mode)
    ir.lower_to_b200(module)
    for op in module.functions[0].block.operations:
        if op.name in ("kernel.b200.rms_norm", "kernel.b200.rope", "kernel.b200.decode_attention",
                       "kernel.b200.linear"):
            assert op.attributes["numerical_mode"] == mode, op.name
    forced = load("decode", mode)
    ir.lower_to_b200(forced, numerical_mode="pytorch_compatible")
    assert all(op.attributes["numerical_mode"] == "pytorch_compatible"
               for op in forced.functions[0].block.operations if op.name == "kernel.b200.rms_norm")
    with pytest.raises(ValueError):
        ir.lower_to_b200(load("decode", mode), numerical_mode="exact")


def test_lowering_is_idempotent_and_keeps_unknown_ops_unlowered():
    module = load("decode", "fast")
    ir.lower_to_b200(module)
    snapshot = json.dumps(ir.module_to_json(module), sort_keys=True)
    ir.lower_to_b200(module)
    assert json.dumps(ir.module_to_json(module), sort_keys=True) == snapshot
    # an op of an unknown dialect is never claimed (tests/test_lowering.py:97-114 upstream)
    function = module.functions[0]
    odd = ir.Operation("kernel.vendor.magic", [function.block.arguments[0]],
                       [ir.Value("%odd", "tensor<1xf32, cpu>")])
    function.block.operations.insert(0, odd)
    function.returns.append(odd.results[0])
    ir.lower_to_b200(module)
    coverage = ir.analyze_lowering_coverage(module)
    assert coverage.unlowered_by_name == {"kernel.vendor.magic": 1}
    with pytest.raises(ir.LoweringCoverageError, match="kernel.vendor.magic"):
        ir.require_full_lowering(module)


def test_without_epilogue_fusion_the_adds_stay_separate_kernels():
    module = load("prefill", "fast")
    ir.lower_to_b200(module, fuse_epilogues=False)
    names = Counter(op.name for op in module.functions[0].block.operations)
    assert names["kernel.b200.add"] == 4
    ir.require_full_lowering(module)


def test_json_round_trip_preserves_the_graph():
    module = load("prefill", "fast")
    again = ir.module_from_json(json.dumps(ir.module_to_json(module)))
    assert ir.module_to_json(again) == ir.module_to_json(module)


def test_strict_executor_refuses_before_running_anything():
    from llm_compiler_b200.executor import B200Executor

    module = load("decode", "fast")  # still the reference's partial lowering
    with pytest.raises(ir.LoweringCoverageError):
        B200Executor(strict=True).run(module, [])


# the reference's src directory, where a checkout of it is present (see tests/golden/make_golden.py)
# (LLM_COMPILER_REFERENCE_SRC, or a "reference" checkout beside this repository)
REFERENCE_SRC = Path(os.environ.get("LLM_COMPILER_REFERENCE_SRC") or
                     Path(__file__).resolve().parents[2] / "reference" / "src") / "stateful_llm_compiler"


@pytest.mark.skipif(not REFERENCE_SRC.is_dir(), reason="reference package not present")
def test_pass_accepts_the_reference_module_objects():
    """Where the reference is installed its own Module objects go straight into the pass."""

    sys.path.insert(0, str(REFERENCE_SRC.parent))
    try:
        import torch
        from stateful_llm_compiler.compiler import CompileOptions, compile_exported_program
        from stateful_llm_compiler.frontend import export_qwen2_causal_lm_prefill
        from stateful_llm_compiler.lowering import LoweringCoverageError as UpstreamError
        from stateful_llm_compiler.qwen2 import (Qwen2CompatConfig, StatefulQwen2ForCausalLM,
                                                 make_qwen2_prefill_inputs)

        cfg = Qwen2CompatConfig(hidden_size=128, intermediate_size=256, num_layers=1, num_heads=2,
                                num_kv_heads=1, vocab_size=64, tie_word_embeddings=True)
        model = StatefulQwen2ForCausalLM(cfg).bfloat16().eval()
        inputs = make_qwen2_prefill_inputs(cfg, 2, 4, seed=0)
        program = export_qwen2_causal_lm_prefill(model, inputs, max_batch=4, max_prompt_length=16)
        with pytest.raises(UpstreamError):  # upstream cannot satisfy --require-full-lowering
            compile_exported_program(program, options=CompileOptions(
                prefill_kv_state=True, kv_capacity=32, require_full_lowering=True))
        artifact = compile_exported_program(program, options=CompileOptions(
            prefill_kv_state=True, kv_capacity=32, numerical_mode="pytorch_compatible"))
        report = ir.lower_to_b200(artifact.module)
        ir.require_full_lowering(artifact.module)
        names = Counter(op.name for op in artifact.module.functions[0].block.operations)
        assert names["kernel.b200.rope_table"] == 1 and names["kernel.b200.swiglu"] == 0
        assert names["kernel.b200.interleave_rows"] == 1 and names["kernel.b200.pack_rows"] == 2
        assert names.get("kernel.b200.cast", 0) == 0  # bf16: the only real casts are in the table
        assert report.coverage.is_complete
    finally:
        sys.path.remove(str(REFERENCE_SRC.parent))
