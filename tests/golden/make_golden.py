"""Generates the golden fixtures in this directory by RUNNING THE REFERENCE ITSELF.

    python tests/golden/make_golden.py [/path/to/reference/src]

Needs the reference package (stateful_llm_compiler) importable -- by default from
/root/reference/src -- and is therefore only run where the reference is mounted; the
fixtures it writes are committed and are what travels to machines without the reference.

Fixtures
  ops.pt              per-operator cases (inputs + outputs) produced by the reference's CPU
                      executor methods (ReferenceExecutor._serve_*, PreallocatedKVCacheState.*,
                      native_kv_store, Qwen2RotaryEmbedding); shapes and seeds follow the
                      reference's own GPU tests (tests/test_triton_backend.py:380-466,
                      tests/test_prefill_attention.py:33-253, tests/test_rope.py:228-290,
                      tests/test_linear.py:123-163).
  qwen2_tiny_fp32.pt  the 2-layer fp32 stateful decode: export -> import -> passes ->
  qwen2_tiny_bf16.pt  ReferenceExecutor on the ServeIR (prefill of 3 x 5 ids into a capacity-64
                      state, then 4 greedy decode steps); ids, logits, tokens, lengths and KV
                      buffers. Weights are NOT stored: they are N(0, 0.02) from seed 0 in
                      parameter order and the script asserts that llm_compiler_b200.qwen2
                      .make_weights regenerates them bit for bit.
  kernel_ir_tiny_*.json  the reference's KernelIR for those two graphs (op names, operands,
                      attributes, types), for the executor's structural tests.
"""

from __future__ import annotations

import json
import sys
from pathlib import Path

import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
REFERENCE_SRC = sys.argv[1] if len(sys.argv) > 1 else "/root/reference/src"
sys.path.insert(0, REFERENCE_SRC)
sys.path.insert(0, str(REPO))

from stateful_llm_compiler.compiler import CompileOptions, compile_exported_program  # noqa: E402
from stateful_llm_compiler.execution import (  # noqa: E402
    PreallocatedKVCacheState,
    ReferenceExecutor,
    bind_exported_program_arguments,
    bind_stateful_decode_arguments,
    native_kv_store,
)
from stateful_llm_compiler.frontend import (  # noqa: E402
    export_qwen2_causal_lm_decode,
    export_qwen2_causal_lm_prefill,
)
from stateful_llm_compiler.importer import import_exported_program  # noqa: E402
from stateful_llm_compiler.optimizer import default_pass_manager  # noqa: E402
from stateful_llm_compiler.qwen2 import (  # noqa: E402
    Qwen2CompatConfig,
    Qwen2RotaryEmbedding,
    StatefulQwen2ForCausalLM,
    make_qwen2_prefill_inputs,
)

import llm_compiler_b200.qwen2 as mine  # noqa: E402

sys.path.insert(0, str(HERE))
import cases  # noqa: E402


# ----------------------------------------------------------------- per-op cases ----
def op_cases():
    """Reference OUTPUTS for the seeded inputs of tests/golden/cases.py."""

    out = {}
    for name in cases.KV_STORE:
        x = cases.kv_store_inputs(name)
        kout, vout = x["key_buffer"].clone(), x["value_buffer"].clone()
        native_kv_store(kout, vout, x["key"], x["value"], x["positions"])
        out[name] = dict(key_out=kout, value_out=vout)
    for name in cases.ROPE:
        x = cases.rope_inputs(name)
        cfg = Qwen2CompatConfig(hidden_size=x["q_heads"] * x["head_dim"], num_heads=x["q_heads"],
                                num_kv_heads=x["kv_heads"], rope_theta=x["theta"])
        cos, sin = Qwen2RotaryEmbedding(cfg)(x["query"], x["position_ids"])
        qo, ko = ReferenceExecutor._serve_rope([x["query"], x["key"], cos, sin],
                                               {"head_dim": x["head_dim"]})
        out[name] = dict(cosine=cos, sine=sin, query_out=qo, key_out=ko)
    for name in cases.RMS_NORM:
        x = cases.rms_norm_inputs(name)
        attrs = {"epsilon": x["epsilon"], "round_before_weight": x["round_before_weight"]}
        out[name] = dict(output=ReferenceExecutor._serve_rms_norm([x["input"], x["weight"]], attrs))
    for name in cases.DECODE_ATTENTION:
        x = cases.decode_attention_inputs(name)
        capacity = x["key_buffer"].shape[1]
        state = PreallocatedKVCacheState((x["key_buffer"],), (x["value_buffer"],),
                                         (x["lengths"],), capacity)
        out[name] = dict(output=state.decode_attention(0, x["query"], x["mask"],
                                                       groups=x["groups"], scale=x["scale"]))
    for name in cases.PREFILL_ATTENTION:
        x = cases.prefill_attention_inputs(name)
        attrs = {"groups": x["groups"], "scale": x["scale"], "causal": "mask"}
        out[name] = dict(output=ReferenceExecutor._serve_prefill_attention(
            [x["query"], x["key"], x["value"], x["mask"]], attrs))
    for name in cases.LINEAR:
        x = cases.linear_inputs(name)
        operands = [x["input"], x["weight"]] + ([x["bias"]] if x["bias"] is not None else [])
        out[name] = dict(output=ReferenceExecutor._serve_linear(
            operands, {"has_bias": x["bias"] is not None}))
    for name in cases.ROPE_TABLE:
        x = cases.rope_table_inputs(name)
        cfg = Qwen2CompatConfig(hidden_size=4 * x["head_dim"], num_heads=4, num_kv_heads=2,
                                rope_theta=x["theta"])
        cos, sin = Qwen2RotaryEmbedding(cfg)(torch.zeros(1, dtype=x["dtype"]), x["position_ids"])
        out[name] = dict(cosine=cos, sine=sin)
    return out


# ------------------------------------------------------------ whole-model cases ----
def module_to_json(module):
    def type_str(t):
        return str(t)

    functions = []
    for function in module.functions:
        functions.append({
            "name": function.name,
            "arguments": [{"name": a.name, "type": type_str(a.type)} for a in function.block.arguments],
            "operations": [{
                "name": op.name,
                "operands": [v.name for v in op.operands],
                "results": [{"name": r.name, "type": type_str(r.type)} for r in op.results],
                "attributes": op.attributes,
            } for op in function.block.operations],
            "returns": [v.name for v in function.returns],
        })
    return {"functions": functions}


def tiny_model_case(dtype, tag):
    cfg = Qwen2CompatConfig(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4,
                            num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=10000.0,
                            vocab_size=1024, tie_word_embeddings=True)
    model = StatefulQwen2ForCausalLM(cfg)
    torch.manual_seed(0)
    with torch.no_grad():
        for parameter in model.parameters():
            parameter.normal_(0.0, 0.02)
    model = model.to(dtype).eval()
    regenerated = mine.make_weights(mine.TINY_FP32, seed=0, dtype=dtype)
    for name, tensor in model.state_dict().items():
        assert torch.equal(tensor, regenerated[name]), f"weight regeneration mismatch: {name}"

    batch, prompt, capacity, steps = 3, 5, 64, 4
    ids, mask, pos = make_qwen2_prefill_inputs(cfg, batch, prompt, seed=0)
    assert torch.equal(ids, mine.make_prompt_ids(mine.TINY_FP32, batch, prompt, seed=0))

    program = export_qwen2_causal_lm_prefill(model, (ids, mask, pos), max_batch=8,
                                             max_prompt_length=32)
    module = import_exported_program(program)
    default_pass_manager(prefill_kv_state=True, kv_capacity=capacity).run(module)
    result = ReferenceExecutor().run(module, bind_exported_program_arguments(program, (ids, mask, pos)))
    prefill_logits, state = result.outputs

    past = tuple((torch.zeros(batch, 2, prompt, 64, dtype=dtype),
                  torch.zeros(batch, 2, prompt, 64, dtype=dtype)) for _ in range(2))
    decode_program = export_qwen2_causal_lm_decode(
        model, (ids[:, :1], torch.zeros(batch, 1, 1, prompt + 1), pos[:, :1], past),
        max_batch=8, max_cache_length=capacity - 1)
    decode_module = import_exported_program(decode_program)
    default_pass_manager(preallocate_kv=True, kv_capacity=capacity).run(decode_module)

    tokens = [prefill_logits[:, -1].argmax(dim=-1)]
    step_logits = []
    for step in range(steps):
        length = prompt + step
        args = bind_stateful_decode_arguments(
            decode_program, tokens[-1].view(batch, 1), torch.zeros(batch, 1, 1, length + 1), state,
            extra_user_inputs={"position_ids": torch.full((batch, 1), length, dtype=torch.int64)},
            primary_input_name="input_ids")
        logits, state = ReferenceExecutor().run(decode_module, args).outputs
        step_logits.append(logits[:, 0].clone())
        tokens.append(logits[:, 0].argmax(dim=-1))

    fixture = dict(
        config=dict(hidden_size=256, intermediate_size=512, num_layers=2, num_heads=4,
                    num_kv_heads=2, rms_norm_eps=1e-6, rope_theta=10000.0, vocab_size=1024,
                    tie_word_embeddings=True),
        dtype=str(dtype), seed=0, batch=batch, prompt=prompt, capacity=capacity, steps=steps,
        input_ids=ids, prefill_logits=prefill_logits, decode_logits=torch.stack(step_logits, 0),
        tokens=torch.stack(tokens, 1), lengths=torch.stack(list(state.lengths), 0),
        keys=torch.stack([k[:, :prompt + steps] for k in state.keys], 0),
        values=torch.stack([v[:, :prompt + steps] for v in state.values], 0))
    torch.save(fixture, HERE / f"qwen2_tiny_{tag}.pt")

    if tag == "fp32":
        for kind, prog, opts in (
            ("prefill", program, CompileOptions(prefill_kv_state=True, kv_capacity=capacity)),
            ("decode", decode_program, CompileOptions(preallocate_kv=True, kv_capacity=capacity)),
        ):
            for mode in ("fast", "pytorch_compatible"):
                artifact = compile_exported_program(
                    prog, options=CompileOptions(**{**opts.__dict__, "numerical_mode": mode}))
                path = HERE / f"kernel_ir_tiny_{kind}_{mode}.json"
                path.write_text(json.dumps(module_to_json(artifact.module), indent=0))
    print(tag, "tokens", fixture["tokens"].tolist())


if __name__ == "__main__":
    torch.save(op_cases(), HERE / "ops.pt")
    tiny_model_case(torch.float32, "fp32")
    tiny_model_case(torch.bfloat16, "bf16")
    for path in sorted(HERE.iterdir()):
        print(f"{path.name:40s} {path.stat().st_size:>9d} bytes")
