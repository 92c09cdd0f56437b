"""Per-operation contracts of the B200 dialect and the run-time symbol guards, on the reference's
own graphs (golden JSON): every lowered graph verifies, and one deliberately broken operation
per contract is caught -- the checks the reference verifier applies by op name
(ir.py:462-835) and its executor applies to run-time extents (execution.py:1323-1347)."""

import gzip
import json
from pathlib import Path

import pytest
import torch

from llm_compiler_b200 import contracts
from llm_compiler_b200 import kernel_ir as ir

GOLDEN = Path(__file__).resolve().parent / "golden"


def lowered(name, **options):
    path = GOLDEN / name
    text = gzip.open(path).read() if name.endswith(".gz") else path.read_text()
    module = ir.module_from_json(json.loads(text))
    ir.lower_to_b200(module, **options)
    return module


ALL_GRAPHS = [f"kernel_ir_tiny_{kind}_{mode}.json" for kind in ("prefill", "decode")
              for mode in ("fast", "pytorch_compatible")] + \
    [f"kernel_ir_tiny_bf16_{kind}_fast.json" for kind in ("prefill", "decode")] + \
    [f"kernel_ir_qwen2_0_5b_{kind}_fast.json.gz" for kind in ("prefill", "decode")]


@pytest.mark.parametrize("name", ALL_GRAPHS)
@pytest.mark.parametrize("fuse", [True, False])
def test_every_lowered_graph_satisfies_the_contracts(name, fuse):
    module = lowered(name, fuse_graph=fuse, fuse_epilogues=fuse)
    assert contracts.operation_contract_errors(module) == []
    ir.verify_module(module)


def first(module, name):
    return next(op for op in module.functions[0].block.operations if op.name == name)


def retyped(value, text):
    value.type = text
    return value


BREAKAGES = {
    # contract -> (graph, mutation, expected message)
    "linear_k": ("decode", lambda m: first(m, "kernel.b200.linear").attributes.update(input_features=7),
                 "input_features attribute does not match"),
    "linear_bias": ("decode", lambda m: first(m, "kernel.b200.linear").attributes.update(has_bias=False),
                    "disagree with the operand count"),
    "linear_epilogue": ("decode", lambda m: first(m, "kernel.b200.linear").attributes.update(epilogue="gelu"),
                        "unknown epilogue"),
    "decode_groups": ("decode", lambda m: first(m, "kernel.b200.decode_attention").attributes.update(groups=3),
                      "query heads must equal KV heads x groups"),
    "decode_scale": ("decode", lambda m: first(m, "kernel.b200.decode_attention").attributes.update(scale=0.0),
                     "scale must be a positive number"),
    "decode_slot": ("decode", lambda m: first(m, "kernel.b200.decode_attention").attributes.update(slot=9),
                    "outside the state's 2 layers"),
    "prefill_causal": ("prefill", lambda m: first(m, "kernel.b200.prefill_attention").attributes.update(causal="no"),
                       "causal must be true"),
    "prefill_groups": ("prefill", lambda m: first(m, "kernel.b200.prefill_attention").attributes.update(groups=4),
                       "query heads must equal KV heads x groups"),
    "rope_head_dim": ("prefill", lambda m: first(m, "kernel.b200.rope").attributes.update(head_dim=32),
                      "head_dim must be static, even and equal to the attribute"),
    "rope_store_head_dim": ("decode", lambda m: first(m, "kernel.b200.rope_kv_store").attributes.update(head_dim=2),
                            "head_dim must be static, even and equal to the attribute"),
    "rms_norm_weight": ("decode", lambda m: retyped(first(m, "kernel.b200.rms_norm").operands[1],
                                                    "tensor<255xf32, cpu>"),
                        "weight must be a vector of the input's last dimension"),
    "advance_delta": ("decode", lambda m: first(m, "runtime.kv.advance").attributes.update(delta=0),
                      "delta must be a positive integer"),
    "store_slot": ("prefill", lambda m: first(m, "kernel.b200.kv_prefill_store").attributes.update(slot=-1),
                   "outside the state's 2 layers"),
    "pack_rows": ("decode", lambda m: retyped(first(m, "kernel.b200.pack_rows").results[0],
                                              "tensor<500x256xf32, cpu>"),
                  "must be the sum of the operands'"),
}


@pytest.mark.parametrize("case", sorted(BREAKAGES))
def test_one_broken_operation_per_contract_is_caught(case):
    kind, mutate, message = BREAKAGES[case]
    module = lowered(f"kernel_ir_tiny_{kind}_fast.json")
    mutate(module)
    errors = contracts.operation_contract_errors(module)
    assert any(message in error for error in errors), errors
    with pytest.raises(ValueError, match=message.split("(")[0].strip()[:40]):
        ir.verify_module(module)


def test_type_strings_parse():
    tensor = contracts.parse_type("tensor<s13<VR[1, 8]>x1x1xs11 + 1<VR[2, 64]>xf32, cpu>")
    assert tensor.rank == 4 and tensor.dtype == "f32" and tensor.shape[1:3] == (1, 1)
    assert contracts.symbol_of(tensor.shape[0]) == ("s13", 1, 8)
    assert contracts.symbol_of(tensor.shape[3]) == ("s11 + 1", 2, 64)
    assert contracts.symbol_of(7) is None
    state = contracts.parse_type("!serve.kv_state<bf16, layers=2, heads=2, head_dim=64, "
                                 "layout=contiguous_bshd, resource=kv.cache, capacity=64>")
    assert (state.dtype, state.layers, state.heads, state.head_dim, state.capacity) == ("bf16", 2, 2, 64, 64)
    assert contracts.parse_type("symint") is None


def test_run_time_symbols_are_bound_and_guarded():
    module = lowered("kernel_ir_tiny_decode_fast.json")
    arguments = module.functions[0].block.arguments
    by_name = {a.name: a for a in arguments}
    declared = [by_name["%input_ids"], by_name["%attention_mask"], by_name["%position_ids"]]

    def values(batch, mask_len, position_batch=None):
        return [torch.zeros(batch, 1, dtype=torch.int64), torch.zeros(batch, 1, 1, mask_len),
                torch.zeros(position_batch or batch, 1, dtype=torch.int64)]

    assert contracts.bind_symbols(declared, values(3, 6)) == {"s13": 3, "s11 + 1": 6}
    with pytest.raises(contracts.SymbolError, match="breaks the equality of symbol s13"):
        contracts.bind_symbols(declared, values(3, 6, position_batch=2))
    with pytest.raises(contracts.SymbolError, match="above the exporter's upper bound 8"):
        contracts.bind_symbols(declared, values(9, 6))
    with pytest.raises(contracts.SymbolError, match="below the exporter's lower bound 2"):
        contracts.bind_symbols(declared, values(3, 1))
    with pytest.raises(contracts.SymbolError, match="the graph fixes it at 1"):
        contracts.bind_symbols(declared[:1], [torch.zeros(3, 2, dtype=torch.int64)])
