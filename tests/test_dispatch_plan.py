"""Profile-guided dispatch plan: schema, bucketing rule, plan attributes, run-time resolution.

The bucketing rule and the decision record are the reference's (cost_model.py:126-245,
tests/test_cost_model.py:25-194): one variant per profiled value of the bucketed dimension,
owning the values up to floor(sqrt(this * next)); no plan -> "default", a plan without a
matching bucket -> "fallback", otherwise "profile". Expected thresholds below are worked out
by hand.
"""

import json
from pathlib import Path

import pytest

from llm_compiler_b200 import kernel_ir as kir
from llm_compiler_b200.dispatch_plan import (DispatchCostModel, ProfileError, resolve_dispatch_plan,
                                             select_variant, split_tokens_of)

GOLDEN = Path(__file__).parent / "golden"
LAYOUT = {"q_heads": 14, "kv_heads": 2, "head_dim": 64, "dtype": "bf16"}


def profile():
    rows = []
    for length, costs in ((256, {"split:0": 4.0, "split:512": 5.0}),
                          (4096, {"split:0": 30.0, "split:2048": 24.0, "split:1024": 33.0}),
                          (16384, {"split:0": 95.0, "split:4096": 90.0})):
        rows.append({"op": "decode_attention", "batch": 64, **LAYOUT, "length": length,
                     "variants_us": costs})
    rows.append({"op": "decode_attention", "batch": 8, **LAYOUT, "length": 4096,
                 "variants_us": {"split:0": 13.0, "split:512": 12.0}})
    for tokens, costs in ((128, {"tcgen05": 9.0, "mma.sync": 7.0}), (2048, {"tcgen05": 150.0, "mma.sync": 260.0})):
        rows.append({"op": "prefill_attention", **LAYOUT, "tokens": tokens, "variants_us": costs})
    for m, costs in ((16, {"tcgen05": 9.0, "mma.sync": 8.5}), (64, {"tcgen05": 9.5, "mma.sync": 9.4}),
                     (4096, {"tcgen05": 12.0, "mma.sync": 40.0})):
        rows.append({"op": "linear", "k": 256, "n": 256, "dtype": "float32", "m": m, "variants_us": costs})
    return {"schema_version": 1, "target": {"device_name": "NVIDIA B200", "compute_capability": "10.0"},
            "results": rows}


def test_buckets_are_bounded_by_the_geometric_mean_of_neighbouring_profiled_values():
    model = DispatchCostModel.from_dict(profile(), source="unit")
    variants = model.variants("decode_attention", batch=64, **LAYOUT)
    assert [(v.min_value, v.max_value, v.profile_value, v.variant) for v in variants] == [
        (1, 1024, 256, "split:0"),            # floor(sqrt(256 * 4096)) = 1024
        (1025, 8192, 4096, "split:2048"),     # floor(sqrt(4096 * 16384)) = 8192
        (8193, None, 16384, "split:4096")]
    assert variants[1].estimated_us == 24.0
    linear = model.variants("linear", k=256, n=256, dtype="fp32")
    assert [(v.min_value, v.max_value, v.variant) for v in linear] == [
        (1, 32, "mma.sync"), (33, 512, "mma.sync"), (513, None, "tcgen05")]
    assert model.variants("linear", k=999, n=256, dtype="fp32") == []


def test_the_built_in_plan_keeps_its_place_inside_the_noise_margin():
    rows = [{"op": "decode_attention", "batch": 64, **LAYOUT, "length": length, "variants_us": costs}
            for length, costs in ((4096, {"split:0": 24.82, "split:2048": 24.65}),       # 0.7 % cheaper: noise
                                  (16384, {"split:0": 97.0, "split:8192": 80.2}))]        # 17 % cheaper: taken
    variants = DispatchCostModel.from_dict(rows).variants("decode_attention", batch=64, **LAYOUT)
    assert [(v.variant, v.estimated_us) for v in variants] == [("split:0", 24.82), ("split:8192", 80.2)]


def test_allowed_variants_and_dtype_aliases():
    model = DispatchCostModel.from_dict(profile())
    only = model.variants("prefill_attention", allowed=["tcgen05"], q_heads=14, kv_heads=2,
                          head_dim=64, dtype="torch.bfloat16")
    assert [v.variant for v in only] == ["tcgen05", "tcgen05"]
    with pytest.raises(ProfileError):
        model.variants("prefill_attention", allowed=["nothing"], **LAYOUT)


def test_resolution_sources_default_profile_fallback():
    model = DispatchCostModel.from_dict(profile(), source="unit")
    plan = model.plan_attribute("decode_attention", batch=64, fallback="split:0", **LAYOUT)
    assert plan["schema_version"] == 1 and plan["bucketed_by"] == "length"
    assert plan["key"] == {"batch": 64, **LAYOUT} and plan["profile_source"] == "unit"
    json.dumps(plan)  # an attribute must serialise
    decision = resolve_dispatch_plan(plan, 4300)
    assert (decision.variant, decision.source, decision.profile_value) == ("split:2048", "profile", 4096)
    assert split_tokens_of(decision.variant) == 2048
    assert resolve_dispatch_plan(None, 10, default_variant="split:0").source == "default"
    hollow = dict(plan, variants=[v for v in plan["variants"] if v["max_value"] is not None])
    late = resolve_dispatch_plan(hollow, 100000)
    assert (late.variant, late.source) == ("split:0", "fallback")
    with pytest.raises(ProfileError):
        resolve_dispatch_plan(plan, 0)
    assert select_variant(plan["variants"], 1024).profile_value == 256
    assert split_tokens_of(None) == 0 and split_tokens_of("tcgen05") == 0


def test_schema_errors_and_the_reference_row_format():
    with pytest.raises(ProfileError):
        DispatchCostModel.from_dict({"schema_version": 2, "results": []})
    with pytest.raises(ProfileError):
        DispatchCostModel.from_dict("rows")
    with pytest.raises(ProfileError):
        DispatchCostModel.from_dict([{"op": "conv", "variants_us": {"a": 1.0}}])
    with pytest.raises(ProfileError):
        DispatchCostModel.from_dict([{"op": "linear", "k": 8, "n": 8, "dtype": "bf16", "m": 0,
                                      "variants_us": {"tcgen05": 1.0}}])
    with pytest.raises(ProfileError):
        DispatchCostModel.from_dict([{"op": "linear", "k": 8, "n": 8, "dtype": "bf16", "m": 4,
                                      "variants_us": {"tcgen05": -1.0}}])
    # rows as the reference's RMSNorm profiler writes them (bare list, cost_model.py:100-103)
    reference_rows = [
        {"rows": 1, "hidden_size": 896, "dtype": "float16", "native_eager_us": 20.0, "triton_us": 8.0},
        {"rows": 64, "hidden_size": 896, "dtype": "float16", "native_eager_us": 21.0, "triton_us": 9.0,
         "inductor_us": 7.5},
    ]
    model = DispatchCostModel.from_dict(reference_rows)
    variants = model.variants("rms_norm", hidden_size=896, dtype="fp16")
    assert [(v.min_value, v.max_value, v.variant) for v in variants] == [(1, 8, "triton"), (9, None, "inductor")]


def test_load_round_trip(tmp_path):
    path = tmp_path / "profile.json"
    path.write_text(json.dumps(profile()))
    model = DispatchCostModel.load(path)
    assert model.source == str(path) and model.target.device_name == "NVIDIA B200"
    assert len(model.entries) == 9


@pytest.mark.parametrize("name", ["kernel_ir_tiny_decode_fast.json", "kernel_ir_tiny_prefill_fast.json"])
def test_selection_pass_writes_plans_on_the_reference_graphs(name):
    module = kir.module_from_json(json.loads((GOLDEN / name).read_text()))
    kir.lower_to_b200(module)
    tiny = {"q_heads": 4, "kv_heads": 2, "head_dim": 64, "dtype": "fp32"}
    model = DispatchCostModel.from_dict([
        {"op": "linear", "k": 256, "n": 256, "dtype": "fp32", "m": 4, "variants_us": {"tcgen05": 5.0, "mma.sync": 4.0}},
        {"op": "decode_attention", "batch": 3, **tiny, "length": 64, "variants_us": {"split:0": 5.0, "split:32": 4.0}},
        {"op": "prefill_attention", **tiny, "tokens": 16, "variants_us": {"tcgen05": 5.0, "mma.sync": 4.0}},
    ])
    stats = kir.select_dispatch_plans(module, model)
    assert stats["changed"] and stats["planned_operations"] > 0
    operations = [op for function in module.functions for op in function.block.operations]
    planned = [op for op in operations if "lowering_plan" in op.attributes or "lowering_plans" in op.attributes]
    assert len(planned) == stats["planned_operations"]
    attention = [op for op in operations if op.name.endswith("_attention")]
    assert attention and all(("lowering_plans" if op.name.endswith("decode_attention") else "lowering_plan")
                             in op.attributes for op in attention)
    for op in attention:
        if op.name.endswith("decode_attention"):
            assert op.attributes["lowering_plans"]["3"]["variants"][0]["variant"] == "split:32"
    again = kir.select_dispatch_plans(module, model)
    assert not again["changed"]  # idempotent
    kir.module_from_json(kir.module_to_json(module))  # plans survive serialisation
