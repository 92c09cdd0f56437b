"""KernelIR for the B200 target: a host-side mirror of the reference's SSA containers, the
lowering pass that finishes what the reference's LowerToKernelIRPass starts, and the
coverage check behind `--require-full-lowering`.

The reference's lowering (lowering.py:91-208) renames the six serving ops to
`kernel.triton.*` / `kernel.cuda.*` / `kernel.cublas.*` and leaves 13-14 ATen op kinds to
PyTorch eager, so `require_full_lowering` fails on every real graph
(docs/qwen2-0.5b-validation.md:96-118). `lower_to_b200` takes a ServeIR module or the
reference's partly lowered KernelIR and rewrites EVERY op into `kernel.b200.*` (a launch of
libb200serve.so) or `runtime.*` (host metadata: views, shapes, KV state bookkeeping), fusing
where that is free:

  aten.to/unsqueeze/view/mul/cat/cos/sin/to chain of the RoPE table   -> kernel.b200.rope_table
  aten.silu + aten.mul                                                 -> kernel.b200.swiglu
  linear whose only user is a residual aten.add                        -> kernel.b200.linear(+residual)
  identity and dead aten.to.dtype                                      -> removed
  view / reshape / transpose / unsqueeze / sym_size                    -> runtime.view.*

The containers are duck-type compatible with the reference's (ir.py:124-158): the pass and
the executor read only `.functions`, `.block.arguments/.operations`, `.returns`,
`.name/.operands/.results/.attributes` and `str(value.type)`, so they accept the reference's
own Module objects as well as modules loaded from JSON (which is how graphs reach machines
where the reference package is not installed).
"""

from __future__ import annotations

import json
import re
from collections import Counter
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, Iterable, List, Optional


# ------------------------------------------------------------------ containers ----
@dataclass(eq=False)
class Value:
    name: str
    type: Any = ""

    def __str__(self) -> str:
        return self.name


@dataclass
class Operation:
    name: str
    operands: List[Value]
    results: List[Value]
    attributes: Dict[str, Any] = field(default_factory=dict)
    effects: tuple = ()


@dataclass
class Block:
    arguments: List[Value] = field(default_factory=list)
    operations: List[Operation] = field(default_factory=list)


@dataclass
class Function:
    name: str
    block: Block
    returns: List[Value]


@dataclass
class Module:
    functions: List[Function] = field(default_factory=list)


def module_from_json(data: Dict[str, Any] | str) -> Module:
    """Rebuilds a module from the JSON form written by `module_to_json`."""

    if isinstance(data, str):
        data = json.loads(data)
    module = Module()
    for entry in data["functions"]:
        values: Dict[str, Value] = {}
        block = Block()
        for argument in entry["arguments"]:
            value = Value(argument["name"], argument["type"])
            values[value.name] = value
            block.arguments.append(value)
        for item in entry["operations"]:
            operands = [values[name] for name in item["operands"]]
            results = [Value(r["name"], r["type"]) for r in item["results"]]
            for value in results:
                values[value.name] = value
            block.operations.append(Operation(item["name"], operands, results,
                                              dict(item.get("attributes", {}))))
        module.functions.append(Function(entry["name"], block,
                                         [values[name] for name in entry["returns"]]))
    return module


def module_to_json(module) -> Dict[str, Any]:
    functions = []
    for function in module.functions:
        functions.append({
            "name": function.name,
            "arguments": [{"name": a.name, "type": str(a.type)} for a in function.block.arguments],
            "operations": [{
                "name": op.name, "operands": [v.name for v in op.operands],
                "results": [{"name": r.name, "type": str(r.type)} for r in op.results],
                "attributes": op.attributes,
            } for op in function.block.operations],
            "returns": [v.name for v in function.returns],
        })
    return {"functions": functions}


# ------------------------------------------------------------------ type strings ----
_TENSOR_TYPE = re.compile(r"tensor<(.*)x([a-z]+\d*), *([^>]+)>$")


def value_dtype(value) -> Optional[str]:
    """dtype token ('f32', 'bf16', 'i64', ...) of a tensor-typed value, else None."""

    dtype = getattr(value.type, "dtype", None)
    if isinstance(dtype, str):
        return dtype
    match = _TENSOR_TYPE.match(str(value.type))
    return match.group(2) if match else None


def value_rank(value) -> Optional[int]:
    shape = getattr(value.type, "shape", None)
    if shape is not None:
        return len(shape)
    match = _TENSOR_TYPE.match(str(value.type))
    if not match:
        return None
    # dimensions are separated by 'x'; symbolic ones look like s13<VR[1, 8]> or "s11 + 1<...>"
    depth, count = 0, 1
    for char in match.group(1):
        if char == "<":
            depth += 1
        elif char == ">":
            depth -= 1
        elif char == "x" and depth == 0:
            count += 1
    return count


# ------------------------------------------------------------------ target tables ----
_SERVING_OPS = {
    "rms_norm": ("serve.rms_norm", "kernel.triton.rms_norm", "kernel.cuda.rms_norm"),
    "linear": ("serve.linear", "kernel.triton.linear", "kernel.cublas.linear"),
    "rope": ("serve.rope", "kernel.triton.rope", "kernel.cuda.rope"),
    "prefill_attention": ("serve.prefill_attention", "kernel.triton.prefill_attention",
                          "kernel.cuda.prefill_attention"),
    "decode_attention": ("serve.decode_attention", "kernel.triton.decode_attention",
                         "kernel.cuda.decode_attention"),
    "kv_store": ("serve.kv.store", "kernel.triton.kv_store"),
    "kv_prefill_store": ("serve.kv.prefill_store", "kernel.triton.kv_prefill_store"),
}
_KERNEL_SOURCES = {source: f"kernel.b200.{target}" for target, sources in _SERVING_OPS.items()
                   for source in sources}
_RUNTIME_SOURCES = {
    "serve.kv.init": "runtime.kv.init", "serve.kv.length": "runtime.kv.length",
    "serve.kv.advance": "runtime.kv.advance",
    "aten.view.default": "runtime.view.view", "aten.reshape.default": "runtime.view.reshape",
    "aten.transpose.int": "runtime.view.transpose", "aten.unsqueeze.default": "runtime.view.unsqueeze",
    "aten.sym_size.int": "runtime.view.sym_size",
}
_ELEMENTWISE_SOURCES = {
    "aten.embedding.default": "kernel.b200.embedding", "aten.add.Tensor": "kernel.b200.add",
    "aten.contiguous.default": "kernel.b200.contiguous", "aten.to.dtype": "kernel.b200.cast",
}

EXECUTABLE_OPERATIONS = frozenset(_KERNEL_SOURCES.values()) | frozenset(_RUNTIME_SOURCES.values()) | \
    frozenset(_ELEMENTWISE_SOURCES.values()) | frozenset({
        "runtime.kv.init", "runtime.kv.length", "runtime.kv.advance",
        "kernel.b200.rope_table", "kernel.b200.swiglu",
        # produced by the graph-level fusion passes (fusion.py)
        "kernel.b200.pack_rows", "kernel.b200.interleave_rows", "runtime.view.slice",
        "runtime.view.last_token",
        "kernel.b200.rope_kv_store", "kernel.b200.scale_columns", "kernel.b200.norm_linear",
        "kernel.b200.qkv_decode_attention", "runtime.kv.advance_all"})

NUMERICAL_MODES = ("fast", "pytorch_compatible")


@dataclass(frozen=True)
class LoweringCoverage:
    """How far a graph is from zero PyTorch fallback (lowering.py:56-72)."""

    total_operations: int
    lowered_operations: int
    unlowered_operations: int
    coverage: float
    lowered_by_name: Dict[str, int]
    unlowered_by_name: Dict[str, int]

    @property
    def is_complete(self) -> bool:
        return self.unlowered_operations == 0

    def to_dict(self) -> Dict[str, object]:
        return asdict(self)


class LoweringCoverageError(RuntimeError):
    """Strict mode found operations that no B200 kernel or runtime op executes."""

    def __init__(self, coverage: LoweringCoverage) -> None:
        self.coverage = coverage
        details = ", ".join(f"{n}x{c}" for n, c in coverage.unlowered_by_name.items())
        super().__init__(
            f"KernelIR is not fully lowered for the B200 target: {coverage.unlowered_operations}/"
            f"{coverage.total_operations} operations left ({details})")


def analyze_lowering_coverage(module) -> LoweringCoverage:
    lowered, unlowered = Counter(), Counter()
    for function in module.functions:
        for operation in function.block.operations:
            (lowered if operation.name in EXECUTABLE_OPERATIONS else unlowered)[operation.name] += 1
    done, left = sum(lowered.values()), sum(unlowered.values())
    total = done + left
    return LoweringCoverage(total, done, left, 1.0 if total == 0 else done / total,
                            dict(sorted(lowered.items())), dict(sorted(unlowered.items())))


def require_full_lowering(module) -> LoweringCoverage:
    coverage = analyze_lowering_coverage(module)
    if not coverage.is_complete:
        raise LoweringCoverageError(coverage)
    return coverage


# ------------------------------------------------------------------ the pass ----
def decode_attribute(value: Any, environment: Dict[str, Any]) -> Any:
    """Resolves the JSON argument tree the importer stores in attributes["args"]
    (importer.py:96-128; decoder execution.py:1052-1070)."""

    if isinstance(value, dict):
        if set(value) == {"ssa"}:
            return environment[value["ssa"]]
        if set(value) == {"tuple"}:
            return tuple(decode_attribute(item, environment) for item in value["tuple"])
        return {key: decode_attribute(item, environment) for key, item in value.items()}
    if isinstance(value, list):
        return [decode_attribute(item, environment) for item in value]
    return value


def _users(function) -> Dict[str, List[Any]]:
    users: Dict[str, List[Any]] = {}
    for operation in function.block.operations:
        for operand in operation.operands:
            users.setdefault(operand.name, []).append(operation)
    for value in function.returns:
        users.setdefault(value.name, []).append("return")
    return users


def _replace_uses(function, old, new) -> None:
    def swap(tree):
        if isinstance(tree, dict):
            if set(tree) == {"ssa"} and tree["ssa"] == old.name:
                return {"ssa": new.name}
            return {key: swap(item) for key, item in tree.items()}
        if isinstance(tree, list):
            return [swap(item) for item in tree]
        return tree

    for operation in function.block.operations:
        if any(operand is old or operand.name == old.name for operand in operation.operands):
            operation.operands = [new if (o is old or o.name == old.name) else o
                                  for o in operation.operands]
            if "args" in operation.attributes:
                operation.attributes["args"] = swap(operation.attributes["args"])
            if "kwargs" in operation.attributes:
                operation.attributes["kwargs"] = swap(operation.attributes["kwargs"])
    function.returns = [new if (v is old or v.name == old.name) else v for v in function.returns]


_PURE_PREFIXES = ("aten.", "kernel.b200.rope_table", "kernel.b200.swiglu", "runtime.view.",
                  "kernel.b200.pack_rows", "kernel.b200.interleave_rows", "kernel.b200.scale_columns")


def _is_pure(operation) -> bool:
    if getattr(operation, "effects", ()):
        return False
    return operation.name.startswith(_PURE_PREFIXES) or operation.name in (
        "kernel.b200.cast", "kernel.b200.add", "kernel.b200.embedding", "kernel.b200.contiguous")


def _eliminate_dead(function) -> int:
    removed = 0
    while True:
        users = _users(function)
        dead = [op for op in function.block.operations
                if _is_pure(op) and op.results and all(not users.get(r.name) for r in op.results)]
        if not dead:
            return removed
        dead_ids = {id(op) for op in dead}
        function.block.operations = [op for op in function.block.operations
                                     if id(op) not in dead_ids]
        removed += len(dead)


def _cast_target(operation) -> Optional[str]:
    args = operation.attributes.get("args")
    if isinstance(args, dict) and "tuple" in args and len(args["tuple"]) >= 2 and \
            isinstance(args["tuple"][1], str):
        return args["tuple"][1]
    return operation.attributes.get("dtype")


def _fold_identity_casts(function) -> int:
    folded = 0
    for operation in list(function.block.operations):
        if operation.name != "aten.to.dtype" or len(operation.operands) != 1:
            continue
        source = operation.operands[0]
        if _cast_target(operation) is not None and _cast_target(operation) == value_dtype(source):
            _replace_uses(function, operation.results[0], source)
            function.block.operations.remove(operation)
            folded += 1
    return folded


def _producer_map(function) -> Dict[str, Any]:
    return {result.name: op for op in function.block.operations for result in op.results}


def _fuse_rope_table(function) -> int:
    """cos(cat(f, f)) / sin(cat(f, f)) with f = unsqueeze(to_f32(position_ids)) * view(inv_freq),
    each followed by a cast to the model dtype (Qwen2RotaryEmbedding.forward, qwen2.py:136-149)."""

    producers = _producer_map(function)

    def through(value, names):
        while value.name in producers and producers[value.name].name in names:
            value = producers[value.name].operands[0]
        return value

    fused = 0
    for cat in list(function.block.operations):
        if cat.name != "aten.cat.default" or len(cat.operands) != 2 or \
                cat.operands[0].name != cat.operands[1].name:
            continue
        mul = producers.get(cat.operands[0].name)
        if mul is None or mul.name != "aten.mul.Tensor" or len(mul.operands) != 2:
            continue
        users = _users(function)
        cos_ops = [u for u in users.get(cat.results[0].name, []) if u != "return" and
                   u.name == "aten.cos.default"]
        sin_ops = [u for u in users.get(cat.results[0].name, []) if u != "return" and
                   u.name == "aten.sin.default"]
        if len(cos_ops) != 1 or len(sin_ops) != 1 or len(users[cat.results[0].name]) != 2:
            continue
        shape_ops = {"aten.to.dtype", "aten.unsqueeze.default", "aten.view.default"}
        first, second = through(mul.operands[0], shape_ops), through(mul.operands[1], shape_ops)
        if value_dtype(first) == "i64":
            positions, inv_freq = first, second
        elif value_dtype(second) == "i64":
            positions, inv_freq = second, first
        else:
            continue
        outputs = []
        for trig in (cos_ops[0], sin_ops[0]):
            result = trig.results[0]
            trig_users = users.get(result.name, [])
            if len(trig_users) == 1 and trig_users[0] != "return" and \
                    trig_users[0].name == "aten.to.dtype":
                outputs.append((trig, trig_users[0], trig_users[0].results[0]))
            else:
                outputs.append((trig, None, result))
        dtype = value_dtype(outputs[0][2])
        if dtype is None or dtype != value_dtype(outputs[1][2]):
            continue
        anchor = function.block.operations.index(cos_ops[0])
        table = Operation("kernel.b200.rope_table", [positions, inv_freq],
                          [outputs[0][2], outputs[1][2]],
                          {"dtype": dtype, "lowered_from": "aten.cos.default+aten.sin.default"})
        function.block.operations.insert(anchor, table)
        for trig, cast, _ in outputs:
            function.block.operations.remove(trig)
            if cast is not None:
                function.block.operations.remove(cast)
        fused += 1
    return fused


def _fuse_swiglu(function) -> int:
    producers = _producer_map(function)
    users = _users(function)
    fused = 0
    for mul in list(function.block.operations):
        if mul.name != "aten.mul.Tensor" or len(mul.operands) != 2:
            continue
        for index in (0, 1):
            silu = producers.get(mul.operands[index].name)
            if silu is not None and silu.name == "aten.silu.default" and \
                    len(users.get(silu.results[0].name, [])) == 1:
                mul.name = "kernel.b200.swiglu"
                mul.operands = [silu.operands[0], mul.operands[1 - index]]
                mul.attributes = {"lowered_from": "aten.silu.default+aten.mul.Tensor"}
                function.block.operations.remove(silu)
                fused += 1
                break
    return fused


def _fuse_residual_epilogues(function) -> int:
    producers = _producer_map(function)
    users = _users(function)
    fused = 0
    for add in list(function.block.operations):
        if add.name != "kernel.b200.add" or len(add.operands) != 2:
            continue
        for index in (1, 0):
            linear = producers.get(add.operands[index].name)
            if linear is None or linear.name != "kernel.b200.linear" or \
                    linear.attributes.get("epilogue") or \
                    len(users.get(linear.results[0].name, [])) != 1:
                continue
            residual = add.operands[1 - index]
            if str(residual.type) != str(linear.results[0].type):
                continue
            function.block.operations.remove(linear)
            linear.operands = list(linear.operands) + [residual]
            linear.results = add.results
            linear.attributes["epilogue"] = "residual"
            linear.attributes.pop("args", None)
            function.block.operations[function.block.operations.index(add)] = linear
            fused += 1
            break
    return fused


@dataclass
class LoweringReport:
    numerical_mode: str
    lowered_rules: Dict[str, int]
    removed_casts: int
    removed_dead: int
    coverage: LoweringCoverage


def lower_to_b200(module, *, numerical_mode: Optional[str] = None,
                  fuse_epilogues: bool = True, fuse_graph: bool = True,
                  causal_mask_arguments: Iterable[str] = (),
                  zero_mask_arguments: Iterable[str] = (),
                  fuse_decode_chain: bool = True,
                  last_token_logits: bool = False) -> LoweringReport:
    """Rewrites `module` in place for the B200 target. `numerical_mode` overrides the mode the
    reference's pass recorded on each op (attribute `numerical_mode`, or implied by a
    `kernel.cuda.*` / `kernel.cublas.*` name); default "fast". `fuse_graph` runs the
    graph-level passes of fusion.py (packed q|k|v and gate|up projections, fused rope + KV
    store of a decode step); `causal_mask_arguments` names graph inputs the caller declares to
    be causal masks, which turns the prefill attention they feed into the mask-free causal
    form. `fuse_decode_chain` (fast bf16 ops only) folds each RMSNorm into the projection behind
    it and, where `zero_mask_arguments` names the decode step's mask input as all zero, turns a
    decode layer's projection -> RoPE -> KV store -> advance -> attention into the fused
    attention op, with the per-slot length updates hoisted into one op at the end.
    `last_token_logits` (opt-in: it changes the first result to B x 1 x V) computes the final norm
    and the LM head of a prefill for the last position only. Idempotent."""

    if numerical_mode is not None and numerical_mode not in NUMERICAL_MODES:
        raise ValueError(f"unknown numerical mode {numerical_mode!r}; choose from {NUMERICAL_MODES}")
    rules: Counter = Counter()
    removed_casts = removed_dead = 0
    for function in module.functions:
        removed_casts += _fold_identity_casts(function)
        removed_dead += _eliminate_dead(function)
        rules["rope_table"] += _fuse_rope_table(function)
        rules["swiglu"] += _fuse_swiglu(function)
        removed_dead += _eliminate_dead(function)
        for operation in function.block.operations:
            source = operation.name
            target = _KERNEL_SOURCES.get(source) or _RUNTIME_SOURCES.get(source) or \
                _ELEMENTWISE_SOURCES.get(source)
            if target is None:
                continue
            if source == "aten.add.Tensor" and len(operation.operands) != 2:
                continue  # tensor + python scalar: not an op of these graphs
            if source in _KERNEL_SOURCES and "kv" not in target:
                # mode: explicit override > what the reference's pass recorded > implied by name
                implied = "pytorch_compatible" if source.startswith("kernel.cuda.") or \
                    operation.attributes.get("backend_selection") == "pytorch_compatible" else "fast"
                operation.attributes["numerical_mode"] = (
                    numerical_mode or operation.attributes.get("numerical_mode") or implied)
            operation.attributes.setdefault("lowered_from", source)
            operation.name = target
            rules[f"{source}->{target}"] += 1
        if fuse_epilogues:
            rules["linear+residual"] += _fuse_residual_epilogues(function)
        if fuse_graph:
            from . import fusion

            rules["pack_qkv"] += fusion.pack_qkv(function)
            rules["pack_gate_up"] += fusion.pack_gate_up(function)
            rules["rope+kv_store"] += fusion.fuse_rope_kv_store(function)
            if fuse_decode_chain:
                rules["norm+linear"] += fusion.fuse_norm_linear(function)
                rules["qkv+attention"] += fusion.fuse_qkv_attention(function, tuple(zero_mask_arguments))
                rules["advance_all"] += fusion.hoist_kv_advances(function)
                removed_dead += _eliminate_dead(function)  # shape values only the fused ops' views used
        if causal_mask_arguments:
            from . import fusion

            rules["causal_mask"] += fusion.mark_causal_masks(function, tuple(causal_mask_arguments))
        if last_token_logits:
            from . import fusion

            rules["last_token_logits"] += fusion.take_last_token_logits(function)
    return LoweringReport(numerical_mode or "per-op", {k: v for k, v in sorted(rules.items()) if v},
                          removed_casts, removed_dead, analyze_lowering_coverage(module))


def static_dims(value) -> Optional[List[Optional[int]]]:
    """Dimensions of a tensor-typed value: ints where static, None where symbolic."""

    shape = getattr(value.type, "shape", None)
    if shape is not None:
        return [getattr(dim, "value", None) if not isinstance(dim, int) else dim for dim in shape]
    match = _TENSOR_TYPE.match(str(value.type))
    if not match:
        return None
    parts, depth, current = [], 0, ""
    for char in match.group(1):
        if char == "<":
            depth += 1
        elif char == ">":
            depth -= 1
        if char == "x" and depth == 0:
            parts.append(current)
            current = ""
        else:
            current += char
    parts.append(current)
    return [int(part) if part.strip().isdigit() else None for part in parts]


_PLAN_DTYPES = {"bf16": "bf16", "f32": "fp32", "f16": "fp16"}


def select_dispatch_plans(module, cost_model) -> Dict[str, Any]:
    """Writes profile-guided `lowering_plan` attributes onto the lowered operations that have
    kernel variants, the way the reference's SelectRMSNormLoweringPass does for serve.rms_norm
    (passes/lowering_selection.py:24-71): linear by (k, n, dtype), bucketed by rows at run time;
    prefill attention by the head layout, bucketed by tokens; decode attention by the head
    layout, one plan per profiled batch size (`lowering_plans`), bucketed by context length.
    Returns the pass statistics. `cost_model` is a dispatch_plan.DispatchCostModel."""

    from .dispatch_plan import OPERATORS

    planned = missing = 0
    chosen: Counter = Counter()
    changed = False

    def attach(operation, name: str, plan) -> None:
        nonlocal planned, missing, changed
        variants = plan["variants"] if "variants" in plan else \
            [v for family in plan.values() for v in family["variants"]]
        if not variants:
            missing += 1
            return
        planned += 1
        chosen.update(variant["variant"] for variant in variants)
        if operation.attributes.get(name) != plan:
            operation.attributes[name] = plan
            changed = True

    for function in module.functions:
        for operation in function.block.operations:
            if operation.name == "kernel.b200.linear":
                dtype = _PLAN_DTYPES.get(value_dtype(operation.results[0]) or "")
                k, n = operation.attributes.get("input_features"), operation.attributes.get("output_features")
                if dtype is None or not isinstance(k, int) or not isinstance(n, int):
                    missing += 1
                    continue
                attach(operation, "lowering_plan", cost_model.plan_attribute("linear", k=k, n=n, dtype=dtype))
            elif operation.name in ("kernel.b200.prefill_attention", "kernel.b200.decode_attention"):
                decode = operation.name.endswith("decode_attention")
                query = operation.operands[1] if decode else operation.operands[0]
                dims, dtype = static_dims(query), _PLAN_DTYPES.get(value_dtype(query) or "")
                groups = operation.attributes.get("groups")
                if dims is None or len(dims) != 4 or dims[1] is None or dims[3] is None or \
                        dtype is None or not isinstance(groups, int) or groups <= 0:
                    missing += 1
                    continue
                layout = {"q_heads": dims[1], "kv_heads": dims[1] // groups, "head_dim": dims[3],
                          "dtype": dtype}
                if not decode:
                    attach(operation, "lowering_plan",
                           cost_model.plan_attribute("prefill_attention", **layout))
                    continue
                batches = sorted({dict(entry.key)["batch"] for entry in cost_model.entries
                                  if entry.op == "decode_attention" and
                                  all(dict(entry.key)[name] == layout[name] for name in layout)})
                attach(operation, "lowering_plans",
                       {str(batch): cost_model.plan_attribute("decode_attention", batch=batch, **layout)
                        for batch in batches} or {"none": {"variants": []}})
    assert set(OPERATORS) >= {"linear", "prefill_attention", "decode_attention"}
    return {"changed": changed, "planned_operations": planned, "missing_profile": missing,
            "variants": dict(sorted(chosen.items()))}


def verify_module(module) -> None:
    """SSA sanity (unique definitions, operands defined before use, ir.py:220-260) and the
    per-operation contracts of the kernel.b200.* / runtime.kv.* dialect (contracts.py: shapes,
    dtypes, bias / epilogue operands, GQA groups, slots, as ir.py:462-835 checks them for the
    reference's own op names). Raises ValueError listing every violation."""

    from .contracts import operation_contract_errors

    errors = []
    for function in module.functions:
        defined = {argument.name for argument in function.block.arguments}
        if len(defined) != len(function.block.arguments):
            errors.append(f"@{function.name}: duplicate argument names")
        for index, operation in enumerate(function.block.operations):
            for operand in operation.operands:
                if operand.name not in defined:
                    errors.append(f"@{function.name} op {index} {operation.name} uses undefined "
                                  f"{operand.name}")
            for result in operation.results:
                if result.name in defined:
                    errors.append(f"@{function.name} op {index} {operation.name} redefines "
                                  f"{result.name}")
                defined.add(result.name)
        for value in function.returns:
            if value.name not in defined:
                errors.append(f"@{function.name} returns undefined {value.name}")
    errors.extend(operation_contract_errors(module))
    if errors:
        raise ValueError("\n".join(errors))
