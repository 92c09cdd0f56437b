"""Graph-level fusion passes of the B200 lowering.

The reference lowers op by op and names the graph-level forms as its own next steps: a fused
SwiGLU op and fused q|k|v / gate|up projections (docs/rope-lowering.md:162-163,
docs/qwen2-0.5b-validation.md:200) and a compiler-proved `causal: true` prefill attention
(docs/prefill-attention.md:43-45). These passes do that on the KernelIR itself, after
`kernel_ir.lower_to_b200` has renamed every op, so that a module compiled by the reference
and run by `B200Executor` launches the same kernels as a hand-wired engine:

  pack_qkv            three linears on one input  -> pack_rows (weights, once) + ONE linear
                                                     + three runtime.view.slice views
  pack_gate_up        swiglu(linear, linear)      -> interleave_rows (once) + ONE linear whose
                                                     epilogue is SwiGLU
  mark_causal_masks   prefill_attention whose mask is a caller-declared causal argument
                                                  -> causal: true (the mask is not read)
  fuse_rope_kv_store  rope -> kv.length -> kv_store of ONE token
                                                  -> kernel.b200.rope_kv_store (one launch)
  chain_decode_layers (fast bf16 decode graphs)   -> the 5-launch decode layer: RMSNorm folded
                                                     into the next projection, split-K
                                                     projections that add their residual,
                                                     q|k|v reduction + RoPE + KV store inside
                                                     the attention launch

Weight-preparation ops carry `"constant": true`: their operands are graph parameters, the
executor evaluates them once per set of weight tensors and caches the result.
"""

from __future__ import annotations

import re
from typing import Any, Dict, List, Optional, Sequence

from .kernel_ir import Operation, Value, _producer_map, _users, value_dtype

_DIMS = re.compile(r"^tensor<(.*)x([a-z]+\d*), *([^>]+)>$")


def _split_dims(text: str) -> List[str]:
    parts, depth, current = [], 0, ""
    for char in text:
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
    return parts


def retype(value, axis: int, extent: int) -> str:
    """Type string of `value` with dimension `axis` replaced by the static `extent`."""

    match = _DIMS.match(str(value.type))
    if not match:
        raise ValueError(f"not a tensor type: {value.type}")
    dims = _split_dims(match.group(1))
    dims[axis] = str(int(extent))
    return f"tensor<{'x'.join(dims)}x{match.group(2)}, {match.group(3)}>"


def _static_extent(value, axis: int) -> Optional[int]:
    match = _DIMS.match(str(value.type))
    if not match:
        return None
    text = _split_dims(match.group(1))[axis].strip()
    return int(text) if text.isdigit() else None


def _is_parameter(function, value) -> bool:
    return any(argument is value or argument.name == value.name
               for argument in function.block.arguments)


def _fresh(function, stem: str) -> str:
    taken = {a.name for a in function.block.arguments} | \
        {r.name for op in function.block.operations for r in op.results}
    index = 0
    while f"%{stem}_{index}" in taken:
        index += 1
    return f"%{stem}_{index}"


def _mode_of(operation) -> str:
    return operation.attributes.get("numerical_mode", "fast")


# ------------------------------------------------------------------ q|k|v packing ----
def pack_qkv(function) -> int:
    """Groups of >= 2 `kernel.b200.linear` ops without an epilogue that read the same input
    and whose weights (and biases) are graph parameters become one projection over the
    row-concatenated weight. Only groups of exactly three with equal bias presence are packed
    (q, k, v); gate / up pairs are left to `pack_gate_up`."""

    packed = 0
    by_input: Dict[str, List[Any]] = {}
    for operation in function.block.operations:
        if operation.name == "kernel.b200.linear" and not operation.attributes.get("epilogue"):
            by_input.setdefault(operation.operands[0].name, []).append(operation)
    for group in by_input.values():
        if len(group) != 3:
            continue
        has_bias = [bool(op.attributes.get("has_bias")) for op in group]
        if len(set(has_bias)) != 1:
            continue
        if not all(_is_parameter(function, operand) for op in group for operand in op.operands[1:]):
            continue
        if len({value_dtype(op.results[0]) for op in group}) != 1 or \
                len({_mode_of(op) for op in group}) != 1:
            continue
        widths = [_static_extent(op.operands[1], 0) for op in group]
        if any(width is None for width in widths):
            continue
        first = function.block.operations.index(group[0])
        total = sum(widths)
        weight = Value(_fresh(function, "packed_weight"), retype(group[0].operands[1], 0, total))
        prepared = [Operation("kernel.b200.pack_rows", [op.operands[1] for op in group], [weight],
                              {"constant": True, "lowered_from": "weight preparation"})]
        operands = [group[0].operands[0], weight]
        if has_bias[0]:
            bias = Value(_fresh(function, "packed_bias"), retype(group[0].operands[2], 0, total))
            prepared.append(Operation("kernel.b200.pack_rows", [op.operands[2] for op in group],
                                      [bias], {"constant": True, "lowered_from": "weight preparation"}))
            operands.append(bias)
        output = Value(_fresh(function, "qkv"), retype(group[0].results[0], -1, total))
        attributes = {key: value for key, value in group[0].attributes.items()
                      if key not in ("args", "fx_name", "lowering_plan")}
        attributes.update({"output_features": total, "has_bias": has_bias[0],
                           "lowered_from": "+".join(["kernel.b200.linear"] * 3),
                           "packed": [int(width) for width in widths]})
        fused = Operation("kernel.b200.linear", operands, [output], attributes)
        slices, offset = [], 0
        for op, width in zip(group, widths):
            slices.append(Operation(
                "runtime.view.slice", [output], list(op.results),
                {"args": {"tuple": [{"ssa": output.name}, -1, offset, offset + width]},
                 "lowered_from": "kernel.b200.linear"}))
            offset += width
        # everything goes where the first projection stood: its operands are defined before it,
        # and the users of the second and third projection come later still
        remaining = [op for op in function.block.operations if all(op is not g for g in group)]
        function.block.operations = remaining[:first] + prepared + [fused] + slices + remaining[first:]
        packed += 1
    return packed


# ---------------------------------------------------------------- gate|up packing ----
def pack_gate_up(function) -> int:
    """swiglu(linear(x, Wg), linear(x, Wu)) with parameter weights and no other users of the
    two products becomes one linear over the row-interleaved weight with a SwiGLU epilogue."""

    producers = _producer_map(function)
    users = _users(function)
    packed = 0
    for swiglu in list(function.block.operations):
        if swiglu.name != "kernel.b200.swiglu":
            continue
        gate, up = (producers.get(operand.name) for operand in swiglu.operands)
        if gate is None or up is None or gate is up:
            continue
        if any(op.name != "kernel.b200.linear" or op.attributes.get("epilogue") or
               op.attributes.get("has_bias") or len(users.get(op.results[0].name, [])) != 1
               for op in (gate, up)):
            continue
        if gate.operands[0].name != up.operands[0].name or \
                not _is_parameter(function, gate.operands[1]) or \
                not _is_parameter(function, up.operands[1]) or _mode_of(gate) != _mode_of(up):
            continue
        width = _static_extent(gate.operands[1], 0)
        if width is None or width != _static_extent(up.operands[1], 0):
            continue
        weight = Value(_fresh(function, "gate_up_weight"), retype(gate.operands[1], 0, 2 * width))
        prepared = Operation("kernel.b200.interleave_rows", [gate.operands[1], up.operands[1]],
                             [weight], {"constant": True, "lowered_from": "weight preparation"})
        attributes = {key: value for key, value in gate.attributes.items()
                      if key not in ("args", "fx_name", "lowering_plan")}
        attributes.update({"output_features": 2 * width, "epilogue": "swiglu",
                           "lowered_from": "kernel.b200.linear+kernel.b200.linear+kernel.b200.swiglu"})
        fused = Operation("kernel.b200.linear", [gate.operands[0], weight], list(swiglu.results),
                          attributes)
        operations = function.block.operations
        anchor = min(operations.index(gate), operations.index(up))  # nothing removed lies before it
        rest = [op for op in operations if op is not gate and op is not up and op is not swiglu]
        function.block.operations = rest[:anchor] + [prepared, fused] + rest[anchor:]
        producers = _producer_map(function)
        users = _users(function)
        packed += 1
    return packed


# ----------------------------------------------------------------- causal masks ----
def _through_casts(value, producers):
    while value.name in producers and producers[value.name].name in ("kernel.b200.cast",
                                                                     "aten.to.dtype"):
        value = producers[value.name].operands[0]
    return value


def mark_causal_masks(function, causal_mask_arguments: Sequence[str]) -> int:
    """`causal_mask_arguments` names graph inputs the caller promises to be causal masks (0 on
    and below the diagonal, -inf above): prefill attention fed by one of them is rewritten to
    the mask-free causal form. The operand stays (the signature is unchanged); the kernel does
    not read it. Graph inputs nobody vouches for keep `causal: "mask"`; the executor may still
    classify the tensor at run time."""

    names = {name if name.startswith("%") else f"%{name}" for name in causal_mask_arguments}
    producers = _producer_map(function)
    marked = 0
    for operation in function.block.operations:
        if operation.name != "kernel.b200.prefill_attention" or len(operation.operands) != 4:
            continue
        source = _through_casts(operation.operands[3], producers)
        if source.name in names and _is_parameter(function, source) and \
                operation.attributes.get("causal") is not True:
            operation.attributes["causal"] = True
            operation.attributes["causal_proof"] = f"declared:{source.name}"
            marked += 1
    return marked


# ------------------------------------------------------------- rope + kv.store ----
def fuse_rope_kv_store(function) -> int:
    """Decode graphs: rope(q, k) -> kv.length(slot) -> kv_store(state, k', v, positions) with
    one token per sequence becomes `kernel.b200.rope_kv_store` (rotates q and k, writes k' and v
    into the slot at the slot's positions, returns q' and the state) when k' has no other user."""

    users = _users(function)
    producers = _producer_map(function)
    fused = 0
    for store in list(function.block.operations):
        if store.name != "kernel.b200.kv_store" or len(store.operands) != 4:
            continue
        state, key, value, positions = store.operands
        rope = producers.get(key.name)
        length = producers.get(positions.name)
        if rope is None or rope.name != "kernel.b200.rope" or rope.results[1].name != key.name or \
                length is None or length.name != "runtime.kv.length" or \
                length.operands[0].name != state.name or \
                int(length.attributes.get("slot", 0)) != int(store.attributes.get("slot", 0)):
            continue
        if len(users.get(key.name, [])) != 1 or _static_extent(rope.results[0], 2) != 1:
            continue
        operations = function.block.operations
        if not operations.index(rope) < operations.index(store):
            continue
        if any(user == "return" or operations.index(user) < operations.index(store)
               for user in users.get(rope.results[0].name, [])):
            continue  # the rotated query is needed before the store: keep the ops apart
        merged = Operation(
            "kernel.b200.rope_kv_store",
            [state, rope.operands[0], rope.operands[1], value, rope.operands[2], rope.operands[3]],
            [rope.results[0], store.results[0]],
            {"slot": int(store.attributes.get("slot", 0)), "head_dim": rope.attributes.get("head_dim"),
             "numerical_mode": _mode_of(rope),
             "lowered_from": "kernel.b200.rope+runtime.kv.length+kernel.b200.kv_store"})
        position = operations.index(store)
        operations[position] = merged
        operations.remove(rope)
        if len(users.get(positions.name, [])) == 1:
            operations.remove(length)
        users = _users(function)
        producers = _producer_map(function)
        fused += 1
    return fused


# ------------------------------------------------------------- the decode chain ----
def _single_user(users, value) -> Optional[Any]:
    found = users.get(value.name, [])
    return found[0] if len(found) == 1 and found[0] != "return" else None


def fuse_norm_linear(function) -> int:
    """rms_norm(x, w) whose only user is a bias-free or biased `kernel.b200.linear` without a
    residual (fast mode, bf16, parameter weights) becomes
    `kernel.b200.norm_linear` [x, w, W, scale_columns(W, w), bias?]: at run time, up to 64 rows,
    ONE launch on the un-normalised rows with the norm weight folded into W's columns and the
    row factor applied to the accumulator; beyond that the executor runs the two kernels."""

    users = _users(function)
    fused = 0
    for norm in list(function.block.operations):
        if norm.name != "kernel.b200.rms_norm" or _mode_of(norm) != "fast" or \
                value_dtype(norm.results[0]) != "bf16":
            continue
        linear = _single_user(users, norm.results[0])
        if linear is None or linear.name != "kernel.b200.linear" or _mode_of(linear) != "fast" or \
                linear.operands[0].name != norm.results[0].name or \
                (linear.attributes.get("epilogue") or "none") not in ("none", "swiglu"):
            continue
        weight = linear.operands[1]
        producer = _producer_map(function).get(weight.name)
        prepared = producer is not None and producer.attributes.get("constant") is True
        # (a weight with other readers -- a tied LM head is also the embedding table -- keeps its
        # plain copy for them; the folded copy costs its size in memory, nothing per step)
        if not (_is_parameter(function, weight) or prepared) or \
                not _is_parameter(function, norm.operands[1]):
            continue
        folded = Value(_fresh(function, "folded_weight"), str(weight.type))
        prepare = Operation("kernel.b200.scale_columns", [weight, norm.operands[1]], [folded],
                            {"constant": True, "lowered_from": "weight preparation"})
        attributes = {key: value for key, value in linear.attributes.items()
                      if key not in ("args", "fx_name")}
        attributes.update({"epsilon": norm.attributes.get("epsilon"),
                           "round_before_weight": bool(norm.attributes.get("round_before_weight", False)),
                           "lowered_from": "kernel.b200.rms_norm+" + str(linear.attributes.get(
                               "lowered_from", "kernel.b200.linear"))})
        merged = Operation("kernel.b200.norm_linear",
                           [norm.operands[0], norm.operands[1], weight, folded] + list(linear.operands[2:]),
                           list(linear.results), attributes)
        operations = function.block.operations
        position = operations.index(linear)
        operations[position:position + 1] = [prepare, merged]
        operations.remove(norm)
        users = _users(function)
        fused += 1
    return fused


def _view_chain(users, producers, value, names):
    """Follows `value` through single-user ops named in `names`; returns the last value."""
    while True:
        user = _single_user(users, value)
        if user is None or user.name not in names or user.operands[0].name != value.name:
            return value
        value = user.results[0]


def fuse_qkv_attention(function, zero_mask_arguments: Sequence[str]) -> int:
    """One decode layer's norm_linear(q|k|v) -> slices / views / transposes -> rope_kv_store ->
    kv.advance -> decode_attention -> transpose / reshape becomes
    `kernel.b200.qkv_decode_attention` [state, x, norm_w, W, folded W, bias?, cos, sin, mask]
    -> (context B x 1 x Hq D, advanced state): up to 64 rows at run time it is two launches (the
    split-K partial products of the packed projection, then the attention kernel that reduces
    them, applies the folded norm, bias and RoPE, stores the new K / V row and attends).
    Only where the caller declares the decode mask all zero (`zero_mask_arguments`): the fused
    kernel reads no mask."""

    names = {name if name.startswith("%") else f"%{name}" for name in zero_mask_arguments}
    if not names:
        return 0
    fused = 0
    for attention in list(function.block.operations):
        if attention.name != "kernel.b200.decode_attention" or _mode_of(attention) != "fast":
            continue
        producers = _producer_map(function)
        users = _users(function)
        mask = _through_casts(attention.operands[2], producers)
        if mask.name not in names or not _is_parameter(function, mask):
            continue
        advance = producers.get(attention.operands[0].name)
        store = producers.get(advance.operands[0].name) if advance is not None and \
            advance.name == "runtime.kv.advance" and int(advance.attributes.get("delta", 1)) == 1 else None
        if store is None or store.name != "kernel.b200.rope_kv_store" or \
                store.results[0].name != attention.operands[1].name or \
                len({int(op.attributes.get("slot", 0)) for op in (attention, advance, store)}) != 1 or \
                len(users.get(store.results[0].name, [])) != 1 or \
                len(users.get(store.results[1].name, [])) != 1 or \
                len(users.get(advance.results[0].name, [])) < 1:
            continue
        # q, k, v each come from the packed projection through slice -> view -> transpose
        sources, chain_ops = [], []
        for operand in store.operands[1:4]:
            value, path = operand, []
            for expected in ("runtime.view.transpose", "runtime.view.view", "runtime.view.slice"):
                op = producers.get(value.name)
                if op is None or op.name != expected or len(users.get(op.results[0].name, [])) != 1:
                    path = None
                    break
                path.append(op)
                value = op.operands[0]
            if path is None:
                break
            sources.append(value)
            chain_ops.extend(path)
        if len(sources) != 3 or len({value.name for value in sources}) != 1:
            continue
        projection = producers.get(sources[0].name)
        if projection is None or projection.name != "kernel.b200.norm_linear" or \
                projection.attributes.get("epilogue") or "packed" not in projection.attributes or \
                len(users.get(projection.results[0].name, [])) != 3 or \
                value_dtype(projection.results[0]) != "bf16":
            continue
        offsets = [decode_attribute_static(op.attributes["args"]) for op in chain_ops
                   if op.name == "runtime.view.slice"]
        widths = projection.attributes["packed"]
        expected_offsets = [(0, widths[0]), (widths[0], widths[0] + widths[1]),
                            (widths[0] + widths[1], sum(widths))]
        if [tuple(item[2:4]) for item in offsets] != expected_offsets:
            continue
        # the context leaves as B x 1 x (Hq D) through transpose(1, 2) + reshape
        context = attention.results[0]
        transpose = _single_user(users, context)
        reshape = _single_user(users, transpose.results[0]) if transpose is not None and \
            transpose.name == "runtime.view.transpose" else None
        if reshape is None or reshape.name not in ("runtime.view.reshape", "runtime.view.view"):
            continue
        head_dim = store.attributes.get("head_dim")
        q_heads = _static_extent(store.operands[1], 1)
        kv_heads = _static_extent(store.operands[2], 1)
        if not isinstance(head_dim, int) or q_heads is None or kv_heads is None or \
                widths != [q_heads * head_dim, kv_heads * head_dim, kv_heads * head_dim]:
            continue
        attributes = {
            "slot": int(attention.attributes.get("slot", 0)), "groups": attention.attributes["groups"],
            "scale": attention.attributes["scale"], "head_dim": head_dim, "q_heads": q_heads,
            "kv_heads": kv_heads, "has_bias": bool(projection.attributes.get("has_bias")),
            "epsilon": projection.attributes.get("epsilon"),
            "round_before_weight": projection.attributes.get("round_before_weight", False),
            "input_features": projection.attributes.get("input_features"),
            "output_features": projection.attributes.get("output_features"),
            "numerical_mode": "fast", "length_offset": 0, "zero_mask": mask.name,
            "lowered_from": "kernel.b200.norm_linear+kernel.b200.rope_kv_store+runtime.kv.advance+"
                            "kernel.b200.decode_attention",
        }
        merged = Operation(
            "kernel.b200.qkv_decode_attention",
            [store.operands[0]] + list(projection.operands) + [store.operands[4], store.operands[5],
                                                               attention.operands[2]],
            [reshape.results[0], advance.results[0]], attributes)
        operations = function.block.operations
        position = operations.index(reshape)
        operations[position] = merged
        for op in [projection, store, advance, attention, transpose] + chain_ops:
            operations.remove(op)
        fused += 1
    return fused


def take_last_token_logits(function) -> int:
    """Prefill graphs return logits for every position (qwen2.py:418-424) although a serving
    loop samples from the last one only. Where the caller opts in, the hidden rows are cut to the
    last position in front of the final norm (or, if that is not a single-use rms_norm, in front
    of the LM head): `runtime.view.last_token` [x] -> x[:, -1:, :], a view. The first result of
    the function becomes B x 1 x V. Returns 1 if the graph was rewritten."""

    if not function.returns:
        return 0
    producers = _producer_map(function)
    users = _users(function)
    head = producers.get(function.returns[0].name)
    if head is None or head.name not in ("kernel.b200.linear", "kernel.b200.norm_linear") or \
            (head.attributes.get("epilogue") or "none") != "none":
        return 0
    chain = [head]
    if head.name == "kernel.b200.linear":
        norm = producers.get(head.operands[0].name)
        if norm is not None and norm.name == "kernel.b200.rms_norm" and \
                _single_user(users, norm.results[0]) is head:
            chain.insert(0, norm)
    hidden = chain[0].operands[0]
    match = _DIMS.match(str(hidden.type))
    if not match or len(_split_dims(match.group(1))) != 3 or _static_extent(hidden, 1) == 1:
        return 0
    last = Value(_fresh(function, "last_token"), retype(hidden, 1, 1))
    view = Operation("runtime.view.last_token", [hidden], [last],
                     {"axis": 1, "lowered_from": "last-token logits"})
    operations = function.block.operations
    operations.insert(operations.index(chain[0]), view)
    chain[0].operands[0] = last
    for operation in chain:  # B x T x * becomes B x 1 x * down to the returned logits
        for result in operation.results:
            result.type = retype(result, 1, 1)
    for value in function.returns:
        if value.name == head.results[0].name:
            value.type = head.results[0].type
    return 1


def decode_attribute_static(tree):
    """The importer's argument tree with SSA references left as their names."""
    if isinstance(tree, dict):
        if set(tree) == {"ssa"}:
            return tree["ssa"]
        if set(tree) == {"tuple"}:
            return tuple(decode_attribute_static(item) for item in tree["tuple"])
        return {key: decode_attribute_static(item) for key, item in tree.items()}
    if isinstance(tree, list):
        return [decode_attribute_static(item) for item in tree]
    return tree


def hoist_kv_advances(function) -> int:
    """When every layer slot is advanced by exactly one fused attention op, the per-slot length
    updates move into ONE `runtime.kv.advance_all` at the end of the function (one launch over
    the state's length arena instead of one per layer): the fused ops get `length_offset: 1`
    (their lengths are still the ones before the new token) and hand the state on unchanged."""

    fused = [op for op in function.block.operations if op.name == "kernel.b200.qkv_decode_attention"]
    others = [op for op in function.block.operations
              if op.name in ("runtime.kv.advance", "runtime.kv.length", "kernel.b200.decode_attention",
                             "kernel.b200.kv_store", "kernel.b200.rope_kv_store",
                             "kernel.b200.kv_prefill_store")]
    if not fused or others:
        return 0
    slots = sorted(int(op.attributes["slot"]) for op in fused)
    if slots != list(range(len(fused))) or any(op.attributes.get("length_offset") for op in fused):
        return 0
    from .contracts import KVStateT, parse_type

    state_type = parse_type(fused[0].operands[0].type)
    if not isinstance(state_type, KVStateT) or state_type.layers != len(fused):
        return 0
    last = max(fused, key=lambda op: function.block.operations.index(op))
    final_state = last.results[1]
    if not any(value is final_state or value.name == final_state.name for value in function.returns):
        return 0
    for op in fused:
        op.attributes["length_offset"] = 1
    carried = Value(_fresh(function, "kv_state_steps"), str(final_state.type))
    last.results = [last.results[0], carried]
    function.block.operations.append(Operation(
        "runtime.kv.advance_all", [carried], [final_state],
        {"delta": 1, "slots": len(fused), "lowered_from": "runtime.kv.advance x%d" % len(fused)}))
    return len(fused)
