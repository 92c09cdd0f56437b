"""Per-operation contracts of the B200 KernelIR dialect and the run-time symbol guards.

The reference verifier checks, by operation name, the shape / dtype / bias / GQA-group contracts
of its serving ops (ir.py:462-534 linear, 537-609 prefill attention, 612-678 rope, 681-742
decode attention, 745-835 KV ops) and its executor binds every symbolic dimension of the graph
signature to the run-time extent, enforcing equality between uses and the exporter's value
ranges (execution.py:1095-1135, 1323-1360). Those checks name `serve.*` / `kernel.triton.*` ops
only; this module applies the same contracts to the `kernel.b200.*` / `runtime.*` ops that
`kernel_ir.lower_to_b200` produces, on the type strings the graphs carry (so it works on modules
loaded from JSON as well as on the reference's own Module objects).

One deliberate difference: the device recorded in a type is not enforced. The graphs are
exported on a CPU ("tensor<..., cpu>") and executed on CUDA tensors; the executor requires CUDA
tensors for every tensor argument instead.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple, Union

_TENSOR = re.compile(r"^tensor<(.*)x([a-z]+\d*), *([^>]+)>$")
_KV_STATE = re.compile(r"^!serve\.kv_state<(.*)>$")
_SYMBOL = re.compile(r"^(.*?)<(VR\[.*\])>$")
_BOUNDS = re.compile(r"VR\[(-?\d+),\s*(-?\d+|int_oo)\]")

Dim = Union[int, str]  # static extent, or the symbol text ("s13<VR[1, 8]>", "s11 + 1<VR[2, 64]>")


@dataclass(frozen=True)
class TensorT:
    shape: Tuple[Dim, ...]
    dtype: str
    device: str

    @property
    def rank(self) -> int:
        return len(self.shape)


@dataclass(frozen=True)
class KVStateT:
    dtype: str
    layers: int
    heads: int
    head_dim: int
    layout: str
    capacity: Optional[int]


def _split_dims(text: str) -> List[str]:
    parts, depth, current = [], 0, ""
    for char in text:
        if char in "<[":
            depth += 1
        elif char in ">]":
            depth -= 1
        if char == "x" and depth == 0:
            parts.append(current)
            current = ""
        else:
            current += char
    parts.append(current)
    return parts


def parse_type(type_: Any) -> Union[TensorT, KVStateT, None]:
    """TensorT / KVStateT of a value type (a type string or the reference's type object)."""

    text = str(type_)
    match = _TENSOR.match(text)
    if match:
        dims: List[Dim] = []
        for part in _split_dims(match.group(1)):
            part = part.strip()
            dims.append(int(part) if re.fullmatch(r"\d+", part) else part)
        return TensorT(tuple(dims), match.group(2), match.group(3).strip())
    match = _KV_STATE.match(text)
    if match:
        fields = [item.strip() for item in match.group(1).split(",")]
        named = dict(item.split("=", 1) for item in fields[1:] if "=" in item)
        capacity = named.get("capacity")
        return KVStateT(fields[0], int(named.get("layers", 0)), int(named.get("heads", 0)),
                        int(named.get("head_dim", 0)), named.get("layout", ""),
                        int(capacity) if capacity and capacity.isdigit() else None)
    return None


def symbol_of(dim: Dim) -> Optional[Tuple[str, Optional[int], Optional[int]]]:
    """(name, lower, upper) of a symbolic dimension; None for a static one. Derived symbols
    ("s11 + 1") are named by their whole expression: equal text means equal extent."""

    if isinstance(dim, int):
        return None
    match = _SYMBOL.match(dim)
    name, bounds = (match.group(1), match.group(2)) if match else (dim, None)
    lower = upper = None
    if bounds:
        found = _BOUNDS.fullmatch(bounds)
        if found:
            lower = int(found.group(1))
            upper = None if found.group(2) == "int_oo" else int(found.group(2))
    return name.strip(), lower, upper


# ------------------------------------------------------------------ per-op contracts ----
class _Check:
    def __init__(self, function_name: str, index: int, operation) -> None:
        self.prefix = f"@{function_name} op {index} {operation.name}"
        self.operation = operation
        self.errors: List[str] = []

    def fail(self, message: str) -> None:
        self.errors.append(f"{self.prefix}: {message}")

    def tensors(self, values: Sequence[Any], what: str) -> Optional[List[TensorT]]:
        types = [parse_type(value.type) for value in values]
        if not all(isinstance(type_, TensorT) for type_ in types):
            self.fail(f"{what} must all be tensors")
            return None
        return types  # type: ignore[return-value]

    def state(self, value) -> Optional[KVStateT]:
        type_ = parse_type(value.type)
        if not isinstance(type_, KVStateT):
            self.fail("the first operand must be the KV state")
            return None
        return type_

    def slot(self, state: KVStateT) -> None:
        slot = self.operation.attributes.get("slot", 0)
        if not isinstance(slot, int) or slot < 0 or (state.layers and slot >= state.layers):
            self.fail(f"slot {slot!r} outside the state's {state.layers} layers")


def _same(*types: TensorT) -> bool:
    return len({type_.dtype for type_ in types}) == 1


def _linear(c: _Check) -> None:
    op = c.operation
    attributes = op.attributes
    epilogue = attributes.get("epilogue") or "none"
    if epilogue not in ("none", "residual", "swiglu"):
        c.fail(f"unknown epilogue {epilogue!r}")
        return
    has_bias = attributes.get("has_bias")
    expected = 2 + int(bool(has_bias)) + int(epilogue == "residual")
    if len(op.operands) != expected or len(op.results) != 1:
        c.fail("has_bias / epilogue disagree with the operand count (input, weight, [bias], [residual])")
        return
    types = c.tensors(list(op.operands) + list(op.results), "input, weight, bias, residual and result")
    if types is None:
        return
    input_t, weight_t, result_t = types[0], types[1], types[-1]
    if input_t.rank not in (2, 3):
        c.fail("the input must have rank 2 or 3")
        return
    if weight_t.rank != 2:
        c.fail("the weight must be an N x K matrix")
        return
    if result_t.rank != input_t.rank:
        c.fail("the result rank must equal the input rank")
        return
    n, k = weight_t.shape
    out = n // 2 if epilogue == "swiglu" and isinstance(n, int) else n
    if epilogue == "swiglu" and (not isinstance(n, int) or n % 2):
        c.fail("a SwiGLU epilogue needs an even static N (gate and up rows interleaved)")
    if input_t.shape[-1] != k:
        c.fail("the last input dimension must equal the weight's K")
    if result_t.shape[:-1] != input_t.shape[:-1]:
        c.fail("the leading result dimensions must equal the input's")
    if result_t.shape[-1] != out:
        c.fail("the last result dimension must equal the weight's N (N / 2 with SwiGLU)")
    if not _same(input_t, weight_t, result_t):
        c.fail("input, weight and result must share one dtype")
    if has_bias:
        bias_t = types[2]
        if bias_t.shape != (n,) or bias_t.dtype != input_t.dtype:
            c.fail("the bias must be a vector of N elements in the input dtype")
    if epilogue == "residual" and types[-2] != result_t:
        c.fail("the residual must have the result's type")
    for name, dim in (("input_features", k), ("output_features", n)):
        if not isinstance(dim, int) or attributes.get(name) != dim:
            c.fail(f"the {name} attribute does not match the weight")


def _attention_common(c: _Check, query: TensorT, kv_heads: Any, head_dim: Any) -> None:
    attributes = c.operation.attributes
    groups = attributes.get("groups")
    if not isinstance(groups, int) or groups <= 0 or not isinstance(query.shape[1], int) or \
            not isinstance(kv_heads, int) or query.shape[1] != kv_heads * groups:
        c.fail("query heads must equal KV heads x groups (static)")
    if query.shape[3] != head_dim:
        c.fail("head_dim of the query and of K / V differ")
    scale = attributes.get("scale")
    if not isinstance(scale, (int, float)) or isinstance(scale, bool) or float(scale) <= 0:
        c.fail("scale must be a positive number")


def _prefill_attention(c: _Check) -> None:
    op = c.operation
    if len(op.operands) != 4 or len(op.results) != 1:
        c.fail("takes query, key, value, mask and returns the context")
        return
    types = c.tensors(list(op.operands) + list(op.results), "operands and result")
    if types is None:
        return
    query, key, value, mask, context = types
    if any(type_.rank != 4 for type_ in types):
        c.fail("every tensor must have rank 4")
        return
    _attention_common(c, query, key.shape[1], key.shape[3])
    if key != value:
        c.fail("key and value must have one type")
    tokens = query.shape[2]
    if not (query.shape[0] == key.shape[0] == mask.shape[0] and tokens == key.shape[2] and
            tokens == mask.shape[2] == mask.shape[3]):
        c.fail("batch or token extents of query, key and mask differ")
    if mask.shape[1] != 1:
        c.fail("the mask's head dimension must be 1")
    if context != query:
        c.fail("the context must have the query's type")
    if query.dtype != key.dtype:
        c.fail("query and key / value must share one dtype")
    if op.attributes.get("causal") not in (True, "mask"):
        c.fail('causal must be true (proved) or "mask" (taken from the operand)')


def _decode_attention(c: _Check) -> None:
    op = c.operation
    if len(op.operands) != 3 or len(op.results) != 1:
        c.fail("takes state, query, mask and returns the context")
        return
    state = c.state(op.operands[0])
    types = c.tensors([op.operands[1], op.operands[2], op.results[0]], "query, mask and context")
    if state is None or types is None:
        return
    query, mask, context = types
    c.slot(state)
    if state.layout != "contiguous_bshd":
        c.fail("only the contiguous_bshd KV layout is supported")
    if query.rank != 4 or query.shape[2] != 1:
        c.fail("the query must be B x H x 1 x D")
        return
    if mask.rank != 4 or mask.shape[1] != 1 or mask.shape[2] != 1:
        c.fail("the mask must be B x 1 x 1 x S")
    elif mask.shape[0] != query.shape[0]:
        c.fail("mask and query batch differ")
    _attention_common(c, query, state.heads, state.head_dim)
    if context != query:
        c.fail("the context must have the query's type")


def _rope_shapes(c: _Check, query: TensorT, key: TensorT, cosine: TensorT, sine: TensorT) -> None:
    if query.rank != 4 or key.rank != 4:
        c.fail("query and key must be B x H x T x D")
        return
    if cosine.rank != 3 or sine.rank != 3:
        c.fail("cosine and sine must be B x T x D")
        return
    head_dim = query.shape[3]
    if not (query.shape[0] == key.shape[0] and query.shape[2:] == key.shape[2:] and
            cosine.shape == (query.shape[0], query.shape[2], head_dim) and sine == cosine):
        c.fail("batch, token or head_dim extents differ")
    if not _same(query, key, cosine):
        c.fail("query, key, cosine and sine must share one dtype")
    if not isinstance(head_dim, int) or head_dim <= 0 or head_dim % 2 or \
            c.operation.attributes.get("head_dim") != head_dim:
        c.fail("head_dim must be static, even and equal to the attribute")


def _rope(c: _Check) -> None:
    op = c.operation
    if len(op.operands) != 4 or len(op.results) != 2:
        c.fail("takes query, key, cosine, sine and returns two tensors")
        return
    types = c.tensors(list(op.operands) + list(op.results), "operands and results")
    if types is None:
        return
    query, key, cosine, sine, out_query, out_key = types
    _rope_shapes(c, query, key, cosine, sine)
    if out_query != query or out_key != key:
        c.fail("the results must have the types of query and key")
    if op.attributes.get("variant", "qwen2_half_rotation") != "qwen2_half_rotation":
        c.fail("only the qwen2_half_rotation variant is supported")


def _kv_tensor(c: _Check, tensor: TensorT, state: KVStateT, what: str) -> None:
    if tensor.rank != 4:
        c.fail(f"{what} must be B x H x T x D")
        return
    if tensor.shape[1] != state.heads or tensor.shape[3] != state.head_dim:
        c.fail(f"{what} heads / head_dim do not match the KV state")
    if tensor.dtype != state.dtype:
        c.fail(f"{what} dtype does not match the KV state")


def _kv_store(c: _Check) -> None:
    op = c.operation
    prefill = op.name.endswith("prefill_store")
    if len(op.operands) != (3 if prefill else 4) or len(op.results) != 1:
        c.fail("takes state, key, value" + ("" if prefill else ", positions") + " and returns the state")
        return
    state = c.state(op.operands[0])
    types = c.tensors(op.operands[1:], "key, value and positions")
    if state is None or types is None:
        return
    c.slot(state)
    _kv_tensor(c, types[0], state, "key")
    _kv_tensor(c, types[1], state, "value")
    if types[0] != types[1]:
        c.fail("key and value must have one type")
    if not prefill:
        positions = types[2]
        if positions.rank != 1 or positions.dtype != "i64" or positions.shape[0] != types[0].shape[0]:
            c.fail("positions must be an int64 vector of the batch size")
    if not isinstance(parse_type(op.results[0].type), KVStateT):
        c.fail("the result must be the KV state")


def _rope_kv_store(c: _Check) -> None:
    op = c.operation
    if len(op.operands) != 6 or len(op.results) != 2:
        c.fail("takes state, query, key, value, cosine, sine and returns the rotated query and the state")
        return
    state = c.state(op.operands[0])
    types = c.tensors(list(op.operands[1:]) + [op.results[0]], "query, key, value, cosine, sine and result")
    if state is None or types is None:
        return
    query, key, value, cosine, sine, out_query = types
    c.slot(state)
    _rope_shapes(c, query, key, cosine, sine)
    _kv_tensor(c, key, state, "key")
    _kv_tensor(c, value, state, "value")
    if query.rank == 4 and query.shape[2] != 1:
        c.fail("the fused rope + store handles one token per sequence")
    if out_query != query:
        c.fail("the first result must have the query's type")
    if not isinstance(parse_type(op.results[1].type), KVStateT):
        c.fail("the second result must be the KV state")


def _rms_norm(c: _Check) -> None:
    op = c.operation
    if len(op.operands) != 2 or len(op.results) != 1:
        c.fail("takes input, weight and returns one tensor")
        return
    types = c.tensors(list(op.operands) + list(op.results), "input, weight and result")
    if types is None:
        return
    input_t, weight_t, result_t = types
    if weight_t.rank != 1 or input_t.rank < 1 or weight_t.shape[0] != input_t.shape[-1]:
        c.fail("the weight must be a vector of the input's last dimension")
    if result_t.shape != input_t.shape:
        c.fail("the result must have the input's shape")
    epsilon = op.attributes.get("epsilon")
    if not isinstance(epsilon, (int, float)) or isinstance(epsilon, bool) or float(epsilon) < 0:
        c.fail("epsilon must be a non-negative number")
    if op.attributes.get("axis", -1) not in (-1, input_t.rank - 1):
        c.fail("only the last axis is normalised")
    wanted = op.attributes.get("output_dtype")
    if wanted is not None and wanted != result_t.dtype:
        c.fail("output_dtype does not match the result type")


def _kv_runtime(c: _Check) -> None:
    op = c.operation
    if op.name == "runtime.kv.init":
        if not isinstance(op.attributes.get("num_layers"), int) or op.attributes["num_layers"] <= 0 or \
                not isinstance(op.attributes.get("capacity"), int) or op.attributes["capacity"] <= 0:
            c.fail("num_layers and capacity must be positive integers")
        return
    if not op.operands:
        c.fail("takes the KV state")
        return
    state = c.state(op.operands[0])
    if state is None:
        return
    c.slot(state)
    if op.name == "runtime.kv.advance":
        delta = op.attributes.get("delta", 1)
        if not isinstance(delta, int) or delta <= 0:
            c.fail("delta must be a positive integer")
    if op.name == "runtime.kv.length":
        types = c.tensors(op.results, "the result")
        if types is not None and (types[0].rank != 1 or types[0].dtype != "i64"):
            c.fail("the result must be an int64 vector")


def _embedding(c: _Check) -> None:
    op = c.operation
    if len(op.operands) != 2 or len(op.results) != 1:
        c.fail("takes table, ids and returns one tensor")
        return
    types = c.tensors(list(op.operands) + list(op.results), "table, ids and result")
    if types is None:
        return
    table, ids, result = types
    if table.rank != 2 or ids.dtype != "i64":
        c.fail("needs a V x H table and int64 ids")
    elif result.shape != ids.shape + (table.shape[1],) or result.dtype != table.dtype:
        c.fail("the result must be ids.shape + [H] in the table's dtype")


def _rope_table(c: _Check) -> None:
    op = c.operation
    if len(op.operands) != 2 or len(op.results) != 2:
        c.fail("takes position ids, inverse frequencies and returns cosine and sine")
        return
    types = c.tensors(list(op.operands) + list(op.results), "operands and results")
    if types is None:
        return
    positions, inv_freq, cosine, sine = types
    if positions.dtype != "i64" or positions.rank != 2:
        c.fail("position ids must be a B x T int64 tensor")
    if inv_freq.dtype != "f32":
        c.fail("inverse frequencies must be fp32")
    if cosine != sine or cosine.rank != 3 or cosine.dtype != op.attributes.get("dtype"):
        c.fail("cosine and sine must be one B x T x D type in the attribute's dtype")
    elif positions.rank == 2 and cosine.shape[:2] != positions.shape:
        c.fail("cosine / sine batch and token extents must equal the position ids'")


def _elementwise(c: _Check) -> None:
    op = c.operation
    types = c.tensors(list(op.operands) + list(op.results), "operands and result")
    if types is None or len(op.operands) != 2 or len(op.results) != 1:
        if types is not None:
            c.fail("takes two tensors and returns one")
        return
    if not (types[0] == types[1] == types[2]):
        c.fail("both operands and the result must have one type")


def _pack(c: _Check) -> None:
    op = c.operation
    types = c.tensors(list(op.operands) + list(op.results), "operands and result")
    if types is None or len(op.results) != 1 or len(op.operands) < 2:
        return
    rows = [type_.shape[0] for type_ in types[:-1]]
    if not all(isinstance(row, int) for row in rows) or types[-1].shape[0] != sum(rows):
        c.fail("the result's first dimension must be the sum of the operands' (static)")
    if any(type_.shape[1:] != types[0].shape[1:] or type_.dtype != types[0].dtype for type_ in types):
        c.fail("operands and result must agree on dtype and trailing dimensions")
    if op.name.endswith("interleave_rows") and (len(op.operands) != 2 or rows[0] != rows[1]):
        c.fail("interleaves exactly two matrices of one shape")


def _norm_linear(c: _Check) -> None:
    op = c.operation
    has_bias = bool(op.attributes.get("has_bias"))
    if len(op.operands) != 4 + int(has_bias) or len(op.results) != 1:
        c.fail("takes input, norm weight, weight, folded weight, optional bias and returns one tensor")
        return
    types = c.tensors(list(op.operands) + list(op.results), "operands and result")
    if types is None:
        return
    input_t, norm_t, weight_t, folded_t, result_t = types[0], types[1], types[2], types[3], types[-1]
    epilogue = op.attributes.get("epilogue") or "none"
    if epilogue not in ("none", "swiglu"):
        c.fail("the epilogue must be none or swiglu")
    if weight_t.rank != 2 or folded_t != weight_t:
        c.fail("the folded weight must have the weight's N x K type")
        return
    n, k = weight_t.shape
    if norm_t.shape != (k,) or input_t.shape[-1] != k:
        c.fail("the norm weight and the input's last dimension must equal the weight's K")
    out = n // 2 if epilogue == "swiglu" and isinstance(n, int) else n
    if result_t.shape != input_t.shape[:-1] + (out,):
        c.fail("the result must be the input's leading dimensions x N (N / 2 with SwiGLU)")
    if has_bias and types[4].shape != (n,):
        c.fail("the bias must be a vector of N elements")
    epsilon = op.attributes.get("epsilon")
    if not isinstance(epsilon, (int, float)) or isinstance(epsilon, bool) or float(epsilon) < 0:
        c.fail("epsilon must be a non-negative number")
    if not _same(input_t, norm_t, weight_t, result_t):
        c.fail("input, norm weight, weight and result must share one dtype")


def _qkv_decode_attention(c: _Check) -> None:
    op = c.operation
    attributes = op.attributes
    has_bias = bool(attributes.get("has_bias"))
    if len(op.operands) != 8 + int(has_bias) or len(op.results) != 2:
        c.fail("takes state, input, norm weight, weight, folded weight, optional bias, cosine, sine, "
               "mask and returns the context and the state")
        return
    state = c.state(op.operands[0])
    types = c.tensors(list(op.operands[1:]) + [op.results[0]], "tensor operands and the context")
    if state is None or types is None:
        return
    c.slot(state)
    input_t, norm_t, weight_t, context = types[0], types[1], types[2], types[-1]
    q_heads, kv_heads, dim = (attributes.get(name) for name in ("q_heads", "kv_heads", "head_dim"))
    if not all(isinstance(value, int) and value > 0 for value in (q_heads, kv_heads, dim)):
        c.fail("q_heads, kv_heads and head_dim must be positive integers")
        return
    if kv_heads != state.heads or dim != state.head_dim or q_heads != kv_heads * attributes.get("groups", 0):
        c.fail("heads / head_dim / groups do not match the KV state")
    if weight_t.rank != 2 or weight_t.shape[0] != (q_heads + 2 * kv_heads) * dim or \
            weight_t.shape[1] != input_t.shape[-1] or norm_t.shape != (weight_t.shape[1],):
        c.fail("the packed q|k|v weight must be (Hq + 2 Hkv) D x K with K the input's last dimension")
    if context.shape[-1] != q_heads * dim or context.shape[0] != input_t.shape[0]:
        c.fail("the context must be B x 1 x (Hq D)")
    scale = attributes.get("scale")
    if not isinstance(scale, (int, float)) or isinstance(scale, bool) or float(scale) <= 0:
        c.fail("scale must be a positive number")
    if attributes.get("length_offset", 0) not in (0, 1):
        c.fail("length_offset must be 0 or 1")
    if not isinstance(parse_type(op.results[1].type), KVStateT):
        c.fail("the second result must be the KV state")


def _advance_all(c: _Check) -> None:
    op = c.operation
    state = c.state(op.operands[0]) if op.operands else None
    if state is None:
        return
    delta, slots = op.attributes.get("delta", 1), op.attributes.get("slots", state.layers)
    if not isinstance(delta, int) or delta <= 0:
        c.fail("delta must be a positive integer")
    if not isinstance(slots, int) or slots <= 0 or (state.layers and slots > state.layers):
        c.fail("slots must lie in 1 .. the state's layers")


_CONTRACTS = {
    "kernel.b200.norm_linear": _norm_linear,
    "kernel.b200.qkv_decode_attention": _qkv_decode_attention,
    "runtime.kv.advance_all": _advance_all,
    "kernel.b200.scale_columns": lambda c: None if len(c.operation.operands) == 2 else c.fail(
        "takes the weight and the column scales"),
    "kernel.b200.linear": _linear,
    "kernel.b200.prefill_attention": _prefill_attention,
    "kernel.b200.decode_attention": _decode_attention,
    "kernel.b200.rope": _rope,
    "kernel.b200.rope_kv_store": _rope_kv_store,
    "kernel.b200.kv_store": _kv_store,
    "kernel.b200.kv_prefill_store": _kv_store,
    "kernel.b200.rms_norm": _rms_norm,
    "kernel.b200.embedding": _embedding,
    "kernel.b200.rope_table": _rope_table,
    "kernel.b200.swiglu": _elementwise,
    "kernel.b200.add": _elementwise,
    "kernel.b200.pack_rows": _pack,
    "kernel.b200.interleave_rows": _pack,
    "runtime.view.last_token": lambda c: None if len(c.operation.operands) == 1 and
    len(c.operation.results) == 1 else c.fail("takes one tensor and yields one view"),
    "runtime.kv.init": _kv_runtime,
    "runtime.kv.length": _kv_runtime,
    "runtime.kv.advance": _kv_runtime,
}


def operation_contract_errors(module) -> List[str]:
    """Every violated contract of the module's kernel.b200.* / runtime.kv.* operations."""

    errors: List[str] = []
    for function in module.functions:
        for index, operation in enumerate(function.block.operations):
            contract = _CONTRACTS.get(operation.name)
            if contract is None:
                continue
            check = _Check(function.name, index, operation)
            contract(check)
            errors.extend(check.errors)
    return errors


# ------------------------------------------------------------------ run-time guards ----
class SymbolError(ValueError):
    """A run-time extent violates a symbolic dimension's equality or range constraint."""


def bind_symbols(declared_arguments, runtime_values) -> Dict[str, int]:
    """Binds the symbolic dimensions of a function signature to the run-time extents of its
    tensor arguments (execution.py:1323-1347): a symbol must have one extent wherever it is
    used, inside the exporter's value range; static dimensions must match exactly."""

    symbols: Dict[str, int] = {}
    for declared, value in zip(declared_arguments, runtime_values):
        type_ = parse_type(declared.type)
        if not isinstance(type_, TensorT) or not hasattr(value, "shape"):
            continue
        if len(value.shape) != type_.rank:
            raise SymbolError(f"argument {declared.name}: rank {len(value.shape)}, expected {type_.rank}")
        for axis, (actual, dim) in enumerate(zip(value.shape, type_.shape)):
            actual = int(actual)
            symbol = symbol_of(dim)
            if symbol is None:
                if actual != dim:
                    raise SymbolError(f"argument {declared.name}: dimension {axis} is {actual}, "
                                      f"the graph fixes it at {dim}")
                continue
            name, lower, upper = symbol
            known = symbols.get(name)
            if known is not None and known != actual:
                raise SymbolError(f"argument {declared.name}: dimension {axis} = {actual} breaks the "
                                  f"equality of symbol {name} (bound to {known} before)")
            if lower is not None and actual < lower:
                raise SymbolError(f"argument {declared.name}: {name} = {actual} is below the "
                                  f"exporter's lower bound {lower}")
            if upper is not None and actual > upper:
                raise SymbolError(f"argument {declared.name}: {name} = {actual} is above the "
                                  f"exporter's upper bound {upper}")
            symbols[name] = actual
    return symbols
