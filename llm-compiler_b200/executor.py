"""KernelIR executor for the B200 target: same contract as the reference's GPU executor
(`TritonExecutor.run(module, arguments, function_name=None) -> ExecutionResult`,
backends/triton_executor.py:42-130 on top of execution.py:530-579), every op executed by a
kernel of libb200serve.so or by host metadata — there is nothing to fall back to.

`strict=True` (the default here; the reference defaults to False) checks the whole graph
before the first op runs, exactly like `require_full_lowering` upstream, and raises
LoweringCoverageError for anything `kernel_ir.lower_to_b200` did not lower. The run is free
of host synchronisation and of allocations other than torch.empty outputs, so a caller may
capture it in a CUDA graph once shapes are fixed.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from . import kernels
from .contracts import SymbolError, bind_symbols
from .dispatch_plan import resolve_dispatch_plan, split_tokens_of
from .kernel_ir import decode_attribute, require_full_lowering, value_dtype, value_rank
from .kv_state import ExecutionError, PagedKVCacheState, PreallocatedKVCacheState

_DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16,
           "i64": torch.int64, "i32": torch.int32, "i1": torch.bool}


@dataclass
class ExecutionResult:
    outputs: Tuple[Any, ...]
    executed_operations: Tuple[str, ...]
    symbolic_dimensions: Dict[str, int]


def _select_function(module, function_name: Optional[str]):
    if function_name is None:
        if len(module.functions) != 1:
            raise ExecutionError("the module holds several functions: pass function_name")
        return module.functions[0]
    for function in module.functions:
        if function.name == function_name:
            return function
    raise ExecutionError(f"no function @{function_name}")


def _as_state(value: Any) -> PreallocatedKVCacheState:
    """Accepts this package's state or any object with the reference's fields
    (keys, values, lengths, capacity, generation): wrapped without copying."""

    if isinstance(value, PreallocatedKVCacheState):
        return value
    if all(hasattr(value, name) for name in ("keys", "values", "lengths", "capacity")):
        return PreallocatedKVCacheState(tuple(value.keys), tuple(value.values),
                                        tuple(value.lengths), int(value.capacity),
                                        int(getattr(value, "generation", 0)))
    raise ExecutionError("expected a PreallocatedKVCacheState")


def bind_arguments(function, weights: Dict[str, torch.Tensor], inputs: Dict[str, Any]) -> List[Any]:
    """Positional argument list for `function` from named values: the counterpart, for modules
    that travel as JSON, of bind_exported_program_arguments / bind_stateful_decode_arguments
    (execution.py:908-1004), which need the ExportedProgram. `inputs` maps user input names
    (input_ids, attention_mask, position_ids, kv_state, inv_freq) to values; parameters are
    matched by their state_dict name with '.' flattened to '_' (the exporter's
    `p_model_<flattened name>` convention); a buffer ending in `inv_freq` takes inputs["inv_freq"]."""

    flattened = sorted(((name.replace(".", "_"), tensor) for name, tensor in weights.items()),
                       key=lambda item: -len(item[0]))
    arguments = []
    for declared in function.block.arguments:
        name = declared.name.lstrip("%")
        if name in inputs:
            arguments.append(inputs[name])
        elif name.endswith("inv_freq") and "inv_freq" in inputs:
            arguments.append(inputs["inv_freq"])
        else:
            for flat, tensor in flattened:
                if name.endswith(flat):
                    arguments.append(tensor)
                    break
            else:
                raise ExecutionError(f"no value for graph argument {declared.name}")
    return arguments


class B200Executor:
    """`classify_masks`: prefill attention whose graph attribute is still `causal: "mask"` has
    its mask tensor checked on the device once per tensor (one host read, skipped under graph
    capture); a mask proved causal takes the mask-free tcgen05 kernel, anything else the
    general additive-mask kernel."""

    def __init__(self, *, strict: bool = True, classify_masks: bool = True) -> None:
        self.strict = strict
        self.classify_masks = classify_masks
        self.lowering_trace: List[Dict[str, Any]] = []
        self._constants: Dict[Any, Any] = {}  # weight-preparation results, by operand storage
        # Row sums of squares that a cluster split-K projection left beside its output during the
        # current run, by the output's address: (output, squares). The output is held here, so
        # its memory cannot be handed to another tensor while the entry exists.
        self._row_squares: Dict[int, Any] = {}
        self._handlers = {
            "kernel.b200.rms_norm": self._rms_norm,
            "kernel.b200.linear": self._linear,
            "kernel.b200.rope": self._rope,
            "kernel.b200.rope_table": self._rope_table,
            "kernel.b200.prefill_attention": self._prefill_attention,
            "kernel.b200.decode_attention": self._decode_attention,
            "kernel.b200.kv_store": self._kv_store,
            "kernel.b200.kv_prefill_store": self._kv_prefill_store,
            "kernel.b200.embedding": self._embedding,
            "kernel.b200.rope_kv_store": self._rope_kv_store,
            "kernel.b200.scale_columns": lambda o, a, e: kernels.b200_scale_columns(o[0], o[1]),
            "kernel.b200.norm_linear": self._norm_linear,
            "kernel.b200.qkv_decode_attention": self._qkv_decode_attention,
            "runtime.kv.advance_all": lambda o, a, e: _as_state(o[0]).advance_all(
                delta=int(a.get("delta", 1)), slots=a.get("slots")),
            "kernel.b200.pack_rows": lambda o, a, e: kernels.b200_pack_rows(*o),
            "kernel.b200.interleave_rows": lambda o, a, e: kernels.interleave_gate_up(o[0], o[1]),
            "runtime.view.slice": self._slice,
            "runtime.view.last_token": self._last_token,
            "kernel.b200.swiglu": lambda o, a, e: kernels.b200_swiglu(o[0], o[1]),
            "kernel.b200.add": lambda o, a, e: kernels.b200_add(o[0], o[1]),
            "kernel.b200.contiguous": self._contiguous,
            "kernel.b200.cast": self._cast,
            "runtime.kv.init": self._kv_init,
            "runtime.kv.length": lambda o, a, e: _as_state(o[0]).positions(int(a.get("slot", 0))),
            "runtime.kv.advance": lambda o, a, e: _as_state(o[0]).advance(
                int(a.get("slot", 0)), delta=int(a.get("delta", 1))),
            "runtime.view.view": self._view,
            "runtime.view.reshape": self._view,
            "runtime.view.transpose": self._transpose,
            "runtime.view.unsqueeze": self._unsqueeze,
            "runtime.view.sym_size": self._sym_size,
        }

    # ------------------------------------------------------------------ run ----
    def run(self, module, arguments: Sequence[Any], *,
            function_name: Optional[str] = None) -> ExecutionResult:
        if self.strict:
            require_full_lowering(module)  # before any op runs (triton_executor.py:60-62)
        function = _select_function(module, function_name)
        if len(arguments) != len(function.block.arguments):
            raise ExecutionError(
                f"@{function.name} takes {len(function.block.arguments)} arguments, "
                f"got {len(arguments)}")
        environment: Dict[str, Any] = {}
        for declared, runtime_value in zip(function.block.arguments, arguments):
            self._validate_argument(declared, runtime_value)
            environment[declared.name] = runtime_value
        try:  # symbol equality and the exporter's value ranges (execution.py:1323-1347)
            symbols = bind_symbols(function.block.arguments, arguments)
        except SymbolError as error:
            raise ExecutionError(str(error)) from error
        trace = []
        self._row_squares.clear()
        for operation in function.block.operations:
            handler = self._handlers.get(operation.name)
            if handler is None:
                raise ExecutionError(
                    f"the B200 executor has no kernel for {operation.name}: run "
                    "kernel_ir.lower_to_b200 on the module first (there is no eager fallback)")
            operands = [environment[value.name] for value in operation.operands]
            if operation.attributes.get("constant") is True:
                results = self._constant(operation, handler, operands, environment)
            else:
                results = handler(operands, operation.attributes, environment)
            expected = len(operation.results)
            if expected == 1:
                results = (results,)
            elif expected == 0:
                results = ()
            elif not isinstance(results, (tuple, list)) or len(results) != expected:
                raise ExecutionError(f"{operation.name} must produce {expected} results")
            for declared, runtime_value in zip(operation.results, results):
                environment[declared.name] = runtime_value
            trace.append(operation.name)
        self._row_squares.clear()
        outputs = tuple(environment[value.name] for value in function.returns)
        return ExecutionResult(outputs, tuple(trace), symbols)

    def _constant(self, operation, handler, operands, environment):
        """Weight-preparation ops (`constant: true`) depend on graph parameters only: evaluated
        once per set of weight tensors (same storage, same version) and kept."""

        key = (operation.name, operation.results[0].name,
               tuple((t.data_ptr(), tuple(t.shape), t._version) for t in operands))
        if key not in self._constants:
            if torch.cuda.is_current_stream_capturing():
                raise ExecutionError(
                    f"{operation.name} prepares weights: run the module once before capturing it")
            self._constants[key] = handler(operands, operation.attributes, environment)
        return self._constants[key]

    @staticmethod
    def _validate_argument(declared, runtime_value) -> None:
        dtype = value_dtype(declared)
        if dtype is None:
            return
        if not isinstance(runtime_value, torch.Tensor):
            raise ExecutionError(f"argument {declared.name} must be a tensor")
        if not runtime_value.is_cuda:
            raise ExecutionError(f"argument {declared.name} must live on a CUDA device")
        expected = _DTYPES.get(dtype)
        if expected is not None and runtime_value.dtype != expected:
            raise ExecutionError(f"argument {declared.name}: dtype {runtime_value.dtype}, "
                                 f"expected {expected}")
        rank = value_rank(declared)
        if rank is not None and runtime_value.ndim != rank:
            raise ExecutionError(f"argument {declared.name}: rank {runtime_value.ndim}, "
                                 f"expected {rank}")

    # ------------------------------------------------------------- kernel ops ----
    def _rms_norm(self, operands, attributes, environment):
        if len(operands) != 2:
            raise ExecutionError("rms_norm takes input and weight")
        mode = attributes.get("numerical_mode", "fast")
        rows = operands[0].numel() // operands[0].shape[-1]
        self.lowering_trace.append({"backend": "b200", "source": "kernel_ir", "rows": rows,
                                    "numerical_mode": mode})
        return kernels.b200_rms_norm(
            operands[0], operands[1], epsilon=float(attributes["epsilon"]),
            output_dtype=attributes.get("output_dtype"),
            round_before_weight=bool(attributes.get("round_before_weight", False)),
            numerical_mode=mode)

    def _decide(self, op: str, attributes, value: int, plan_key: str = "lowering_plan",
                family_key: Optional[int] = None):
        """Resolves the operation's profile-guided plan with the run-time value of its bucketed
        dimension and records the decision in lowering_trace (the reference records
        backend / source / rows for serve.rms_norm, backends/triton_executor.py:299-308)."""

        plan = attributes.get(plan_key)
        if plan_key == "lowering_plans" and isinstance(plan, dict):
            # one plan per profiled batch size: the nearest one on a log scale
            sizes = [int(k) for k in plan if k.isdigit()]
            plan = plan[str(min(sizes, key=lambda b: abs(math.log(b / max(family_key, 1)))))] \
                if sizes and family_key else None
        decision = resolve_dispatch_plan(plan, max(int(value), 1))
        self.lowering_trace.append({"backend": "b200", "op": op, "source": decision.source,
                                    "variant": decision.variant, "value": int(value),
                                    "profile_value": decision.profile_value})
        return decision.variant

    def _linear(self, operands, attributes, environment):
        has_bias = bool(attributes.get("has_bias"))
        epilogue = attributes.get("epilogue") or "none"
        expected = 2 + int(has_bias) + int(epilogue == "residual")
        if len(operands) != expected:
            raise ExecutionError("linear: has_bias / epilogue disagree with the operand count")
        tensor, weight = operands[0], operands[1]
        bias = operands[2] if has_bias else None
        residual = operands[-1] if epilogue == "residual" else None
        rows = tensor.numel() // tensor.shape[-1]
        variant = self._decide("linear", attributes, rows) if "lowering_plan" in attributes else None
        if epilogue == "residual" and bias is None and variant is None and \
                tensor.dtype == torch.bfloat16 and rows <= 256 and weight.shape[0] % 4 == 0:
            # few N tiles at decode sizes: the cluster split-K projection that adds the residual
            # itself (same rounding points as the plain kernel's residual epilogue)
            chain = rows <= self._chain_rows(weight)  # a folded RMSNorm may follow: leave it the row squares
            flat = kernels.b200_linear_splitk_residual(
                tensor.reshape(rows, tensor.shape[-1]), weight, residual.reshape(rows, weight.shape[0]),
                row_squares=chain)
            if chain:
                flat, squares = flat
                if squares is not None:
                    self._row_squares[flat.data_ptr()] = (flat, squares)
            return flat.view(residual.shape)
        with kernels.kernel_variants(linear=variant):
            return kernels.b200_linear(tensor, weight, bias, residual=residual, epilogue=epilogue)

    # The decode chain (fusion.fuse_norm_linear / fuse_qkv_attention): up to this many rows the
    # folded-norm kernels run (one or two rows per idle-warp thread); beyond, the same ops are
    # executed as their unfused kernels.
    CHAIN_ROWS = 128

    def _chain_rows(self, weight) -> int:
        return min(self.CHAIN_ROWS, kernels.decode_chain_rows(weight))

    def _norm_linear(self, operands, attributes, environment):
        has_bias = bool(attributes.get("has_bias"))
        if len(operands) != 4 + int(has_bias):
            raise ExecutionError("norm_linear takes input, norm weight, weight, folded weight and optional bias")
        tensor, norm_weight, weight, folded = operands[:4]
        bias = operands[4] if has_bias else None
        epilogue = attributes.get("epilogue") or "none"
        epsilon = float(attributes["epsilon"])
        rows = tensor.numel() // tensor.shape[-1]
        self.lowering_trace.append({"backend": "b200", "op": "norm_linear", "rows": rows,
                                    "folded": rows <= self._chain_rows(weight)})
        if rows <= self._chain_rows(weight) and tensor.dtype == torch.bfloat16:
            rows_2d = tensor.reshape(rows, tensor.shape[-1])
            left = self._row_squares.get(rows_2d.data_ptr())
            squares = None
            if left is not None and left[0].shape == rows_2d.shape and left[1].shape[1] == rows:
                squares = left[1]  # what the projection that produced these rows left
            flat = kernels.b200_linear_rms_input(rows_2d, folded, bias, epsilon=epsilon,
                                                 epilogue=epilogue, row_squares=squares)
            return flat.view(*tensor.shape[:-1], flat.shape[-1])
        normed = kernels.b200_rms_norm(tensor, norm_weight, epsilon=epsilon,
                                       round_before_weight=bool(attributes.get("round_before_weight")),
                                       numerical_mode=attributes.get("numerical_mode", "fast"))
        return kernels.b200_linear(normed, weight, bias, epilogue=epilogue)

    def _qkv_decode_attention(self, operands, attributes, environment):
        has_bias = bool(attributes.get("has_bias"))
        if len(operands) != 8 + int(has_bias):
            raise ExecutionError("qkv_decode_attention takes state, input, norm weight, weight, folded "
                                 "weight, optional bias, cosine, sine and mask")
        state = _as_state(operands[0])
        tensor, norm_weight, weight, folded = operands[1:5]
        bias = operands[5] if has_bias else None
        cosine, sine, mask = operands[-3:]
        slot = int(attributes.get("slot", 0))
        q_heads, kv_heads, dim = (int(attributes[name]) for name in ("q_heads", "kv_heads", "head_dim"))
        epsilon, scale = float(attributes["epsilon"]), float(attributes["scale"])
        offset = int(attributes.get("length_offset", 0))
        rows = tensor.numel() // tensor.shape[-1]
        if isinstance(state, PagedKVCacheState):
            return self._qkv_decode_attention_paged(state, slot, tensor, norm_weight, weight, folded, bias,
                                                    cosine, sine, mask, q_heads, kv_heads, dim, epsilon,
                                                    scale, offset, attributes)
        key_buffer, value_buffer, lengths = state._slot(slot)
        if key_buffer.shape[0] != rows or key_buffer.shape[2] != kv_heads or key_buffer.shape[3] != dim:
            raise ExecutionError("qkv_decode_attention: the KV state does not match batch, heads or head_dim")
        bound = mask.shape[-1] if mask is not None else state.capacity
        if bound > state.capacity:
            raise ExecutionError("decode attention mask is longer than the KV capacity")
        self.lowering_trace.append({"backend": "b200", "op": "qkv_decode_attention", "rows": rows,
                                    "fused": rows <= self._chain_rows(weight), "length_offset": offset})
        if rows <= self._chain_rows(weight) and tensor.dtype == torch.bfloat16:
            flat = tensor.reshape(rows, tensor.shape[-1])
            partials, squares = kernels.b200_linear_partial(flat, folded, row_squares=True)
            if offset == 0:  # the graph advances this slot here: lengths then count the new token
                state = state.advance(slot, delta=1)
            split = kernels._profiled_split_tokens(rows, q_heads, kv_heads, dim, tensor.dtype, bound)
            context = kernels.b200_qkv_decode_attention(
                partials, bias, cosine, sine, key_buffer, value_buffer, lengths, q_heads=q_heads,
                scale=scale, split_tokens=split, max_length_hint=bound, length_offset=offset,
                norm_row_squares=squares, norm_hidden=flat.shape[1], norm_epsilon=epsilon)
            return context.view(rows, 1, q_heads * dim), state
        # more rows than the fused kernels take: the same ops, one kernel each
        normed = kernels.b200_rms_norm(tensor, norm_weight, epsilon=epsilon,
                                       round_before_weight=bool(attributes.get("round_before_weight")),
                                       numerical_mode="fast")
        qkv = kernels.b200_linear(normed, weight, bias).view(rows, q_heads + 2 * kv_heads, dim)
        query = kernels.b200_rope_kv_store(qkv[:, :q_heads], qkv[:, q_heads:q_heads + kv_heads],
                                           qkv[:, q_heads + kv_heads:], cosine, sine, key_buffer,
                                           value_buffer, lengths)
        if offset == 0:
            state = state.advance(slot, delta=1)
            attention_lengths = lengths
        else:  # the advance is deferred to the end of the step: attend over lengths + 1
            attention_lengths = torch.empty_like(lengths)
            attention_lengths.copy_(lengths)
            kernels.b200_advance_lengths(attention_lengths, 1, state.capacity)
        context = kernels.b200_decode_attention(query, key_buffer, value_buffer, attention_lengths, mask,
                                                scale=scale, max_length_hint=bound)
        return context.view(rows, 1, q_heads * dim), state

    @staticmethod
    def _rope(operands, attributes, environment):
        if len(operands) != 4:
            raise ExecutionError("rope takes query, key, cosine and sine")
        if operands[0].shape[-1] != int(attributes["head_dim"]):
            raise ExecutionError("rope: head_dim does not match the attribute")
        return kernels.b200_rope(*operands)

    @staticmethod
    def _rope_table(operands, attributes, environment):
        positions, inv_freq = operands
        dtype = _DTYPES[attributes["dtype"]]
        return kernels.b200_rope_table(positions, inv_freq.reshape(-1), dtype)

    def _prefill_attention(self, operands, attributes, environment):
        if len(operands) != 4:
            raise ExecutionError("prefill_attention takes q, k, v and mask")
        query, key, value, mask = operands
        if query.shape[1] != key.shape[1] * int(attributes["groups"]):
            raise ExecutionError("prefill_attention: GQA groups mismatch")
        variant = self._decide("prefill_attention", attributes, query.shape[2]) \
            if "lowering_plan" in attributes else None
        causal = attributes.get("causal") is True
        proof = attributes.get("causal_proof") if causal else None
        if not causal and self.classify_masks and mask is not None and \
                not torch.cuda.is_current_stream_capturing():
            causal = kernels.b200_mask_is_causal(mask)
            proof = "classified" if causal else None
        self.lowering_trace.append({"backend": "b200", "op": "prefill_attention.mask",
                                    "causal": causal, "proof": proof})
        with kernels.kernel_variants(prefill_attention=variant):
            return kernels.b200_prefill_attention(
                query, key, value, None if causal else mask, scale=float(attributes["scale"]),
                causal=causal, numerical_mode=attributes.get("numerical_mode", "fast"))

    def _decode_attention(self, operands, attributes, environment):
        if len(operands) != 3:
            raise ExecutionError("decode_attention takes state, query and mask")
        state = _as_state(operands[0])
        options = {}
        if "lowering_plans" in attributes:
            # bucketed by the context bound the host knows: the mask length (or the capacity)
            bound = operands[2].shape[-1] if operands[2] is not None else state.capacity
            variant = self._decide("decode_attention", attributes, bound, "lowering_plans",
                                   operands[1].shape[0])
            options["split_tokens"] = split_tokens_of(variant)
        return state.decode_attention(
            int(attributes.get("slot", 0)), operands[1], operands[2],
            groups=int(attributes["groups"]), scale=float(attributes["scale"]),
            numerical_mode=attributes.get("numerical_mode", "fast"), **options)

    @staticmethod
    def _kv_store(operands, attributes, environment):
        if len(operands) != 4:
            raise ExecutionError("kv_store takes state, key, value and positions")
        state = _as_state(operands[0])
        return state.store(int(attributes.get("slot", 0)), operands[1], operands[2], operands[3])

    @staticmethod
    def _rope_kv_store(operands, attributes, environment):
        if len(operands) != 6:
            raise ExecutionError("rope_kv_store takes state, query, key, value, cosine and sine")
        state = _as_state(operands[0])
        query, key, value, cosine, sine = operands[1:]
        if query.shape[-1] != int(attributes["head_dim"]):
            raise ExecutionError("rope_kv_store: head_dim does not match the attribute")
        slot = int(attributes.get("slot", 0))
        if isinstance(state, PagedKVCacheState):  # paged storage: rotate, then store through the table
            rotated, rotated_key = kernels.b200_rope(query, key, cosine, sine)
            return rotated, state.store(slot, rotated_key, value, state.positions(slot))
        key_buffer, value_buffer, positions = state._slot(slot)
        rotated = kernels.b200_rope_kv_store(query, key, value, cosine, sine, key_buffer,
                                             value_buffer, positions)
        return rotated, state

    def _qkv_decode_attention_paged(self, state, slot, tensor, norm_weight, weight, folded, bias, cosine,
                                    sine, mask, q_heads, kv_heads, dim, epsilon, scale, offset, attributes):
        """The fused decode-layer op on a paged state: up to CHAIN_ROWS bf16 rows the same two
        launches as on the contiguous layout, through the block table; beyond, the same ops one
        kernel each through the state's own store / attention methods."""

        rows = tensor.numel() // tensor.shape[-1]
        bound = mask.shape[-1] if mask is not None else state.capacity
        if bound > state.capacity:
            raise ExecutionError("decode attention mask is longer than the KV capacity")
        self.lowering_trace.append({"backend": "b200", "op": "qkv_decode_attention", "rows": rows,
                                    "fused": rows <= self._chain_rows(weight), "length_offset": offset,
                                    "layout": "paged"})
        if rows <= self._chain_rows(weight) and tensor.dtype == torch.bfloat16:
            flat = tensor.reshape(rows, tensor.shape[-1])
            partials, squares = kernels.b200_linear_partial(flat, folded, row_squares=True)
            pool_key, pool_value, lengths = state._slot(slot)
            if offset == 0:  # the graph advances this slot here: lengths then count the new token
                state = state.advance(slot, delta=1)
            context = kernels.b200_paged_qkv_decode_attention(
                partials, bias, cosine, sine, pool_key, pool_value, state.block_table, lengths,
                q_heads=q_heads, scale=scale, max_length_hint=bound, length_offset=offset,
                norm_row_squares=squares, norm_hidden=flat.shape[1], norm_epsilon=epsilon)
            return context.view(rows, 1, q_heads * dim), state
        normed = kernels.b200_rms_norm(tensor, norm_weight, epsilon=epsilon,
                                       round_before_weight=bool(attributes.get("round_before_weight")),
                                       numerical_mode="fast")
        qkv = kernels.b200_linear(normed, weight, bias).view(rows, 1, q_heads + 2 * kv_heads, dim)
        query = qkv[:, :, :q_heads].transpose(1, 2)
        key = qkv[:, :, q_heads:q_heads + kv_heads].transpose(1, 2)
        value = qkv[:, :, q_heads + kv_heads:].transpose(1, 2)
        query, key = kernels.b200_rope(query, key, cosine, sine)
        state.store(slot, key, value, state.positions(slot))
        lengths = state.positions(slot)
        if offset == 0:
            state = state.advance(slot, delta=1)
            attention_state = state
        else:  # the advance is deferred to the end of the step: attend over lengths + 1
            attention_lengths = torch.empty_like(lengths)
            attention_lengths.copy_(lengths)
            kernels.b200_advance_lengths(attention_lengths, 1, state.capacity)
            attention_state = state._derive(state.generation)
            object.__setattr__(attention_state, "lengths",
                               tuple(attention_lengths if i == slot else l for i, l in enumerate(state.lengths)))
        context = attention_state.decode_attention(slot, query, mask, groups=q_heads // kv_heads, scale=scale)
        return context.view(rows, 1, q_heads * dim), state

    @staticmethod
    def _slice(operands, attributes, environment):
        tensor, axis, start, stop = decode_attribute(attributes["args"], environment)
        return tensor.narrow(int(axis), int(start), int(stop) - int(start))

    @staticmethod
    def _last_token(operands, attributes, environment):
        if len(operands) != 1 or operands[0].ndim < 2:
            raise ExecutionError("last_token takes one tensor of rank 2 or more")
        axis = int(attributes.get("axis", 1))
        return operands[0].narrow(axis, operands[0].shape[axis] - 1, 1)

    @staticmethod
    def _kv_prefill_store(operands, attributes, environment):
        if len(operands) != 3:
            raise ExecutionError("kv_prefill_store takes state, key and value")
        state = _as_state(operands[0])
        return state.prefill_store(int(attributes.get("slot", 0)), operands[1], operands[2])

    @staticmethod
    def _kv_init(operands, attributes, environment):
        if len(operands) != 1 or not isinstance(operands[0], torch.Tensor):
            raise ExecutionError("kv.init takes one key tensor as its template")
        return PreallocatedKVCacheState.empty_from_key_template(
            operands[0], num_layers=int(attributes["num_layers"]),
            capacity=int(attributes["capacity"]))

    @staticmethod
    def _embedding(operands, attributes, environment):
        table, ids = operands
        return kernels.b200_embedding(table, ids)

    @staticmethod
    def _contiguous(operands, attributes, environment):
        tensor = operands[0]
        return tensor if tensor.is_contiguous() else kernels.b200_contiguous(tensor)

    @staticmethod
    def _cast(operands, attributes, environment):
        args = decode_attribute(attributes["args"], environment)
        tensor, dtype = args[0], _DTYPES[args[1]]
        if tensor.dtype == dtype:
            return tensor
        floats = (torch.float32, torch.bfloat16, torch.float16)
        if tensor.dtype not in floats or dtype not in floats:
            raise ExecutionError(f"no B200 kernel casts {tensor.dtype} to {dtype}")
        return kernels.b200_contiguous(tensor, dtype)

    # ------------------------------------------------------------ metadata ops ----
    @staticmethod
    def _view(operands, attributes, environment):
        tensor, shape = decode_attribute(attributes["args"], environment)
        shape = [int(extent) for extent in shape]
        try:
            return tensor.view(shape)
        except RuntimeError:
            # strides do not allow a view: densify with the library's own copy kernel
            return kernels.b200_contiguous(tensor).view(shape)

    @staticmethod
    def _transpose(operands, attributes, environment):
        tensor, first, second = decode_attribute(attributes["args"], environment)
        return tensor.transpose(int(first), int(second))

    @staticmethod
    def _unsqueeze(operands, attributes, environment):
        tensor, axis = decode_attribute(attributes["args"], environment)
        return tensor.unsqueeze(int(axis))

    @staticmethod
    def _sym_size(operands, attributes, environment):
        tensor, axis = decode_attribute(attributes["args"], environment)
        return int(tensor.shape[int(axis)])
