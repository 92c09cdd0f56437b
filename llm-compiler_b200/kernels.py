"""Python wrappers over the C ABI, one per kernel wrapper of the reference backend.

Names, argument order and error behaviour follow the reference's Triton wrappers
(backends/__init__.py:3-19): precondition failures raise ValueError before anything is
launched; outputs are allocated with torch.empty on the inputs' device; kernels launch on
torch's current stream and never synchronise, so every call is legal under CUDA graph
capture. PyTorch is used for memory and streams only: all arithmetic runs in
libb200serve.so, and a missing library or a CPU tensor is an error, never a fallback.
"""

from __future__ import annotations

import contextlib
import math
from typing import Optional, Tuple

import torch

from . import _lib

# (fp16 runs on the generic CUDA-core kernels: the reference's kernels accept it,
# backends/triton_linear.py:100-105, and no benchmark configuration uses it)
_DTYPE_CODES = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.float16: _lib.F16}
_MODES = {"fast": _lib.MODE_FAST, "pytorch_compatible": _lib.MODE_PYTORCH_COMPATIBLE}
_EPILOGUES = {"none": _lib.EPILOGUE_NONE, "residual": _lib.EPILOGUE_RESIDUAL,
              "swiglu": _lib.EPILOGUE_SWIGLU}


class KernelStatusError(RuntimeError):
    """A kernel flagged a device-side error (KV overflow, bad token id, ...)."""


# --------------------------------------------------------------------------- runtime ----
class DeviceRuntime:
    """Per-device scratch owned by Python: the int32 status word and named workspaces.

    Workspaces only grow; they are zero-filled when (re)allocated because the split-K
    linear kernel keeps tile counters there that must start at zero (it leaves them at
    zero after every call). A workspace that is outgrown is retired, never freed: a CUDA
    graph captured earlier has its address baked into its launches, and a replay must keep
    finding memory that nothing else owns (with its counters still at zero). Growth is
    geometric, so the retired buffers of a name sum to less than the live one.
    """

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self._workspaces: dict[str, torch.Tensor] = {}
        self._retired: list[torch.Tensor] = []
        self.launches = 0

    def workspace(self, name: str, nbytes: int) -> Optional[torch.Tensor]:
        if nbytes <= 0:
            return None
        current = self._workspaces.get(name)
        if current is None or current.numel() < nbytes:
            if current is not None:
                self._retired.append(current)
                nbytes = max(int(nbytes), 2 * current.numel())
            current = torch.zeros(int(nbytes), dtype=torch.uint8, device=self.device)
            self._workspaces[name] = current
        return current

    def reserve(self, name: str, nbytes: int) -> None:
        """Pre-sizes a workspace (call before CUDA graph capture)."""

        self.workspace(name, nbytes)

    def check_status(self) -> None:
        """Host read of the status word (synchronises); raises and clears on error."""

        value = int(self.status.item())
        if value == 0:
            return
        self.status.zero_()
        reasons = []
        if value & _lib.STATUS_KV_OVERFLOW:
            reasons.append("KV position beyond capacity (write skipped / length clamped)")
        if value & _lib.STATUS_LENGTH_OVER_MASK:
            reasons.append("KV length above the attention mask length (clamped)")
        if value & _lib.STATUS_BAD_TOKEN_ID:
            reasons.append("token id outside the vocabulary (row zeroed)")
        if value & _lib.STATUS_BAD_POSITION:
            reasons.append("negative KV position (write skipped)")
        if value & _lib.STATUS_WAIT_TIMEOUT:
            reasons.append("a bounded in-kernel wait gave up (result invalid)")
        raise KernelStatusError("; ".join(reasons) or f"status word {value}")


_RUNTIMES: dict[int, DeviceRuntime] = {}


def runtime(device: torch.device | None = None) -> DeviceRuntime:
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    index = device.index if device.index is not None else torch.cuda.current_device()
    found = _RUNTIMES.get(index)
    if found is None:
        found = DeviceRuntime(torch.device("cuda", index))
        _RUNTIMES[index] = found
    return found


def launch_count(device: torch.device | None = None) -> int:
    return runtime(device).launches


# ------------------------------------------------------------------------- helpers ----
@contextlib.contextmanager
def launch_mode(*, programmatic: bool, constant_weights: bool = False,
                stable_kv_prefix: bool = False):
    """Scope in which the decode-chain kernels are launched with programmatic dependent launch
    (each may become resident while its predecessor still runs and waits on the device before
    touching a tensor). constant_weights promises that no kernel in flight writes a weight
    tensor, which lets the tcgen05 linear fetch weight tiles before that wait; stable_kv_prefix
    promises the same for lengths[] and every KV row below lengths[b] - 1, which lets decode
    attention fill its pipeline before the wait. The mode belongs to the calling thread (the
    library keeps it thread-local: engines on other threads are not affected); launches captured
    into a CUDA graph keep the mode they were captured with."""

    flags = (_lib.LAUNCH_PROGRAMMATIC if programmatic else 0) | \
        (_lib.LAUNCH_CONSTANT_WEIGHTS if constant_weights else 0) | \
        (_lib.LAUNCH_STABLE_KV_PREFIX if stable_kv_prefix else 0)
    library = _lib.load()
    previous = library.b200_set_launch_mode(flags)
    if previous < 0:
        raise ValueError(f"b200_set_launch_mode: {_lib.error_string(previous)}")
    try:
        yield
    finally:
        library.b200_set_launch_mode(previous)


@contextlib.contextmanager
def kernel_variants(*, linear: Optional[str] = None, prefill_attention: Optional[str] = None):
    """Scope in which b200_linear / b200_prefill_attention use the named variant ("tcgen05" or
    "mma.sync"; None leaves the library's own choice): how a resolved dispatch plan reaches the
    library. Other launch-mode flags are kept."""

    for name, value in (("linear", linear), ("prefill_attention", prefill_attention)):
        if value not in (None, "tcgen05", "mma.sync"):
            raise ValueError(f"unknown {name} variant {value!r}")
    library = _lib.load()
    previous = library.b200_get_launch_mode()
    flags = previous & ~(_lib.LAUNCH_LINEAR_WARP_LEVEL | _lib.LAUNCH_PREFILL_WARP_LEVEL)
    if linear == "mma.sync":
        flags |= _lib.LAUNCH_LINEAR_WARP_LEVEL
    if prefill_attention == "mma.sync":
        flags |= _lib.LAUNCH_PREFILL_WARP_LEVEL
    library.b200_set_launch_mode(flags)
    try:
        yield
    finally:
        library.b200_set_launch_mode(previous)


def _guard_current_device(device: torch.device) -> None:
    """The C ABI launches on the calling thread's current device and on its current stream;
    operands that live on another GPU would be dereferenced by the wrong GPU (an illegal
    address without peer access, a silent NVLink detour with it). Refused before any launch."""

    current = torch.cuda.current_device()
    if device.index is not None and device.index != current:
        raise ValueError(
            f"operands live on cuda:{device.index} but the current device is cuda:{current}: "
            "call under torch.cuda.device(...) of the operands' GPU")


def _require_cuda(*tensors: torch.Tensor) -> torch.device:
    device = None
    for tensor in tensors:
        if tensor is None:
            continue
        if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
            raise ValueError("the B200 backend only runs CUDA tensors (there is no CPU fallback)")
        if device is None:
            device = tensor.device
        elif tensor.device != device:
            raise ValueError("all operands must live on the same CUDA device")
    assert device is not None
    _guard_current_device(device)
    return device


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODES[dtype]
    except KeyError as error:
        raise ValueError(f"unsupported dtype {dtype}: the B200 backend runs f32, bf16 and f16") from error


def _mode(numerical_mode: str) -> int:
    try:
        return _MODES[numerical_mode]
    except KeyError as error:
        raise ValueError(f"unknown numerical mode {numerical_mode!r}") from error


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(code: int, what: str) -> None:
    if code == 0:
        return
    message = f"{what}: {_lib.error_string(code)}"
    if code in (_lib.ERR_LAUNCH,):
        raise RuntimeError(message)
    raise ValueError(message)


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    return None if tensor is None else tensor.data_ptr()


def _count(rt: DeviceRuntime, launches: int = 1) -> None:
    rt.launches += launches


def _dense(tensor: torch.Tensor) -> torch.Tensor:
    """Contiguous version of a floating-point tensor, copied by this library's own kernel."""

    if tensor.is_contiguous():
        return tensor
    return b200_contiguous(tensor)


def _dense_index(tensor: torch.Tensor, what: str) -> torch.Tensor:
    if not tensor.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    return tensor


# ------------------------------------------------------------------------ KV store ----
def b200_kv_store(key_buffer: torch.Tensor, value_buffer: torch.Tensor, key: torch.Tensor,
                  value: torch.Tensor, positions: torch.Tensor) -> None:
    """buf[b, positions[b]+t, h, :] = x[b, h, t, :] for K and V, in place, one launch.

    Mirrors triton_kv_store (backends/triton_kv.py:71-129).
    """

    device = _require_cuda(key_buffer, value_buffer, key, value, positions)
    if key_buffer.ndim != 4 or key_buffer.shape != value_buffer.shape:
        raise ValueError("KV buffers must be B x C x H x D tensors of one shape")
    if key.ndim != 4 or key.shape != value.shape:
        raise ValueError("key/value must be B x H x T x D tensors of one shape")
    batch, capacity, heads, dim = key_buffer.shape
    if key.shape[0] != batch or key.shape[1] != heads or key.shape[3] != dim:
        raise ValueError("key/value batch, heads or head_dim do not match the KV buffers")
    if not key_buffer.is_contiguous() or not value_buffer.is_contiguous():
        raise ValueError("KV buffers must be contiguous")
    if len({key_buffer.dtype, value_buffer.dtype, key.dtype, value.dtype}) != 1:
        raise ValueError("KV buffers and key/value must share one dtype")
    if positions.shape != (batch,) or positions.dtype != torch.int64:
        raise ValueError("positions must be a one-dimensional int64 batch tensor")
    positions = _dense_index(positions, "positions")
    rt = runtime(device)
    tokens = key.shape[2]
    code = _lib.load().b200_kv_store(
        key_buffer.data_ptr(), value_buffer.data_ptr(), key.data_ptr(), value.data_ptr(),
        positions.data_ptr(), batch, capacity, heads, tokens, dim,
        _lib.i64_array(key.stride()), _lib.i64_array(value.stride()), _code(key.dtype),
        rt.status.data_ptr(), _stream())
    _check(code, "b200_kv_store")
    _count(rt)


# ---------------------------------------------------------------------------- RoPE ----
def b200_rope(query: torch.Tensor, key: torch.Tensor, cosine: torch.Tensor,
              sine: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Qwen2 half-rotation RoPE on Q and K in one launch; returns new contiguous tensors.

    Mirrors triton_rope (backends/triton_rope.py:299-390).
    """

    device = _require_cuda(query, key, cosine, sine)
    if query.ndim != 4 or key.ndim != 4:
        raise ValueError("query/key must be B x H x T x D")
    batch, q_heads, tokens, dim = query.shape
    if key.shape[0] != batch or key.shape[2] != tokens or key.shape[3] != dim:
        raise ValueError("query and key disagree on batch, tokens or head_dim")
    if dim % 2:
        raise ValueError("head_dim must be even")
    if cosine.shape != (batch, tokens, dim) or sine.shape != (batch, tokens, dim):
        raise ValueError("cosine/sine must be B x T x D")
    if len({query.dtype, key.dtype, cosine.dtype, sine.dtype}) != 1:
        raise ValueError("query, key, cosine and sine must share one dtype")
    kv_heads = key.shape[1]
    query_out = torch.empty((batch, q_heads, tokens, dim), dtype=query.dtype, device=device)
    key_out = torch.empty((batch, kv_heads, tokens, dim), dtype=key.dtype, device=device)
    rt = runtime(device)
    code = _lib.load().b200_rope(
        query.data_ptr(), key.data_ptr(), cosine.data_ptr(), sine.data_ptr(),
        query_out.data_ptr(), key_out.data_ptr(), batch, q_heads, kv_heads, tokens, dim,
        _lib.i64_array(query.stride()), _lib.i64_array(key.stride()),
        _lib.i64_array(cosine.stride()), _lib.i64_array(sine.stride()), _code(query.dtype),
        _stream())
    _check(code, "b200_rope")
    _count(rt)
    return query_out, key_out


def b200_rope_kv_store(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                       cosine: torch.Tensor, sine: torch.Tensor, key_buffer: torch.Tensor,
                       value_buffer: torch.Tensor, positions: torch.Tensor,
                       query_out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Decode fusion (T == 1): rope(q) -> query_out, rope(k) and v -> KV buffers at positions.

    query/key/value are B x H x 1 x D (or B x H x D) views with a contiguous last dim;
    cosine/sine are B x 1 x D. Returns the rotated query, B x Hq x 1 x D contiguous.
    """

    device = _require_cuda(query, key, value, cosine, sine, key_buffer, value_buffer, positions)

    def squeeze(tensor: torch.Tensor) -> torch.Tensor:
        if tensor.ndim == 4:
            if tensor.shape[2] != 1:
                raise ValueError("the fused rope + store kernel handles one token per sequence")
            return tensor[:, :, 0, :]
        return tensor

    q3, k3, v3 = squeeze(query), squeeze(key), squeeze(value)
    batch, q_heads, dim = q3.shape
    kv_heads = k3.shape[1]
    if k3.shape != (batch, kv_heads, dim) or v3.shape != (batch, kv_heads, dim):
        raise ValueError("key/value must be B x Hkv x D")
    if key_buffer.shape != value_buffer.shape or key_buffer.shape[0] != batch or \
            key_buffer.shape[2] != kv_heads or key_buffer.shape[3] != dim:
        raise ValueError("KV buffers do not match key/value")
    cos2 = cosine.reshape(batch, dim) if cosine.ndim == 3 else cosine
    sin2 = sine.reshape(batch, dim) if sine.ndim == 3 else sine
    if cos2.stride() != sin2.stride():
        sin2 = _dense(sin2)
        cos2 = _dense(cos2)
    for tensor in (q3, k3, v3, cos2, sin2):
        if tensor.stride(-1) != 1:
            raise ValueError("last dimension must be contiguous")
    if positions.shape != (batch,) or positions.dtype != torch.int64:
        raise ValueError("positions must be a one-dimensional int64 batch tensor")
    if query_out is None:
        query_out = torch.empty((batch, q_heads, 1, dim), dtype=query.dtype, device=device)
    rt = runtime(device)
    code = _lib.load().b200_rope_kv_store(
        q3.data_ptr(), k3.data_ptr(), v3.data_ptr(), cos2.data_ptr(), sin2.data_ptr(),
        query_out.data_ptr(), key_buffer.data_ptr(), value_buffer.data_ptr(),
        positions.data_ptr(), batch, q_heads, kv_heads, dim, key_buffer.shape[1],
        q3.stride(0), q3.stride(1), k3.stride(0), k3.stride(1), v3.stride(0), v3.stride(1),
        cos2.stride(0), _code(query.dtype), rt.status.data_ptr(), _stream())
    _check(code, "b200_rope_kv_store")
    _count(rt)
    return query_out


def b200_rope_table(position_ids: torch.Tensor, inv_freq: torch.Tensor,
                    dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables B x T x D from int64 position ids and fp32 inverse frequencies.

    Replaces the eager to/unsqueeze/mul/cat/cos/sin chain of Qwen2RotaryEmbedding.forward
    (qwen2.py:136-149).
    """

    device = _require_cuda(position_ids, inv_freq)
    if position_ids.dtype != torch.int64 or position_ids.ndim != 2:
        raise ValueError("position_ids must be a B x T int64 tensor")
    if inv_freq.dtype != torch.float32 or inv_freq.ndim != 1:
        raise ValueError("inv_freq must be a one-dimensional fp32 tensor")
    position_ids = _dense_index(position_ids, "position_ids")
    inv_freq = _dense(inv_freq)
    batch, tokens = position_ids.shape
    half = inv_freq.shape[0]
    cosine = torch.empty((batch, tokens, 2 * half), dtype=dtype, device=device)
    sine = torch.empty_like(cosine)
    rt = runtime(device)
    code = _lib.load().b200_rope_table(position_ids.data_ptr(), inv_freq.data_ptr(),
                                       cosine.data_ptr(), sine.data_ptr(), batch * tokens, half,
                                       _code(dtype), _stream())
    _check(code, "b200_rope_table")
    _count(rt)
    return cosine, sine


# ------------------------------------------------------------------------- RMSNorm ----
def b200_rms_norm(tensor: torch.Tensor, weight: torch.Tensor, *, epsilon: float,
                  output_dtype=None, round_before_weight: bool = False,
                  numerical_mode: str = "fast") -> torch.Tensor:
    """RMSNorm over the last dimension. Mirrors triton_rms_norm
    (backends/triton_rmsnorm.py:205-443); `pytorch_compatible` reproduces the CPU
    executor's result bit for bit (execution.py:686-692)."""

    device = _require_cuda(tensor, weight)
    hidden = tensor.shape[-1]
    if weight.shape != (hidden,):
        raise ValueError("weight must be a vector of the hidden size")
    out_dtype = _resolve_dtype(output_dtype, tensor.dtype)
    if not (tensor.dtype == weight.dtype == out_dtype):
        raise ValueError("input, weight and output dtype must agree")
    if tensor.is_contiguous():
        source, row_stride = tensor, hidden
    elif tensor.ndim == 2 and tensor.stride(1) == 1 and tensor.stride(0) >= hidden:
        source, row_stride = tensor, tensor.stride(0)
    else:
        source, row_stride = _dense(tensor), hidden
    rows = source.numel() // hidden if hidden else 0
    weight = _dense(weight)
    output = torch.empty(tensor.shape, dtype=out_dtype, device=device)
    rt = runtime(device)
    code = _lib.load().b200_rms_norm(
        source.data_ptr(), weight.data_ptr(), output.data_ptr(), rows, hidden, row_stride,
        float(epsilon), int(bool(round_before_weight)), _code(tensor.dtype), _code(weight.dtype),
        _code(out_dtype), _mode(numerical_mode), _stream())
    _check(code, "b200_rms_norm")
    _count(rt)
    return output


def _resolve_dtype(value, default: torch.dtype) -> torch.dtype:
    if value is None:
        return default
    if isinstance(value, torch.dtype):
        return value
    names = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}
    if value not in names:
        raise ValueError(f"unsupported output dtype {value!r}")
    return names[value]


# ---------------------------------------------------------------- decode attention ----
_packaged_plans: dict = {}


def _profiled_split_tokens(batch: int, q_heads: int, kv_heads: int, dim: int, dtype: torch.dtype,
                           context_bound: int) -> int:
    """Split size of decode attention from the packaged dispatch profile: the plan of the
    nearest profiled batch size (log scale) for this head layout, resolved with the context
    bound; 0 (built-in plan) without matching rows. Plans are built once per layout."""

    from .dispatch_plan import DispatchCostModel, ProfileError, resolve_dispatch_plan, split_tokens_of

    layout = (q_heads, kv_heads, dim, str(dtype))
    if layout not in _packaged_plans:
        plans = {}
        try:
            model = _packaged_plans.get("model") or DispatchCostModel.packaged()
            _packaged_plans["model"] = model
            for entry in model.entries:
                key = dict(entry.key)
                if entry.op == "decode_attention" and key["batch"] not in plans:
                    try:
                        plan = model.plan_attribute("decode_attention", batch=key["batch"],
                                                    q_heads=q_heads, kv_heads=kv_heads,
                                                    head_dim=dim, dtype=str(dtype))
                    except ProfileError:
                        continue
                    if plan["variants"]:
                        plans[key["batch"]] = plan
        except (OSError, ValueError):
            plans = {}
        _packaged_plans[layout] = plans
    plans = _packaged_plans[layout]
    if not plans:
        return 0
    nearest = min(plans, key=lambda size: abs(math.log(size / max(batch, 1))))
    return split_tokens_of(resolve_dispatch_plan(plans[nearest], max(context_bound, 1)).variant)


def decode_attention_workspace_bytes(batch: int, q_heads: int, kv_heads: int, head_dim: int,
                                     max_length: int, split_tokens: int = 0) -> int:
    return int(_lib.load().b200_decode_attention_workspace_bytes(
        batch, q_heads, kv_heads, head_dim, max_length, split_tokens))


def b200_decode_attention(query: torch.Tensor, key_buffer: torch.Tensor,
                          value_buffer: torch.Tensor, lengths: torch.Tensor,
                          attention_mask: Optional[torch.Tensor], *, scale: float,
                          numerical_mode: str = "fast", split_tokens: Optional[int] = None,
                          max_length_hint: int = 0,
                          output: Optional[torch.Tensor] = None,
                          sequence_order: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One-token GQA attention over the physical KV buffers. Mirrors
    triton_decode_attention (backends/triton_attention.py:134-210).

    sequence_order (int32 [B], a permutation of the batch; bf16 only): the order in which the
    sequences are handed to the GPU. With more (sequence, KV head) pairs than the GPU holds at
    once, listing the longest sequences first keeps the last wave short (sequence_order_of).

    attention_mask is B x 1 x 1 x S additive (S <= capacity) or None for an all-zero mask
    of length `capacity`. Returns B x Hq x 1 x D (memory order B, Hq, D).
    split_tokens: tokens per KV split; 0 = the library's built-in plan; None (default) = the
    profile-guided plan (the measured profile that ships with the package, resolved with the
    batch and the context bound of this call; the built-in plan where it has no matching rows).
    """

    device = _require_cuda(query, key_buffer, value_buffer, lengths, attention_mask)
    if query.ndim != 4 or query.shape[2] != 1:
        raise ValueError("query must be B x H x 1 x D")
    if key_buffer.ndim != 4 or key_buffer.shape != value_buffer.shape:
        raise ValueError("KV buffers must be B x C x H x D tensors of one shape")
    batch, q_heads, _, dim = query.shape
    _, capacity, kv_heads, buffer_dim = key_buffer.shape
    if key_buffer.shape[0] != batch or buffer_dim != dim:
        raise ValueError("query batch or head_dim does not match the KV buffers")
    if kv_heads <= 0 or q_heads % kv_heads:
        raise ValueError("query heads must be a multiple of KV heads")
    if not key_buffer.is_contiguous() or not value_buffer.is_contiguous():
        raise ValueError("KV buffers must be contiguous")
    if lengths.shape != (batch,) or lengths.dtype != torch.int64:
        raise ValueError("lengths must be a one-dimensional int64 batch tensor")
    if not (query.dtype == key_buffer.dtype == value_buffer.dtype):
        raise ValueError("query and KV buffers must share one dtype")
    if query.stride(3) != 1:
        query = _dense(query)
    mask_len, mask_stride, mask_code = capacity, 0, _lib.F32
    if attention_mask is not None:
        if attention_mask.ndim != 4 or attention_mask.shape[1] != 1 or \
                attention_mask.shape[2] != 1 or attention_mask.shape[0] != batch:
            raise ValueError("attention_mask must be B x 1 x 1 x S")
        mask_len = attention_mask.shape[3]
        if mask_len > capacity or mask_len <= 0:
            raise ValueError("mask length must be in [1, capacity]")
        if attention_mask.stride(3) != 1:
            attention_mask = _dense(attention_mask)
        mask_stride = attention_mask.stride(0)
        mask_code = _code(attention_mask.dtype)
    lengths = _dense_index(lengths, "lengths")
    if output is None:
        output = torch.empty((batch, q_heads, 1, dim), dtype=query.dtype, device=device)
    rt = runtime(device)
    library = _lib.load()
    max_length = min(max_length_hint, mask_len) if max_length_hint > 0 else mask_len
    if split_tokens is None:
        split_tokens = _profiled_split_tokens(batch, q_heads, kv_heads, dim, query.dtype, max_length)
    need = 0
    if query.dtype == torch.bfloat16:
        need = int(library.b200_decode_attention_workspace_bytes(
            batch, q_heads, kv_heads, dim, max_length, split_tokens))
    workspace = rt.workspace("decode_attention", need)
    if sequence_order is not None:
        _require_cuda(query, sequence_order)
        if sequence_order.dtype != torch.int32 or sequence_order.shape != (batch,) or \
                not sequence_order.is_contiguous():
            raise ValueError("sequence_order must be a contiguous int32 vector of B entries")
        if query.dtype != torch.bfloat16:
            raise ValueError("a sequence order is taken by the bf16 kernel only")
        code = library.b200_decode_attention_ordered(
            query.data_ptr(), key_buffer.data_ptr(), value_buffer.data_ptr(), lengths.data_ptr(),
            _ptr(attention_mask), output.data_ptr(), sequence_order.data_ptr(), batch, q_heads,
            kv_heads, dim, capacity, mask_len, query.stride(0), query.stride(1), mask_stride,
            mask_code, float(scale), _code(query.dtype), _mode(numerical_mode), int(split_tokens),
            int(max_length_hint), _ptr(workspace), need, rt.status.data_ptr(), _stream())
    else:
        code = library.b200_decode_attention(
            query.data_ptr(), key_buffer.data_ptr(), value_buffer.data_ptr(), lengths.data_ptr(),
            _ptr(attention_mask), output.data_ptr(), batch, q_heads, kv_heads, dim, capacity,
            mask_len, query.stride(0), query.stride(1), mask_stride, mask_code, float(scale),
            _code(query.dtype), _mode(numerical_mode), int(split_tokens), int(max_length_hint),
            _ptr(workspace), need, rt.status.data_ptr(), _stream())
    _check(code, "b200_decode_attention")
    _count(rt)
    return output


def _order_pointer(sequence_order: Optional[torch.Tensor], batch: int, device) -> Optional[int]:
    if sequence_order is None:
        return None
    if sequence_order.dtype != torch.int32 or sequence_order.shape != (batch,) or \
            not sequence_order.is_contiguous() or sequence_order.device != device:
        raise ValueError("sequence_order must be a contiguous int32 vector of B entries on the operands' device")
    return sequence_order.data_ptr()


def sequence_order_of(lengths: torch.Tensor) -> torch.Tensor:
    """Longest-first service order for b200_decode_attention(sequence_order=...): the batch
    indices sorted by descending length (stable), int32, on the lengths' device. Lengths that
    all grow by one per step keep their order, so a serving loop computes this once per batch."""

    return torch.argsort(lengths, descending=True, stable=True).to(torch.int32)


def b200_decode_attention_no_alloc(query: torch.Tensor, key_buffer: torch.Tensor,
                                   value_buffer: torch.Tensor, lengths: torch.Tensor,
                                   attention_mask: Optional[torch.Tensor], output: torch.Tensor, *,
                                   scale: float, numerical_mode: str = "fast",
                                   split_tokens: int = 0, max_length_hint: int = 0) -> torch.Tensor:
    """Decode attention for callers that must not allocate on the device.

    Some users of this backend cannot let a call reach cudaMalloc or torch's caching
    allocator: a step being captured into a CUDA graph, a serving loop whose memory budget is
    frozen after start-up, a host framework that hands its plugins a fixed arena. This
    variant takes the output tensor from the caller and keeps the split-KV scratch in an
    8 MiB array inside the library (one per GPU, alive until the process exits) instead of a
    workspace tensor. Nothing is allocated by this call or in the library (the one exception:
    the very first use of this package on a GPU creates that GPU's 4-byte status word, so touch
    `kernels.runtime(device)` once at start-up); tensors that would need a contiguous copy are
    rejected. Requests whose partial sums do not fit the array raise
    ValueError (raise split_tokens to shrink the need). Calls on one GPU share the array, so
    calls that overlap on different streams race; the first call on a device should happen
    outside graph capture because it looks the array's address up. bf16 only.
    """

    device = _require_cuda(query, key_buffer, value_buffer, lengths, attention_mask, output)
    if query.ndim != 4 or query.shape[2] != 1 or query.stride(3) != 1:
        raise ValueError("query must be B x H x 1 x D with a contiguous last dimension")
    if key_buffer.ndim != 4 or key_buffer.shape != value_buffer.shape or \
            not key_buffer.is_contiguous() or not value_buffer.is_contiguous():
        raise ValueError("KV buffers must be contiguous B x C x H x D tensors of one shape")
    batch, q_heads, _, dim = query.shape
    _, capacity, kv_heads, buffer_dim = key_buffer.shape
    if key_buffer.shape[0] != batch or buffer_dim != dim or kv_heads <= 0 or q_heads % kv_heads:
        raise ValueError("query does not match the KV buffers")
    if lengths.shape != (batch,) or lengths.dtype != torch.int64 or not lengths.is_contiguous():
        raise ValueError("lengths must be a contiguous one-dimensional int64 batch tensor")
    if not (query.dtype == key_buffer.dtype == value_buffer.dtype == output.dtype):
        raise ValueError("query, KV buffers and output must share one dtype")
    if output.shape != (batch, q_heads, 1, dim) or not output.is_contiguous():
        raise ValueError("output must be a contiguous B x H x 1 x D tensor")
    mask_len, mask_stride, mask_code = capacity, 0, _lib.F32
    if attention_mask is not None:
        if attention_mask.ndim != 4 or attention_mask.shape[:3] != (batch, 1, 1) or \
                attention_mask.stride(3) != 1:
            raise ValueError("attention_mask must be B x 1 x 1 x S with a contiguous last dimension")
        mask_len = attention_mask.shape[3]
        if mask_len > capacity or mask_len <= 0:
            raise ValueError("mask length must be in [1, capacity]")
        mask_stride = attention_mask.stride(0)
        mask_code = _code(attention_mask.dtype)
    rt = runtime(device)
    code = _lib.load().b200_decode_attention_static_scratch(
        query.data_ptr(), key_buffer.data_ptr(), value_buffer.data_ptr(), lengths.data_ptr(),
        _ptr(attention_mask), output.data_ptr(), batch, q_heads, kv_heads, dim, capacity,
        mask_len, query.stride(0), query.stride(1), mask_stride, mask_code, float(scale),
        _code(query.dtype), _mode(numerical_mode), int(split_tokens), int(max_length_hint),
        rt.status.data_ptr(), _stream())
    if code == _lib.ERR_TOO_LARGE:
        raise ValueError(
            "b200_decode_attention_static_scratch: the split partials do not fit the library's "
            f"{_lib.load().b200_decode_attention_static_scratch_bytes()} byte scratch array; "
            "use a larger split_tokens or the workspace entry point")
    _check(code, "b200_decode_attention_static_scratch")
    _count(rt)
    return output


# ------------------------------------------------------------------- paged KV ----
def b200_paged_kv_store(key_pool: torch.Tensor, value_pool: torch.Tensor, block_table: torch.Tensor,
                        key: torch.Tensor, value: torch.Tensor, positions: torch.Tensor) -> None:
    """serve.kv.store through a block table: pool[table[b, (pos+t) // bs], (pos+t) % bs, h, :] =
    x[b, h, t, :] for K and V. Pools are blocks x block_size x H x D, the table int32 B x
    max_blocks_per_sequence. The paged counterpart of b200_kv_store (the reference lists the
    layout as future work, README.md:295)."""

    device = _require_cuda(key_pool, value_pool, block_table, key, value, positions)
    if key_pool.ndim != 4 or key_pool.shape != value_pool.shape or not key_pool.is_contiguous() or \
            not value_pool.is_contiguous():
        raise ValueError("KV pools must be contiguous blocks x block_size x H x D tensors of one shape")
    if key.ndim != 4 or key.shape != value.shape:
        raise ValueError("key/value must be B x H x T x D tensors of one shape")
    blocks, block_size, heads, dim = key_pool.shape
    batch, _, tokens, _ = key.shape
    if key.shape[1] != heads or key.shape[3] != dim:
        raise ValueError("key/value heads or head_dim do not match the pools")
    if block_table.dtype != torch.int32 or block_table.ndim != 2 or block_table.shape[0] != batch or \
            not block_table.is_contiguous():
        raise ValueError("block_table must be a contiguous int32 B x max_blocks tensor")
    if positions.shape != (batch,) or positions.dtype != torch.int64 or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous int64 batch vector")
    if len({key_pool.dtype, value_pool.dtype, key.dtype, value.dtype}) != 1:
        raise ValueError("pools and key/value must share one dtype")
    rt = runtime(device)
    code = _lib.load().b200_paged_kv_store(
        key_pool.data_ptr(), value_pool.data_ptr(), block_table.data_ptr(), key.data_ptr(),
        value.data_ptr(), positions.data_ptr(), batch, heads, tokens, dim, blocks, block_size,
        block_table.shape[1], _lib.i64_array(key.stride()), _lib.i64_array(value.stride()),
        _code(key.dtype), rt.status.data_ptr(), _stream())
    _check(code, "b200_paged_kv_store")
    _count(rt)


def b200_paged_decode_attention(query: torch.Tensor, key_pool: torch.Tensor, value_pool: torch.Tensor,
                                block_table: torch.Tensor, lengths: torch.Tensor,
                                attention_mask: Optional[torch.Tensor], *, scale: float,
                                numerical_mode: str = "fast", split_tokens: int = 0,
                                max_length_hint: int = 0) -> torch.Tensor:
    """serve.decode_attention over paged KV: the kernel of b200_decode_attention reading every
    32-token step through the block table. bf16; returns B x Hq x 1 x D."""

    device = _require_cuda(query, key_pool, value_pool, block_table, lengths, attention_mask)
    if query.ndim != 4 or query.shape[2] != 1:
        raise ValueError("query must be B x H x 1 x D")
    if key_pool.ndim != 4 or key_pool.shape != value_pool.shape or not key_pool.is_contiguous() or \
            not value_pool.is_contiguous():
        raise ValueError("KV pools must be contiguous blocks x block_size x H x D tensors of one shape")
    batch, q_heads, _, dim = query.shape
    blocks, block_size, kv_heads, pool_dim = key_pool.shape
    if pool_dim != dim or kv_heads <= 0 or q_heads % kv_heads:
        raise ValueError("query does not match the pools")
    if not (query.dtype == key_pool.dtype == value_pool.dtype == torch.bfloat16):
        raise ValueError("paged decode attention runs bf16")
    if block_table.dtype != torch.int32 or block_table.ndim != 2 or block_table.shape[0] != batch or \
            not block_table.is_contiguous():
        raise ValueError("block_table must be a contiguous int32 B x max_blocks tensor")
    if lengths.shape != (batch,) or lengths.dtype != torch.int64 or not lengths.is_contiguous():
        raise ValueError("lengths must be a contiguous int64 batch vector")
    if query.stride(3) != 1:
        query = _dense(query)
    capacity = block_table.shape[1] * block_size
    mask_len, mask_stride, mask_code = capacity, 0, _lib.F32
    if attention_mask is not None:
        if attention_mask.ndim != 4 or attention_mask.shape[:3] != (batch, 1, 1):
            raise ValueError("attention_mask must be B x 1 x 1 x S")
        mask_len = attention_mask.shape[3]
        if mask_len > capacity or mask_len <= 0:
            raise ValueError("mask length must be in [1, capacity]")
        if attention_mask.stride(3) != 1:
            attention_mask = _dense(attention_mask)
        mask_stride = attention_mask.stride(0)
        mask_code = _code(attention_mask.dtype)
    output = torch.empty((batch, q_heads, 1, dim), dtype=query.dtype, device=device)
    rt = runtime(device)
    library = _lib.load()
    max_length = min(max_length_hint, mask_len) if max_length_hint > 0 else mask_len
    need = int(library.b200_decode_attention_workspace_bytes(batch, q_heads, kv_heads, dim, max_length,
                                                            split_tokens))
    workspace = rt.workspace("decode_attention", need)
    code = library.b200_paged_decode_attention(
        query.data_ptr(), key_pool.data_ptr(), value_pool.data_ptr(), block_table.data_ptr(),
        lengths.data_ptr(), _ptr(attention_mask), output.data_ptr(), batch, q_heads, kv_heads, dim,
        blocks, block_size, block_table.shape[1], mask_len, query.stride(0), query.stride(1),
        mask_stride, mask_code, float(scale), _mode(numerical_mode), int(split_tokens),
        int(max_length_hint), _ptr(workspace), need, rt.status.data_ptr(), _stream())
    _check(code, "b200_paged_decode_attention")
    _count(rt)
    return output


# --------------------------------------------------------------- prefill attention ----
def b200_prefill_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                           attention_mask: Optional[torch.Tensor], *, scale: float,
                           causal: bool = False, numerical_mode: str = "fast") -> torch.Tensor:
    """T-token GQA attention with an additive B x 1 x T x T mask (or proven causality).
    Mirrors triton_prefill_attention (backends/triton_prefill_attention.py:152-232).

    Returns a B x Hq x T x D tensor whose memory order is B, T, Hq, D, so that the
    transpose(1, 2) + reshape that follows in Qwen2 graphs is a view.
    """

    device = _require_cuda(query, key, value, attention_mask)
    if query.ndim != 4 or key.ndim != 4 or key.shape != value.shape:
        raise ValueError("query must be B x Hq x T x D and key/value B x Hkv x T x D")
    batch, q_heads, tokens, dim = query.shape
    kv_heads = key.shape[1]
    if key.shape[0] != batch or key.shape[2] != tokens or key.shape[3] != dim:
        raise ValueError("query and key/value disagree on batch, tokens or head_dim")
    if kv_heads <= 0 or q_heads % kv_heads:
        raise ValueError("query heads must be a multiple of KV heads")
    if not (query.dtype == key.dtype == value.dtype):
        raise ValueError("query, key and value must share one dtype")
    if attention_mask is None and not causal:
        raise ValueError("a mask is required unless causality is proven")
    mask_strides = None
    mask_code = _lib.F32
    if attention_mask is not None:
        if attention_mask.ndim != 4 or attention_mask.shape[1] != 1 or \
                attention_mask.shape[2] != tokens or attention_mask.shape[3] != tokens or \
                attention_mask.shape[0] not in (1, batch):
            raise ValueError("attention_mask must be B x 1 x T x T")
        strides = list(attention_mask.stride())
        if attention_mask.shape[0] == 1:
            strides[0] = 0
        mask_strides = _lib.i64_array(strides)
        mask_code = _code(attention_mask.dtype)
    query = query if query.stride(3) == 1 else _dense(query)
    key = key if key.stride(3) == 1 else _dense(key)
    value = value if value.stride(3) == 1 else _dense(value)
    storage = torch.empty((batch, tokens, q_heads, dim), dtype=query.dtype, device=device)
    rt = runtime(device)
    library = _lib.load()
    need = 0
    if attention_mask is not None and not causal and query.dtype == torch.bfloat16:
        need = int(library.b200_prefill_attention_workspace_bytes(batch, tokens))  # mask tile classes
    workspace = rt.workspace("prefill_attention", need)
    code = library.b200_prefill_attention(
        query.data_ptr(), key.data_ptr(), value.data_ptr(), _ptr(attention_mask),
        storage.data_ptr(), batch, q_heads, kv_heads, tokens, dim,
        _lib.i64_array(query.stride()), _lib.i64_array(key.stride()),
        _lib.i64_array(value.stride()), mask_strides, mask_code, float(scale), int(bool(causal)),
        _code(query.dtype), _mode(numerical_mode), _ptr(workspace), need, rt.status.data_ptr(),
        _stream())
    _check(code, "b200_prefill_attention")
    _count(rt)
    return storage.transpose(1, 2)


_causal_verdicts: dict = {}


def b200_mask_is_causal(attention_mask: torch.Tensor) -> bool:
    """Run-time proof that an additive B x 1 x T x T mask is exactly the causal mask (0 on and
    below the diagonal, -inf above): one pass of a classifier kernel over the mask and ONE host
    read of its verdict (a synchronisation), remembered per (storage, shape, strides, version)
    so that the layers of a model, which all receive the same tensor, pay it once. The
    reference names the proved form as the follow-up of its `causal: "mask"` contract
    (docs/prefill-attention.md:43-45). Never call it under CUDA-graph capture."""

    device = _require_cuda(attention_mask)
    if attention_mask.ndim != 4 or attention_mask.shape[1] != 1 or \
            attention_mask.shape[2] != attention_mask.shape[3]:
        return False
    if attention_mask.dtype not in _DTYPE_CODES:
        return False
    key = (device.index, attention_mask.data_ptr(), tuple(attention_mask.shape),
           tuple(attention_mask.stride()), attention_mask._version, attention_mask.dtype)
    verdict = _causal_verdicts.get(key)
    if verdict is None:
        rt = runtime(device)
        flag = torch.empty(1, dtype=torch.int32, device=device)
        strides = list(attention_mask.stride())
        if attention_mask.shape[0] == 1:
            strides[0] = 0
        code = _lib.load().b200_classify_causal_mask(
            attention_mask.data_ptr(), attention_mask.shape[0], attention_mask.shape[2],
            _lib.i64_array(strides), _code(attention_mask.dtype), flag.data_ptr(), _stream())
        _check(code, "b200_classify_causal_mask")
        _count(rt, 2)
        verdict = bool(flag.item())
        if len(_causal_verdicts) > 64:
            _causal_verdicts.clear()
        _causal_verdicts[key] = verdict
    return verdict


def b200_pack_rows(*tensors: torch.Tensor) -> torch.Tensor:
    """Weight preparation: rows of several matrices (or entries of several vectors) one after
    the other, e.g. q|k|v projection weights into one matrix. A one-time device copy."""

    device = _require_cuda(*tensors)
    first = tensors[0]
    if any(t.shape[1:] != first.shape[1:] or t.dtype != first.dtype for t in tensors):
        raise ValueError("packed tensors must agree on dtype and trailing dimensions")
    rows = sum(t.shape[0] for t in tensors)
    packed = torch.empty((rows, *first.shape[1:]), dtype=first.dtype, device=device)
    offset = 0
    for tensor in tensors:
        packed[offset:offset + tensor.shape[0]].copy_(tensor)
        offset += tensor.shape[0]
    return packed


# -------------------------------------------------------------------------- linear ----
def linear_workspace_bytes(m: int, k: int, n: int, dtype: torch.dtype,
                           epilogue: str = "none") -> int:
    return int(_lib.load().b200_linear_workspace_bytes(m, k, n, _code(dtype),
                                                       _EPILOGUES[epilogue]))


def b200_linear(tensor: torch.Tensor, weight: torch.Tensor,
                bias: Optional[torch.Tensor] = None, *, residual: Optional[torch.Tensor] = None,
                epilogue: str = "none") -> torch.Tensor:
    """y = x W^T (+ bias) with fp32 accumulation. Mirrors triton_linear
    (backends/triton_linear.py:87-148).

    epilogue "residual": y = r(r(x W^T + b) + residual) (same shape as y).
    epilogue "swiglu": weight holds 2N rows, gate_j and up_j alternating, and the result has
    N columns: r(r(silu(r(gate))) * r(up)).
    """

    device = _require_cuda(tensor, weight, bias, residual)
    if weight.ndim != 2:
        raise ValueError("weight must be N x K")
    n, k = weight.shape
    if tensor.ndim < 1 or tensor.shape[-1] != k:
        raise ValueError("the last input dimension must equal the weight's K")
    if tensor.dtype != weight.dtype:
        raise ValueError("input and weight must share one dtype")
    if bias is not None and (bias.shape != (n,) or bias.dtype != tensor.dtype):
        raise ValueError("bias must be a vector of N elements in the input dtype")
    if epilogue not in _EPILOGUES:
        raise ValueError(f"unknown epilogue {epilogue!r}")
    weight = _dense(weight)
    source = _dense(tensor) if tensor.ndim <= 4 else tensor
    if not source.is_contiguous():
        raise ValueError("inputs of rank > 4 must be contiguous")
    m = source.numel() // k
    out_features = n // 2 if epilogue == "swiglu" else n
    output = torch.empty((*tensor.shape[:-1], out_features), dtype=tensor.dtype, device=device)
    if epilogue == "residual":
        if residual is None or residual.shape != output.shape or residual.dtype != tensor.dtype:
            raise ValueError("residual must match the output shape and dtype")
        residual = _dense(residual)
    elif residual is not None:
        raise ValueError("residual given without the residual epilogue")
    if bias is not None:
        bias = _dense(bias)
    rt = runtime(device)
    library = _lib.load()
    code_dtype = _code(tensor.dtype)
    need = int(library.b200_linear_workspace_bytes(m, k, n, code_dtype, _EPILOGUES[epilogue]))
    workspace = rt.workspace("linear", need)
    code = library.b200_linear(source.data_ptr(), weight.data_ptr(), _ptr(bias), _ptr(residual),
                               output.data_ptr(), m, k, n, k, code_dtype, _EPILOGUES[epilogue],
                               _ptr(workspace), need, rt.status.data_ptr(), _stream())
    _check(code, "b200_linear")
    _count(rt)
    return output


def linear_partial_splits(m: int, k: int, n: int) -> int:
    return int(_lib.load().b200_linear_partial_splits(m, k, n))


def b200_linear_partial(tensor: torch.Tensor, weight: torch.Tensor,
                        partials: Optional[torch.Tensor] = None, *, row_squares: bool = False):
    """Decode-size projection without its epilogue: fp32 partial sums [splits, M, N] over K
    slices, to be reduced by the operator that follows (b200_reduce_*). M <= 128, bf16.
    row_squares=True (M <= 128) also returns fp32 [splits, M]: the sum of squares of every input
    row over each K slice, for a consumer that applies an RMSNorm folded into this projection."""

    device = _require_cuda(tensor, weight, partials)
    if weight.ndim != 2 or tensor.ndim != 2 or tensor.shape[1] != weight.shape[1]:
        raise ValueError("input must be M x K and weight N x K")
    if tensor.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise ValueError("the partial-sum producer runs bf16")
    if tensor.stride(1) != 1 or not weight.is_contiguous():
        raise ValueError("input rows and the weight must be contiguous")
    m, k = tensor.shape
    n = weight.shape[0]
    library = _lib.load()
    splits = int(library.b200_linear_partial_splits(m, k, n))
    if partials is None:
        partials = torch.empty((splits, m, n), dtype=torch.float32, device=device)
    elif partials.shape != (splits, m, n) or partials.dtype != torch.float32 or \
            not partials.is_contiguous():
        raise ValueError(f"partials must be a contiguous fp32 tensor of shape {(splits, m, n)}")
    squares = torch.empty((splits, m), dtype=torch.float32, device=device) if row_squares else None
    rt = runtime(device)
    code = library.b200_linear_partial(tensor.data_ptr(), weight.data_ptr(), partials.data_ptr(),
                                       _ptr(squares), m, k, n, tensor.stride(0), splits,
                                       rt.status.data_ptr(), _stream())
    _check(code, "b200_linear_partial")
    _count(rt)
    return (partials, squares) if row_squares else partials


def b200_reduce_residual_rms_norm(partials: torch.Tensor, residual: Optional[torch.Tensor],
                                  norm_weight: Optional[torch.Tensor], *, epsilon: float,
                                  numerical_mode: str = "fast"):
    """x = r(r(sum of partials) + residual); h = RMSNorm(x) * w (Qwen2 rounding order).
    Returns (x, h); h is None when norm_weight is None."""

    device = _require_cuda(partials, residual, norm_weight)
    if partials.ndim != 3 or partials.dtype != torch.float32 or not partials.is_contiguous():
        raise ValueError("partials must be a contiguous fp32 [splits, rows, hidden] tensor")
    splits, rows, hidden = partials.shape
    if residual is not None and (residual.shape != (rows, hidden) or not residual.is_contiguous()
                                 or residual.dtype != torch.bfloat16):
        raise ValueError("residual must be a contiguous bf16 rows x hidden tensor")
    x_out = torch.empty((rows, hidden), dtype=torch.bfloat16, device=device)
    h_out = torch.empty_like(x_out) if norm_weight is not None else None
    rt = runtime(device)
    code = _lib.load().b200_reduce_residual_rms_norm(
        partials.data_ptr(), splits, _ptr(residual), _ptr(norm_weight), x_out.data_ptr(),
        _ptr(h_out), rows, hidden, float(epsilon), _mode(numerical_mode), _stream())
    _check(code, "b200_reduce_residual_rms_norm")
    _count(rt)
    return x_out, h_out


def b200_reduce_rope_kv_store(partials: torch.Tensor, bias: Optional[torch.Tensor],
                              cosine: torch.Tensor, sine: torch.Tensor, key_buffer: torch.Tensor,
                              value_buffer: torch.Tensor, positions: torch.Tensor, *,
                              q_heads: int) -> torch.Tensor:
    """q|k|v = r(sum of partials + bias); RoPE on q and k; k, v into the KV buffers at
    positions[b]. Returns the rotated query, B x Hq x 1 x D."""

    device = _require_cuda(partials, bias, cosine, sine, key_buffer, value_buffer, positions)
    splits, batch, width = partials.shape
    _, capacity, kv_heads, dim = key_buffer.shape
    if width != (q_heads + 2 * kv_heads) * dim or key_buffer.shape[0] != batch:
        raise ValueError("partials do not match the head layout of the KV buffers")
    cos2, sin2 = cosine.reshape(batch, dim), sine.reshape(batch, dim)
    if not (cos2.is_contiguous() and sin2.is_contiguous()):
        raise ValueError("cosine / sine must be contiguous")
    query_out = torch.empty((batch, q_heads, 1, dim), dtype=torch.bfloat16, device=device)
    rt = runtime(device)
    code = _lib.load().b200_reduce_rope_kv_store(
        partials.data_ptr(), splits, _ptr(bias), cos2.data_ptr(), sin2.data_ptr(),
        query_out.data_ptr(), key_buffer.data_ptr(), value_buffer.data_ptr(), positions.data_ptr(),
        batch, q_heads, kv_heads, dim, capacity, rt.status.data_ptr(), _stream())
    _check(code, "b200_reduce_rope_kv_store")
    _count(rt)
    return query_out


def b200_qkv_decode_attention(partials: torch.Tensor, bias: Optional[torch.Tensor],
                              cosine: torch.Tensor, sine: torch.Tensor, key_buffer: torch.Tensor,
                              value_buffer: torch.Tensor, lengths: torch.Tensor, *, q_heads: int,
                              scale: float, split_tokens: int = 0, max_length_hint: int = 0,
                              length_offset: int = 0,
                              norm_row_squares: Optional[torch.Tensor] = None,
                              norm_hidden: int = 0, norm_epsilon: float = 0.0,
                              sequence_order: Optional[torch.Tensor] = None) -> torch.Tensor:
    """b200_reduce_rope_kv_store + b200_decode_attention of a decode step in one launch: the
    q|k|v partials are reduced (+ bias, RoPE) inside the attention kernel, the new token's K / V
    row is stored at row lengths[b] - 1 and attends from registers. lengths are the attention
    lengths (the new token counted; with length_offset=1 they are the lengths before it and the
    kernel adds one, for callers that advance every slot once at the end of the step).
    norm_row_squares (what b200_linear_partial(...,
    row_squares=True) returned) with norm_hidden and norm_epsilon: the RMSNorm in front of the
    projection was folded into it, and the reduced sums are scaled by rsqrt(mean(x^2) +
    norm_epsilon) here. Returns B x Hq x 1 x D."""

    device = _require_cuda(partials, bias, cosine, sine, key_buffer, value_buffer, lengths,
                           norm_row_squares)
    if norm_row_squares is not None and (
            norm_row_squares.shape != partials.shape[:2] or norm_row_squares.dtype != torch.float32
            or not norm_row_squares.is_contiguous() or norm_hidden <= 0):
        raise ValueError("norm_row_squares must be contiguous fp32 [splits, B] with norm_hidden > 0")
    splits, batch, width = partials.shape
    _, capacity, kv_heads, dim = key_buffer.shape
    if partials.dtype != torch.float32 or key_buffer.dtype != torch.bfloat16:
        raise ValueError("fp32 partials and bf16 KV buffers expected")
    if width != (q_heads + 2 * kv_heads) * dim or key_buffer.shape[0] != batch:
        raise ValueError("partials do not match the head layout of the KV buffers")
    if not (key_buffer.is_contiguous() and value_buffer.is_contiguous() and partials.is_contiguous()):
        raise ValueError("partials and KV buffers must be contiguous")
    cos2, sin2 = cosine.reshape(batch, dim), sine.reshape(batch, dim)
    if not (cos2.is_contiguous() and sin2.is_contiguous()):
        raise ValueError("cosine / sine must be contiguous")
    lengths = _dense_index(lengths, "lengths")
    output = torch.empty((batch, q_heads, 1, dim), dtype=torch.bfloat16, device=device)
    rt = runtime(device)
    library = _lib.load()
    max_length = min(max_length_hint, capacity) if max_length_hint > 0 else capacity
    need = int(library.b200_decode_attention_workspace_bytes(batch, q_heads, kv_heads, dim,
                                                            max_length, split_tokens))
    workspace = rt.workspace("decode_attention", need)
    code = library.b200_qkv_decode_attention(
        partials.data_ptr(), splits, _ptr(bias), cos2.data_ptr(), sin2.data_ptr(),
        key_buffer.data_ptr(), value_buffer.data_ptr(), lengths.data_ptr(), output.data_ptr(),
        batch, q_heads, kv_heads, dim, capacity, capacity, float(scale), int(split_tokens),
        int(max_length_hint), int(length_offset), _ptr(norm_row_squares), int(norm_hidden),
        float(norm_epsilon), _order_pointer(sequence_order, batch, device), _ptr(workspace),
        need, rt.status.data_ptr(), _stream())
    _check(code, "b200_qkv_decode_attention")
    _count(rt)
    return output


def b200_paged_qkv_decode_attention(partials: torch.Tensor, bias: Optional[torch.Tensor],
                                    cosine: torch.Tensor, sine: torch.Tensor, key_pool: torch.Tensor,
                                    value_pool: torch.Tensor, block_table: torch.Tensor,
                                    lengths: torch.Tensor, *, q_heads: int, scale: float,
                                    split_tokens: int = 0, max_length_hint: int = 0,
                                    length_offset: int = 0,
                                    norm_row_squares: Optional[torch.Tensor] = None,
                                    norm_hidden: int = 0, norm_epsilon: float = 0.0,
                                    sequence_order: Optional[torch.Tensor] = None) -> torch.Tensor:
    """b200_qkv_decode_attention on the paged layout: K / V pools [blocks, block_size, Hkv, D]
    and an int32 block table [B, max_blocks]; the new token's row goes to the block the table
    names for position lengths[b] - 1 (a missing block raises the KV-overflow status bit)."""

    device = _require_cuda(partials, bias, cosine, sine, key_pool, value_pool, block_table, lengths,
                           norm_row_squares)
    if norm_row_squares is not None and (
            norm_row_squares.shape != partials.shape[:2] or norm_row_squares.dtype != torch.float32
            or not norm_row_squares.is_contiguous() or norm_hidden <= 0):
        raise ValueError("norm_row_squares must be contiguous fp32 [splits, B] with norm_hidden > 0")
    splits, batch, width = partials.shape
    blocks, block_size, kv_heads, dim = key_pool.shape
    if partials.dtype != torch.float32 or key_pool.dtype != torch.bfloat16:
        raise ValueError("fp32 partials and bf16 KV pools expected")
    if width != (q_heads + 2 * kv_heads) * dim or value_pool.shape != key_pool.shape:
        raise ValueError("partials do not match the head layout of the KV pools")
    if block_table.dtype != torch.int32 or block_table.ndim != 2 or block_table.shape[0] != batch \
            or not block_table.is_contiguous():
        raise ValueError("block_table must be a contiguous int32 [B, max_blocks] tensor")
    if block_size % 32 != 0:
        raise ValueError("block_size must be a multiple of 32 tokens")
    if not (key_pool.is_contiguous() and value_pool.is_contiguous() and partials.is_contiguous()):
        raise ValueError("partials and KV pools must be contiguous")
    cos2, sin2 = cosine.reshape(batch, dim), sine.reshape(batch, dim)
    if not (cos2.is_contiguous() and sin2.is_contiguous()):
        raise ValueError("cosine / sine must be contiguous")
    lengths = _dense_index(lengths, "lengths")
    output = torch.empty((batch, q_heads, 1, dim), dtype=torch.bfloat16, device=device)
    rt = runtime(device)
    library = _lib.load()
    max_blocks = block_table.shape[1]
    capacity = max_blocks * block_size
    max_length = min(max_length_hint, capacity) if max_length_hint > 0 else capacity
    need = int(library.b200_decode_attention_workspace_bytes(batch, q_heads, kv_heads, dim,
                                                            max_length, split_tokens))
    workspace = rt.workspace("decode_attention", need)
    code = library.b200_paged_qkv_decode_attention(
        partials.data_ptr(), splits, _ptr(bias), cos2.data_ptr(), sin2.data_ptr(),
        key_pool.data_ptr(), value_pool.data_ptr(), block_table.data_ptr(), lengths.data_ptr(),
        output.data_ptr(), batch, q_heads, kv_heads, dim, blocks, block_size, max_blocks, capacity,
        float(scale), int(split_tokens), int(max_length_hint), int(length_offset),
        _ptr(norm_row_squares), int(norm_hidden), float(norm_epsilon),
        _order_pointer(sequence_order, batch, device), _ptr(workspace), need,
        rt.status.data_ptr(), _stream())
    _check(code, "b200_paged_qkv_decode_attention")
    _count(rt)
    return output


def b200_scale_columns(weight: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Weight preparation: weight[n, k] * scale[k], rounded to the weight dtype -- a norm
    weight folded into the projection that follows the norm. A one-time device pass."""

    device = _require_cuda(weight, scale)
    if weight.ndim != 2 or scale.shape != (weight.shape[1],) or scale.dtype != weight.dtype:
        raise ValueError("scale must be a vector of the weight's K in the weight's dtype")
    weight, scale = _dense(weight), _dense(scale)
    output = torch.empty_like(weight)
    rt = runtime(device)
    code = _lib.load().b200_scale_columns(weight.data_ptr(), scale.data_ptr(), output.data_ptr(),
                                          weight.shape[0], weight.shape[1], _code(weight.dtype),
                                          _stream())
    _check(code, "b200_scale_columns")
    _count(rt)
    return output


def decode_chain_rows(weight) -> int:
    """Rows up to which the five-launch decode layer's kernels (folded-norm projection, cluster
    split-K, fused q|k|v attention) are the faster form of a projection with this weight (a
    tensor, or its size in bytes): 128
    while the matrix is small enough for the launch to be a chain of latencies (a Qwen2-0.5B
    layer at 96 sequences: 1.82 -> 1.69 ms per step), 64 for large matrices, where the 128-row
    tiles of those kernels re-read the activations through L2 once per 64 columns and lose to
    the split-K partial producers (Qwen2-7B layers at 128 sequences: 10.1 -> 11.8 ms)."""

    nbytes = weight if isinstance(weight, int) else weight.numel() * weight.element_size()
    return 128 if nbytes <= (32 << 20) else 64


def b200_linear_rms_input(tensor: torch.Tensor, folded_weight: torch.Tensor,
                          bias: Optional[torch.Tensor] = None, *, epsilon: float,
                          epilogue: str = "none",
                          row_squares: Optional[torch.Tensor] = None) -> torch.Tensor:
    """serve.rms_norm + serve.linear in one launch (fast mode, bf16, at most 128 rows): `tensor`
    is the un-normalised input, `folded_weight` the projection weight with the norm weight
    multiplied into its columns (b200_scale_columns); the kernel scales each accumulator row by
    rsqrt(mean(x^2) + epsilon) before the bias / SwiGLU epilogue. `row_squares` (fp32
    [slices, M], what b200_linear_splitk_residual(..., row_squares=True) left for these very
    rows): the kernel adds the slices instead of squaring the rows itself."""

    device = _require_cuda(tensor, folded_weight, bias)
    if tensor.ndim != 2 or folded_weight.ndim != 2 or tensor.shape[1] != folded_weight.shape[1]:
        raise ValueError("input must be M x K and weight N x K")
    if tensor.dtype != torch.bfloat16 or folded_weight.dtype != torch.bfloat16:
        raise ValueError("the folded-norm projection runs bf16")
    if tensor.stride(1) != 1 or not folded_weight.is_contiguous():
        raise ValueError("input rows and the weight must be contiguous")
    if epilogue not in ("none", "swiglu"):
        raise ValueError(f"unsupported epilogue {epilogue!r}")
    m, k = tensor.shape
    n = folded_weight.shape[0]
    if bias is not None and (bias.shape != (n,) or bias.dtype != torch.bfloat16):
        raise ValueError("bias must be a bf16 vector of N elements")
    slices = 0
    if row_squares is not None:
        _require_cuda(tensor, row_squares)
        if row_squares.dtype != torch.float32 or row_squares.ndim != 2 or \
                row_squares.shape[1] != m or not row_squares.is_contiguous():
            raise ValueError("row_squares must be a contiguous fp32 [slices, M] tensor")
        slices = row_squares.shape[0]
    output = torch.empty((m, n // 2 if epilogue == "swiglu" else n), dtype=torch.bfloat16,
                         device=device)
    rt = runtime(device)
    code = _lib.load().b200_linear_rms_input(
        tensor.data_ptr(), folded_weight.data_ptr(), _ptr(bias), output.data_ptr(),
        _ptr(row_squares) if slices else None, slices, m, k, n,
        tensor.stride(0), float(epsilon), _EPILOGUES[epilogue], rt.status.data_ptr(), _stream())
    _check(code, "b200_linear_rms_input")
    _count(rt)
    return output


def b200_linear_splitk_residual(tensor: torch.Tensor, weight: torch.Tensor,
                                residual: torch.Tensor, *, row_squares: bool = False):
    """serve.linear + aten.add in one launch at decode sizes (bf16, at most 256 rows):
    r(r(x W^T) + residual). The K slices of an output tile are the CTAs of one thread-block
    cluster and add their fp32 accumulators through distributed shared memory. With
    `row_squares` the result is (output, squares): fp32 [slices, M] partial sums of the squared
    output rows for a folded RMSNorm behind this projection (b200_linear_rms_input), or None
    where the shape runs without a cluster and leaves none."""

    device = _require_cuda(tensor, weight, residual)
    if tensor.ndim != 2 or weight.ndim != 2 or tensor.shape[1] != weight.shape[1]:
        raise ValueError("input must be M x K and weight N x K")
    if tensor.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or \
            residual.dtype != torch.bfloat16:
        raise ValueError("the split-K projection runs bf16")
    m, k = tensor.shape
    n = weight.shape[0]
    if residual.shape != (m, n) or not residual.is_contiguous():
        raise ValueError("residual must be a contiguous M x N tensor")
    if tensor.stride(1) != 1 or not weight.is_contiguous():
        raise ValueError("input rows and the weight must be contiguous")
    output = torch.empty((m, n), dtype=torch.bfloat16, device=device)
    rt = runtime(device)
    library = _lib.load()
    squares = None
    if row_squares:
        slices = library.b200_linear_splitk_slices(m, k, n) if m <= 256 else 0
        if slices > 0:
            squares = torch.empty((slices, m), dtype=torch.float32, device=device)
    code = library.b200_linear_splitk_residual(
        tensor.data_ptr(), weight.data_ptr(), residual.data_ptr(), output.data_ptr(),
        _ptr(squares), m, k, n, tensor.stride(0), rt.status.data_ptr(), _stream())
    if code == _lib.ERR_UNSUPPORTED:  # no cluster plan for this shape: the general projection
        output = b200_linear(tensor, weight, residual=residual, epilogue="residual")
        return (output, None) if row_squares else output
    _check(code, "b200_linear_splitk_residual")
    _count(rt)
    return (output, squares) if row_squares else output


def interleave_gate_up(gate_weight: torch.Tensor, up_weight: torch.Tensor) -> torch.Tensor:
    """Row-interleaves gate and up projection weights (gate_0, up_0, gate_1, ...) for the
    SwiGLU epilogue. A one-time weight repack done at load time with a device copy."""

    if gate_weight.shape != up_weight.shape:
        raise ValueError("gate and up weights must have one shape")
    n, k = gate_weight.shape
    packed = torch.empty((2 * n, k), dtype=gate_weight.dtype, device=gate_weight.device)
    packed[0::2].copy_(gate_weight)
    packed[1::2].copy_(up_weight)
    return packed


# ------------------------------------------------- ops the reference leaves to eager ----
def b200_embedding(table: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """aten.embedding.default: rows of `table` gathered by int64 ids."""

    device = _require_cuda(table, ids)
    if table.ndim != 2 or ids.dtype != torch.int64:
        raise ValueError("embedding needs a V x H table and int64 ids")
    table = _dense(table)
    ids = _dense_index(ids, "ids")
    vocab, hidden = table.shape
    output = torch.empty((*ids.shape, hidden), dtype=table.dtype, device=device)
    rt = runtime(device)
    code = _lib.load().b200_embedding(table.data_ptr(), ids.data_ptr(), output.data_ptr(),
                                      ids.numel(), hidden, vocab, _code(table.dtype),
                                      rt.status.data_ptr(), _stream())
    _check(code, "b200_embedding")
    _count(rt)
    return output


def b200_swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """aten.silu.default + aten.mul.Tensor: r(r(silu(gate)) * up)."""

    device = _require_cuda(gate, up)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("gate and up must share shape and dtype")
    gate = _dense(gate)
    up = _dense(up)
    output = torch.empty_like(gate)
    rt = runtime(device)
    code = _lib.load().b200_swiglu(gate.data_ptr(), up.data_ptr(), output.data_ptr(),
                                   gate.numel(), _code(gate.dtype), _stream())
    _check(code, "b200_swiglu")
    _count(rt)
    return output


def b200_add(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """aten.add.Tensor on same-shape tensors: r(a + b)."""

    device = _require_cuda(a, b)
    if a.shape != b.shape or a.dtype != b.dtype:
        raise ValueError("add operands must share shape and dtype")
    a = _dense(a)
    b = _dense(b)
    output = torch.empty_like(a)
    rt = runtime(device)
    code = _lib.load().b200_add(a.data_ptr(), b.data_ptr(), output.data_ptr(), a.numel(),
                                _code(a.dtype), _stream())
    _check(code, "b200_add")
    _count(rt)
    return output


def b200_contiguous(tensor: torch.Tensor, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """aten.contiguous.default / a real aten.to.dtype: dense copy of a (<= 4-D) strided view,
    optionally converting between f32, bf16 and f16."""

    device = _require_cuda(tensor)
    dtype = dtype or tensor.dtype
    if tensor.ndim > 4:
        raise ValueError("strided copies handle at most 4 dimensions")
    sizes = [1] * (4 - tensor.ndim) + list(tensor.shape)
    strides = [0] * (4 - tensor.ndim) + list(tensor.stride())
    output = torch.empty(tensor.shape, dtype=dtype, device=device)
    rt = runtime(device)
    code = _lib.load().b200_copy_4d(tensor.data_ptr(), output.data_ptr(), _lib.i64_array(sizes),
                                    _lib.i64_array(strides), _code(tensor.dtype), _code(dtype),
                                    _stream())
    _check(code, "b200_copy_4d")
    _count(rt)
    return output


def b200_advance_lengths(lengths: torch.Tensor, delta: int, capacity: int) -> None:
    """runtime.kv.advance in place: lengths += delta, clamped at capacity with a status bit.
    `lengths` is int64 of shape [batch] or [slots, batch], contiguous."""

    device = _require_cuda(lengths)
    if lengths.dtype != torch.int64 or not lengths.is_contiguous() or lengths.ndim not in (1, 2):
        raise ValueError("lengths must be a contiguous int64 tensor of rank 1 or 2")
    if delta <= 0:
        raise ValueError("advance delta must be positive")
    slots = lengths.shape[0] if lengths.ndim == 2 else 1
    batch = lengths.shape[-1]
    rt = runtime(device)
    code = _lib.load().b200_advance_lengths(lengths.data_ptr(), slots, batch, int(delta),
                                            int(capacity), rt.status.data_ptr(), _stream())
    _check(code, "b200_advance_lengths")
    _count(rt)


def b200_argmax(logits: torch.Tensor, output: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Greedy token per row of a [..., V] logits tensor (lowest index wins ties)."""

    device = _require_cuda(logits)
    vocab = logits.shape[-1]
    source = _dense(logits)
    rows = source.numel() // vocab
    if output is None:
        output = torch.empty(logits.shape[:-1], dtype=torch.int64, device=device)
    rt = runtime(device)
    code = _lib.load().b200_argmax(source.data_ptr(), output.data_ptr(), rows, vocab, vocab,
                                   _code(logits.dtype), _stream())
    _check(code, "b200_argmax")
    _count(rt)
    return output


def default_scale(head_dim: int) -> float:
    return 1.0 / math.sqrt(head_dim)
