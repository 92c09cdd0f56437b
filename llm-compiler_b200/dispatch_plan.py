"""Profile-guided dispatch plan: measured variant costs -> shape-bucketed plan -> run-time pick.

The reference does this for serve.rms_norm only: a profile JSON (schema version 1) is loaded
into RMSNormCostModel (cost_model.py:87-123), turned into a multi-version `lowering_plan`
attribute whose variants own row buckets bounded by floor(sqrt(a * b)) of neighbouring profiled
row counts (cost_model.py:126-186), written onto the operation by SelectRMSNormLoweringPass
(passes/lowering_selection.py:24-71) and resolved with the run-time row count by
resolve_lowering_plan (cost_model.py:220-245). This module keeps the schema, the bucketing rule
and the decision record, and generalises them to the operators whose B200 kernels have variants:

    op                  bucketed by   key (exact match)                         variants
    decode_attention    length        batch, q_heads, kv_heads, head_dim, dtype  "split:<tokens>" (0 = built-in plan)
    prefill_attention   tokens        q_heads, kv_heads, head_dim, dtype         "tcgen05", "mma.sync"
    linear              m             k, n, dtype                                "tcgen05", "mma.sync"
    rms_norm            rows          hidden_size, dtype                         the reference's own rows are accepted

Profile rows: {"op": ..., <key fields>, <bucket field>, "variants_us": {variant: microseconds}}.
A reference RMSNorm row ({"rows", "hidden_size", "dtype", "native_eager_us", "triton_us",
"inductor_us"?}) is read as op "rms_norm" with variants native / triton / inductor.
`python llm-compiler_b200/profile_dispatch.py` measures such a file on the GPU.
"""

from __future__ import annotations

import json
import math
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, Iterable, List, Optional, Tuple


class ProfileError(ValueError):
    """The profile does not follow schema version 1."""


# op -> (bucket field, key fields)
OPERATORS: Dict[str, Tuple[str, Tuple[str, ...]]] = {
    "decode_attention": ("length", ("batch", "q_heads", "kv_heads", "head_dim", "dtype")),
    "prefill_attention": ("tokens", ("q_heads", "kv_heads", "head_dim", "dtype")),
    "linear": ("m", ("k", "n", "dtype")),
    "rms_norm": ("rows", ("hidden_size", "dtype")),
}

# The variant a kernel picks by itself, and how much cheaper (as a fraction) a measured
# alternative must be to replace it: differences inside the measurement noise of a profile
# must not move a call off the plan that was tuned inside the whole decode step.
BUILT_IN_VARIANT: Dict[str, str] = {"decode_attention": "split:0"}
NOISE_MARGIN = 0.05

_DTYPE_ALIASES = {"f16": "fp16", "float16": "fp16", "half": "fp16", "bfloat16": "bf16",
                  "float32": "fp32", "f32": "fp32", "float": "fp32"}


def normalize_dtype(dtype: str) -> str:
    text = str(dtype).lower().replace("torch.", "")
    return _DTYPE_ALIASES.get(text, text)


@dataclass(frozen=True)
class TargetProfile:
    device_name: str = "unknown"
    compute_capability: str = "unknown"
    torch_version: str = "unknown"
    library_version: str = "unknown"


@dataclass(frozen=True)
class ProfileEntry:
    op: str
    key: Tuple[Tuple[str, Any], ...]
    value: int  # the bucketed dimension at which the costs were measured
    costs: Tuple[Tuple[str, float], ...]

    def variant_costs(self) -> Dict[str, float]:
        return dict(self.costs)


@dataclass(frozen=True)
class DispatchVariant:
    min_value: int
    max_value: Optional[int]
    profile_value: int
    variant: str
    estimated_us: float

    def contains(self, value: int) -> bool:
        return value >= self.min_value and (self.max_value is None or value <= self.max_value)


@dataclass(frozen=True)
class DispatchDecision:
    variant: Optional[str]
    source: str  # "default" (no plan), "profile" (a bucket matched), "fallback" (plan, no bucket)
    profile_value: Optional[int] = None
    estimated_us: Optional[float] = None


def _positive_int(row: Dict[str, Any], name: str) -> int:
    value = row.get(name)
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ProfileError(f"profile row: {name} must be a positive integer, got {value!r}")
    return value


def _parse_entry(row: Any) -> ProfileEntry:
    if not isinstance(row, dict):
        raise ProfileError("profile rows must be objects")
    op = row.get("op")
    if op is None and "hidden_size" in row and "rows" in row:  # a row of the reference's own profiler
        op = "rms_norm"
        costs = {name: row[field_name] for name, field_name in
                 (("native", "native_eager_us"), ("triton", "triton_us"), ("inductor", "inductor_us"))
                 if row.get(field_name) is not None}
    else:
        costs = row.get("variants_us")
    if op not in OPERATORS:
        raise ProfileError(f"profile row: unknown op {op!r}")
    if not isinstance(costs, dict) or not costs:
        raise ProfileError(f"profile row of {op}: variants_us must be a non-empty object")
    bucket_field, key_fields = OPERATORS[op]
    key = []
    for name in key_fields:
        if name not in row:
            raise ProfileError(f"profile row of {op}: missing {name}")
        key.append((name, normalize_dtype(row[name]) if name == "dtype" else _positive_int(row, name)))
    parsed = []
    for variant, cost in costs.items():
        if not isinstance(cost, (int, float)) or isinstance(cost, bool) or not cost > 0 or \
                not math.isfinite(cost):
            raise ProfileError(f"profile row of {op}: cost of {variant!r} must be a positive number")
        parsed.append((str(variant), float(cost)))
    return ProfileEntry(op, tuple(key), _positive_int(row, bucket_field), tuple(sorted(parsed)))


def _key(op: str, fields: Dict[str, Any]) -> Tuple[Tuple[str, Any], ...]:
    if op not in OPERATORS:
        raise ProfileError(f"unknown op {op!r}")
    out = []
    for name in OPERATORS[op][1]:
        if name not in fields:
            raise ProfileError(f"{op}: key field {name} is missing")
        out.append((name, normalize_dtype(fields[name]) if name == "dtype" else int(fields[name])))
    return tuple(out)


@dataclass
class DispatchCostModel:
    """Measured costs of kernel variants, queried per operator and key."""

    target: TargetProfile = field(default_factory=TargetProfile)
    entries: List[ProfileEntry] = field(default_factory=list)
    source: str = "memory"

    @classmethod
    def load(cls, path: str | Path) -> "DispatchCostModel":
        path = Path(path)
        return cls.from_dict(json.loads(path.read_text(encoding="utf-8")), source=str(path))

    @classmethod
    def packaged(cls) -> "DispatchCostModel":
        """The profile measured on a B200 with `profile_dispatch.py` that ships with the package."""

        return cls.load(Path(__file__).resolve().parent / "dispatch_profile_b200.json")

    @classmethod
    def from_dict(cls, payload: Any, *, source: str = "memory") -> "DispatchCostModel":
        if isinstance(payload, list):  # the reference also accepts a bare list of rows
            target_data, rows = {}, payload
        elif isinstance(payload, dict):
            if payload.get("schema_version") != 1:
                raise ProfileError("unsupported profile schema_version")
            target_data, rows = payload.get("target", {}), payload.get("results", [])
        else:
            raise ProfileError("a profile is an object or a list of rows")
        if not isinstance(rows, list) or not isinstance(target_data, dict):
            raise ProfileError("profile: results must be a list and target an object")
        target = TargetProfile(
            device_name=str(target_data.get("device_name", "unknown")),
            compute_capability=str(target_data.get("compute_capability", "unknown")),
            torch_version=str(target_data.get("torch_version", "unknown")),
            library_version=str(target_data.get("library_version",
                                                target_data.get("triton_version", "unknown"))))
        return cls(target, [_parse_entry(row) for row in rows], source)

    def variants(self, op: str, *, allowed: Optional[Iterable[str]] = None,
                 **key_fields: Any) -> List[DispatchVariant]:
        """One variant per profiled value of the bucketed dimension: the cheapest allowed one
        (the kernel's built-in choice unless another is more than NOISE_MARGIN cheaper), owning
        the values up to floor(sqrt(this * next)) (cost_model.py:150-153)."""

        key = _key(op, key_fields)
        allowed_set = None if allowed is None else set(allowed)
        candidates = sorted((e for e in self.entries if e.op == op and e.key == key),
                            key=lambda entry: entry.value)
        merged: Dict[int, Dict[str, float]] = {}
        for entry in candidates:  # rows measured at the same value complement each other
            merged.setdefault(entry.value, {}).update(entry.variant_costs())
        values = sorted(merged)
        thresholds = [math.floor(math.sqrt(a * b)) for a, b in zip(values, values[1:])]
        out, minimum = [], 1
        for index, value in enumerate(values):
            maximum = thresholds[index] if index < len(thresholds) else None
            costs = {name: cost for name, cost in merged[value].items()
                     if allowed_set is None or name in allowed_set}
            if not costs:
                raise ProfileError(f"{op} at {OPERATORS[op][0]}={value}: no allowed variant")
            best = min(sorted(costs), key=costs.get)
            built_in = BUILT_IN_VARIANT.get(op)
            if built_in in costs and costs[built_in] <= costs[best] * (1.0 + NOISE_MARGIN):
                best = built_in
            out.append(DispatchVariant(minimum, maximum, value, best, costs[best]))
            minimum = maximum + 1 if maximum is not None else minimum
        return out

    def plan_attribute(self, op: str, *, fallback: Optional[str] = None,
                       allowed: Optional[Iterable[str]] = None, **key_fields: Any) -> Dict[str, Any]:
        """The `lowering_plan` attribute of one operation (cost_model.py:188-204)."""

        variants = self.variants(op, allowed=allowed, **key_fields)
        return {"schema_version": 1, "profile_source": self.source, "target": asdict(self.target),
                "op": op, "bucketed_by": OPERATORS[op][0], "key": dict(_key(op, key_fields)),
                "fallback": fallback, "variants": [asdict(variant) for variant in variants]}


def select_variant(variants: Iterable[Any], value: int) -> Optional[DispatchVariant]:
    for item in variants:
        variant = item if isinstance(item, DispatchVariant) else DispatchVariant(**item)
        if variant.contains(value):
            return variant
    return None


def resolve_dispatch_plan(plan: Optional[Dict[str, Any]], value: int, *,
                          default_variant: Optional[str] = None) -> DispatchDecision:
    """Picks the variant for a run-time value of the bucketed dimension
    (resolve_lowering_plan, cost_model.py:220-245)."""

    if value <= 0:
        raise ProfileError("the run-time value of the bucketed dimension must be positive")
    if not plan:
        return DispatchDecision(default_variant, "default")
    variant = select_variant(plan.get("variants", []), value)
    if variant is None:
        return DispatchDecision(plan.get("fallback", default_variant), "fallback")
    return DispatchDecision(variant.variant, "profile", variant.profile_value, variant.estimated_us)


def split_tokens_of(variant: Optional[str]) -> int:
    """"split:<tokens>" -> tokens; anything else (None, the built-in plan) -> 0."""

    if variant and variant.startswith("split:"):
        tokens = int(variant[len("split:"):])
        if tokens < 0:
            raise ProfileError(f"bad decode attention variant {variant!r}")
        return tokens
    return 0
