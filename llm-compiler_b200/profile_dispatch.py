"""Measures the kernel variants the profile-guided dispatch plan chooses between and writes a
schema-version-1 profile (dispatch_plan.py), the B200 counterpart of the reference's RMSNorm
profile benchmark (benchmarks/bench_rmsnorm.py -> cost_model.py:94-123):

    python llm-compiler_b200/profile_dispatch.py --output dispatch_profile.json

  decode attention   split sizes, by (batch, context length), all sequences at full length
  prefill attention  tcgen05 or warp-level kernel, by tokens
  linear             tcgen05 or warp-level kernel, by rows, for the Qwen2-0.5B weight shapes

`kernel_ir.select_dispatch_plans(module, DispatchCostModel.from_file(path))` turns the file into
`lowering_plan` attributes; the profile that ships as dispatch_profile_b200.json was measured
with this tool. Timing: CUDA events on the launching stream around replays of a CUDA graph of
the launches, rotating over enough independent buffer sets that one round exceeds the 126 MB L2.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import llm_compiler_b200 as b200  # noqa: E402
from llm_compiler_b200 import kernels  # noqa: E402

L2_BYTES = 126 * 1024 * 1024


def time_launches(launch, sets, warmup, iters):
    for index in range(warmup):
        launch(index % sets)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for index in range(iters):
        launch(index % sets)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e-3 / iters


def graph_time(launch, sets, warmup, iters):
    """Same, but the `sets` launches of one round are replayed from a CUDA graph so that host
    launch overhead does not pollute kernels that last a few microseconds."""

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for index in range(sets):
            launch(index)
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for index in range(sets):
            launch(index)
    rounds = max(1, iters // sets)
    for _ in range(max(1, warmup // sets)):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(rounds):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) * 1e-3 / (rounds * sets)


def sets_for(bytes_per_set, limit=16):
    return int(min(limit, max(1, -(-2 * L2_BYTES // max(1, bytes_per_set)))))


def decode_attention_case(args, batch, length):
    hq, hkv, d = args.q_heads, args.kv_heads, args.head_dim
    capacity = args.capacity or max(length, 64)
    generator = torch.Generator(device="cuda").manual_seed(batch * 10000 + length)
    lengths = torch.randint(min(64, length), length + 1, (batch,), generator=generator,
                            device="cuda") if not args.full_length else \
        torch.full((batch,), length, device="cuda", dtype=torch.int64)
    total = int(lengths.sum())
    kv_bytes = 2 * total * hkv * d * 2
    sets = sets_for(kv_bytes)
    # only the first max(len) rows of each buffer are touched: allocate what is read
    rows = int(lengths.max())
    keys = [torch.randn(batch, rows, hkv, d, generator=generator, device="cuda",
                        dtype=torch.float32).bfloat16() for _ in range(sets)]
    values = [torch.randn_like(k) for k in keys]
    query = torch.randn(batch, hq, 1, d, device="cuda", dtype=torch.bfloat16)
    output = torch.empty_like(query)

    order = kernels.sequence_order_of(lengths) if getattr(args, "longest_first", False) else None

    def launch(index):
        kernels.b200_decode_attention(query, keys[index], values[index], lengths, None,
                                      scale=d ** -0.5, split_tokens=args.split_tokens,
                                      max_length_hint=length, output=output,
                                      numerical_mode=args.mode, sequence_order=order)

    timer = time_launches if args.no_graph else graph_time
    seconds = timer(launch, sets, args.warmup, args.iters)
    algorithmic = kv_bytes + 2 * batch * hq * d * 2 + 8 * batch
    flops = 4 * hq * d * total
    return {"op": "decode_attention", "batch": batch, "max_length": length, "buffer_rows": rows,
            "sum_lengths": total, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
            "split_tokens": args.split_tokens, "longest_first": order is not None,
            "buffer_sets": sets, "us": seconds * 1e6,
            "gbs": algorithmic / seconds / 1e9, "tflops": flops / seconds / 1e12,
            "algorithmic_bytes": algorithmic}


def prefill_attention_case(args):
    b, t, hq, hkv, d = args.batch, args.tokens, args.q_heads, args.kv_heads, args.head_dim
    generator = torch.Generator(device="cuda").manual_seed(b * 10000 + t)
    q = torch.randn(b, t, hq, d, generator=generator, device="cuda").bfloat16().transpose(1, 2)
    k = torch.randn(b, t, hkv, d, generator=generator, device="cuda").bfloat16().transpose(1, 2)
    v = torch.randn(b, t, hkv, d, generator=generator, device="cuda").bfloat16().transpose(1, 2)
    mask = None
    if args.general_mask:
        future = torch.triu(torch.ones(t, t, dtype=torch.bool, device="cuda"), diagonal=1)
        mask = torch.zeros(b, 1, t, t, device="cuda").masked_fill(future, float("-inf"))

    def launch(_):
        kernels.b200_prefill_attention(q, k, v, mask, scale=d ** -0.5, causal=mask is None,
                                       numerical_mode=args.mode)

    seconds = time_launches(launch, 1, args.warmup, args.iters)
    flops = 2 * b * hq * t * t * d
    return {"op": "prefill_attention", "batch": b, "tokens": t, "general_mask": bool(args.general_mask),
            "us": seconds * 1e6, "tflops_causal": flops / seconds / 1e12}


def linear_case(args):
    m, k, n = args.m, args.k, args.n
    sets = sets_for(n * k * 2)
    x = torch.randn(m, k, device="cuda").bfloat16()
    weights = [(torch.randn(n, k, device="cuda") * 0.02).bfloat16() for _ in range(sets)]
    residual = torch.randn(m, n, device="cuda").bfloat16() if args.epilogue == "residual" else None

    def launch(index):
        kernels.b200_linear(x, weights[index], residual=residual, epilogue=args.epilogue)

    timer = time_launches if m > 1024 else graph_time
    seconds = timer(launch, sets, args.warmup, args.iters)
    nbytes = (m * k + n * k + m * n) * 2
    return {"op": "linear", "m": m, "k": k, "n": n, "epilogue": args.epilogue, "us": seconds * 1e6,
            "gbs": nbytes / seconds / 1e9, "tflops": 2 * m * k * n / seconds / 1e12}


def profile_case(args):
    """Measures the variants the dispatch plan chooses between and writes a schema-version-1
    profile (dispatch_plan.py): decode attention split sizes by (batch, context length), prefill
    attention and linear kernel paths by tokens / rows. All sequences at full length."""

    import copy

    rows = []
    probe = copy.copy(args)
    probe.full_length, probe.no_graph, probe.general_mask = True, False, False
    probe.warmup, probe.iters = max(3, args.warmup // 2), max(10, args.iters // 4)
    layout = {"q_heads": args.q_heads, "kv_heads": args.kv_heads, "head_dim": args.head_dim,
              "dtype": "bf16"}
    for batch in (1, 8, 16, 32, 64, 128, 256):
        for length in (256, 1024, 4096, 16384, 32768):
            costs = {}
            for split in (0, 512, 1024, 2048, 4096, 8192):
                if split > length:
                    continue
                probe.split_tokens = split
                costs[f"split:{split}"] = decode_attention_case(probe, batch, length)["us"]
            rows.append({"op": "decode_attention", "batch": batch, **layout, "length": length,
                         "variants_us": costs})
            print(json.dumps(rows[-1]), flush=True)
    for tokens in (128, 512, 2048, 4096):
        probe.batch, probe.tokens = 4, tokens
        costs = {}
        for variant in ("tcgen05", "mma.sync"):
            with kernels.kernel_variants(prefill_attention=variant):
                costs[variant] = prefill_attention_case(probe)["us"]
        rows.append({"op": "prefill_attention", **layout, "tokens": tokens, "variants_us": costs})
        print(json.dumps(rows[-1]), flush=True)
    probe.epilogue = "none"
    for k, n in ((896, 1152), (896, 9728), (4864, 896)):
        for m in (16, 64, 512, 4096):
            probe.m, probe.k, probe.n = m, k, n
            costs = {}
            for variant in ("tcgen05", "mma.sync"):
                with kernels.kernel_variants(linear=variant):
                    costs[variant] = linear_case(probe)["us"]
            rows.append({"op": "linear", "k": k, "n": n, "dtype": "bf16", "m": m, "variants_us": costs})
            print(json.dumps(rows[-1]), flush=True)
    properties = torch.cuda.get_device_properties(0)
    payload = {"schema_version": 1,
               "target": {"device_name": properties.name,
                          "compute_capability": f"{properties.major}.{properties.minor}",
                          "torch_version": torch.__version__,
                          "library_version": str(b200._lib.load().b200_abi_version())},
               "results": rows}
    Path(args.output).write_text(json.dumps(payload, indent=1) + "\n", encoding="utf-8")
    return {"op": "profile", "rows": len(rows), "output": args.output}


def measurement_arguments(parser: argparse.ArgumentParser) -> None:
    """The options the case functions read (shared with the repository's microbench.py)."""

    parser.add_argument("--batch", type=int, default=64)
    parser.add_argument("--length", type=int, default=4096)
    parser.add_argument("--tokens", type=int, default=512)
    parser.add_argument("--capacity", type=int, default=0)
    parser.add_argument("--q-heads", type=int, default=14)
    parser.add_argument("--kv-heads", type=int, default=2)
    parser.add_argument("--head-dim", type=int, default=64)
    parser.add_argument("--split-tokens", type=int, default=None,
                        help="decode attention: tokens per KV split; 0 = the library's built-in "
                             "plan; default: the profile-guided plan")
    parser.add_argument("--m", type=int, default=64)
    parser.add_argument("--k", type=int, default=896)
    parser.add_argument("--n", type=int, default=896)
    parser.add_argument("--epilogue", default="none")
    parser.add_argument("--mode", default="fast")
    parser.add_argument("--general-mask", action="store_true")
    parser.add_argument("--longest-first", action="store_true",
                        help="decode attention: hand the sequences to the GPU longest first")
    parser.add_argument("--full-length", action="store_true",
                        help="every sequence at --length instead of uniform [64, length]")
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--iters", type=int, default=100)


def main():
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--output", default="dispatch_profile.json", help="file to write")
    measurement_arguments(parser)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("profile_dispatch.py needs a CUDA device")
    print(json.dumps(profile_case(args)))
    kernels.runtime().check_status()


if __name__ == "__main__":
    main()
