"""Per-kernel micro-benchmarks of the serve.* operator surface (one JSON line per case).

    python llm-compiler_b200/microbench.py decode_attention --batch 64 --length 4096
    python llm-compiler_b200/microbench.py decode_attention --sweep
    python llm-compiler_b200/microbench.py prefill_attention --batch 4 --tokens 4096
    python llm-compiler_b200/microbench.py linear --m 64 --k 896 --n 9728 --epilogue swiglu
    python llm-compiler_b200/microbench.py kv_store --batch 16 --tokens 4096
    python llm-compiler_b200/microbench.py timeline --batch 64 --length 4096   (trace build only)
    python llm-compiler_b200/microbench.py profile --output dispatch_profile.json

Timing: CUDA events on the launching stream around `--iters` launches after `--warmup`
launches, rotating over enough independent buffer sets that one round exceeds the 126 MB L2
(so every launch reads from HBM). Reported bytes / flops are the algorithmic ones:
  decode attention  512 * sum(len) + 3592 * B bytes at 14/2 heads x 64 (K and V read once, Q,
                    O, lengths); 4 * Hq * D * sum(len) flops
  prefill attention 2 * B * Hq * T^2 * D flops (causal half of 4 * B * Hq * T^2 * D)
  KV store          2 * (read + write) * B * Hkv * T * D * 2 bytes
  linear            2 * M * K * N flops; (M*K + N*K + M*N) * 2 bytes
Also the small-case target for `ncu -k regex:<kernel>` captures.
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

    def launch(index):
        kernels.b200_decode_attention(query, keys[index], values[index], lengths, None,
                                      scale=d ** -0.5, split_tokens=args.split_tokens,
                                      max_length_hint=length, output=output,
                                      numerical_mode=args.mode)

    timer = time_launches if args.no_graph else graph_time
    seconds = timer(launch, sets, args.warmup, args.iters)
    algorithmic = kv_bytes + 2 * batch * hq * d * 2 + 8 * batch
    flops = 4 * hq * d * total
    return {"op": "decode_attention", "batch": batch, "max_length": length, "buffer_rows": rows,
            "sum_lengths": total, "q_heads": hq, "kv_heads": hkv, "head_dim": d,
            "split_tokens": args.split_tokens, "buffer_sets": sets, "us": seconds * 1e6,
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


def kv_store_case(args):
    b, t, hkv, d = args.batch, args.tokens, args.kv_heads, args.head_dim
    capacity = args.capacity or 2 * t
    nbytes = 2 * 2 * b * hkv * t * d * 2
    sets = sets_for(nbytes)
    keys = [torch.randn(b, t, hkv, d, device="cuda").bfloat16().transpose(1, 2) for _ in range(sets)]
    buffers = [torch.zeros(b, capacity, hkv, d, device="cuda", dtype=torch.bfloat16)
               for _ in range(sets)]
    positions = torch.zeros(b, dtype=torch.int64, device="cuda")

    def launch(index):
        kernels.b200_kv_store(buffers[index], buffers[index], keys[index], keys[index], positions)

    seconds = graph_time(launch, sets, args.warmup, args.iters)
    return {"op": "kv_store", "batch": b, "tokens": t, "us": seconds * 1e6,
            "gbs": nbytes / seconds / 1e9, "algorithmic_bytes": nbytes}


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


def rms_norm_case(args):
    rows, hidden = args.m, args.k
    sets = sets_for(rows * hidden * 4)
    xs = [torch.randn(rows, hidden, device="cuda").bfloat16() for _ in range(sets)]
    w = torch.randn(hidden, device="cuda").bfloat16()

    def launch(index):
        kernels.b200_rms_norm(xs[index], w, epsilon=1e-6, round_before_weight=True,
                              numerical_mode=args.mode)

    seconds = graph_time(launch, sets, args.warmup, args.iters)
    return {"op": "rms_norm", "rows": rows, "hidden": hidden, "mode": args.mode,
            "us": seconds * 1e6, "gbs": rows * hidden * 4 / seconds / 1e9}


def prefill_step_case(args):
    """Stateful prefill of --batch prompts of --tokens tokens through Qwen2Engine.prefill (Qwen2-0.5B
    or, with --model qwen2-7b, Qwen2-7B architecture; random weights, random token ids): embedding,
    RoPE table, then per layer RMSNorm, q|k|v GEMM, RoPE, KV store, causal attention, o GEMM with the
    residual, RMSNorm, gate|up GEMM with SwiGLU, down GEMM with the residual; last-position logits
    and the greedy token. Prompt tokens per second, device-timed."""

    from llm_compiler_b200 import qwen2 as q2
    from llm_compiler_b200.engine import Qwen2Engine

    device = torch.device("cuda", torch.cuda.current_device())
    config = q2.QWEN2_7B if args.model == "qwen2-7b" else q2.QWEN2_0_5B
    weights = q2.make_weights(config, seed=0, dtype=torch.bfloat16, device=device, reproducible=False)
    engine = Qwen2Engine(config, weights, batch=args.batch, capacity=args.tokens + 64)
    ids = torch.randint(0, config.vocab_size, (args.batch, args.tokens), device=device)
    seconds = time_launches(lambda _: engine.prefill(ids), 1, min(args.warmup, 3), min(args.iters, 10))
    layer_params = (config.hidden_size * (config.q_size + 2 * config.kv_size) + config.q_size * config.hidden_size +
                    3 * config.hidden_size * config.intermediate_size)
    tokens = args.batch * args.tokens
    gemm_flops = 2 * tokens * layer_params * config.num_layers
    attention_flops = 2 * args.batch * config.num_heads * args.tokens ** 2 * config.head_dim * config.num_layers
    return {"op": "prefill_step", "model": args.model, "batch": args.batch, "tokens": args.tokens,
            "ms": seconds * 1e3, "prompt_tokens_per_s": tokens / seconds,
            "tflops": (gemm_flops + attention_flops) / seconds / 1e12,
            "gemm_tflop": gemm_flops / 1e12, "causal_attention_tflop": attention_flops / 1e12}


def timeline_case(args):
    """Per-launch device timeline of one replayed decode step (Qwen2-0.5B architecture, random
    weights, synthetic KV of --length tokens). Needs the library built with
    B200_NVCC_EXTRA=-DB200_TRACE: thread 0 of every CTA of the chain kernels then records
    %globaltimer at its top, after its dependency wait, once in the middle and at its end.
    Printed per launch, in microseconds from the first record: when its CTAs became resident
    (top), when the dependency wait returned (wait), the middle mark (GEMM: accumulator
    complete; attention: streaming done) and the end marks."""

    import ctypes
    import statistics

    from llm_compiler_b200 import _lib
    from llm_compiler_b200 import qwen2 as q2
    from llm_compiler_b200.engine import Qwen2Engine

    library = _lib.load()
    if not hasattr(library, "b200_trace_attach"):
        raise SystemExit("this libb200serve.so was built without -DB200_TRACE "
                         "(B200_NVCC_EXTRA=-DB200_TRACE python llm-compiler_b200/build.py --force)")
    library.b200_trace_attach.argtypes = [ctypes.c_void_p]
    device = torch.device("cuda", torch.cuda.current_device())
    config = q2.QWEN2_0_5B
    weights = q2.make_weights(config, seed=0, dtype=torch.bfloat16, device=device,
                              reproducible=False)
    engine = Qwen2Engine(config, weights, batch=args.batch, capacity=args.length + 128)
    engine.max_length_hint = args.length + 128
    generator = torch.Generator(device=device).manual_seed(0)
    for layer in range(config.num_layers):
        engine.state.keys[layer].normal_(generator=generator)
        engine.state.values[layer].normal_(generator=generator)
    engine.load_context(torch.full((args.batch,), args.length),
                        next_ids=torch.randint(0, config.vocab_size, (args.batch,)))
    engine.capture()
    for _ in range(5):
        engine.decode_step()
    torch.cuda.synchronize()
    records = 65536
    buffer = torch.zeros(1 + 8 * records + 1 + 64 * 512, dtype=torch.int64, device=device)
    library.b200_trace_attach(buffer.data_ptr())
    engine.decode_step()
    torch.cuda.synchronize()
    library.b200_trace_attach(None)
    host = buffer.cpu()
    count = min(int(host[0]), records)
    names = {1: "linear_tcgen05", 2: "reduce_residual_rms_norm", 3: "reduce_rope_kv_store",
             4: "decode_attention"}
    rows = []
    for r in host[1:1 + 8 * count].view(count, 8).tolist():
        rows.append({"kernel": names.get(r[0] & 0xffff, str(r[0] & 0xffff)), "top": r[1],
                     "wait": r[3], "end": r[5], "middle": r[7]})
    rows.sort(key=lambda r: r["wait"] or r["top"])
    origin = min(r["top"] for r in rows)
    launches = []
    for r in rows:
        if launches and launches[-1][0]["kernel"] == r["kernel"] and \
                r["wait"] - launches[-1][0]["wait"] < 1500:
            launches[-1].append(r)
        else:
            launches.append([r])

    def us(values):
        values = [(v - origin) / 1000.0 for v in values if v]
        return (min(values), statistics.median(values), max(values)) if values else (0, 0, 0)

    print(f"{len(rows)} CTA records, {len(launches)} launches; microseconds from the first record")
    print(f"{'kernel':26s} {'ctas':>4s} {'top max':>8s} {'wait':>8s} {'mid min':>8s} {'mid max':>8s} "
          f"{'end min':>8s} {'end med':>8s} {'end max':>8s} {'wait->end':>9s}")
    for launch in launches[:args.launches]:
        top, wait = us([r["top"] for r in launch]), us([r["wait"] for r in launch])
        middle, end = us([r["middle"] for r in launch]), us([r["end"] for r in launch])
        print(f"{launch[0]['kernel']:26s} {len(launch):4d} {top[2]:8.2f} {wait[2]:8.2f} {middle[0]:8.2f} "
              f"{middle[2]:8.2f} {end[0]:8.2f} {end[1]:8.2f} {end[2]:8.2f} {end[2] - wait[2]:9.2f}")
    return {"op": "timeline", "batch": args.batch, "context": args.length, "launches": len(launches),
            "records": len(rows)}


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
    for batch in (1, 8, 64, 256):
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


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("op", choices=["decode_attention", "prefill_attention", "kv_store", "linear",
                                       "rms_norm", "timeline", "profile", "prefill_step"])
    parser.add_argument("--model", default="qwen2-0.5b", choices=["qwen2-0.5b", "qwen2-7b"],
                        help="prefill_step: architecture")
    parser.add_argument("--output", default="dispatch_profile.json", help="profile: file to write")
    parser.add_argument("--launches", type=int, default=40, help="timeline: launches to print")
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
    parser.add_argument("--full-length", action="store_true",
                        help="every sequence at --length instead of uniform [64, length]")
    parser.add_argument("--sweep", action="store_true",
                        help="decode attention over batch {1,8,64,256} x length {64,1024,4096,32768}")
    parser.add_argument("--no-graph", action="store_true")
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--iters", type=int, default=100)
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("microbench.py needs a CUDA device")
    if args.op == "decode_attention":
        shapes = [(b, l) for b in (1, 8, 64, 256) for l in (64, 1024, 4096, 32768)] \
            if args.sweep else [(args.batch, args.length)]
        for batch, length in shapes:
            print(json.dumps(decode_attention_case(args, batch, length)), flush=True)
    elif args.op == "prefill_attention":
        print(json.dumps(prefill_attention_case(args)))
    elif args.op == "kv_store":
        print(json.dumps(kv_store_case(args)))
    elif args.op == "linear":
        print(json.dumps(linear_case(args)))
    elif args.op == "timeline":
        print(json.dumps(timeline_case(args)))
    elif args.op == "profile":
        print(json.dumps(profile_case(args)))
    elif args.op == "prefill_step":
        print(json.dumps(prefill_step_case(args)))
    else:
        print(json.dumps(rms_norm_case(args)))
    kernels.runtime().check_status()


if __name__ == "__main__":
    main()
