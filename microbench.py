"""Per-kernel measurements of the serve.* operator surface (one JSON line per case): the numbers
behind profiles/, the small-case targets of the ncu captures, and the side-by-side run against
the reference's own Triton kernels.

    python microbench.py decode_attention --batch 64 --length 4096
    python microbench.py decode_attention --sweep
    python microbench.py prefill_attention --batch 4 --tokens 4096
    python microbench.py linear --m 64 --k 896 --n 9728 --epilogue swiglu
    python microbench.py linear_splitk --m 64 --k 4864 --n 896        (o / down of the decode chain)
    python microbench.py linear_rms --m 64 --k 896 --n 9728 --epilogue swiglu   (gate|up, folded norm)
    python microbench.py kv_store --batch 16 --tokens 4096
    python microbench.py prefill_step --model qwen2-0.5b --batch 4 --tokens 4096
    python microbench.py timeline --batch 64 --length 4096      (a -DB200_TRACE build only)
    python microbench.py compare                                (needs baseline/_ref, see below)

Timing: CUDA events on the launching stream around `--iters` launches after `--warmup`
launches, rotating over enough independent buffer sets that one round exceeds the 126 MB L2
(so every launch reads from HBM). Reported bytes / flops are the algorithmic ones:
  decode attention  512 * sum(len) + 3592 * B bytes at 14/2 heads x 64 (K and V read once, Q,
                    O, lengths); 4 * Hq * D * sum(len) flops
  prefill attention 2 * B * Hq * T^2 * D flops (causal half of 4 * B * Hq * T^2 * D)
  KV store          2 * (read + write) * B * Hkv * T * D * 2 bytes
  linear            2 * M * K * N flops; (M*K + N*K + M*N) * 2 bytes

`compare` times this library beside the reference's Triton kernels (triton_decode_attention,
triton_prefill_attention, triton_linear, triton_kv_store, triton_rope, triton_rms_norm), PyTorch
SDPA and F.linear on the same seeded inputs with the reference's own method
(triton.testing.do_bench, 20 ms warm-up, 80 ms of repetitions, median;
benchmarks/bench_decode_attention.py:131-147) and reports the max-abs difference between the two
implementations. The reference package is imported from baseline/_ref (installed there with
`pip install --no-deps --target baseline/_ref <reference checkout>`; not part of this
repository); a reference kernel that fails to compile or run is recorded with its message and
skipped. The product never imports it: the comparison lives in this tool only.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parent))

import llm_compiler_b200 as b200  # noqa: E402,F401
from llm_compiler_b200 import kernels  # noqa: E402
from llm_compiler_b200.profile_dispatch import (  # noqa: E402
    decode_attention_case, graph_time, linear_case, measurement_arguments, prefill_attention_case,
    sets_for, time_launches)

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


def decode_gemm_case(args, form):
    """The two decode-layer projections that have no stand-alone reference op: `splitk` is
    serve.linear + residual add as a cluster split-K launch (o / down), `rms` is serve.rms_norm
    folded into serve.linear (gate|up with --epilogue swiglu). Launched back to back with
    programmatic dependent launch, each launch reading the one before (the residual stream), the
    way the decode chain runs them; weights rotate through more than L2."""

    m, k, n = args.m, args.k, args.n
    sets = sets_for(n * k * 2)
    g = torch.Generator(device="cuda").manual_seed(m + k + n)
    weights = [(torch.randn(n, k, generator=g, device="cuda") * k ** -0.5).bfloat16() for _ in range(sets)]
    x = torch.randn(m, k, generator=g, device="cuda").bfloat16()
    residual = torch.randn(m, n, generator=g, device="cuda").bfloat16()
    norm = (1 + 0.1 * torch.randn(k, generator=g, device="cuda")).bfloat16()
    folded = [kernels.b200_scale_columns(w, norm) for w in weights] if form == "rms" else None
    carry = [residual]

    def launch(index):
        with kernels.launch_mode(programmatic=True, constant_weights=True):
            if form == "splitk":
                carry[0] = kernels.b200_linear_splitk_residual(x, weights[index], carry[0])
            else:
                kernels.b200_linear_rms_input(x, folded[index], epsilon=1e-6, epilogue=args.epilogue)

    seconds = (time_launches if args.no_graph else graph_time)(launch, sets, args.warmup, args.iters)
    return {"op": f"linear_{form}", "m": m, "k": k, "n": n, "epilogue": args.epilogue, "us": seconds * 1e6,
            "gbs": (m * k + n * k + m * n) * 2 / seconds / 1e9}


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
    ids = torch.randint(0, config.vocab_size, (args.batch, args.tokens), device=device)
    if args.path == "executor":
        return prefill_graph_case(args, config, weights, ids)
    engine = Qwen2Engine(config, weights, batch=args.batch, capacity=args.tokens + 64)
    if args.all_logits:
        seconds = time_launches(lambda _: engine.prefill(ids, all_logits=True), 1, min(args.warmup, 3),
                                min(args.iters, 10))
    else:
        seconds = time_launches(lambda _: engine.prefill(ids), 1, min(args.warmup, 3), min(args.iters, 10))
    layer_params = (config.hidden_size * (config.q_size + 2 * config.kv_size) + config.q_size * config.hidden_size +
                    3 * config.hidden_size * config.intermediate_size)
    tokens = args.batch * args.tokens
    gemm_flops = 2 * tokens * layer_params * config.num_layers
    attention_flops = 2 * args.batch * config.num_heads * args.tokens ** 2 * config.head_dim * config.num_layers
    return {"op": "prefill_step", "model": args.model, "batch": args.batch, "tokens": args.tokens,
            "path": "engine", "all_logits": bool(args.all_logits),
            "ms": seconds * 1e3, "prompt_tokens_per_s": tokens / seconds,
            "tflops": (gemm_flops + attention_flops) / seconds / 1e12,
            "gemm_tflop": gemm_flops / 1e12, "causal_attention_tflop": attention_flops / 1e12}


def prefill_graph_case(args, config, weights, ids):
    """The drop-in path for prefill: the reference's own KernelIR of the Qwen2-0.5B prefill
    (exported and compiled by the reference, tests/golden/...json.gz: logits for every position,
    the additive mask an argument of the graph), finished by lower_to_b200 and interpreted by
    B200Executor, eagerly as the reference's executor runs it. Three ways of treating the mask:
    declared causal by the caller, classified on the device by the executor, taken as data."""

    import gzip

    from llm_compiler_b200 import kernel_ir
    from llm_compiler_b200 import qwen2 as q2
    from llm_compiler_b200.executor import B200Executor, bind_arguments

    if args.model != "qwen2-0.5b":
        raise SystemExit("--path executor runs the shipped Qwen2-0.5B prefill graph")
    batch, tokens = ids.shape
    device = ids.device
    future = torch.triu(torch.ones(tokens, tokens, dtype=torch.bool, device=device), diagonal=1)
    mask = torch.zeros(batch, 1, tokens, tokens, device=device).masked_fill(future, float("-inf"))
    positions = torch.arange(tokens, device=device).repeat(batch, 1)
    path = Path(__file__).resolve().parent / "tests" / "golden" / "kernel_ir_qwen2_0_5b_prefill_fast.json.gz"
    rows = []
    for label, declared, classify, last in (("declared causal", ("attention_mask",), True, False),
                                            ("classified on the device", (), True, False),
                                            ("mask as data", (), False, False),
                                            ("declared causal, last-token logits", ("attention_mask",), True, True)):
        module = kernel_ir.module_from_json(json.loads(gzip.open(path).read()))
        kernel_ir.lower_to_b200(module, causal_mask_arguments=declared, last_token_logits=last)
        kernel_ir.require_full_lowering(module)
        executor = B200Executor(strict=True, classify_masks=classify)
        arguments = bind_arguments(module.functions[0], weights, {
            "input_ids": ids, "attention_mask": mask, "position_ids": positions,
            "inv_freq": q2.inverse_frequency(config, device)})
        before = kernels.launch_count(device)
        executor.run(module, arguments)
        launches = kernels.launch_count(device) - before
        seconds = time_launches(lambda _: executor.run(module, arguments), 1, 1, min(args.iters, 5))
        rows.append({"op": "prefill_step", "model": args.model, "batch": batch, "tokens": tokens,
                     "path": "executor", "mask": label, "all_logits": not last, "kernels": launches,
                     "ms": seconds * 1e3, "prompt_tokens_per_s": batch * tokens / seconds})
        print(json.dumps(rows[-1]), flush=True)
        if last:  # the same run captured once and replayed: no interpreter, no launch gaps
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                executor.run(module, arguments)
            seconds = time_launches(lambda _: graph.replay(), 1, 1, min(args.iters, 5))
            rows.append(dict(rows[-1], mask=label + ", one CUDA graph", ms=seconds * 1e3,
                             prompt_tokens_per_s=batch * tokens / seconds))
            print(json.dumps(rows[-1]), flush=True)
            del graph
        del executor, module, arguments
        torch.cuda.empty_cache()
    return {"op": "prefill_step", "path": "executor", "variants": len(rows)}


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
    if args.model == "qwen2-7b":  # four full-width layers show the chain; the rest only repeat it
        import dataclasses
        config = dataclasses.replace(q2.QWEN2_7B, num_layers=4)
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


def compare_case(args):
    """This library beside the reference's Triton kernels, SDPA and F.linear: same seeded
    inputs, the reference's timing method, max-abs difference between the two."""

    reference_root = Path(__file__).resolve().parent / "baseline" / "_ref"
    if not (reference_root / "stateful_llm_compiler").is_dir():
        print(json.dumps({"op": "compare", "unavailable": "baseline/_ref holds no reference install"}))
        return
    sys.path.insert(0, str(reference_root))
    import torch.nn.functional as F
    import triton.testing

    try:
        from stateful_llm_compiler import backends as reference
    except Exception as error:  # the whole package failed to import: say so once
        print(json.dumps({"op": "compare", "unavailable": f"{type(error).__name__}: {error}"[:300]}))
        return

    def bench(call):
        return triton.testing.do_bench(call, warmup=20, rep=80, return_mode="median") * 1e3  # us

    def row(op, shape, ours, theirs, extra=None, unit_bytes=None, flops=None):
        """Times `ours` and the callables in `theirs` (name -> call); a reference call that
        raises is recorded with its message and not retried."""
        result = {"op": op, **shape}
        mine = ours()
        result["b200_us"] = bench(ours)
        for name, call in theirs.items():
            try:
                value = call()
                result[f"{name}_us"] = bench(call)
                if isinstance(value, torch.Tensor) and value.shape == mine.shape:
                    result[f"max_abs_vs_{name}"] = float((value.float() - mine.float()).abs().max())
            except Exception as error:
                result[f"{name}_error"] = f"{type(error).__name__}: {error}"[:200]
        if unit_bytes:
            result["b200_gbs"] = unit_bytes / result["b200_us"] / 1e3
        if flops:
            result["b200_tflops"] = flops / result["b200_us"] / 1e6
        if extra:
            result.update(extra)
        print(json.dumps(result), flush=True)

    hq, hkv, d = 14, 2, 64
    for batch in (8, 64):
        for length in (1024, 4096):
            g = torch.Generator(device="cuda").manual_seed(batch * 10000 + length)
            q = torch.randn(batch, hq, 1, d, generator=g, device="cuda").bfloat16()
            k = torch.randn(batch, length, hkv, d, generator=g, device="cuda").bfloat16()
            v = torch.randn(batch, length, hkv, d, generator=g, device="cuda").bfloat16()
            lengths = torch.full((batch,), length, device="cuda", dtype=torch.int64)
            mask = torch.zeros(batch, 1, 1, length, device="cuda")

            def sdpa():
                key = k.permute(0, 2, 1, 3).repeat_interleave(hq // hkv, dim=1)
                value = v.permute(0, 2, 1, 3).repeat_interleave(hq // hkv, dim=1)
                return F.scaled_dot_product_attention(q, key, value, attn_mask=mask.to(q.dtype),
                                                      dropout_p=0.0, scale=d ** -0.5)

            row("decode_attention", {"batch": batch, "capacity": length, "length": length},
                lambda: kernels.b200_decode_attention(q, k, v, lengths, mask, scale=d ** -0.5),
                {"reference_triton": lambda: reference.triton_decode_attention(q, k, v, lengths, mask,
                                                                               scale=d ** -0.5),
                 "torch_sdpa": sdpa},
                unit_bytes=4 * hkv * d * batch * length)
    for tokens in (512, 2048):
        batch = 4
        g = torch.Generator(device="cuda").manual_seed(batch * 10000 + tokens)
        q = torch.randn(batch, tokens, hq, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
        k = torch.randn(batch, tokens, hkv, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
        v = torch.randn(batch, tokens, hkv, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
        future = torch.triu(torch.ones(tokens, tokens, dtype=torch.bool, device="cuda"), diagonal=1)
        mask = torch.zeros(batch, 1, tokens, tokens, device="cuda").masked_fill(future, float("-inf"))

        def sdpa_prefill():
            return F.scaled_dot_product_attention(q, k.repeat_interleave(hq // hkv, dim=1),
                                                  v.repeat_interleave(hq // hkv, dim=1), is_causal=True,
                                                  scale=d ** -0.5)

        shape = {"batch": batch, "tokens": tokens}
        flops = 2 * batch * hq * tokens * tokens * d
        row("prefill_attention(mask)", shape,
            lambda: kernels.b200_prefill_attention(q, k, v, mask, scale=d ** -0.5),
            {"reference_triton": lambda: reference.triton_prefill_attention(q, k, v, mask, scale=d ** -0.5)},
            flops=flops)
        row("prefill_attention(causal proved)", shape,
            lambda: kernels.b200_prefill_attention(q, k, v, None, scale=d ** -0.5, causal=True),
            {"reference_triton": lambda: reference.triton_prefill_attention(q, k, v, mask, scale=d ** -0.5),
             "torch_sdpa": sdpa_prefill}, flops=flops)
    for m in (64, 4096):
        for name, k_dim, n_dim, bias in (("q|k|v", 896, 1152, True), ("o", 896, 896, False),
                                         ("gate", 896, 4864, False), ("down", 4864, 896, False),
                                         ("lm_head", 896, 151936, False)):
            if m == 4096 and name == "lm_head":
                continue
            g = torch.Generator(device="cuda").manual_seed(m + k_dim + n_dim)
            x = torch.randn(m, k_dim, generator=g, device="cuda").bfloat16()
            w = (torch.randn(n_dim, k_dim, generator=g, device="cuda") * k_dim ** -0.5).bfloat16()
            b = torch.randn(n_dim, generator=g, device="cuda").bfloat16() if bias else None
            row("linear", {"name": name, "m": m, "k": k_dim, "n": n_dim},
                lambda: kernels.b200_linear(x, w, b),
                {"reference_triton": lambda: reference.triton_linear(x, w, b),
                 "torch_f_linear": lambda: F.linear(x, w, b)},
                unit_bytes=(m * k_dim + n_dim * k_dim + m * n_dim) * 2, flops=2 * m * k_dim * n_dim)
    for batch, tokens in ((64, 1), (4, 2048)):
        g = torch.Generator(device="cuda").manual_seed(tokens)
        capacity = 4096
        key = torch.randn(batch, tokens, hkv, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
        value = torch.randn(batch, tokens, hkv, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
        positions = torch.full((batch,), 7, device="cuda", dtype=torch.int64)
        mine = [torch.zeros(batch, capacity, hkv, d, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
        theirs = [torch.zeros_like(mine[0]) for _ in range(2)]

        def ours_store():
            kernels.b200_kv_store(mine[0], mine[1], key, value, positions)
            return mine[0]

        def their_store():
            reference.triton_kv_store(theirs[0], theirs[1], key, value, positions)
            return theirs[0]

        row("kv_store", {"batch": batch, "tokens": tokens}, ours_store, {"reference_triton": their_store},
            unit_bytes=2 * 2 * batch * hkv * tokens * d * 2)
        q = torch.randn(batch, tokens, hq, d, generator=g, device="cuda").bfloat16().transpose(1, 2)
        cosine = torch.randn(batch, tokens, d, generator=g, device="cuda").bfloat16()
        sine = torch.randn(batch, tokens, d, generator=g, device="cuda").bfloat16()
        row("rope", {"batch": batch, "tokens": tokens},
            lambda: kernels.b200_rope(q, key, cosine, sine)[0],
            {"reference_triton": lambda: reference.triton_rope(q, key, cosine, sine)[0]})
    for rows in (64, 16384):
        g = torch.Generator(device="cuda").manual_seed(rows)
        x = torch.randn(rows, 896, generator=g, device="cuda").bfloat16()
        w = (1 + 0.1 * torch.randn(896, generator=g, device="cuda")).bfloat16()
        row("rms_norm", {"rows": rows, "hidden": 896},
            lambda: kernels.b200_rms_norm(x, w, epsilon=1e-6, round_before_weight=True),
            {"reference_triton": lambda: reference.triton_rms_norm(x, w, epsilon=1e-6,
                                                                   round_before_weight=True)},
            unit_bytes=rows * 896 * 4)


def cpu_baseline_case(args):
    """The CPU oracle (the restatement of the reference's CPU executor) timed on this machine's
    host cores: per operator on the benchmark configurations' shapes, and the whole Qwen2-0.5B
    architecture (24 layers, vocabulary 151936) through a 512-token prefill and decode steps at
    batch 1 and 16. No GPU work: the numbers stand beside the GPU tables."""

    import os
    import statistics
    import time

    from llm_compiler_b200 import qwen2 as q2
    from oracle import qwen2_model, serve_ops

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)

    def timed(fn, repeats=3):
        fn()
        samples = []
        for _ in range(repeats):
            start = time.perf_counter()
            fn()
            samples.append(time.perf_counter() - start)
        return statistics.median(samples)

    def emit(op, case, seconds, **extra):
        print(json.dumps({"op": op, **case, "cpu_ms": seconds * 1e3, "threads": threads, **extra}), flush=True)

    g = torch.Generator().manual_seed(0)
    hq, hkv, d = 14, 2, 64
    with torch.no_grad():
        for batch, length in ((8, 1024), (8, 4096), (64, 4096)):
            q = torch.randn(batch, hq, 1, d, generator=g).bfloat16()
            k = torch.randn(batch, length, hkv, d, generator=g).bfloat16()
            v = torch.randn(batch, length, hkv, d, generator=g).bfloat16()
            lengths = torch.full((batch,), length)
            mask = torch.zeros(batch, 1, 1, length)
            emit("decode_attention", {"batch": batch, "length": length},
                 timed(lambda: serve_ops.decode_attention(q, k, v, lengths, mask, groups=hq // hkv, scale=d ** -0.5)))
        for batch, tokens in ((4, 512), (4, 2048), (1, 4096)):
            q = torch.randn(batch, hq, tokens, d, generator=g).bfloat16()
            k = torch.randn(batch, hkv, tokens, d, generator=g).bfloat16()
            v = torch.randn(batch, hkv, tokens, d, generator=g).bfloat16()
            mask = serve_ops.causal_mask(batch, tokens)
            emit("prefill_attention", {"batch": batch, "tokens": tokens},
                 timed(lambda: serve_ops.prefill_attention(q, k, v, mask, groups=hq // hkv, scale=d ** -0.5)))
        for m in (64, 4096):
            for name, (k_dim, n) in {"q|k|v": (896, 1152), "gate": (896, 4864), "down": (4864, 896),
                                     "lm_head": (896, 151936)}.items():
                if name == "lm_head" and m != 64:
                    continue
                x = torch.randn(m, k_dim, generator=g).bfloat16()
                w = (torch.randn(n, k_dim, generator=g) * 0.02).bfloat16()
                emit("linear", {"name": name, "m": m, "k": k_dim, "n": n}, timed(lambda: serve_ops.linear(x, w)))
        x = torch.randn(16384, 896, generator=g).bfloat16()
        w = torch.ones(896).bfloat16()
        emit("rms_norm", {"rows": 16384, "hidden": 896},
             timed(lambda: serve_ops.rms_norm(x, w, 1e-6, round_before_weight=True)))
        q = torch.randn(4, hq, 2048, d, generator=g).bfloat16()
        k = torch.randn(4, hkv, 2048, d, generator=g).bfloat16()
        cos = torch.randn(4, 2048, d, generator=g).bfloat16()
        sin = torch.randn(4, 2048, d, generator=g).bfloat16()
        emit("rope", {"batch": 4, "tokens": 2048}, timed(lambda: serve_ops.rope(q, k, cos, sin)))
        kbuf = torch.zeros(4, 8192, hkv, d).bfloat16()
        vbuf = torch.zeros_like(kbuf)
        positions = torch.zeros(4, dtype=torch.int64)
        emit("kv_store", {"batch": 4, "tokens": 2048},
             timed(lambda: serve_ops.kv_store(kbuf, vbuf, k, k, positions)))

        # the whole model, in full: prefill of 512 tokens, then decode steps
        config = q2.QWEN2_0_5B
        weights = q2.make_weights(config, seed=0, dtype=torch.bfloat16)
        for batch in (1, 16):
            prompt = q2.make_prompt_ids(config, batch, 512, seed=batch)
            start = time.perf_counter()
            logits, state = qwen2_model.prefill(config, weights, prompt, capacity=640)
            prefill_s = time.perf_counter() - start
            ids = logits[:, -1].argmax(-1).view(-1, 1)
            steps = []
            for _ in range(5):
                start = time.perf_counter()
                logits = qwen2_model.decode(config, weights, ids, state)
                ids = logits[:, 0].argmax(-1).view(-1, 1)
                steps.append(time.perf_counter() - start)
            step_s = statistics.median(steps[1:])
            emit("qwen2_0.5b_full_model", {"batch": batch, "prompt_tokens": 512}, prefill_s,
                 prefill_tokens_per_s=batch * 512 / prefill_s, decode_ms_per_step=step_s * 1e3,
                 decode_tokens_per_s=batch / step_s)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("op", choices=["decode_attention", "prefill_attention", "kv_store", "linear",
                                       "rms_norm", "timeline", "prefill_step", "compare",
                                       "linear_splitk", "linear_rms", "cpu_baseline"])
    parser.add_argument("--model", default="qwen2-0.5b", choices=["qwen2-0.5b", "qwen2-7b"],
                        help="prefill_step, timeline: architecture")
    parser.add_argument("--launches", type=int, default=40, help="timeline: launches to print")
    parser.add_argument("--path", default="engine", choices=["engine", "executor"],
                        help="prefill_step: Qwen2Engine.prefill, or the reference's prefill KernelIR "
                             "through lower_to_b200 + B200Executor")
    parser.add_argument("--all-logits", action="store_true",
                        help="prefill_step --path engine: logits for every position, as the reference's graph")
    parser.add_argument("--sweep", action="store_true",
                        help="decode attention over batch {1,8,64,256} x length {64,1024,4096,32768}")
    measurement_arguments(parser)
    args = parser.parse_args()
    if args.op == "cpu_baseline":  # host cores only
        cpu_baseline_case(args)
        return
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
    elif args.op == "compare":
        compare_case(args)
    elif args.op in ("linear_splitk", "linear_rms"):
        print(json.dumps(decode_gemm_case(args, args.op.split("_")[1])))
    elif args.op == "prefill_step":
        print(json.dumps(prefill_step_case(args)))
    else:
        print(json.dumps(rms_norm_case(args)))
    kernels.runtime().check_status()


if __name__ == "__main__":
    main()
