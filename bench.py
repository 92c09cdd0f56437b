"""Headline benchmark: Qwen2-0.5B-architecture bf16 greedy decode, tokens/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (the shape the decode target is quoted on): 24-layer Qwen2-0.5B architecture, bf16,
random N(0, 0.02) weights with tied embedding / LM head; per GPU a batch of 64 sequences whose
4096-token prompts (uniform synthetic ids) are prefilled by this backend into the preallocated
KV buffers; then K greedy decode steps replay one CUDA graph over fixed KV / length / token
addresses. One step reads 0.99 GB of weights + 3.2 GB of KV: inputs are far larger than the
126 MB L2, so no flush is needed between steps. N > 1: one process per GPU, each a full
replica with its own 64 sequences (weak scaling); the only exchange is the NCCL all-gather of
the sampled token ids, issued every step inside the timed region.

Printed JSON (rank 0, one line):
  value      tokens/s over all GPUs, device-timed with CUDA events, inputs resident in HBM
  e2e        the same metric through Qwen2Engine.step(): host ids in (pinned, H2D), one step,
             host tokens out (D2H) every step, wall-clock between synchronisations
  roofline   decode-attention kernel alone over the same 24 KV buffers: algorithmic bytes
             (512 * sum(len) + 3592 * B per launch) / CUDA-event time, against the measured
             HBM copy peak of MEASURED_PEAKS.json
  cpu_baseline  the CPU oracle (a port of the reference's ReferenceExecutor arithmetic) on the
             host cores, on a bounded sample of the same workload
`--impl reference` times only that CPU path and prints it as its own line.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

REPO = Path(__file__).resolve().parent
sys.path.insert(0, str(REPO))

BATCH_PER_GPU = 64
CONTEXT = 4096
METRIC = "qwen2_0.5b_bf16_decode_tokens_per_s"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
RESULT_STREAM = sys.stdout  # main() replaces it with a private copy of the process's stdout
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-attention launch over 64 x 4096 =
# 262144 tokens, from the ncu capture summarised in profiles/decode_attention_b64_l4096_ncu_full.md;
# scaled to the bench launch by the tokens it processes (traffic is proportional to the tokens read)
NCU_TRAFFIC_BYTES, NCU_TRAFFIC_TOKENS = 138_843_776, 262_144


def metric_name(args):
    return METRIC if args.model == "qwen2-0.5b" else METRIC.replace("qwen2_0.5b", "qwen2_7b")


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--batch", type=int, default=BATCH_PER_GPU)
    parser.add_argument("--context", type=int, default=CONTEXT)
    parser.add_argument("--layers", type=int, default=0, help="override the layer count (debug)")
    parser.add_argument("--split-tokens", type=int, default=0)
    parser.add_argument("--context-source", default="prefill", choices=["prefill", "synthetic"])
    parser.add_argument("--cpu-sample-batch", type=int, default=8)
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--model", default="qwen2-0.5b", choices=["qwen2-0.5b", "qwen2-7b"],
                        help="architecture (the headline metric is quoted on qwen2-0.5b)")
    parser.add_argument("--context-min", type=int, default=0,
                        help="with --context-source synthetic: per-sequence contexts uniform in "
                             "[context-min, context] instead of all at --context")
    return parser.parse_args()


def workload_config(args, n_gpus):
    return {
        "workload": f"{args.model}-architecture greedy decode, batch {args.batch}/GPU, context "
                    + (f"uniform in [{args.context_min}, {args.context}]" if args.context_min > 0
                       else f"{args.context}")
                    + f", bf16, CUDA-graph step, KV from a {args.context_source} prompt",
        "global_batch": args.batch * n_gpus,
        "context": args.context,
        "layers": args.layers or (24 if args.model == "qwen2-0.5b" else 28),
        "parallelism": f"replicas x{n_gpus} (batch-partitioned, NCCL all-gather of token ids)",
        "l2": "inputs larger than L2 (0.99 GB weights + 3.2 GB KV read per step)"
              if args.model == "qwen2-0.5b" and args.context == CONTEXT and args.batch == BATCH_PER_GPU
              else "inputs larger than L2 (all weights and every valid KV row are read once per step)",
    }


# ------------------------------------------------------------------ clock sampling ----
class ClockSampler:
    """Samples SM clock and clock-event reasons of this process's GPU with NVML while the
    benchmark runs (read-only queries)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, device_index: int) -> None:
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{uuid}".encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.nvml = pynvml
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception as error:  # no NVML: the clocks key says so
            self.nvml, self.error = None, repr(error)

    def _loop(self):
        nvml = self.nvml
        while not self._stop.is_set():
            try:
                self.samples.append(nvml.nvmlDeviceGetClockInfo(self.handle, nvml.NVML_CLOCK_SM))
                mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nvml is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self):
        if self.nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "error": self.error}
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------- CPU baseline ----
def cpu_decode_baseline(config, weights_cpu, context, sample_batch, steps, warmup):
    """Times the CPU oracle's decode step (same arithmetic as the reference's CPU executor)
    on `sample_batch` sequences at the full context, all layers, all host threads."""

    from oracle import qwen2_model

    generator = torch.Generator().manual_seed(1)
    dtype = weights_cpu["embed_tokens.weight"].dtype
    capacity = context + steps + warmup + 1
    state = qwen2_model.OracleKVState([], [], [], capacity)
    for _ in range(config.num_layers):
        shape = (sample_batch, capacity, config.num_kv_heads, config.head_dim)
        state.keys.append(torch.randn(shape, generator=generator).to(dtype))
        state.values.append(torch.randn(shape, generator=generator).to(dtype))
        state.lengths.append(torch.full((sample_batch,), context, dtype=torch.int64))
    ids = torch.randint(0, config.vocab_size, (sample_batch, 1), generator=generator)
    times = []
    with torch.no_grad():
        for index in range(warmup + steps):
            start = time.perf_counter()
            logits = qwen2_model.decode(config, weights_cpu, ids, state)
            ids = logits[:, 0].argmax(-1).view(-1, 1)
            if index >= warmup:
                times.append(time.perf_counter() - start)
    step_s = statistics.median(times)
    return sample_batch / step_s, step_s


def reference_arm(args, config):
    """`--impl reference`: the reference's CPU implementation of the path (the oracle port;
    the reference package itself cannot travel to the GPU box) on the host cores."""

    from llm_compiler_b200 import qwen2 as q2

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    weights = q2.make_weights(config, seed=0, dtype=torch.bfloat16, device="cpu",
                              reproducible=False)
    steps = max(1, min(args.steps, 5))
    warmup = max(1, min(args.warmup, 1))
    value, step_s = cpu_decode_baseline(config, weights, args.context, args.cpu_sample_batch,
                                        steps, warmup)
    sample = (f"{args.cpu_sample_batch} of the {args.batch} sequences, all {config.num_layers} "
              f"layers, context {args.context}, median of {steps} steps after {warmup} warm-up")
    print(json.dumps({
        "impl": "reference", "metric": metric_name(args), "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }), file=RESULT_STREAM, flush=True)


# ------------------------------------------------------------------------ B200 arm ----
def measured_hbm_peak():
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def attention_roofline(engine, lengths_sum, rounds):
    """Decode-attention kernel alone, one launch per layer over the engine's own KV buffers
    (24 x 134 MB, far beyond L2), captured in a graph so that host launch gaps do not count."""

    from llm_compiler_b200 import kernels

    config = engine.config
    batch = engine.batch
    query = torch.randn(batch, config.num_heads, 1, config.head_dim, device=engine.device,
                        dtype=torch.bfloat16)
    outputs = torch.empty_like(query)

    def launches():
        for index in range(config.num_layers):
            kernels.b200_decode_attention(
                query, engine.state.keys[index], engine.state.values[index],
                engine.attention_lengths, None, scale=engine.scale, numerical_mode=engine.mode,
                split_tokens=engine.split_tokens, max_length_hint=engine.max_length_hint,
                output=outputs)

    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        launches()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launches()
    for _ in range(3):
        graph.replay()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(rounds):
        graph.replay()
    stop.record()
    torch.cuda.synchronize()
    per_launch_s = start.elapsed_time(stop) * 1e-3 / (rounds * config.num_layers)
    # K and V of every valid token once, q in and o out once, the lengths
    bytes_per_launch = 4 * config.num_kv_heads * config.head_dim * lengths_sum + \
        (4 * config.num_heads * config.head_dim + 8) * batch
    return bytes_per_launch, per_launch_s


def b200_arm(args, config):
    import torch.distributed as dist

    from llm_compiler_b200 import kernels
    from llm_compiler_b200 import qwen2 as q2
    from llm_compiler_b200.engine import Qwen2Engine
    from llm_compiler_b200.serving import TokenGather

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the B200 backend has no CPU path")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    n_gpus = world

    steps, warmup = args.steps, max(args.warmup, 3)
    capacity = args.context + 2 * (steps + warmup) + 64
    weights = q2.make_weights(config, seed=rank, dtype=torch.bfloat16, device=device,
                              reproducible=False)
    engine = Qwen2Engine(config, weights, batch=args.batch, capacity=capacity)
    engine.split_tokens = args.split_tokens
    engine.max_length_hint = capacity

    if args.context_source == "prefill":
        prompt = q2.make_prompt_ids(config, args.batch, args.context, seed=100 + rank)
        chunk = 8  # sequences per prefill call: bounds the activation footprint
        if args.batch % chunk == 0 and args.batch > chunk:
            helper = Qwen2Engine(config, weights, batch=chunk, capacity=args.context)
            first = []
            for begin in range(0, args.batch, chunk):
                helper.prefill(prompt[begin:begin + chunk])
                for layer in range(config.num_layers):
                    engine.state.keys[layer][begin:begin + chunk, :args.context].copy_(
                        helper.state.keys[layer])
                    engine.state.values[layer][begin:begin + chunk, :args.context].copy_(
                        helper.state.values[layer])
                first.append(helper.next_ids.clone())
            del helper
            engine.load_context(torch.full((args.batch,), args.context), next_ids=torch.cat(first))
        else:
            engine.prefill(prompt)
    else:
        generator = torch.Generator(device=device).manual_seed(rank)
        for layer in range(config.num_layers):
            engine.state.keys[layer].normal_(generator=generator)
            engine.state.values[layer].normal_(generator=generator)
        contexts = torch.full((args.batch,), args.context)
        if args.context_min > 0:
            contexts = torch.randint(args.context_min, args.context + 1, (args.batch,),
                                     generator=torch.Generator().manual_seed(rank))
        engine.load_context(contexts, next_ids=torch.randint(0, config.vocab_size, (args.batch,)))
    torch.cuda.synchronize()
    # the split plan of decode attention comes from the measured profile that ships with the
    # package (profile-guided dispatch), resolved with this engine's batch and context bound
    from llm_compiler_b200.dispatch_plan import DispatchCostModel
    if args.split_tokens == 0:
        decision = engine.use_dispatch_profile(DispatchCostModel.packaged(), capacity)
    else:
        decision = None
    engine.capture()
    step_tokens_read = int(engine.attention_lengths.sum().item())  # KV rows one step reads, at the start
    gather = TokenGather(args.batch * world, device=device) if world > 1 else None

    def run_steps(count):
        pending = None
        for _ in range(count):
            tokens = engine.decode_step()
            if gather is not None:
                if pending is not None:
                    pending.wait()
                gather.send.copy_(tokens)
                pending = dist.all_gather_into_tensor(gather.padded, gather.send, async_op=True)
        if pending is not None:
            pending.wait()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    with ClockSampler(local_rank) as clocks:
        run_steps(warmup)
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches_before = kernels.launch_count(device)
        start.record()
        run_steps(steps)
        stop.record()
        barrier()
        elapsed = torch.tensor([start.elapsed_time(stop) * 1e-3], device=device)
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        device_s = float(elapsed.item())

        # end to end through the public host API: H2D ids, step, D2H tokens, every step
        host_ids = engine.next_ids.cpu()
        for _ in range(3):
            host_ids = engine.step(host_ids).clone()
        barrier()
        wall = time.perf_counter()
        for _ in range(steps):
            host_ids = engine.step(host_ids)
        torch.cuda.synchronize()
        e2e_local = time.perf_counter() - wall
        e2e_t = torch.tensor([e2e_local], device=device)
        if world > 1:
            dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
        e2e_s = float(e2e_t.item())

        roofline = None
        if rank == 0:
            lengths_sum = int(engine.attention_lengths.sum().item())
            bytes_per_launch, launch_s = attention_roofline(engine, lengths_sum, rounds=10)
            peak, peak_kind = measured_hbm_peak()
            achieved = bytes_per_launch / launch_s / 1e9
            roofline = {"bound": "hbm", "kernel": "decode_attention_kernel", "achieved": achieved,
                        "peak": peak, "peak_source": f"{peak_kind} copy bandwidth", "unit": "GB/s",
                        "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0,
                        "traffic": NCU_TRAFFIC_BYTES * lengths_sum / NCU_TRAFFIC_TOKENS
                        if args.batch == BATCH_PER_GPU and args.model == "qwen2-0.5b" else None,
                        "algorithmic_bytes_per_launch": bytes_per_launch,
                        "us_per_launch": launch_s * 1e6}
    engine.state.check()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    total_tokens = args.batch * world * steps
    kv_bytes_per_token = config.num_layers * 4 * config.num_kv_heads * config.head_dim
    step_bytes = 2 * q2.parameter_count(config) + kv_bytes_per_token * step_tokens_read
    result = {
        "metric": metric_name(args), "value": total_tokens / device_s, "unit": UNIT, "n_gpus": n_gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": device_s / steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, n_gpus),
        "e2e": {"value": total_tokens / e2e_s, "unit": UNIT,
                "h2d_bytes_per_step": args.batch * 8, "d2h_bytes_per_step": args.batch * 8,
                "ms_per_step": e2e_s / steps * 1e3},
        "gpu_launches": engine.kernels_per_step * steps,
        "kernels_per_step": engine.kernels_per_step,
        "dispatch": None if decision is None else {
            "op": "decode_attention", "variant": decision.variant, "source": decision.source,
            "profile_value": decision.profile_value},
        "clocks": clocks.summary(),
        "roofline": roofline,
        "step_bandwidth": {"algorithmic_gb_per_step": step_bytes / 1e9,
                           "achieved_gbs_per_gpu": step_bytes / (device_s / steps) / 1e9,
                           "frac_of_measured_hbm": step_bytes / (device_s / steps) / 1e9 /
                           measured_hbm_peak()[0]},
    }
    if world == 1 and not args.skip_cpu_baseline:
        weights_cpu = {name: tensor.cpu() for name, tensor in weights.items()}
        value, step_s = cpu_decode_baseline(config, weights_cpu, args.context,
                                            args.cpu_sample_batch, 3, 1)
        result["cpu_baseline"] = {
            "value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{args.cpu_sample_batch} of the {args.batch} sequences, all "
                      f"{config.num_layers} layers, context {args.context}, median of 3 steps "
                      f"after 1 warm-up ({step_s:.2f} s/step)"}
    print(json.dumps(result), file=RESULT_STREAM, flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    # The JSON line must be the only thing on stdout, but libraries write there too (NCCL prints
    # its version banner): keep the real stdout for the result and point fd 1 at stderr.
    global RESULT_STREAM
    sys.stdout.flush()
    RESULT_STREAM = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    from llm_compiler_b200 import qwen2 as q2

    config = q2.QWEN2_0_5B if args.model == "qwen2-0.5b" else q2.QWEN2_7B
    if args.layers:
        config = q2.Qwen2Config(**{**config.__dict__, "num_layers": args.layers})
    if args.impl == "reference":
        reference_arm(args, config)
    else:
        b200_arm(args, config)


if __name__ == "__main__":
    main()
