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

The timed region of K steps is repeated (contexts reset between repeats, outside the timing)
until about a second of device time has been measured; `value` and `ms_per_step` are the median
repeat, `ms_per_step_min` / `ms_per_step_max` the spread. Before timing, the logits of one
decode step for two sequences are compared with the CPU oracle on the same KV rows (`parity`).

`--model qwen2-7b` runs the serving configuration instead: Qwen2-7B architecture, a GLOBAL batch
of 512 sequences with contexts uniform in [1024, 8192] (seeded), KV pre-filled with N(0, 1),
sequences dealt to the ranks by context length (serving.balanced_assignment) so that every GPU
streams about the same KV bytes; strong scaling. One GPU cannot hold 512 contiguous KV slots
(242 GB): at N = 1 the batch is served as two sub-batches of 256, one after the other.
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
# 262144 tokens, from one ncu --set full capture of decode_attention_kernel (the kernel's streaming
# loop has not changed since; captured at commit a29196d); scaled to the bench launch by the
# tokens it processes (traffic is proportional to the tokens read)
NCU_TRAFFIC_BYTES, NCU_TRAFFIC_TOKENS, NCU_TRAFFIC_COMMIT = 138_338_944, 262_144, "a29196d"
MIN_TIMED_SECONDS = 1.0


def metric_name(args):
    return METRIC if args.model == "qwen2-0.5b" else METRIC.replace("qwen2_0.5b", "qwen2_7b")


def parse_args():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--batch", type=int, default=0,
                        help="sequences per GPU (default 64 for qwen2-0.5b; for qwen2-7b the global "
                             "batch of 512 is split over the GPUs unless this is given)")
    parser.add_argument("--global-batch", type=int, default=512,
                        help="qwen2-7b serving configuration: sequences over all GPUs")
    parser.add_argument("--context", type=int, default=0, help="default 4096 (qwen2-7b: 8192)")
    parser.add_argument("--layers", type=int, default=0, help="override the layer count (debug)")
    parser.add_argument("--split-tokens", type=int, default=0)
    parser.add_argument("--context-source", default="", choices=["", "prefill", "synthetic"])
    parser.add_argument("--cpu-sample-batch", type=int, default=8)
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--skip-parity", action="store_true")
    parser.add_argument("--model", default="qwen2-0.5b", choices=["qwen2-0.5b", "qwen2-7b"],
                        help="architecture (the headline metric is quoted on qwen2-0.5b)")
    parser.add_argument("--context-min", type=int, default=-1,
                        help="with --context-source synthetic: per-sequence contexts uniform in "
                             "[context-min, context] instead of all at --context")
    parser.add_argument("--kv-layout", default="contiguous", choices=["contiguous", "paged"],
                        help="paged: K / V in block pools behind a block table (PagedKVCacheState)")
    parser.add_argument("--block-size", type=int, default=128, help="tokens per KV block (paged layout)")
    parser.add_argument("--path", default="engine", choices=["engine", "executor"],
                        help="engine: Qwen2Engine; executor: the reference-compiled KernelIR of the "
                             "decode step (tests/golden) through lower_to_b200 + B200Executor")
    parser.add_argument("--min-seconds", type=float, default=MIN_TIMED_SECONDS,
                        help="repeat the K timed steps until this much device time is measured")
    args = parser.parse_args()
    serving = args.model == "qwen2-7b"
    args.serving = serving and args.batch == 0  # the 512-sequence serving configuration
    if args.context == 0:
        args.context = 8192 if serving else CONTEXT
    if args.context_min < 0:
        args.context_min = 1024 if serving else 0
    if not args.context_source:
        args.context_source = "synthetic" if serving else "prefill"
    if args.batch == 0:
        args.batch = BATCH_PER_GPU  # (the serving configuration sizes its batches from --global-batch)
    return args


def workload_config(args, n_gpus):
    if args.serving:
        per = args.global_batch // n_gpus
        sub = 2 if n_gpus == 1 and per > 256 else 1
        return {
            "workload": f"qwen2-7b-architecture serving: global batch {args.global_batch}, contexts "
                        f"uniform in [{args.context_min}, {args.context}] (seed 512), KV pre-filled "
                        "with N(0,1), greedy decode, bf16, CUDA-graph step, sequences dealt to the "
                        "GPUs by context length"
                        + (f"; one GPU cannot hold {args.global_batch} contiguous KV slots: served as "
                           f"{sub} sub-batches of {per // sub} in turn" if sub > 1 else "")
                        + (f"; KV in pools of {args.block_size}-token blocks behind a block table"
                           if args.kv_layout == "paged" else ""),
            "kv_layout": args.kv_layout,
            "global_batch": args.global_batch, "context": args.context, "layers": args.layers or 28,
            "parallelism": f"replicas x{n_gpus} (batch-partitioned, NCCL all-gather of token ids)",
            "l2": "inputs larger than L2 (all weights and every valid KV row are read once per step)",
        }
    return {
        "workload": f"{args.model}-architecture greedy decode, batch {args.batch}/GPU, context "
                    + (f"uniform in [{args.context_min}, {args.context}]" if args.context_min > 0
                       else f"{args.context}")
                    + f", bf16, CUDA-graph step, KV from a {args.context_source} prompt"
                    + (f", KV in pools of {args.block_size}-token blocks behind a block table"
                       if args.kv_layout == "paged" else ""),
        "kv_layout": args.kv_layout,
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


def host_threads():
    """All host cores for the CPU legs. torch.distributed.run exports OMP_NUM_THREADS=1 to its
    ranks; the CPU arm runs on rank 0 alone and may use the whole machine."""

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    return torch.get_num_threads()


def reference_arm(args, config):
    """`--impl reference`: the reference's CPU implementation of the path (the oracle port;
    the reference package itself cannot travel to the GPU box) on the host cores."""

    from llm_compiler_b200 import qwen2 as q2

    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = host_threads()
    weights = q2.make_weights(config, seed=0, dtype=torch.bfloat16, device="cpu",
                              reproducible=False)
    steps = max(1, min(args.steps, 5))
    warmup = max(1, min(args.warmup, 1))
    # the serving configuration's contexts average (min + max) / 2: the sample runs at that length
    context = (args.context + args.context_min) // 2 if args.context_min > 0 else args.context
    sample_batch = min(args.cpu_sample_batch, 4) if args.model == "qwen2-7b" else args.cpu_sample_batch
    value, step_s = cpu_decode_baseline(config, weights, context, sample_batch, steps, warmup)
    total = args.global_batch if args.serving else args.batch * args.gpus
    sample = (f"{sample_batch} of the {total} sequences, all {config.num_layers} "
              f"layers, context {context}, median of {steps} steps after {warmup} warm-up")
    print(json.dumps({
        "impl": "reference", "metric": metric_name(args), "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.serving else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
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


def restore_lengths(engine, saved):
    """Puts back a saved copy of the length arena (the rows the undone steps wrote are rewritten
    by the next ones); on the paged layout the engine's host mirror of the lengths follows."""

    engine.state._length_arena.copy_(saved)
    if engine.paged:
        engine.sync_host_lengths()


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
            if engine.paged:
                kernels.b200_paged_decode_attention(
                    query, engine.state.keys[index], engine.state.values[index],
                    engine.state.block_table, engine.attention_lengths, None, scale=engine.scale,
                    numerical_mode=engine.mode, split_tokens=engine.split_tokens,
                    max_length_hint=engine.max_length_hint)
                continue
            kernels.b200_decode_attention(
                query, engine.state.keys[index], engine.state.values[index],
                engine.attention_lengths, None, scale=engine.scale, numerical_mode=engine.mode,
                split_tokens=engine.split_tokens, max_length_hint=engine.max_length_hint,
                output=outputs)

    # The step launches the fused form of this kernel, which (head_dim 64) serves a CTA's tokens
    # with 16 warps where the plain operator uses 8: time the plain operator in the step's shape.
    forced = os.environ.get("B200_DECODE_ATTENTION_WARPS")
    if forced is None and getattr(engine, "attention_is_fused", False) and config.head_dim == 64:
        os.environ["B200_DECODE_ATTENTION_WARPS"] = "16"
    try:
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            launches()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            launches()
    finally:
        if forced is None:
            os.environ.pop("B200_DECODE_ATTENTION_WARPS", None)
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


def oracle_step_parity(engine, config, weights, rows=(0, 1)):
    """One decode step on the engine (not timed, lengths restored afterwards) against the CPU
    oracle on the same KV rows, ids and weights for a few sequences: max-abs logit difference,
    the largest reference logit, and whether the greedy tokens agree."""

    from oracle import qwen2_model

    rows = [r for r in rows if r < engine.batch]
    index = torch.tensor(rows, device=engine.device)
    lengths = engine.positions[index].cpu()
    used = int(lengths.max()) + 1
    state = qwen2_model.OracleKVState([], [], [], used)
    for layer in range(config.num_layers):
        if engine.paged:  # rows of each sequence gathered through the block table
            rows_k = [engine.state.gather(layer, r, used) for r in rows]
            state.keys.append(torch.stack([k for k, _ in rows_k]).cpu())
            state.values.append(torch.stack([v for _, v in rows_k]).cpu())
        else:
            state.keys.append(engine.state.keys[layer][index, :used].cpu())
            state.values.append(engine.state.values[layer][index, :used].cpu())
        state.lengths.append(lengths.clone())
    ids = engine.input_ids[index].cpu()
    saved = engine.state._length_arena.clone()
    engine.decode_step(feed_back=False)
    actual = engine.logits.view(engine.batch, -1)[index].float().cpu()
    tokens = engine.next_ids[index].cpu()
    restore_lengths(engine, saved)  # the row the step wrote is rewritten by the next one
    torch.cuda.synchronize()
    weights_cpu = {name: tensor.cpu() for name, tensor in weights.items()}
    with torch.no_grad():
        expected = qwen2_model.decode(config, weights_cpu, ids.view(-1, 1), state)[:, 0].float()
    scale = float(expected.abs().max())
    diff = float((actual - expected).abs().max())
    picked = expected.gather(1, tokens.view(-1, 1)).view(-1)
    return {"sequences": len(rows), "max_abs_logit_diff": diff, "logit_scale": scale,
            "tokens_equal": bool(torch.equal(tokens, expected.argmax(-1))),
            "picked_token_margin": float((expected.max(-1).values - picked).max()),
            "within_2e-2": diff <= 2e-2}


class ExecutorStepper:
    """The drop-in path as a decode loop: the reference's own KernelIR of the Qwen2-0.5B decode
    step (exported and compiled by the reference, shipped as tests/golden/...json.gz), finished
    by lower_to_b200 and interpreted by B200Executor over the engine's KV state, with the greedy
    token pick and the position update, all captured in one CUDA graph. Same interface as the
    part of Qwen2Engine the benchmark uses."""

    def __init__(self, engine, weights):
        import gzip

        from llm_compiler_b200 import kernel_ir, kernels
        from llm_compiler_b200.executor import B200Executor, bind_arguments
        from llm_compiler_b200.kv_state import PreallocatedKVCacheState

        self.engine, self.kernels = engine, kernels
        path = REPO / "tests" / "golden" / "kernel_ir_qwen2_0_5b_decode_fast.json.gz"
        self.module = kernel_ir.module_from_json(json.loads(gzip.open(path).read()))
        self.report = kernel_ir.lower_to_b200(self.module, zero_mask_arguments=("attention_mask",))
        kernel_ir.require_full_lowering(self.module)
        self.executor = B200Executor(strict=True)
        batch, device = engine.batch, engine.device
        layers = engine.config.num_layers
        # the engine's arena, seen as the state object the graph takes (slot lengths only)
        self.state = PreallocatedKVCacheState(engine.state.keys, engine.state.values,
                                              engine.state.lengths, engine.state.capacity)
        object.__setattr__(self.state, "_length_arena", engine.state._length_arena[:layers])
        self.ids = torch.zeros(batch, 1, dtype=torch.int64, device=device)
        self.positions = torch.zeros(batch, 1, dtype=torch.int64, device=device)
        self.mask = torch.zeros(batch, 1, 1, engine.capacity, device=device)
        self.next_ids = torch.zeros(batch, dtype=torch.int64, device=device)
        self.arguments = bind_arguments(self.module.functions[0], weights, {
            "input_ids": self.ids, "attention_mask": self.mask, "position_ids": self.positions,
            "kv_state": self.state, "inv_freq": engine.inv_freq})
        self.graph = None
        self.kernels_per_step = 0

    def _step(self):
        before = self.kernels.launch_count(self.engine.device)
        with self.kernels.launch_mode(programmatic=True, constant_weights=True, stable_kv_prefix=True):
            logits, _ = self.executor.run(self.module, self.arguments).outputs
        self.logits = logits
        self.kernels.b200_argmax(logits.view(self.engine.batch, -1), self.next_ids)
        self.ids.view(-1).copy_(self.next_ids)
        self.kernels.b200_advance_lengths(self.positions.view(-1), 1, self.engine.capacity)
        self.kernels_per_step = self.kernels.launch_count(self.engine.device) - before

    def sync_from_engine(self):
        self.ids.view(-1).copy_(self.engine.input_ids)
        self.positions.view(-1).copy_(self.engine.positions)

    def capture(self):
        saved = self.engine.state._length_arena.clone()
        self.sync_from_engine()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            self._step()  # sizes workspaces, prepares the packed / folded weights
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        restore_lengths(self.engine, saved)
        self.sync_from_engine()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self._step()
        self.graph = graph
        restore_lengths(self.engine, saved)
        self.sync_from_engine()

    def decode_step(self):
        self.graph.replay()
        return self.next_ids


def serving_contexts(args):
    """The serving configuration's per-sequence context lengths (seeded, the same on every rank)."""

    generator = torch.Generator().manual_seed(512)
    return torch.randint(args.context_min, args.context + 1, (args.global_batch,), generator=generator)


def b200_arm(args, config):
    import torch.distributed as dist

    from llm_compiler_b200 import kernels
    from llm_compiler_b200 import qwen2 as q2
    from llm_compiler_b200.engine import Qwen2Engine
    from llm_compiler_b200.serving import ReplicaServer, balanced_assignment

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
    weights = q2.make_weights(config, seed=rank, dtype=torch.bfloat16, device=device,
                              reproducible=False)
    # ---- which sequences this rank serves, and in how many sub-batches ----
    imbalance = None
    if args.serving:
        contexts_all = serving_contexts(args)
        buckets = balanced_assignment(contexts_all.tolist(), world)
        mine = torch.tensor(buckets[rank])
        kv_sums = [int(contexts_all[torch.tensor(bucket)].sum()) for bucket in buckets]
        imbalance = {"kv_tokens_per_rank": kv_sums,
                     "max_over_mean": max(kv_sums) / (sum(kv_sums) / len(kv_sums))}
        per_rank = len(buckets[rank])
        sub_batches = 2 if per_rank > 256 else 1
        # sub-batches are dealt the same way, so that each holds the same mix of lengths
        parts = balanced_assignment(contexts_all[mine].tolist(), sub_batches)
        batches = [contexts_all[mine[torch.tensor(part)]] for part in parts]
    else:
        contexts = torch.full((args.batch,), args.context)
        if args.context_min > 0:
            contexts = torch.randint(args.context_min, args.context + 1, (args.batch,),
                                     generator=torch.Generator().manual_seed(rank))
        batches = [contexts]
    batch = len(batches[0])
    if any(len(part) != batch for part in batches):
        raise SystemExit("the global batch must divide evenly over ranks and sub-batches")
    capacity = args.context + 2 * (steps + warmup) + 64
    engine = Qwen2Engine(config, weights, batch=batch, capacity=capacity, kv_layout=args.kv_layout,
                         block_size=args.block_size)
    capacity = engine.capacity  # (whole blocks on the paged layout)
    engine.split_tokens = args.split_tokens
    engine.max_length_hint = capacity

    def fill_context(contexts, seed):
        generator = torch.Generator(device=device).manual_seed(seed)
        for layer in range(config.num_layers):
            engine.state.keys[layer].normal_(generator=generator)
            engine.state.values[layer].normal_(generator=generator)
        engine.load_context(contexts, next_ids=torch.randint(0, config.vocab_size, (batch,)))

    if args.context_source == "prefill":
        prompt = q2.make_prompt_ids(config, batch, args.context, seed=100 + rank)
        chunk = 8  # sequences per prefill call: bounds the activation footprint
        if batch % chunk == 0 and batch > chunk:
            helper = Qwen2Engine(config, weights, batch=chunk, capacity=args.context)
            first = []
            if engine.paged:  # the prompts' rows, then one store per layer through the block table
                shape = (batch, args.context, config.num_kv_heads, config.head_dim)
                rows_k = [torch.empty(shape, dtype=engine.dtype, device=device) for _ in range(config.num_layers)]
                rows_v = [torch.empty(shape, dtype=engine.dtype, device=device) for _ in range(config.num_layers)]
            for begin in range(0, batch, chunk):
                helper.prefill(prompt[begin:begin + chunk])
                for layer in range(config.num_layers):
                    if engine.paged:
                        rows_k[layer][begin:begin + chunk].copy_(helper.state.keys[layer])
                        rows_v[layer][begin:begin + chunk].copy_(helper.state.values[layer])
                        continue
                    engine.state.keys[layer][begin:begin + chunk, :args.context].copy_(
                        helper.state.keys[layer])
                    engine.state.values[layer][begin:begin + chunk, :args.context].copy_(
                        helper.state.values[layer])
                first.append(helper.next_ids.clone())
            del helper
            engine.load_context(torch.full((batch,), args.context), next_ids=torch.cat(first))
            if engine.paged:
                zeros = torch.zeros(batch, dtype=torch.int64, device=device)
                for layer in range(config.num_layers):
                    engine.state.store(layer, rows_k[layer].transpose(1, 2), rows_v[layer].transpose(1, 2), zeros)
                del rows_k, rows_v
        else:
            engine.prefill(prompt)
    else:
        fill_context(batches[0], rank)
    torch.cuda.synchronize()
    # the split plan of decode attention comes from the measured profile that ships with the
    # package (profile-guided dispatch), resolved with this engine's batch and context bound
    from llm_compiler_b200.dispatch_plan import DispatchCostModel
    if args.split_tokens == 0:
        decision = engine.use_dispatch_profile(DispatchCostModel.packaged(), capacity)
    else:
        decision = None
    engine.capture()
    parity = None
    if rank == 0 and not args.skip_parity:
        parity = oracle_step_parity(engine, config, weights)
    stepper = None
    if args.path == "executor":
        if args.model != "qwen2-0.5b" or args.layers:
            raise SystemExit("--path executor runs the shipped Qwen2-0.5B decode graph")
        if engine.paged:
            raise SystemExit("--path executor measures the contiguous layout")
        stepper = ExecutorStepper(engine, weights)
        stepper.capture()
        # the same step through both paths from the same state: they launch the same kernels
        saved = engine.state._length_arena.clone()
        engine.decode_step(feed_back=False)
        engine_logits, engine_tokens = engine.logits.float().clone(), engine.next_ids.clone()
        restore_lengths(engine, saved)
        stepper.sync_from_engine()
        stepper.decode_step()
        difference = float((stepper.logits.view(batch, -1).float() - engine_logits.view(batch, -1)).abs().max())
        if parity is not None:
            parity["executor_vs_engine_max_abs_logit_diff"] = difference
            parity["executor_vs_engine_tokens_equal"] = bool(torch.equal(stepper.next_ids, engine_tokens))
        restore_lengths(engine, saved)
        stepper.sync_from_engine()
    step_tokens_read = sum(int(part.sum()) + len(part) for part in batches)  # KV rows read per global step
    global_batch = batch * len(batches) * world
    server = ReplicaServer(engine, batch * world, failure_timeout_s=60.0) if world > 1 else None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    barrier()  # rank 0 has just spent seconds in the CPU oracle: start the steps together

    def run_steps(count):
        pending = None
        for _ in range(count):
            if stepper is not None:
                tokens = stepper.decode_step()
            else:
                tokens = engine.decode_step() if server is None else server.local_step()
            if server is not None:
                if pending is not None:
                    pending.wait()
                pending = server.gather_async(tokens)
        if pending is not None:
            pending.wait()

    def timed(count):
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run_steps(count)
        stop.record()
        barrier()
        elapsed = torch.tensor([start.elapsed_time(stop) * 1e-3], device=device)
        if world > 1:
            dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
        return float(elapsed.item())

    saved_lengths = [None] * len(batches)

    def repeat_seconds():
        """K steps on every sub-batch in turn, each from its starting context (restored outside
        the timed regions); returns the device seconds of the K global steps."""
        total = 0.0
        for index, part in enumerate(batches):
            if len(batches) > 1:
                fill_context(part, rank * 16 + index)
            elif saved_lengths[0] is not None:
                restore_lengths(engine, saved_lengths[0])
                if stepper is not None:
                    stepper.sync_from_engine()
            if saved_lengths[index] is None:
                saved_lengths[index] = engine.state._length_arena.clone()
            run_steps(3 if len(batches) > 1 else 0)  # (a refilled sub-batch warms up again)
            total += timed(steps)
        return total

    with ClockSampler(local_rank) as clocks:
        run_steps(warmup)
        saved_lengths[0] = None
        launches_before = kernels.launch_count(device)
        repeats = [repeat_seconds()]
        wanted = args.min_seconds
        while sum(repeats) < wanted and len(repeats) < 200:
            repeats.append(repeat_seconds())
        # (every rank sees the same max-over-ranks times, so all run the same number of repeats)
        device_s = statistics.median(repeats)

        # end to end through the public host API: H2D ids, step, all-gather of the tokens where
        # there are several ranks, D2H tokens, every step
        restore_lengths(engine, saved_lengths[-1])
        host_ids = engine.next_ids.cpu()
        if stepper is not None:
            stepper.sync_from_engine()
            pinned_in = torch.zeros(batch, dtype=torch.int64).pin_memory()
            pinned_out = torch.zeros(batch, dtype=torch.int64).pin_memory()

        def host_step(ids):
            if stepper is not None:  # host ids in, graph replay, host tokens out
                pinned_in.copy_(ids)
                stepper.ids.view(-1).copy_(pinned_in, non_blocking=True)
                stepper.decode_step()
                pinned_out.copy_(stepper.next_ids, non_blocking=True)
                torch.cuda.current_stream().synchronize()
                return pinned_out
            tokens = engine.step(ids)
            if server is not None:
                server.gather_host(engine.next_ids)
            return tokens

        for _ in range(3):
            host_ids = host_step(host_ids).clone()
        barrier()
        wall = time.perf_counter()
        for _ in range(steps):
            host_ids = host_step(host_ids)
        torch.cuda.synchronize()
        e2e_local = (time.perf_counter() - wall) * len(batches)  # (one sub-batch timed; all are alike)
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
            headline = batch == BATCH_PER_GPU and args.model == "qwen2-0.5b"
            roofline = {"bound": "hbm", "kernel": "decode_attention_kernel", "achieved": achieved,
                        "peak": peak, "peak_source": f"{peak_kind} copy bandwidth", "unit": "GB/s",
                        "frac": achieved / peak, "frac_of_nominal_8000": achieved / 8000.0,
                        "traffic": NCU_TRAFFIC_BYTES * lengths_sum / NCU_TRAFFIC_TOKENS if headline else None,
                        "traffic_capture_commit": NCU_TRAFFIC_COMMIT if headline else None,
                        "algorithmic_bytes_per_launch": bytes_per_launch,
                        "us_per_launch": launch_s * 1e6}
    engine.state.check()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    total_tokens = global_batch * steps
    kv_bytes_per_token = config.num_layers * 4 * config.num_kv_heads * config.head_dim
    # per GPU and global step: the weights once per sub-batch, every valid KV row once
    step_bytes = 2 * q2.parameter_count(config) * len(batches) + kv_bytes_per_token * step_tokens_read
    if not config.tie_word_embeddings:  # an untied embedding table is only gathered, not streamed
        step_bytes -= 2 * config.vocab_size * config.hidden_size * len(batches)
    result = {
        "metric": metric_name(args), "value": total_tokens / device_s, "unit": UNIT, "n_gpus": n_gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": device_s / steps * 1e3,
        "ms_per_step_min": min(repeats) / steps * 1e3, "ms_per_step_max": max(repeats) / steps * 1e3,
        "repeats": len(repeats),
        "higher_is_better": True, "scaling": "strong" if args.serving else "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(args, n_gpus),
        "e2e": {"value": total_tokens / e2e_s, "unit": UNIT,
                "h2d_bytes_per_step": batch * 8 * len(batches), "d2h_bytes_per_step": batch * 8 * len(batches),
                "ms_per_step": e2e_s / steps * 1e3},
        "path": args.path,
        "gpu_launches": (stepper or engine).kernels_per_step * steps * len(batches),
        "kernels_per_step": (stepper or engine).kernels_per_step * len(batches),
        "dispatch": None if decision is None else {
            "op": "decode_attention", "variant": decision.variant, "source": decision.source,
            "profile_value": decision.profile_value},
        "clocks": clocks.summary(),
        "roofline": roofline,
        "parity": parity,
        "step_bandwidth": {"algorithmic_gb_per_step": step_bytes / 1e9,
                           "achieved_gbs_per_gpu": step_bytes / (device_s / steps) / 1e9,
                           "frac_of_measured_hbm": step_bytes / (device_s / steps) / 1e9 /
                           measured_hbm_peak()[0]},
    }
    if imbalance is not None:
        result["balance"] = imbalance
    if world == 1 and not args.skip_cpu_baseline:
        cores = host_threads()
        weights_cpu = {name: tensor.cpu() for name, tensor in weights.items()}
        context = (args.context + args.context_min) // 2 if args.context_min > 0 else args.context
        sample_batch = min(args.cpu_sample_batch, 4) if args.model == "qwen2-7b" else args.cpu_sample_batch
        value, step_s = cpu_decode_baseline(config, weights_cpu, context, sample_batch, 3, 1)
        result["cpu_baseline"] = {
            "value": value, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{sample_batch} of the {global_batch} sequences, all "
                      f"{config.num_layers} layers, context {context}, median of 3 steps "
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
