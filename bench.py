"""Benchmark of the sparse-decode attention path at 128K context.

Workload (the reference's long-context batched decode configuration): a
Qwen3-8B-shaped decoder - 36 layers, 32 query / 8 KV heads, head_dim 128 - at
131072 tokens of context per sequence, 1024-4096 communities per (layer, KV
head) with Zipf(1.1) sizes, 2048-token retrieval budget, bf16 K/V.  One "step"
is one decode step of the attention path: for every layer, every sequence and
every KV head, centroid scoring -> budgeted community selection -> gather +
segmented attention -> merge -> online assignment.  Layers run one after the
other (a real decoder's layers depend on each other); all sequences and heads of
a layer share one library call.  KV heads are sharded across the GPUs, each GPU
keeps 8/N heads of ``--batch-per-gpu * N`` sequences (weak scaling), and every
layer's head outputs are all-gathered.

Prints one JSON line (rank 0).  ``--impl reference`` times the CPU restatement of
the reference's algorithm on the host cores instead.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from concurrent.futures import ProcessPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

LAYERS = 36
QUERY_HEADS = 32
KV_HEADS = 8
HEAD_DIM = 128
CONTEXT = 131072
# ncu DRAM bytes of one layer launch, written by the profiling step next to its summary
TRAFFIC_FILE = ROOT / "profiles" / "decode_cluster_kernel.traffic.json"
CPU_DECODE_CAPACITY = 4096  # decode slots of a CPU worker's unit (far more than the time bound allows)
BLAS_THREAD_VARIABLES = ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS", "NUMEXPR_NUM_THREADS")
BUDGET = 2048
NUM_SINK = 10
COMMUNITIES = (1024, 4096)
ZIPF = 1.1
SCALE = HEAD_DIM**-0.5
METRIC = "sparse decode tokens/sec at 128K ctx (attention path, all 36 layers)"


def parse_args() -> argparse.Namespace:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["b200", "reference"], default="b200")
    parser.add_argument("--batch-per-gpu", type=int, default=0, help="0: largest of 8/4/2/1 that fits")
    parser.add_argument("--layers", type=int, default=LAYERS)
    parser.add_argument("--context", type=int, default=CONTEXT)
    parser.add_argument("--splits", type=int, default=0, help="attention CTAs per head; 0: fill one wave")
    parser.add_argument("--layers-per-launch", type=int, default=1)
    parser.add_argument("--cpu-seconds", type=float, default=15.0)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-prefill", action="store_true", help="skip the prefill kernel's sub-record")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--exchange", choices=["peer", "nccl"], default="peer",
                        help="N>1: head outputs by in-kernel peer stores (default) or an NCCL all-gather per layer")
    parser.add_argument("--peer-wait", choices=["node", "launch"], default="node",
                        help="peer exchange: wait for the peers' rows in a one-thread kernel after each layer "
                             "(node) or inside the layer launch itself (launch)")
    parser.add_argument("--update", choices=["inline", "deferred"], default="deferred",
                        help="online graph update inside the layer launch (inline), or as its own launch on a "
                             "second stream that runs beside the next layer's launch (deferred)")
    parser.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                        help="weak: --batch-per-gpu sequences per GPU (8N in all); strong: 16 sequences in all, "
                             "the stated batch of the long-context configuration, whatever N (needs N >= 2)")
    parser.add_argument("--sweep-context", type=int, default=1_048_576)
    parser.add_argument("--workload", choices=["decode", "prefill", "sweep", "model"], default="decode",
                        help="prefill: the score-graph emission kernel at S=16384 (a second, separate line); "
                             "model: a random-init Qwen3-8B-shaped decoder driven through the Hugging Face plug-in")
    parser.add_argument("--prompt-length", type=int, default=32768)
    parser.add_argument("--new-tokens", type=int, default=128)
    parser.add_argument("--model-layers", type=int, default=36)
    parser.add_argument("--online-assignment", choices=["modularity", "nearest_centroid"], default="modularity",
                        help="--workload model: the reference's modularity-gain rule, or the nearest-centroid "
                             "variant (one more centroid scan per layer and token)")
    parser.add_argument("--prefill-length", type=int, default=16384)
    return parser.parse_args()


# --------------------------------------------------------------------------- #
# CPU arm: the oracle port on the host cores
# --------------------------------------------------------------------------- #
def _cpu_worker(task: tuple[int, int, float]) -> tuple[int, float]:
    """Time oracle layer transitions of one (sequence, layer, KV head) unit."""

    seed, context, seconds = task
    import torch

    torch.set_num_threads(1)
    from community_kv_b200.runtime import convert_prefill_tensors
    from community_kv_b200.synthetic import make_layer, make_query
    from oracle import decode_oracle

    generator = torch.Generator().manual_seed(seed)
    count = int(torch.randint(COMMUNITIES[0], COMMUNITIES[1] + 1, (1,), generator=generator))
    layer = make_layer(
        seed=seed, kv_heads=1, group_size=4, seq_len=context, communities=count,
        num_sink=NUM_SINK, max_decode_tokens=CPU_DECODE_CAPACITY, zipf_exponent=ZIPF,
    )
    converted = convert_prefill_tensors(**layer.prepare_kwargs())
    sinks = torch.arange(NUM_SINK, dtype=torch.int32)
    done = 0
    begin = time.perf_counter()
    while True:
        decode_oracle.decode_layer(
            query=make_query(seed=seed * 131 + done, query_heads=4),
            key=layer.key,
            value=layer.value,
            csr=converted.csr,
            state=converted.mutable,
            sink_positions=sinks,
            current_position=converted.current_position,
            softmax_scale=SCALE,
            lam=0.5,
            token_budget=BUDGET,
            num_sink=NUM_SINK,
            exact=False,
        )
        done += 1
        elapsed = time.perf_counter() - begin
        if elapsed >= seconds or done >= CPU_DECODE_CAPACITY - 8:  # the second bound: decode slots of the sample
            return done, elapsed


def cpu_baseline(seconds: float, context: int, layers: int, seed: int = 0) -> dict:
    """Whole-host throughput of the CPU restatement on a bounded sample of the workload."""

    import multiprocessing

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    context_for_sample = context
    tasks = [(seed * 1000 + worker, context_for_sample, seconds) for worker in range(cores)]
    # One process per core, each strictly single-threaded: the BLAS / OpenMP pools read
    # these variables when the worker imports numpy and torch, so they are set before the
    # workers are spawned (otherwise every worker starts a pool as wide as the machine and
    # the processes fight over the cores).
    saved = {name: os.environ.get(name) for name in BLAS_THREAD_VARIABLES}
    os.environ.update({name: "1" for name in BLAS_THREAD_VARIABLES})
    try:
        with ProcessPoolExecutor(max_workers=cores, mp_context=multiprocessing.get_context("spawn")) as pool:
            results = list(pool.map(_cpu_worker, tasks))
    finally:
        for name, value in saved.items():
            if value is None:
                os.environ.pop(name, None)
            else:
                os.environ[name] = value
    unit_rate = sum(done / elapsed for done, elapsed in results)
    units_per_token = layers * KV_HEADS
    return {
        "value": unit_rate / units_per_token,
        "unit": "tokens/s",
        "cores": cores,
        "threads_per_process": 1,
        "kind": "port",
        "sample": (
            f"{cores} processes x one (sequence, layer, KV head) unit each at ctx {context_for_sample}, "
            f"{sum(d for d, _ in results)} unit-steps in ~{seconds:.0f}s; a token = {units_per_token} units"
        ),
    }


def run_reference(args: argparse.Namespace) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    per_step = []
    total_steps = args.warmup + args.steps
    seconds = max(2.0, min(args.cpu_seconds, 150.0 / max(total_steps, 1)))
    last = None
    for step in range(total_steps):
        last = cpu_baseline(seconds, args.context, args.layers, seed=step)
        if step >= args.warmup:
            per_step.append(last["value"])
    value = statistics.mean(per_step)
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": value,
        "unit": "tokens/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": 1000.0 / value,
        "higher_is_better": True,
        "scaling": args.scaling,
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(
            args, batch=16 if args.scaling == "strong" else (args.batch_per_gpu or 8) * args.gpus, world=args.gpus,
            exchange_mode=default_exchange_mode(args, args.gpus),
        ),
        "cpu_baseline": {**last, "value": value},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def default_exchange_mode(args: argparse.Namespace, world: int) -> str:
    if world == 1:
        return "none"
    if args.exchange == "nccl":
        return "nccl all-gather per layer"
    return "peer stores from the merge phase; wait for the peers' rows: " + args.peer_wait


def workload_config(args: argparse.Namespace, *, batch: int, world: int, exchange_mode: str = "none") -> dict:
    return {
        "workload": (
            "batched long-context decode (Qwen3-8B attention shapes): "
            f"{args.layers} layers x {batch} sequences x {KV_HEADS} KV heads, ctx {args.context}, "
            f"{COMMUNITIES[0]}-{COMMUNITIES[1]} Zipf({ZIPF}) communities per head, budget {BUDGET}"
        ),
        "global_batch": batch,
        "context": args.context,
        "token_budget": BUDGET,
        "parallelism": f"kv-head shard x{world}",
        "exchange": exchange_mode,
        "layers_per_launch": args.layers_per_launch,
        "splits": args.splits,
        "update": args.update,
        "l2": "inputs larger than L2 (each step gathers rows scattered over the whole KV cache)",
    }


def measured_traffic(units_per_launch: int, kernels_per_layer: int) -> tuple[int | None, str | None]:
    """DRAM bytes of one layer launch as the profiler counted them (None without a capture).

    The capture is taken on a smaller launch (fewer units); traffic grows in proportion to
    the units a launch processes, so it is scaled by the unit count.
    """

    if kernels_per_layer != 1 or not TRAFFIC_FILE.exists():
        return None, None
    try:
        record = json.loads(TRAFFIC_FILE.read_text())
        per_unit = float(record["dram_bytes_per_launch"]) / float(record["units_per_launch"])
    except (ValueError, KeyError, ZeroDivisionError):
        return None, None
    source = (
        "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch with "
        f"{record['units_per_launch']} units, scaled to {units_per_launch} units"
    )
    return int(per_unit * units_per_launch), source


# --------------------------------------------------------------------------- #
# clocks
# --------------------------------------------------------------------------- #
class ClockSampler:
    FIELDS = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int) -> None:
        self.index = index
        self.samples: list[list[str]] = []
        self.process: subprocess.Popen | None = None
        self.thread: threading.Thread | None = None

    def start(self) -> None:
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True,
            )
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self) -> None:
        assert self.process is not None and self.process.stdout is not None
        for line in self.process.stdout:
            self.samples.append([part.strip() for part in line.split(",")])

    def stop(self) -> dict:
        if self.process is not None:
            self.process.terminate()
            try:
                self.process.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.process.kill()
        clocks, maxima, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for sample in self.samples:
            if len(sample) < 7:
                continue
            try:
                clocks.append(float(sample[0]))
                maxima.append(float(sample[1]))
            except ValueError:
                continue
            for name, flag in zip(names, sample[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max(maxima) if maxima else None,
            "samples": len(clocks),
            "reasons": sorted(reasons),
        }


# --------------------------------------------------------------------------- #
# GPU arm
# --------------------------------------------------------------------------- #
def pick_batch(requested: int, args: argparse.Namespace, heads_local: int, torch) -> int:
    if requested > 0:
        return requested
    free, _ = torch.cuda.mem_get_info()
    rows = args.context + 512
    per_sequence = args.layers * heads_local * rows * HEAD_DIM * 2 * 2
    per_sequence += args.layers * heads_local * (args.context * 12 + 5000 * 140)
    for candidate in (8, 4, 2, 1):
        if candidate * per_sequence < 0.86 * free:
            return candidate
    return 1


def run_b200(args: argparse.Namespace) -> None:
    import torch
    import torch.distributed as dist

    from community_kv_b200 import native, ops
    from community_kv_b200.workload import build_decode_workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if KV_HEADS % world:
        raise SystemExit("the number of GPUs must divide the 8 KV heads")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    heads_local = KV_HEADS // world
    query_local = heads_local * (QUERY_HEADS // KV_HEADS)
    if args.scaling == "strong":
        if world < 2:
            raise SystemExit("--scaling strong keeps 16 sequences in all: that needs at least two GPUs")
        batch = 16
    else:
        per_gpu = pick_batch(args.batch_per_gpu, args, KV_HEADS, torch)
        batch = per_gpu * world
    total_steps = args.warmup + args.steps
    e2e_steps = max(3, min(args.steps, 10))
    extra_steps = 4 + e2e_steps + 2 + 3 + 4  # e2e steps, three event-timed passes, one phase-stamped pass
    max_decode = total_steps + extra_steps + 8

    build_begin = time.perf_counter()
    work = build_decode_workload(
        layers=args.layers, batch=batch, kv_heads=heads_local, group_size=QUERY_HEADS // KV_HEADS,
        seq_len=args.context, communities=COMMUNITIES, token_budget=BUDGET, num_sink=NUM_SINK,
        max_decode_tokens=max_decode, device=device, seed=args.seed, zipf_exponent=ZIPF,
        head_offset=rank * heads_local, layers_per_launch=args.layers_per_launch, splits=args.splits or None,
    )
    torch.cuda.synchronize()
    build_seconds = time.perf_counter() - build_begin
    launches, slots = work.launches, work.slots

    # One contiguous output arena so that a step's result is a single tensor.
    exchange = None
    exchange_mode = "none"
    if world > 1 and args.exchange == "peer":
        try:
            from community_kv_b200.distributed import PeerOutputExchange

            exchange = PeerOutputExchange(launches=launches, slots=slots, heads=query_local, head_dim=HEAD_DIM,
                                          units=slots * heads_local, device=device)
            ok = torch.ones((1,), device=device)
        except Exception as error:  # symmetric memory unavailable: every rank falls back together
            print(f"[bench] rank {rank}: peer exchange unavailable ({error!r}); using NCCL", file=sys.stderr)
            ok = torch.zeros((1,), device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if float(ok) == 0.0:
            exchange = None
    if world > 1:
        exchange_mode = default_exchange_mode(args, world) if exchange else "nccl all-gather per layer"
    if exchange is not None:
        out_full = exchange.gathered
        out_local = None
    else:
        out_local = torch.zeros((launches, slots, query_local, HEAD_DIM), dtype=torch.bfloat16, device=device)
        out_full = (
            torch.zeros((launches, world, slots, query_local, HEAD_DIM), dtype=torch.bfloat16, device=device)
            if world > 1 else None
        )
    # One staging buffer holds a step's inputs, layer by layer: a layer's queries, then its new
    # K rows, then its new V rows.  The end-to-end loop can so bring the first layers' inputs
    # from the host in one copy and the remaining layers' in a second that runs beside them.
    query_count = slots * query_local * HEAD_DIM
    row_count = slots * heads_local * HEAD_DIM
    staged = torch.zeros((launches, query_count + 2 * row_count), dtype=torch.bfloat16, device=device)
    q_cur = staged[:, :query_count].view(launches, slots, query_local, HEAD_DIM)
    new_key = staged[:, query_count:query_count + row_count].view(launches, slots, heads_local, HEAD_DIM)
    new_value = staged[:, query_count + row_count:].view(launches, slots, heads_local, HEAD_DIM)
    generator = torch.Generator(device=device).manual_seed(args.seed + 17 + rank)
    stream = torch.cuda.Stream(device)
    packed = []
    with torch.cuda.stream(stream):
        for launch in range(launches):
            state = work.state(launch)
            state.workspace.attention.output = (
                exchange.local_output(launch) if exchange is not None else out_local[launch]
            )
            packed.append(
                work.runtime.pack(launch, query=q_cur[launch], key=work.key[launch],
                                  value=work.value[launch], softmax_scale=SCALE)
            )
            if exchange is not None:
                exchange.attach(packed[-1], launch, wait_in_kernel=args.peer_wait == "launch")

    # Deferred update: the layer launch stops after the head outputs, the neighbour
    # candidates and the log-sum-exp are written; the online assignment of that layer runs
    # as a second launch on a side stream (nothing downstream of the attention output
    # depends on it) and is joined before the step ends, i.e. before the layer's next step.
    deferred = args.update == "deferred"
    side = torch.cuda.Stream(device) if deferred else None
    attend_args, update_args = [], []
    for launch in range(launches if deferred else 0):
        attend = native.LayerArgs.from_buffer_copy(packed[launch])
        attend.flags |= native.FLAG_SKIP_UPDATE
        attend_args.append(attend)
        update = native.LayerArgs.from_buffer_copy(packed[launch])
        update.peer_count = 0
        update.peer_wait_flag = None
        update_args.append(update)

    def enqueue_step(first: int = 0, last: int = launches, after_layer=None) -> None:
        handle = stream.cuda_stream
        for launch in range(first, last):
            if deferred:
                native.call("ckv_decode_layer", attend_args[launch], handle)
                attended = torch.cuda.Event()
                attended.record(stream)
                side.wait_event(attended)
                native.call("ckv_online_update", update_args[launch], side.cuda_stream)
            else:
                native.call("ckv_decode_layer", packed[launch], handle)
            if exchange is not None:
                if args.peer_wait == "node":
                    exchange.wait(launch, handle)  # the next consumer needs every rank's heads
            elif world > 1:
                dist.all_gather_into_tensor(out_full[launch], out_local[launch])
            if after_layer is not None:
                after_layer(launch)
        if deferred:
            updated = torch.cuda.Event()
            updated.record(side)
            stream.wait_event(updated)

    def new_queries(count: int) -> "torch.Tensor":
        return torch.randn((count, launches, slots, query_local, HEAD_DIM), generator=generator,
                           device=device, dtype=torch.float32).to(torch.bfloat16)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (direct launches), then capture one step in a CUDA graph ----
    q_all = new_queries(total_steps)
    with torch.cuda.stream(stream):
        for step in range(args.warmup):
            q_cur.copy_(q_all[step])
            enqueue_step()
    barrier()
    if exchange is not None:
        # the rows the peers stored here must be exactly what a collective would deliver
        exchange.check()
        mine = exchange.gathered[:, rank].contiguous()
        reference = torch.empty_like(exchange.gathered).transpose(0, 1).contiguous()
        dist.all_gather_into_tensor(reference, mine)
        if not torch.equal(reference.transpose(0, 1), exchange.gathered):
            raise RuntimeError("peer-stored head outputs differ from an all-gather of the local outputs")
        barrier()
    graph = torch.cuda.CUDAGraph()
    use_graph = True
    try:
        with torch.cuda.graph(graph, stream=stream):
            enqueue_step()
        # the capture itself does not execute; state is untouched
    except Exception as error:  # pragma: no cover - depends on NCCL capture support
        use_graph = False
        if rank == 0:
            print(f"[bench] graph capture unavailable ({type(error).__name__}); direct launches", file=sys.stderr)
    barrier()

    def run_step() -> None:
        if use_graph:
            graph.replay()
        else:
            enqueue_step()

    # ---- timed region: K steps, CUDA events on the launching stream ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    with torch.cuda.stream(stream):
        begin.record()
        for step in range(args.warmup, total_steps):
            q_cur.copy_(q_all[step])
            run_step()
        end.record()
    barrier()
    elapsed_ms = torch.tensor([begin.elapsed_time(end)], device=device)
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed_ms) / args.steps
    work.runtime.assert_no_overflow()

    # ---- dominant kernel: the per-layer launch(es), event-timed one layer at a time ----
    layer_ms = []
    solo = []  # the same launches without the cross-GPU stores: these passes are not synchronised
    for launch in range(launches):
        # the launch the timed step uses: without the online update when that runs as its own launch
        clone = native.LayerArgs.from_buffer_copy(attend_args[launch] if deferred else packed[launch])
        clone.peer_count = 0
        clone.peer_wait_flag = None
        solo.append(clone)
    with torch.cuda.stream(stream):
        for repeat in range(3):
            events = []
            for launch in range(launches):
                first, second = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                first.record()
                native.call("ckv_decode_layer", solo[launch], stream.cuda_stream)
                second.record()
                events.append((first, second))
            stream.synchronize()
            if repeat > 0:
                layer_ms.extend(a.elapsed_time(b) for a, b in events)
    layer_launch_ms = statistics.mean(layer_ms)
    kernels_per_layer = int(native.library().ckv_decode_layer_kernels(ctypes.byref(packed[0])))
    work.runtime.assert_no_overflow()

    # ---- where a layer launch spends its time: per-CTA phase timestamps (one extra pass) ----
    phases_us = None
    if kernels_per_layer == 1:
        units = slots * heads_local
        stamps = torch.zeros((launches, units, 8, 16), dtype=torch.int64, device=device)
        with torch.cuda.stream(stream):
            for launch in range(launches):
                clone = native.LayerArgs.from_buffer_copy(solo[launch])
                clone.phase_times = stamps[launch].data_ptr()
                native.call("ckv_decode_layer", clone, stream.cuda_stream)
            stream.synchronize()
        t = stamps[:, :, : packed[0].splits, :10].cpu().numpy().astype("float64") / 1e3
        t0 = t[..., 0].min(axis=(1, 2), keepdims=True)
        span = lambda a, b, ranks=slice(None): (t[:, :, ranks, b] - t[:, :, ranks, a])
        stat = lambda x: {"mean": round(float(x.mean()), 2), "max": round(float(x.max(axis=(1, 2)).mean()), 2)}
        phases_us = {
            "score": stat(span(0, 1)),
            "select_wait_for_cluster": stat(span(1, 2)),
            "select_exchanges": stat(span(2, 5)),
            "select_detail": {"histograms": stat(span(2, 3)), "threshold_scan_publish": stat(span(3, 4)),
                              "count": stat(span(4, 5))},
            "resolve_positions": stat(span(5, 6)),
            "gather_attention": stat(span(6, 7)),
            "wait_for_cluster": stat(span(7, 8, slice(0, 1))),
            "merge_update": stat(span(8, 9, slice(0, 1))),
            "launch_total": stat((t[:, :, 0:1, 9] - t0)),
            "note": "per CTA, microseconds; max = slowest CTA of a launch, averaged over the layers",
        }
        work.runtime.assert_no_overflow()

    # ---- the gather + attention kernel alone, same way ----
    attn_args = []
    for launch in range(launches):
        clone = native.LayerArgs.from_buffer_copy(solo[launch])
        clone.flags = native.FLAG_ATTENTION_ONLY | native.FLAG_SKIP_UPDATE
        attn_args.append(clone)
    kernel_ms = []
    with torch.cuda.stream(stream):
        for repeat in range(3):
            events = []
            for launch in range(launches):
                first, second = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                first.record()
                native.call("ckv_segmented_attention", attn_args[launch], stream.cuda_stream)
                second.record()
                events.append((first, second))
            stream.synchronize()
            if repeat > 0:
                kernel_ms.extend(a.elapsed_time(b) for a, b in events)
    attention_ms = statistics.mean(kernel_ms)
    clocks = sampler.stop() if rank == 0 else {}

    # ---- end to end: host queries and new K/V rows in, head outputs out, every step ----
    # A token is two graph replays.  The first holds the leading layers, whose inputs come in a
    # small copy; the second holds the other layers, whose inputs come in a second copy that
    # runs on the copy stream beside the first replay.  Inside the second replay the head
    # outputs go back to the host a few layers at a time on the copy stream, beside the layers
    # still to run; only the last piece is read after the last layer.  The row the new K/V
    # land in is a device cursor that the token advances itself.
    pinned_in = torch.randn((e2e_steps, launches, query_count + 2 * row_count))
    pinned_in[:, :, query_count:] *= SCALE
    pinned_in = pinned_in.to(torch.bfloat16).pin_memory()
    # every rank reads back the head outputs it computed (together the ranks read the whole result once)
    pinned_out = torch.empty((launches, slots, query_local, HEAD_DIM), dtype=torch.bfloat16).pin_memory()
    result = exchange.gathered[:, rank] if exchange is not None else out_local
    cursor = work.state(0).current_position.max().to(torch.int32).reshape(1).clone()
    copies = torch.cuda.Stream(device)
    lead = launches // 9  # a ninth of the layers: 4 of 36
    pieces = 4 if launches >= 8 else 1
    piece_ends = [launches * (piece + 1) // pieces for piece in range(pieces)]

    def append_rows(first: int, last: int) -> None:
        ops.append_kv(work.key[first:last], work.value[first:last], new_key[first:last],
                      new_value[first:last], cursor)

    def read_back(launch: int) -> None:
        if launch + 1 not in piece_ends[:-1]:
            return
        index = piece_ends.index(launch + 1)
        begin = piece_ends[index - 1] if index else 0
        produced = torch.cuda.Event()
        produced.record(stream)
        copies.wait_event(produced)
        with torch.cuda.stream(copies):
            pinned_out[begin:launch + 1].copy_(result[begin:launch + 1], non_blocking=True)

    def enqueue_lead() -> None:
        append_rows(0, lead)
        enqueue_step(0, lead)

    def enqueue_rest() -> None:
        append_rows(lead, launches)
        cursor.add_(1)
        enqueue_step(lead, launches, after_layer=read_back)
        begin = piece_ends[-2] if pieces > 1 else 0
        pinned_out[begin:].copy_(result[begin:], non_blocking=True)
        if pieces > 1:
            returned = torch.cuda.Event()
            returned.record(copies)
            stream.wait_event(returned)

    lead_graph = rest_graph = None
    if use_graph:
        rest_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(rest_graph, stream=stream):
            enqueue_rest()
        if lead:
            lead_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(lead_graph, stream=stream):
                enqueue_lead()

    def replay_or_enqueue(graph, enqueue) -> None:
        if graph is not None:
            graph.replay()
        else:
            enqueue()

    def token(step: int) -> None:
        source = pinned_in[step]
        if lead:
            staged[:lead].copy_(source[:lead], non_blocking=True)
            first_arrived, all_arrived = torch.cuda.Event(), torch.cuda.Event()
            first_arrived.record(stream)
            copies.wait_event(first_arrived)  # one copy at a time in this direction
            with torch.cuda.stream(copies):
                staged[lead:].copy_(source[lead:], non_blocking=True)
                all_arrived.record(copies)
            replay_or_enqueue(lead_graph, enqueue_lead)
            stream.wait_event(all_arrived)
        else:
            staged.copy_(source, non_blocking=True)
        replay_or_enqueue(rest_graph, enqueue_rest)
        stream.synchronize()  # the caller reads the token's output before the next token

    with torch.cuda.stream(stream):
        for warm in range(2):  # untimed: the first replays of a new graph also upload it
            token(warm)
    barrier()
    e2e_begin, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e2e_begin.record()
        for step in range(e2e_steps):
            token(step)
        e2e_end.record()
    barrier()
    e2e_ms = torch.tensor([e2e_begin.elapsed_time(e2e_end)], device=device)
    if world > 1:
        dist.all_reduce(e2e_ms, op=dist.ReduceOp.MAX)
    e2e_ms_per_step = float(e2e_ms) / e2e_steps
    if not torch.equal(pinned_out, result.cpu()):
        raise RuntimeError("the head outputs read back piece by piece differ from the ones on the device")
    work.runtime.assert_no_overflow()
    if exchange is not None:
        exchange.check()

    # ---- roofline ----
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    if peaks_path.exists():
        peak = float(json.loads(peaks_path.read_text())["hbm_gbs"])
        peak_source = "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_source = 6650.0, "fallback"
    units_per_launch = slots * heads_local
    kv_bytes_per_unit = 2 * BUDGET * HEAD_DIM * 2
    attention_gbs = units_per_launch * kv_bytes_per_unit / (attention_ms * 1e-3) / 1e9
    centroid_bytes = sum(work.community_counts) * HEAD_DIM
    step_bytes = centroid_bytes + launches * units_per_launch * kv_bytes_per_unit
    layer_bytes = step_bytes // launches  # centroids + selected KV of one launch (mean over layers)
    # Average duration of a layer launch inside the timed region: the launches of a step run
    # back to back on the stream, each starting its prologue under the tail of the one before
    # (programmatic dependent launch), so the step time divided by the launches is what one
    # launch costs there.  `launch_ms_isolated` is the same launch bracketed by events of its own.
    launch_ms_in_step = ms_per_step / launches
    layer_gbs = layer_bytes / (launch_ms_in_step * 1e-3) / 1e9
    isolated_gbs = layer_bytes / (layer_launch_ms * 1e-3) / 1e9
    step_gbs = step_bytes / (ms_per_step * 1e-3) / 1e9

    traffic, traffic_source = measured_traffic(units_per_launch, kernels_per_layer)
    if rank != 0:
        finish(world, dist)
        return
    line = {
        "metric": METRIC,
        "value": batch / (ms_per_step * 1e-3),
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "us_per_step": ms_per_step * 1e3,
        "higher_is_better": True,
        "scaling": args.scaling,
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": workload_config(args, batch=batch, world=world, exchange_mode=exchange_mode),
        "roofline": {
            "kernel": (
                "decode_cluster_kernel (one launch per layer: centroid scoring, selection, KV gather + "
                "segmented flash-decode, split merge" + ("" if deferred else ", online update") + ")"
                if kernels_per_layer == 1 else
                "score_kernel + select_kernel + attention_kernel + merge_update_kernel (one layer)"
            ),
            "bound": "hbm",
            "achieved": layer_gbs,
            "peak": peak,
            "unit": "GB/s",
            "frac": layer_gbs / peak,
            "peak_source": peak_source,
            "traffic": traffic,
            "traffic_source": traffic_source,
            "algorithmic_bytes_per_launch": layer_bytes,
            "launch_ms": launch_ms_in_step,
            "launch_ms_isolated": layer_launch_ms,
            "frac_isolated": isolated_gbs / peak,
            "kernels_per_layer": kernels_per_layer,
            "attention_kernel_alone": {
                "achieved": attention_gbs,
                "frac": attention_gbs / peak,
                "algorithmic_bytes_per_launch": units_per_launch * kv_bytes_per_unit,
                "launch_ms": attention_ms,
            },
        },
        "step_roofline": {
            "bytes_per_step_per_gpu": step_bytes,
            "achieved": step_gbs,
            "frac": step_gbs / peak,
            "note": "centroids + selected KV of all layers / whole-step time",
        },
        "e2e": {
            "value": batch / (e2e_ms_per_step * 1e-3),
            "unit": "tokens/s",
            "ms_per_step": e2e_ms_per_step,
            "steps": e2e_steps,
            "h2d_bytes_per_step": int(pinned_in[0].numel() * 2),
            "d2h_bytes_per_step": int(pinned_out.numel() * 2),
        },
        "phases_us": phases_us,
        "gpu_launches": args.steps * launches * (kernels_per_layer + (1 if deferred else 0)),
        "cuda_graph": use_graph,
        "clocks": clocks,
        "build_seconds": build_seconds,
    }
    if world == 1 and not args.no_prefill:
        # the other kernel of the path, measured in the same run: prefill score-graph emission
        del work, packed, attend_args, update_args, solo, attn_args
        torch.cuda.empty_cache()
        line["prefill"] = measure_prefill(args, device, steps=5, warmup=3)
        work = None
    if world == 1 and not args.no_cpu_baseline:
        work = None
        torch.cuda.empty_cache()
        line["cpu_baseline"] = cpu_baseline(args.cpu_seconds, args.context, args.layers)
    print(json.dumps(line), flush=True)
    finish(world, dist)


def finish(world: int, dist) -> None:
    """Leave a multi-rank run without tearing NCCL down.

    The process group is still referenced by the captured CUDA graph; destroying
    it at this point can block for ever.  Everything has been measured and
    printed, so the ranks meet at a barrier and exit directly.
    """

    if world > 1:
        dist.barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def measure_prefill(args: argparse.Namespace, device, steps: int, warmup: int) -> dict:
    """Times the prefill score-graph emission kernel: one layer, 32/8 heads, causal, planted key clusters."""

    import torch

    from community_kv_b200.prefill import (
        check_status,
        prefill_attention,
        prefill_attention_edges,
        prefill_attention_topk,
    )

    length = args.prefill_length
    generator = torch.Generator(device=device).manual_seed(args.seed)
    centres = torch.randn((KV_HEADS, 256, HEAD_DIM), generator=generator, device=device)
    labels = torch.randint(0, 256, (length, KV_HEADS), generator=generator, device=device)
    key = centres[torch.arange(KV_HEADS, device=device).view(1, -1), labels]
    key = ((key + 0.3 * torch.randn(key.shape, generator=generator, device=device)) * SCALE).to(torch.bfloat16)[None]
    value = (torch.randn((1, length, KV_HEADS, HEAD_DIM), generator=generator, device=device) * SCALE).to(torch.bfloat16)
    query = torch.randn((1, length, QUERY_HEADS, HEAD_DIM), generator=generator, device=device).to(torch.bfloat16)
    flops = 2.0 * length * length * HEAD_DIM * QUERY_HEADS  # causal Q.K^T + P.V
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["bf16_tflops"]) if peaks_path.exists() else 1590.0
    # one status word for the whole run: the calls queue without a host round trip and the
    # word is read after each timed loop
    status = torch.zeros((1,), dtype=torch.int32, device=device)
    variants = {
        "attention_only": lambda: prefill_attention(query, key, value, softmax_scale=SCALE, status=status),
        "reference_top8": lambda: prefill_attention_topk(
            query, key, value, softmax_scale=SCALE, num_sink=NUM_SINK, status=status),
        "exact_top16_per_kv_head": lambda: prefill_attention_edges(
            query, key, value, softmax_scale=SCALE, num_sink=NUM_SINK, edges_per_row=16, status=status),
    }
    timings = {}
    rescanned = None
    for name, run in variants.items():
        for _ in range(max(warmup, 3)):
            result = run()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(steps):
            result = run()
        end.record()
        torch.cuda.synchronize()
        timings[name] = begin.elapsed_time(end) / steps
        check_status(status)
        if name == "exact_top16_per_kv_head":
            rescanned = int(result[4].sum())
    headline = timings["exact_top16_per_kv_head"]
    return {
        "workload": "prefill score-graph emission: 1 layer, 32 Q / 8 KV heads, head_dim 128, "
                    f"S={length}, causal, 256 planted key clusters",
        "variants_ms": timings,
        "rows_rescanned": rescanned,
        "steps": steps,
        "flops": flops,
        "roofline": {
            "kernel": "prefill_pair_kernel (tcgen05 Q.K^T and P.V, P in tensor memory)",
            "bound": "tensor",
            "achieved": flops / (timings["attention_only"] * 1e-3) / 1e12,
            "achieved_with_reference_top8": flops / (timings["reference_top8"] * 1e-3) / 1e12,
            "achieved_with_edges": flops / (headline * 1e-3) / 1e12,
            "peak": peak,
            "unit": "TFLOP/s",
            "frac": flops / (timings["attention_only"] * 1e-3) / 1e12 / peak,
            "traffic": None,
        },
    }


def run_prefill(args: argparse.Namespace) -> None:
    """Prefill score-graph emission as a line of its own."""

    import torch

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    sampler = ClockSampler(device.index or 0)
    sampler.start()
    record = measure_prefill(args, device, args.steps, args.warmup)
    clocks = sampler.stop()
    headline = record["variants_ms"]["exact_top16_per_kv_head"]
    line = {
        "metric": "prefill score-graph emission, ms per layer (S=%d, 32/8 heads, top-16 edges per KV head)"
                  % args.prefill_length,
        "value": headline,
        "unit": "ms",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": max(args.warmup, 3),
        "ms_per_step": headline,
        "higher_is_better": False,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": record["workload"], "l2": "each step streams 2*S*8*256 B of K/V per query tile"},
        "variants_ms": record["variants_ms"],
        "rows_rescanned": record["rows_rescanned"],
        "roofline": record["roofline"],
        "gpu_launches": args.steps * 3,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def run_sweep(args: argparse.Namespace) -> None:
    """Sequence-sharded single-layer stress: one sequence of 1M tokens,
    32/8 heads, 16384 planted clusters, budget 8192, K/V rows split across the GPUs."""

    import torch
    import torch.distributed as dist

    from community_kv_b200 import distributed as ckv_dist
    from community_kv_b200.config import CommunityKVConfig
    from community_kv_b200.sequence_shard import SequenceShardedLayer
    from community_kv_b200.workload import build_planted_layer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    clusters, budget, sinks = 16384, 8192, NUM_SINK
    steps_total = args.warmup + args.steps + 2
    converted, key, value = build_planted_layer(
        seq_len=args.sweep_context, clusters=clusters, kv_heads=KV_HEADS, group_size=QUERY_HEADS // KV_HEADS,
        num_sink=sinks, max_decode_tokens=steps_total + 4, device=device, seed=args.seed,
    )
    total_rows = key.shape[1]
    begin, end = ckv_dist.sequence_shard(total_rows, world, rank)
    config = CommunityKVConfig(token_budget=budget, num_sink=sinks, lam=0.5, aggregation="query_group")
    layer = SequenceShardedLayer(
        converted=converted, key_shard=key[:, begin:end].contiguous(), value_shard=value[:, begin:end].contiguous(),
        row_begin=begin, total_rows=total_rows, config=config, splits=args.splits or 8,
    )
    del key, value
    torch.cuda.empty_cache()
    generator = torch.Generator(device=device).manual_seed(args.seed + 99)  # same on every rank
    queries = torch.randn((steps_total, QUERY_HEADS, HEAD_DIM), generator=generator, device=device).to(torch.bfloat16)
    new_keys = (torch.randn((steps_total, KV_HEADS, HEAD_DIM), generator=generator, device=device) * SCALE).to(torch.bfloat16)

    q_cur = torch.zeros_like(queries[0])
    k_cur = torch.zeros_like(new_keys[0])
    stream = torch.cuda.Stream(device)
    # The step's inputs are picked on the device by a cursor that the step itself advances,
    # so that a whole step - input selection included - is one CUDA-graph replay (at 60-130 us
    # per step, separate copy launches would make the host the bottleneck).
    cursor = torch.zeros((1,), dtype=torch.int64, device=device)

    def enqueue() -> "torch.Tensor":
        torch.index_select(queries, 0, cursor, out=q_cur.unsqueeze(0))
        torch.index_select(new_keys, 0, cursor, out=k_cur.unsqueeze(0))
        cursor.add_(1)
        return layer.decode(q_cur, k_cur, SCALE)

    graph = None

    def step(index: int) -> None:
        with torch.cuda.stream(stream):
            if graph is not None:
                graph.replay()
            else:
                enqueue()

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(device.index or 0) if rank == 0 else None
    for index in range(args.warmup):
        step(index)
    barrier()
    # the whole step (kernels, the small combining tensor ops, the collectives) as one CUDA graph
    use_graph = True
    try:
        candidate = torch.cuda.CUDAGraph()
        with torch.cuda.graph(candidate, stream=stream):
            enqueue()
        graph = candidate
    except Exception as error:  # pragma: no cover - depends on capture support
        use_graph = False
        if rank == 0:
            print(f"[bench] graph capture unavailable ({type(error).__name__}: {error}); direct launches", file=sys.stderr)
    barrier()
    if sampler:
        sampler.start()
    first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        first.record()
    for index in range(args.warmup, args.warmup + args.steps):
        step(index)
    with torch.cuda.stream(stream):
        last.record()
    barrier()
    elapsed = torch.tensor([first.elapsed_time(last)], device=device)
    if world > 1:
        dist.all_reduce(elapsed, op=dist.ReduceOp.MAX)
    ms_per_step = float(elapsed) / args.steps
    clocks = sampler.stop() if sampler else {}
    layer.converted.mutable  # keep alive
    if int(layer.workspace.update.overflow.max()) != 0:
        raise RuntimeError("overflow during the sweep")
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["hbm_gbs"]) if peaks_path.exists() else 6650.0
    centroid_bytes = int(converted.mutable.community_counts.sum()) * HEAD_DIM
    kv_bytes = KV_HEADS * 2 * budget * HEAD_DIM * 2
    bytes_per_gpu = centroid_bytes + kv_bytes // world  # centroids are replicated, selected rows are split
    if rank != 0:
        finish(world, dist)
        return
    line = {
        "metric": "sequence-sharded sparse decode, microseconds per step (1 sequence, one layer, ctx %d, budget %d)"
                  % (args.sweep_context, budget),
        "value": ms_per_step * 1e3,
        "unit": "us",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms_per_step,
        "higher_is_better": False,
        "scaling": "strong",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {
            "workload": f"sequence-sharded single-layer decode: batch 1, 32 Q / 8 KV heads, ctx {args.sweep_context}, "
                        f"{clusters} planted clusters per head, budget {budget}, rows split x{world}",
            "exchange": "one NCCL all-gather of the ranks' merged (acc, max, sum) rows and top-8 candidates, "
                        "merged in place by ckv_merge_partials" if world > 1 else "none",
            "l2": "inputs larger than L2 (each step gathers rows scattered over the whole KV cache)",
        },
        "roofline": {
            "kernel": "score_kernel + select_kernel + attention_kernel + merge_update_kernel"
                      + (" + all-gather + merge_update_kernel over the ranks' rows" if world > 1 else ""),
            "bound": "hbm",
            "achieved": bytes_per_gpu / (ms_per_step * 1e-3) / 1e9,
            "peak": peak,
            "unit": "GB/s",
            "frac": bytes_per_gpu / (ms_per_step * 1e-3) / 1e9 / peak,
            "traffic": None,
            "algorithmic_bytes_per_launch": bytes_per_gpu,
        },
        "gpu_launches": args.steps * (4 if world == 1 else 5),
        "cuda_graph": use_graph,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    finish(world, dist)


def run_model(args: argparse.Namespace) -> None:
    """Whole-model decode behind the Hugging Face plug-in: a random-init Qwen3-8B-shaped decoder
    (36 layers, hidden 4096, 32/8 heads, head_dim 128, FFN 12288, vocab 151936, bf16), batch 1, a prompt of
    uniform-random token ids, greedy generation.  512 communities per (layer, KV head) with Zipf(1.1) sizes from
    the synthetic partitioner, budget 2048.  Reports whole-step tokens/s (Hugging Face eager loop: projections,
    MLP, norms, sampling and Python included) and, separately, the attention path (CUDA events around every
    decode-layer call)."""

    import torch
    from transformers import Qwen3Config, Qwen3ForCausalLM

    from community_kv_b200 import CommunityKVAttention, CommunityKVConfig, CommunityKVRuntime, PartitionConfig
    from community_kv_b200.synthetic import SyntheticPartitioner

    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    layers = args.model_layers
    config = Qwen3Config(
        hidden_size=4096, intermediate_size=12288, num_hidden_layers=layers, num_attention_heads=QUERY_HEADS,
        num_key_value_heads=KV_HEADS, head_dim=HEAD_DIM, vocab_size=151936,
        max_position_embeddings=args.prompt_length + args.new_tokens + 8, tie_word_embeddings=False,
    )
    torch.manual_seed(args.seed)
    build_begin = time.perf_counter()
    with torch.device(device):
        previous = torch.get_default_dtype()
        torch.set_default_dtype(torch.bfloat16)
        try:
            model = Qwen3ForCausalLM(config).eval()
        finally:
            torch.set_default_dtype(previous)
    build_seconds = time.perf_counter() - build_begin
    generator = torch.Generator().manual_seed(args.seed)
    prompt = torch.randint(0, config.vocab_size, (1, args.prompt_length), generator=generator).to(device)
    ckv = CommunityKVConfig(token_budget=BUDGET, num_sink=NUM_SINK, lam=0.5, aggregation="query_group",
                            online_assignment=args.online_assignment)
    partitioner = SyntheticPartitioner(communities=512, zipf_exponent=ZIPF, seed=args.seed)
    sampler = ClockSampler(device.index or 0)
    with CommunityKVRuntime(config=ckv, partition=PartitionConfig(), num_layers=layers,
                            max_decode_tokens=args.new_tokens, partitioner=partitioner) as runtime:
        model.config._attn_implementation = CommunityKVAttention(runtime).register()
        decode = runtime.decode_runtime.decode
        spans: list[tuple] = []

        def timed_decode(**kwargs):
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            out = decode(**kwargs)
            end.record()
            spans.append((begin, end))
            return out

        runtime.decode_runtime.decode = timed_decode
        first_decode = {}
        ensure_ready = runtime.ensure_ready

        def mark_ready():
            if "t" not in first_decode:
                torch.cuda.synchronize()
                first_decode["t"] = time.perf_counter()
            ensure_ready()

        runtime.ensure_ready = mark_ready
        sampler.start()
        torch.cuda.synchronize()
        begin = time.perf_counter()
        with torch.no_grad():
            output = runtime.generate(model, prompt, max_new_tokens=args.new_tokens)
        torch.cuda.synchronize()
        end = time.perf_counter()
        clocks = sampler.stop()
    decode_tokens = args.new_tokens - 1
    decode_seconds = end - first_decode["t"]
    attention_ms = sum(a.elapsed_time(b) for a, b in spans)
    per_token_attention_ms = attention_ms / max(decode_tokens, 1)
    peaks_path = ROOT / "MEASURED_PEAKS.json"
    peak = float(json.loads(peaks_path.read_text())["hbm_gbs"]) if peaks_path.exists() else 6650.0
    bytes_per_token = layers * KV_HEADS * (512 * HEAD_DIM + 2 * BUDGET * HEAD_DIM * 2)
    line = {
        "metric": "whole-model sparse decode tokens/s behind the Hugging Face plug-in (batch 1)",
        "value": decode_tokens / decode_seconds,
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": decode_tokens,
        "warmup": 0,
        "ms_per_step": 1e3 * decode_seconds / max(decode_tokens, 1),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic",
        "config": {
            "workload": f"random-init Qwen3-8B-shaped decoder ({layers} layers, hidden 4096, 32/8 heads, FFN 12288, "
                        f"vocab 151936), batch 1, prompt {args.prompt_length} random ids, {args.new_tokens} new tokens, "
                        f"512 Zipf({ZIPF}) communities per (layer, KV head), budget {BUDGET}, "
                        f"online assignment: {args.online_assignment}",
            "loop": "Hugging Face generate, eager (no CUDA graph): projections, MLP, norms and sampling included",
        },
        "prefill_seconds": first_decode["t"] - begin,
        "attention_path": {
            "ms_per_token": per_token_attention_ms,
            "us_per_layer_call": 1e3 * attention_ms / max(len(spans), 1),
            "calls": len(spans),
            "algorithmic_bytes_per_token": bytes_per_token,
            "achieved_gbs": bytes_per_token / (per_token_attention_ms * 1e-3) / 1e9,
            "frac_of_hbm_peak": bytes_per_token / (per_token_attention_ms * 1e-3) / 1e9 / peak,
            "note": "CUDA events around every decode-layer call (one launch each); one sequence gives a launch "
                    "only 8 units, so this is the latency of the phase chain, not a bandwidth figure",
        },
        "generated": int(output.shape[-1] - args.prompt_length),
        "gpu_launches": len(spans),
        "clocks": clocks,
        "build_seconds": build_seconds,
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    args = parse_args()
    if args.workload == "model" and args.impl != "reference":
        run_model(args)
        return
    if args.workload == "prefill" and args.impl != "reference":
        run_prefill(args)
        return
    if args.workload == "sweep" and args.impl != "reference":
        run_sweep(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
