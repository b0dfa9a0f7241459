#!/usr/bin/env python
"""Headline benchmark: one Qwen3-8B dense decode layer per step (batch 1, KV
length 4096, bf16), tensor-parallel over N GPUs of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

One JSON line on rank 0.  ``value`` is the achieved HBM bandwidth of the whole
job: algorithmic bytes of one layer step (every weight and every valid KV row
once; the same total at every N, so scaling is "strong") divided by the device
time of a step, timed with CUDA events over exactly K steps replayed from a CUDA
graph, max over ranks.  Steps rotate over four independent sets of layer weights
and KV caches (1.6 GB), so no step finds its inputs in L2.  The timed steps are
enqueued directly behind ``--lead-in`` untimed ones (no host synchronisation in
between), so with several ranks the processes' launch skew is absorbed before the
first timed step and the clock samples describe the load the steps run under.
At batch 1 a step is ONE kernel launch per GPU (the whole layer as a persistent
kernel; with several ranks both sums over ranks happen inside it, over NVLink peer
memory); at one GPU ``roofline`` describes that kernel and ``weight_streaming_leg``
the stand-alone GEMV kernel the other paths are built on.  Above batch 8 the ranks
run three local parts with the library's own all-reduce kernel in between
(``--exchange nccl`` puts NCCL there; ``--exchange-only`` times the sums alone).
The process returns normally (exit hooks run); with several ranks the process
group is destroyed under a guard timer.

Further legs, all outside the timed region of ``value``:
  e2e          the same layer through the operator API with the step's input and
               result in pinned host memory: a copy-in kernel, the layer (whose last
               kernel stores into the pinned result buffer), stream sync and a host
               read, every step (weights and KV cache are resident state).
  roofline     one GPU, batch 1: the single-kernel layer, from the timed region
               itself; otherwise the weight-streaming GEMV timed alone on a
               gate/up-sized weight; both against the measured HBM copy peak.
  cpu_baseline the CPU oracle (torch on the host cores) on the same layer.
``--impl reference`` times that CPU path as its own arm.
"""

from __future__ import annotations

import argparse
import json
import os
import signal
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

NUM_WEIGHT_SETS = 4
METRIC = "qwen3_8b_decode_layer_achieved_hbm_gbs"
UNIT = "GB/s"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--exchange", choices=["auto", "fused", "nccl", "peer"], default="auto",
                    help="N > 1: how the two sums over ranks of a layer are done")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=["qwen3-8b", "qwen3-32b"], default="qwen3-8b")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--no-graph", action="store_true", help="time eager launches instead of a CUDA graph")
    ap.add_argument("--skip-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--calls", choices=["auto", "layer", "stack"], default="auto",
                    help="layer: one C call per step (the reference operator's granularity).  stack: the timed steps are "
                         "issued as multi-layer calls (ezb_qwen3_decode_stack / ..._tp_fused); a step is still one layer, "
                         "but at N > 1 a layer's second sum is folded into the next layer's first kernel.  auto: layer at "
                         "N = 1, stack at N > 1 when the fused exchange applies")
    ap.add_argument("--stack", action="store_true", help="same as --calls stack")
    ap.add_argument("--roofline-only", action="store_true",
                    help="run only the roofline leg (a few launches of the dominant kernel): the command an ncu capture wraps")
    ap.add_argument("--exchange-only", action="store_true",
                    help="N > 1: time only the two NCCL all-reduces of a layer ([batch, hidden] fp32 each), no compute: "
                         "the collective's share of a step of --exchange nccl")
    ap.add_argument("--lead-in", type=int, default=200,
                    help="untimed steps issued directly in front of the timed ones (same stream, no host sync in between)")
    ap.add_argument("--no-cross-call-pdl", action="store_true",
                    help="order the first kernel of every layer call fully after the previous call")
    return ap.parse_args()


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


# ----------------------------------------------------------------- clocks ---
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the
    timed region runs (read-only queries)."""

    BAD = {
        0x0000000000000008: "hw_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
    }
    NOTED = {0x0000000000000004: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.0004):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if index < len(ids) and ids[index].isdigit():
                    phys = int(ids[index])
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM)
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
                for bit, name in {**self.BAD, **self.NOTED}.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self._nvml is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


# ------------------------------------------------------------- CPU oracle ---
def cpu_layer_arm(shape, batch, seq_len, budget_s=15.0, max_calls=50, min_calls=3):
    """Times the CPU oracle of the layer on the host cores with every thread the
    process may use.  Returns (seconds per call, calls, threads)."""
    from ezops_b200 import workloads as wl
    from oracle import ezops_oracle as orc

    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    data = wl.decode_layer_inputs(shape, batch, seq_len)
    heads = (shape.num_heads, shape.num_kv_heads, shape.head_dim)
    orc.qwen3_dense_decode_ref(*data, *heads)  # warm-up
    times = []
    t_start = time.perf_counter()
    while len(times) < max_calls and (len(times) < min_calls or time.perf_counter() - t_start < budget_s):
        t0 = time.perf_counter()
        orc.qwen3_dense_decode_ref(*data, *heads)
        times.append(time.perf_counter() - t0)
    times.sort()
    return times[len(times) // 2], len(times), torch.get_num_threads()


def run_reference_arm(args, shape, total_bytes):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from ezops_b200 import workloads as wl
    from oracle import ezops_oracle as orc

    steps = args.steps if args.steps is not None else 20
    warmup = args.warmup if args.warmup is not None else 3
    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    data = wl.decode_layer_inputs(shape, args.batch, args.seq_len)
    heads = (shape.num_heads, shape.num_kv_heads, shape.head_dim)
    for _ in range(warmup):
        orc.qwen3_dense_decode_ref(*data, *heads)
    t0 = time.perf_counter()
    for _ in range(steps):
        orc.qwen3_dense_decode_ref(*data, *heads)
    dt = (time.perf_counter() - t0) / steps
    value = total_bytes / dt / 1e9
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": dt * 1e3, "us_per_layer": dt * 1e6, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (seeded torch.randn, N(0,0.02) weights)",
        "config": workload_config(args, shape, args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": f"{steps} full layer steps of the CPU oracle (the reference's torch _ref_forward restated)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def resolve_calls(args, n):
    """How the timed steps are issued: 'layer' (one C call per step) or 'stack' (multi-layer calls).  The rule is
    shared by both arms so that their ``config`` objects are equal."""
    if getattr(args, "stack", False) or args.calls == "stack":
        return "stack"
    if args.calls == "layer":
        return "layer"
    exchange = args.exchange
    if exchange == "auto":
        exchange = "fused" if args.batch <= 8 else "peer"
    return "stack" if n > 1 and exchange == "fused" else "layer"


def workload_config(args, shape, n):
    return {
        "workload": (f"{shape.name} dense decode layer, batch {args.batch}, kv_len {args.seq_len}, bf16, tp{n}"
                     + (" - EXCHANGE ONLY: the layer's two all-reduces, no compute" if getattr(args, "exchange_only", False) else "")),
        "hidden": shape.hidden, "intermediate": shape.inter, "heads": f"{shape.num_heads}q/{shape.num_kv_heads}kv x {shape.head_dim}",
        "parallelism": f"tp{n}",
        "cache_policy": f"inputs larger than L2: steps rotate over {NUM_WEIGHT_SETS * n} weight+KV sets per GPU",
        "pdl_across_calls": not getattr(args, "no_cross_call_pdl", False),
        "calls": "one multi-layer call per graph" if resolve_calls(args, n) == "stack" else "one call per layer",
    }


def ncu_traffic(kernel: str, rows: int, cols: int, batch: int):
    """DRAM bytes (read + write) of one launch, from the ncu captures summarised under profiles/ (the table
    profiles/ncu_dram_traffic.json names the summary each entry comes from).  An entry for the same kernel, batch
    and row length but another number of rows is scaled by the rows (traffic is the weight stream: it grows in
    proportion); returns (bytes or None, how)."""
    path = ROOT / "profiles" / "ncu_dram_traffic.json"
    try:
        table = json.loads(path.read_text())["entries"]
    except Exception:
        return None, "no table"
    same = [e for e in table if e["kernel"] == kernel and e["cols"] == cols and e["batch"] == batch]
    for e in same:
        if e["rows"] == rows:
            return e["dram_read_bytes"] + e["dram_write_bytes"], f"ncu capture ({e['summary']})"
    if same and kernel != "decode_layer_b1_kernel":  # the whole-layer kernel's traffic is not proportional to one size
        e = same[0]
        scaled = (e["dram_read_bytes"] + e["dram_write_bytes"]) * rows / e["rows"]
        return int(scaled), f"scaled by rows from the ncu capture at {e['rows']} rows ({e['summary']})"
    return None, "no capture of this shape"


def roofline_leg(sets, nsets, hidden0, B, H, device, n_roof):
    """The dominant kernel timed alone: a GEMV over a gate/up-sized weight (rank 0's shard at N > 1)."""
    import torch

    from ezops_b200 import _lib

    peaks, peak_kind = measured_peaks()
    lib = _lib.load()
    rows_local = sets[0][4].shape[0]
    Y = torch.empty(B, rows_local, dtype=torch.bfloat16, device=device)
    ws = torch.zeros(lib.ezb_gemv_workspace_bytes(B, rows_local, H), dtype=torch.uint8, device=device)
    X = hidden0

    def roof_launch(i):
        W = sets[i % nsets][4]
        _lib.check(lib.ezb_gemv_batched_bf16(X.data_ptr(), W.data_ptr(), Y.data_ptr(), ws.data_ptr(), ws.numel(), B,
                                             rows_local, H, torch.cuda.current_stream().cuda_stream))

    for i in range(8):
        roof_launch(i)
    torch.cuda.synchronize()
    r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    r0.record()
    for i in range(n_roof):
        roof_launch(i)
    r1.record()
    torch.cuda.synchronize()
    launch_s = r0.elapsed_time(r1) * 1e-3 / n_roof
    kernel_bytes = 2 * (rows_local * H + B * H + B * rows_local)
    achieved = kernel_bytes / launch_s / 1e9
    traffic, traffic_how = ncu_traffic("gemv_rows8_kernel" if B <= 8 else "gemm_tc_kernel", rows_local, H, B)
    roofline = {
        "bound": "hbm", "kernel": "gemv_rows8_kernel" if B <= 8 else "gemm_tc_kernel", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
        "frac": achieved / peaks["hbm_gbs"], "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs, burst copy)",
        "traffic": traffic, "traffic_source": traffic_how, "bytes_per_launch": kernel_bytes, "us_per_launch": launch_s * 1e6,
        "workload": f"W [{rows_local}, {H}] bf16 (gate/up-sized), batch {B}, {n_roof} back-to-back launches over {nsets} weights",
    }
    return roofline


# ------------------------------------------------------------------- main ---
def main():
    args = parse_args()
    from ezops_b200 import workloads as wl

    shape = wl.QWEN3_8B if args.model == "qwen3-8b" else wl.QWEN3_32B
    total_bytes = shape.algorithmic_bytes(args.batch, args.seq_len)

    if args.impl == "reference":
        run_reference_arm(args, shape, total_bytes)
        return

    import torch.distributed as dist

    import ezops_b200 as ez
    from ezops_b200 import _lib
    from ezops_b200 import tp as tpm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run --nproc-per-node N")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    tp = world
    # A decode loop over resident, immutable weights: let the first kernel of a
    # layer request its weight tiles while the previous layer's last kernel drains.
    _lib.set_tuning(pdl_across_calls=0 if args.no_cross_call_pdl else 1)
    steps = args.steps if args.steps is not None else 1000
    warmup = max(3, args.warmup if args.warmup is not None else 20)
    B, S, H, I = args.batch, args.seq_len, shape.hidden, shape.inter
    NH, NKV, D = shape.num_heads, shape.num_kv_heads, shape.head_dim

    # ---- resident state: nsets layers' weights and KV caches (a rank's shard shrinks
    # with the number of ranks, so the number of sets grows with it: every rank
    # always rotates over more than four times the L2 capacity) ----
    nsets = NUM_WEIGHT_SETS * tp
    gen = torch.Generator(device=device)
    sets, full0 = [], None
    for i in range(nsets):
        gen.manual_seed(1000 + i)  # same seed on every rank: consistent shards
        rn = lambda *s, std=1.0: (torch.randn(*s, generator=gen, device=device, dtype=torch.float32) * std).to(torch.bfloat16)
        Wqkv, Wo = rn(shape.q_rows + 2 * shape.kv_rows, H, std=0.02), rn(H, shape.q_rows, std=0.02)
        Wgu, Wd = rn(2 * I, H, std=0.02), rn(H, I, std=0.02)
        Kc, Vc = rn(B, NKV, S, D), rn(B, NKV, S, D)
        if tp > 1:
            if i == 0 and rank == 0:
                full0 = (Kc, Vc, Wqkv, Wo, Wgu, Wd)  # the unsharded layer, for the check against the torch reference
            Wqkv, Wo, Wgu, Wd = tpm.shard_layer_weights(Wqkv, Wo, Wgu, Wd, NH, NKV, D, tp, rank)
            Kc, Vc = tpm.shard_kv_cache(Kc, tp, rank), tpm.shard_kv_cache(Vc, tp, rank)
        sets.append((Kc, Vc, Wqkv, Wo, Wgu, Wd))
        torch.cuda.empty_cache()
    gen.manual_seed(7)
    hidden0 = torch.randn(B, H, generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)

    if args.roofline_only:
        print(json.dumps({"roofline": roofline_leg(sets, nsets, hidden0, B, H, device, 4)}), flush=True)
        return

    lay, stacks, e2e_graphs = None, {}, None
    if tp == 1:
        op = ez.Qwen3DenseDecodeOp(B, S, H, I, NH, D, backend="cuda", num_kv_heads=NKV)
        kernel = op._kernel
        launches_per_step = 5

        def layer(hidden, wset, out):
            return kernel(hidden, *wset, out=out)
    else:
        # Sums over ranks inside the projection kernels (peer stores over NVLink) when the
        # batch allows it, NCCL all-reduce between the three local parts otherwise.
        exchange = args.exchange
        if exchange == "auto":
            # the sums inside the kernels win where a layer is latency-bound (batch <= 8); above that the three
            # parts with the library's own all-reduce over peer memory in between (measured faster than NCCL's:
            # Qwen3-32B batch 64 on 2 / 4 GPUs 318.7 / 231.6 us per layer against 329.8 / 243.9)
            exchange = "fused" if B <= 8 else "peer"
        lay = tpm.TensorParallelDecodeLayer(B, S, H, I, NH, D, NKV, exchange=exchange)
        launches_per_step = 6 if exchange == "fused" else (10 if exchange == "peer" else 7)

        def layer(hidden, wset, out):
            return lay(hidden, *wset, out=out)

        if args.exchange_only:
            partial = torch.zeros(B, H, dtype=torch.float32, device=device)

            def layer(hidden, wset, out):  # noqa: F811 - the layer's two sums over ranks and nothing else
                if exchange == "peer":
                    comm = lay._fused_comm(device)
                    s = torch.cuda.current_stream().cuda_stream
                    for which in (0, 1):
                        _lib.check(_lib.load().ezb_tp_allreduce_f32(partial.data_ptr(), comm["bases"], tp, rank, which, B, H, s))
                    return out
                dist.all_reduce(partial)
                dist.all_reduce(partial)
                return out

    bufs = [torch.empty_like(hidden0) for _ in range(2)]

    def run_steps(n, first=0):
        h = hidden0
        for i in range(n):
            out = bufs[(first + i) & 1]
            layer(h, sets[(first + i) % nsets], out)
            h = out

    if args.calls == "stack":
        args.stack = True
    elif args.calls == "auto" and tp > 1 and exchange == "fused":
        args.stack = True
    if args.stack:
        names = ("K_cache", "V_cache", "Wqkv", "Wo", "Wgu", "Wd")
        as_layers = [dict(zip(names, wset)) for wset in sets]
        # `stacks`: multi-layer executors by layer count (created in the same order on every rank)

        def stack_for(n):
            if n not in stacks:
                if tp == 1:
                    stacks[n] = ez.get_kernel("qwen3_decode_stack", "cuda")(B, S, H, I, NH, D, n, num_kv_heads=NKV)
                else:
                    stacks[n] = tpm.TensorParallelDecodeStack(B, S, H, I, NH, D, NKV, n)
            return stacks[n]

        def run_steps(n, first=0):  # noqa: F811 - the multi-layer form of the loop above
            stack_for(n)(hidden0, [as_layers[(first + i) % nsets] for i in range(n)], None, None, out=bufs[0])

        def layer(hidden, wset, out):  # noqa: F811 - one-layer stack call (self-check and e2e leg)
            return stack_for(1)(hidden, [dict(zip(names, wset))], None, None, out=out)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # One step checked against the torch reference on the unsharded weights (every rank takes part in the step,
    # rank 0 holds the reference): the correctness bit of this line, at every N.
    ref_op = ez.Qwen3DenseDecodeOp(B, S, H, I, NH, D, backend="ref", num_kv_heads=NKV)
    got = layer(hidden0, (sets[0][0].clone(), sets[0][1].clone()) + sets[0][2:], torch.empty_like(hidden0))
    sync_all()
    check = None
    if rank == 0 and not args.exchange_only:
        ref_set = sets[0] if tp == 1 else full0
        ref = ref_op._ref_forward(hidden0, ref_set[0].clone(), ref_set[1].clone(), *ref_set[2:])
        check = bool(ref_op.check(got, ref))
        del ref
    full0 = None
    torch.cuda.empty_cache()

    run_steps(warmup)
    sync_all()
    # launches per step, counted by the library while one step is issued eagerly
    lib_ = _lib.load()
    n0 = lib_.ezb_launch_count()
    run_steps(1)
    launches_per_step = int(lib_.ezb_launch_count() - n0)
    sync_all()

    unroll = 1
    graph = None
    if not args.no_graph:
        unroll = max(d for d in range(1, 65) if steps % d == 0)
        if args.stack:  # the executor for `unroll` layers allocates on first use: not inside a capture
            run_steps(unroll)
            sync_all()
        try:
            graph = torch.cuda.CUDAGraph()
            n0 = lib_.ezb_launch_count()
            with torch.cuda.graph(graph):
                run_steps(unroll)
            launches_per_step = (lib_.ezb_launch_count() - n0) / unroll  # what one replay launches, per step
            graph.replay()  # untimed: first replay pays graph upload
            sync_all()
        except Exception as exc:  # pragma: no cover - depends on the runtime
            print(f"[bench] CUDA graph capture failed ({type(exc).__name__}: {exc}); timing eager launches", file=sys.stderr)
            graph, unroll = None, 1
            torch.cuda.synchronize()

    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def issue_steps(n):
        if graph is not None:
            for _ in range(n // unroll):
                graph.replay()
        else:
            run_steps(n)

    # The timed steps follow untimed steps of the same kind on the stream with no host synchronisation in between:
    # the ranks are then coupled on the device (by the exchange inside the steps) before t0, so host launch skew
    # between the processes is not charged to the first timed step; the clock sampler sees the same load before
    # and during the timed region (a 20-step region alone is shorter than one NVML query).
    lead_in = max(unroll, (max(args.lead_in, 1) + unroll - 1) // unroll * unroll)
    sync_all()
    with ClockSampler(local_rank) as clocks:
        issue_steps(lead_in)
        t0.record()
        issue_steps(steps)
        t1.record()
        torch.cuda.synchronize()
    sync_all()
    elapsed_ms = torch.tensor([t0.elapsed_time(t1)], device=device)
    if world > 1:
        dist.all_reduce(elapsed_ms, op=dist.ReduceOp.MAX)
    elapsed_ms = elapsed_ms.item()
    ms_per_step = elapsed_ms / steps
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    status = _lib.device_status()

    # ---- e2e: operator API, step input in pinned host memory ----
    e2e = None
    if not args.skip_e2e:
        n_e2e = min(steps, 300)
        host_in = torch.empty(B, H, dtype=torch.bfloat16).pin_memory()
        hidden0_host = hidden0.cpu()
        host_in.copy_(hidden0_host)
        host_out = torch.empty(B, H, dtype=torch.bfloat16).pin_memory()
        dev_in, dev_out = torch.empty_like(hidden0), torch.empty_like(hidden0)
        stream = torch.cuda.current_stream()

        # One GPU: the operator itself takes the pinned host buffers (a copy-in kernel, ezb_copy_pinned, and the layer
        # as one dependency chain; the layer's last kernel stores the result into the pinned buffer).  Tensor
        # parallel: torch copies around the rank-local call.
        host_io_by_op = tp == 1 and not args.stack

        def e2e_eager(i):
            if host_io_by_op:
                layer(host_in, sets[i % nsets], host_out)
                return
            if tp > 1:
                # the same two steps through the C ABI: a copy-in kernel, then the rank-local call with the pinned
                # result buffer as its output (device-addressable: the last kernel stores into it)
                _lib.check(lib_.ezb_copy_pinned(dev_in.data_ptr(), host_in.data_ptr(), B * H * 2, torch.cuda.current_stream().cuda_stream))
                layer(dev_in, sets[i % nsets], host_out)
                return
            dev_in.copy_(host_in, non_blocking=True)
            layer(dev_in, sets[i % nsets], dev_out)
            host_out.copy_(dev_out, non_blocking=True)

        # One CUDA graph per weight set holding the whole step (copy in, the operator call, copy out), as a
        # serving loop would keep it: a step then costs one graph launch and one stream synchronisation.
        if not args.no_graph:
            try:
                for i in range(nsets):
                    e2e_eager(i)  # everything the call allocates exists before the capture
                sync_all()
                e2e_graphs = []
                for i in range(nsets):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g):
                        e2e_eager(i)
                    e2e_graphs.append(g)
                sync_all()
            except Exception as exc:  # pragma: no cover - depends on the runtime
                print(f"[bench] e2e graph capture failed ({type(exc).__name__}: {exc}); using eager launches", file=sys.stderr)
                e2e_graphs = None
                torch.cuda.synchronize()

        def e2e_step(i):
            host_in[0, 0] = hidden0_host[0, 0]  # the step's input is produced on the host
            if e2e_graphs is not None:
                e2e_graphs[i % nsets].replay()
            else:
                e2e_eager(i)
            stream.synchronize()
            return float(host_out[0, 0])  # the step's result is consumed on the host

        for i in range(10):
            e2e_step(i)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_e2e):
            e2e_step(i)
        e1.record()
        sync_all()
        e_ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(e_ms, op=dist.ReduceOp.MAX)
        e_step = e_ms.item() / n_e2e
        # the host-side result of an end-to-end step is the result of the same step issued on device tensors
        e2e_step(0)
        same = torch.empty_like(hidden0)
        layer(hidden0, sets[0], same)
        sync_all()
        e2e_same = bool(torch.equal(host_out, same.cpu()))
        e2e = {"value": total_bytes / (e_step * 1e-3) / 1e9, "unit": UNIT, "us_per_step": e_step * 1e3, "steps": n_e2e,
               "h2d_bytes_per_step": B * H * 2, "d2h_bytes_per_step": B * H * 2, "result_equals_device_call": e2e_same,
               "launch": "one CUDA graph per step (copy in, operator call, copy out)" if e2e_graphs is not None else "eager",
               "copies": ("by the operator: pinned host tensors passed to the call (copy-in kernel ezb_copy_pinned; the layer's last "
                          "kernel stores the result into the pinned buffer)") if host_io_by_op else
                         ("copy-in kernel ezb_copy_pinned, then the rank-local call with the pinned result buffer as its output" if tp > 1
                          else "torch copy_ around the call"),
               "note": "weights and KV cache are resident device state; per-step input/output cross PCIe"}

    peaks, peak_kind = measured_peaks()
    gemv_leg = roofline_leg(sets, nsets, hidden0, B, H, device, 200)
    if tp == 1 and launches_per_step == 1:
        # One launch is the whole step: the dominant kernel's duration is the step time measured above.
        traffic, traffic_how = ncu_traffic("decode_layer_b1_kernel", S, H, B)
        roofline = {
            "bound": "hbm", "kernel": "decode_layer_b1_kernel", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": value / peaks["hbm_gbs"], "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs, burst copy)",
            "traffic": traffic, "traffic_source": traffic_how, "bytes_per_launch": total_bytes, "us_per_launch": ms_per_step * 1e3,
            "workload": f"the whole layer in one launch (weights + KV once), {steps} launches of the timed region",
        }
    else:
        roofline = gemv_leg

    # ---- CPU oracle beside it (rank 0, single-GPU run only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.skip_cpu:
        sec, calls, threads = cpu_layer_arm(shape, B, S)
        cpu = {"value": total_bytes / sec / 1e9, "unit": UNIT, "cores": threads, "kind": "port", "us_per_layer": sec * 1e6,
               "sample": f"median of {calls} full layer steps of the CPU oracle (torch, bf16 staging of the reference)"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "us_per_layer": ms_per_step * 1e3, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded torch.randn on device: N(0,1) activations/KV, N(0,0.02) weights)",
            "config": workload_config(args, shape, world),
            "algorithmic_bytes_per_step": total_bytes,
            "frac_of_8tbs": value / 8000.0, "frac_of_measured_hbm": value / peaks["hbm_gbs"],
            "timing": f"CUDA events around {steps} steps " + (f"replayed from a CUDA graph of {unroll} steps" if graph is not None else "launched eagerly")
                      + f", directly behind {lead_in} untimed steps on the same stream; max over ranks",
            "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(round(steps * launches_per_step)),
            "roofline": roofline, "weight_streaming_leg": gemv_leg, "cpu_baseline": cpu, "check_vs_torch_ref": check, "device_status": status,
        }
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()
    # Leave the normal way (interpreter exit hooks run).  With several ranks, first drop everything that holds NCCL
    # kernels or peer mappings, then destroy the process group; a guard ends the process if that teardown blocks.
    graph = e2e_graphs = None
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        for obj in [lay] + list(stacks.values()):
            if obj is not None and hasattr(obj, "close"):
                obj.close()
        guard = threading.Timer(90.0, lambda: (sys.stderr.write("[bench] process-group teardown blocked; leaving\n"), os._exit(0)))
        guard.daemon = True
        guard.start()
        dist.destroy_process_group()
        guard.cancel()


def _watchdog(signum, frame):  # a benchmark must never sit in a hang until the caller's limit
    print(json.dumps({"error": "bench.py watchdog: no result within the time limit", "impl": "ours"}), flush=True)
    os._exit(3)


if __name__ == "__main__":
    signal.signal(signal.SIGALRM, _watchdog)
    signal.alarm(int(os.environ.get("EZB_BENCH_LIMIT_S", "900")))
    main()
    signal.alarm(0)
