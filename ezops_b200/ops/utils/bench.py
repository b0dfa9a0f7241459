"""Device-side latency measurement (ezops/ops/utils/bench.py:24-150).

Protocol: eager warm-up with an L2 flush before every call; capture one call in
a CUDA graph (eager fallback with a warning if capture fails); graph warm-up;
then ``n_trials`` x ``n_repeat`` iterations of {flush L2, event, replay, event};
the result is the median of the per-trial means, in milliseconds.  The flush
buffer is as large as the device's L2 and is zeroed, so every timed call starts
with cold weights even when the workload itself would fit in L2.
"""

from __future__ import annotations

import statistics
from typing import Any, Callable

import torch

_flush_buf: torch.Tensor | None = None
_POOL = 3
_POOL_LIMIT = 1 << 30


def l2_flush_buffer() -> torch.Tensor:
    global _flush_buf
    if _flush_buf is None:
        size = torch.cuda.get_device_properties(torch.cuda.current_device()).L2_cache_size
        if size <= 0:
            size = 256_000_000
        _flush_buf = torch.empty(size // 4, dtype=torch.int32, device="cuda")
    return _flush_buf


def _clone_tensors(args):
    return tuple(a.clone() if isinstance(a, torch.Tensor) else a for a in args)


def bench_kernel(
    fn: Callable,
    args: tuple[Any, ...] = (),
    n_warmup: int = 10,
    n_repeat: int = 50,
    n_trials: int = 3,
) -> float:
    flush = l2_flush_buffer()

    # rotate over a few copies of the inputs while that stays under 1 GiB
    pool = [tuple(args)]
    if args:
        nbytes = sum(a.nbytes for a in args if isinstance(a, torch.Tensor))
        if nbytes * _POOL <= _POOL_LIMIT:
            pool = [_clone_tensors(args) for _ in range(_POOL)]

    def eager(i: int):
        return fn(*pool[i % len(pool)])

    for i in range(n_warmup):
        flush.zero_()
        eager(i)
    torch.cuda.synchronize()

    graph = None
    try:
        static = _clone_tensors(args)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn(*static)
        torch.cuda.synchronize()
        graph = g
    except Exception as exc:  # capture is best effort, as in the reference
        print(
            f"Warning: CUDA Graph capture failed for {getattr(fn, '__name__', fn)!r} "
            f"({type(exc).__name__}: {exc}); timing eagerly, host dispatch included."
        )

    if graph is not None:
        for _ in range(n_warmup):
            flush.zero_()
            graph.replay()
        torch.cuda.synchronize()

    means = []
    for _ in range(n_trials):
        marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_repeat)]
        for i, (t0, t1) in enumerate(marks):
            flush.zero_()
            t0.record()
            if graph is not None:
                graph.replay()
            else:
                eager(i)
            t1.record()
        torch.cuda.synchronize()
        means.append(sum(t0.elapsed_time(t1) for t0, t1 in marks) / n_repeat)

    del pool
    torch.cuda.empty_cache()
    return statistics.median(means)
