"""CUDA-event timing of kernel launches, by CUDA-graph replay where capture succeeds.

Mirrors the reference's protocol (python/cleave/runtime/timer.py:14-108): ``batch`` back-to-back
launches are captured once on a side stream and the graph is replayed, which keeps Python
dispatch out of the timed region; if capture fails a plain launch loop is timed instead and a
warning is issued.
"""

from __future__ import annotations

import warnings


def capture_launch_graph(kernel, args, batch: int):
    """A CUDA graph of ``batch`` back-to-back ``kernel(*args)`` launches, or None."""
    import torch

    try:
        graph = torch.cuda.CUDAGraph()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            kernel(*args)  # lazy set-up (workspace, function attributes) happens outside capture
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        with torch.cuda.graph(graph):
            for _ in range(batch):
                kernel(*args)
    except Exception:  # noqa: BLE001 - capture is an optimisation, not a requirement
        return None
    return graph


def time_rounds(body, repeats: int = 1) -> list:
    """CUDA-event milliseconds of ``body()`` for each of ``repeats`` rounds."""
    import torch

    rounds = []
    for _ in range(repeats):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        body()
        stop.record()
        torch.cuda.synchronize()
        rounds.append(start.elapsed_time(stop))
    return rounds


def replay_rounds(graph, replays: int, *, repeats: int = 1, warmup: int = 1) -> list:
    import torch

    for _ in range(warmup):
        graph.replay()
    torch.cuda.synchronize()

    def body():
        for _ in range(replays):
            graph.replay()

    return time_rounds(body, repeats)


def launch_rounds(kernel, args, launches: int, *, repeats: int = 1) -> list:
    def body():
        for _ in range(launches):
            kernel(*args)

    return time_rounds(body, repeats)


def mean_launch_ms(kernel, args, *, warmup: int = 0, iters: int = 1, batch: int = 100) -> float:
    """Mean ms per launch over at least ``iters`` launches, replayed in graphs of ``batch``."""
    if warmup < 0:
        raise ValueError(f"warmup_iters must be >= 0, got {warmup}")
    if iters <= 0:
        raise ValueError(f"profile_iters must be > 0, got {iters}")
    import torch

    args = list(args)
    for _ in range(warmup):
        kernel(*args)
    torch.cuda.synchronize()
    batch = min(iters, batch)
    graph = capture_launch_graph(kernel, args, batch)
    if graph is not None:
        replays = -(-iters // batch)
        (elapsed,) = replay_rounds(graph, replays)
        return elapsed / (replays * batch)
    warnings.warn("CUDA graph capture failed for this kernel; timing a plain launch loop, "
                  "which includes per-call Python dispatch overhead", RuntimeWarning, stacklevel=2)
    (elapsed,) = launch_rounds(kernel, args, iters)
    return elapsed / iters


def min_launch_us(kernel, args, *, batch: int = 20, repeats: int = 5, warmup: int = 3) -> float:
    """Minimum over ``repeats`` rounds of the mean microseconds per launch of a ``batch``-launch
    graph (the autotuner's reading, python/cleave/runtime/autotune.py:101-139)."""
    import torch

    args = list(args)
    for _ in range(warmup):
        kernel(*args)
    torch.cuda.synchronize()
    graph = capture_launch_graph(kernel, args, batch)
    if graph is None:
        return min(launch_rounds(kernel, args, batch, repeats=repeats)) / batch * 1e3
    return min(replay_rounds(graph, 1, repeats=repeats)) / batch * 1e3
