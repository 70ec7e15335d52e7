"""Device timing of kernel launches.

Protocol (the one the reference times candidates with, python/cleave/runtime/timer.py:76-108 and
python/cleave/runtime/autotune.py:36-43): a batch of back-to-back launches is captured once into a CUDA
graph, the graph is replayed, and CUDA events on the replay stream bracket the replays, so neither Python
dispatch nor the C-ABI call overhead is inside the timed region. ``mean_launch_ms`` is the candidate
benchmark (mean over at least ``iters`` launches), ``min_launch_us`` the autotuner's reading (best of a few
rounds). When a launch cannot be captured the same number of plain launches is timed instead, with a warning.
"""

from __future__ import annotations

import warnings


class LaunchTimer:
    """Times ``launch()`` (a zero-argument callable that enqueues one kernel on the current stream)."""

    def __init__(self, launch, batch: int):
        if batch <= 0:
            raise ValueError(f"batch must be positive, got {batch}")
        self.launch, self.batch = launch, int(batch)
        self.graph = None

    def warm(self, n: int) -> None:
        import torch

        for _ in range(n):
            self.launch()
        torch.cuda.synchronize()

    def capture(self) -> bool:
        """Capture ``batch`` launches into a graph; False (and no graph) when capture is refused."""
        import torch

        side = torch.cuda.Stream()
        try:
            # one launch on the capture stream first: whatever a first call sets up lazily (a workspace,
            # function attributes) must not happen while the stream is capturing
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.launch()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(self.batch):
                    self.launch()
        except Exception:  # noqa: BLE001 - timing falls back to plain launches
            self.graph = None
            return False
        self.graph = graph
        return True

    def _enqueue(self, times: int) -> None:
        if self.graph is not None:
            for _ in range(times):
                self.graph.replay()
        else:
            for _ in range(times * self.batch):
                self.launch()

    def rounds_ms(self, rounds: int, batches_per_round: int = 1) -> list:
        """Elapsed milliseconds of each round of ``batches_per_round * batch`` launches."""
        import torch

        out = []
        for _ in range(rounds):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            self._enqueue(batches_per_round)
            t1.record()
            t1.synchronize()
            out.append(t0.elapsed_time(t1))
        return out


def _timer_for(kernel, args, batch: int, warmup: int) -> LaunchTimer:
    bound = tuple(args)
    timer = LaunchTimer(lambda: kernel(*bound), batch)
    timer.warm(warmup)
    if not timer.capture():
        warnings.warn("CUDA graph capture failed for this kernel; timing a plain launch loop, "
                      "which includes per-call Python dispatch overhead", RuntimeWarning, stacklevel=3)
    return timer


def mean_launch_ms(kernel, args, *, warmup: int = 0, iters: int = 1, batch: int = 100) -> float:
    """Mean milliseconds per launch over at least ``iters`` launches, in graphs of ``batch``."""
    if warmup < 0:
        raise ValueError(f"warmup_iters must be >= 0, got {warmup}")
    if iters <= 0:
        raise ValueError(f"profile_iters must be > 0, got {iters}")
    per_graph = min(int(iters), int(batch))
    timer = _timer_for(kernel, args, per_graph, warmup)
    n_graphs = (iters + per_graph - 1) // per_graph
    if timer.graph is not None:
        timer.rounds_ms(1)  # first replay: the graph is instantiated and uploaded outside the reading
    (ms,) = timer.rounds_ms(1, n_graphs)
    return ms / (n_graphs * per_graph)


def min_launch_us(kernel, args, *, batch: int = 20, repeats: int = 5, warmup: int = 3) -> float:
    """Best of ``repeats`` rounds of the mean microseconds per launch of one ``batch``-launch graph."""
    timer = _timer_for(kernel, args, batch, warmup)
    if timer.graph is not None:
        timer.rounds_ms(1)
    return min(timer.rounds_ms(repeats)) * 1e3 / batch
