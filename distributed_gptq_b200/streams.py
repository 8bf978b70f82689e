"""Side streams for independent per-layer chains.

The damped inverse and the block quantization of one layer are long chains of short,
dependent kernels that leave most of the GPU idle.  Layers are independent once their
Hessians are complete, so their chains are put on a few high-priority side streams, where
they run beside each other and beside whatever the caller's stream goes on to do (a
host-to-device copy, a collective, another layer's ``add_batch`` while that one waits for
its data).  Enqueueing a chain costs the host milliseconds (hundreds of launches); with
``threads=True`` every side stream gets its own host thread for that (the library calls
and torch's launches release the interpreter lock).  On the layer sweep of ``bench.py`` the
device, not the host, bounds the chains, and the threads bought nothing, so they are off
by default.

The streams (and threads) are meant to be made once and reused: torch's caching allocator
keeps its pool of freed blocks per stream, and a fresh stream starts with an empty pool.
"""
from __future__ import annotations

from concurrent.futures import Future, ThreadPoolExecutor
from typing import Any, Callable, Iterable, List, Optional

import torch


class ChainPool:
    """A round-robin pool of high-priority CUDA streams.

    ``submit(fn)`` arranges for ``fn()`` to run with the next side stream current, ordered
    after everything queued so far on the caller's current stream, and returns a future of
    ``fn``'s result (available once the chain is *enqueued*, not once the device has run it).
    ``join()`` waits for all enqueueing to end and makes the caller's current stream wait for
    every chain submitted so far.  ``fn`` must not synchronise with the host if the chains are
    to overlap; ``GPTQ.quantize_launch`` / ``GPTQ.quantize_finish`` are split for that.
    """

    def __init__(self, device: torch.device, n_streams: int = 4, threads: bool = False):
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("ChainPool needs a CUDA device")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        n = max(1, n_streams)
        self.streams = [torch.cuda.Stream(device=self.device, priority=-1) for _ in range(n)]
        self._workers = ([ThreadPoolExecutor(max_workers=1, thread_name_prefix=f"dgq-chain{i}")
                          for i in range(n)] if threads else None)
        self._next = 0
        self._jobs: List[Future] = []

    def submit(self, fn: Callable[[], Any], uses: Iterable[torch.Tensor] = (),
               after: Optional[torch.cuda.Event] = None) -> Future:
        i = self._next % len(self.streams)
        self._next += 1
        side = self.streams[i]
        if after is None:
            after = torch.cuda.Event()
            after.record(torch.cuda.current_stream(self.device))
        for t in uses:
            if t is not None and t.is_cuda:
                t.record_stream(side)

        def run():
            torch.cuda.set_device(self.device)
            side.wait_event(after)
            with torch.cuda.stream(side):
                out = fn()
            done = torch.cuda.Event()
            done.record(side)
            return out, done

        if self._workers is None:
            fut: Future = Future()
            try:
                fut.set_result(run())
            except BaseException as e:      # delivered by result(), like the threaded form
                fut.set_exception(e)
        else:
            fut = self._workers[i].submit(run)
        self._jobs.append(fut)
        out_fut: Future = Future()

        def deliver(f):
            if f.exception() is not None:
                out_fut.set_exception(f.exception())
            else:
                out_fut.done_event = f.result()[1]     # recorded on the side stream after fn
                out_fut.set_result(f.result()[0])

        fut.add_done_callback(deliver)
        return out_fut

    def stream_wait(self, stream: torch.cuda.Stream, futures: Iterable[Future]) -> None:
        """Makes ``stream`` wait for the chains behind ``futures`` (as returned by
        :meth:`submit`); blocks the host only until those chains are enqueued."""
        for f in futures:
            f.result()
            stream.wait_event(f.done_event)

    def join(self) -> None:
        cur = torch.cuda.current_stream(self.device)
        jobs, self._jobs = self._jobs, []
        first_error = None
        for fut in jobs:
            try:
                _, done = fut.result()
                cur.wait_event(done)
            except BaseException as e:
                first_error = first_error or e
        if first_error is not None:
            raise first_error

    def shutdown(self) -> None:
        self.join()
        if self._workers is not None:
            for w in self._workers:
                w.shutdown(wait=True)
            self._workers = None
