"""Capturing launches into a CUDA graph without outside interference.

While a stream is being captured, CUDA refuses "potentially unsafe" calls made by
the process (``cudaFree``, ``cudaGraphExecDestroy``, a synchronous copy ...) and a
refused call *invalidates the capture*: every later launch fails with
``cudaErrorStreamCaptureInvalidated``.  Such calls need not come from the code
being captured.  Python's cyclic garbage collector runs whenever enough
containers have been allocated, and an object it frees then (an old engine whose
graphs are destroyed, a pinned buffer) makes exactly such a call from inside the
capture, at a moment that depends on what other threads allocated.

:func:`capture` therefore (1) keeps the collector off until the capture has
ended (what it would have freed is freed right after; a full collection before
the capture would cost tens of milliseconds in a process with a large heap, as
much as several steps) and (2) captures in CUDA's ``relaxed`` mode, in which
calls that do not touch the capturing stream are not policed at all.  The
reference captures its decode graphs at start-up only
(tinyvllm/runtime/graphs.py:49-125), where no garbage with device resources
exists yet; this engine also captures steps while it serves.
"""

from __future__ import annotations

import contextlib
import gc

import torch


@contextlib.contextmanager
def capture(graph: "torch.cuda.CUDAGraph", *, pool=None, stream: "torch.cuda.Stream | None" = None):
    """``with capture(graph, pool=..., stream=...):`` records the launches of the body into
    ``graph`` on ``stream`` (torch's own capture stream if None)."""
    if stream is None:
        stream = torch.cuda.Stream()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        # torch.cuda.graph() would also hand every cached block of the allocator back to the driver
        # first; while an engine serves that makes the steps after the capture allocate anew
        torch.cuda.synchronize()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            if pool is None:
                graph.capture_begin(capture_error_mode="relaxed")
            else:
                graph.capture_begin(pool=pool, capture_error_mode="relaxed")
            try:
                yield
            finally:
                graph.capture_end()
        torch.cuda.current_stream().wait_stream(stream)
    finally:
        if was_enabled:
            gc.enable()
