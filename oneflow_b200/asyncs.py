"""``flow.asyncs``: run a block of ops asynchronously to the main line of work
(reference: python/oneflow/asyncs/thread.py:18-52).  The reference gives the block its own virtual-machine worker
thread; on one GPU the unit of asynchrony is the CUDA stream, so a :class:`Thread` owns a side stream and
``with flow.asyncs.thread(t):`` launches everything inside on it.  The side stream first waits for what the current
stream has queued (inputs are ready), and :meth:`Thread.join` makes the current stream wait for the side work."""
import torch


class Thread:
    def __init__(self, device=None):
        self.stream = torch.cuda.Stream(device) if torch.cuda.is_available() else None

    def join(self):
        """Order the current stream after everything launched on this worker so far."""
        if self.stream is not None:
            torch.cuda.current_stream().wait_stream(self.stream)

    def synchronize(self):
        if self.stream is not None:
            self.stream.synchronize()


class thread:
    """Context manager (and decorator) that launches the enclosed ops on ``worker_thread``'s stream."""

    def __init__(self, worker_thread: Thread):
        self.worker_thread_ = worker_thread
        self._ctx = None

    def __enter__(self):
        s = self.worker_thread_.stream
        if s is not None:
            s.wait_stream(torch.cuda.current_stream())
            self._ctx = torch.cuda.stream(s)
            self._ctx.__enter__()
        return self.worker_thread_

    def __exit__(self, *exc):
        if self._ctx is not None:
            self._ctx.__exit__(*exc)
            self._ctx = None
        return False

    def __call__(self, fn):
        import functools

        @functools.wraps(fn)
        def wrapped(*a, **k):
            with thread(self.worker_thread_):
                return fn(*a, **k)
        return wrapped
