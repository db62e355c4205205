"""Two pieces of work on one rank taking turns at their communication points.

DualPipeV runs the forward of one micro-batch and the backward of another in the same slot so that the expert-parallel
all-to-all of one hides behind the compute of the other (torchtitan/distributed/dual_pipe_v.py:33-330: two threads and
hooks around the MoE dispatch / combine that pass control back and forth). The same idea here, without hooks on
modules: the two pieces run in two Python threads that share the compute stream and hold a baton; a collective that can
run in the background (``parallel/ep.py``'s all-to-all) is launched asynchronously, the thread hands the baton over
(:func:`yield_point`) and waits for the collective only when it gets the baton back. Exactly one thread issues work
at any time, so kernels reach the compute stream in a deterministic order and nothing races on module state; what
overlaps is the collective (on the communication library's own stream) with the other thread's kernels.
"""

from __future__ import annotations

import threading

import torch

__all__ = ["active", "yield_point", "run_overlapped"]

_tls = threading.local()


class _Baton:
    def __init__(self):
        self._cv = threading.Condition()
        self._turn = 0
        self._done = [False, False]

    def wait_turn(self, me: int) -> None:
        with self._cv:
            while self._turn != me and not self._done[1 - me]:
                self._cv.wait()

    def switch(self, me: int) -> None:
        with self._cv:
            if self._done[1 - me]:
                return
            self._turn = 1 - me
            self._cv.notify_all()
            while self._turn != me and not self._done[1 - me]:
                self._cv.wait()

    def finish(self, me: int) -> None:
        with self._cv:
            self._done[me] = True
            self._turn = 1 - me
            self._cv.notify_all()


def active() -> bool:
    """True inside :func:`run_overlapped`: collectives may then be issued asynchronously around a yield point."""
    return getattr(_tls, "baton", None) is not None


def yield_point() -> None:
    """Let the other piece of work run until its next yield point (no-op outside :func:`run_overlapped`)."""
    b = getattr(_tls, "baton", None)
    if b is not None:
        b[0].switch(b[1])


def run_overlapped(first, second):
    """Run ``first()`` (in this thread) and ``second()`` (in a helper thread) taking turns at yield points; returns both
    results. ``first`` starts. An exception in either is raised here after both have stopped."""
    baton = _Baton()
    out = [None, None]
    err: list = [None, None]
    stream = torch.cuda.current_stream() if torch.cuda.is_available() else None
    grad_mode = torch.is_grad_enabled()

    def side(i, fn):
        _tls.baton = (baton, i)
        try:
            baton.wait_turn(i)
            out[i] = fn()
        except BaseException as e:  # noqa: BLE001  (re-raised by the caller's thread)
            err[i] = e
        finally:
            _tls.baton = None
            baton.finish(i)

    def helper():
        if stream is not None:
            torch.cuda.set_device(stream.device)
            torch.cuda.set_stream(stream)          # the helper thread issues on the same compute stream
        torch.set_grad_enabled(grad_mode)
        side(1, second)

    t = threading.Thread(target=helper, name="pp-overlap", daemon=True)
    t.start()
    side(0, first)
    t.join()
    for e in err:
        if e is not None:
            raise e
    return out[0], out[1]
