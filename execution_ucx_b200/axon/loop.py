"""An asyncio event loop that spins briefly before it sleeps (not in the reference).

The runtime's context threads hand every completion to the event loop through an eventfd. A loop that is
asleep in ``epoll_wait`` when the completion arrives pays a kernel wake-up, on both sides of a call.
``SpinningSelector`` watches, without the GIL, the one word in which the native layer counts the
completions it has queued, for up to ``spin_us`` microseconds, and only then sleeps in the selector as
usual::

    axon.run(main())                                  # asyncio.run with the spinning loop
    asyncio.run(main(), loop_factory=axon.new_event_loop)

While it spins the loop does not look at its other file descriptors, so unrelated I/O of the same loop
sees up to ``spin_us`` more latency, and a loop that wakes often with nothing to do keeps a core busy for
that long each time. ``spin_us=0`` (or ``EUX_PY_SPIN_US=0``) gives the plain selector loop.

Opt-in, and worth it only where wake-ups are slow: on a virtual machine with 8 cores a 4 KiB host echo went
from 185 to 165 us per round trip; on the bare-metal hosts of the B200s it made no difference (131.7
against 132.9 us for a 4 KiB device echo between two GPUs), so nothing in this package turns it on.
"""
from __future__ import annotations

import asyncio
import os
import selectors
from typing import Optional

from . import _axon

DEFAULT_SPIN_US = 150.0


def _spin_seconds(spin_us: Optional[float]) -> float:
    if spin_us is None:
        env = os.environ.get("EUX_PY_SPIN_US")
        spin_us = float(env) if env not in (None, "") else DEFAULT_SPIN_US
    if spin_us < 0:
        raise ValueError("spin_us must not be negative")
    return spin_us * 1e-6


class SpinningSelector(selectors.DefaultSelector):
    """The platform's selector; a ``select`` that would sleep first spins for the native layer's next completion."""

    def __init__(self, spin_us: Optional[float] = None):
        super().__init__()
        self._spin = _spin_seconds(spin_us)

    def select(self, timeout=None):
        spin = self._spin
        if spin and (timeout is None or timeout > 0):
            budget = spin if timeout is None else min(spin, timeout)
            if _axon._spin_for_wake(budget):
                return super().select(0)
            if timeout is not None:
                timeout = max(0.0, timeout - budget)
        return super().select(timeout)


def new_event_loop(spin_us: Optional[float] = None) -> asyncio.AbstractEventLoop:
    """A selector event loop on a ``SpinningSelector`` (``spin_us``: default ``EUX_PY_SPIN_US``, else 150)."""
    return asyncio.SelectorEventLoop(SpinningSelector(spin_us))


def run(main, *, spin_us: Optional[float] = None, debug: Optional[bool] = None):
    """``asyncio.run(main)`` on the spinning loop."""
    return asyncio.run(main, debug=debug, loop_factory=lambda: new_event_loop(spin_us))
