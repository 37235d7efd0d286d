"""The host-side watchdog around collectives (no GPU, no NCCL: the communicator is a stand-in)."""

import time

import pytest

from quark_b200.runtime.nccl import NcclError, Watchdog


class _Comm:
    def __init__(self):
        self.aborted = 0

    def abort(self):
        self.aborted += 1


def test_watchdog_leaves_a_region_that_finishes_in_time_alone():
    c = _Comm()
    wd = Watchdog(c, timeout_s=5.0)
    with wd.guard():
        time.sleep(0.01)
    assert c.aborted == 0 and not wd.fired


def test_watchdog_aborts_the_communicator_when_a_frame_overruns():
    """A rank that never joins leaves its peers inside a collective; the timer thread aborts the communicator
    (which is what lets the blocked call return) and the guard reports it."""
    c = _Comm()
    wd = Watchdog(c, timeout_s=0.05)
    t0 = time.monotonic()
    with pytest.raises(NcclError, match="aborted"):
        with wd.guard():
            while c.aborted == 0 and time.monotonic() - t0 < 5.0:  # stands for a host call blocked on the stream
                time.sleep(0.005)
    assert c.aborted == 1 and wd.fired and time.monotonic() - t0 < 2.0


def test_watchdog_does_not_mask_an_error_of_the_guarded_region():
    c = _Comm()
    wd = Watchdog(c, timeout_s=5.0)
    with pytest.raises(ZeroDivisionError):
        with wd.guard():
            1 / 0
    assert c.aborted == 0
    with pytest.raises(ValueError):
        Watchdog(c, timeout_s=0)
