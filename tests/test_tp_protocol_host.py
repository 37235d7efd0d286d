"""The epoch protocol of the fused cross-GPU reduction (``quark_b200/csrc/tp.cu``), modelled on the host.

Every rank is a thread; the arenas are numpy arrays that all threads see, standing for peer-mapped device memory.
Each rank repeats what a rank's stream does per reduction: its GEMM overwrites its partial (y slot ``call & 1``, or
for the pushed schedule the owners' staging blocks), then its kernel announces the epoch to every peer, waits for
every peer's announcement, reads the partials, and (two-shot) writes its share of the result rows into every
rank's x slot ``call & 1``, announces that, and waits for everybody's rows.  Random delays shake the interleaving.
Every value carries the epoch it was written in, so a read that sees anything else has hit a buffer that was
rewritten too early or read too early: the buffer-reuse argument of the kernel (two y slots, two x slots, one staging
area) is what is being checked, for all three schedules, together with freedom from deadlock.
"""

import random
import threading
import time

import numpy as np
import pytest


class Arena:
    def __init__(self, world, rows):
        self.y_ready = np.zeros(world, np.int64)
        self.x_arrived = np.zeros(world, np.int64)
        self.y = np.zeros((2, rows), np.int64)          # two y slots: the epoch each row of this rank's partial belongs to
        self.staging = np.zeros((world, rows // world), np.int64)  # pushed schedule: per source rank, this owner's rows
        self.x = np.zeros((2, rows), np.int64)          # two x slots


def _rank(r, world, rows, calls, schedule, arenas, errors, seed):
    rnd = random.Random(seed)
    mine = arenas[r]
    rpo = rows // world
    nap = lambda: time.sleep(rnd.random() * 0.0004) if rnd.random() < 0.5 else None  # noqa: E731

    def wait(flags, e):
        t0 = time.monotonic()
        while np.any(flags < e):
            if time.monotonic() - t0 > 20.0:
                raise TimeoutError(f"rank {r} waited for epoch {e}: {flags}")
            time.sleep(0)

    try:
        for e in range(1, calls + 1):
            slot = e & 1
            # ---- the rank's GEMM: it may run only after the rank's previous kernel has ended (stream order)
            nap()
            if schedule == "pushed":
                for o in range(world):
                    arenas[o].staging[r, :] = e
            else:
                mine.y[slot, :] = e
            if e > 1:  # the residual of this call is the x of the call before, read from the other slot during the kernel
                prev_x = mine.x[1 - slot].copy() if schedule != "one-shot" else None
            # ---- the kernel
            nap()
            for p in range(world):
                arenas[p].y_ready[r] = e
            wait(mine.y_ready, e)
            nap()
            if schedule == "one-shot":
                seen = np.stack([arenas[p].y[slot] for p in range(world)])
            elif schedule == "two-shot":
                seen = np.stack([arenas[p].y[slot, r * rpo : (r + 1) * rpo] for p in range(world)])
            else:
                seen = mine.staging.copy()
            if np.any(seen != e):
                errors.append(f"rank {r} call {e}: read partial rows of epochs {sorted(set(seen.ravel().tolist()))}")
            if schedule != "one-shot":
                if e > 1 and np.any(prev_x != e - 1):
                    errors.append(f"rank {r} call {e}: residual rows of epochs {sorted(set(prev_x.tolist()))}")
                nap()
                for p in range(world):
                    arenas[p].x[slot, r * rpo : (r + 1) * rpo] = e
                for p in range(world):
                    arenas[p].x_arrived[r] = e
                wait(mine.x_arrived, e)
                if np.any(mine.x[slot] != e):
                    errors.append(f"rank {r} call {e}: result rows of epochs {sorted(set(mine.x[slot].tolist()))}")
    except Exception as exc:  # a deadlock shows up as the timeout above
        errors.append(repr(exc))


@pytest.mark.parametrize("schedule", ["one-shot", "two-shot", "pushed"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_no_buffer_is_rewritten_or_read_too_early(world, schedule):
    rows, calls = 8 * world, 40
    arenas = [Arena(world, rows) for _ in range(world)]
    errors = []
    threads = [threading.Thread(target=_rank, args=(r, world, rows, calls, schedule, arenas, errors, 1000 * world + r)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(60)
    assert not any(t.is_alive() for t in threads), "a rank never finished"
    assert not errors, errors[:5]


def test_one_y_slot_would_not_be_enough_for_the_one_shot_schedule():
    """The model is sharp enough to see the hazard the second y slot removes: with a single slot a fast rank's next GEMM
    can overwrite the partial that a slow peer has not read yet."""
    world, rows = 2, 16
    arenas = [Arena(world, rows) for _ in range(world)]
    a0, a1 = arenas
    # rank 0: call 1 complete (it read both partials), then its GEMM of call 2 writes the same slot; rank 1 is still reading call 1
    a0.y[0, :] = 1
    a1.y[0, :] = 1
    a0.y[0, :] = 2  # single slot reused
    assert np.any(np.stack([a0.y[0], a1.y[0]]) != 1)  # rank 1's late read of call 1 would see epoch 2
