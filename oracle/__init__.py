"""CPU oracle for the Waypoint-1.5 DiT per-NFE hot path.

TEST INFRASTRUCTURE ONLY.  This package is a numpy restatement of the reference's
per-kernel CPU references (``src/quark/kernels/*/reference.py``, ``src/quark/runtime/npconv.py``
and the host-side conditioning math in ``src/quark/models/_waypoint_15_io.py``).  It is the
checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``.  Nothing in ``quark_b200/`` imports it: the product
path runs only the CUDA library and fails loudly when that library is missing.

Parity pin: every function here is checked against the reference's own Python oracles,
imported from the reference tree, on seeded inputs (``tests/golden/make_golden.py`` generates
the committed fixtures in ``tests/golden/*.npz``; ``tests/test_oracle_golden.py`` replays them).
The reference ships no golden vectors of its own for this path.
"""

from . import codec, ops, model  # noqa: F401
