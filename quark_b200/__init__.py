"""B200-native Waypoint-1.5 DiT hot path behind the reference's ``quark`` call surface.

``quark_b200.functional`` (``qf``) mirrors ``quark.functional``; ``QuarkTensor`` mirrors the
reference tensor; ``Engine`` mirrors ``quark.Engine`` (``append_frame`` / ``gen_frame``).  All
compute runs in ``libquark_b200.so`` (hand-written sm_100a CUDA) through ctypes.
"""

from . import _lib, runtime  # noqa: F401
from . import functional  # noqa: F401
from . import functional as qf  # noqa: F401
from .runtime.tensor import QuarkTensor  # noqa: F401

__all__ = ["QuarkTensor", "qf", "functional", "runtime", "Engine", "CtrlInput", "Waypoint15", "Waypoint15Config", "QuantConfig"]


def __getattr__(name):
    if name in ("Engine", "CtrlInput"):
        from . import engine

        return getattr(engine, name)
    if name in ("Waypoint15", "Waypoint15Config", "QuantConfig", "GenerateFrame"):
        from .models import waypoint_15 as m

        return getattr(m, name)
    raise AttributeError(name)
