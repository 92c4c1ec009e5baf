"""B200-native pi0.5 action-chunk engine: one persistent sm_100a kernel behind a C ABI.

``Pi05Arm`` is the drop-in arm for the reference's benchmark harness; ``fixture``
holds the geometry and the seeded synthetic inputs.  The native library is loaded
when an arm is created and its absence is an error (no CPU path exists).
"""

from .fixture import ORDER, SEEDS, Geometry, make_batch, make_inputs, sol  # noqa: F401


def __getattr__(name):
    if name in ("Pi05Arm", "PagedPrefix"):
        from . import arm
        return getattr(arm, name)
    raise AttributeError(name)
