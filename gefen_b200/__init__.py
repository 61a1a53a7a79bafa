"""gefen_b200: the Gefen optimizer-step hot path on B200 (sm_100a).

`Gefen` and `GefenMuon` carry the reference package's public names (reference: __init__.py:1-13) and,
like there, are resolved on first use, so that `import gefen_b200` does no device work and loads no
native code. Two wrappers have no reference counterpart: `Zero1Gefen` / `Zero1GefenMuon` (sharded
state over the GPUs of one machine) and `HostStreamedGefen` (gradients from and parameters to pinned
host memory, copies overlapped).
"""
import importlib

_EXPORTS = {
    "Gefen": "gefen",
    "GefenMuon": "gefen_muon",
    "HostStreamedGefen": "host_stream",
    "Zero1Gefen": "zero1",
    "Zero1GefenMuon": "zero1",
}
__all__ = sorted(_EXPORTS)


def __getattr__(name):
    module = _EXPORTS.get(name)
    if module is None:
        raise AttributeError("module {!r} has no attribute {!r}".format(__name__, name))
    value = getattr(importlib.import_module("." + module, __name__), name)
    globals()[name] = value
    return value
