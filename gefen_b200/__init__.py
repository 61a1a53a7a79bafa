"""gefen_b200: the Gefen optimizer-step hot path on B200 (sm_100a).

Same public names as the reference package (reference: __init__.py:1-13): `Gefen`, `GefenMuon`,
imported lazily so that `import gefen_b200` does no device work and loads no native code. Two
wrappers without a reference counterpart: `Zero1Gefen` (sharded state over the GPUs of one machine)
and `HostStreamedGefen` (gradients from and parameters to pinned host memory, copies overlapped).
"""
__all__ = ["Gefen", "GefenMuon", "HostStreamedGefen", "Zero1Gefen"]


def __getattr__(name):
    if name == "Gefen":
        from .gefen import Gefen

        return Gefen
    if name == "GefenMuon":
        from .gefen_muon import GefenMuon

        return GefenMuon
    if name == "HostStreamedGefen":
        from .host_stream import HostStreamedGefen

        return HostStreamedGefen
    if name == "Zero1Gefen":
        from .zero1 import Zero1Gefen

        return Zero1Gefen
    raise AttributeError("module {!r} has no attribute {!r}".format(__name__, name))
