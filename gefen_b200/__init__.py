"""gefen_b200: the Gefen optimizer-step hot path on B200 (sm_100a).

Same public names as the reference package (reference: __init__.py:1-13): `Gefen`, `GefenMuon`,
imported lazily so that `import gefen_b200` does no device work and loads no native code.
"""
__all__ = ["Gefen", "GefenMuon"]


def __getattr__(name):
    if name == "Gefen":
        from .gefen import Gefen

        return Gefen
    if name == "GefenMuon":
        from .gefen_muon import GefenMuon

        return GefenMuon
    raise AttributeError("module {!r} has no attribute {!r}".format(__name__, name))
