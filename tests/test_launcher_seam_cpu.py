"""The hand-written typed launchers of btb_b200.launcher against the reference's GENERATED ones
(btb/engine/card_launch.py, written by the reference's `build.py bindings` from its kernels' signatures): driven with the
same arguments into a recording launcher, both must make the same `launch(name, grid, block, args, stream, shared)` call -
the kernel's name, and one ctypes value of the same type and payload per kernel parameter, in the kernel's order.

Runs where a reference checkout is at hand (BTB_REFERENCE, or a `reference` folder beside this repository); the GPU box
has none and skips it."""

import importlib.util
import inspect
import os
import sys

import pytest

from btb_b200 import launcher as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _checkout():
    for c in (os.environ.get("BTB_REFERENCE"), os.path.join(os.path.dirname(ROOT), "reference")):
        if c and os.path.exists(os.path.join(c, "btb", "engine", "card_launch.py")):
            return c
    return None


class Recorder:
    def __init__(self):
        self.calls = []

    def launch(self, name, grid, block, args, stream=None, shared=0):
        self.calls.append((name, tuple(grid), tuple(block), [(type(a).__name__, a.value) for a in args], stream, shared))


def _reference_module(ref):
    """card_launch.py by file path: it needs torch and the reference's btb.kinds (plain NewTypes), nothing of the engine"""
    kinds = importlib.util.spec_from_file_location("btb.kinds", os.path.join(ref, "btb", "kinds.py"))
    pkg = type(sys)("btb")
    pkg.__path__ = []  # a bare namespace: nothing else of the reference is imported
    saved = {k: sys.modules.get(k) for k in ("btb", "btb.kinds")}
    try:
        sys.modules["btb"] = pkg
        km = importlib.util.module_from_spec(kinds)
        sys.modules["btb.kinds"] = km
        kinds.loader.exec_module(km)
        spec = importlib.util.spec_from_file_location("_ref_card_launch", os.path.join(ref, "btb", "engine", "card_launch.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v


def test_typed_launchers_make_the_generated_launchers_calls():
    ref = _checkout()
    if ref is None:
        pytest.skip("no reference checkout at hand")
    theirs = _reference_module(ref)
    mine = {n: f for n, f in vars(L).items() if n.startswith("btb_") and inspect.isfunction(f)}
    assert len(mine) >= 18
    for name, f in sorted(mine.items()):
        g = getattr(theirs, name, None)
        assert g is not None, f"{name}: the reference generates no such launcher"
        pa = [p for p in inspect.signature(f).parameters.values() if p.kind == p.POSITIONAL_OR_KEYWORD][1:]
        pb = [p for p in inspect.signature(g).parameters.values() if p.kind == p.POSITIONAL_OR_KEYWORD][1:]
        assert len(pa) == len(pb), name
        assert [p.name.rstrip("_") for p in pa] == [p.name.rstrip("_") for p in pb], name  # the same parameters, in order
        vals = []
        for i, p in enumerate(pb):
            if p.name in ("grid", "block"):
                vals.append((3 + i, 2, 1))
            elif p.name in ("eps", "scale"):
                vals.append(0.25 + i)
            elif p.name in ("D", "M"):
                vals.append(8)
            else:
                vals.append(1000 + 16 * i)
        ra, rb = Recorder(), Recorder()
        f(ra, *vals, stream="s", shared=48)
        g(rb, *vals, stream="s", shared=48)
        assert ra.calls == rb.calls, name
        assert L.B200Launcher.__dict__  # the class is importable without a device
    served = [rx for rx, _h in L.B200Launcher.FAMILIES]
    assert len(served) >= 18
