"""sps_b200.install() against the reference's own modules: every name it is meant to rebind exists
there and takes the same arguments.  The reference is looked for under REFERENCE_ROOT (its
checkout; the package lies in src/) or in baseline/_ref (a pip --target install of it); the test
is skipped when neither is there."""

import importlib
import inspect
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_path():
    env = os.environ.get("REFERENCE_ROOT")
    cands = [os.path.join(env, "src")] if env else []
    cands += [os.path.join(ROOT, "baseline", "_ref")]
    for c in cands:
        if os.path.isdir(os.path.join(c, "modeling", "models")):
            return c
    return None


def test_install_rebinds_every_name_with_the_reference_signature(monkeypatch):
    path = _reference_path()
    if path is None:
        pytest.skip("the reference's modeling package is not on this machine")
    monkeypatch.syspath_prepend(path)
    monkeypatch.setattr(sys, "dont_write_bytecode", True)
    try:
        importlib.import_module("modeling.models.sps.core")
    except Exception as e:            # e.g. triton missing
        pytest.skip(f"the reference does not import here: {e!r}")
    inst = importlib.import_module("sps_b200.install")
    originals = {}
    for mod_name, attr, _fn in inst._BINDINGS:
        mod = importlib.import_module(mod_name)
        originals[(mod_name, attr)] = getattr(mod, attr)
    try:
        done = inst.install(strict=True)
        assert len(done) == len(inst._BINDINGS) == 8
        for mod_name, attr, fn in inst._BINDINGS:
            mod = importlib.import_module(mod_name)
            assert getattr(mod, attr) is fn
            ref_sig = inspect.signature(originals[(mod_name, attr)])
            our_sig = inspect.signature(fn)
            assert list(ref_sig.parameters) == list(our_sig.parameters), (attr, ref_sig, our_sig)
            for name, p in ref_sig.parameters.items():
                q = our_sig.parameters[name]
                assert p.kind == q.kind and p.default == q.default, (attr, name)
    finally:
        for (mod_name, attr), orig in originals.items():
            setattr(importlib.import_module(mod_name), attr, orig)
