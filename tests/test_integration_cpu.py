"""The reference-side binding builds from a checkout of the reference (skipped where there is none):
the five edits of tests/integration/make_binding.py still find their places in the reference's host
file, the result compiles against torch and libcs2d.so, and the module keeps the reference's
``fwd`` / ``bwd`` signatures."""
import importlib.util
import os
import sys

import pytest

from conftest import ROOT


def _reference():
    for cand in (os.environ.get("CS2D_REFERENCE", ""), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "kernels", "selective_nd_scan", "src", "cusoflex",
                                                "selective_scan_oflex.cpp")):
            return cand
    return None


@pytest.mark.skipif(_reference() is None, reason="no checkout of the reference project")
def test_binding_builds_and_keeps_the_reference_signatures():
    import torch  # noqa: F401  (the module links against torch's libraries)
    sys.path.insert(0, os.path.join(ROOT, "tests", "integration"))
    import make_binding
    so = make_binding.build(_reference())
    spec = importlib.util.spec_from_file_location("selective_nd_scan_cuda_oflex", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    assert mod.fwd.__doc__.count("arg") == 10 and mod.bwd.__doc__.count("arg") == 13
    assert "list[torch.Tensor]" in mod.fwd.__doc__ and "list[torch.Tensor]" in mod.bwd.__doc__
    assert not os.path.exists(os.path.join(ROOT, "tests", "integration", "_build", "selective_scan_oflex_on_cs2d.cpp"))
