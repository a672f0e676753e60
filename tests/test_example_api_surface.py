"""Every name the reference's example program takes from the `dpnp` namespace exists in this
library under the same name.  Runs on the CPU where a checkout of the reference is present (the
example is read as text, nothing of it is executed); tests/test_gpu_dropin.py executes the file
itself where there is both a checkout and a GPU."""

import ast
import os

import pytest

REFERENCE_ROOT = os.environ.get("DPNP_REFERENCE_ROOT") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")


def test_names_used_by_example_bs_exist():
    path = os.path.join(REFERENCE_ROOT, "examples", "example_bs.py")
    if not os.path.exists(path):
        pytest.skip("no checkout of the reference on this machine")
    import dpnp              # the alias package of this repository
    import dpnp_b200

    assert dpnp is dpnp_b200
    tree = ast.parse(open(path).read())
    alias = None
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                if a.name == "dpnp":
                    alias = a.asname or "dpnp"
    assert alias is not None

    def dotted(node):
        parts = []
        while isinstance(node, ast.Attribute):
            parts.append(node.attr)
            node = node.value
        if isinstance(node, ast.Name) and node.id == alias:
            return list(reversed(parts))
        return None

    used = set()
    for node in ast.walk(tree):
        if isinstance(node, ast.Attribute):
            d = dotted(node)
            if d:
                used.add(tuple(d))
    assert ("log",) in used and ("random", "uniform") in used
    for chain in sorted(used):
        obj = dpnp
        for name in chain:
            assert hasattr(obj, name), f"dpnp.{'.'.join(chain)} is missing"
            obj = getattr(obj, name)
