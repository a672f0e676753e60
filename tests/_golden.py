"""Loader of the committed known-answer fixtures (tests/golden)."""

import json
import os

import numpy as np

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_cases():
    with open(os.path.join(_DIR, "known_answers.json")) as fh:
        cases = json.load(fh)
    data = np.load(os.path.join(_DIR, "known_answers.npz"))
    for c in cases:
        c["x"] = data[f"{c.get('x_from', c['name'])}__x"]
        c["expected"] = data[f"{c['name']}__expected"]
        for key in ("y", "cond"):
            k = f"{c['name']}__{key}"
            c[key] = data[k] if k in data.files else None
    return cases


def apply_view(x, steps, xp):
    """Apply the view steps of a case to a NumPy array (xp=np) or a device array."""
    for kind, arg in steps:
        if kind == "flip":
            x = xp.flip(x, axis=arg) if arg is not None else xp.flip(x)
        elif kind == "permute":
            x = xp.transpose(x, arg) if xp is np else x.transpose(*arg)
        elif kind == "slice":
            x = x[tuple(slice(*s) for s in arg)]
        elif kind == "reshape":
            x = x.reshape(arg)
        else:
            raise ValueError(kind)
    return x


def axis_of(params):
    ax = params.get("axis", None)
    return tuple(ax) if isinstance(ax, list) else ax
