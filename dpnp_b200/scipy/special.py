"""``dpnp.scipy.special``: the error function (dpnp/scipy/special/_erf.py:125-132)."""
from .._ufuncs import erf

__all__ = ["erf"]
