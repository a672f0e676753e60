"""SciPy-compatible namespace (only ``special.erf`` lies on the elementwise path)."""
from . import special
