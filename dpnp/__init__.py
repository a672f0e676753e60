"""Alias so that code written as ``import dpnp as np`` runs on this library:
the module object of ``dpnp_b200`` is installed under the name ``dpnp``."""

import sys

import dpnp_b200

sys.modules[__name__] = dpnp_b200
