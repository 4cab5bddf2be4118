"""numpy under the name ``jax.numpy`` (see the package docstring)."""
from numpy import *  # noqa: F401,F403
from numpy import ndarray, float32, asarray  # noqa: F401
