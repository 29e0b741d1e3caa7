"""NumPy stand-in for the part of `flax` the reference's model files use (test infrastructure)."""
from . import linen  # noqa: F401
