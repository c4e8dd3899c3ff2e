"""Op library: hand-written sm_100a kernels with plain-PyTorch CPU definitions."""
from . import functional, reference  # noqa: F401
