"""fitre_b200: B200-native CUDA implementation of FITRE's CNN gradient / Hessian-vector /
KFAC-factor path behind the reference's operator interface.  See include/fitre_b200.h for
the C ABI and fitre_b200.api for the host-side mirror of the reference's functions."""
from . import _structs as structs  # noqa: F401
from . import layout  # noqa: F401

__all__ = ["structs", "layout"]
