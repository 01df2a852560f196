"""`megagemm`: the reference's package name, served by mgrrmsnorm_b200.

Code written against the reference (`from megagemm import RMSNorm, MegaGemmTriton`) runs unchanged
with this repository on the path; every name resolves lazily to the sm_100a implementation.
"""
import mgrrmsnorm_b200 as _impl

__version__ = _impl.__version__
__all__ = list(_impl.__all__)


def __getattr__(name):
    return getattr(_impl, name)
