"""`megagemm.swiglu` under the reference's module path (megagemm/swiglu.py)."""
from mgrrmsnorm_b200.swiglu import MegaGemmFunction, MegaGemmTriton  # noqa: F401
