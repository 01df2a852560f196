"""`megagemm.rmsnorm` under the reference's module path (megagemm/rmsnorm.py)."""
from mgrrmsnorm_b200.rmsnorm import RMSNorm, RMSNormFunction  # noqa: F401
