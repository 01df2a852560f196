"""Top-level `rmsnorm_cuda_ops`, the module name the reference's scripts import
(megagemm/rmsnorm.py:12, test_rmsnorm.py:2); it re-exports the C-ABI-backed implementation."""
from mgrrmsnorm_b200.rmsnorm_cuda_ops import *  # noqa: F401,F403
from mgrrmsnorm_b200.rmsnorm_cuda_ops import rmsnorm_backward, rmsnorm_forward  # noqa: F401
