"""Helpers shared by the tests: tolerances and seeded inputs. Test code only."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle

TORCH_DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}

# Tolerances (the contract the kernels are held to):
#   fp32   : within 1e-5 relative of the fp64 truth -- elementwise |err| <= 1e-5*|truth| + 1e-6*max|truth|
#            (the second term covers elements that are the difference of two large products);
#   fp16 / bf16: within 1e-2 max-abs of the truth where the output type can express that, and never
#            worse than one rounding of the truth: |err| <= 0.5 ulp_dtype(truth) + the fp32 bound above.
#            (Half an ulp of bf16 at |v| in [4, 8) is 0.0156 > 1e-2, so for such elements the rounding
#            bound is the binding one.)
F32_RTOL = 1e-5
F32_ATOL_SCALE = 1e-6
HALF_MAXABS = 1e-2


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def assert_matches_truth(got: torch.Tensor | np.ndarray, truth: np.ndarray, dtype: str, what: str, slack: float = 1.0):
    g = to_np(got).astype(np.float64) if isinstance(got, torch.Tensor) else np.asarray(got, np.float64)
    truth = np.asarray(truth, np.float64)
    assert g.shape == truth.shape, f"{what}: shape {g.shape} vs {truth.shape}"
    err = np.abs(g - truth)
    scale = float(np.max(np.abs(truth))) if truth.size else 0.0
    bound = slack * (F32_RTOL * np.abs(truth) + F32_ATOL_SCALE * scale)
    if dtype != "f32":
        half_ulp = 0.5 * oracle.ulp_of(truth, dtype)
        bound = bound + half_ulp
        # literal 1e-2 max-abs wherever one rounding of the truth can meet it
        lit = err[half_ulp < HALF_MAXABS / 2]
        assert lit.size == 0 or float(lit.max()) <= HALF_MAXABS, f"{what}: max-abs {float(lit.max())} > 1e-2"
    bad = err > bound
    assert not bad.any(), (f"{what} [{dtype}]: {int(bad.sum())} of {err.size} elements out of tolerance; "
                           f"worst err {float(err.max()):.3e} at truth {float(truth.flat[int(err.argmax())]):.6g}")


def seeded_rmsnorm_inputs(rows: int, cols: int, dtype: str, seed: int = 1234, x_scale: float = 1.0):
    """x ~ N(0, x_scale^2), w = 1 + 0.1 N(0,1), dy ~ N(0,1), drawn on CPU in fp32 in that order from one
    generator, then rounded to `dtype` -- the input recipe of the benchmark configurations."""
    g = torch.Generator().manual_seed(seed)
    x = x_scale * torch.randn(rows, cols, generator=g)
    w = 1.0 + 0.1 * torch.randn(cols, generator=g)
    dy = torch.randn(rows, cols, generator=g)
    td = TORCH_DTYPES[dtype]
    return x.to(td), w.to(td), dy.to(td)
