"""Generates the golden vectors under tests/golden/ by running the REFERENCE's own code on CPU.

Needs the reference tree (its location comes from MGR_REFERENCE_DIR; see REF below for the default) and
oracle/_ref/libmgr_ref.so (make -C oracle ref). The committed .npz files are its output; the tests
only read them, so they run where the reference tree does not exist.

What runs from the reference, unmodified:
  * rmsnorm_cpu (rmsnorm_standalone.cu:17-30) through oracle/_ref           -> rmsnorm forward, fp32
  * the Triton kernels _mg_swiglu_fwd_kernel / _mg_swiglu_bwd_kernel (megagemm/swiglu.py:18-79)
    through MegaGemmFunction, executed by the Triton interpreter (TRITON_INTERPRET=1) -> activation
  * MegaGemmTriton (megagemm/swiglu.py:138-172) and PyTorchSwiGLU (benchmark_swiglu.py:40-58) with the
    weight mapping of benchmark_swiglu.py:85-89                               -> whole MLP, fwd + bwd
The reference has no CPU code for the RMSNorm backward; the vectors for it come from the formula its
own test differentiates (test_rmsnorm.py:55-60), evaluated by torch autograd in fp64.

Run:  python tests/golden/make_golden.py
"""
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REF = Path(os.environ.get("MGR_REFERENCE_DIR") or ROOT.parent / "reference")   # default: `reference` beside this repository
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(REF))

import numpy as np
import torch

from oracle import oracle


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def f16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16).to(torch.float32)


def rmsnorm_cases():
    ref = oracle.ref_lib()
    assert ref is not None, "build oracle/_ref first: make -C oracle ref"
    g = torch.Generator().manual_seed(1234)
    out = {}
    for name, rows, cols, eps, rnd in [
        ("f32_a", 10, 256, 1e-5, None),        # eps of RMSNorm's default (megagemm/rmsnorm.py:68)
        ("f32_b", 5, 1000, 1e-6, None),        # ragged row count, cols % 16 != 0
        ("f16", 6, 512, 1e-6, f16_round),
        ("bf16", 6, 512, 1e-6, bf16_round),
    ]:
        x = torch.randn(rows, cols, generator=g)
        w = 1.0 + 0.1 * torch.randn(cols, generator=g)
        dy = torch.randn(rows, cols, generator=g)
        if rnd is not None:
            x, w, dy = rnd(x), rnd(w), rnd(dy)
        # the reference's CPU forward (fp32, its own evaluation order)
        y_ref_cpu = ref.cpu_forward(x.numpy(), w.numpy(), eps)
        # the formula its test differentiates, in fp64 (test_rmsnorm.py:55-60)
        x64 = x.double().requires_grad_(True)
        w64 = w.double().requires_grad_(True)
        y64 = x64 * torch.rsqrt(x64.pow(2).mean(-1, keepdim=True) + float(np.float32(eps))) * w64
        y64.backward(dy.double())
        out.update({
            f"{name}_x": x.numpy(), f"{name}_w": w.numpy(), f"{name}_dy": dy.numpy(),
            f"{name}_eps": np.float32(eps),
            f"{name}_y_refcpu": y_ref_cpu,
            f"{name}_y": y64.detach().numpy(), f"{name}_dx": x64.grad.numpy(), f"{name}_dw": w64.grad.numpy(),
        })
    np.savez_compressed(HERE / "rmsnorm.npz", **out)


def swiglu_cases():
    from megagemm.swiglu import MegaGemmFunction, MegaGemmTriton   # the reference package
    from benchmark_swiglu import PyTorchSwiGLU                      # the reference's baseline module

    g = torch.Generator().manual_seed(4321)
    out = {}
    # activation alone, through the reference's Triton kernels (interpreted)
    for name, m, f, dt in [("act_f32", 9, 96, torch.float32), ("act_f16", 5, 160, torch.float16),
                           ("act_bf16", 5, 160, torch.bfloat16)]:
        gv = (1.5 * torch.randn(m, 2 * f, generator=g)).to(dt).requires_grad_(True)
        dh = torch.randn(m, f, generator=g).to(dt)
        h = MegaGemmFunction.apply(gv, f)
        h.backward(dh)
        out.update({f"{name}_gv": gv.detach().float().numpy(), f"{name}_dh": dh.float().numpy(),
                    f"{name}_h": h.detach().float().numpy(), f"{name}_dgv": gv.grad.float().numpy()})
    # whole MLP, fp32, through the reference module
    torch.manual_seed(99)
    d_model, mult = 64, 32
    mlp = MegaGemmTriton(d_model, multiple_of=mult)
    base = PyTorchSwiGLU(d_model, multiple_of=mult)
    with torch.no_grad():                                           # benchmark_swiglu.py:85-89, reversed
        base.w1.weight.copy_(mlp.w12.weight[:mlp.hidden])
        base.w2.weight.copy_(mlp.w12.weight[mlp.hidden:])
        base.w3.weight.copy_(mlp.w3.weight)
    x = torch.randn(2, 12, d_model, generator=g).requires_grad_(True)
    dy = torch.randn(2, 12, d_model, generator=g)
    y = mlp(x)
    y.backward(dy)
    y_base = base(x.detach())
    out.update({
        "mlp_hidden": np.int64(mlp.hidden), "mlp_x": x.detach().numpy(), "mlp_dy": dy.numpy(),
        "mlp_w12": mlp.w12.weight.detach().numpy(), "mlp_w3": mlp.w3.weight.detach().numpy(),
        "mlp_y": y.detach().numpy(), "mlp_y_pytorchswiglu": y_base.detach().numpy(),
        "mlp_dx": x.grad.numpy(), "mlp_dw12": mlp.w12.weight.grad.numpy(), "mlp_dw3": mlp.w3.weight.grad.numpy(),
    })
    # hidden-size rule of the constructor (megagemm/swiglu.py:158-160) at the sizes the configs use
    rule = []
    for dm, mo, hm in [(4096, 256, 5 / 3), (2048, 256, 5 / 3), (8192, 256, 3.5), (64, 32, 5 / 3), (100, 8, 2.0)]:
        hidden = int(dm * hm)
        hidden = mo * ((hidden + mo - 1) // mo)
        rule.append((dm, mo, hm, hidden))
    chk = MegaGemmTriton(100, multiple_of=8, hidden_multiple=2.0)
    assert chk.hidden == rule[-1][3] and tuple(chk.w12.weight.shape) == (2 * chk.hidden, 100)
    assert tuple(chk.w3.weight.shape) == (100, chk.hidden)
    out["hidden_rule"] = np.array(rule, dtype=np.float64)
    np.savez_compressed(HERE / "swiglu.npz", **out)


def add_rmsnorm_cases():
    """The residual add in front of the norm, written the way a user of the reference writes it:
    h = x + residual (torch), y = rmsnorm(h) -- forward by the reference's rmsnorm_cpu, forward and
    backward by the formula its test differentiates, in fp64 -- with a gradient arriving through h as
    well as through y (dh_total = d_norm/dh + dres). Inputs are rounded to the case's dtype and h is
    rounded again after the add, as torch's add of two half-precision tensors does."""
    ref = oracle.ref_lib()
    assert ref is not None, "build oracle/_ref first: make -C oracle ref"
    g = torch.Generator().manual_seed(2468)
    out = {}
    for name, rows, cols, eps, dt in [("f32", 5, 264, 1e-6, torch.float32), ("f16", 4, 256, 1e-6, torch.float16),
                                      ("bf16", 5, 512, 1e-5, torch.bfloat16)]:
        x = torch.randn(rows, cols, generator=g).to(dt)
        res = torch.randn(rows, cols, generator=g).to(dt)
        w = (1.0 + 0.1 * torch.randn(cols, generator=g)).to(dt)
        dy = torch.randn(rows, cols, generator=g).to(dt)
        dres = torch.randn(rows, cols, generator=g).to(dt)
        h = (x + res)                                   # torch's add in the case's dtype: the reference user's first line
        y_ref_cpu = ref.cpu_forward(h.float().numpy(), w.float().numpy(), eps)
        h64 = h.double().requires_grad_(True)
        w64 = w.double().requires_grad_(True)
        y64 = h64 * torch.rsqrt(h64.pow(2).mean(-1, keepdim=True) + float(np.float32(eps))) * w64
        (y64 * dy.double()).sum().backward()
        out.update({
            f"{name}_x": x.float().numpy(), f"{name}_res": res.float().numpy(), f"{name}_w": w.float().numpy(),
            f"{name}_dy": dy.float().numpy(), f"{name}_dres": dres.float().numpy(), f"{name}_eps": np.float32(eps),
            f"{name}_h": h.float().numpy(), f"{name}_y_refcpu": y_ref_cpu, f"{name}_y": y64.detach().numpy(),
            f"{name}_dh": (h64.grad + dres.double()).numpy(), f"{name}_dw": w64.grad.numpy(),
        })
    np.savez_compressed(HERE / "add_rmsnorm.npz", **out)


if __name__ == "__main__":
    rmsnorm_cases()
    swiglu_cases()
    add_rmsnorm_cases()
    for p in sorted(HERE.glob("*.npz")):
        print(p.name, p.stat().st_size, "bytes")
