"""Runs ONE entry point of the library a few times on seeded inputs: the command a profiler wraps.

    python -m mgrrmsnorm_b200.profile_case --case rmsnorm --rows 65536 --cols 2048 --dtype bf16 --iters 3
    ncu --set full --clock-control none -k regex:rms_ -c 6 -o out python -m mgrrmsnorm_b200.profile_case ...

Cases: rmsnorm (forward + backward), add_rmsnorm (residual add fused, forward + backward), swiglu_act
(stand-alone activation forward + backward; --cols is the hidden size f, the projected tensor is [rows, 2f]),
peer_allreduce (the cross-rank sum of a --cols long fp32 vector run as a ONE-rank group in this process, which is
the only form a profiler may wrap: the kernel stores to and reads from its own buffer; --rows is ignored).
--path reg|ring|scalar pins the RMSNorm kernel family (MGR_RMSNORM_PATH); the default is the library's own
choice for the shape, which is what the profiles under profiles/ document. Inputs are generated on the
device before the first call; keep them larger than L2 (126 MB) and small enough for a profiler's replays.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch

DTYPES = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--case", choices=["rmsnorm", "add_rmsnorm", "swiglu_act", "peer_allreduce"], required=True)
    ap.add_argument("--rows", type=int, required=True)
    ap.add_argument("--cols", type=int, required=True)
    ap.add_argument("--dtype", choices=sorted(DTYPES), default="bf16")
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--path", choices=["reg", "ring", "scalar"], default=None)
    args = ap.parse_args(argv)
    if args.path:
        os.environ["MGR_RMSNORM_PATH"] = args.path
    from . import rmsnorm_cuda_ops as ops

    if not torch.cuda.is_available():
        print("profile_case needs a CUDA device", file=sys.stderr)
        return 2
    dev = torch.device("cuda", 0)
    dt = DTYPES[args.dtype]
    g = torch.Generator(device=dev).manual_seed(1234)
    rows, cols = args.rows, args.cols

    def rnd(*shape):
        return torch.randn(*shape, device=dev, generator=g).to(dt)

    if args.case == "peer_allreduce":
        import ctypes

        from . import _capi

        L = _capi.lib()
        n = cols // 4 * 4
        buf = torch.zeros(int(L.mgr_peer_allreduce_buffer_bytes(1, n)), dtype=torch.uint8, device=dev)
        calls = torch.zeros(_capi.MGR_PEER_ALLREDUCE_CTAS, dtype=torch.int32, device=dev)
        src, out = torch.randn(n, device=dev, generator=g), torch.empty(n, device=dev, dtype=dt)
        ptrs = (ctypes.c_void_p * 1)(buf.data_ptr())
        for _ in range(args.iters):
            _capi.check("mgr_peer_allreduce_f32", L.mgr_peer_allreduce_f32(ptrs, 0, 1, src.data_ptr(), None, out.data_ptr(), ops._DTYPES[dt], n, n,
                                                                          calls.data_ptr(), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        assert torch.equal(out, src.to(dt))
    elif args.case == "swiglu_act":
        gv, dh = rnd(rows, 2 * cols), rnd(rows, cols)
        for _ in range(args.iters):
            ops.swiglu_act_forward(gv, cols)
            ops.swiglu_act_backward(dh, gv, cols)
    else:
        x, dy = rnd(rows, cols), rnd(rows, cols)
        w = (1 + 0.1 * torch.randn(cols, device=dev, generator=g)).to(dt)
        if args.case == "rmsnorm":
            for _ in range(args.iters):
                _, inv = ops.rmsnorm_forward(x, w, 1e-6)
                ops.rmsnorm_backward(dy, x, w, inv)
        else:
            res, dres = rnd(rows, cols), rnd(rows, cols)
            for _ in range(args.iters):
                _, h, inv = ops.add_rmsnorm_forward(x, res, w, 1e-6)
                ops.add_rmsnorm_backward(dy, dres, h, w, inv)
    torch.cuda.synchronize()
    ops.device_status()
    print(f"ok: {args.case} {rows}x{cols} {args.dtype} x{args.iters}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
