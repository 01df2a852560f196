"""RMSNorm forward+backward over tensors that live in HOST memory.

When x and dy sit in (pinned) host memory and y, dx have to end up there too, the step is bound by the
PCIe link, not by the kernels: at 65536 x 8192 bf16 the copies move 4 GiB while the kernels need under a
millisecond. Rows are independent, so the step is cut into row chunks and pipelined over three streams:

    copy-in stream : x[c], dy[c]  host -> device      (chunk c+1 while chunk c computes)
    compute stream : mgr_rmsnorm_fwd / mgr_rmsnorm_bwd on chunk c
    copy-out stream: y[c], dx[c]  device -> host      (chunk c-1 meanwhile)

PCIe is full duplex, so inbound and outbound copies overlap and the step takes about as long as the
larger of the two directions instead of their sum. dW is the fp32 sum of the chunks' fp32 partial
sums, added in chunk order (so it is bit-reproducible for a given chunking) and rounded once.

The arithmetic is the library's (C ABI); torch supplies streams, events and memory only.
"""
from __future__ import annotations

import os
from pathlib import Path

import torch

from . import _capi
from .rmsnorm_cuda_ops import _DTYPES


class HostRMSNormPipeline:
    """Reusable pipeline for one (rows, cols, dtype, device): device staging buffers are allocated once.

    run(x_host, dy_host, weight_dev, eps, y_host, dx_host) -> dW (device tensor, weight dtype)
    run(..., return_f32=True) -> the fp32 column sum before its rounding: what a rank that holds a row
    block of a larger batch all-reduces across ranks first (sharding.allreduce_dw) so that dW is rounded
    once, after the cross-rank sum. The returned tensor is the pipeline's own buffer, valid until the next run.
    Host tensors should be pinned (torch.Tensor.pin_memory) for the copies to be asynchronous.
    """

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, device: torch.device, chunk_rows: int | None = None,
                 depth: int = 3):
        if dtype not in _DTYPES:
            raise RuntimeError("Unsupported dtype. Use float32, float16, or bfloat16.")
        self.rows, self.cols, self.dtype, self.device = rows, cols, dtype, torch.device(device)
        if chunk_rows is None:
            # 32 MiB per tensor and chunk. The first chunk's inbound copy and the last chunk's outbound copy have
            # nothing to overlap with, so smaller chunks shorten the step until per-chunk launch and event costs
            # take over: at 65536 x 8192 bf16, 128 / 64 / 32 / 16 / 8 MiB chunks take 48.7 / 46.8 / 46.6 / 48.0 /
            # 51.1 ms on a B200 host.
            chunk_rows = max(256, (32 << 20) // max(1, cols * torch.empty(0, dtype=dtype).element_size()))
        self.chunk = max(1, min(chunk_rows, rows))
        self.depth = depth
        self.code = _DTYPES[dtype]
        self.L = _capi.lib()
        with torch.cuda.device(self.device):
            mk = lambda: torch.empty((self.chunk, cols), dtype=dtype, device=self.device)
            self.slots = [dict(x=mk(), dy=mk(), y=mk(), dx=mk(), inv=torch.empty(self.chunk, dtype=torch.float32, device=self.device),
                               loaded=torch.cuda.Event(), computed=torch.cuda.Event(), drained=torch.cuda.Event())
                          for _ in range(depth)]
            ws_bytes = int(self.L.mgr_rmsnorm_bwd_workspace_bytes(self.chunk, cols, self.code))
            self.ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=self.device)
            self.dw_part = torch.empty(cols, dtype=torch.float32, device=self.device)
            self.dw_sum = torch.empty(cols, dtype=torch.float32, device=self.device)
            self.s_in = torch.cuda.Stream(self.device)
            self.s_out = torch.cuda.Stream(self.device)

    def run(self, x_host, dy_host, weight, eps: float, y_host, dx_host, return_f32: bool = False) -> torch.Tensor:
        L, cols, code = self.L, self.cols, self.code
        for t in (x_host, dy_host, y_host, dx_host):
            if t.dtype != self.dtype or tuple(t.shape) != (self.rows, cols) or not t.is_contiguous():
                raise RuntimeError("host tensors must be contiguous [rows, cols] of the pipeline's dtype")
        if weight.dtype != self.dtype or weight.device != self.device or tuple(weight.shape) != (cols,):
            raise RuntimeError("weight must be a device tensor [cols] of the pipeline's dtype")
        main = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(main)
        self.s_out.wait_stream(main)
        self.dw_sum.zero_()
        nchunks = (self.rows + self.chunk - 1) // self.chunk
        for c in range(nchunks):
            r0 = c * self.chunk
            n = min(self.chunk, self.rows - r0)
            slot = self.slots[c % self.depth]
            with torch.cuda.stream(self.s_in):
                if c >= self.depth:
                    self.s_in.wait_event(slot["drained"])       # the slot's previous outputs have left the device
                slot["x"][:n].copy_(x_host[r0:r0 + n], non_blocking=True)
                slot["dy"][:n].copy_(dy_host[r0:r0 + n], non_blocking=True)
                slot["loaded"].record(self.s_in)
            main.wait_event(slot["loaded"])
            sp = main.cuda_stream
            _capi.check("mgr_rmsnorm_fwd", L.mgr_rmsnorm_fwd(slot["y"].data_ptr(), slot["inv"].data_ptr(), slot["x"].data_ptr(),
                                                             weight.data_ptr(), n, cols, float(eps), code, sp))
            _capi.check("mgr_rmsnorm_bwd", L.mgr_rmsnorm_bwd(slot["dx"].data_ptr(), None, self.dw_part.data_ptr(), slot["dy"].data_ptr(),
                                                             slot["x"].data_ptr(), weight.data_ptr(), slot["inv"].data_ptr(), n, cols,
                                                             code, self.ws.data_ptr(), self.ws.numel(), sp))
            self.dw_sum.add_(self.dw_part)                        # chunk order: fixed summation order
            slot["computed"].record(main)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(slot["computed"])
                y_host[r0:r0 + n].copy_(slot["y"][:n], non_blocking=True)
                dx_host[r0:r0 + n].copy_(slot["dx"][:n], non_blocking=True)
                slot["drained"].record(self.s_out)
        main.wait_stream(self.s_out)
        return self.dw_sum if return_f32 else self.dw_sum.to(self.dtype)


# ---------------------------------------------------------------------------------------------------
# where the host side of a rank runs
# ---------------------------------------------------------------------------------------------------

def _cpulist(text: str) -> set[int]:
    cpus: set[int] = set()
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        cpus.update(range(int(lo), int(hi or lo) + 1))
    return cpus


def gpu_numa_node(device) -> int | None:
    """NUMA node the GPU's PCIe slot hangs off (sysfs), or None where the platform does not say."""
    try:
        p = torch.cuda.get_device_properties(device)
        pci = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int((Path("/sys/bus/pci/devices") / pci / "numa_node").read_text())
        return node if node >= 0 else None
    except (OSError, ValueError, AttributeError, RuntimeError):
        return None


def place_near_gpu(device) -> dict:
    """Restricts the calling process to the CPUs of the GPU's NUMA node (where the scheduler allows any of
    them), so that pinned buffers allocated afterwards come from the memory next to that GPU's PCIe root and
    the copies do not cross the socket interconnect. With several ranks on one host this is what keeps each
    rank's host traffic on its own side of the machine. Returns what was found and done; never raises."""
    info = {"gpu_numa_node": gpu_numa_node(device), "bound": False}
    try:
        nodes = sorted(int(d.name[4:]) for d in Path("/sys/devices/system/node").glob("node[0-9]*"))
        info["numa_nodes"] = len(nodes)
        allowed = os.sched_getaffinity(0)
        info["cpus_allowed"] = len(allowed)
        if info["gpu_numa_node"] is not None and len(nodes) > 1:
            local = _cpulist((Path("/sys/devices/system/node") / f"node{info['gpu_numa_node']}" / "cpulist").read_text()) & allowed
            if local and local != allowed:
                os.sched_setaffinity(0, local)
                info["bound"] = True
                info["cpus_allowed"] = len(local)
    except (OSError, ValueError, AttributeError):
        pass
    return info
