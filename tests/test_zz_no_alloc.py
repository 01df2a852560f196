"""mgr_rmsnorm_bwd_noalloc: the RMSNorm backward for hosts that cannot allocate device memory.

Some users of the library have nobody to ask for scratch memory at call time: a C or C++ program that
links libmgr_b200.so without torch's caching allocator, or a service that, once warmed up, keeps
cudaMalloc and cudaFree out of its request path because both stall the whole GPU and can fail late when
memory is fragmented. For them the backward's scratch (the per-CTA partial sums of dW) lives in a fixed
16 MiB array inside the library. This test calls that entry point through the C ABI and checks it
against the regular entry point (caller-provided workspace) on the same inputs, twice in a row with
different shapes, because the array is shared between calls and keeps what the previous call left.

Collected last on purpose (file name): a run that stops at the first failure has then already run every
other test. It does not depend on them: it passes alone in a fresh process as well.
"""
import pytest
import torch

from mgrrmsnorm_b200 import _capi
from tests.util import seeded_rmsnorm_inputs

pytestmark = pytest.mark.gpu

CODES = {"f32": _capi.MGR_F32, "f16": _capi.MGR_F16, "bf16": _capi.MGR_BF16}


def both_backwards(L, rows, cols, dtype, seed):
    """Runs forward, then the backward through both entry points. Returns ((dx, dw, dw32), (dx, dw, dw32))."""
    code = CODES[dtype]
    x, w, dy = (t.cuda() for t in seeded_rmsnorm_inputs(rows, cols, dtype, seed))
    stream = torch.cuda.current_stream().cuda_stream
    y = torch.empty_like(x)
    inv = torch.empty(rows, dtype=torch.float32, device="cuda")
    assert L.mgr_rmsnorm_fwd(y.data_ptr(), inv.data_ptr(), x.data_ptr(), w.data_ptr(), rows, cols, 1e-6, code, stream) == 0

    def outputs():
        # poisoned, so that an entry point that wrote nothing cannot pass by accident
        return (torch.full_like(x, float("nan")), torch.full_like(w, float("nan")),
                torch.full((cols,), float("nan"), dtype=torch.float32, device="cuda"))

    ref = outputs()
    nbytes = int(L.mgr_rmsnorm_bwd_workspace_bytes(rows, cols, code))
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device="cuda")
    st = L.mgr_rmsnorm_bwd(ref[0].data_ptr(), ref[1].data_ptr(), ref[2].data_ptr(), dy.data_ptr(), x.data_ptr(), w.data_ptr(),
                           inv.data_ptr(), rows, cols, code, ws.data_ptr(), ws.numel(), stream)
    assert st == 0, _capi.status_str(st)
    got = outputs()
    st = L.mgr_rmsnorm_bwd_noalloc(got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), dy.data_ptr(), x.data_ptr(),
                                   w.data_ptr(), inv.data_ptr(), rows, cols, code, stream)
    assert st == 0, _capi.status_str(st)
    torch.cuda.synchronize()
    return ref, got


def assert_same(ref, got, dtype):
    # Same kernels, same launch plan, same fixed summation order: the two entry points agree to the
    # last bit. The tolerance the other tests allow against the oracle (half an output ulp plus 1e-5
    # relative) is therefore met with room to spare; equality is asserted because it is what holds.
    for a, b, name in zip(ref, got, ("dx", "dw", "dw_f32")):
        assert not torch.isnan(b).any(), f"{name}: the allocation-free entry point left values unwritten"
        assert torch.equal(a, b), f"{name}: differs from mgr_rmsnorm_bwd, max |diff| {float((a.float() - b.float()).abs().max())}"


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
def test_noalloc_backward_matches_regular_entry_point_twice_in_a_row(built_lib, dtype):
    L = built_lib
    # first call: many partial rows (one per resident CTA) fill a large part of the shared array
    assert_same(*both_backwards(L, 6000, 8192, dtype, seed=101), dtype)
    # second call, straight after, smaller and differently shaped: must not see the first call's leftovers
    assert_same(*both_backwards(L, 333, 1000 if dtype == "f32" else 2048, dtype, seed=202), dtype)
    # and a third on the bulk-copy-ring family's home ground (32 KB rows), again right behind
    assert_same(*both_backwards(L, 2000, 16384 if dtype == "bf16" else 8192, dtype, seed=303), dtype)
    assert L.mgr_device_status(1) == 0


def test_noalloc_backward_refuses_what_does_not_fit(built_lib):
    L = built_lib
    t = torch.zeros(1 << 16, device="cuda")
    p = t.data_ptr()
    rows, cols = 4096, 32768
    assert int(L.mgr_rmsnorm_bwd_workspace_bytes(rows, cols, _capi.MGR_BF16)) > (16 << 20)
    st = L.mgr_rmsnorm_bwd_noalloc(p, p, None, p, p, p, p, rows, cols, _capi.MGR_BF16, None)   # refused before any launch
    assert st == _capi.MGR_ERR_TOO_LARGE and "maximum" in _capi.status_str(st)
    assert L.mgr_rmsnorm_bwd_noalloc(p, p, None, p, p, p, p, -1, 64, _capi.MGR_F32, None) == _capi.MGR_ERR_BAD_SHAPE
    assert L.mgr_rmsnorm_bwd_noalloc(p, p, None, p, p, p, p, 4, 64, 9, None) == _capi.MGR_ERR_BAD_DTYPE
    assert L.mgr_rmsnorm_bwd_noalloc(None, p, None, p, p, p, p, 4, 64, _capi.MGR_F32, None) == _capi.MGR_ERR_NULL_PTR


def test_noalloc_backward_from_several_host_threads_one_call_at_a_time(built_lib):
    """Host threads may share the entry point (its per-device address lookup is held in an atomic), but the
    scratch array is one per GPU: a call is two launches that hand partial rows through it, so callers take
    turns -- here under a lock, all on one stream. Every thread's results equal the regular entry point's."""
    import threading

    L = built_lib
    shapes = [(700, 4096, "bf16"), (300, 8192, "f32"), (1000, 1024, "f16"), (129, 1000, "f32"), (2000, 2048, "bf16"), (64, 5120, "f16")]
    turn = threading.Lock()
    failures = []

    def work(i):
        rows, cols, dtype = shapes[i]
        try:
            for rep in range(3):
                with turn:
                    ref, got = both_backwards(L, rows, cols, dtype, seed=500 + 10 * i + rep)
                assert_same(ref, got, dtype)
        except Exception as e:  # noqa: BLE001 -- surfaced below; an exception in a thread would otherwise pass silently
            failures.append((shapes[i], repr(e)))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(shapes))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures
    assert L.mgr_device_status(1) == 0
