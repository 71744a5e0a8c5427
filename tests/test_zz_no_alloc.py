"""rwkv_mm8_one_static: the mm8_one entry point for hosts that cannot hand the library a
workspace (it keeps its split-K scratch in a fixed array of the library's device image).

Called straight through the C ABI, twice in a row on different inputs, and compared with
rwkv_mm8_one on a caller-provided workspace: same kernel and split plan, so the outputs have to
agree to the tolerance the other mm8_one tests use.  The second call finds the first call's
leftovers in the shared array and must not be disturbed by them.  This file sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(N, M, seed):
    g = torch.Generator().manual_seed(seed)
    P = (M + 15) // 16 * 16
    w = torch.randint(0, 256, (N, P), dtype=torch.uint8, generator=g).cuda()[:, :M]
    mx = (torch.randn(M, generator=g) * 0.01).half().cuda()
    rx = (torch.rand(M, generator=g) * 0.01).half().cuda()
    my = (torch.randn(N, generator=g) * 0.01).half().cuda()
    ry = (torch.rand(N, generator=g) * 0.01).half().cuda()
    x = torch.randn(N, generator=g).half().cuda()
    return x, w, mx, rx, my, ry


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from chatrwkv_b200 import _lib
    L = _lib.lib()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (N, M, seed) in enumerate([(4096, 4096, 11), (1024, 12000, 12)]):
        x, w, mx, rx, my, ry = _case(N, M, seed)
        ptrs = (x.data_ptr(), w.data_ptr(), w.stride(0), mx.data_ptr(), rx.data_ptr(), my.data_ptr(), ry.data_ptr())
        y_ws = torch.zeros(M, dtype=torch.float32, device="cuda")
        nbytes = L.rwkv_mm8_one_workspace_bytes(N, M)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
        assert L.rwkv_mm8_one(N, M, *ptrs, _lib.F16, y_ws.data_ptr(), ws.data_ptr(), nbytes, stream) == 0
        y_st = torch.zeros(M, dtype=torch.float32, device="cuda")
        assert L.rwkv_mm8_one_static(N, M, *ptrs, _lib.F16, y_st.data_ptr(), stream) == 0
        torch.cuda.synchronize()
        scale = max(1.0, y_ws.abs().max().item())
        assert (y_st - y_ws).abs().max().item() <= 2e-5 * scale, f"call {call}"
        assert y_ws.abs().max().item() > 0


def test_static_scratch_entry_point_rejects_oversize():
    from chatrwkv_b200 import _lib
    L = _lib.lib()
    x, w, mx, rx, my, ry = _case(32, 64, 1)
    y = torch.zeros(64, dtype=torch.float32, device="cuda")
    rc = L.rwkv_mm8_one_static(32, 40000, x.data_ptr(), w.data_ptr(), 40000, mx.data_ptr(), rx.data_ptr(),
                               my.data_ptr(), ry.data_ptr(), _lib.F16, y.data_ptr(), None)
    assert rc == -6
    assert b"32768" in L.rwkv_b200_error_string(rc)
