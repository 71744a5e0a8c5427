"""rwkv_mm8_one_static: the mm8_one entry point for hosts that cannot hand the library a
workspace (it keeps its split-K scratch in a fixed array of the library's device image).

Called straight through the C ABI and compared with rwkv_mm8_one on a fresh caller-provided
workspace.  The scratch is only touched by the split-K ("ticket") kernel, so every case makes that
kernel run: either by forcing it (`rwkv_mm8_one_set_cluster(-1, 0)`) or with a matrix the cluster
kernel cannot take (contiguous rows of odd length).  Calls follow one another on different shapes,
so each one finds the previous call's partial sums in the shared array and must not be disturbed by
them; the largest case reaches the top of the array.  This file sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(N, M, seed, stride=None):
    g = torch.Generator().manual_seed(seed)
    P = stride if stride is not None else (M + 15) // 16 * 16
    w = torch.randint(0, 256, (N, P), dtype=torch.uint8, generator=g).cuda()[:, :M]
    mx = (torch.randn(M, generator=g) * 0.01).half().cuda()
    rx = (torch.rand(M, generator=g) * 0.01).half().cuda()
    my = (torch.randn(N, generator=g) * 0.01).half().cuda()
    ry = (torch.rand(N, generator=g) * 0.01).half().cuda()
    x = torch.randn(N, generator=g).half().cuda()
    return x, w, mx, rx, my, ry


def _both(L, _lib, N, M, seed, stride=None):
    stream = torch.cuda.current_stream().cuda_stream
    x, w, mx, rx, my, ry = _case(N, M, seed, stride)
    ptrs = (x.data_ptr(), w.data_ptr(), w.stride(0), mx.data_ptr(), rx.data_ptr(), my.data_ptr(), ry.data_ptr())
    y_ws = torch.zeros(M, dtype=torch.float32, device="cuda")
    nbytes = L.rwkv_mm8_one_workspace_bytes(N, M)
    ws = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    assert L.rwkv_mm8_one(N, M, *ptrs, _lib.F16, y_ws.data_ptr(), ws.data_ptr(), nbytes, stream) == 0
    y_st = torch.zeros(M, dtype=torch.float32, device="cuda")
    assert L.rwkv_mm8_one_static(N, M, *ptrs, _lib.F16, y_st.data_ptr(), stream) == 0
    torch.cuda.synchronize()
    return y_st, y_ws


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from chatrwkv_b200 import _lib
    L = _lib.lib()
    L.rwkv_mm8_one_set_cluster(-1, 0)           # split-K through scratch: the kernel that uses the array
    try:
        # two calls in a row, different shapes: the second finds the first one's partial sums
        for call, (N, M, seed) in enumerate([(4096, 4096, 11), (1024, 12000, 12), (2048, 32768, 13), (4096, 4096, 14)]):
            y_st, y_ws = _both(L, _lib, N, M, seed)
            scale = max(1.0, y_ws.abs().max().item())
            assert (y_st - y_ws).abs().max().item() <= 2e-5 * scale, f"call {call}"
            assert y_ws.abs().max().item() > 0
    finally:
        L.rwkv_mm8_one_set_cluster(0, 0)


def test_static_scratch_entry_point_on_unaligned_rows():
    """Contiguous rows of odd length take the split-K kernel without any forcing."""
    from chatrwkv_b200 import _lib
    L = _lib.lib()
    for call, (N, M, seed) in enumerate([(2048, 12001, 21), (3000, 4099, 22)]):
        y_st, y_ws = _both(L, _lib, N, M, seed, stride=M)
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
