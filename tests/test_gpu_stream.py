"""The persistent decode kernel (rwkv_mm8_stream_*) through the C ABI: phases of plain mm8_one problems
on seeded inputs against the CPU oracle's exactly rounded sums, including column counts that do not
divide by four or by the CTA count, more CTAs than column quads, 20480 in-features, one-signed and
outlier activations, results that feed the next phase, and bit-identical repeats."""
import ctypes as C

import pytest
import torch

from oracle import rwkv_oracle as orc

pytestmark = pytest.mark.gpu


def _run(phases, xs):
    """phases: list of lists of (name, N, M, epilogue, x_key); xs: dict of input vectors (fp16, CPU)."""
    from chatrwkv_b200 import _lib, ops
    from tests.util import packed_case
    L = _lib.lib()
    dev = torch.device("cuda", torch.cuda.current_device())
    bufs = {k: v.to(dev) for k, v in xs.items()}
    cpu_w, problems, counts, outs, keep = {}, [], [], {}, []
    for ph in phases:
        counts.append(len(ph))
        for (name, N, M, epi, xkey) in ph:
            cpu, dv = packed_case(N, M, seed=N * 7 + M)
            cpu_w[name] = cpu
            y = torch.zeros(M, dtype=torch.float32 if epi in (_lib.EPI_ACC_F32, _lib.EPI_STORE_F32) else torch.float16, device=dev)
            outs[name] = y
            bufs[name] = y
            problems.append(ops.make_problem(bufs[xkey], *dv, y, epi))
            keep.append(dv)
    arr = (_lib.Mm8Problem * len(problems))(*problems)
    cnt = (C.c_int32 * len(counts))(*counts)
    G = L.rwkv_mm8_stream_ctas()
    nbytes = L.rwkv_mm8_stream_weight_bytes(arr, len(problems), G)
    wstream = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    assert L.rwkv_mm8_stream_pack(arr, len(problems), G, wstream.data_ptr(), nbytes, stream) == 0
    tbytes = L.rwkv_mm8_stream_table_bytes(len(counts))
    host = torch.zeros(tbytes, dtype=torch.uint8)
    assert L.rwkv_mm8_stream_plan(arr, cnt, len(counts), _lib.F16, G, host.data_ptr(), tbytes) == 0
    table = host.to(dev)
    sync = torch.zeros(16, dtype=torch.int32, device=dev)
    results = []
    for _ in range(2):
        for y in outs.values():
            y.zero_()
        assert L.rwkv_mm8_stream_run(table.data_ptr(), host.data_ptr(), wstream.data_ptr(), sync.data_ptr(), None, stream) == 0
        e = C.c_int(0)
        assert L.rwkv_mm8_stream_take_error(sync.data_ptr(), stream, C.byref(e)) == 0 and e.value == 0
        results.append({k: v.clone().cpu() for k, v in outs.items()})
    for k in outs:
        assert torch.equal(results[0][k], results[1][k]), k
    return results[0], cpu_w


@pytest.mark.parametrize("kind", ["gauss", "one_signed", "outlier"])
def test_stream_phases_match_oracle(kind):
    from chatrwkv_b200 import _lib
    g = torch.Generator().manual_seed(5)
    def vec(n):
        v = torch.randn(n, generator=g)
        if kind == "one_signed":
            v = v.clamp(min=0) ** 2
        if kind == "outlier":
            v = v * 0.01
            v[n // 3] = 50.0
        return v.half()
    xs = {"x0": vec(512), "x1": vec(20480), "x2": vec(768)}
    phases = [
        [("a", 512, 1000, _lib.EPI_STORE_F32, "x0"), ("b", 512, 301, _lib.EPI_STORE_F32, "x0"), ("c", 512, 64, _lib.EPI_ACC_F32, "x0")],
        [("d", 20480, 520, _lib.EPI_STORE_F32, "x1")],
        [("e", 768, 50277, _lib.EPI_STORE_F32, "x2"), ("f", 768, 3, _lib.EPI_ACC_F32, "x2")],
    ]
    got, cpu_w = _run(phases, xs)
    for ph in phases:
        for (name, N, M, epi, xkey) in ph:
            ref = orc.mm8_kernel(xs[xkey], *cpu_w[name])
            # The streamed sum is exact; what remains is the fp32 combination rx * sum + mx * sum(x) + sum(x * my), whose
            # terms cancel when x is one-signed (they are then ~100 times the result): fp32 round-off of the largest term.
            tol = (2e-5 if kind == "one_signed" else 4e-6) * max(1.0, ref.abs().max().item())
            if epi == _lib.EPI_STORE_F32:
                ref16 = ref.half().float()
                # the rounding to fp16 may fall on the other side for sums within that round-off of a tie
                d = (got[name] - ref16).abs()
                assert (d <= ref.abs() * 2 ** -10 + tol).all(), (name, d.max().item())
                assert (got[name] != ref16).float().mean().item() < (0.06 if kind == "one_signed" else 0.02), name
            else:
                assert (got[name] - ref).abs().max().item() <= tol, name


def test_stream_phase_consumes_previous_phase():
    """Phase 2 multiplies what phase 1 stored (fp16 sigmoid outputs), after the grid barrier."""
    from chatrwkv_b200 import _lib
    g = torch.Generator().manual_seed(6)
    xs = {"x0": torch.randn(1024, generator=g).half()}
    phases = [[("h", 1024, 4096, _lib.EPI_SIGMOID, "x0")], [("o", 4096, 777, _lib.EPI_ACC_F32, "h")]]
    got, cpu_w = _run(phases, xs)
    h = torch.sigmoid(orc.mm8_kernel(xs["x0"], *cpu_w["h"]).half().float()).half()
    assert (got["h"].float() - h.float()).abs().max().item() <= 1e-3
    ref = orc.mm8_kernel(got["h"], *cpu_w["o"])
    assert (got["o"] - ref).abs().max().item() <= 2e-5 * max(1.0, ref.abs().max().item())   # x = sigmoid(.) > 0: one-signed
