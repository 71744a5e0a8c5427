"""Helpers shared by the GPU parity tests."""
import torch

from oracle import rwkv_oracle as orc


def packed_case(N, M, seed, device="cuda", std=0.02, atype=torch.float16):
    """Seeded fp16-valued weights N(0, std) packed by the ORACLE packer (CPU), moved to the
    device with the padded row stride the loader uses."""
    from chatrwkv_b200 import ops
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(N, M, generator=g) * std).half().float()
    q, mx, rx, my, ry = orc.quantize_weight(w, atype)
    P = ops.padded_stride(M)
    qd = torch.zeros((N, P), dtype=torch.uint8, device=device)
    qd[:, :M].copy_(q)
    cpu = (q, mx, rx, my, ry)
    dev = (qd[:, :M], mx.to(device), rx.to(device), my.to(device), ry.to(device))
    return cpu, dev
