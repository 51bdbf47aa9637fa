"""Seeded input builders and error metrics shared by the parity tests."""
import math

import torch

import polar_oracle as oracle


def rand_layer(out_f, in_f_padded, bits, seed, device="cpu"):
    """Random codes / fp16 norms / Lloyd-Max table, generated on the CPU from a seed
    (the reference's kernel tests use random codes and |randn|+0.1 norms:
    tests/test_kernel_correctness.py:42-83)."""
    g = torch.Generator().manual_seed(seed)
    levels = 1 << bits
    codes = torch.randint(0, levels, (out_f, in_f_padded), generator=g, dtype=torch.int16).to(torch.uint8).view(torch.int8)
    norms = (torch.randn(out_f, in_f_padded // 128, generator=g).abs() * 0.02 + 0.002).half()
    cts = oracle.ct_scaled(bits)
    return codes.to(device), norms.to(device), cts.to(device)


def rand_x(batch, in_f, seed, dtype=torch.float16, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(batch, in_f, generator=g).to(dtype).to(device)


def max_rel(y, ref):
    """max |y - ref| / max |ref| -- the tolerance metric of the parity tests."""
    y, ref = y.double().cpu(), ref.double().cpu()
    return float((y - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def ref_metrics(y, ref):
    """The reference's own acceptance metrics: cosine similarity and mean element-wise
    relative error (tests/test_kernel_correctness.py:128-139)."""
    y, ref = y.double().cpu().flatten(), ref.double().cpu().flatten()
    cos = float(torch.nn.functional.cosine_similarity(y, ref, dim=0))
    mre = float(((y - ref).abs() / (ref.abs() + 1e-8)).mean())
    return cos, mre
