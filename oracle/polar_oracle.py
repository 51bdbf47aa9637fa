"""CPU oracle for the PolarEngine quantized-linear path.  TEST INFRASTRUCTURE ONLY.

This module restates, on the CPU, the arithmetic the reference project
(caiovicentino/polarengine-vllm) defines for its quantized-linear forward and for
the data formats either side of it.  It exists to check the CUDA kernels; nothing
in the product package imports it.  Only the test-suite, the smoke check and the
CPU-baseline leg of the benchmark may call it.

Parity status: pinned.  Every function below is checked in
``tests/test_oracle_golden.py`` against vectors produced by importing the reference
itself (``tests/golden/make_golden.py`` wrote them) and against the known-answer
bytes the reference's own tests hold (0xC3 / 0x0F nibble placement, the H2 literal,
Hadamard involution).  The MoE composition has no counterpart arithmetic in the
reference (its MoE method forwards to vLLM's bf16 fused MoE), so ``moe_forward`` is
a composition of the pinned pieces and is itself "parity unpinned".

Each function cites the reference file:line it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import numpy as np
import torch

BLOCK = 128


# --------------------------------------------------------------------------- centroids
def lloyd_max_centroids(n_levels: int, n_iter: int = 100) -> np.ndarray:
    """Lloyd-Max levels for N(0,1); float64 in, float32 out.

    Follows polarengine_vllm/utils.py:21-68: interior boundaries start at
    linspace(-4, 4, L+1) with infinite ends; 100 rounds of
    {conditional mean per cell (midpoint if the cell mass <= 1e-10); midpoints}.
    """
    from scipy.stats import norm

    edges = np.linspace(-4, 4, n_levels + 1)
    edges[0], edges[-1] = -np.inf, np.inf
    levels = np.zeros(n_levels)
    for _ in range(n_iter):
        levels = np.zeros(n_levels)
        for i in range(n_levels):
            lo, hi = edges[i], edges[i + 1]
            mass = norm.cdf(hi) - norm.cdf(lo)
            levels[i] = (norm.pdf(lo) - norm.pdf(hi)) / mass if mass > 1e-10 else (lo + hi) / 2
        nxt = np.zeros(n_levels + 1)
        nxt[0], nxt[-1] = -np.inf, np.inf
        for i in range(1, n_levels):
            nxt[i] = (levels[i - 1] + levels[i]) / 2
        edges = nxt
    return levels.astype(np.float32)


_CT: Dict[int, np.ndarray] = {}


def centroids(bits: int) -> np.ndarray:
    """polarengine_vllm/utils.py:78-100 (valid range 2..8, cached)."""
    if bits < 2 or bits > 8:
        raise ValueError(f"bits must be in [2, 8], got {bits}")
    if bits not in _CT:
        _CT[bits] = lloyd_max_centroids(1 << bits)
    return _CT[bits]


def ct_scaled(bits: int, block: int = BLOCK) -> torch.Tensor:
    """Runtime table: centroids / sqrt(block) in fp32 (linear_method.py:131-135)."""
    return torch.from_numpy(centroids(bits).copy()) / math.sqrt(block)


# --------------------------------------------------------------------------- rotation
_H: Dict[int, torch.Tensor] = {}


def hadamard(n: int) -> torch.Tensor:
    """Normalised Sylvester matrix, built level by level with a /sqrt(2) per level
    (polarengine_vllm/kernels/fwht.py:54-62); fp32, symmetric, its own inverse."""
    assert n >= 1 and n & (n - 1) == 0
    if n not in _H:
        if n == 1:
            _H[n] = torch.tensor([[1.0]])
        else:
            h = hadamard(n // 2)
            _H[n] = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0) / math.sqrt(2)
    return _H[n]


def fwht(x: torch.Tensor, block: int = BLOCK) -> torch.Tensor:
    """Block-wise rotation as one matmul (kernels/fwht.py:102-108)."""
    assert x.shape[-1] % block == 0
    return (x.reshape(-1, block) @ hadamard(block).to(x.dtype)).reshape(x.shape)


def fwht_butterfly(x: torch.Tensor) -> torch.Tensor:
    """Seven add/sub stages with strides 1..64 then 1/sqrt(n)
    (kernels/fwht.py:180-190; kernels/cuda/fwht_cuda.cu:59-81)."""
    n = x.shape[-1]
    y = x.clone().reshape(-1, n)
    h = 1
    while h < n:
        y = y.reshape(-1, n // (2 * h), 2, h)
        a, b = y[:, :, 0, :], y[:, :, 1, :]
        y = torch.stack([a + b, a - b], 2).reshape(-1, n)
        h *= 2
    return (y / math.sqrt(n)).reshape(x.shape)


# --------------------------------------------------------------------------- quantizer
def quantize_tensor(weight: torch.Tensor, bits: int, block: int = BLOCK) -> Dict[str, torch.Tensor]:
    """Offline producer of codes / norms / ct_scaled (quantizer.py:206-257).

    Same torch operators in the same order as the reference so that codes and norms
    come out bit-identical: pad K, per-block L2 norm clamped at 1e-10, divide,
    64-row chunks of (u @ H) * sqrt(block), argmin of |r - c_j| (first minimum).
    """
    ct = torch.from_numpy(centroids(bits).copy())
    H = hadamard(block)
    n, k = weight.shape
    kp = (k + block - 1) // block * block
    nb = kp // block
    w = weight.detach().float()
    if kp > k:
        w = torch.nn.functional.pad(w, (0, kp - k))
    blocks = w.view(n, nb, block)
    norms = blocks.norm(dim=2).clamp(min=1e-10)
    unit = blocks / norms.unsqueeze(2)
    codes = torch.empty(n, nb, block, dtype=torch.int8)
    s = math.sqrt(block)
    ctv = ct.view(1, 1, 1, -1)
    for i in range(0, n, 64):
        j = min(i + 64, n)
        r = ((unit[i:j].reshape(-1, block) @ H) * s).view(j - i, nb, block)
        codes[i:j] = (r.unsqueeze(-1) - ctv).abs().argmin(dim=-1).to(torch.int8)
    return {"codes": codes.reshape(n, kp), "norms": norms.half(), "ct_scaled": ct / s}


# --------------------------------------------------------------------------- layouts
def pack_nibble(codes: np.ndarray, block: int = BLOCK) -> np.ndarray:
    """Half-block nibble layout: byte i of a block = code[64+i] << 4 | code[i]
    (packing.py:45-60; kernels/polar_gemv.py:275-283; utils.py:211-260)."""
    c = np.asarray(codes).astype(np.uint8)
    *lead, k = c.shape
    assert k % block == 0
    b = c.reshape(*lead, k // block, block)
    h = block // 2
    return ((b[..., h:] << 4) | b[..., :h]).reshape(*lead, k // 2)


def unpack_nibble(packed: np.ndarray, block: int = BLOCK) -> np.ndarray:
    """Inverse of pack_nibble (packing.py:63-94)."""
    p = np.asarray(packed).astype(np.uint8)
    *lead, kh = p.shape
    h = block // 2
    b = p.reshape(*lead, kh // h, h)
    return np.concatenate([b & 15, b >> 4], -1).reshape(*lead, kh * 2).astype(np.int8)


def pack_q5(codes: np.ndarray) -> np.ndarray:
    """"v5" disk layout, LSB-first, 8 codes -> 5 bytes (packing.py:109-114, 149-153)."""
    c = np.asarray(codes).astype(np.int64) & 0xFF
    *lead, k = c.shape
    g = c.reshape(*lead, k // 8, 8)
    c0, c1, c2, c3, c4, c5, c6, c7 = [g[..., i] for i in range(8)]
    out = np.stack([
        c0 | c1 << 5,
        c1 >> 3 | c2 << 2 | c3 << 7,
        c3 >> 1 | c4 << 4,
        c4 >> 4 | c5 << 1 | c6 << 6,
        c6 >> 2 | c7 << 3,
    ], -1) & 0xFF
    return out.astype(np.uint8).reshape(*lead, k * 5 // 8)


def unpack_q5(packed: np.ndarray) -> np.ndarray:
    """Inverse of pack_q5 (packing.py:163-209)."""
    p = np.asarray(packed).astype(np.int64)
    *lead, kp = p.shape
    b = p.reshape(*lead, kp // 5, 5)
    b0, b1, b2, b3, b4 = [b[..., i] for i in range(5)]
    out = np.stack([
        b0, b0 >> 5 | b1 << 3, b1 >> 2, b1 >> 7 | b2 << 1,
        b2 >> 4 | b3 << 4, b3 >> 1, b3 >> 6 | b4 << 2, b4 >> 3,
    ], -1) & 31
    return out.astype(np.int8).reshape(*lead, kp * 8 // 5)


def pack_q5_hlwq(codes: np.ndarray) -> np.ndarray:
    """HLWQ 5-bit layout, MSB-first (packing.py:274-290)."""
    c = np.asarray(codes).astype(np.int64)
    *lead, k = c.shape
    pad = (-k) % 8
    if pad:
        c = np.concatenate([c, np.zeros((*lead, pad), np.int64)], -1)
        k += pad
    g = c.reshape(*lead, k // 8, 8)
    c0, c1, c2, c3, c4, c5, c6, c7 = [g[..., i] for i in range(8)]
    out = np.stack([
        c0 << 3 | c1 >> 2,
        (c1 & 3) << 6 | c2 << 1 | c3 >> 4,
        (c3 & 15) << 4 | c4 >> 1,
        (c4 & 1) << 7 | c5 << 2 | c6 >> 3,
        (c6 & 7) << 5 | c7,
    ], -1) & 0xFF
    return out.astype(np.uint8).reshape(*lead, -1)


def unpack_q5_hlwq(packed: np.ndarray, total: Optional[int] = None) -> np.ndarray:
    """Inverse of pack_q5_hlwq (packing.py:229-271)."""
    p = np.asarray(packed).astype(np.int64)
    *lead, kp = p.shape
    b = p.reshape(*lead, kp // 5, 5)
    b0, b1, b2, b3, b4 = [b[..., i] for i in range(5)]
    out = np.stack([
        b0 >> 3,
        (b0 & 7) << 2 | b1 >> 6,
        b1 >> 1,
        (b1 & 1) << 4 | b2 >> 4,
        (b2 & 15) << 1 | b3 >> 7,
        b3 >> 2,
        (b3 & 3) << 3 | b4 >> 5,
        b4,
    ], -1) & 31
    out = out.astype(np.int8).reshape(*lead, -1)
    return out if total is None else out[..., :total]


# --------------------------------------------------------------------------- forward
def dequant_fp32(codes: torch.Tensor, norms: torch.Tensor, cts: torch.Tensor,
                 block: int = BLOCK) -> torch.Tensor:
    """fp32 weight (ct_scaled[codes] @ H) * norm; the math of weight_converter.py:54-67
    without its final bf16 cast (ct_scaled already carries the 1/sqrt(block))."""
    n, kp = codes.shape
    nb = kp // block
    v = cts.float()[codes.long() & 0xFF].view(n * nb, block) @ hadamard(block)
    return (v.view(n, nb, block) * norms.float().view(n, nb, 1)).reshape(n, kp)


def linear_dequant(x: torch.Tensor, codes: torch.Tensor, norms: torch.Tensor,
                   cts: torch.Tensor, in_f: Optional[int] = None) -> torch.Tensor:
    """The oracle: y = x.float() @ dequant.T in fp32 ("fp32 dequant reference")."""
    w = dequant_fp32(codes, norms, cts)
    k = in_f if in_f is not None else x.shape[-1]
    return x.float().reshape(-1, k) @ w[:, :k].T


def linear_hadamard_domain(x: torch.Tensor, codes: torch.Tensor, norms: torch.Tensor,
                           cts: torch.Tensor, block: int = BLOCK) -> torch.Tensor:
    """Same result without the inverse rotation (tests/test_kernel_correctness.py:86-108):
    y[m, r] = sum_blk norm[r, blk] * <ct_scaled[codes[r, blk, :]], FWHT(x)[m, blk, :]>."""
    n, kp = codes.shape
    nb = kp // block
    xf = x.float().reshape(-1, x.shape[-1])
    if xf.shape[1] < kp:
        xf = torch.nn.functional.pad(xf, (0, kp - xf.shape[1]))
    xt = fwht(xf, block).view(-1, nb, block)
    vals = cts.float()[codes.long() & 0xFF].view(n, nb, block) * norms.float().view(n, nb, 1)
    return torch.einsum("rnk,mnk->mr", vals, xt)


def apply_forward(x: torch.Tensor, codes: torch.Tensor, norms: torch.Tensor, cts: torch.Tensor,
                  in_f: int, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Semantics of PolarQuantLinearMethod.apply (linear_method.py:184-222):
    flatten, fp32, pad, rotate, matmul, cast to fp16, restore leading dims, add bias.half()."""
    lead = x.shape[:-1]
    y = linear_hadamard_domain(x.reshape(-1, in_f), codes, norms, cts).half()
    y = y.view(*lead, codes.shape[0])
    return y + bias.half() if bias is not None else y


# --------------------------------------------------------------------------- MoE
def moe_route(x: torch.Tensor, gate_w: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax over fp32 logits, top-k, renormalise (nemotron_offload.py:180-189)."""
    p = torch.softmax(x.float() @ gate_w.float().T, dim=-1)
    w, ids = p.topk(top_k, dim=-1)
    return w / w.sum(-1, keepdim=True), ids


def moe_forward(x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor, experts: list) -> torch.Tensor:
    """sum_k w_k * down(silu(gate(x)) * up(x)) per token (nemotron_offload.py:199-226),
    every projection being the quantized linear above.  ``experts[e]`` is a dict with
    keys gate/up/down -> (codes int8, norms fp16, ct_scaled fp32, in_f)."""
    t = x.shape[0]
    out_f = experts[0]["down"][0].shape[0]
    y = torch.zeros(t, out_f)
    xf = x.float()
    for e in topk_ids.unique().tolist():
        tok, slot = (topk_ids == e).nonzero(as_tuple=True)
        ex = experts[e]
        g = linear_hadamard_domain(xf[tok], *ex["gate"][:3])
        u = linear_hadamard_domain(xf[tok], *ex["up"][:3])
        h = torch.nn.functional.silu(g) * u
        d = linear_hadamard_domain(h, *ex["down"][:3])
        y.index_add_(0, tok, d * topk_w[tok, slot].float().unsqueeze(1))
    return y
