"""Lloyd-Max tables and the mixed-bit layer table.

Mirrors the public names of polarengine_vllm/utils.py in the reference project:
``compute_lloyd_max_centroids`` (utils.py:21-68), ``get_centroids`` (78-100),
``DEFAULT_BIT_ASSIGNMENT`` (112-125), ``get_bits_for_layer`` (146-204) and the
half-block nibble helpers (211-286).
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import numpy as np
import torch

BLOCK_SIZE = 128


def compute_lloyd_max_centroids(n_levels: int, n_iter: int = 100) -> torch.Tensor:
    """MSE-optimal scalar quantizer levels for a standard normal, as fp32.

    Alternates, in float64, between the conditional mean of each cell,
    (pdf(a) - pdf(b)) / (cdf(b) - cdf(a)), and cell edges at the midpoints of
    neighbouring levels.  The first edge set is linspace(-4, 4) with open ends; a cell
    whose probability is <= 1e-10 takes its midpoint.  (Reference: utils.py:21-68.)
    """
    from scipy.stats import norm as gauss

    edge = np.linspace(-4, 4, n_levels + 1)
    edge[0] = -np.inf
    edge[-1] = np.inf
    level = np.zeros(n_levels)
    for _ in range(n_iter):
        level = np.zeros(n_levels)
        for i in range(n_levels):
            a, b = edge[i], edge[i + 1]
            p = gauss.cdf(b) - gauss.cdf(a)
            level[i] = (gauss.pdf(a) - gauss.pdf(b)) / p if p > 1e-10 else (a + b) / 2
        mid = np.zeros(n_levels + 1)
        mid[0] = -np.inf
        mid[-1] = np.inf
        for i in range(1, n_levels):
            mid[i] = (level[i - 1] + level[i]) / 2
        edge = mid
    return torch.tensor(level, dtype=torch.float32)


_TABLES: Dict[int, torch.Tensor] = {}


def get_centroids(bits: int) -> torch.Tensor:
    """Cached table of 2**bits levels; bits must be 2..8 (ValueError otherwise)."""
    if not 2 <= bits <= 8:
        raise ValueError(f"bits must be in [2, 8], got {bits}")
    tab = _TABLES.get(bits)
    if tab is None:
        tab = _TABLES[bits] = compute_lloyd_max_centroids(1 << bits)
    return tab


def get_ct_scaled(bits: int, block_size: int = BLOCK_SIZE) -> torch.Tensor:
    """Runtime table: levels / sqrt(block_size) (linear_method.py:131-135)."""
    return get_centroids(bits) / math.sqrt(block_size)


for _bits in (2, 3, 4, 5, 6):  # the widths the layer table uses
    get_centroids(_bits)

DEFAULT_BIT_ASSIGNMENT: Dict[str, int] = {
    "embed": 5, "lm_head": 6,
    "q_proj": 5, "k_proj": 5, "v_proj": 5, "o_proj": 6, "out_proj": 6,
    "gate_up_proj": 3, "gate_proj": 3, "up_proj": 3, "down_proj": 4,
    "in_proj": 5,
}

_KEEP_FP16_LOWER = ("norm", "layernorm", "rmsnorm", "a_log", "dt_bias", "dt_proj", "conv1d")
_KEEP_FP16_EXACT = (".D", "A_log")  # compared without lower-casing


def get_bits_for_layer(name: str, param: torch.Tensor, assignment: Optional[Mapping[str, int]] = None) -> int:
    """Bit width for a named parameter, 16 meaning "leave as fp16".

    fp16: fewer than two dims or under 256 elements; norm / Mamba state names; 1-D
    biases; MoE routers (``*.gate.weight`` or "router").  Otherwise the longest key of
    ``assignment`` contained in the name decides; 5 when none matches.
    """
    table = DEFAULT_BIT_ASSIGNMENT if assignment is None else assignment
    if param.ndim < 2 or param.numel() < 256:
        return 16
    low = name.lower()
    if any(s in low for s in _KEEP_FP16_LOWER) or any(s in name for s in _KEEP_FP16_EXACT):
        return 16
    if "bias" in name and param.ndim == 1:
        return 16
    if name.endswith(".gate.weight") or "router" in name:
        return 16
    for key in sorted(table, key=len, reverse=True):
        if key in name:
            return table[key]
    return 5


def pack_codes_half_block(codes: torch.Tensor, block_size: int = BLOCK_SIZE) -> torch.Tensor:
    """(..., K) codes 0..15 -> (..., K/2) bytes; within each block byte i carries
    code[i] in its low and code[block/2 + i] in its high nibble."""
    *lead, k = codes.shape
    if k % block_size:
        raise ValueError(f"Last dimension ({k}) must be a multiple of block_size ({block_size})")
    half = block_size // 2
    b = codes.reshape(*lead, k // block_size, block_size).to(torch.uint8)
    return ((b[..., half:] << 4) | b[..., :half]).reshape(*lead, k // 2)


def unpack_codes_half_block(packed: torch.Tensor, block_size: int = BLOCK_SIZE) -> torch.Tensor:
    """Inverse of :func:`pack_codes_half_block`; int8 result."""
    *lead, kh = packed.shape
    half = block_size // 2
    b = packed.reshape(*lead, kh // half, half)
    return torch.cat([b & 15, (b >> 4) & 15], -1).to(torch.int8).reshape(*lead, kh * 2)
