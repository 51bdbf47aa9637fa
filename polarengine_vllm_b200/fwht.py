"""Block-wise Walsh-Hadamard rotation (reference: polarengine_vllm/kernels/fwht.py).

``fwht_matmul`` keeps the reference's name and meaning -- rotate every block of
``block_size`` along the last dimension by the normalised Hadamard matrix -- but on a
CUDA tensor with block_size 128 it runs the native warp-shuffle kernel
(``pe_fwht128``).  CPU tensors (the offline quantizer) and other block sizes multiply
by the cached matrix, which is also the definition the quantizer's codes depend on.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

_H: Dict[Tuple[int, str], torch.Tensor] = {}


def build_hadamard(n: int, device: Optional[torch.device] = None) -> torch.Tensor:
    """Normalised Sylvester-Hadamard matrix (n a power of two), cached per device.
    Built by doubling with a 1/sqrt(2) at every level, so H @ H = I and H = H.T."""
    assert n >= 1 and (n & (n - 1)) == 0, f"n must be a power of 2, got {n}"
    if (n, "cpu") not in _H:
        h = torch.ones(1, 1)
        size = 1
        while size < n:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0) / math.sqrt(2)
            size *= 2
            _H[(size, "cpu")] = h
        _H.setdefault((1, "cpu"), torch.ones(1, 1))
    if device is None:
        return _H[(n, "cpu")]
    key = (n, str(device))
    if key not in _H:
        _H[key] = _H[(n, "cpu")].to(device)
    return _H[key]


def fwht128(x: torch.Tensor, in_f_padded: Optional[int] = None, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """Native rotation of a CUDA tensor (..., in_f): zero-pads the last dimension to
    ``in_f_padded`` (default: next multiple of 128) inside the kernel."""
    from . import _native as nv
    dev = nv.require_cuda(x)
    in_f = x.shape[-1]
    kp = in_f_padded if in_f_padded is not None else (in_f + 127) // 128 * 128
    x2 = x.reshape(-1, in_f)
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    out = torch.empty(x2.shape[0], kp, dtype=out_dtype, device=dev)
    if x2.shape[0]:
        nv.check(nv.lib().pe_fwht128(x2.data_ptr(), nv.dtype_code(x2), x2.stride(0), out.data_ptr(),
                                     nv.dtype_code(out), out.stride(0), x2.shape[0], in_f, kp, nv.stream_ptr(dev)),
                 "pe_fwht128")
    return out.reshape(*x.shape[:-1], kp)


def fwht_matmul(x: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """Rotate every ``block_size`` block of the last dimension; same shape and dtype."""
    k = x.shape[-1]
    assert k % block_size == 0, f"in_features ({k}) must be divisible by block_size ({block_size})"
    if x.is_cuda and block_size == 128 and x.dtype in (torch.float32, torch.float16, torch.bfloat16):
        return fwht128(x, k, x.dtype)
    h = build_hadamard(block_size, x.device).to(x.dtype)
    return (x.reshape(-1, block_size) @ h).reshape(x.shape)


def fwht_butterfly(x: torch.Tensor) -> torch.Tensor:
    """Slow cross-check: log2(n) add/subtract stages over the last dimension, then
    1/sqrt(n)."""
    n = x.shape[-1]
    assert n >= 1 and (n & (n - 1)) == 0, f"last dimension must be a power of 2, got {n}"
    y = x.reshape(-1, n).clone()
    h = 1
    while h < n:
        y = y.view(-1, n // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], 2).reshape(-1, n)
        h *= 2
    return (y / math.sqrt(n)).reshape(x.shape)


class FWHTCache:
    """Single-entry memo of the last rotation, keyed by (storage pointer, in_features),
    so projections that read the same hidden state rotate it once."""

    def __init__(self) -> None:
        self.clear()

    def get(self, x: torch.Tensor, in_f: int) -> Optional[torch.Tensor]:
        return self._value if (x.data_ptr(), in_f) == self._key else None

    def put(self, x: torch.Tensor, in_f: int, result: torch.Tensor) -> None:
        self._key, self._value = (x.data_ptr(), in_f), result

    def clear(self) -> None:
        self._key, self._value = (-1, -1), None
