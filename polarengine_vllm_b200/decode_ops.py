"""Glue ops of a decoder layer (residual add + RMSNorm, rotary + KV-cache write, SiLU * up)
as single native launches.  The reference leaves these to vLLM; they are used by the
measurement decoder (``decoder.QuantDecoder``) so that a decode step is a short chain of
kernels around the quantized projections."""
from __future__ import annotations

from typing import Optional, Union

import torch

from . import _native as nv


def add_rmsnorm(x: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x`` (rows, hidden) fp16 is updated in place with ``x += delta.half()`` (if delta is
    given, fp16 or fp32); returns ``(x.float() * rsqrt(mean(x^2) + eps)).half() * weight``."""
    dev = nv.require_cuda(x, weight)
    if x.dtype != torch.float16 or weight.dtype != torch.float16 or not x.is_contiguous():
        raise ValueError("add_rmsnorm wants a contiguous fp16 residual stream and fp16 weights")
    rows, hidden = x.shape
    if delta is not None:
        if delta.shape != x.shape or not delta.is_contiguous() or delta.dtype not in (torch.float16, torch.float32):
            raise ValueError("delta must match x (contiguous, fp16 or fp32)")
    out = torch.empty_like(x)
    nv.check(nv.lib().pe_add_rmsnorm(x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                     nv.dtype_code(delta) if delta is not None else nv.PE_F16, weight.data_ptr(),
                                     out.data_ptr(), rows, hidden, float(eps), nv.stream_ptr(dev)), "pe_add_rmsnorm")
    return out


def rope_cache(qkv: torch.Tensor, pos0: Union[int, torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor, batch: int,
               t: int, hq: int, hkv: int, head_dim: int, theta: float) -> torch.Tensor:
    """qkv (batch*t, (hq + 2 hkv) * head_dim) fp16 -> rotated queries (batch, hq, t, head_dim);
    rotated keys and values are written into the caches (batch, hkv, max_len, head_dim) at
    positions pos0 .. pos0 + t - 1.  ``pos0`` is an int or a 0-d int64 device tensor."""
    dev = nv.require_cuda(qkv, k_cache, v_cache)
    if qkv.dtype != torch.float16 or qkv.stride(1) != 1 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise ValueError("rope_cache wants fp16 qkv rows and contiguous caches")
    q = torch.empty(batch, hq, t, head_dim, dtype=torch.float16, device=dev)
    dev_pos = pos0 if torch.is_tensor(pos0) else None
    if dev_pos is not None and (dev_pos.dtype != torch.int64 or dev_pos.device != dev):
        raise ValueError("a device position must be an int64 tensor on the same device")
    nv.check(nv.lib().pe_rope_cache(qkv.data_ptr(), qkv.stride(0), dev_pos.data_ptr() if dev_pos is not None else None,
                                    0 if dev_pos is not None else int(pos0), q.data_ptr(), k_cache.data_ptr(),
                                    v_cache.data_ptr(), batch, t, hq, hkv, head_dim, k_cache.shape[2], float(theta),
                                    nv.stream_ptr(dev)), "pe_rope_cache")
    return q


def silu_mul(gate_up: torch.Tensor, inter: int) -> torch.Tensor:
    """(rows, 2*inter) fp16 -> silu(gate_up[:, :inter]) * gate_up[:, inter:]."""
    dev = nv.require_cuda(gate_up)
    if gate_up.dtype != torch.float16 or gate_up.stride(1) != 1:
        raise ValueError("silu_mul wants fp16 rows")
    out = torch.empty(gate_up.shape[0], inter, dtype=torch.float16, device=dev)
    nv.check(nv.lib().pe_silu_mul(gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), out.stride(0), gate_up.shape[0],
                                  inter, nv.stream_ptr(dev)), "pe_silu_mul")
    return out


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, pos: Union[int, torch.Tensor]) -> torch.Tensor:
    """One new token per sequence: q (batch, hq, 1, head_dim) against the cache positions
    0 .. pos (the token written last).  Returns (batch, hq * head_dim) fp16."""
    dev = nv.require_cuda(q, k_cache, v_cache)
    batch, hq, t, d = q.shape
    if t != 1 or q.dtype != torch.float16 or not q.is_contiguous():
        raise ValueError("decode_attention wants contiguous fp16 queries of one token per sequence")
    hkv, max_len = k_cache.shape[1], k_cache.shape[2]
    out = torch.empty(batch, hq * d, dtype=torch.float16, device=dev)
    dev_pos = pos if torch.is_tensor(pos) else None
    need = nv.lib().pe_decode_attention_workspace_bytes(batch, hq, hkv, d)
    ws = _attention_scratch(dev, need) if need else None
    nv.check(nv.lib().pe_decode_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                          dev_pos.data_ptr() if dev_pos is not None else None,
                                          0 if dev_pos is not None else int(pos), out.data_ptr(), batch, hq, hkv, d, max_len,
                                          ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                          nv.stream_ptr(dev)), "pe_decode_attention")
    return out


def rope_attention(qkv: torch.Tensor, pos: Union[int, torch.Tensor], k_cache: torch.Tensor, v_cache: torch.Tensor, hq: int, hkv: int,
                   head_dim: int, theta: float) -> torch.Tensor:
    """One new token per sequence, rotary embedding + KV-cache write + attention in one launch: qkv (batch,
    (hq + 2 hkv) * head_dim) fp16 is the raw fused projection; returns (batch, hq * head_dim) fp16 and leaves the
    rotated key and the value in the caches at ``pos``."""
    dev = nv.require_cuda(qkv, k_cache, v_cache)
    if qkv.dtype != torch.float16 or qkv.stride(1) != 1 or not k_cache.is_contiguous() or not v_cache.is_contiguous():
        raise ValueError("rope_attention wants fp16 qkv rows and contiguous caches")
    batch, max_len = qkv.shape[0], k_cache.shape[2]
    out = torch.empty(batch, hq * head_dim, dtype=torch.float16, device=dev)
    dev_pos = pos if torch.is_tensor(pos) else None
    need = nv.lib().pe_decode_attention_workspace_bytes(batch, hq, hkv, head_dim)
    ws = _attention_scratch(dev, need) if need else None
    nv.check(nv.lib().pe_rope_attention(qkv.data_ptr(), qkv.stride(0), dev_pos.data_ptr() if dev_pos is not None else None,
                                        0 if dev_pos is not None else int(pos), k_cache.data_ptr(), v_cache.data_ptr(),
                                        out.data_ptr(), batch, hq, hkv, head_dim, max_len, float(theta),
                                        ws.data_ptr() if ws is not None else None, ws.numel() if ws is not None else 0,
                                        nv.stream_ptr(dev)), "pe_rope_attention")
    return out


_att_ws = {}


def _attention_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch of the split attention, one per (device, stream); the kernel leaves its
    ticket counters at zero, so consecutive calls on a stream share it."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _att_ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _att_ws[key] = buf
    return buf
