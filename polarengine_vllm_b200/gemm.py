"""Prefill-size path: thin wrapper over ``pe_gemm`` (tcgen05 tensor-core kernel)."""
from __future__ import annotations

from typing import Optional

import torch

from . import _native as nv


def quant_gemm(codes: torch.Tensor, packed: bool, norms: torch.Tensor, ct: torch.Tensor, x: torch.Tensor, rotated: bool,
               out_f: int, in_f: int, in_f_padded: int, y: torch.Tensor, bias: Optional[torch.Tensor] = None,
               check_status: bool = False) -> torch.Tensor:
    """Fill ``y`` (m, out_f) from x (m, in_f | in_f_padded).  Arguments are already
    normalised by ``kernels.quant_matmul`` (contiguous rows, fp16 norms, fp32 table)."""
    dev = x.device
    l = nv.lib()
    m = x.shape[0]
    ws = nv.gemm_workspace(dev, l.pe_gemm_workspace_bytes_splitk(m, out_f, in_f_padded))
    nv.check(l.pe_gemm(codes.data_ptr(), int(packed), codes.stride(0) * codes.element_size(), norms.data_ptr(),
                       norms.stride(0), ct.data_ptr(), ct.numel(), x.data_ptr(),
                       nv.PE_X_ROTATED if rotated else nv.PE_X_RAW, nv.dtype_code(x), x.stride(0), in_f, y.data_ptr(),
                       nv.dtype_code(y), y.stride(0), bias.data_ptr() if bias is not None else None, m, out_f,
                       in_f_padded, ws.data_ptr(), ws.numel(), nv.stream_ptr(dev)), "pe_gemm")
    if check_status:
        code = int(ws[:4].view(torch.int32).item())
        if code:
            raise RuntimeError(f"pe_gemm: device-side wait {code} timed out")
    return y
