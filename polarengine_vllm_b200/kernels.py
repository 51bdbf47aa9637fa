"""Python face of the native matmul kernels, under the reference's function names.

Reference: polarengine_vllm/kernels/polar_gemm.py:425-534 (``polar_matmul``),
polar_gemv.py:181-283 (``polar_gemv``, ``polar_gemv_packed``, ``pack_codes_int4``),
polar_gemv_splitk.py:421-569, polar_gemm.py:312-418.  Argument order and meaning are
kept; every one of them ends in the same native entry point, which chooses its own
split of the K range, so the split-K names are aliases.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _native as nv
from .packing import pack_codes_half_block

GEMV_MAX_BATCH = 16


def pack_codes_int4(codes: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    return pack_codes_half_block(codes, block_size)


def retile(codes: torch.Tensor, packed: bool, norms: torch.Tensor) -> torch.Tensor:
    """Layer in the decode kernel's tiled layout (``pe_retile``): a flat uint8 buffer."""
    dev = nv.require_cuda(codes, norms)
    out_f = codes.shape[0]
    kp = norms.shape[-1] * 128
    if norms.dtype != torch.float16 or norms.stride(-1) != 1:
        norms = norms.to(torch.float16).contiguous()
    if codes.stride(-1) != 1:
        codes = codes.contiguous()
    l = nv.lib()
    out = torch.empty(l.pe_retile_bytes(int(packed), out_f, kp), dtype=torch.uint8, device=dev)
    nv.check(l.pe_retile(codes.data_ptr(), int(packed), codes.stride(0) * codes.element_size(), norms.data_ptr(),
                         norms.stride(0), out.data_ptr(), out_f, kp, nv.stream_ptr(dev)), "pe_retile")
    return out


SMALL_BATCH_MAX = 8


def small_batch_takes(codes: torch.Tensor, packed: bool, norms: torch.Tensor, out_f: int, in_f_padded: int) -> bool:
    """True if batches of 3..8 rows of this layer run on the row-major arrays (column-owner tensor-core kernel):
    such batches need no tiled copy of the layer."""
    return bool(nv.lib().pe_gemv_small_batch_takes(int(packed), codes.stride(0) * codes.element_size(), norms.data_ptr(),
                                                   norms.stride(0), out_f, in_f_padded))


def quant_matmul(codes: torch.Tensor, packed: bool, norms: torch.Tensor, ct_scaled: torch.Tensor, x: torch.Tensor,
                 rotated: bool, out_f: int, in_f: int, in_f_padded: int, out_dtype: torch.dtype = torch.float32,
                 bias: Optional[torch.Tensor] = None, tiles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y (batch, out_f) for x (batch, in_f or in_f_padded); the single entry to the
    native kernels used by everything else in the package.  ``tiles`` (from
    :func:`retile`) lets batches of 3..16 rows stream the tiled copy of the layer; one or
    two rows, and 3..8 rows of the layers :func:`small_batch_takes` accepts, read the row-major arrays (whole
    weight rows per CTA, no scratch traffic)."""
    dev = nv.require_cuda(codes, norms, ct_scaled, x)
    nv.ensure_init(dev)
    if x.dim() != 2 or x.stride(1) != 1:
        x = x.reshape(-1, x.shape[-1]).contiguous()
    if norms.dtype != torch.float16:
        norms = norms.to(torch.float16)
    norms = norms.reshape(out_f, -1)
    if norms.stride(1) != 1:
        norms = norms.contiguous()
    if codes.stride(-1) != 1:
        codes = codes.contiguous()
    ct = ct_scaled if ct_scaled.dtype == torch.float32 else ct_scaled.float()
    if bias is not None and (bias.dtype != torch.float16 or not bias.is_contiguous()):
        bias = bias.to(torch.float16).contiguous()
    batch = x.shape[0]
    y = torch.empty(batch, out_f, dtype=out_dtype, device=dev)
    if batch == 0:
        return y
    l = nv.lib()
    st = nv.stream_ptr(dev)
    if batch <= GEMV_MAX_BATCH:
        need = l.pe_gemv_workspace_bytes(min(batch, GEMV_MAX_BATCH), out_f, in_f_padded)
        ws = nv.gemv_scratch(dev, need)
        for m0 in range(0, batch, GEMV_MAX_BATCH):
            m1 = min(batch, m0 + GEMV_MAX_BATCH)
            xs, ys = x[m0:m1], y[m0:m1]
            if tiles is not None and batch > 2 and not (batch <= SMALL_BATCH_MAX and small_batch_takes(codes, packed, norms, out_f, in_f_padded)):
                nv.check(l.pe_gemv_tiled(tiles.data_ptr(), int(packed), ct.data_ptr(), ct.numel(), xs.data_ptr(),
                                         nv.PE_X_ROTATED if rotated else nv.PE_X_RAW, nv.dtype_code(xs), xs.stride(0),
                                         in_f, ys.data_ptr(), nv.dtype_code(ys), ys.stride(0),
                                         bias.data_ptr() if bias is not None else None, m1 - m0, out_f, in_f_padded,
                                         ws.data_ptr(), ws.numel(), st), "pe_gemv_tiled")
                continue
            nv.check(l.pe_gemv(codes.data_ptr(), int(packed), codes.stride(0) * codes.element_size(),
                               norms.data_ptr(), norms.stride(0), ct.data_ptr(), ct.numel(),
                               xs.data_ptr(), nv.PE_X_ROTATED if rotated else nv.PE_X_RAW, nv.dtype_code(xs),
                               xs.stride(0), in_f, ys.data_ptr(), nv.dtype_code(ys), ys.stride(0),
                               bias.data_ptr() if bias is not None else None, m1 - m0, out_f, in_f_padded,
                               ws.data_ptr(), ws.numel(), st), "pe_gemv")
        return y
    from .gemm import quant_gemm
    return quant_gemm(codes, packed, norms, ct, x, rotated, out_f, in_f, in_f_padded, y, bias)


def quant_matmul_pro(codes: torch.Tensor, packed: bool, norms: torch.Tensor, ct_scaled: torch.Tensor, prologue: int,
                     x: torch.Tensor, in_f: int, out_f: int, in_f_padded: int, out_dtype: torch.dtype = torch.float16, *,
                     delta: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                     resid_out: Optional[torch.Tensor] = None, eps: float = 0.0,
                     bias: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """One-token matmul with the glue op in front of it folded into the launch (``pe_gemv_pro``).

    ``prologue`` = ``PE_PRO_ADD_RMSNORM``: ``x`` is the fp16 residual row (in_f), ``delta`` (fp16 / fp32, optional) is
    added to it, the sum goes to ``resid_out`` and its RMSNorm times ``norm_weight`` is the matmul input;
    ``PE_PRO_SILU_MUL``: ``x`` is ``[gate | up]`` (2 * in_f) and the input is ``silu(gate) * up``.
    Returns y (1, out_f), or None when the batch-1 kernel does not take the layer's shape (the caller then runs the
    glue op and :func:`quant_matmul`)."""
    dev = nv.require_cuda(codes, norms, ct_scaled, x)
    nv.ensure_init(dev)
    width = in_f if prologue == nv.PE_PRO_ADD_RMSNORM else 2 * in_f
    if x.dtype != torch.float16 or x.numel() != width or not x.is_contiguous():
        raise ValueError("the fused prologues take one contiguous fp16 activation row")
    for t in (delta, resid_out):
        if t is not None and (t.numel() != in_f or not t.is_contiguous()):
            raise ValueError("delta / resid_out must be contiguous rows of in_f elements")
    if resid_out is not None and (resid_out.dtype != torch.float16 or resid_out.data_ptr() == x.data_ptr()):
        raise ValueError("resid_out must be an fp16 row other than x")
    norms = norms.reshape(out_f, -1)
    y = torch.empty(1, out_f, dtype=out_dtype, device=dev)
    rc = nv.lib().pe_gemv_pro(codes.data_ptr(), int(packed), codes.stride(0) * codes.element_size(), norms.data_ptr(),
                              norms.stride(0), ct_scaled.data_ptr(), ct_scaled.numel(), prologue, x.data_ptr(), in_f,
                              delta.data_ptr() if delta is not None else None,
                              nv.dtype_code(delta) if delta is not None else nv.PE_F16,
                              norm_weight.data_ptr() if norm_weight is not None else None,
                              resid_out.data_ptr() if resid_out is not None else None, float(eps), y.data_ptr(),
                              nv.dtype_code(y), bias.data_ptr() if bias is not None else None, out_f, in_f_padded,
                              nv.stream_ptr(dev))
    if rc == -2:  # PE_ERR_SHAPE: not a layer of the batch-1 kernel
        return None
    nv.check(rc, "pe_gemv_pro")
    return y


def polar_matmul(codes: Optional[torch.Tensor], x_transformed: torch.Tensor, norms: torch.Tensor,
                 ct_scaled: torch.Tensor, out_f: int, in_f_padded: int, n_blocks: int, block_size: int = 128,
                 packed: bool = False, packed_codes: Optional[torch.Tensor] = None,
                 in_f_half: Optional[int] = None) -> torch.Tensor:
    """fp32 product of rotated activations with a quantized weight.  A 1-D input
    gives a 1-D output; a 2-D input keeps its batch dimension."""
    if block_size != 128:
        raise ValueError("block_size must be 128")
    use_packed = bool(packed and packed_codes is not None and in_f_half is not None)
    w = packed_codes if use_packed else codes
    if w is None:
        raise ValueError("codes (or packed_codes with packed=True) are required")
    x2 = x_transformed.reshape(1, -1) if x_transformed.dim() == 1 else x_transformed
    assert x2.shape[-1] == in_f_padded == n_blocks * block_size
    y = quant_matmul(w, use_packed, norms, ct_scaled, x2, True, out_f, in_f_padded, in_f_padded)
    return y.reshape(out_f) if x_transformed.dim() == 1 else y


def polar_gemv(codes, x_transformed, norms, ct_scaled, out_f, in_f_padded, n_blocks, block_size=128):
    return polar_matmul(codes, x_transformed.reshape(-1), norms, ct_scaled, out_f, in_f_padded, n_blocks, block_size)


def polar_gemv_packed(codes_packed, x_transformed, norms, ct_scaled, out_f, in_f_half, n_blocks, block_size=128):
    return polar_matmul(None, x_transformed.reshape(-1), norms, ct_scaled, out_f, 2 * in_f_half, n_blocks,
                        block_size, True, codes_packed, in_f_half)


def polar_gemm(codes, x_transformed, norms, ct_scaled, out_f, in_f_padded, n_blocks, block_size=128):
    return polar_matmul(codes, x_transformed.reshape(-1, in_f_padded), norms, ct_scaled, out_f, in_f_padded,
                        n_blocks, block_size)


def polar_gemm_packed(codes_packed, x_transformed, norms, ct_scaled, out_f, in_f_half, n_blocks, block_size=128):
    return polar_matmul(None, x_transformed.reshape(-1, 2 * in_f_half), norms, ct_scaled, out_f, 2 * in_f_half,
                        n_blocks, block_size, True, codes_packed, in_f_half)


polar_gemv_splitk = polar_gemv
polar_gemv_packed_splitk = polar_gemv_packed


def quant_embedding(codes: torch.Tensor, packed: bool, norms: torch.Tensor, ct_scaled: torch.Tensor, ids: torch.Tensor,
                    hidden: int, out_dtype: torch.dtype = torch.float16) -> torch.Tensor:
    """Rows ``ids`` of a quantized embedding table, dequantised on the fly: (*ids.shape, hidden)."""
    dev = nv.require_cuda(codes, norms, ct_scaled, ids)
    flat = ids.reshape(-1).to(torch.int64).contiguous()
    hp = norms.shape[-1] * 128
    out = torch.empty(flat.numel(), hidden, dtype=out_dtype, device=dev)
    if flat.numel():
        nv.check(nv.lib().pe_embedding(codes.data_ptr(), int(packed), codes.stride(0) * codes.element_size(), norms.data_ptr(),
                                       norms.stride(0), ct_scaled.data_ptr(), ct_scaled.numel(), flat.data_ptr(),
                                       codes.shape[0], out.data_ptr(), nv.dtype_code(out), out.stride(0), flat.numel(),
                                       hidden, hp, nv.stream_ptr(dev)), "pe_embedding")
    return out.reshape(*ids.shape, hidden)
