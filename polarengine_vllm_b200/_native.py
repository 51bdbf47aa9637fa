"""ctypes binding of libpolar_b200.so (the C ABI declared in include/polar_b200.h).

There is no fallback: if the shared library is missing or a call returns an error
code, a RuntimeError is raised.  Pointers are taken from torch tensors; torch only
supplies device memory and the current stream.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_LIB_NAME = "libpolar_b200.so"
_lib: Optional[ctypes.CDLL] = None

PE_F32, PE_F16, PE_BF16 = 0, 1, 2
PE_X_ROTATED, PE_X_RAW = 0, 1
PE_PRO_ADD_RMSNORM, PE_PRO_SILU_MUL = 1, 2

_DTYPE = {torch.float32: PE_F32, torch.float16: PE_F16, torch.bfloat16: PE_BF16}

# name -> (restype, argtypes); also the list of symbols the header declares
_vp, _i, _i64, _sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_size_t
SIGNATURES = {
    "pe_version": (_i, []),
    "pe_error_string": (ctypes.c_char_p, [_i]),
    "pe_last_cuda_error": (_i, []),
    "pe_init": (_i, [_i]),
    "pe_set_wait_limit_us": (_i, [_i64]),
    "pe_fwht128": (_i, [_vp, _i, _i64, _vp, _i, _i64, _i, _i, _i, _vp]),
    "pe_embedding": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _i, _vp, _i64, _vp, _i, _i64, _i, _i, _i, _vp]),
    "pe_quantize": (_i, [_vp, _i, _i64, _i64, _i, _i, _vp, _i, _vp, _i64, _vp, _i64, _vp]),
    "pe_pack_nibble": (_i, [_vp, _vp, _i64, _i64, _vp]),
    "pe_gemv_workspace_bytes": (_sz, [_i, _i, _i]),
    "pe_gemv": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _i, _vp, _i, _i, _i64, _i, _vp, _i, _i64, _vp, _i, _i, _i,
                     _vp, _sz, _vp]),
    "pe_gemv_grouped_workspace_bytes": (_sz, [_i, _i, _i]),
    "pe_gemv_grouped": (_i, [_vp, _i, _i64, _i64, _vp, _i64, _i64, _vp, _i, _vp, _i, _i, _i64, _i, _vp, _vp, _i, _i64, _vp,
                            _i, _i, _i, _i, _vp, _sz, _vp]),
    "pe_moe_route": (_i, [_vp, _i, _i64, _i, _i, _i, _i, _vp, _vp, _vp]),
    "pe_moe_plan": (_i, [_vp, _vp, _i, _i, _i, _i, _i, _i, _vp, _vp, _vp, _vp, _vp]),
    "pe_gemm_grouped_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "pe_gemm_grouped": (_i, [_vp, _i, _i64, _i64, _vp, _i64, _i64, _vp, _i, _vp, _i, _i, _i64, _i, _vp, _vp, _i, _i64, _vp,
                            _i, _i, _i, _i, _vp, _sz, _vp]),
    "pe_moe_combine": (_i, [_vp, _i64, _vp, _vp, _i, _i, _vp, _i, _i64, _i, _vp]),
    "pe_allreduce_buffer_bytes": (_sz, [_i, _i, _i]),
    "pe_allreduce_add_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, ctypes.c_float, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "pe_retile_bytes": (_sz, [_i, _i64, _i64]),
    "pe_retile": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _i64, _i64, _vp]),
    "pe_gemv_tiled": (_i, [_vp, _i, _vp, _i, _vp, _i, _i, _i64, _i, _vp, _i, _i64, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "pe_gemm_workspace_bytes": (_sz, [_i, _i]),
    "pe_gemm_workspace_bytes_splitk": (_sz, [_i, _i, _i]),
    "pe_gemm": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _i, _vp, _i, _i, _i64, _i, _vp, _i, _i64, _vp, _i, _i, _i,
                     _vp, _sz, _vp]),
    "pe_add_rmsnorm": (_i, [_vp, _vp, _i, _vp, _vp, _i, _i, ctypes.c_float, _vp]),
    "pe_rope_cache": (_i, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, ctypes.c_float, _vp]),
    "pe_silu_mul": (_i, [_vp, _i64, _vp, _i64, _i, _i, _vp]),
    "pe_decode_attention_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "pe_decode_attention": (_i, [_vp, _vp, _vp, _vp, _i64, _vp, _i, _i, _i, _i, _i, _vp, _sz, _vp]),
    "pe_gemv_pro": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _i, _i, _vp, _i, _vp, _i, _vp, _vp, ctypes.c_float, _vp, _i, _vp, _i, _i, _vp]),
    "pe_gemv_status": (_i, [_vp, _sz, _i, _vp]),
    "pe_gemv_small_batch_takes": (_i, [_i, _i64, _vp, _i64, _i, _i]),
    "pe_gemv_noalloc_status": (_i, [_i, _vp]),
    "pe_rope_attention": (_i, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i, _i, _i, _i, _i, ctypes.c_float, _vp, _sz, _vp]),
    "pe_gemv_noalloc_max_bytes": (_sz, []),
    "pe_gemv_noalloc": (_i, [_vp, _i, _i64, _vp, _i64, _vp, _i, _vp, _i, _i, _i64, _i, _vp, _i, _i64, _vp, _i, _i, _i,
                             _vp]),
}


def library_path() -> str:
    """The in-tree build, or the file POLAR_B200_LIB names (a supported way to load a build kept elsewhere,
    e.g. one compiled with other flags for an A/B comparison)."""
    return os.environ.get("POLAR_B200_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), _LIB_NAME)


def lib() -> ctypes.CDLL:
    """Load the shared library once; fail loudly when it has not been built."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise RuntimeError(
                f"{path} not found: build it with `make -C polarengine_vllm_b200/csrc` "
                "(or __graft_entry__.build()); this package has no CPU or Triton fallback")
        handle = ctypes.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        l = lib()
        msg = l.pe_error_string(code).decode()
        extra = f" (cudaError {l.pe_last_cuda_error()})" if code == -5 else ""
        raise RuntimeError(f"{what} failed: {msg}{extra}")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}; expected float32, float16 or bfloat16") from None


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if t is not None and (not t.is_cuda or t.device != dev):
            raise RuntimeError("polarengine_vllm_b200 kernels need CUDA tensors on one device (no CPU path)")
    return dev


_inited = set()


def ensure_init(device: torch.device) -> None:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _inited:
        check(lib().pe_init(idx), "pe_init")
        _inited.add(idx)


# one scratch buffer per (device, stream); zero-filled once, kernels leave it zeroed
_scratch = {}


def gemv_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 22), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


_grouped_scratch = {}


def grouped_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    """Scratch of the grouped launches (its own buffer: the counter zone differs from pe_gemv's)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _grouped_scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 8 << 20), dtype=torch.uint8, device=device)
        _grouped_scratch[key] = buf
    return buf


_gemm_ws = {}


def gemm_workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Grow-only per-(device, stream) buffer for pe_gemm (status word + bf16 activations)."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _gemm_ws.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes + (nbytes >> 2), dtype=torch.uint8, device=device)
        _gemm_ws[key] = buf
    return buf
