"""On-disk / in-memory code layouts (reference: polarengine_vllm/packing.py).

* half-block nibbles for widths <= 4 (packing.py:22-94)
* "v5" 5-bit, least-significant-bit first, 8 codes in 5 bytes (packing.py:97-209)
* HLWQ 5-bit, most-significant-bit first (packing.py:229-290)
* ``pack_model_codes`` packs every eligible layer of a module tree (packing.py:293-364)

Tensors on a CUDA device are nibble-packed by the native kernel; CPU tensors (offline
tooling, checkpoint writing) by plain tensor arithmetic.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from . import utils


def pack_codes_half_block(codes: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """(out_f, K) int8 codes in 0..15 -> (out_f, K/2) uint8."""
    assert block_size % 2 == 0, f"block_size must be even, got {block_size}"
    assert codes.dim() == 2 and codes.shape[1] % block_size == 0, (
        f"in_f_padded ({codes.shape[-1]}) must be a multiple of block_size ({block_size})")
    if codes.is_cuda and block_size == 128 and codes.dtype in (torch.int8, torch.uint8):
        from . import _native as nv
        src = codes.contiguous()
        out = torch.empty(src.shape[0], src.shape[1] // 2, dtype=torch.uint8, device=src.device)
        nv.check(nv.lib().pe_pack_nibble(src.data_ptr(), out.data_ptr(), src.shape[0], src.shape[1],
                                         nv.stream_ptr(src.device)), "pe_pack_nibble")
        return out
    as_u8 = codes.to(torch.uint8)
    assert bool((as_u8 <= 15).all()), f"codes must be in [0, 15] for nibble packing, max={int(as_u8.max())}"
    return utils.pack_codes_half_block(as_u8, block_size)


def unpack_codes_half_block(packed: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    assert block_size % 2 == 0
    assert packed.shape[-1] % (block_size // 2) == 0, "packed width must be a whole number of half blocks"
    return utils.unpack_codes_half_block(packed, block_size)


def _groups(t: torch.Tensor, n: int):
    g = t.to(torch.long).reshape(*t.shape[:-1], t.shape[-1] // n, n)
    return [g[..., i] for i in range(n)]


def pack_codes_q5(codes: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    """5-bit codes, LSB first: bit 5*i+j of each 40-bit group is bit j of code i."""
    assert block_size % 8 == 0
    k = codes.shape[-1]
    assert k % block_size == 0, f"Last dimension ({k}) must be a multiple of block_size ({block_size})"
    c = _groups(codes.to(torch.long) & 0xFF, 8)
    assert all(bool((x <= 31).all()) for x in c), "codes must be in [0, 31] for Q5 packing"
    word = sum(c[i] << (5 * i) for i in range(8))
    out = torch.stack([(word >> (8 * j)) & 0xFF for j in range(5)], -1).to(torch.uint8)
    return out.reshape(*codes.shape[:-1], k * 5 // 8)


def unpack_codes_q5(packed: torch.Tensor, block_size: int = 128) -> torch.Tensor:
    kp = packed.shape[-1]
    assert kp % (block_size * 5 // 8) == 0, "packed width must be a whole number of 5-bit blocks"
    b = _groups(packed, 5)
    word = sum(b[j] << (8 * j) for j in range(5))
    out = torch.stack([(word >> (5 * i)) & 31 for i in range(8)], -1).to(torch.int8)
    return out.reshape(*packed.shape[:-1], kp * 8 // 5)


def pack_codes_q5_hlwq(codes: torch.Tensor) -> torch.Tensor:
    """5-bit codes, MSB first: code 0 occupies the top five bits of byte 0."""
    k = codes.shape[-1]
    if k % 8:
        codes = torch.nn.functional.pad(codes, (0, 8 - k % 8))
    c = _groups(codes, 8)
    word = sum(c[i] << (5 * (7 - i)) for i in range(8))
    out = torch.stack([(word >> (8 * (4 - j))) & 0xFF for j in range(5)], -1).to(torch.uint8)
    return out.reshape(*codes.shape[:-1], -1)


def unpack_codes_q5_hlwq(packed: torch.Tensor, total: Optional[int] = None) -> torch.Tensor:
    assert packed.shape[-1] % 5 == 0, f"HLWQ bit-packed codes need a multiple of 5 bytes, got {packed.shape[-1]}"
    b = _groups(packed, 5)
    word = sum(b[j] << (8 * (4 - j)) for j in range(5))
    out = torch.stack([(word >> (5 * (7 - i))) & 31 for i in range(8)], -1).to(torch.int8)
    out = out.reshape(*packed.shape[:-1], -1)
    return out if total is None else out[..., :total]


def verify_packing_roundtrip(codes: torch.Tensor, block_size: int = 128) -> bool:
    return bool(torch.equal(unpack_codes_half_block(pack_codes_half_block(codes, block_size), block_size),
                            codes.to(torch.int8)))


def verify_q5_roundtrip(codes: torch.Tensor, block_size: int = 128) -> bool:
    return bool(torch.equal(unpack_codes_q5(pack_codes_q5(codes, block_size), block_size), codes.to(torch.int8)))


def pack_model_codes(model: Any, block_size: int = 128) -> Dict[str, Any]:
    """Nibble-pack, in place, every sub-module that has ``bits <= 4`` and a ``codes``
    buffer; returns counts and byte totals."""
    stats = {"layers_packed": 0, "layers_skipped": 0, "bytes_before": 0, "bytes_after": 0}
    for _, mod in model.named_modules():
        codes = getattr(mod, "codes", None)
        bits = getattr(mod, "bits", None)
        if codes is None or bits is None:
            continue
        if bits > 4 or getattr(mod, "packed", False):
            stats["layers_skipped"] += 1
            continue
        packed = pack_codes_half_block(codes, block_size)
        stats["bytes_before"] += codes.numel() * codes.element_size()
        stats["bytes_after"] += packed.numel()
        if "codes" in getattr(mod, "_buffers", {}):
            del mod._buffers["codes"]
        elif hasattr(mod, "codes"):
            delattr(mod, "codes")
        if hasattr(mod, "register_buffer"):
            mod.register_buffer("codes_packed", packed)
        else:
            mod.codes_packed = packed
        mod.in_f_half = packed.shape[1]
        mod.packed = True
        stats["layers_packed"] += 1
    saved = stats["bytes_before"] - stats["bytes_after"]
    stats["bytes_saved"] = saved
    stats["savings_pct"] = 100.0 * saved / stats["bytes_before"] if stats["bytes_before"] else 0.0
    return stats
