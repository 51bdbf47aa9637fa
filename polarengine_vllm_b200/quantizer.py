"""Offline producer of the kernels' inputs (reference: polarengine_vllm/quantizer.py:178-257).

The codes a checkpoint carries depend on floating-point summation order, so
``quantize_tensor`` performs the reference's torch operations in the reference's
order (pad, block norm clamped at 1e-10, normalise, 64-row chunks of
``(u @ H) * sqrt(block)``, first-minimum argmin of |r - c|).  On the CPU this
reproduces reference checkpoints bit for bit.
"""
from __future__ import annotations

import math
from typing import Dict, Mapping, Optional

import torch
import torch.nn.functional as F

from .fwht import build_hadamard
from .utils import DEFAULT_BIT_ASSIGNMENT, get_bits_for_layer, get_centroids, get_ct_scaled
from .packing import pack_codes_half_block, pack_codes_q5


class PolarQuantizer:
    def __init__(self, block_size: int = 128, bit_assignment: Optional[Mapping[str, int]] = None) -> None:
        self.block_size = block_size
        self.bit_assignment = dict(bit_assignment or DEFAULT_BIT_ASSIGNMENT)

    def quantize_tensor(self, weight: torch.Tensor, bits: int) -> Dict[str, torch.Tensor]:
        """(out_f, in_f) float -> codes int8 (out_f, in_f_padded), norms fp16
        (out_f, n_blocks), ct_scaled fp32 (2**bits)."""
        bs = self.block_size
        dev = weight.device
        levels = get_centroids(bits).to(dev)
        had = build_hadamard(bs, dev)
        rows, cols = weight.shape
        padded = -(-cols // bs) * bs
        nblk = padded // bs
        w = weight.detach().float()
        if padded != cols:
            w = F.pad(w, (0, padded - cols))
        blocks = w.view(rows, nblk, bs)
        norms = blocks.norm(dim=2).clamp(min=1e-10)
        unit = blocks / norms.unsqueeze(2)
        codes = torch.empty(rows, nblk, bs, dtype=torch.int8, device=dev)
        root = math.sqrt(bs)
        lv = levels.view(1, 1, 1, -1)
        for lo in range(0, rows, 64):
            hi = min(lo + 64, rows)
            rot = ((unit[lo:hi].reshape(-1, bs) @ had) * root).view(hi - lo, nblk, bs)
            codes[lo:hi] = (rot.unsqueeze(-1) - lv).abs().argmin(dim=-1).to(torch.int8)
        return {"codes": codes.reshape(rows, padded), "norms": norms.half(), "ct_scaled": levels / root}

    def quantize_tensor_gpu(self, weight: torch.Tensor, bits: int) -> Dict[str, torch.Tensor]:
        """:meth:`quantize_tensor` as one native launch (``pe_quantize``) for a CUDA tensor: same outputs, seconds
        instead of minutes for a whole model.  Summation orders differ from the CPU path, so codes that sit on a
        cell boundary can differ (measured: a few per million); checkpoints that must match the reference bit for
        bit are made with :meth:`quantize_tensor` on the CPU."""
        from . import _native as nv
        if self.block_size != 128:
            raise ValueError("the native quantizer supports block_size 128 only")
        dev = nv.require_cuda(weight)
        nv.ensure_init(dev)
        w = weight.detach()
        if w.dtype not in (torch.float32, torch.float16, torch.bfloat16):
            w = w.float()
        if w.stride(1) != 1:
            w = w.contiguous()
        rows, cols = w.shape
        padded = -(-cols // 128) * 128
        levels = get_centroids(bits).to(dev)
        codes = torch.empty(rows, padded, dtype=torch.int8, device=dev)
        norms = torch.empty(rows, padded // 128, dtype=torch.float16, device=dev)
        nv.check(nv.lib().pe_quantize(w.data_ptr(), nv.dtype_code(w), w.stride(0), rows, cols, padded, levels.data_ptr(),
                                      levels.numel(), codes.data_ptr(), codes.stride(0), norms.data_ptr(), norms.stride(0),
                                      nv.stream_ptr(dev)), "pe_quantize")
        return {"codes": codes, "norms": norms, "ct_scaled": get_ct_scaled(bits, 128).to(dev)}  # table divided on the host, as the CPU path has it

    def quantize_state_dict(self, state: Mapping[str, torch.Tensor], pack: bool = True):
        """Quantize every eligible 2-D ``*.weight``; returns (tensors, polar_config dict)
        in the on-disk naming of quantizer.py:341-403."""
        out: Dict[str, torch.Tensor] = {}
        layers: Dict[str, dict] = {}
        any_q5 = False
        for name, t in state.items():
            bits = get_bits_for_layer(name, t, self.bit_assignment)
            if bits == 16 or t.ndim != 2 or not name.endswith(".weight"):
                out[name] = t.half() if t.is_floating_point() else t
                continue
            q = self.quantize_tensor(t, bits)
            prefix = name[: -len(".weight")]
            codes, is_packed, q5 = q["codes"], False, False
            if pack and bits <= 4:
                codes, is_packed = pack_codes_half_block(codes, self.block_size), True
            elif pack and bits == 5:
                codes, q5, any_q5 = pack_codes_q5(codes, self.block_size), True, True
            out[prefix + ".codes"], out[prefix + ".norms"], out[prefix + ".ct_scaled"] = codes, q["norms"], q["ct_scaled"]
            meta = {"in_features": t.shape[1], "out_features": t.shape[0],
                    "in_features_padded": q["codes"].shape[1], "n_blocks": q["codes"].shape[1] // self.block_size,
                    "bits": bits, "block_size": self.block_size, "packed": is_packed, "scale_dtype": "float16"}
            if q5:
                meta["packed_q5"] = True
            layers[prefix] = meta
        cfg = {"format": "polar_engine_v5" if any_q5 else "polar_engine_v4", "quantization": "polarengine",
               "block_size": self.block_size, "bit_assignment": self.bit_assignment, "layers": layers}
        return out, cfg


def save_checkpoint(tensors: Mapping[str, torch.Tensor], polar_config: dict, output_dir: str,
                    max_shard_bytes: int = 5 * 1024 ** 3) -> Dict[str, str]:
    """Write the output of :meth:`PolarQuantizer.quantize_state_dict` the way the reference's
    ``quantize_model`` does (quantizer.py:85-137, 386-403): safetensors shards of at most
    ``max_shard_bytes`` named ``model-0000i-of-0000n.safetensors`` filled in insertion order,
    ``model.safetensors.index.json`` (total size + weight map) and ``polar_config.json``.
    Returns the weight map."""
    import json
    import os
    from safetensors.torch import save_file
    os.makedirs(output_dir, exist_ok=True)
    shards, current, used = [], {}, 0
    for name, t in tensors.items():
        nbytes = t.numel() * t.element_size()
        if current and used + nbytes > max_shard_bytes:
            shards.append(current)
            current, used = {}, 0
        current[name] = t.contiguous()
        used += nbytes
    if current:
        shards.append(current)
    weight_map: Dict[str, str] = {}
    for i, shard in enumerate(shards):
        fname = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file(shard, os.path.join(output_dir, fname))
        weight_map.update({k: fname for k in shard})
    with open(os.path.join(output_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": sum(t.numel() * t.element_size() for t in tensors.values())},
                   "weight_map": weight_map}, f, indent=2)
    with open(os.path.join(output_dir, "polar_config.json"), "w") as f:
        json.dump(polar_config, f, indent=2)
    return weight_map
