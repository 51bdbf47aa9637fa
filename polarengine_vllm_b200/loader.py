"""Checkpoint side of the plugin: PolarEngine safetensors -> the tensors the kernels read.

Reference: polarengine_vllm/loader.py:35-551 (``load_polar_config``, ``get_weight_map``,
``PolarWeightLoader``).  On-disk formats, unchanged:

* ``polar_engine_v4`` / ``polar_engine_v5``: per quantized layer ``<name>.codes`` (int8
  ``(N, K)``; uint8 half-block nibbles ``(N, K/2)`` when packed; uint8 ``(N, K*5/8)`` when
  the layer's entry in ``polar_config.json`` says ``packed_q5``), ``<name>.norms`` fp16
  ``(N, K/128)``, ``<name>.ct_scaled`` fp32 (or legacy ``<name>.ct``, scaled by
  1/sqrt(block) on load), optional ``<name>.bias``;
* ``hlwq-q5``: ``<name>.weight__packed`` (MSB-first 5-bit stream), ``.weight__norms``,
  ``.weight__meta`` = [out_f, n_blocks, block, total_codes(, in_f)]; the table is the
  canonical Lloyd-Max one.

What is added to the reference's behaviour: a layer can be loaded as a tensor-parallel
shard (rows for column-parallel, whole 128-blocks of K for row-parallel layers, the way
``parallel.shard_*`` cut them), and ``fill_linear`` writes the result into the parameters
``PolarQuantLinearMethod.create_weights`` registered.  The reference unpacks every ``hlwq-*``
format with the 5-bit routine (loader.py:333-364); here ``hlwq-q4`` / ``hlwq-q3`` are refused
instead of being decoded with the wrong width.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

from . import parallel
from .packing import unpack_codes_q5, unpack_codes_q5_hlwq
from .utils import get_centroids

KNOWN_FORMATS = ("polar_engine_v4", "polar_engine_v5", "hlwq-q5", "hlwq-q4", "hlwq-q3")
_SUFFIXES = (".codes", ".norms", ".ct_scaled", ".ct", ".weight__packed", ".weight__norms", ".weight__meta")


def load_polar_config(model_dir: str) -> dict:
    """``polar_config.json`` of a checkpoint directory (FileNotFoundError if absent)."""
    path = os.path.join(model_dir, "polar_config.json")
    with open(path) as f:
        cfg = json.load(f)
    if str(cfg.get("format", "unknown")).lower() not in KNOWN_FORMATS:
        import warnings
        warnings.warn(f"unrecognised PolarEngine format {cfg.get('format')!r}; treating it as polar_engine_v4")
    return cfg


def get_weight_map(model_dir: str) -> Dict[str, str]:
    """tensor key -> safetensors file, from ``model.safetensors.index.json`` when present,
    else by listing the keys of every ``*.safetensors`` file in the directory."""
    index = os.path.join(model_dir, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as f:
            return dict(json.load(f)["weight_map"])
    from safetensors import safe_open
    out: Dict[str, str] = {}
    for name in sorted(os.listdir(model_dir)):
        if name.endswith(".safetensors"):
            with safe_open(os.path.join(model_dir, name), framework="pt") as f:
                for key in f.keys():
                    out[key] = name
    if not out:
        raise FileNotFoundError(f"no safetensors files in {model_dir}")
    return out


class PolarCheckpoint:
    """Lazy reader of one checkpoint directory."""

    def __init__(self, model_dir: str, polar_config: Optional[dict] = None) -> None:
        self.model_dir = model_dir
        self.config = polar_config if polar_config is not None else load_polar_config(model_dir)
        self.weight_map = get_weight_map(model_dir)
        self.block_size = int(self.config.get("block_size", 128))
        self.format = str(self.config.get("format", "polar_engine_v4")).lower()
        self._files: Dict[str, object] = {}

    # ---- file handling
    def _file(self, name: str):
        from safetensors import safe_open
        if name not in self._files:
            self._files[name] = safe_open(os.path.join(self.model_dir, name), framework="pt")
        return self._files[name]

    def close(self) -> None:
        self._files.clear()

    def __enter__(self) -> "PolarCheckpoint":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def load_tensor(self, key: str) -> torch.Tensor:
        if key not in self.weight_map:
            raise KeyError(f"tensor {key!r} is not in the checkpoint")
        return self._file(self.weight_map[key]).get_tensor(key)

    # ---- layer metadata
    def layer_names(self) -> List[str]:
        """Base names of all quantized layers, sorted."""
        names = set()
        for key in self.weight_map:
            for suf in (".codes", ".weight__packed"):
                if key.endswith(suf):
                    names.add(key[: -len(suf)])
        return sorted(names)

    def is_quantized_layer(self, name: str) -> bool:
        return (name in self.config.get("layers", {}) or name + ".codes" in self.weight_map
                or name + ".weight__packed" in self.weight_map)

    def layer_bits(self, name: str) -> int:
        meta = self.config.get("layers", {}).get(name, {})
        if "bits" in meta:
            return int(meta["bits"])
        if self.format.startswith("hlwq-q"):
            return int(self.format[-1])
        for key in (name + ".ct_scaled", name + ".ct"):
            if key in self.weight_map:
                return int(round(math.log2(self.load_tensor(key).numel())))
        raise KeyError(f"cannot tell the bit width of {name!r}")

    # ---- loading
    def load_layer(self, name: str, tp_rank: int = 0, tp_size: int = 1, parallel_mode: Optional[str] = None) -> Dict[str, torch.Tensor]:
        """Tensors of one layer on the CPU.  Quantized: ``codes`` (int8 ``(N, K)``, or uint8
        nibbles ``(N, K/2)`` exactly as stored when the checkpoint packed them), ``norms`` fp16,
        ``ct_scaled`` fp32, ``packed`` (bool), ``in_f`` (true width when the file records it),
        optional ``bias``.  Otherwise ``weight`` (+ ``bias``).  ``parallel_mode`` "column" / "row"
        returns the rank's shard (bias of a row-parallel layer only on rank 0)."""
        if parallel_mode not in (None, "column", "row"):
            raise ValueError("parallel_mode must be None, 'column' or 'row'")
        out: Dict[str, torch.Tensor] = {}
        if not self.is_quantized_layer(name):
            key = name + ".weight" if name + ".weight" in self.weight_map else name
            w = self.load_tensor(key)
            if parallel_mode and tp_size > 1:
                dim = 0 if parallel_mode == "column" else 1
                if w.shape[dim] % tp_size:
                    raise ValueError(f"{name}: dimension {dim} ({w.shape[dim]}) is not divisible by {tp_size}")
                w = w.chunk(tp_size, dim)[tp_rank].contiguous()
            out["weight"] = w
        elif self.format.startswith("hlwq-"):
            if self.format != "hlwq-q5":
                raise ValueError(f"{self.format}: only the 5-bit HLWQ stream layout is defined (packing.unpack_codes_q5_hlwq)")
            meta = [int(v) for v in self.load_tensor(name + ".weight__meta").flatten().tolist()]
            out_f, n_blocks, bs, total = meta[:4]
            codes = unpack_codes_q5_hlwq(self.load_tensor(name + ".weight__packed"), total=total)
            out["codes"] = codes.reshape(out_f, n_blocks * bs).to(torch.int8)
            out["norms"] = self.load_tensor(name + ".weight__norms").to(torch.float16).reshape(out_f, n_blocks)
            out["ct_scaled"] = (get_centroids(5) / math.sqrt(bs)).to(torch.float32)
            out["in_f"] = meta[4] if len(meta) >= 5 else n_blocks * bs
            out["packed"] = False
        else:
            codes = self.load_tensor(name + ".codes")
            norms = self.load_tensor(name + ".norms").to(torch.float16)
            if name + ".ct_scaled" in self.weight_map:
                ct = self.load_tensor(name + ".ct_scaled").to(torch.float32)
            elif name + ".ct" in self.weight_map:
                ct = (self.load_tensor(name + ".ct").to(torch.float32) / math.sqrt(self.block_size))
            else:
                raise KeyError(f"no centroids for {name!r}: neither {name}.ct_scaled nor {name}.ct")
            meta = self.config.get("layers", {}).get(name, {})
            bs = int(meta.get("block_size", self.block_size))
            if meta.get("packed_q5", False):
                codes = unpack_codes_q5(codes, bs)
            k_padded = norms.shape[-1] * bs
            packed = codes.dtype == torch.uint8 and codes.shape[-1] * 2 == k_padded
            out["codes"] = codes if packed else codes.to(torch.int8)
            out["norms"], out["ct_scaled"], out["packed"] = norms, ct, packed
            if "in_features" in meta:
                out["in_f"] = int(meta["in_features"])
        if name + ".bias" in self.weight_map:
            out["bias"] = self.load_tensor(name + ".bias")
        if "codes" in out and parallel_mode and tp_size > 1:
            dim = 0 if parallel_mode == "column" else 1
            out["codes"] = parallel.shard_codes_for_tp(out["codes"], tp_rank, tp_size, dim, bool(out["packed"]), self.block_size)
            out["norms"] = parallel.shard_norms_for_tp(out["norms"], tp_rank, tp_size, dim)
            if dim == 1 and "in_f" in out:  # the rank's share of the true width
                per = out["norms"].shape[1] * self.block_size
                out["in_f"] = max(0, min(per, int(out["in_f"]) - tp_rank * per))
        if "bias" in out and parallel_mode and tp_size > 1:
            if parallel_mode == "column":
                out["bias"] = out["bias"].chunk(tp_size, 0)[tp_rank].contiguous()
            elif tp_rank != 0:
                del out["bias"]
        return out


def fill_linear(layer, tensors: Dict[str, torch.Tensor]) -> None:
    """Copy a loaded layer into the parameters ``PolarQuantLinearMethod.create_weights``
    registered (``codes`` int8, ``norms`` fp16, ``ct_scaled`` fp32).  Nibble-packed
    checkpoints are attached as ``codes_packed`` directly (``process_weights_after_loading``
    then only builds the tiled copy)."""
    from .packing import unpack_codes_half_block
    if "codes" not in tensors:
        raise ValueError("fill_linear needs a quantized layer (codes / norms / ct_scaled)")
    codes = tensors["codes"]
    if tensors.get("packed", False):
        codes = unpack_codes_half_block(codes)
    if tuple(codes.shape) != tuple(layer.codes.shape):
        raise ValueError(f"codes {tuple(codes.shape)} do not fit the layer {tuple(layer.codes.shape)}")
    if tuple(tensors["norms"].shape) != tuple(layer.norms.shape):
        raise ValueError(f"norms {tuple(tensors['norms'].shape)} do not fit the layer {tuple(layer.norms.shape)}")
    layer.codes.data.copy_(codes.to(layer.codes.dtype))
    layer.norms.data.copy_(tensors["norms"])
    ct = tensors["ct_scaled"]
    if ct.numel() != layer.ct_scaled.numel():
        raise ValueError(f"{ct.numel()} centroids for a {int(math.log2(layer.ct_scaled.numel()))}-bit layer")
    layer.ct_scaled.data.copy_(ct.to(layer.ct_scaled.dtype))
