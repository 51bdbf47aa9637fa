"""vLLM quantization config registered as ``"polarengine"``.

Reference: polarengine_vllm/config.py:62-270.  Parses ``polar_config.json``
(``block_size``, ``format``, ``bit_assignment``, ``layers``) and hands a method object
to each layer: embeddings stay unquantized, fused-MoE layers get the MoE method,
linear layers get :class:`PolarQuantLinearMethod` with the resolved bit width (an exact
per-layer entry first, otherwise the longest ``bit_assignment`` key contained in the
layer prefix, otherwise unquantized).
"""
from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional

import torch

log = logging.getLogger(__name__)

try:
    from vllm.model_executor.layers.quantization.base_config import QuantizationConfig, QuantizeMethodBase
    HAVE_VLLM = True
except Exception:  # pragma: no cover
    HAVE_VLLM = False

    class QuantizationConfig:  # type: ignore[no-redef]
        """Placeholder base when vLLM is absent."""

    class QuantizeMethodBase:  # type: ignore[no-redef]
        """Placeholder base when vLLM is absent."""

try:
    from vllm.model_executor.layers.quantization import register_quantization_config as _register
except Exception:  # pragma: no cover
    _register = None

KNOWN_FORMATS = frozenset({"polar_engine_v4", "polar_engine_v5", "hlwq-q5", "hlwq-q4", "hlwq-q3"})


class PolarQuantConfig(QuantizationConfig):
    def __init__(self, block_size: int = 128, bit_assignment: Optional[Dict[str, int]] = None,
                 layers_meta: Optional[Dict[str, Dict[str, Any]]] = None, fmt: str = "polar_engine_v4") -> None:
        if HAVE_VLLM:
            try:
                super().__init__()
            except Exception:
                pass
        self.block_size = block_size
        self.bit_assignment: Dict[str, int] = bit_assignment or {}
        self.layers_meta: Dict[str, Dict[str, Any]] = layers_meta or {}
        self.format = fmt
        self.quantize_experts = False  # True: MoE experts carry PolarQuant codes (PolarQuantMoEMethod)
        self.packed_modules_mapping: Dict[str, Any] = {}

    def __repr__(self) -> str:
        widths = sorted(set(self.bit_assignment.values()))
        return f"PolarQuantConfig(block_size={self.block_size}, bits={widths}, layers={len(self.layers_meta)})"

    # ---- interface vLLM queries
    @staticmethod
    def get_name() -> str:
        return "polarengine"

    @staticmethod
    def get_supported_act_dtypes() -> List[torch.dtype]:
        return [torch.float16, torch.bfloat16]

    @staticmethod
    def get_min_capability() -> int:
        # kept at the reference's value (config.py:112-115) so that config probing on
        # other devices behaves the same; the kernels themselves require sm_100
        return 70

    @staticmethod
    def get_config_filenames() -> List[str]:
        return ["polar_config.json"]

    @classmethod
    def from_config(cls, config: Dict[str, Any]) -> "PolarQuantConfig":
        fmt = config.get("format", "polar_engine_v4")
        if fmt not in KNOWN_FORMATS:
            log.warning("Unrecognised PolarEngine/HLWQ format '%s'; weight loading may fail.", fmt)
        out = cls(block_size=config.get("block_size", 128), bit_assignment=config.get("bit_assignment", {}),
                  layers_meta=config.get("layers", {}), fmt=fmt)
        out.quantize_experts = bool(config.get("quantize_experts", False))
        return out

    def get_quant_method(self, layer: torch.nn.Module, prefix: str) -> Optional["QuantizeMethodBase"]:
        from .linear_method import PolarQuantLinearMethod
        from vllm.model_executor.layers.linear import UnquantizedLinearMethod
        from vllm.model_executor.layers.vocab_parallel_embedding import (UnquantizedEmbeddingMethod,
                                                                         VocabParallelEmbedding)
        kind = type(layer).__name__
        if isinstance(layer, VocabParallelEmbedding) or "Embedding" in kind:
            return UnquantizedEmbeddingMethod()
        if any(tag in kind for tag in ("MoE", "Moe", "moe")) or hasattr(layer, "num_experts"):
            from .moe_method import make_moe_method
            return make_moe_method(self, layer, prefix)
        if not isinstance(layer, torch.nn.Linear) and "Linear" not in kind:
            return UnquantizedLinearMethod()
        bits = self._resolve_bits(prefix)
        if bits is None:
            return UnquantizedLinearMethod()
        return PolarQuantLinearMethod(block_size=self.block_size, bits=bits, layer_meta=self.layers_meta.get(prefix, {}))

    def _resolve_bits(self, prefix: str) -> Optional[int]:
        meta = self.layers_meta.get(prefix)
        if meta and "bits" in meta:
            return int(meta["bits"])
        hits = [k for k in self.bit_assignment if k in prefix]
        return int(self.bit_assignment[max(hits, key=len)]) if hits else None


if _register is not None:
    try:
        PolarQuantConfig = _register("polarengine")(PolarQuantConfig)
    except Exception as exc:  # already registered by another copy of the plugin
        log.debug("polarengine quantization config not re-registered: %s", exc)
elif HAVE_VLLM:  # pragma: no cover - old vLLM without the decorator
    try:
        from vllm.model_executor.layers.quantization import QUANTIZATION_METHODS
        if "polarengine" not in QUANTIZATION_METHODS:
            QUANTIZATION_METHODS["polarengine"] = PolarQuantConfig
    except Exception:
        log.warning("Could not register the polarengine quantization config with vLLM.")
