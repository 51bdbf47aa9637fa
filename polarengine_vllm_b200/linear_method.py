"""Quantized linear layer behind vLLM's linear-method interface.

Reference: polarengine_vllm/linear_method.py:59-258 (``PolarQuantLinearMethod``).
Same three entry points and the same layer attributes (``codes`` / ``codes_packed``,
``norms``, ``ct_scaled``, ``in_f``, ``out_f``, ``in_f_padded``, ``n_blocks``, ``bits``,
``block_size``, ``packed``, ``in_f_half``); the forward keeps the reference's meaning
(flatten, pad, rotate, multiply, cast to fp16, add ``bias.half()``) but is one native
launch for up to 16 tokens: padding, rotation, dequantisation, dot products, the
split-K reduction, the cast and the bias all happen inside ``pe_gemv``.

Differences from the reference that a vLLM integrator should know:
* the class derives from vLLM's ``LinearMethodBase`` when vLLM is importable, so the
  loader calls ``process_weights_after_loading``;
* ``codes`` and ``norms`` are non-trainable Parameters carrying ``input_dim`` /
  ``output_dim`` / ``weight_loader`` attributes, sized from the per-rank partition
  (``input_size_per_partition``, ``sum(output_partition_sizes)``) so tensor-parallel
  shards load correctly; a row-parallel shard must cover whole 128-blocks.
"""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import torch

from .kernels import SMALL_BATCH_MAX, pack_codes_int4, quant_matmul, retile, small_batch_takes
from .packing import unpack_codes_half_block, unpack_codes_q5
from .utils import get_ct_scaled

try:  # vLLM is optional: the class must stay importable for offline tooling
    from vllm.model_executor.layers.linear import LinearMethodBase as _Base
    from vllm.model_executor.utils import set_weight_attrs
except Exception:  # pragma: no cover - exercised only without vLLM
    class _Base:  # type: ignore[no-redef]
        pass

    def set_weight_attrs(weight: torch.Tensor, attrs: Optional[Dict[str, Any]]) -> None:
        for k, v in (attrs or {}).items():
            setattr(weight, k, v)


def codes_to_int8(w: torch.Tensor, in_f_padded: int) -> torch.Tensor:
    """One byte per code from any of the on-disk layouts of a ``<prefix>.codes`` tensor: half-block nibbles
    (uint8, K/2 columns: quantizer.py:349-351), LSB-first 5-bit packing (uint8, 5K/8 columns: quantizer.py:352-354;
    the reference unpacks it at load, loader.py:412-417) or int8 as is."""
    cols = w.shape[-1]
    if cols == in_f_padded:
        return w.view(torch.int8) if w.dtype == torch.uint8 else w.to(torch.int8)
    if cols * 2 == in_f_padded:
        return unpack_codes_half_block(w.view(torch.uint8) if w.dtype == torch.int8 else w).to(torch.int8)
    if cols * 8 == in_f_padded * 5:
        return unpack_codes_q5(w.view(torch.uint8) if w.dtype == torch.int8 else w).to(torch.int8)
    raise ValueError(f"codes tensor of width {cols} fits none of the layouts of a layer with {in_f_padded} padded input features")


def _checkpoint_loader(inner, kind: str, in_f_padded: int):
    """The ``weight_loader`` vLLM calls for a parameter of a quantized layer: brings the checkpoint tensor into
    the parameter's layout, then hands it to the layer's own loader (``inner``: vLLM's, which narrows to the
    rank's shard along ``output_dim`` / ``input_dim`` and places fused q/k/v or gate/up sections), or copies it
    when the layer has none.  The centroid table is the same for every section of a fused layer."""
    def loader(param: torch.nn.Parameter, loaded_weight: torch.Tensor, *args: Any, **kwargs: Any) -> None:
        w = loaded_weight
        if kind == "codes":
            w = codes_to_int8(w, in_f_padded)
        elif kind == "norms":
            w = w.to(torch.float16)
        else:  # ct_scaled
            param.data.copy_(w.to(param.dtype).reshape(param.shape))
            return
        if inner is not None:
            inner(param, w, *args, **kwargs)
        else:
            param.data.copy_(w)
    return loader


class PolarQuantLinearMethod(_Base):
    def __init__(self, block_size: int = 128, bits: int = 4, layer_meta: Optional[Dict[str, Any]] = None) -> None:
        if block_size != 128:
            raise ValueError("the B200 kernels support block_size 128 only")
        self.block_size = block_size
        self.bits = bits
        self.layer_meta = layer_meta or {}
        # The tiled copy of a layer (codes and norms interleaved per 16-row x 128-column tile) serves batches of
        # 3..16 rows only; it is built the first time such a batch arrives, so a layer that only ever sees one
        # token at a time, or prefill, keeps a single copy of its codes in HBM.
        self.decode_tiled = True

    # ------------------------------------------------------------------ weights
    def create_weights(self, layer: torch.nn.Module, input_size_per_partition: int,
                       output_partition_sizes: List[int], input_size: int, output_size: int,
                       params_dtype: torch.dtype, **extra_weight_attrs: Any) -> None:
        bs = self.block_size
        in_f = int(input_size_per_partition)
        out_f = int(sum(output_partition_sizes))
        if in_f != input_size and in_f % bs:
            raise ValueError(f"a K-shard of a PolarQuant layer must be a multiple of {bs}, got {in_f}")
        padded = -(-in_f // bs) * bs
        nblk = padded // bs
        codes = torch.nn.Parameter(torch.zeros(out_f, padded, dtype=torch.int8), requires_grad=False)
        norms = torch.nn.Parameter(torch.zeros(out_f, nblk, dtype=torch.float16), requires_grad=False)
        # vLLM's model loaders look parameters up by checkpoint name (`<prefix>.codes`, `.norms`, `.ct_scaled`) and
        # call their `weight_loader`: ours unpacks the on-disk code layouts first (the reference unpacks in its own
        # loader, loader.py:300-445, which vLLM never calls), then vLLM's shards and places the tensor.  The
        # full (un-sharded) padded width tells the layouts apart whatever the rank's slice is.
        inner = extra_weight_attrs.get("weight_loader")
        full_padded = -(-int(input_size) // bs) * bs
        ct = torch.nn.Parameter(get_ct_scaled(self.bits, bs).clone(), requires_grad=False)
        for prm, kind in ((codes, "codes"), (norms, "norms"), (ct, "ct_scaled")):
            attrs = {"weight_loader": _checkpoint_loader(inner if kind != "ct_scaled" else None, kind, full_padded)}
            if kind != "ct_scaled":
                attrs.update(input_dim=1, output_dim=0)
            set_weight_attrs(prm, attrs)
        layer.register_parameter("codes", codes)
        layer.register_parameter("norms", norms)
        layer.register_parameter("ct_scaled", ct)
        layer.in_f, layer.out_f = in_f, out_f
        layer.in_f_padded, layer.n_blocks = padded, nblk
        layer.bits, layer.block_size, layer.packed = self.bits, bs, False

    def process_weights_after_loading(self, layer: torch.nn.Module) -> None:
        """Move the table next to the codes and nibble-pack widths <= 4 (native kernel)."""
        dev = layer.codes.device if hasattr(layer, "codes") else layer.codes_packed.device
        if layer.ct_scaled.device != dev:
            layer.ct_scaled.data = layer.ct_scaled.data.to(dev)
        if layer.bits <= 4 and not getattr(layer, "packed", False):
            packed = pack_codes_int4(layer.codes.data, layer.block_size)
            if "codes" in layer._parameters:
                del layer._parameters["codes"]
            elif "codes" in layer._buffers:
                del layer._buffers["codes"]
            else:
                del layer.codes
            layer.codes_packed = packed
            layer.in_f_half = layer.n_blocks * (layer.block_size // 2)
            layer.packed = True
        layer.codes_tiled = None

    # ------------------------------------------------------------------ forward
    def apply(self, layer: torch.nn.Module, x: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, layer.in_f)
        packed = bool(getattr(layer, "packed", False))
        w = layer.codes_packed if packed else layer.codes
        if (self.decode_tiled and 3 <= x2.shape[0] <= 16 and getattr(layer, "codes_tiled", None) is None
                and not torch.cuda.is_current_stream_capturing()
                and not (x2.shape[0] <= SMALL_BATCH_MAX
                         and small_batch_takes(w.data, packed, layer.norms.data.reshape(layer.out_f, -1), layer.out_f, layer.in_f_padded))):
            layer.codes_tiled = retile(w.data, packed, layer.norms.data)
        # one native entry for every batch size: <= 16 rows run the fused decode kernel,
        # more rows the tensor-core kernel (rotation is done by its preparation launch)
        y = quant_matmul(w, packed, layer.norms, layer.ct_scaled, x2, False, layer.out_f, layer.in_f,
                         layer.in_f_padded, torch.float16, bias, tiles=getattr(layer, "codes_tiled", None))
        return y.view(*lead, layer.out_f)


def create_fwht_clear_hook(linear_method: PolarQuantLinearMethod):
    """The reference installs this forward pre-hook to empty the method's memo of rotated activations
    (linear_method.py:265-288).  Here the rotation happens inside the matmul launch and nothing is memoised,
    so the hook has nothing to clear; it exists so that code written against the reference keeps working."""
    def hook(module: torch.nn.Module, args: Any) -> None:
        return None
    return hook
