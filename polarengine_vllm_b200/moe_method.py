"""MoE methods behind vLLM's fused-MoE interface.

Reference: polarengine_vllm/moe_method.py:18-107.  The reference keeps expert weights in
bf16 and forwards to vLLM's unquantized fused MoE (``PolarPassthroughMoEMethod``, kept
here unchanged in behaviour).  ``PolarQuantMoEMethod`` is the quantized counterpart the
reference lists as future work: experts are stored as PolarQuant codes (gate/up fused as
``w13``, Q3 by default; down ``w2``, Q4) and every expert projection runs through the
same native kernels as a linear layer.  Routing and activation follow the reference's
MoE layer (nemotron_offload.py:180-226): softmax, top-k, renormalise, silu(gate) * up,
weighted sum over the selected experts.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _native as nv
from .decode_ops import silu_mul
from .kernels import quant_matmul
from .packing import pack_codes_half_block
from .utils import get_ct_scaled


class PolarPassthroughMoEMethod:
    """Delegates to vLLM's ``UnquantizedFusedMoEMethod``; built lazily because vLLM asks
    for the method before the FusedMoE layer is fully constructed."""

    def __init__(self) -> None:
        self._inner = None

    def _lazy_init(self, layer) -> bool:
        if self._inner is None:
            try:
                from vllm.model_executor.layers.fused_moe.unquantized_fused_moe_method import UnquantizedFusedMoEMethod
                self._inner = UnquantizedFusedMoEMethod(moe=layer)
            except (AttributeError, TypeError, ImportError):
                return False
        return True

    def create_weights(self, layer, num_experts, hidden_size, intermediate_size_per_partition, params_dtype, **kw):
        if self._lazy_init(layer):
            return self._inner.create_weights(layer, num_experts=num_experts, hidden_size=hidden_size,
                                              intermediate_size_per_partition=intermediate_size_per_partition,
                                              params_dtype=params_dtype, **kw)
        for name, shape in (("w13_weight", (num_experts, 2 * intermediate_size_per_partition, hidden_size)),
                            ("w2_weight", (num_experts, hidden_size, intermediate_size_per_partition))):
            layer.register_parameter(name, torch.nn.Parameter(torch.empty(*shape, dtype=params_dtype), requires_grad=False))

    def apply(self, layer, x, *args, **kwargs):
        if not self._lazy_init(layer):
            raise RuntimeError("PolarPassthroughMoEMethod: vLLM's fused MoE method could not be constructed")
        return self._inner.apply(layer, x, *args, **kwargs)

    def get_fused_moe_quant_config(self, *args):
        if self._inner is not None and hasattr(self._inner, "get_fused_moe_quant_config"):
            return self._inner.get_fused_moe_quant_config(*args)
        return None


def route_softmax_topk(router_logits: torch.Tensor, top_k: int, renormalize: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 softmax over experts, top-k, optional renormalisation (nemotron_offload.py:180-189).  On the GPU one launch
    (``pe_moe_route``); the torch ops below are the same math for CPU tensors."""
    if router_logits.is_cuda and router_logits.dim() == 2 and router_logits.shape[1] <= 1024 and top_k <= 32 \
            and router_logits.dtype in (torch.float32, torch.float16, torch.bfloat16):
        from . import _native as nv
        dev = router_logits.device
        nv.ensure_init(dev)
        lg = router_logits if router_logits.stride(1) == 1 else router_logits.contiguous()
        t, e = lg.shape
        w = torch.empty(t, top_k, dtype=torch.float32, device=dev)
        ids = torch.empty(t, top_k, dtype=torch.int64, device=dev)
        if t:
            nv.check(nv.lib().pe_moe_route(lg.data_ptr(), nv.dtype_code(lg), lg.stride(0), t, e, top_k, int(bool(renormalize)),
                                           w.data_ptr(), ids.data_ptr(), nv.stream_ptr(dev)), "pe_moe_route")
        return w, ids
    p = torch.softmax(router_logits.float(), dim=-1)
    w, ids = p.topk(top_k, dim=-1)
    if renormalize:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, ids


class PolarQuantMoEMethod:
    """Quantized experts.  Layer tensors (E = local experts, I = intermediate, H = hidden,
    K padded to multiples of 128):

        w13_codes  uint8 (E, 2I, H_pad/2) nibbles if w13_bits <= 4 else int8 (E, 2I, H_pad)
        w13_norms  fp16  (E, 2I, H_pad/128)
        w2_codes   uint8 (E, H, I_pad/2)  or int8 (E, H, I_pad)
        w2_norms   fp16  (E, H, I_pad/128)
        w13_ct_scaled / w2_ct_scaled  fp32 tables

    ``expert_map`` (optional int tensor of size global experts, -1 = not on this rank)
    supports expert-parallel placement: tokens routed elsewhere contribute zero here and
    the caller all-reduces.
    """

    def __init__(self, w13_bits: int = 3, w2_bits: int = 4, block_size: int = 128) -> None:
        self.w13_bits, self.w2_bits, self.block_size = w13_bits, w2_bits, block_size

    @staticmethod
    def _pad(n: int, b: int = 128) -> int:
        return -(-n // b) * b

    def create_weights(self, layer, num_experts, hidden_size, intermediate_size_per_partition, params_dtype, **kw):
        e, h, i = num_experts, hidden_size, intermediate_size_per_partition
        hp, ip = self._pad(h), self._pad(i)
        def codes(rows, kp, bits):
            return torch.zeros(e, rows, kp // 2 if bits <= 4 else kp, dtype=torch.uint8 if bits <= 4 else torch.int8)
        for name, t in (("w13_codes", codes(2 * i, hp, self.w13_bits)),
                        ("w13_norms", torch.zeros(e, 2 * i, hp // 128, dtype=torch.float16)),
                        ("w2_codes", codes(h, ip, self.w2_bits)),
                        ("w2_norms", torch.zeros(e, h, ip // 128, dtype=torch.float16))):
            prm = torch.nn.Parameter(t, requires_grad=False)
            if "weight_loader" in kw:
                prm.weight_loader = kw["weight_loader"]
            layer.register_parameter(name, prm)
        layer.register_buffer("w13_ct_scaled", get_ct_scaled(self.w13_bits).clone())
        layer.register_buffer("w2_ct_scaled", get_ct_scaled(self.w2_bits).clone())
        layer.moe_hidden, layer.moe_inter, layer.moe_hidden_padded, layer.moe_inter_padded = h, i, hp, ip
        layer.moe_w13_bits, layer.moe_w2_bits = self.w13_bits, self.w2_bits

    def load_expert(self, layer, e: int, gate: dict, up: dict, down: dict) -> None:
        """Copy one expert's quantizer outputs (dicts with int8 ``codes`` and ``norms``)."""
        i = layer.moe_inter
        for lo, src in ((0, gate), (i, up)):
            c = src["codes"]
            layer.w13_codes.data[e, lo:lo + i] = (pack_codes_half_block(c) if self.w13_bits <= 4 else c).to(layer.w13_codes.device)
            layer.w13_norms.data[e, lo:lo + i] = src["norms"].to(layer.w13_norms.device)
        c = down["codes"]
        layer.w2_codes.data[e] = (pack_codes_half_block(c) if self.w2_bits <= 4 else c).to(layer.w2_codes.device)
        layer.w2_norms.data[e] = down["norms"].to(layer.w2_norms.device)

    def process_weights_after_loading(self, layer) -> None:
        dev = layer.w13_codes.device
        layer.w13_ct_scaled = layer.w13_ct_scaled.to(dev)
        layer.w2_ct_scaled = layer.w2_ct_scaled.to(dev)

    def apply(self, layer, x, a, b, *rest, expert_map: Optional[torch.Tensor] = None, **kwargs):
        """Both calling conventions of vLLM's fused-MoE methods:
        ``apply(layer, x, topk_weights, topk_ids, ...)`` (routing done by the caller, vLLM 0.2x) and
        ``apply(layer, x, router_logits, top_k, renormalize, ...)`` (the reference's, moe_method.py:74-78)."""
        if torch.is_tensor(b) and not b.is_floating_point():
            topk_weights, topk_ids = a, b
        else:
            renorm = rest[0] if rest else kwargs.get("renormalize", True)
            topk_weights, topk_ids = route_softmax_topk(a, int(b), bool(renorm))
        return self.moe_forward(layer, x, topk_weights, topk_ids, expert_map)

    # average (token, expert) pairs per local expert up to which the grouped launches are
    # used; beyond it every expert has enough rows to fill the tensor-core kernel by itself
    # (measured on 128 experts: grouped 6.5 ms against 21.8 ms per-expert at 128 rows each)
    GROUPED_MAX_ROWS_PER_EXPERT = 512
    # average rows per expert from which the grouped launches run on the tensor cores (a 256 x 256
    # tile per expert and weight tile costs the same for 1 or 256 rows; below this the streaming
    # decode-size kernel is cheaper)
    TENSOR_CORE_MIN_ROWS_PER_EXPERT = 12

    def moe_forward(self, layer, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                    expert_map: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y[t] = sum_k w[t,k] * down_e(silu(gate_e(x[t])) * up_e(x[t])), e = ids[t,k]; fp16 out.
        Decode-size batches: two grouped launches over all experts (``pe_gemv_grouped``),
        nothing read back to the host.  Prefill-size batches: per-expert tensor-core matmuls."""
        n_local = layer.w13_codes.shape[0]
        if self.expected_local_pairs(topk_ids.numel(), n_local, expert_map) <= self.GROUPED_MAX_ROWS_PER_EXPERT * n_local \
                and x.dtype in (torch.float16, torch.bfloat16):
            out = self._moe_forward_grouped(layer, x, topk_weights, topk_ids, expert_map)
            if out is not None:
                return out
        return self._moe_forward_per_expert(layer, x, topk_weights, topk_ids, expert_map)

    @staticmethod
    def expected_local_pairs(pairs: int, n_local: int, expert_map: Optional[torch.Tensor]) -> int:
        """(token, expert) pairs this rank expects to own: all of them without an expert map, else
        the local share of uniformly routed pairs (kernel choices only; buffers hold every pair)."""
        n_global = int(expert_map.numel()) if expert_map is not None else n_local
        return max(1, pairs * n_local // max(n_global, 1))

    def _moe_forward_grouped(self, layer, x, topk_weights, topk_ids, expert_map) -> Optional[torch.Tensor]:
        lead = x.shape[:-1]
        h, i = layer.moe_hidden, layer.moe_inter
        hp, ip = layer.moe_hidden_padded, layer.moe_inter_padded
        x2 = x.reshape(-1, h)
        if x2.stride(1) != 1:
            x2 = x2.contiguous()
        dev = nv.require_cuda(x2, layer.w13_codes, layer.w2_codes)
        nv.ensure_init(dev)
        t, k = topk_ids.shape
        n_local = layer.w13_codes.shape[0]
        pairs = t * k
        ids = topk_ids.reshape(-1).to(torch.int64).contiguous()
        emap = expert_map.to(device=dev, dtype=torch.int64).contiguous() if expert_map is not None else None
        # rows per problem: 8 while experts see few tokens (lighter kernel), else 16
        local_pairs = self.expected_local_pairs(pairs, n_local, expert_map)
        rpp = 8 if local_pairs <= 6 * n_local else 16
        max_problems = min(n_local, pairs) + pairs // rpp
        l = nv.lib()
        if min(l.pe_gemv_grouped_workspace_bytes(max_problems, 2 * i, hp), l.pe_gemv_grouped_workspace_bytes(max_problems, h, ip)) == 0:
            return None  # more problems than the scratch counter zone holds: the caller takes the per-expert path
        tok_sorted = torch.empty(pairs, dtype=torch.int32, device=dev)   # token of every grouped row
        pos = torch.empty(pairs, dtype=torch.int32, device=dev)          # grouped row of every pair (-1: other rank)
        desc = torch.empty(max_problems, 4, dtype=torch.int32, device=dev)
        expert_rows = torch.empty(n_local, 2, dtype=torch.int32, device=dev)  # (first grouped row, rows) per expert
        st = nv.stream_ptr(dev)
        nv.check(l.pe_moe_plan(ids.data_ptr(), emap.data_ptr() if emap is not None else None,
                               int(emap.numel()) if emap is not None else 0, pairs, k, n_local, rpp,
                               max_problems, tok_sorted.data_ptr(), pos.data_ptr(), desc.data_ptr(), expert_rows.data_ptr(), st),
                 "pe_moe_plan")
        # many rows per expert: the tensor-core kernel over all experts (tile list built on the device);
        # few: the decode-size kernel, which streams every expert's codes once per 8 or 16 rows
        tensor_cores = local_pairs >= self.TENSOR_CORE_MIN_ROWS_PER_EXPERT * n_local

        def grouped(codes, packed, norms, ct, xin, x_rows, in_f, kp, y):
            if tensor_cores and codes.stride(0) == codes.shape[1] * codes.stride(1):
                need = l.pe_gemm_grouped_workspace_bytes(n_local, pairs, y.shape[1], kp)
                ws = nv.gemm_workspace(dev, need)
                nv.check(l.pe_gemm_grouped(codes.data_ptr(), int(packed), codes.stride(1) * codes.element_size(),
                                           codes.stride(0) * codes.element_size(), norms.data_ptr(), norms.stride(1),
                                           norms.stride(0), ct.data_ptr(), ct.numel(), xin.data_ptr(), nv.PE_X_RAW,
                                           nv.dtype_code(xin), xin.stride(0), in_f, x_rows.data_ptr() if x_rows is not None else None,
                                           y.data_ptr(), nv.dtype_code(y), y.stride(0), expert_rows.data_ptr(), n_local, pairs,
                                           y.shape[1], kp, ws.data_ptr(), ws.numel(), st), "pe_gemm_grouped")
                return
            ws = nv.grouped_scratch(dev, l.pe_gemv_grouped_workspace_bytes(max_problems, y.shape[1], kp))
            nv.check(l.pe_gemv_grouped(codes.data_ptr(), int(packed), codes.stride(1) * codes.element_size(),
                                       codes.stride(0) * codes.element_size(), norms.data_ptr(), norms.stride(1), norms.stride(0),
                                       ct.data_ptr(), ct.numel(), xin.data_ptr(), nv.PE_X_RAW, nv.dtype_code(xin), xin.stride(0),
                                       in_f, x_rows.data_ptr() if x_rows is not None else None, y.data_ptr(), nv.dtype_code(y),
                                       y.stride(0), desc.data_ptr(), max_problems, rpp, y.shape[1], kp, ws.data_ptr(), ws.numel(), st),
                     "pe_gemv_grouped")
        gu = torch.empty(pairs, 2 * i, dtype=torch.float16, device=dev)   # rows beyond the local pairs stay unused
        grouped(layer.w13_codes, self.w13_bits <= 4, layer.w13_norms, layer.w13_ct_scaled, x2, tok_sorted, h, hp, gu)
        act = silu_mul(gu, i)
        d = torch.empty(pairs, h, dtype=torch.float32, device=dev)
        grouped(layer.w2_codes, self.w2_bits <= 4, layer.w2_norms, layer.w2_ct_scaled, act, None, i, ip, d)
        out = torch.empty(t, h, dtype=torch.float16, device=dev)
        wts = topk_weights.reshape(-1).to(torch.float32).contiguous()
        nv.check(l.pe_moe_combine(d.data_ptr(), d.stride(0), pos.data_ptr(), wts.data_ptr(), t, k, out.data_ptr(), nv.PE_F16,
                                  out.stride(0), h, st), "pe_moe_combine")
        return out.view(*lead, h)

    def _moe_forward_per_expert(self, layer, x: torch.Tensor, topk_weights: torch.Tensor, topk_ids: torch.Tensor,
                                expert_map: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Tokens are grouped by expert on the device; each expert's tokens go through the
        two projections as one batch (tensor-core path for more than 16 rows)."""
        lead = x.shape[:-1]
        h, i = layer.moe_hidden, layer.moe_inter
        x2 = x.reshape(-1, h)
        t, k = topk_ids.shape
        ids = topk_ids.reshape(-1)
        if expert_map is not None:  # ids outside the map belong to nobody (same rule as pe_moe_plan)
            em = expert_map.to(ids.device)
            inside = (ids >= 0) & (ids < em.numel())
            ids = torch.where(inside, em[ids.long().clamp(0, em.numel() - 1)], torch.full_like(ids, -1))
        order = torch.argsort(ids, stable=True)
        sorted_ids = ids[order]
        n_local = layer.w13_codes.shape[0]
        skipped = int((sorted_ids < 0).sum()) if expert_map is not None else 0  # routed to other ranks; sorted first
        counts = torch.bincount(sorted_ids[skipped:], minlength=n_local)
        tok = (order // k)
        wts = topk_weights.reshape(-1)[order].float()
        out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
        pos = skipped
        for e, n in enumerate(counts.tolist()):
            if n == 0:
                continue
            sel = tok[pos:pos + n]
            xe = x2.index_select(0, sel)
            gu = quant_matmul(layer.w13_codes[e], self.w13_bits <= 4, layer.w13_norms[e], layer.w13_ct_scaled, xe, False,
                              2 * i, h, layer.moe_hidden_padded, torch.float32)
            act = torch.nn.functional.silu(gu[:, :i]) * gu[:, i:]
            d = quant_matmul(layer.w2_codes[e], self.w2_bits <= 4, layer.w2_norms[e], layer.w2_ct_scaled, act, False,
                             h, i, layer.moe_inter_padded, torch.float32)
            out.index_add_(0, sel, d * wts[pos:pos + n].unsqueeze(1))
            pos += n
        return out.to(torch.float16).view(*lead, h)

    def get_fused_moe_quant_config(self, *args):
        return None


def make_moe_method(config, layer, prefix):
    """Quantized experts when the checkpoint's bit table names them, else the reference's pass-through."""
    bits13 = config._resolve_bits(prefix + ".experts.0.gate_proj") if hasattr(config, "_resolve_bits") else None
    bits2 = config._resolve_bits(prefix + ".experts.0.down_proj") if hasattr(config, "_resolve_bits") else None
    if bits13 is not None and bits2 is not None and getattr(config, "quantize_experts", False):
        return PolarQuantMoEMethod(bits13, bits2, config.block_size)
    return PolarPassthroughMoEMethod()


try:
    from vllm.model_executor.layers.fused_moe.layer import FusedMoEMethodBase
    FusedMoEMethodBase.register(PolarPassthroughMoEMethod)
    FusedMoEMethodBase.register(PolarQuantMoEMethod)
except Exception:
    pass
