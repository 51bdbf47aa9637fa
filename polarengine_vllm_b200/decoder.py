"""Minimal dense decoder built on the quantized layers, for end-to-end decode measurement.

This is measurement scaffolding around the quantized-linear path, not a model zoo: a
9B-class decoder (hidden 4096, 32 query / 8 KV heads of 128, intermediate 12288, 36
layers, vocabulary 151936) whose every projection, the embedding and the LM head run
through the native kernels.  Residual add + RMSNorm, rotary embedding + KV-cache write and
SiLU * up are single native launches (``decode_ops``); decode-step attention over the KV cache is one native launch too
(prefill attention is torch's SDPA); none of these is the path under test.  ``rms_norm`` and ``rope`` below are the op-by-op torch
formulations the fused ops are tested against.

Tensor parallelism follows vLLM's layout, which is also the only place where ranks
exchange data: q/k/v and gate/up are column parallel (heads / intermediate split), o and
down are row parallel with one all-reduce each (``parallel.QuantLinearShard``), the LM
head is column parallel over the vocabulary with an all-gather of the per-rank maxima.
Weights are synthetic: codes are Lloyd-Max cells of N(0,1) draws, norms ~ 0.02*sqrt(128).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .decode_ops import add_rmsnorm, decode_attention, rope_attention, rope_cache, silu_mul
from . import _native as nv
from .kernels import SMALL_BATCH_MAX, quant_embedding, quant_matmul, quant_matmul_pro, retile, small_batch_takes
from .packing import pack_codes_half_block
from .parallel import PeerExchange, shard_codes_for_tp, shard_norms_for_tp
from .utils import get_centroids, get_ct_scaled


@dataclass
class DecoderConfig:
    hidden: int = 4096
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 12288
    n_layers: int = 36
    vocab: int = 151936
    bits_qkv: int = 5
    bits_o: int = 6
    bits_gate_up: int = 3
    bits_down: int = 4
    bits_embed: int = 5
    bits_head: int = 6
    rms_eps: float = 1e-6
    rope_theta: float = 1e6


def synth_weight(out_f: int, in_f: int, bits: int, dev, gen: torch.Generator):
    """Synthetic quantizer output for a (out_f, in_f) weight: int8 codes (Lloyd-Max cells of N(0,1) draws) and
    fp16 block norms ~ 0.02 * sqrt(128)."""
    ct = get_centroids(bits).to(dev)
    bounds = (ct[1:] + ct[:-1]) / 2
    codes = torch.empty(out_f, in_f, dtype=torch.int8, device=dev)
    step = max(1, (1 << 26) // in_f)
    for r0 in range(0, out_f, step):  # bounded temporaries for vocabulary-sized tables
        r1 = min(out_f, r0 + step)
        codes[r0:r1] = torch.bucketize(torch.randn(r1 - r0, in_f, device=dev, generator=gen), bounds).to(torch.int8)
    norms = (0.02 * math.sqrt(128) * (1 + 0.05 * torch.randn(out_f, in_f // 128, device=dev, generator=gen))).half()
    return codes, norms


class QWeight:
    """Quantized (out_f, in_f) weight resident on one device, from int8 codes and fp16 norms."""

    def __init__(self, codes: torch.Tensor, norms: torch.Tensor, bits: int):
        self.packed = bits <= 4
        self.codes = pack_codes_half_block(codes) if self.packed else codes.contiguous()
        self.norms = norms.contiguous()
        self.ct = get_ct_scaled(bits).to(codes.device)
        self.out_f, self.in_f = codes.shape
        self.tiles = None  # streaming copy for batches of 3..16 rows, built the first time one arrives

    @classmethod
    def synthetic(cls, out_f: int, in_f: int, bits: int, dev, gen: torch.Generator) -> "QWeight":
        return cls(*synth_weight(out_f, in_f, bits, dev, gen), bits)

    def fused(self, prologue: int, x: torch.Tensor, out_dtype=torch.float16, **kw) -> Optional[torch.Tensor]:
        """One token with the glue op in front of the projection folded into the launch; None if the layer's
        shape is not one the batch-1 kernel takes."""
        return quant_matmul_pro(self.codes, self.packed, self.norms, self.ct, prologue, x, self.in_f, self.out_f, self.in_f,
                                out_dtype, **kw)

    def __call__(self, x: torch.Tensor, out_dtype=torch.float16) -> torch.Tensor:
        if (self.tiles is None and 3 <= x.shape[0] <= 16 and not torch.cuda.is_current_stream_capturing()
                and not (x.shape[0] <= SMALL_BATCH_MAX and small_batch_takes(self.codes, self.packed, self.norms, self.out_f, self.in_f))):
            self.tiles = retile(self.codes, self.packed, self.norms)
        return quant_matmul(self.codes, self.packed, self.norms, self.ct, x, False, self.out_f, self.in_f, self.in_f, out_dtype,
                            tiles=self.tiles)


def shard_fused_rows(codes, norms, sections, rank: int, world: int):
    """Column-parallel shard of a fused projection: the rank's rows of every section (q | k | v, gate | up),
    concatenated in section order -- the slicing vLLM's loader applies to fused ``qkv_proj`` / ``gate_up_proj``
    shards (the reference's row helper is loader.py:558-598)."""
    cs, ns, r0 = [], [], 0
    for n in sections:
        cs.append(shard_codes_for_tp(codes[r0:r0 + n], rank, world, 0))
        ns.append(shard_norms_for_tp(norms[r0:r0 + n], rank, world, 0))
        r0 += n
    return torch.cat(cs, 0), torch.cat(ns, 0)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def rope(x: torch.Tensor, pos: torch.Tensor, theta: float) -> torch.Tensor:
    """x (B, H, T, D), pos (T,) absolute positions; rotate-half form."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, None], ang.sin()[None, None]
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1).to(x.dtype)


class QuantDecoder:
    def __init__(self, cfg: DecoderConfig, dev, tp_rank: int = 0, tp_size: int = 1, group=None, seed: int = 1000,
                 max_len: int = 640, batch: int = 1, fused_allreduce: bool = False):
        assert cfg.n_kv_heads % tp_size == 0 and (cfg.intermediate // tp_size) % 128 == 0
        self.cfg, self.dev, self.rank, self.tp, self.group = cfg, dev, tp_rank, tp_size, group
        self.hq, self.hkv = cfg.n_heads // tp_size, cfg.n_kv_heads // tp_size
        self.inter = cfg.intermediate // tp_size
        d = cfg.head_dim
        self.layers: List[dict] = []
        # Every rank draws the SAME full layer from the seed and keeps its shard (rows for the column-parallel
        # projections, whole 128-blocks of K for the row-parallel ones), so a sharded model computes the same
        # function as the un-sharded one and their outputs can be compared.
        for li in range(cfg.n_layers):
            g = torch.Generator(device=dev).manual_seed(seed + 16 * li)
            nq, nkv = cfg.n_heads * d, cfg.n_kv_heads * d
            c, n = synth_weight(nq + 2 * nkv, cfg.hidden, cfg.bits_qkv, dev, g)
            qkv = QWeight(*shard_fused_rows(c, n, (nq, nkv, nkv), tp_rank, tp_size), cfg.bits_qkv)
            c, n = synth_weight(cfg.hidden, nq, cfg.bits_o, dev, g)
            o = QWeight(shard_codes_for_tp(c, tp_rank, tp_size, 1), shard_norms_for_tp(n, tp_rank, tp_size, 1), cfg.bits_o)
            c, n = synth_weight(2 * cfg.intermediate, cfg.hidden, cfg.bits_gate_up, dev, g)
            gate_up = QWeight(*shard_fused_rows(c, n, (cfg.intermediate, cfg.intermediate), tp_rank, tp_size), cfg.bits_gate_up)
            c, n = synth_weight(cfg.hidden, cfg.intermediate, cfg.bits_down, dev, g)
            down = QWeight(shard_codes_for_tp(c, tp_rank, tp_size, 1), shard_norms_for_tp(n, tp_rank, tp_size, 1), cfg.bits_down)
            del c, n
            self.layers.append({
                "qkv": qkv, "o": o, "gate_up": gate_up, "down": down,
                "ln1": torch.ones(cfg.hidden, dtype=torch.float16, device=dev),
                "ln2": torch.ones(cfg.hidden, dtype=torch.float16, device=dev),
            })
        ge = torch.Generator(device=dev).manual_seed(seed + 900)  # same table on every rank
        self.embed = QWeight.synthetic(cfg.vocab, cfg.hidden, cfg.bits_embed, dev, ge)
        assert cfg.vocab % tp_size == 0
        gh = torch.Generator(device=dev).manual_seed(seed + 901)
        c, n = synth_weight(cfg.vocab, cfg.hidden, cfg.bits_head, dev, gh)
        self.head = QWeight(shard_codes_for_tp(c, tp_rank, tp_size, 0), shard_norms_for_tp(n, tp_rank, tp_size, 0), cfg.bits_head)
        del c, n
        self.final_ln = torch.ones(cfg.hidden, dtype=torch.float16, device=dev)
        self.max_len = max_len
        self.n_sms = torch.cuda.get_device_properties(dev).multi_processor_count
        self.fuse_glue = True   # fold norm / activation into the projections' launches when one token is decoded
        self.fused_allreduce = fused_allreduce
        self.xchg = None
        self.alloc_cache(batch)

    def alloc_cache(self, batch: int) -> None:
        """(Re)allocate the KV cache and the exchange buffers for `batch` sequences (a collective call when the
        fused row-parallel epilogue is on: every rank must make it)."""
        cfg, dev, d = self.cfg, self.dev, self.cfg.head_dim
        self.batch = batch
        # decode steps of a sharded model: all-reduce + residual add + norm as one launch over peer memory
        if self.fused_allreduce and (self.xchg is None or self.xchg.max_rows < batch):
            self.xchg = PeerExchange(dev, self.rank, self.tp, max(batch, 1), cfg.hidden, self.group)
        self.k_cache = [torch.zeros(batch, self.hkv, self.max_len, d, dtype=torch.float16, device=dev) for _ in range(cfg.n_layers)]
        self.v_cache = [torch.zeros(batch, self.hkv, self.max_len, d, dtype=torch.float16, device=dev) for _ in range(cfg.n_layers)]

    # ---- collectives (the only exchanges on the path)
    def _all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.tp > 1:
            dist.all_reduce(t, group=self.group)
        return t

    def weight_bytes_per_step(self) -> int:
        """Algorithmic code + norm bytes one decode step streams on this rank."""
        total = 0
        for L in self.layers:
            for k in ("qkv", "o", "gate_up", "down"):
                total += L[k].codes.numel() * L[k].codes.element_size() + L[k].norms.numel() * 2
        return total + self.head.codes.numel() + self.head.norms.numel() * 2

    def forward(self, ids: torch.Tensor, pos0, return_logits: bool = False) -> torch.Tensor:
        """ids (B, T) -> next-token ids (B,), or the fp32 logits (B, vocab) of the last position (gathered over
        the ranks) when ``return_logits`` is set.  ``pos0`` is an int (prefill) or a 0-d device
        tensor (decode under a CUDA graph); the KV cache is written at pos0..pos0+T-1."""
        cfg, d = self.cfg, self.cfg.head_dim
        b, t = ids.shape
        x = quant_embedding(self.embed.codes, self.embed.packed, self.embed.norms, self.embed.ct, ids, cfg.hidden)
        x = x.view(b * t, cfg.hidden)  # residual stream, updated in place by add_rmsnorm
        delta = None                   # output of the previous layer's down projection, not yet added
        fused = self.xchg is not None and b * t <= self.xchg.max_rows

        def reduce_add_norm(partial, w):   # x += sum over ranks of partial; returns norm(x) * w
            if fused:
                return self.xchg.allreduce_add_rmsnorm(partial, x, w, cfg.rms_eps)
            return add_rmsnorm(x, self._all_reduce(partial), w, cfg.rms_eps)

        # One token on one rank: the residual add + RMSNorm in front of q/k/v and gate/up and the SiLU * up in
        # front of down are computed by the projection's own launch (6 launches per layer instead of 9).  The
        # residual alternates between two buffers because every CTA of such a launch reads the old one.
        one = b * t == 1 and self.fuse_glue
        fold_norm = one and self.tp == 1   # with several ranks the all-reduce kernel does the add + norm
        x_alt = torch.empty_like(x) if fold_norm else None

        def norm_proj(W, delta, w, out_dtype=torch.float16):   # W(norm(x += delta))
            nonlocal x, x_alt
            if fold_norm:
                y = W.fused(nv.PE_PRO_ADD_RMSNORM, x, out_dtype, delta=delta, norm_weight=w, eps=cfg.rms_eps,
                            resid_out=x_alt if delta is not None else None)
                if y is not None:
                    if delta is not None:
                        x, x_alt = x_alt, x
                    return y
            h = add_rmsnorm(x, None, w, cfg.rms_eps) if delta is None else reduce_add_norm(delta, w)
            return W(h, out_dtype)

        for li, L in enumerate(self.layers):
            qkv = norm_proj(L["qkv"], delta, L["ln1"])
            if t == 1 and d == 128 and self.fuse_glue and b * self.hkv * 4 < self.n_sms:  # few sequences: rotary, cache write and attention in one launch
                att = rope_attention(qkv, pos0, self.k_cache[li], self.v_cache[li], self.hq, self.hkv, d, cfg.rope_theta)
            elif t == 1 and d == 128:
                q = rope_cache(qkv, pos0, self.k_cache[li], self.v_cache[li], b, t, self.hq, self.hkv, d, cfg.rope_theta)
                att = decode_attention(q, self.k_cache[li], self.v_cache[li], pos0)
            else:
                q = rope_cache(qkv, pos0, self.k_cache[li], self.v_cache[li], b, t, self.hq, self.hkv, d, cfg.rope_theta)
                p0 = int(pos0)
                att = F.scaled_dot_product_attention(q, self.k_cache[li][:, :, : p0 + t], self.v_cache[li][:, :, : p0 + t],
                                                     is_causal=(p0 == 0 and t > 1), enable_gqa=True)
                att = att.transpose(1, 2).reshape(b * t, self.hq * d)
            gate_up = norm_proj(L["gate_up"], L["o"](att, torch.float32), L["ln2"])
            delta = L["down"].fused(nv.PE_PRO_SILU_MUL, gate_up, torch.float32) if one else None
            if delta is None:
                delta = L["down"](silu_mul(gate_up, self.inter), torch.float32)
        if fold_norm:
            logits = self.head.fused(nv.PE_PRO_ADD_RMSNORM, x, torch.float32, delta=delta, norm_weight=self.final_ln,
                                     eps=cfg.rms_eps, resid_out=x_alt)
        else:
            logits = None
        if logits is None:
            h = reduce_add_norm(delta, self.final_ln).view(b, t, cfg.hidden)[:, -1]
            logits = self.head(h, torch.float32)                  # (B, vocab / tp)
        if return_logits:
            if self.tp == 1:
                return logits
            parts = [torch.empty_like(logits) for _ in range(self.tp)]
            dist.all_gather(parts, logits.contiguous(), group=self.group)
            return torch.cat(parts, dim=-1)
        val, idx = logits.max(dim=-1)
        if self.tp > 1:
            vals = [torch.empty_like(val) for _ in range(self.tp)]
            idxs = [torch.empty_like(idx) for _ in range(self.tp)]
            dist.all_gather(vals, val, group=self.group)
            dist.all_gather(idxs, idx + self.rank * (cfg.vocab // self.tp), group=self.group)
            best = torch.stack(vals, 0).argmax(0)
            idx = torch.stack(idxs, 0).gather(0, best[None])[0]
        return idx
