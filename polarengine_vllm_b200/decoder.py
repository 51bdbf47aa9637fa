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

from .decode_ops import add_rmsnorm, decode_attention, rope_cache, silu_mul
from .kernels import quant_embedding, quant_matmul, retile
from .packing import pack_codes_half_block
from .parallel import PeerExchange
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


class QWeight:
    """Synthetic quantized (out_f, in_f) weight resident on one device."""

    def __init__(self, out_f: int, in_f: int, bits: int, dev, gen: torch.Generator):
        ct = get_centroids(bits).to(dev)
        bounds = (ct[1:] + ct[:-1]) / 2
        codes = torch.empty(out_f, in_f, dtype=torch.int8, device=dev)
        step = max(1, (1 << 26) // in_f)
        for r0 in range(0, out_f, step):  # bounded temporaries for vocabulary-sized tables
            r1 = min(out_f, r0 + step)
            codes[r0:r1] = torch.bucketize(torch.randn(r1 - r0, in_f, device=dev, generator=gen), bounds).to(torch.int8)
        self.packed = bits <= 4
        self.codes = pack_codes_half_block(codes) if self.packed else codes
        self.norms = (0.02 * math.sqrt(128) * (1 + 0.05 * torch.randn(out_f, in_f // 128, device=dev, generator=gen))).half()
        self.ct = get_ct_scaled(bits).to(dev)
        self.tiles = retile(self.codes, self.packed, self.norms)  # streaming copy for decode-size batches
        self.out_f, self.in_f = out_f, in_f

    def __call__(self, x: torch.Tensor, out_dtype=torch.float16) -> torch.Tensor:
        return quant_matmul(self.codes, self.packed, self.norms, self.ct, x, False, self.out_f, self.in_f, self.in_f, out_dtype,
                            tiles=self.tiles)


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
        for li in range(cfg.n_layers):
            g = torch.Generator(device=dev).manual_seed(seed + 16 * li + 4099 * tp_rank)
            self.layers.append({
                "qkv": QWeight((self.hq + 2 * self.hkv) * d, cfg.hidden, cfg.bits_qkv, dev, g),
                "o": QWeight(cfg.hidden, self.hq * d, cfg.bits_o, dev, g),          # K slice of the row-parallel o
                "gate_up": QWeight(2 * self.inter, cfg.hidden, cfg.bits_gate_up, dev, g),
                "down": QWeight(cfg.hidden, self.inter, cfg.bits_down, dev, g),     # K slice of the row-parallel down
                "ln1": torch.ones(cfg.hidden, dtype=torch.float16, device=dev),
                "ln2": torch.ones(cfg.hidden, dtype=torch.float16, device=dev),
            })
        ge = torch.Generator(device=dev).manual_seed(seed + 900)  # same table on every rank
        self.embed = QWeight(cfg.vocab, cfg.hidden, cfg.bits_embed, dev, ge)
        assert cfg.vocab % tp_size == 0
        gh = torch.Generator(device=dev).manual_seed(seed + 901 + 4099 * tp_rank)
        self.head = QWeight(cfg.vocab // tp_size, cfg.hidden, cfg.bits_head, dev, gh)
        self.final_ln = torch.ones(cfg.hidden, dtype=torch.float16, device=dev)
        self.max_len, self.batch = max_len, batch
        # decode steps of a sharded model: all-reduce + residual add + norm as one launch over peer memory
        self.xchg = PeerExchange(dev, tp_rank, tp_size, max(batch, 1), cfg.hidden, group) if fused_allreduce else None
        self.k_cache = [torch.zeros(batch, self.hkv, max_len, d, dtype=torch.float16, device=dev) for _ in range(cfg.n_layers)]
        self.v_cache = [torch.zeros(batch, self.hkv, max_len, d, dtype=torch.float16, device=dev) for _ in range(cfg.n_layers)]

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

    def forward(self, ids: torch.Tensor, pos0) -> torch.Tensor:
        """ids (B, T) -> next-token ids (B,).  ``pos0`` is an int (prefill) or a 0-d device
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

        for li, L in enumerate(self.layers):
            h = add_rmsnorm(x, None, L["ln1"], cfg.rms_eps) if delta is None else reduce_add_norm(delta, L["ln1"])
            qkv = L["qkv"](h)
            q = rope_cache(qkv, pos0, self.k_cache[li], self.v_cache[li], b, t, self.hq, self.hkv, d, cfg.rope_theta)
            if t == 1 and d == 128:  # decode: one launch over the cache, length from the position scalar
                att = decode_attention(q, self.k_cache[li], self.v_cache[li], pos0)
            else:
                p0 = int(pos0)
                att = F.scaled_dot_product_attention(q, self.k_cache[li][:, :, : p0 + t], self.v_cache[li][:, :, : p0 + t],
                                                     is_causal=(p0 == 0 and t > 1), enable_gqa=True)
                att = att.transpose(1, 2).reshape(b * t, self.hq * d)
            h = reduce_add_norm(L["o"](att, torch.float32), L["ln2"])
            act = silu_mul(L["gate_up"](h), self.inter)
            delta = L["down"](act, torch.float32)
        h = reduce_add_norm(delta, self.final_ln).view(b, t, cfg.hidden)[:, -1]
        logits = self.head(h, torch.float32)                      # (B, vocab / tp)
        val, idx = logits.max(dim=-1)
        if self.tp > 1:
            vals = [torch.empty_like(val) for _ in range(self.tp)]
            idxs = [torch.empty_like(idx) for _ in range(self.tp)]
            dist.all_gather(vals, val, group=self.group)
            dist.all_gather(idxs, idx + self.rank * (cfg.vocab // self.tp), group=self.group)
            best = torch.stack(vals, 0).argmax(0)
            idx = torch.stack(idxs, 0).gather(0, best[None])[0]
        return idx
