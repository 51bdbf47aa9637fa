"""Tensor-parallel and expert-parallel placement of quantized layers.

Reference: polarengine_vllm/loader.py:558-638 (``shard_codes_for_tp`` /
``shard_norms_for_tp``): pure slicing, no collectives (the all-reduce after a
row-parallel layer is vLLM's).  Output rows are independent units and every 128-block
of K is independent (rotation and nibble packing are block-local), so

* column parallel (q/k/v, gate/up, LM head): rows ``[r0, r1)`` of codes and norms; no
  exchange;
* row parallel (o, down): whole blocks ``[b0, b1)`` of K -- ``codes[:, b0*128 : b1*128]``
  (``packed[:, b0*64 : b1*64]`` for nibbles), ``norms[:, b0:b1]`` -- each rank rotates only
  its slice of the activations; ONE all-reduce of the partial outputs follows.

Unlike the reference helper, the K split returns the rank's slice (the reference returns
the full tensor for ``dim=1``) and refuses splits that would cut a block.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def _bounds(total: int, rank: int, world: int, what: str) -> Tuple[int, int]:
    if total % world:
        raise ValueError(f"{what} ({total}) is not divisible by the tensor-parallel size ({world})")
    step = total // world
    return rank * step, (rank + 1) * step


def shard_codes_for_tp(codes: torch.Tensor, tp_rank: int, tp_size: int, dim: int = 0, packed: bool = False,
                       block_size: int = 128) -> torch.Tensor:
    """Rank's slice of a codes tensor.  dim 0 = output rows, dim 1 = input features."""
    if tp_size == 1:
        return codes
    if dim == 0:
        lo, hi = _bounds(codes.shape[0], tp_rank, tp_size, "out_features")
        return codes[lo:hi].contiguous()
    per_block = block_size // 2 if packed else block_size
    if codes.shape[1] % per_block:
        raise ValueError("codes width is not a whole number of blocks")
    lo, hi = _bounds(codes.shape[1] // per_block, tp_rank, tp_size, "n_blocks")
    return codes[:, lo * per_block:hi * per_block].contiguous()


def shard_norms_for_tp(norms: torch.Tensor, tp_rank: int, tp_size: int, dim: int = 0) -> torch.Tensor:
    if tp_size == 1:
        return norms
    lo, hi = _bounds(norms.shape[dim], tp_rank, tp_size, "out_features" if dim == 0 else "n_blocks")
    return (norms[lo:hi] if dim == 0 else norms[:, lo:hi]).contiguous()


def shard_activation_for_row_parallel(x: torch.Tensor, tp_rank: int, tp_size: int, in_f_padded: int) -> torch.Tensor:
    """Columns of x that feed this rank's K slice (x zero-padded to in_f_padded first if ragged)."""
    if x.shape[-1] < in_f_padded:
        x = torch.nn.functional.pad(x, (0, in_f_padded - x.shape[-1]))
    lo, hi = _bounds(in_f_padded // 128, tp_rank, tp_size, "n_blocks")
    return x[..., lo * 128:hi * 128]


def expert_placement(num_experts: int, ep_rank: int, ep_size: int) -> torch.Tensor:
    """int64 map global expert -> local index on this rank, -1 elsewhere (contiguous blocks)."""
    lo, hi = _bounds(num_experts, ep_rank, ep_size, "num_experts")
    m = torch.full((num_experts,), -1, dtype=torch.long)
    m[lo:hi] = torch.arange(hi - lo)
    return m


class QuantLinearShard:
    """One rank's piece of a quantized linear layer plus its collective.

    ``mode`` "column": y_local = x @ W[r0:r1].T (no exchange; ``gather_output`` optional).
    ``mode`` "row": y = all_reduce(x[:, k0:k1] @ W[:, k0:k1].T); bias is added on rank 0 only.
    """

    def __init__(self, codes, packed, norms, ct_scaled, out_f, in_f, mode: str, group=None):
        assert mode in ("column", "row")
        self.codes, self.packed, self.norms, self.ct = codes, packed, norms, ct_scaled
        self.out_f, self.in_f, self.mode, self.group = out_f, in_f, mode, group

    @classmethod
    def from_full(cls, codes, packed, norms, ct_scaled, mode, rank, world, group=None):
        dim = 0 if mode == "column" else 1
        c = shard_codes_for_tp(codes, rank, world, dim, packed)
        n = shard_norms_for_tp(norms, rank, world, dim)
        return cls(c, packed, n, ct_scaled, c.shape[0], n.shape[1] * 128, mode, group)

    def forward(self, x_local: torch.Tensor, bias: Optional[torch.Tensor] = None, out_dtype=torch.float16) -> torch.Tensor:
        import torch.distributed as dist
        from .kernels import quant_matmul
        if self.mode == "column":
            return quant_matmul(self.codes, self.packed, self.norms, self.ct, x_local, False, self.out_f, self.in_f,
                                self.in_f, out_dtype, bias)
        rank = dist.get_rank(self.group) if dist.is_initialized() else 0
        y = quant_matmul(self.codes, self.packed, self.norms, self.ct, x_local, False, self.out_f, self.in_f, self.in_f,
                         torch.float32, bias if rank == 0 else None)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y, group=self.group)
        return y.to(out_dtype)


class PeerExchange:
    """Exchange buffers of the fused all-reduce + residual add + RMSNorm kernel
    (``pe_allreduce_add_rmsnorm``): one buffer per rank, mapped into every rank.

    With one rank the buffer is ordinary device memory (the kernel then exchanges with
    itself, which is how the protocol is tested on a single GPU).  With several ranks the
    buffers come from torch's symmetric-memory allocator, which only provides the peer
    mappings; every load and store on them is issued by the kernel of this package.
    """

    def __init__(self, device, rank: int, world: int, max_rows: int, hidden: int, group=None):
        from . import _native as nv
        self.rank, self.world, self.max_rows, self.hidden = rank, world, max_rows, hidden
        nbytes = nv.lib().pe_allreduce_buffer_bytes(world, max_rows, hidden)
        if nbytes == 0:
            raise ValueError("exchange buffer: unsupported world size / rows / hidden")
        if world == 1:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            ptrs = [self.buf.data_ptr()]
        else:
            import os
            import torch.distributed as dist
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer mappings only
            import torch.distributed._symmetric_memory as symm_mem
            self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
            self.buf.zero_()
            handle = symm_mem.rendezvous(self.buf, group if group is not None else dist.group.WORLD)
            ptrs = [int(p) for p in handle.buffer_ptrs]
            self._handle = handle
            torch.cuda.synchronize(device)
            dist.barrier(group)  # every buffer reads zero before anyone's first launch
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.seq = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)

    def allreduce_add_rmsnorm(self, partial: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        """x (rows, hidden) fp16 += fp16(sum over ranks of partial (rows, hidden) fp32), in place;
        returns RMSNorm(x) * weight.  Every rank must make the same sequence of calls."""
        from . import _native as nv
        rows, hidden = x.shape
        if hidden != self.hidden or rows > self.max_rows or partial.shape != x.shape:
            raise ValueError("exchange: shape does not fit the buffer")
        if partial.dtype != torch.float32 or x.dtype != torch.float16 or not partial.is_contiguous() or not x.is_contiguous():
            raise ValueError("exchange: fp32 partials and an fp16 residual stream, both contiguous")
        out = torch.empty_like(x)
        nv.check(nv.lib().pe_allreduce_add_rmsnorm(partial.data_ptr(), x.data_ptr(), weight.data_ptr(), out.data_ptr(), rows, hidden,
                                                   float(eps), self.peers.data_ptr(), self.rank, self.world, self.max_rows,
                                                   self.seq.data_ptr(), self.status.data_ptr(), nv.stream_ptr(x.device)),
                 "pe_allreduce_add_rmsnorm")
        return out

    def timed_out(self) -> bool:
        """True if any call so far gave up waiting for a peer (reads the status word back)."""
        return bool(int(self.status.item()))
