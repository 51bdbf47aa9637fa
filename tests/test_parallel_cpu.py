"""Sharding helpers and the row-parallel reduction on two CPU ranks (gloo).  The shards
are evaluated with the CPU oracle; the product kernels are exercised by the GPU tests."""
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import polar_oracle as oracle
from polarengine_vllm_b200 import parallel
from polarengine_vllm_b200.utils import pack_codes_half_block


def test_shard_shapes_and_errors():
    codes = torch.arange(8 * 512, dtype=torch.int16).reshape(8, 512).to(torch.int8)
    norms = torch.arange(8 * 4, dtype=torch.float32).reshape(8, 4).half()
    assert parallel.shard_codes_for_tp(codes, 1, 2, dim=0).equal(codes[4:])
    assert parallel.shard_codes_for_tp(codes, 1, 2, dim=1).equal(codes[:, 256:])
    packed = pack_codes_half_block(codes & 15)
    assert parallel.shard_codes_for_tp(packed, 0, 4, dim=1, packed=True).equal(packed[:, :64])
    assert parallel.shard_norms_for_tp(norms, 1, 4, dim=1).equal(norms[:, 1:2])
    assert parallel.shard_norms_for_tp(norms, 0, 1) is norms
    with pytest.raises(ValueError):
        parallel.shard_codes_for_tp(codes, 0, 3, dim=1)       # 4 blocks over 3 ranks
    with pytest.raises(ValueError):
        parallel.shard_norms_for_tp(norms, 0, 3, dim=0)
    m = parallel.expert_placement(128, 3, 8)
    assert (m >= 0).sum() == 16 and m[48] == 0 and m[63] == 15 and m[64] == -1
    x = torch.randn(2, 300)
    assert parallel.shard_activation_for_row_parallel(x, 1, 3, 384).shape == (2, 128)


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        w = torch.randn(96, 512, generator=g) * 0.02
        q = oracle.quantize_tensor(w, 4)
        x = torch.randn(3, 512, generator=g).half()
        full = oracle.linear_dequant(x, q["codes"], q["norms"], q["ct_scaled"])
        packed = torch.from_numpy(oracle.pack_nibble(q["codes"].numpy()))
        # row parallel: K slices of the packed codes, partial products, one all-reduce
        c = parallel.shard_codes_for_tp(packed, rank, world, dim=1, packed=True)
        n = parallel.shard_norms_for_tp(q["norms"], rank, world, dim=1)
        xs = parallel.shard_activation_for_row_parallel(x, rank, world, 512)
        part = oracle.linear_dequant(xs, torch.from_numpy(oracle.unpack_nibble(c.numpy())), n, q["ct_scaled"])
        dist.all_reduce(part)
        row_err = float((part - full).abs().max() / full.abs().max())
        # column parallel: row slices, all-gather
        c = parallel.shard_codes_for_tp(q["codes"], rank, world, dim=0)
        n = parallel.shard_norms_for_tp(q["norms"], rank, world, dim=0)
        loc = oracle.linear_dequant(x, c, n, q["ct_scaled"])
        parts = [torch.empty_like(loc) for _ in range(world)]
        dist.all_gather(parts, loc)
        col_err = float((torch.cat(parts, 1) - full).abs().max() / full.abs().max())
        if rank == 0:
            ret["row"], ret["col"] = row_err, col_err
    finally:
        dist.destroy_process_group()


def test_row_and_column_parallel_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = 29500 + os.getpid() % 500
        procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
            assert p.exitcode == 0
        assert ret["row"] < 1e-5 and ret["col"] < 1e-6


def _moe_worker(rank, world, port, ret):
    """Expert parallel: every rank evaluates only the experts its placement map keeps
    (oracle arithmetic), the all-reduce restores the full layer output."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        e, h, i, k, t = 8, 256, 128, 2, 12
        g = torch.Generator().manual_seed(5)
        experts = []
        for _ in range(e):
            ex = {}
            for name, (rows, cols, bits) in {"gate": (i, h, 3), "up": (i, h, 3), "down": (h, i, 4)}.items():
                q = oracle.quantize_tensor(torch.randn(rows, cols, generator=g) * 0.02, bits)
                ex[name] = (q["codes"], q["norms"], q["ct_scaled"], cols)
            experts.append(ex)
        x = torch.randn(t, h, generator=g).half()
        w, ids = oracle.moe_route(x, (torch.randn(e, h, generator=g) * 0.02).half(), k)
        full = oracle.moe_forward(x, w, ids, experts)
        emap = parallel.expert_placement(e, rank, world)
        local = emap[ids] >= 0                                   # pairs whose expert lives here
        part = oracle.moe_forward(x, w * local, ids, experts)     # remote pairs weigh nothing
        dist.all_reduce(part)
        if rank == 0:
            ret["moe"] = float((part - full).abs().max() / full.abs().max())
            ret["share"] = int(local.sum())
    finally:
        dist.destroy_process_group()


def test_expert_parallel_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        ret = mgr.dict()
        port = 30100 + os.getpid() % 500
        procs = [ctx.Process(target=_moe_worker, args=(r, 2, port, ret)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
        assert ret["moe"] < 1e-5 and 0 < ret["share"] < 24


def test_expected_local_pairs():
    from polarengine_vllm_b200.moe_method import PolarQuantMoEMethod as M
    assert M.expected_local_pairs(512, 128, None) == 512
    assert M.expected_local_pairs(512, 16, parallel.expert_placement(128, 0, 8)) == 64
    assert M.expected_local_pairs(3, 16, parallel.expert_placement(128, 0, 8)) == 1
