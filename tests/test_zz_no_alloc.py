"""pe_gemv_noalloc: the decode matmul for hosts that cannot allocate device memory.

A serving process usually hands all free HBM to its own cache when it starts; code that
runs later, inside a layer, may find cudaMalloc failing and has no allocator of its own.
This entry point therefore takes no scratch buffer: it uses an 8 MiB array that ships
inside the library.  The test calls it through the C ABI twice in a row (two different
shapes, so the second call sees the first one's leftovers in the shared array) and checks
each result against the ordinary pe_gemv entry point on the same inputs.
"""
import pytest
import torch

import polar_oracle as oracle
from helpers import max_rel, rand_layer, rand_x

pytestmark = pytest.mark.gpu
TOL = 1e-2  # same bound as the other parity tests


def _both(n, k, bits, batch, seed):
    from polarengine_vllm_b200 import _native as nv, packing
    dev = torch.device("cuda")
    nv.ensure_init(dev)
    lib = nv.lib()
    codes, norms, cts = rand_layer(n, k, bits, seed)
    x = rand_x(batch, k, seed + 1).to(dev)
    packed = bits <= 4
    w = packing.pack_codes_half_block(codes.to(dev)) if packed else codes.to(dev)
    nd, cd = norms.to(dev), cts.to(dev)
    st = nv.stream_ptr(dev)
    common = lambda y: (w.data_ptr(), int(packed), w.stride(0), nd.data_ptr(), nd.stride(0), cd.data_ptr(), cd.numel(),
                        x.data_ptr(), nv.PE_X_RAW, nv.PE_F16, x.stride(0), k, y.data_ptr(), nv.PE_F32, y.stride(0),
                        None, batch, n, k)
    y_ref = torch.empty(batch, n, device=dev)
    need = lib.pe_gemv_workspace_bytes(batch, n, k)
    ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    nv.check(lib.pe_gemv(*common(y_ref), ws.data_ptr(), ws.numel(), st), "pe_gemv")
    y_new = torch.full((batch, n), float("nan"), device=dev)
    # One call first (it looks up the array's address and lets the driver finish loading the kernels), then
    # the free device memory the driver reports must not move across a further call: that figure sees an
    # allocation made by anybody in the process, the library included.  (By reading, the entry point calls
    # cudaGetDevice, cudaGetSymbolAddress once, cudaMemsetAsync and the kernel launch, nothing that allocates.)
    nv.check(lib.pe_gemv_noalloc(*common(y_new), st), "pe_gemv_noalloc")
    torch.cuda.synchronize()
    y_new.fill_(float("nan"))
    free_before, _ = torch.cuda.mem_get_info(dev)
    nv.check(lib.pe_gemv_noalloc(*common(y_new), st), "pe_gemv_noalloc")
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before
    assert lib.pe_gemv_noalloc_status(0, st) == 0   # no bounded wait ran out
    cpu_ref = oracle.linear_dequant(x.cpu(), codes, norms, cts)
    return y_new, y_ref, cpu_ref


def test_noalloc_matches_pe_gemv_on_two_calls_in_a_row():
    # the tile kernel (uses the array's counters and partials), again with another shape, then a batch-1 layer
    # (row-owning kernel: only the status word of the array is involved)
    for n, k, bits, batch, seed in [(4096, 12288, 4, 3, 11), (6144, 4096, 5, 16, 12), (4096, 4096, 4, 1, 13)]:
        y_new, y_ref, cpu_ref = _both(n, k, bits, batch, seed)
        assert torch.isfinite(y_new).all()
        assert max_rel(y_new, y_ref) <= TOL
        assert torch.equal(y_new, y_ref)          # same kernel, same split: bit-identical
        assert max_rel(y_new, cpu_ref) <= TOL


def test_noalloc_rejects_shapes_beyond_its_array():
    from polarengine_vllm_b200 import _native as nv
    lib = nv.lib()
    assert lib.pe_gemv_noalloc_max_bytes() == 8 << 20
    assert lib.pe_gemv_workspace_bytes(16, 151936, 4096) > lib.pe_gemv_noalloc_max_bytes()
    d = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p = d.data_ptr()
    rc = lib.pe_gemv_noalloc(p, 0, 4096, p, 32, p, 64, p, nv.PE_X_RAW, nv.PE_F16, 4096, 4096, p, nv.PE_F32, 151936,
                             None, 16, 151936, 4096, None)
    assert rc == -7 and lib.pe_error_string(rc) == b"size beyond a compiled-in maximum"
