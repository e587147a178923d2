"""The allocation-free sort entry point, through the C ABI, against the ordinary one.

cgx_sort_pairs_static keeps its scratch in a fixed array inside the library, for callers that are not allowed
to allocate device memory when they sort (fixed memory budgets, frozen pools, allocator-free latency paths).
It has to give exactly the pairs cgx_sort_pairs gives, call after call, although every call reuses the same
scratch bytes.  This file sorts last on purpose, so a run that stops at the first failure has already run
every other test."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _sorted_both_ways(n, end_bit, seed, dev, tiles_max=7500):
    from diff_gaussian_rasterization import _lib

    l = _lib.lib()
    gen = torch.Generator().manual_seed(seed)
    tiles = torch.randint(0, tiles_max, (n,), generator=gen, dtype=torch.int64)
    depth = torch.rand(n, generator=gen).mul(50).add(0.1).view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    keys = ((tiles << 32) | depth).to(dev)
    vals = torch.arange(n, dtype=torch.int32, device=dev)
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run(static):
        kin, vin = keys.clone(), vals.clone()
        kout, vout = torch.empty_like(kin), torch.empty_like(vin)
        if static:
            rc = l.cgx_sort_pairs_static(n, end_bit, kin.data_ptr(), vin.data_ptr(), kout.data_ptr(), vout.data_ptr(), st)
        else:
            ws = torch.empty(l.cgx_sort_workspace_bytes(n), dtype=torch.uint8, device=dev)
            rc = l.cgx_sort_pairs(n, end_bit, kin.data_ptr(), vin.data_ptr(), kout.data_ptr(), vout.data_ptr(),
                                  ws.data_ptr(), ws.numel(), st)
        assert rc == 0
        torch.cuda.synchronize()
        return kout.cpu(), vout.cpu()

    return run(False), run(True), keys.cpu()


def test_static_sort_matches_workspace_sort_twice_in_a_row(cuda_device):
    # two different inputs back to back: the second call finds the first call's leftovers in the scratch
    for n, seed in ((1_000_003, 11), (300_001, 12)):
        (k_ref, v_ref), (k_st, v_st), keys = _sorted_both_ways(n, 45, seed, cuda_device)
        assert torch.equal(k_st, k_ref) and torch.equal(v_st, v_ref)          # integer work: bit-exact
        order = torch.sort(keys & ((1 << 45) - 1), stable=True)[1]
        assert torch.equal(v_st.long(), order)


def test_static_sort_at_its_ceiling_with_the_widest_keys(cuda_device):
    # exactly as many pairs as the fixed scratch is sized for, keys of a 3840x2160 tile grid (47 sorted bits)
    n = 1 << 22
    (k_ref, v_ref), (k_st, v_st), keys = _sorted_both_ways(n, 47, 13, cuda_device, tiles_max=32400)
    assert torch.equal(k_st, k_ref) and torch.equal(v_st, v_ref)
    order = torch.sort(keys & ((1 << 47) - 1), stable=True)[1]
    assert torch.equal(v_st.long(), order)


def test_static_sort_rejects_sizes_beyond_its_scratch(cuda_device):
    from diff_gaussian_rasterization import _lib

    l = _lib.lib()
    limit = l.cgx_sort_pairs_static_max()
    assert limit == 1 << 22
    rc = l.cgx_sort_pairs_static(limit + 1, 45, None, None, None, None, None)
    assert rc == _lib.CGX_ENOMEM
    assert b"fixed scratch" in l.cgx_last_cuda_error()
