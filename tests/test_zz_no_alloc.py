"""The allocation-free attention entry point, for hosts that cannot call cudaMalloc while they
serve (all of HBM already belongs to their own pool, or allocation is forbidden because it
synchronises the device).  It must give exactly what dc_sparse_attend gives with a caller's
scratch buffer — its scratch is a fixed array inside the library that every call shares and that
still holds the previous call's partials, so the check is repeated on a second, different call.

This file sorts last on purpose: a run that stops at the first failure has then already run
every other test."""
import numpy as np
import pytest
import torch

from tests import util

pytestmark = pytest.mark.gpu


def _problem(seed, P, G, D, n, n_sel, res_len):
    Hkv = 2
    k, v, q = util.small_problem(P // Hkv, Hkv, G, n, D, seed=seed)
    rng = np.random.default_rng(seed)
    sel = np.stack([rng.permutation(n)[:n_sel] for _ in range(P)]).astype(np.int32)
    res = torch.randn(2, P // Hkv, Hkv, res_len + 1, D, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)
    new = torch.randn(2, P, D, generator=torch.Generator().manual_seed(seed + 1)).to(torch.bfloat16)
    return dict(P=P, Hkv=Hkv, G=G, D=D, n=n, n_sel=n_sel, res_len=res_len, k=k.cuda().reshape(P, n, D),
                v=v.cuda().reshape(P, n, D), q=q.cuda(), sel=torch.from_numpy(sel).cuda(), res_k=res[0].cuda(),
                res_v=res[1].cuda(), k_new=new[0].cuda(), v_new=new[1].cuda())


def _attend(lib, pr, noalloc: bool):
    P, G, D = pr["P"], pr["G"], pr["D"]
    out = torch.zeros((P * G, D), dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(P * G, dtype=torch.float32, device="cuda")
    rk, rv = pr["res_k"].clone(), pr["res_v"].clone()
    sb, sh = rk.stride(0), rk.stride(1)
    st = int(torch.cuda.current_stream().cuda_stream)
    head = (pr["k"].data_ptr(), pr["v"].data_ptr(), pr["n"] * D, pr["n"], P, pr["Hkv"], G, D, 0, pr["q"].data_ptr(),
            pr["sel"].data_ptr(), pr["n_sel"], pr["n_sel"], 0, pr["k_new"].data_ptr(), pr["v_new"].data_ptr(),
            rk.data_ptr(), rv.data_ptr(), sb, sh, pr["res_len"], 0.0, out.data_ptr(), lse.data_ptr(), None, None)
    if noalloc:
        # what the name promises: device memory in use is the same after the call as before it.  The
        # scratch variant ran first, so the kernels are already loaded; nothing between the two readings
        # allocates through torch.  (Repeated so that a one-off change made by something else on the
        # device cannot fail the test.)
        for attempt in range(3):
            free_before = torch.cuda.mem_get_info()[0]
            rc = lib.dc_sparse_attend_noalloc(*head, st)
            torch.cuda.synchronize()
            free_after = torch.cuda.mem_get_info()[0]
            if rc != 0 or free_after >= free_before:
                break
        assert rc != 0 or free_after >= free_before, f"free device memory fell from {free_before} to {free_after}"
    else:
        scratch = torch.zeros(int(lib.dc_attend_scratch_bytes(P, G, D)), dtype=torch.uint8, device="cuda")
        rc = lib.dc_sparse_attend(*head, scratch.data_ptr(), st)
    assert rc == 0, lib.dc_last_error()
    torch.cuda.synchronize()
    return out.cpu(), lse.cpu(), rk.cpu()


def test_noalloc_attention_equals_scratch_attention_twice():
    from diffcache_b200 import _lib

    lib = _lib.load()
    # two calls in a row with different shapes: the second one finds the first one's partials in the array
    for pr in (_problem(91, 8, 4, 128, 3000, 700, 40), _problem(92, 4, 7, 128, 2000, 333, 17)):
        want_out, want_lse, want_rk = _attend(lib, pr, noalloc=False)
        got_out, got_lse, got_rk = _attend(lib, pr, noalloc=True)
        # same kernels, same split, same summation order: the 16-bit outputs must be identical;
        # the tolerance the other attention tests use (2e-3 rel / 1e-3 abs) is the fallback bound
        assert torch.allclose(got_out.float(), want_out.float(), rtol=2e-3, atol=1e-3)
        assert torch.equal(got_out, want_out)
        assert torch.allclose(got_lse, want_lse, rtol=1e-6, atol=1e-6)
        assert torch.equal(got_rk, want_rk)  # the new token was appended the same way


def test_noalloc_rejects_problems_beyond_the_static_array():
    from diffcache_b200 import _lib

    lib = _lib.load()
    pr = _problem(93, 4, 4, 128, 256, 64, 4)
    st = int(torch.cuda.current_stream().cuda_stream)
    out = torch.zeros((4 * 4, 128), dtype=torch.bfloat16, device="cuda")
    # 8192 problems x 8 heads x head_dim 256 needs tens of MB of partials: refused before any launch
    rc = lib.dc_sparse_attend_noalloc(pr["k"].data_ptr(), pr["v"].data_ptr(), 256 * 256, 256, 8192, 2, 8, 256, 0,
                                      pr["q"].data_ptr(), pr["sel"].data_ptr(), 64, 64, 0, None, None, None, None, 0, 0,
                                      0, 0.0, out.data_ptr(), None, None, None, st)
    assert rc == -1
    msg = lib.dc_last_error().decode()
    assert "DC_NOALLOC_SCRATCH_BYTES" in msg and "bytes" in msg
    torch.cuda.synchronize()
