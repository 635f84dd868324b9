"""The entry point that allocates nothing, against the regular one.

tcab_chain_reduce_noalloc exists for hosts that cannot let the library call cudaMalloc: a process
whose device memory is already handed out in full, code that runs while a stream is being captured,
a loop that cannot afford the device-wide synchronisation cudaMalloc implies. It runs the multi-CTA
split reduction with the partial results in a fixed array inside the library's device image instead
of a buffer from cudaMalloc. This file checks, through the C ABI, that it gives what
tcab_chain_reduce gives, on two calls in a row (the array is shared and keeps the first call's
contents), that it stays correct whichever of the two is called first in the process, and that it
turns away problems its fixed array cannot hold. The file name sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

import tcacomp_b200 as T

pytestmark = pytest.mark.gpu

EXPR = "(0.5f*p0 + 0.25f) * (0.5f*p0 + 0.25f)"


def _pair(dev, rows, cols, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    return torch.rand((rows, cols), generator=g, device=dev) * 2 - 1


def test_noalloc_matches_regular_entry_on_two_calls_in_a_row(oracle, cuda):
    from oracle import checks
    # two different problems back to back: the second call finds the first call's partials in the array
    x1 = _pair(cuda, 3, 400000, 1)
    x2 = _pair(cuda, 5, 123457, 2)   # odd length: the scalar path; fewer partial slots in use than before
    out1 = torch.full((3,), -12345.0, device=cuda)
    out2 = torch.full((5,), -12345.0, device=cuda)
    before = torch.cuda.memory_allocated(cuda)
    T.chain_reduce_noalloc([x1], EXPR, out=out1)
    T.chain_reduce_noalloc([x2], EXPR, out=out2)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(cuda) == before  # nothing came from torch's allocator either
    for x, got in ((x1, out1), (x2, out2)):
        want = T.chain_reduce([x], EXPR)                # the existing entry point
        g, w = got.cpu().numpy(), want.cpu().numpy()
        assert (np.abs(g - w) <= 1e-5 * np.abs(w)).all()
        assert checks.rowsum_close(g, x.cpu().numpy())  # and both against the oracle


def test_noalloc_other_combiners_init_and_piped_map(cuda):
    x = _pair(cuda, 4, 300000, 3)
    out = torch.empty((4,), device=cuda)
    T.chain_reduce_noalloc([x], "p0", out=out, combine_expr="fmaxf(p0, p1)", init=0.25)
    assert torch.equal(out, T.chain_reduce([x], "p0", combine_expr="fmaxf(p0, p1)", init=0.25))  # max: bit-exact
    z = _pair(cuda, 4, 300000, 4).abs()
    T.chain_reduce_noalloc([x, z], "(p0 * p0) * p1", out=out, post_expr="p0 * rsqrtf(p0 * c0 + c1)",
                           captures=(1.0 / 300000, 1e-5))
    want = T.chain_reduce([x, z], "(p0 * p0) * p1", post_expr="p0 * rsqrtf(p0 * c0 + c1)",
                          captures=(1.0 / 300000, 1e-5))
    assert torch.allclose(out, want, rtol=1e-5, atol=0)
    # short rows and a single element still go through the fixed array
    s = _pair(cuda, 7, 5, 5)
    o7 = torch.empty((7,), device=cuda)
    T.chain_reduce_noalloc([s], "p0", out=o7)
    assert torch.allclose(o7, s.sum(1), rtol=1e-6, atol=1e-6)
    e = torch.zeros((3, 0), device=cuda)
    o3 = torch.empty((3,), device=cuda)
    T.chain_reduce_noalloc([e], "p0", out=o3, init=2.5)
    assert (o3 == 2.5).all()  # an empty reduction returns init


def test_noalloc_rejects_what_its_array_cannot_hold(cuda):
    rows = T._lib.NOALLOC_MAX_ROWS + 1
    x = torch.zeros((rows, 8), device=cuda)
    out = torch.empty((rows,), device=cuda)
    with pytest.raises(T.TcabError) as e:
        T.chain_reduce_noalloc([x], "p0", out=out)
    assert e.value.status == T._lib.ERR_TOO_LARGE and "TCAB_NOALLOC_MAX_ROWS" in e.value.message
    ok = torch.ones((T._lib.NOALLOC_MAX_ROWS, 8), device=cuda)
    o = torch.empty((T._lib.NOALLOC_MAX_ROWS,), device=cuda)
    T.chain_reduce_noalloc([ok], "p0", out=o)  # exactly at the limit: one slot per row
    assert (o == 8).all()
    with pytest.raises(T.TcabError) as e:
        T.chain_reduce_noalloc([ok], "p0", out=torch.empty((3,), device=cuda))
    assert e.value.status == T._lib.ERR_SHAPE
