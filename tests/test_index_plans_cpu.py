"""Index arithmetic of three kernels restated on the host and swept: every element is visited exactly once.

The device code is the authority (tcacomp_b200/csrc/chain_kernels.cuh, reduce_outer.cu); these are the same
formulas in Python, so that a change of either side that breaks the cover shows up without a GPU. The GPU
parity tests check the results; these check the plan over many more shapes than a GPU test can afford.
"""
import ctypes as C

import numpy as np
import pytest


def ragged_row_cover(row, nk, tpr):
    """fold_row_share_ragged: thread t of tpr takes the row's whole 16-byte vectors t, t + tpr, ... and the edge
    elements t, t + tpr (two per thread with four threads per row, one otherwise)."""
    e0 = row * nk
    head = min((4 - (e0 & 3)) & 3, nk)
    v0 = (e0 + head) >> 2
    nfull = (nk - head) >> 2
    tail = nk - head - 4 * nfull
    edges = 1 if tpr >= 6 else 2
    seen = []
    for t in range(tpr):
        for q in range(edges):
            e = t + q * tpr
            if e < head + tail:
                seen.append(e0 + e if e < head else e0 + 4 * nfull + e)
        for idx in range(t, nfull, tpr):
            assert (v0 + idx) * 4 % 4 == 0                      # an aligned vector of the flat operand
            seen.extend(range(4 * (v0 + idx), 4 * (v0 + idx) + 4))
    return seen


@pytest.mark.parametrize("tpr", [4, 32, 256])
def test_ragged_rows_are_covered_once(tpr):
    rng = np.random.default_rng(tpr)
    shapes = [(r, nk) for nk in (65, 66, 67, 69, 127, 129, 255, 1023, 1025, 2563) for r in (0, 1, 2, 3, 7, 1000003)]
    shapes += [(int(rng.integers(0, 1 << 20)), int(rng.integers(65, 5000)) | 1) for _ in range(60)]
    for row, nk in shapes:
        if nk % 4 == 0:
            continue
        seen = ragged_row_cover(row, nk, tpr)
        assert sorted(seen) == list(range(row * nk, row * nk + nk)), (row, nk, tpr)


def rows32e_copy_cover(row_base, rows, nk):
    """chain_inner_rows32e: a warp's 32 rows start at element 32 m nk (a multiple of 32) and are copied as whole
    vectors; the last, shorter group of rows ends with up to three single elements."""
    nrows = min(32, rows - row_base)
    total = nrows * nk
    nvec = total >> 2
    e0 = row_base * nk
    assert e0 % 32 == 0
    seen = []
    for lane in range(32):
        for v in range(lane, nvec, 32):
            seen.extend(range(e0 + 4 * v, e0 + 4 * v + 4))
        if lane < (total & 3):
            seen.append(e0 + 4 * nvec + lane)
    return nrows, seen


def test_rows32e_copies_every_element_of_its_rows():
    for nk in (1, 2, 3, 5, 6, 7, 13, 33, 62, 63):
        for rows in (1, 31, 32, 33, 64, 95, 1027):
            for row_base in range(0, rows, 32):
                nrows, seen = rows32e_copy_cover(row_base, rows, nk)
                assert sorted(seen) == list(range(row_base * nk, (row_base + nrows) * nk)), (nk, rows, row_base)
                assert max(seen) < rows * nk                    # nothing beyond the operand


def flat_ranges_cover(nk, g, ksplit, klen, unroll):
    """chain_outer_flat / reduce_outer_flat with ksplit > 1: CTA `ks` takes rows [ks klen, min(nk, (ks + 1) klen)),
    its eight warps interleave steps of 32 / g rows times `unroll`."""
    rows_per_step = 32 // g
    seen = []
    for ks in range(ksplit):
        first = min(ks * klen, nk)
        kend = nk if nk - first < klen else first + klen
        for warp in range(8):
            kstep = rows_per_step * unroll
            kbeg = min(first + warp * kstep, kend)
            kstep *= 8
            for kr in range(rows_per_step):                    # the lanes' rows inside a step (lanes beyond g * (32 / g) idle)
                k0 = kbeg + kr
                while k0 < kend:
                    for u in range(unroll):
                        k = k0 + u * rows_per_step
                        if k < kend:
                            seen.append(k)
                    k0 += kstep
    return seen


def test_flat_ranges_visit_every_row_once(tcab_lib):
    for nb, nk, nc in [(1, 100003, 4), (1, 1 << 16, 16), (3, 50001, 8), (1, 70000, 12), (2, 9000, 20), (1, 4097, 64),
                       (1, 30000, 3), (1, 2049, 7), (5, 12345, 48)]:
        g, r, kl = C.c_uint32(), C.c_uint32(), C.c_uint32()
        assert tcab_lib.tcab_plan_outer_flat_ranges(nb, nk, nc, 148, 262144, C.byref(g), C.byref(r), C.byref(kl)) == 0
        assert g.value != 0 and r.value >= 1
        unroll = 4 if nc % 4 == 0 else 16
        seen = flat_ranges_cover(nk, g.value, r.value, kl.value, unroll) if r.value > 1 else list(range(nk))
        assert sorted(seen) == list(range(nk)), (nb, nk, nc, g.value, r.value, kl.value)
