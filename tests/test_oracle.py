"""CPU tests of the oracle: golden vectors, the reference's test expressions, and the
C restatement of the kernel arithmetic against the torch restatement."""
import math

import numpy as np
import torch

from conftest import load_golden, tol_ratio
from oracle import c_oracle as CO
from oracle import ref_semantics as R


def f32(a):
    return torch.from_numpy(np.asarray(a)).float()


def test_exact_bmm_golden():
    g = load_golden("exact_bmm")
    A, B = f32(g["A"]), f32(g["B"])
    want = torch.from_numpy(g["C"]).float()
    assert torch.equal(R.bmm(A, B), want)
    assert torch.equal(CO.bmm(A, B), want)
    assert torch.equal(R.bmm(A[0], B[0]), want[0])  # 2-D inputs (bmm.py:78-81,127-129)


def test_exact_min_golden_and_tie_rule():
    g = load_golden("exact_min")
    A, B = f32(g["A"]), f32(g["B"])
    for dim in (1, 2):
        wv, wi = f32(g[f"v_dim{dim}"]), torch.from_numpy(g[f"i_dim{dim}"])
        for impl in (R.min_bmm, lambda a, b, dim: CO.min_bmm(a, b, dim)):
            v, i = impl(A, B, dim=dim)
            assert torch.equal(v, wv)
            assert torch.equal(i, wi)
    # planted ties: columns 200.. duplicate columns 0.., so no dim-2 answer may be >= 200
    assert int(torch.from_numpy(g["i_dim2"]).max()) < 200
    assert int(torch.from_numpy(g["i_dim1"]).max()) < 140
    # 2-D inputs: dim is bumped by one (minbmm.py:86-90)
    v, i = R.min_bmm(A[0], B[0], dim=1)
    assert torch.equal(v, f32(g["v_dim2"])[0]) and torch.equal(i, torch.from_numpy(g["i_dim2"])[0])


def test_exact_topk_golden():
    g = load_golden("exact_topk")
    A, B, k = f32(g["A"]), f32(g["B"]), int(g["k"])
    for dim in (1, 2):
        want = f32(g[f"v_dim{dim}"])
        v, i = R.topk_bmm(A, B, k=k, dim=dim)
        assert torch.equal(v, want)
        cv, ci = CO.topk_bmm(A, B, k, dim)
        assert torch.equal(cv, want)
        R.check_topk(cv, ci, A, B, k, dim)
    # output layout: k is the last axis for both dims (topkbmm.py:119-127)
    assert R.topk_bmm(A, B, k=k, dim=1)[0].shape == (1, B.shape[2], k)
    assert R.topk_bmm(A, B, k=k, dim=2)[0].shape == (1, A.shape[1], k)


def test_topk_short_rows_pad():
    g = load_golden("exact_topk_short")
    A, B, k = f32(g["A"]), f32(g["B"]), int(g["k"])
    v, i = R.topk_bmm(A, B, k=k, dim=2)
    assert torch.equal(v, torch.from_numpy(g["v_dim2"])) and torch.equal(i, torch.from_numpy(g["i_dim2"]))
    assert bool(torch.isneginf(v[..., 5:]).all()) and bool((i[..., 5:] == -1).all())
    cv, ci = CO.topk_bmm(A, B, k, 2)
    assert torch.equal(cv, v)
    assert bool((ci[..., 5:] == -1).all())


def test_exact_mbmm_golden():
    g = load_golden("exact_mbmm")
    A, B = f32(g["A"]), f32(g["B"])
    l, m, _ = A.shape
    n = B.shape[2]
    mask = torch.from_numpy(np.unpackbits(g["mask"], axis=-1)[..., :n].astype(bool))
    want = torch.from_numpy(g["C"]).float()
    bm, tm, em = R.make_masks(mask)
    assert bm.shape == (l, math.ceil(m / 128), math.ceil(n / 128)) and tm.shape == (l, math.ceil(m / 8), math.ceil(n / 8))
    assert bm.dtype == tm.dtype == em.dtype == torch.uint8
    assert torch.equal(R.mbmm(A, B, bm, tm, em), want)
    assert torch.equal(CO.mbmm(A, B, bm, tm, em), want)
    # the reference's own check expression (colab/test_mbmm.ipynb:1342-1343)
    assert torch.equal(torch.bmm(A, B).masked_fill_(~mask, 0), want)
    # fixture really holds an all-masked, an all-kept and a single-element tile
    assert int(bm[0, 0, 1]) == 0 and int(tm[0, :16, 32:].min()) == 64 and int(em[0, 128:256, :128].sum()) == 1


def test_mask_precedence_block_over_thread_over_element():
    """Inconsistent masks: the block mask wins, then the thread mask, then the element
    byte multiplies (kernels/mbmm.cu:251-255,360-363,111-133)."""
    A, B = R.exact_inputs(1, 128, 8, 256, seed=3)
    em = torch.ones(1, 128, 256, dtype=torch.uint8)
    tm = torch.ones(1, 16, 32, dtype=torch.uint8)
    bm = torch.ones(1, 1, 2, dtype=torch.uint8)
    bm[0, 0, 1] = 0
    tm[0, 2, 3] = 0
    em[0, 5, 7] = 3
    full = torch.bmm(A, B)
    for C in (R.mbmm(A, B, bm, tm, em), CO.mbmm(A, B, bm, tm, em)):
        assert bool((C[0, :, 128:] == 0).all())
        assert bool((C[0, 16:24, 24:32] == 0).all())
        assert float(C[0, 5, 7]) == 3 * float(full[0, 5, 7])
        assert torch.equal(C[0, 64:, :128], full[0, 64:, :128])


def test_share_mask():
    A, B = R.exact_inputs(3, 130, 8, 140, seed=4)
    mask = torch.tril(torch.ones(130, 140, dtype=torch.bool))
    bm, tm, em = R.make_masks(mask)
    assert bm.dim() == 2
    C = R.mbmm(A, B, bm, tm, em, share_mask=True)
    assert torch.equal(C, torch.bmm(A, B).masked_fill_(~mask[None].expand(3, -1, -1), 0))
    assert torch.equal(CO.mbmm(A, B, bm, tm, em, share_mask=True), C)


def test_randn_golden_against_both_restatements():
    g = load_golden("randn_small")
    A, B, k = torch.from_numpy(g["A"]), torch.from_numpy(g["B"]), int(g["k"])
    assert tol_ratio(R.bmm(A, B), torch.from_numpy(g["C"])) <= 1e-3  # same code path: near bit-equal
    assert tol_ratio(CO.bmm(A, B), torch.from_numpy(g["C"])) <= 1.0   # fma chain vs blocked sgemm
    for dim in (1, 2):
        v, i = CO.min_bmm(A, B, dim)
        R.check_min(v, i, A, B, dim)
        assert torch.equal(i, torch.from_numpy(g[f"min_i{dim}"]))
        v, i = CO.topk_bmm(A, B, k, dim)
        R.check_topk(v, i, A, B, k, dim)
        assert tol_ratio(v, torch.from_numpy(g[f"topk_v{dim}"])) <= 1.0


def test_dim1_is_rowwise_reduction_of_transposed_product():
    g = torch.Generator().manual_seed(5)
    A, B = torch.randn(2, 33, 20, generator=g), torch.randn(2, 20, 47, generator=g)
    v1, i1 = R.min_bmm(A, B, dim=1)
    v2, i2 = R.min_bmm(B.transpose(1, 2), A.transpose(1, 2), dim=2)
    assert tol_ratio(v1, v2) <= 1.0 and torch.equal(i1, i2)


def test_comparators_reject_wrong_answers():
    g = torch.Generator().manual_seed(6)
    A, B = torch.randn(1, 16, 8, generator=g), torch.randn(1, 8, 32, generator=g)
    v, i = R.min_bmm(A, B, dim=2)
    R.check_min(v, i, A, B, 2)
    bad = i.clone()
    bad[0, 0] = (bad[0, 0] + 1) % 32
    try:
        R.check_min(v, bad, A, B, 2)
        raise RuntimeError("comparator accepted a wrong index")
    except AssertionError:
        pass
    tv, ti = R.topk_bmm(A, B, k=4, dim=2)
    R.check_topk(tv, ti, A, B, 4, 2)
    try:
        R.check_topk(tv + 1e-2, ti, A, B, 4, 2)
        raise RuntimeError("comparator accepted wrong values")
    except AssertionError:
        pass


def test_config_generators_are_seeded_and_shaped():
    a = R.make_inputs("c1", rows=64, cols=96)
    b = R.make_inputs("c1", rows=64, cols=96)
    assert torch.equal(a["A"], b["A"]) and a["A"].shape == (1, 64, 64) and a["B"].shape == (1, 64, 96)
    c3 = R.make_inputs("c3", batches=4, rows=256, cols=256)
    assert c3["mask"].shape == (4, 256, 256) and bool(c3["mask"][0, 0, 0]) and not bool(c3["mask"][0, 0, 1])
    t = c3["mask"][2:].view(2, 4, 64, 4, 64)
    assert bool((t.all(dim=(2, 4)) | (~t).all(dim=(2, 4))).all())  # 64x64 tiles are uniform
    c2 = R.make_inputs("c2", batches=1, rows=8, cols=8)
    assert float(c2["A"].abs().max()) <= 1.0
    assert R.flops(*R.CONFIG_SHAPES["c1"]) == 2.0 * 16384 * 16384 * 64


def test_l2_distance_restatements_agree():
    """squared_l2 (kernels/bmm_helpers.cu:28-35): the torch restatement (direct formula) and
    the C restatement (fmaf chain) agree, and both equal |a|^2 + |b|^2 - 2 a.b in fp64."""
    A, B = R.exact_inputs(2, 20, 6, 30, seed=8, lo=-3, hi=3)
    D = R.product(A, B, "l2")
    ref = (A.double() ** 2).sum(-1)[:, :, None] + (B.double() ** 2).sum(1)[:, None, :] - 2 * torch.bmm(A.double(), B.double())
    assert torch.equal(D.double(), ref)
    for dim in (1, 2):
        v, i = R.min_bmm(A, B, dim=dim, distance="l2")
        cv, ci = CO.min_bmm(A, B, dim, distance="l2")
        assert torch.equal(v, cv) and torch.equal(i, ci)
        tv, _ = R.topk_bmm(A, B, k=4, dim=dim, distance="l2")
        ctv, cti = CO.topk_bmm(A, B, 4, dim, distance="l2")
        assert torch.equal(tv, ctv)
        R.check_topk(ctv, cti, A, B, 4, dim, distance="l2")


def test_kmeans_oracle_step():
    """The k-means restatement on a case small enough to do by hand."""
    X = torch.tensor([[0., 0.], [0., 2.], [10., 10.], [10., 12.], [5., 5.]])
    C = torch.tensor([[0., 1.], [10., 11.], [100., 100.]])
    v, i = R.kmeans_assign(X, C)
    assert i.tolist() == [0, 0, 1, 1, 0]  # (5,5): 41 to the first centroid, 61 to the second
    assert v.tolist() == [1.0, 1.0, 1.0, 1.0, 41.0]
    newc, counts = R.kmeans_update(X, i, C)
    assert counts.tolist() == [3.0, 2.0, 0.0]
    assert torch.allclose(newc, torch.tensor([[5 / 3, 7 / 3], [10., 11.], [100., 100.]], dtype=torch.float64))
