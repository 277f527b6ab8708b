"""Pins the oracle, and libfbmm.so, to outputs of the reference's OWN kernels.

oracle/build_ref.py compiles the reference's kernels/{bmm_helpers,bmm,minbmm,mbmm}.cu as its
wrappers do (placeholders substituted, ``--maxrregcount=128 --use_fast_math``) into cubins
under oracle/_ref/; oracle/ref_kernels.py launches them with the reference's grid and
arguments. Checked here, on shapes that are multiples of 512 (every CTA of the reference's
patch raster then lies inside the matrix):

* the C restatement of the kernel arithmetic (oracle/fbmm_oracle.c: one fp32 fmaf chain over
  ascending k per output) reproduces the reference's bmm / mbmm outputs and min VALUES bit
  for bit, for the inner product and for the squared-l2 and l1 accumulate functions;
* the reference's argmin agrees with the oracle's except where its unsynchronised
  value / index update (kernels/minbmm.cu:76-79) lost a race -- rare, counted, bounded;
* libfbmm.so agrees with the reference's kernels within the stated tolerance (rel 1e-5 /
  abs 1e-4 on each side of an fp32 comparison).

kernels/topkbmm.cu is not run: it takes a global spin mutex (kernels/topkbmm.cu:13-47).
"""
import pytest
import torch

from conftest import tol_ratio
from oracle import c_oracle
from oracle import ref_kernels as K
from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu

MODES = ("nn", "nt", "tn", "tt")


@pytest.fixture(scope="module")
def ref(dev):
    if not K.available():
        pytest.skip("oracle/_ref is not built (python -m oracle.build_ref <reference root>)")
    return K


def as_layout(X, transposed):
    return X.transpose(1, 2).contiguous().transpose(1, 2) if transposed else X


def test_reference_bmm_kernels_pin_the_oracle_and_the_library(ref, dev, lib):
    from custom_matmul_kernels_b200 import BMMCUDA
    op = BMMCUDA()
    for seed, (l, m, k, n) in enumerate([(2, 512, 96, 1024), (1, 1024, 64, 512), (1, 512, 100, 512)]):
        g = torch.Generator().manual_seed(40 + seed)
        A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
        want = c_oracle.bmm(A, B)
        Ad, Bd = A.to(dev), B.to(dev)
        for mode in MODES:
            C_ref = ref.bmm(Ad, Bd, mode)
            assert torch.equal(C_ref.cpu(), want), (mode, float((C_ref.cpu() - want).abs().max()))
            C = op(as_layout(Ad, mode[0] == "t"), as_layout(Bd, mode[1] == "t"))
            assert tol_ratio(C, C_ref) <= 2.0, mode
    assert lib.fbmm_check(None) == 0


def test_reference_min_kernels_pin_the_oracle_and_the_library(ref, dev, lib):
    from custom_matmul_kernels_b200 import MinBMMCUDA
    l, m, k, n = 1, 1024, 64, 2048
    g = torch.Generator().manual_seed(50)
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    Ad, Bd = A.to(dev), B.to(dev)
    for distance in ("inner", "l2"):
        op = MinBMMCUDA(distance=distance)
        for dim in (1, 2):
            wv, wi = c_oracle.min_bmm(A, B, dim, distance)
            for mode in MODES:
                rv, ri = ref.min_bmm(Ad, Bd, dim, mode, distance)
                assert torch.equal(rv.cpu(), wv), (distance, dim, mode)
                lost = int((ri.cpu() != wi).sum())
                assert lost <= wi.numel() // 100, f"{lost} argmin mismatches: more than the reference's race explains"
                v, i = op(as_layout(Ad, mode[0] == "t"), as_layout(Bd, mode[1] == "t"), dim=dim)
                assert tol_ratio(v, rv) <= 2.0, (distance, dim, mode)
                # our index, looked up in the oracle's product, is the minimum up to the tolerance
                R.check_min(v, i, A, B, dim, distance=distance)
    # the l1 accumulate function (kernels/bmm_helpers.cu:46-52) against its restatement
    wv, _ = c_oracle.min_bmm(A, B, 2, "l1")
    rv, _ = ref.min_bmm(Ad, Bd, 2, "nn", "l1")
    assert torch.equal(rv.cpu(), wv)
    # ... and the library's l1 kernel against the reference's (both dims)
    for dim in (1, 2):
        rv, _ = ref.min_bmm(Ad, Bd, dim, "nn", "l1")
        v, i = MinBMMCUDA(distance="l1")(Ad, Bd, dim=dim)
        assert tol_ratio(v, rv) <= 2.0, dim
        R.check_min(v, i, A, B, dim, distance="l1")
    assert lib.fbmm_check(None) == 0


def test_reference_mbmm_kernel_pins_the_oracle_and_the_library(ref, dev, lib):
    from custom_matmul_kernels_b200 import MBMMCUDA, make_masks
    l, m, k, n = 2, 512, 64, 1024
    g = torch.Generator().manual_seed(60)
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    mask = torch.zeros(l, m, n, dtype=torch.bool)
    mask[0] = torch.tril(torch.ones(m, n, dtype=torch.bool))
    tiles = torch.rand(m // 64, n // 64, generator=g) < 0.3
    mask[1] = tiles.repeat_interleave(64, 0).repeat_interleave(64, 1)
    mask[1, 5, 700] = True   # a lone element: its 8x8 tile count is 1
    Ad, Bd = A.to(dev), B.to(dev)
    bm, tm, em = make_masks(mask.to(dev))
    want = c_oracle.mbmm(A, B, bm.cpu(), tm.cpu(), em.cpu())
    C_ref = ref.mbmm(Ad, Bd, bm, tm, em)
    assert torch.equal(C_ref.cpu(), want)
    assert torch.equal(C_ref.cpu() != 0, (want != 0))
    C = MBMMCUDA()(Ad, Bd, bm, tm, em)
    assert tol_ratio(C, C_ref) <= 2.0
    assert bool((C[~mask.to(dev)] == 0).all())
    # shared masks (the kernel text with the mask's batch index replaced by 0, mbmm.py:24)
    bm1, tm1, em1 = make_masks(mask[1].to(dev))
    want1 = c_oracle.mbmm(A, B, bm1.cpu(), tm1.cpu(), em1.cpu(), share_mask=True)
    C_ref1 = ref.mbmm(Ad, Bd, bm1, tm1, em1, share_mask=True)
    assert torch.equal(C_ref1.cpu(), want1)
    assert tol_ratio(MBMMCUDA(share_mask=True)(Ad, Bd, bm1, tm1, em1), C_ref1) <= 2.0
    assert lib.fbmm_check(None) == 0
