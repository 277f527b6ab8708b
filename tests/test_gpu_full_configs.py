"""Whole benchmark configurations on the GPU against a chunked fp32 product (TF32 off) on the
same device: a test-only comparator that can afford every batch and tens of thousands of
full-width rows, beside the CPU-oracle samples of test_gpu_parity.py. Tolerance: rel 1e-5 /
abs 1e-4 on each side of the fp32 comparison (hence the factor 2)."""
import pytest
import torch

from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu


class fp32_matmul:
    """torch matmuls in plain fp32 (no TF32) inside the block."""

    def __enter__(self):
        self.prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False

    def __exit__(self, *exc):
        torch.backends.cuda.matmul.allow_tf32 = self.prev


def outside_tolerance(got, want):
    return int(((got - want).abs() > 2 * (R.ATOL + R.RTOL * want.abs())).sum())


def test_bmm_config2_all_batches(dev, lib):
    from custom_matmul_kernels_b200 import BMMCUDA
    d = R.make_inputs("c2")
    A, B = d["A"].to(dev), d["B"].to(dev)
    C = BMMCUDA()(A, B)
    assert C.shape == (128, 1024, 1024)
    bad = 0
    with fp32_matmul():
        for b0 in range(0, 128, 16):
            bad += outside_tolerance(C[b0:b0 + 16], torch.bmm(A[b0:b0 + 16], B[b0:b0 + 16]))
    assert bad == 0
    # and a CPU-oracle sample (fp64) of batches the slice test does not touch
    for b in (63, 127):
        ok, err = R.values_close(C[b], torch.mm(d["A"][b].double(), d["B"][b].double()))
        assert ok, err
    assert lib.fbmm_check(None) == 0


def test_mbmm_config3_all_batches(dev, lib):
    from custom_matmul_kernels_b200 import MBMMCUDA, make_masks
    d = R.make_inputs("c3")
    A, B, mask = d["A"].to(dev), d["B"].to(dev), d["mask"].to(dev)
    bm, tm, em = make_masks(mask)
    C = MBMMCUDA()(A, B, bm, tm, em)
    assert bool((C[~mask] == 0).all()), "a masked entry is not exactly zero"
    bad = 0
    with fp32_matmul():
        for b0 in range(0, 128, 16):
            want = torch.bmm(A[b0:b0 + 16], B[b0:b0 + 16]).masked_fill_(~mask[b0:b0 + 16], 0)
            bad += outside_tolerance(C[b0:b0 + 16], want)
    assert bad == 0
    for b in (0, 64, 127):   # causal, first random-tile batch, last batch: fp64 oracle
        want = torch.mm(d["A"][b].double(), d["B"][b].double()).masked_fill_(~d["mask"][b], 0)
        ok, err = R.values_close(C[b], want)
        assert ok, err
    assert lib.fbmm_check(None) == 0


def test_topk_config5_65536_rows_at_full_width(dev, lib):
    """65 536 rows of configuration 5 against all 1 048 576 columns, k = 64: values descending
    and within tolerance of the comparator's own top-64, indices in range, unique, and each
    reproducing its value in the comparator's product."""
    from custom_matmul_kernels_b200 import TopkBMMCUDA
    g = torch.Generator(device=dev).manual_seed(1005)
    m, k, n, kk = 65536, 256, 1 << 20, 64
    A = torch.randn(1, m, k, generator=g, device=dev)
    B = torch.randn(1, k, n, generator=g, device=dev)
    v, i = TopkBMMCUDA()(A, B, k=kk, dim=2)
    assert bool((v[..., :-1] >= v[..., 1:]).all()) and bool(((i >= 0) & (i < n)).all())
    srt = i.sort(dim=-1).values
    assert bool((srt[..., 1:] != srt[..., :-1]).all())
    del srt
    bad_val = bad_idx = 0
    rstep, cstep = 4096, 65536
    with fp32_matmul():
        for r0 in range(0, m, rstep):
            Ar, ir, vr = A[0, r0:r0 + rstep], i[0, r0:r0 + rstep], v[0, r0:r0 + rstep]
            best = torch.full((rstep, kk), float("-inf"), device=dev)
            at = torch.empty(rstep, kk, device=dev)
            for c0 in range(0, n, cstep):
                C = Ar @ B[0, :, c0:c0 + cstep]
                best = torch.cat([best, C.topk(kk, dim=1).values], dim=1).topk(kk, dim=1).values
                inside = (ir >= c0) & (ir < c0 + cstep)
                at = torch.where(inside, C.gather(1, (ir - c0).clamp(0, cstep - 1)), at)
            tol = 2 * (R.ATOL + R.RTOL * best.abs())
            bad_val += int(((vr - best).abs() > tol).sum())
            bad_idx += int(((at - vr).abs() > tol).sum())
    assert bad_val == 0 and bad_idx == 0, (bad_val, bad_idx)
    assert lib.fbmm_check(None) == 0
