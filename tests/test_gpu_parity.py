"""GPU parity tests: the CUDA path (through the Python wrappers, which call the C ABI, and
through the C ABI directly) against the CPU oracle on the same seeded inputs.

Tolerance, as the benchmark specification states it: values within rel 1e-5 / abs 1e-4;
indices exact except where competing values are closer than that tolerance (checked by
looking the returned index up in the oracle's fp64 product). Exact-arithmetic fixtures
must match bit for bit, indices included."""
import math

import numpy as np
import pytest
import torch

from conftest import load_golden, tol_ratio
from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(dev, lib):
    from custom_matmul_kernels_b200 import BMMCUDA, MBMMCUDA, MinBMMCUDA, TopkBMMCUDA
    return {"bmm": BMMCUDA(), "mbmm": MBMMCUDA(), "mbmm_shared": MBMMCUDA(share_mask=True), "min": MinBMMCUDA(),
            "topk": TopkBMMCUDA()}


def f32(a):
    return torch.from_numpy(np.asarray(a)).float()


def device_ok(lib):
    assert lib.fbmm_check(None) == 0, lib.fbmm_last_error()


def layouts(A, B):
    """The four stride layouts of the same logical operands (bmm.py:56-66)."""
    At = A.transpose(1, 2).contiguous().transpose(1, 2)
    Bt = B.transpose(1, 2).contiguous().transpose(1, 2)
    return {"nn": (A, B), "tn": (At, B), "nt": (A, Bt), "tt": (At, Bt)}


# ----------------------------------------------------------------------------- bmm
def test_bmm_exact_golden(ops, dev, lib):
    g = load_golden("exact_bmm")
    A, B = f32(g["A"]).to(dev), f32(g["B"]).to(dev)
    want = torch.from_numpy(g["C"]).float()
    for mode, (a, b) in layouts(A, B).items():
        assert ops["bmm"].get_mode(a, b) == mode
        assert torch.equal(ops["bmm"](a, b).cpu(), want), mode
    assert torch.equal(ops["bmm"](A[0], B[0]).cpu(), want[0])  # 2-D in, 2-D out
    device_ok(lib)


@pytest.mark.parametrize("shape", [(1, 128, 32, 128), (2, 256, 96, 384), (3, 200, 100, 300), (1, 77, 50, 130),
                                   (1, 1, 1, 1), (2, 129, 257, 5), (1, 640, 256, 512)])
def test_bmm_randn(ops, dev, lib, shape):
    l, m, k, n = shape
    g = torch.Generator().manual_seed(hash(shape) % 1000)
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    want = R.bmm(A, B, dtype=torch.float64)
    for mode, (a, b) in layouts(A.to(dev), B.to(dev)).items():
        assert tol_ratio(ops["bmm"](a, b), want) <= 1.0, mode
    device_ok(lib)


def test_bmm_golden_randn_and_determinism(ops, dev):
    g = load_golden("randn_small")
    A, B = torch.from_numpy(g["A"]).to(dev), torch.from_numpy(g["B"]).to(dev)
    C1 = ops["bmm"](A, B)
    C2 = ops["bmm"](A, B)
    assert tol_ratio(C1, torch.from_numpy(g["C"])) <= 1.0
    assert torch.equal(C1, C2)


def test_bmm_noncontiguous_views_and_nonfinite(ops, dev, lib):
    g = torch.Generator().manual_seed(3)
    big = torch.randn(2, 70, 90, generator=g).to(dev)
    A = big[:, 3:53, 1:41]            # odd offset, pitch 90: repacked by the wrapper
    B = torch.randn(2, 40, 33, generator=g).to(dev)
    assert tol_ratio(ops["bmm"](A, B), R.bmm(A.cpu(), B.cpu(), dtype=torch.float64)) <= 1.0
    A2 = torch.randn(1, 8, 16, generator=g)
    A2[0, 2, 3] = float("inf")
    B2 = torch.randn(1, 16, 8, generator=g).abs() + 0.5
    C = ops["bmm"](A2.to(dev), B2.to(dev)).cpu()
    assert bool(torch.isinf(C[0, 2]).all()) and bool(torch.isfinite(C[0, :2]).all())
    device_ok(lib)


def test_bmm_config2_slice(ops, dev):
    d = R.make_inputs("c2", batches=4)
    C = ops["bmm"](d["A"].to(dev), d["B"].to(dev))
    assert tol_ratio(C, R.bmm(d["A"], d["B"], dtype=torch.float64)) <= 1.0


# ----------------------------------------------------------------------------- mbmm
def test_mbmm_exact_golden(ops, dev, lib):
    g = load_golden("exact_mbmm")
    A, B = f32(g["A"]), f32(g["B"])
    n = B.shape[2]
    mask = torch.from_numpy(np.unpackbits(g["mask"], axis=-1)[..., :n].astype(bool))
    from custom_matmul_kernels_b200 import make_masks
    bm, tm, em = make_masks(mask.to(dev))
    C = ops["mbmm"](A.to(dev), B.to(dev), bm, tm, em)
    assert torch.equal(C.cpu(), torch.from_numpy(g["C"]).float())
    device_ok(lib)


def test_mbmm_precedence_and_share_mask(ops, dev, lib):
    A, B = R.exact_inputs(3, 130, 8, 260, seed=4)
    em = torch.ones(130, 260, dtype=torch.uint8)
    tm = torch.ones(17, 33, dtype=torch.uint8)
    bm = torch.ones(2, 3, dtype=torch.uint8)
    bm[0, 1] = 0
    tm[2, 3] = 0
    em[5, 7] = 3
    want = R.mbmm(A, B, bm, tm, em, share_mask=True)
    C = ops["mbmm_shared"](A.to(dev), B.to(dev), bm.to(dev), tm.to(dev), em.to(dev))
    assert torch.equal(C.cpu(), want)
    # 2-D inputs with 2-D masks through the non-shared wrapper (mbmm.py:173-179)
    C2 = ops["mbmm"](A[0].to(dev), B[0].to(dev), bm.to(dev), tm.to(dev), em.to(dev))
    assert torch.equal(C2.cpu(), want[0])
    with pytest.raises(NotImplementedError):
        ops["mbmm"](A.to(dev), B.to(dev), bm.to(dev), tm.to(dev), em.to(dev), mode="tt")
    with pytest.raises(ValueError):
        ops["mbmm"](A.to(dev), B.to(dev), bm.to(dev), tm.to(dev), em.to(dev))  # masks lack the batch axis
    device_ok(lib)


def test_mbmm_config3_slice(ops, dev):
    from custom_matmul_kernels_b200 import make_masks
    d = R.make_inputs("c3", batches=4)
    bm, tm, em = make_masks(d["mask"].to(dev))
    C = ops["mbmm"](d["A"].to(dev), d["B"].to(dev), bm, tm, em).cpu()
    want = torch.bmm(d["A"].double(), d["B"].double()).masked_fill_(~d["mask"], 0)
    assert tol_ratio(C, want) <= 1.0
    assert bool((C[~d["mask"]] == 0).all())


# ----------------------------------------------------------------------------- min
def test_min_exact_golden_lowest_index_on_ties(ops, dev, lib):
    g = load_golden("exact_min")
    A, B = f32(g["A"]).to(dev), f32(g["B"]).to(dev)
    for dim in (1, 2):
        for mode, (a, b) in layouts(A, B).items():
            v, i = ops["min"](a, b, dim=dim)
            assert torch.equal(v.cpu(), f32(g[f"v_dim{dim}"])), (dim, mode)
            assert torch.equal(i.cpu(), torch.from_numpy(g[f"i_dim{dim}"])), (dim, mode)
    v, i = ops["min"](A[0], B[0], dim=1)  # 2-D inputs: dim is bumped (minbmm.py:86-90)
    assert torch.equal(i.cpu(), torch.from_numpy(g["i_dim2"])[0])
    device_ok(lib)


@pytest.mark.parametrize("shape", [(1, 128, 64, 128), (2, 300, 40, 500), (1, 2048, 64, 4096), (1, 5, 3, 7),
                                   (1, 130, 256, 1000)])
def test_min_randn(ops, dev, lib, shape):
    l, m, k, n = shape
    g = torch.Generator().manual_seed(sum(shape))
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    for dim in (1, 2):
        v, i = ops["min"](A.to(dev), B.to(dev), dim=dim)
        assert v.dtype == torch.float32 and i.dtype == torch.int64
        assert v.shape == (l, n if dim == 1 else m)
        R.check_min(v, i, A, B, dim)
        v2, i2 = ops["min"](A.to(dev), B.to(dev), dim=dim)
        assert torch.equal(v, v2) and torch.equal(i, i2)  # deterministic
    device_ok(lib)


def test_min_config1_full(ops, dev, lib):
    d = R.make_inputs("c1")
    v, i = ops["min"](d["A"].to(dev), d["B"].to(dev), dim=2)
    r = R.check_min(v, i, d["A"], d["B"], 2)
    assert r["idx_mismatch"] <= 2  # near-ties may flip an index; exact ties cannot occur here
    device_ok(lib)


def test_min_config4_slice_properties(ops, dev, lib):
    """Full width (65536 centroids), 4096 of the 1M points: oracle on all of them, plus the
    row-independence property that a row's answer does not depend on which rows ride along."""
    d = R.make_inputs("c4", rows=4096)
    A, B = d["A"].to(dev), d["B"].to(dev)
    v, i = ops["min"](A, B, dim=2)
    R.check_min(v, i, d["A"], d["B"], 2)
    v2, i2 = ops["min"](A[:, 1000:1300], B, dim=2)
    assert torch.equal(v2, v[:, 1000:1300]) and torch.equal(i2, i[:, 1000:1300])
    device_ok(lib)


def test_min_config4_full_size_all_rows(ops, dev, lib):
    """All 1 048 576 rows of configuration 4 against a chunked fp32 product (TF32 off) on the
    same GPU: a test-only comparator that can afford every row, where the CPU oracle of the
    previous test covers a sample. Values within the fp32 tolerance of both sides; where the
    indices differ, the comparator's product at the returned index must be within tolerance
    of its own minimum (a near-tie)."""
    g = torch.Generator(device=dev).manual_seed(1004)
    m, k, n = 1 << 20, 128, 65536
    A = torch.randn(1, m, k, generator=g, device=dev)
    B = torch.randn(1, k, n, generator=g, device=dev)
    v, i = ops["min"](A, B, dim=2)
    assert v.shape == (1, m) and i.dtype == torch.int64 and bool(((i >= 0) & (i < n)).all())
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        step, bad_val, bad_idx = 16384, 0, 0
        for r0 in range(0, m, step):
            C = A[0, r0:r0 + step] @ B[0]
            wv, wi = C.min(dim=1)
            gv, gi = v[0, r0:r0 + step], i[0, r0:r0 + step]
            tol = 2 * (R.ATOL + R.RTOL * wv.abs())
            bad_val += int(((gv - wv).abs() > tol).sum())
            at = C.gather(1, gi[:, None])[:, 0]
            bad_idx += int(((at - wv).abs() > tol).sum())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert bad_val == 0 and bad_idx == 0, (bad_val, bad_idx)
    device_ok(lib)


def test_topk_config5_full_width_rows_against_gpu_reference(ops, dev, lib):
    """2 048 rows of configuration 5 against all 1 048 576 columns (pre-split, repacked
    planes, paced sweep), k = 64: descending values, unique in-range indices, and every
    (value, index) pair reproduced by a chunked fp32 product (TF32 off) whose own top-64
    values must agree within tolerance."""
    g = torch.Generator(device=dev).manual_seed(1005)
    m, k, n, kk = 2048, 256, 1 << 20, 64
    A = torch.randn(1, m, k, generator=g, device=dev)
    B = torch.randn(1, k, n, generator=g, device=dev)
    v, i = ops["topk"](A, B, k=kk, dim=2)
    assert bool((v[..., :-1] >= v[..., 1:]).all()) and bool(((i >= 0) & (i < n)).all())
    srt = i.sort(dim=-1).values
    assert bool((srt[..., 1:] != srt[..., :-1]).all())
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        best = torch.full((m, kk), float("-inf"), device=dev)
        at = torch.empty(m, kk, device=dev)
        cstep = 65536
        for c0 in range(0, n, cstep):
            C = A[0] @ B[0, :, c0:c0 + cstep]
            best = torch.cat([best, C], dim=1).topk(kk, dim=1).values
            inside = (i[0] >= c0) & (i[0] < c0 + cstep)
            got = C.gather(1, (i[0] - c0).clamp(0, cstep - 1))
            at = torch.where(inside, got, at)
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    tol = 2 * (R.ATOL + R.RTOL * best.abs())
    assert bool(((v[0] - best).abs() <= tol).all()), float((v[0] - best).abs().max())
    assert bool(((at - v[0]).abs() <= tol).all()), "an index does not reproduce its value"
    device_ok(lib)


# ----------------------------------------------------------------------------- top-k
def test_topk_exact_golden(ops, dev, lib):
    g = load_golden("exact_topk")
    A, B, k = f32(g["A"]), f32(g["B"]), int(g["k"])
    for dim in (1, 2):
        for mode, (a, b) in layouts(A.to(dev), B.to(dev)).items():
            v, i = ops["topk"](a, b, k=k, dim=dim)
            assert torch.equal(v.cpu(), f32(g[f"v_dim{dim}"])), (dim, mode)
            R.check_topk(v, i, A, B, k, dim)
    device_ok(lib)


@pytest.mark.parametrize("kk", [32, 64, 96, 128])
def test_topk_exact_ties_with_k_a_multiple_of_32(ops, dev, lib, kk):
    """Small-integer operands: values are exact and ties are everywhere, so the values must
    equal the oracle's bit for bit and equal values must come lowest index first (the
    reference's strict comparisons keep the earlier column). k % 32 == 0 takes the
    one-row-per-lane merge; three row blocks' worth of rows and thousands of columns make
    every row merge many times, and 203 rows leave a warp with rows past the end."""
    A, B = R.exact_inputs(2, 203, 24, 2900, seed=400 + kk, lo=-3, hi=3)
    for dim in (1, 2):
        v, i = ops["topk"](A.to(dev), B.to(dev), k=kk, dim=dim)
        C = torch.bmm(A.double(), B.double())
        if dim == 1:
            C = C.transpose(1, 2).contiguous()
        # stable descending sort = larger value first, lower index first among equals
        order = torch.sort(C, dim=-1, descending=True, stable=True)
        assert torch.equal(v.cpu().double(), order.values[..., :kk]), dim
        assert torch.equal(i.cpu(), order.indices[..., :kk]), dim
    device_ok(lib)


def test_topk_short_rows_pad(ops, dev):
    g = load_golden("exact_topk_short")
    A, B, k = f32(g["A"]), f32(g["B"]), int(g["k"])
    v, i = ops["topk"](A.to(dev), B.to(dev), k=k, dim=2)
    assert torch.equal(v.cpu(), torch.from_numpy(g["v_dim2"]))
    assert bool((i.cpu()[..., 5:] == -1).all()) and bool(torch.isneginf(v.cpu()[..., 5:]).all())
    R.check_topk(v, i, A, B, k, 2)


@pytest.mark.parametrize("case", [(1, 128, 64, 128, 16), (1, 128, 64, 1024, 64), (2, 300, 40, 700, 10),
                                  (1, 256, 64, 4096, 128), (1, 2048, 128, 8192, 64), (1, 130, 32, 50, 64),
                                  (1, 64, 16, 3000, 1), (1, 200, 24, 2500, 97)])
def test_topk_randn(ops, dev, lib, case):
    l, m, k, n, kk = case
    g = torch.Generator().manual_seed(sum(case))
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    for dim in (1, 2):
        v, i = ops["topk"](A.to(dev), B.to(dev), k=kk, dim=dim)
        assert v.shape == (l, n if dim == 1 else m, kk) and v.is_contiguous()
        R.check_topk(v, i, A, B, kk, dim)
        v2, i2 = ops["topk"](A.to(dev), B.to(dev), k=kk, dim=dim)
        assert torch.equal(v, v2) and torch.equal(i, i2)
    device_ok(lib)


def test_topk_config5_slice_and_column_shard_merge(ops, dev, lib):
    """512 queries against 65536 keys at d=256, k=64: oracle on every row; then the same
    answer from 4 column shards merged by fbmm_topk_merge_f32 (the multi-GPU exchange,
    emulated on one device)."""
    d = R.make_inputs("c5", rows=512, cols=65536)
    A, B = d["A"].to(dev), d["B"].to(dev)
    v, i = ops["topk"](A, B, k=64, dim=2)
    R.check_topk(v, i, d["A"], d["B"], 64, 2)
    shards = 4
    w = 65536 // shards
    cv = torch.empty(shards, 512, 64, device=dev)
    ci = torch.empty(shards, 512, 64, device=dev, dtype=torch.int64)
    for s in range(shards):
        sv, si = ops["topk"](A, B[:, :, s * w:(s + 1) * w].contiguous(), k=64, dim=2, index_offset=s * w)
        cv[s], ci[s] = sv[0], si[0]
    mv = torch.empty(512, 64, device=dev)
    mi = torch.empty(512, 64, device=dev, dtype=torch.int64)
    rc = lib.fbmm_topk_merge_f32(None, cv.data_ptr(), ci.data_ptr(), shards, 512, 64, mv.data_ptr(), mi.data_ptr())
    assert rc == 0, lib.fbmm_last_error()
    torch.cuda.synchronize()
    assert torch.equal(mv, v[0]) and torch.equal(mi, i[0])
    device_ok(lib)


# ----------------------------------------------------------------------------- raw C ABI
def test_c_abi_direct_call_with_pitched_operands(dev, lib):
    """Calls fbmm_bmm_f32 with explicit pitches and a pitched C, no wrapper in between."""
    from custom_matmul_kernels_b200 import custom_kernel as ck
    l, m, k, n = 2, 100, 36, 52
    g = torch.Generator().manual_seed(9)
    Abuf = torch.randn(l, m, 40, generator=g).to(dev)      # pitch 40 > k
    Bbuf = torch.randn(l, k, 56, generator=g).to(dev)      # pitch 56 > n
    Cbuf = torch.full((l, m, 60), 7.0, device=dev)         # pitch 60 > n
    rc = lib.fbmm_bmm_f32(torch.cuda.current_stream().cuda_stream, Abuf.data_ptr(), ord("n"), 40, m * 40,
                          Bbuf.data_ptr(), ord("n"), 56, k * 56, Cbuf.data_ptr(), 60, m * 60, l, m, n, k)
    assert rc == 0, lib.fbmm_last_error()
    assert lib.fbmm_check(None) == 0
    want = torch.bmm(Abuf[:, :, :k].double().cpu(), Bbuf[:, :, :n].double().cpu())
    assert tol_ratio(Cbuf[:, :, :n], want) <= 1.0
    assert bool((Cbuf[:, :, n:] == 7.0).all())             # padding columns untouched
    rc = lib.fbmm_bmm_f32(None, Abuf.data_ptr() + 4, ord("n"), 40, m * 40, Bbuf.data_ptr(), ord("n"), 56, k * 56,
                          Cbuf.data_ptr(), 60, m * 60, l, m, n, k)
    assert rc == ck.FBMM_ERR_ALIGN


def test_c_abi_min_workspace_too_small(dev, lib):
    from custom_matmul_kernels_b200 import custom_kernel as ck
    A = torch.zeros(1, 128, 32, device=dev)
    B = torch.zeros(1, 32, 128, device=dev)
    v = torch.empty(1, 128, device=dev)
    i = torch.empty(1, 128, device=dev, dtype=torch.int64)
    ws = torch.empty(64, device=dev, dtype=torch.uint8)
    rc = lib.fbmm_min_bmm_f32(None, A.data_ptr(), ord("n"), 32, 0, B.data_ptr(), ord("n"), 128, 0, v.data_ptr(),
                              i.data_ptr(), 1, 128, 128, 32, 2, 0, ws.data_ptr(), 64)
    assert rc == ck.FBMM_ERR_WORKSPACE


def test_presplit_scratch_gives_identical_bits(dev, lib):
    """With room for pre-split lo planes in the workspace the kernels skip their in-kernel
    splitter; the planes hold the same values either way, so the outputs must not differ
    in a single bit (min and top-k with K <= 128 and K > 128)."""
    g = torch.Generator().manual_seed(31)
    stream = torch.cuda.current_stream().cuda_stream
    # (K <= 64 with pre-split planes is the min kernel with two resident row blocks of A per CTA:
    # 1100 rows leave its last unit a ragged second block, 1408 an absent one, K = 20 one k-block)
    for (m, k, n) in [(1100, 96, 1300), (1024, 160, 1536), (1280, 128, 1100), (1100, 64, 1300), (1408, 20, 1024),
                      (2048, 36, 2500)]:
        A = torch.randn(1, m, k, generator=g).to(dev)
        B = torch.randn(1, k, n, generator=g).to(dev)
        extra = lib.fbmm_presplit_workspace_bytes(1, m, n, k, 2, ord("n"), k, m * k, ord("n"), n, k * n)
        assert extra >= k * n * 4
        outs = []
        for use_extra in (False, True):
            own = (lib.fbmm_min_bmm_workspace_bytes(1, m, n, k, 2, 0) + 255) // 256 * 256
            nbytes = own + (extra if use_extra else 0)
            ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
            v = torch.empty(1, m, device=dev)
            i = torch.empty(1, m, device=dev, dtype=torch.int64)
            rc = lib.fbmm_min_bmm_f32(stream, A.data_ptr(), ord("n"), k, m * k, B.data_ptr(), ord("n"), n, k * n,
                                      v.data_ptr(), i.data_ptr(), 1, m, n, k, 2, 0, ws.data_ptr(), nbytes)
            assert rc == 0, lib.fbmm_last_error()
            own_t = (lib.fbmm_topk_bmm_workspace_bytes(1, m, n, k, 16, 2, 0) + 255) // 256 * 256
            nb_t = own_t + (extra if use_extra else 0)
            ws_t = torch.empty(max(nb_t, 256), device=dev, dtype=torch.uint8)
            tv = torch.empty(1, m, 16, device=dev)
            ti = torch.empty(1, m, 16, device=dev, dtype=torch.int64)
            rc = lib.fbmm_topk_bmm_f32(stream, A.data_ptr(), ord("n"), k, m * k, B.data_ptr(), ord("n"), n, k * n,
                                       tv.data_ptr(), ti.data_ptr(), 1, m, n, k, 16, 2, 0, 0, ws_t.data_ptr(), nb_t)
            assert rc == 0, lib.fbmm_last_error()
            torch.cuda.synchronize()
            outs.append((v, i, tv, ti))
        for a, b in zip(*outs):
            assert torch.equal(a, b)
        R.check_min(outs[1][0], outs[1][1], A.cpu(), B.cpu(), 2)
        R.check_topk(outs[1][2], outs[1][3], A.cpu(), B.cpu(), 16, 2)
    assert lib.fbmm_presplit_workspace_bytes(1, 512, 4096, 64, 2, ord("n"), 64, 0, ord("n"), 4096, 0) == 0
    assert lib.fbmm_check(None) == 0, lib.fbmm_last_error()


def test_two_row_block_min_kernel_l2_and_dim1(dev, lib):
    """The K <= 64 min kernel on pre-split planes (two resident row blocks per CTA) through the
    wrapper, which passes the planes' scratch: squared-l2 distance, both dims, a transposed
    layout, batches; against the oracle, and exact integers bit for bit."""
    from custom_matmul_kernels_b200 import MinBMMCUDA
    g = torch.Generator().manual_seed(77)
    A, B = torch.randn(2, 1300, 48, generator=g), torch.randn(2, 48, 1200, generator=g)
    Ad, Bd = A.to(dev), B.to(dev)
    Bt = Bd.transpose(1, 2).contiguous().transpose(1, 2)
    for distance in ("inner", "l2"):
        op = MinBMMCUDA(distance=distance)
        for dim in (1, 2):
            for b_ in (Bd, Bt):
                v, i = op(Ad, b_, dim=dim)
                R.check_min(v, i, A, B, dim, distance=distance)
    Ae, Be = R.exact_inputs(1, 1536, 64, 1024, seed=9)
    v, i = MinBMMCUDA()(Ae.to(dev), Be.to(dev), dim=2)
    wv, wi = R.min_bmm(Ae, Be, dim=2)
    assert torch.equal(v.cpu(), wv) and torch.equal(i.cpu(), wi)
    device_ok(lib)


def test_topk_and_min_with_pre_split_planes_wider_than_l2(dev, lib):
    """A column operand whose hi and lo planes (2 x 51 MB) exceed what L2 keeps: top-k sweeps
    it paced (every CTA holds back until the others have asked for the range before last),
    min sweeps it in column ranges. Same bits as without pre-split planes, and the oracle's
    answer on a sample of rows (the full product is too much for the CPU side of a test)."""
    m, k, n = 148 * 128 + 60, 64, 200000
    g = torch.Generator().manual_seed(77)
    A = torch.randn(1, m, k, generator=g).to(dev)
    B = torch.randn(1, k, n, generator=g).to(dev)
    stream = torch.cuda.current_stream().cuda_stream
    extra = lib.fbmm_presplit_workspace_bytes(1, m, n, k, 2, ord("n"), k, m * k, ord("n"), n, k * n)
    assert extra >= k * n * 4
    outs = []
    for use_extra in (False, True):
        own = (lib.fbmm_min_bmm_workspace_bytes(1, m, n, k, 2, 0) + 255) // 256 * 256
        nbytes = own + (extra if use_extra else 0)
        ws = torch.empty(nbytes, device=dev, dtype=torch.uint8)
        v = torch.empty(1, m, device=dev)
        i = torch.empty(1, m, device=dev, dtype=torch.int64)
        rc = lib.fbmm_min_bmm_f32(stream, A.data_ptr(), ord("n"), k, m * k, B.data_ptr(), ord("n"), n, k * n,
                                  v.data_ptr(), i.data_ptr(), 1, m, n, k, 2, 0, ws.data_ptr(), nbytes)
        assert rc == 0, lib.fbmm_last_error()
        own_t = (lib.fbmm_topk_bmm_workspace_bytes(1, m, n, k, 32, 2, 0) + 255) // 256 * 256
        nb_t = own_t + (extra if use_extra else 0)
        ws_t = torch.empty(nb_t, device=dev, dtype=torch.uint8)
        tv = torch.empty(1, m, 32, device=dev)
        ti = torch.empty(1, m, 32, device=dev, dtype=torch.int64)
        rc = lib.fbmm_topk_bmm_f32(stream, A.data_ptr(), ord("n"), k, m * k, B.data_ptr(), ord("n"), n, k * n,
                                   tv.data_ptr(), ti.data_ptr(), 1, m, n, k, 32, 2, 0, 0, ws_t.data_ptr(), nb_t)
        assert rc == 0, lib.fbmm_last_error()
        torch.cuda.synchronize()
        outs.append((v, i, tv, ti))
    for a, b in zip(*outs):
        assert torch.equal(a, b)
    rows = torch.cat([torch.arange(0, 160), torch.arange(9000, 9100), torch.arange(m - 130, m)])
    As, Bc = A.cpu()[:, rows], B.cpu()
    R.check_min(outs[1][0][:, rows], outs[1][1][:, rows], As, Bc, 2)
    R.check_topk(outs[1][2][:, rows], outs[1][3][:, rows], As, Bc, 32, 2)
    assert lib.fbmm_check(None) == 0, lib.fbmm_last_error()


def test_topk_and_min_on_a_repacked_column_operand(ops, dev, lib):
    """B stored [k][n] with a million columns (256 MB; the rewrite starts at 64 MB): its planes
    are rewritten k-contiguous before the sweep. Oracle on a sample of rows, and the same bits as with B
    handed over k-contiguous by the caller (layout 't'), where nothing is repacked."""
    m, k, n = 148 * 128, 64, 1 << 20
    g = torch.Generator().manual_seed(78)
    A = torch.randn(1, m, k, generator=g).to(dev)
    Bc = torch.randn(1, k, n, generator=g)
    B = Bc.to(dev)
    Bt = B.transpose(1, 2).contiguous().transpose(1, 2)  # same values, stored [n][k]
    tk, mn = ops["topk"], ops["min"]
    extra = lib.fbmm_presplit_workspace_bytes(1, m, n, k, 2, ord("n"), k, m * k, ord("n"), n, k * n)
    assert extra >= 2 * n * k * 4  # both planes of B
    tv, ti = tk(A, B, k=32, dim=2)
    tv2, ti2 = tk(A, Bt, k=32, dim=2)
    mv, mi = mn(A, B, dim=2)
    mv2, mi2 = mn(A, Bt, dim=2)
    assert torch.equal(tv, tv2) and torch.equal(ti, ti2)
    assert torch.equal(mv, mv2) and torch.equal(mi, mi2)
    rows = torch.cat([torch.arange(0, 40), torch.arange(m - 24, m)])
    As = A.cpu()[:, rows]
    R.check_min(mv[:, rows], mi[:, rows], As, Bc, 2)
    R.check_topk(tv[:, rows], ti[:, rows], As, Bc, 32, 2)
    assert lib.fbmm_check(None) == 0, lib.fbmm_last_error()


# ----------------------------------------------------------------------------- 16-bit operands
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 300, 72, 700), (2, 129, 64, 257), (1, 1100, 200, 1300), (1, 64, 520, 3000)])
def test_min_and_topk_on_16_bit_operands(ops, dev, lib, dtype, shape):
    """fp16 / bf16 operands go to tcgen05.mma.kind::f16 as they are (fp32 accumulation). The
    oracle multiplies the same 16-bit values in fp64, so only the accumulation differs:
    the fp32 tolerance holds. K = 72 and 200 are not multiples of the 64-element k-block,
    K = 520 streams A (more than four k-blocks); both dims, B given [k][n] (repacked by the
    wrapper) and [n][k] (taken as it is)."""
    l, m, k, n = shape
    g = torch.Generator().manual_seed(sum(shape) + (1 if dtype == torch.float16 else 2))
    A = torch.randn(l, m, k, generator=g).to(dtype)
    B = torch.randn(l, k, n, generator=g).to(dtype)
    Bt = B.to(dev).transpose(1, 2).contiguous().transpose(1, 2)
    Af, Bf = A.float(), B.float()
    for dim in (1, 2):
        v, i = ops["min"](A.to(dev), B.to(dev), dim=dim)
        assert v.dtype == torch.float32 and i.dtype == torch.int64
        R.check_min(v, i, Af, Bf, dim)
        v2, i2 = ops["min"](A.to(dev), Bt, dim=dim)
        assert torch.equal(v, v2) and torch.equal(i, i2)
        for kk in (10, 64):
            tv, ti = ops["topk"](A.to(dev), B.to(dev), k=kk, dim=dim)
            R.check_topk(tv, ti, Af, Bf, kk, dim)
    device_ok(lib)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_bmm_on_16_bit_operands(ops, dev, lib, dtype):
    """C comes back in the operands' type: the fp64 product of the same 16-bit values,
    rounded once, may differ from it by the fp32 accumulation error plus half a unit in the
    last place of the 16-bit type (2^-11 relative for fp16, 2^-8 for bf16)."""
    half_ulp = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
    g = torch.Generator().manual_seed(17)
    for (l, m, k, n) in [(2, 300, 72, 264), (1, 129, 520, 257), (3, 1024, 128, 1024)]:
        A = torch.randn(l, m, k, generator=g).to(dtype)
        B = torch.randn(l, k, n, generator=g).to(dtype)
        want = torch.bmm(A.double(), B.double())
        for Bd in (B.to(dev), B.to(dev).transpose(1, 2).contiguous().transpose(1, 2)):
            C = ops["bmm"](A.to(dev), Bd)
            assert C.dtype == dtype and C.shape == (l, m, n)
            err = (C.cpu().double() - want).abs()
            assert bool((err <= 1e-4 + (1e-5 + half_ulp * 1.01) * want.abs()).all()), float(err.max())
    device_ok(lib)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_mbmm_on_16_bit_operands(ops, dev, lib, dtype):
    """Masked bmm with 16-bit operands: zeros exactly where the mask says so, the rounded
    product elsewhere (shapes with ragged edges and with whole dead 128x128 blocks)."""
    from custom_matmul_kernels_b200 import make_masks
    half_ulp = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
    g = torch.Generator().manual_seed(23)
    for (l, m, k, n) in [(2, 300, 72, 264), (2, 512, 64, 640)]:
        A = torch.randn(l, m, k, generator=g).to(dtype)
        B = torch.randn(l, k, n, generator=g).to(dtype)
        mask = torch.rand(l, m, n, generator=g) < 0.4
        mask[0, :128, :256] = False          # dead blocks
        mask[1] = torch.tril(torch.ones(m, n)).bool()
        bm, tm, em = make_masks(mask.to(dev))
        C = ops["mbmm"](A.to(dev), B.to(dev), bm, tm, em)
        assert C.dtype == dtype
        want = torch.bmm(A.double(), B.double()).masked_fill_(~mask, 0)
        got = C.cpu().double()
        assert bool((got[~mask] == 0).all())
        err = (got - want).abs()
        assert bool((err <= 1e-4 + (1e-5 + half_ulp * 1.01) * want.abs()).all()), float(err.max())
    device_ok(lib)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_l2_distance_on_16_bit_operands(dev, lib, dtype):
    """distance="l2" with 16-bit operands: norms of the 16-bit values in fp32, products on
    the tensor cores; the oracle forms sum (a - b)^2 of the same values in fp64."""
    from custom_matmul_kernels_b200 import MinBMMCUDA, TopkBMMCUDA
    g = torch.Generator().manual_seed(29)
    mn, tk = MinBMMCUDA(distance="l2"), TopkBMMCUDA(distance="l2")
    for (l, m, k, n) in [(1, 300, 72, 700), (2, 130, 64, 257)]:
        A = torch.randn(l, m, k, generator=g).to(dtype)
        B = torch.randn(l, k, n, generator=g).to(dtype)
        for dim in (1, 2):
            v, i = mn(A.to(dev), B.to(dev), dim=dim)
            R.check_min(v, i, A.float(), B.float(), dim, distance="l2")
            tv, ti = tk(A.to(dev), B.to(dev), k=9, dim=dim)
            R.check_topk(tv, ti, A.float(), B.float(), 9, dim, distance="l2")
    assert lib.fbmm_check(None) == 0, lib.fbmm_last_error()


def test_16_bit_exact_small_integers(ops, dev, lib):
    """Small-integer operands are exact in fp16 and bf16 and so is every partial sum: the
    16-bit kernels must return the fp32 kernels' values and indices bit for bit."""
    A, B = R.exact_inputs(1, 260, 96, 1500, seed=91, lo=-4, hi=4)
    v32, i32 = ops["min"](A.to(dev), B.to(dev), dim=2)
    t32v, t32i = ops["topk"](A.to(dev), B.to(dev), k=32, dim=2)
    for dtype in (torch.float16, torch.bfloat16):
        v, i = ops["min"](A.to(dev).to(dtype), B.to(dev).to(dtype), dim=2)
        assert torch.equal(v, v32) and torch.equal(i, i32)
        tv, ti = ops["topk"](A.to(dev).to(dtype), B.to(dev).to(dtype), k=32, dim=2)
        assert torch.equal(tv, t32v) and torch.equal(ti, t32i)
    device_ok(lib)


# ----------------------------------------------------------------------------- k-means consumer
def test_kmeans_step_and_fit(dev, lib):
    """assign = min_bmm with the l2 distance, update = fbmm_kmeans_update_f32. One step is
    checked against the oracle (fp64 sums; an empty cluster keeps its centroid), a short
    fit must not increase the summed distance from one iteration to the next."""
    from custom_matmul_kernels_b200 import KMeansCUDA
    g = torch.Generator().manual_seed(5)
    n, d, k = 5000, 48, 37
    blobs = torch.randn(k - 1, d, generator=g) * 4
    X = blobs[torch.randint(0, k - 1, (n,), generator=g)] + torch.randn(n, d, generator=g) * 0.5
    C0 = torch.cat([X[:k - 1].clone(), torch.full((1, d), 1e3)])  # the last centroid attracts nobody
    km = KMeansCUDA()
    dist, idx = km.assign(X.to(dev), C0.to(dev))
    want_v, want_i = R.kmeans_assign(X, C0)
    assert float((dist.cpu().double() - want_v).abs().max()) <= 1e-4 + 1e-5 * float(want_v.abs().max())
    near = (idx.cpu() != want_i)
    if bool(near.any()):  # only where two centroids are equally near within tolerance
        d2 = ((X.double()[near][:, None, :] - C0.double()[None]) ** 2).sum(-1)
        got = d2.gather(1, idx.cpu()[near][:, None])[:, 0]
        assert bool(((got - want_v[near]).abs() <= 1e-4 + 1e-5 * want_v[near].abs()).all())
    newc, counts = km.update(X.to(dev), idx, C0.to(dev))
    want_c, want_n = R.kmeans_update(X, idx.cpu(), C0)
    assert torch.equal(counts.cpu().double(), want_n)
    assert float(want_n[-1]) == 0 and torch.equal(newc.cpu()[-1], C0[-1])
    assert float((newc.cpu().double() - want_c).abs().max()) <= 1e-4
    c, prev = C0.to(dev), None
    for _ in range(4):
        dist, idx = km.assign(X.to(dev), c)
        total = float(dist.sum())
        assert prev is None or total <= prev * (1 + 1e-6)
        prev = total
        c, _ = km.update(X.to(dev), idx, c)
    fc, fi, fd = km.fit(X.to(dev), C0.to(dev), iters=3)
    assert fc.shape == (k, d) and fi.shape == (n,) and fd.shape == (n,)
    # many points, few clusters: the update gathers per-CTA partial sums in shared memory
    n2 = 70001
    X2 = torch.randn(n2, d, generator=g)
    idx2 = torch.randint(0, k, (n2,), generator=g)
    newc2, counts2 = km.update(X2.to(dev), idx2.to(dev), C0.to(dev))
    want_c2, want_n2 = R.kmeans_update(X2, idx2, C0)
    assert torch.equal(counts2.cpu().double(), want_n2)
    assert float((newc2.cpu().double() - want_c2).abs().max()) <= 1e-4
    assert lib.fbmm_check(None) == 0, lib.fbmm_last_error()


# ----------------------------------------------------------------------------- l2 distance
@pytest.mark.parametrize("shape", [(1, 200, 40, 300), (2, 130, 64, 257), (1, 1100, 96, 1300), (1, 64, 200, 520)])
def test_min_and_topk_l2_distance(dev, lib, shape):
    """distance="l2": squared distances sum_k (a - b)^2 (squared_l2 of the reference), both
    dims, all four layouts for one shape; checked against the direct fp64 formula."""
    from custom_matmul_kernels_b200 import MinBMMCUDA, TopkBMMCUDA
    l, m, k, n = shape
    g = torch.Generator().manual_seed(sum(shape) + 1)
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    mn, tk = MinBMMCUDA(distance="l2"), TopkBMMCUDA(distance="euclidean")
    combos = layouts(A.to(dev), B.to(dev)) if shape[1] == 200 else {"nn": (A.to(dev), B.to(dev))}
    for mode, (a, b) in combos.items():
        for dim in (1, 2):
            v, i = mn(a, b, dim=dim)
            R.check_min(v, i, A, B, dim, distance="l2")
            tv, ti = tk(a, b, k=9, dim=dim)
            R.check_topk(tv, ti, A, B, 9, dim, distance="l2")
    device_ok(lib)


def test_l2_distance_exact_and_nonnegative(dev, lib):
    """Integer operands: every squared distance is an exact integer, so values must match
    the oracle bit for bit; a column of B equal to a row of A gives distance exactly 0."""
    from custom_matmul_kernels_b200 import MinBMMCUDA
    A, B = R.exact_inputs(1, 140, 24, 300, seed=41, lo=-4, hi=4)
    B[0, :, 17] = A[0, 5]
    v, i = MinBMMCUDA(distance="l2")(A.to(dev), B.to(dev), dim=2)
    wv, wi = R.min_bmm(A, B, dim=2, distance="l2")
    assert torch.equal(v.cpu(), wv) and torch.equal(i.cpu(), wi)
    assert float(v[0, 5]) == 0.0 and bool((v >= 0).all())
    device_ok(lib)


# ----------------------------------------------------------------------------- l1 distance
@pytest.mark.parametrize("shape", [(1, 200, 40, 300), (2, 130, 64, 257), (1, 1100, 19, 1300), (1, 64, 200, 5200),
                                   (3, 1, 1, 1)])
def test_min_and_topk_l1_distance(dev, lib, shape):
    """distance="l1": sum_k |a - b| (l1 of the reference, kernels/bmm_helpers.cu:46-52), the SIMT
    kernel: both dims, all four layouts for one shape, k below and above 32 and 64, shapes with
    ragged rows / columns / K, several column chunks per row block (64 x 5200), 1 x 1 x 1;
    against the direct fp64 formula."""
    from custom_matmul_kernels_b200 import MinBMMCUDA, TopkBMMCUDA
    l, m, k, n = shape
    g = torch.Generator().manual_seed(sum(shape) + 3)
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    mn, tk = MinBMMCUDA(distance="l1"), TopkBMMCUDA(distance="manhattan")
    combos = layouts(A.to(dev), B.to(dev)) if shape[1] == 200 else {"nn": (A.to(dev), B.to(dev))}
    for mode, (a, b) in combos.items():
        for dim in (1, 2):
            v, i = mn(a, b, dim=dim)
            R.check_min(v, i, A, B, dim, distance="l1")
            for kk in (9, 40, 100):
                tv, ti = tk(a, b, k=kk, dim=dim)
                R.check_topk(tv, ti, A, B, kk, dim, distance="l1")
    device_ok(lib)


def test_l1_distance_exact_packed_and_16_bit(dev, lib):
    """Integer operands: every l1 distance is an exact integer, so values and min indices match the
    oracle bit for bit and a column equal to a row gives exactly 0; the packed candidates equal the
    unpacked result; 16-bit tensors are refused."""
    from custom_matmul_kernels_b200 import MinBMMCUDA, TopkBMMCUDA
    from custom_matmul_kernels_b200 import sharding as S
    A, B = R.exact_inputs(2, 140, 24, 300, seed=43, lo=-4, hi=4)
    B[0, :, 17] = A[0, 5]
    v, i = MinBMMCUDA(distance="l1")(A.to(dev), B.to(dev), dim=2)
    wv, wi = R.min_bmm(A, B, dim=2, distance="l1")
    assert torch.equal(v.cpu(), wv) and torch.equal(i.cpu(), wi)
    assert float(v[0, 5]) == 0.0 and bool((v >= 0).all())
    op = TopkBMMCUDA(distance="l1")
    tv, ti = op(A.to(dev), B.to(dev), k=12, dim=2)
    wtv, _ = R.topk_bmm(A, B, k=12, dim=2, distance="l1")
    assert torch.equal(tv.cpu(), wtv)
    pv, pi = S.unpack_candidates(op.packed(A.to(dev), B.to(dev), k=12, dim=2))
    assert torch.equal(pv, tv) and torch.equal(pi, ti)
    with pytest.raises(NotImplementedError):
        MinBMMCUDA(distance="l1")(A.to(dev).half(), B.to(dev).half(), dim=2)
    with pytest.raises(NotImplementedError):
        op(A.to(dev).bfloat16(), B.to(dev).bfloat16(), k=4, dim=2)
    device_ok(lib)


def test_every_op_on_shapes_that_straddle_row_blocks(dev, lib):
    """A spread of ops, layouts and both dims on shapes with several row blocks and ragged
    edges (300, 1100 and 129 rows), each against the oracle."""
    from custom_matmul_kernels_b200 import BMMCUDA, MBMMCUDA, MinBMMCUDA, TopkBMMCUDA, make_masks
    g = torch.Generator().manual_seed(5)
    for (l, m, k, n) in [(2, 300, 96, 400), (1, 1100, 160, 1300), (1, 129, 40, 77)]:
        A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
        Ad, Bd = A.to(dev), B.to(dev)
        At = Ad.transpose(1, 2).contiguous().transpose(1, 2)
        Bt = Bd.transpose(1, 2).contiguous().transpose(1, 2)
        want = torch.bmm(A.double(), B.double())
        for a, b in ((Ad, Bd), (At, Bt)):
            assert tol_ratio(BMMCUDA()(a, b), want) <= 1.0
            for dim in (1, 2):
                v, i = MinBMMCUDA()(a, b, dim=dim)
                R.check_min(v, i, A, B, dim)
                tv, ti = TopkBMMCUDA()(a, b, k=33, dim=dim)
                R.check_topk(tv, ti, A, B, 33, dim)
        v, i = MinBMMCUDA(distance="l2")(Ad, Bd, dim=2)
        R.check_min(v, i, A, B, 2, distance="l2")
        mask = torch.rand(l, m, n, generator=g) < 0.3
        mask[:, :128, :128] = False
        mask[:, 128:256, :128] = True
        bm, tm, em = make_masks(mask.to(dev))
        C = MBMMCUDA()(Ad, Bd, bm, tm, em).cpu()
        assert tol_ratio(C, want.masked_fill(~mask, 0)) <= 1.0 and bool((C[~mask] == 0).all())
    A, B = R.exact_inputs(1, 300, 32, 640, 7, -2, 2)
    v, i = MinBMMCUDA()(A.to(dev), B.to(dev), dim=2)
    wv, wi = torch.bmm(A, B).min(dim=2)
    assert torch.equal(v.cpu(), wv) and torch.equal(i.cpu(), wi)
    device_ok(lib)
