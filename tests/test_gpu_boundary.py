"""GPU tests of the C-ABI boundary beyond the plain calls: broadcast operands, the packed
candidate format of the column-sharded exchange, the workspace query for dim = 1, and the
bounded-wait failure path (made to run out on purpose by the library's own self-test kernel,
which returns normally: nothing faults, traps or hangs)."""
import pytest
import torch

from conftest import tol_ratio
from custom_matmul_kernels_b200 import custom_kernel as ck
from custom_matmul_kernels_b200 import sharding as S
from oracle import c_oracle
from oracle import ref_semantics as R

pytestmark = pytest.mark.gpu


def stream():
    return torch.cuda.current_stream().cuda_stream


def test_broadcast_operand_through_the_c_abi(dev, lib):
    """One B shared by three batches, passed with batch stride 0 (l = 3)."""
    l, m, k, n = 3, 200, 40, 136
    g = torch.Generator().manual_seed(11)
    A, B = torch.randn(l, m, k, generator=g), torch.randn(1, k, n, generator=g)
    Ad, Bd = A.to(dev), B.to(dev)
    C = torch.empty(l, m, n, device=dev)
    rc = lib.fbmm_bmm_f32(stream(), Ad.data_ptr(), ord("n"), k, m * k, Bd.data_ptr(), ord("n"), n, 0,
                          C.data_ptr(), n, m * n, l, m, n, k)
    assert rc == 0, lib.fbmm_last_error()
    want = R.bmm(A, B.expand(l, k, n), dtype=torch.float64)
    assert tol_ratio(C, want) <= 1.0
    # shared A and per-batch B, min over columns; exact integers so that bits must agree
    Ae, Be = R.exact_inputs(1, 130, 24, 300, seed=5)
    Be3 = torch.cat([Be, Be.flip(2), Be * 2], 0)
    Aed, Bed = Ae.to(dev), Be3.to(dev)
    v = torch.empty(3, 130, device=dev)
    i = torch.empty(3, 130, device=dev, dtype=torch.int64)
    ws_bytes = lib.fbmm_min_bmm_workspace_bytes(3, 130, 300, 24, 2, 0)
    ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
    rc = lib.fbmm_min_bmm_f32(stream(), Aed.data_ptr(), ord("n"), 24, 0, Bed.data_ptr(), ord("n"), 300, 24 * 300,
                              v.data_ptr(), i.data_ptr(), 3, 130, 300, 24, 2, 0, ws.data_ptr(), ws_bytes)
    assert rc == 0, lib.fbmm_last_error()
    wv, wi = c_oracle.min_bmm(Ae.expand(3, 130, 24), Be3, 2)
    assert torch.equal(v.cpu(), wv) and torch.equal(i.cpu(), wi)
    # the wrappers pass an expanded tensor through without copying it
    from custom_matmul_kernels_b200 import BMMCUDA
    C2 = BMMCUDA()(Ad, Bd.expand(l, k, n))
    assert torch.equal(C2, C)
    assert lib.fbmm_check(None) == 0


def test_packed_candidates_equal_the_unpacked_result(dev, lib):
    from custom_matmul_kernels_b200 import TopkBMMCUDA
    op = TopkBMMCUDA()
    g = torch.Generator().manual_seed(12)
    for (m, k, n, kk) in [(300, 24, 1000, 9), (2000, 64, 4096, 64), (128, 32, 40000, 100)]:   # last: several column chunks
        A, B = torch.randn(1, m, k, generator=g).to(dev), torch.randn(1, k, n, generator=g).to(dev)
        v, i = op(A, B, k=kk, dim=2)
        p = op.packed(A, B, k=kk, dim=2)
        assert p.dtype == torch.int64 and p.shape == (1, m, kk)
        pv, pi = S.unpack_candidates(p)
        assert torch.equal(pv, v) and torch.equal(pi, i)
        # column shards -> packed lists -> packed merge == the unsharded answer, bit for bit
        world = 3
        stride = S.shard_stride(n, world, 128)
        lists = []
        for r in range(world):
            c0, c1 = S.shard_range(n, world, r, 128)
            lists.append(op.packed(A, B[:, :, c0:c1].contiguous(), k=kk, dim=2).reshape(m, kk))
        mv, mi = S.merge_packed_cuda(torch.stack(lists).contiguous(), kk, stride)
        assert torch.equal(mv, v[0])
        R.check_topk(mv[None], mi[None], A, B, kk, 2)
        tv, ti = S.merge_packed_torch(torch.stack(lists).cpu(), kk, stride)
        assert torch.equal(mv.cpu(), tv)
    # dim = 1 and fewer entries than k: empty slots are (-inf, -1)
    A, B = torch.randn(1, 20, 16, generator=g).to(dev), torch.randn(1, 16, 50, generator=g).to(dev)
    pv, pi = S.unpack_candidates(op.packed(A, B, k=32, dim=1))
    assert pv.shape == (1, 50, 32) and bool((pi[..., 20:] == -1).all()) and bool(torch.isneginf(pv[..., 20:]).all())
    assert lib.fbmm_check(None) == 0


def test_presplit_query_is_used_for_dim_1(dev, lib):
    """A dim = 1 call whose row operand (B) is the large one: with the dim-aware query the
    scratch fits the planes the kernel wants, and the result has the same bits as without."""
    from custom_matmul_kernels_b200 import MinBMMCUDA
    m, k, n = 2048, 160, 4096          # k > 128: the row operand (here B) streams, so it is split too
    g = torch.Generator().manual_seed(13)
    A, B = torch.randn(1, m, k, generator=g).to(dev), torch.randn(1, k, n, generator=g).to(dev)
    own = (lib.fbmm_min_bmm_workspace_bytes(1, m, n, k, 1, 0) + 255) // 256 * 256
    extra = lib.fbmm_presplit_workspace_bytes(1, m, n, k, 1, ord("n"), k, m * k, ord("n"), n, k * n)
    assert extra > 0
    outs = []
    for ws_bytes in (own, own + extra):
        v = torch.empty(1, n, device=dev)
        i = torch.empty(1, n, device=dev, dtype=torch.int64)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        rc = lib.fbmm_min_bmm_f32(stream(), A.data_ptr(), ord("n"), k, m * k, B.data_ptr(), ord("n"), n, k * n,
                                  v.data_ptr(), i.data_ptr(), 1, m, n, k, 1, 0, ws.data_ptr(), ws_bytes)
        assert rc == 0, lib.fbmm_last_error()
        outs.append((v, i))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])
    wv, wi = MinBMMCUDA()(A, B, dim=1)
    assert torch.equal(wv, outs[1][0])
    R.check_min(outs[1][0], outs[1][1], A, B, 1)


def test_bounded_wait_expiry_is_reported_once(dev, lib):
    """A wait that nothing satisfies gives up after its budget, the kernel returns, and the
    host sees FBMM_ERR_DEVICE exactly once; the device stays usable."""
    assert lib.fbmm_check(None) == 0
    assert lib.fbmm_selftest_wait_expiry(stream()) == 0
    assert lib.fbmm_check(stream()) == ck.FBMM_ERR_DEVICE
    assert b"bounded wait" in lib.fbmm_last_error()
    assert lib.fbmm_check(stream()) == 0
    # and the next real call is unaffected
    from custom_matmul_kernels_b200 import MinBMMCUDA
    d = R.make_inputs("c1", rows=256, cols=512)
    v, i = MinBMMCUDA()(d["A"].to(dev), d["B"].to(dev), dim=2)
    R.check_min(v, i, d["A"], d["B"], 2)
    assert lib.fbmm_check(None) == 0


def test_tensor_map_cache_returns_the_same_answers(dev, lib):
    """Repeated calls on the same buffers (cached descriptors) and on new buffers of the same
    shape (new descriptors) agree."""
    from custom_matmul_kernels_b200 import BMMCUDA
    op = BMMCUDA()
    g = torch.Generator().manual_seed(14)
    A, B = torch.randn(2, 256, 64, generator=g).to(dev), torch.randn(2, 64, 256, generator=g).to(dev)
    C1 = op(A, B)
    C2 = op(A, B)
    A2, B2 = A.clone(), B.clone()
    C3 = op(A2, B2)
    assert torch.equal(C1, C2) and torch.equal(C1, C3)
    for _ in range(40):  # more distinct buffers than the cache holds
        X = torch.randn(1, 128, 32, generator=g).to(dev)
        assert tol_ratio(op(X, X.transpose(1, 2).contiguous()), R.bmm(X.cpu(), X.cpu().transpose(1, 2), dtype=torch.float64)) <= 1.0
    assert torch.equal(op(A, B), C1)


def test_masked_row_softmax_matches_the_oracle(dev, lib):
    """softmax(scale * A @ B with masked entries at -inf) against the fp64 oracle: causal and
    random-tile masks of configuration 3's kind (mask tiles through TMA), a ragged shape with
    an all-masked block and empty rows (masks read from global memory), shared masks.
    Tolerance: abs 2e-6 + rel 1e-4 on the probabilities (fp32 scores are good to 1e-5 rel /
    1e-4 abs, which the exponential turns into a relative error of that size)."""
    from custom_matmul_kernels_b200 import MBMMSoftmaxCUDA, make_masks

    def check(P, want, mask):
        P, want = P.cpu().double(), want.double()
        assert bool((P[~mask] == 0).all()), "a masked entry is not exactly zero"
        err = (P - want).abs()
        assert bool((err <= 2e-6 + 1e-4 * want.abs()).all()), float(err.max())
        rows_kept = mask.any(dim=-1)
        assert bool(((P.sum(-1) - 1).abs()[rows_kept] < 1e-4).all()) and bool((P.sum(-1)[~rows_kept] == 0).all())

    g = torch.Generator().manual_seed(31)
    # configuration-3-like: multiples of 128, causal + 64x64 random tiles
    l, m, k, n = 4, 1024, 64, 1024
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    mask = torch.zeros(l, m, n, dtype=torch.bool)
    mask[:2] = torch.tril(torch.ones(m, n, dtype=torch.bool))
    tiles = torch.rand(2, m // 64, n // 64, generator=g) < 0.3
    mask[2:] = tiles.repeat_interleave(64, 1).repeat_interleave(64, 2)
    bm, tm, em = make_masks(mask.to(dev))
    scale = 1.0 / 8.0
    P = MBMMSoftmaxCUDA()(A.to(dev), B.to(dev), bm, tm, em, scale=scale)
    check(P, R.mbmm_softmax(A, B, bm.cpu(), tm.cpu(), em.cpu(), scale=scale), mask)
    assert torch.equal(P, MBMMSoftmaxCUDA()(A.to(dev), B.to(dev), bm, tm, em, scale=scale))  # deterministic
    # ragged, k > 128 (A streams), a dead block, rows that keep nothing
    l, m, k, n = 2, 200, 160, 300
    A, B = torch.randn(l, m, k, generator=g), torch.randn(l, k, n, generator=g)
    mask = torch.rand(l, m, n, generator=g) < 0.4
    mask[:, :128, 128:256] = False
    mask[0, 7] = False
    mask[1, 150:] = False
    bm, tm, em = make_masks(mask.to(dev))
    P = MBMMSoftmaxCUDA()(A.to(dev), B.to(dev), bm, tm, em, scale=0.5)
    check(P, R.mbmm_softmax(A, B, bm.cpu(), tm.cpu(), em.cpu(), scale=0.5), mask)
    # shared masks, 2-D inputs
    bm1, tm1, em1 = make_masks(mask[0].to(dev))
    P1 = MBMMSoftmaxCUDA(share_mask=True)(A[0].to(dev), B[0].to(dev), bm1, tm1, em1, scale=0.5)
    assert torch.equal(P1, P[0])
    assert lib.fbmm_check(None) == 0
