"""CPU oracle for the fused-BMM hot path. TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this module: only ``tests/``,
``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` do,
and there only as the checker or the timed CPU arm.

What it restates
----------------
The reference (DeMoriarty/custom_matmul_kernels) validates each of its four CUDA ops
against a pure-torch expression in its notebooks. Those expressions are the oracle:

* bmm      ``torch.bmm(A, B)``                               colab/test_bmm.ipynb:2121
* mbmm     ``torch.bmm(A, B).masked_fill_(~mask, 0)``        colab/test_mbmm.ipynb:1342-1343
           with the three uint8 masks derived from a bool mask as in
           colab/test_mbmm.ipynb:1295-1313 and applied with the kernel's precedence
           (block, then 8x8 thread tile, then element)       kernels/mbmm.cu:251-255,360-363,111-133
* min_bmm  ``torch.bmm(A, B).min(dim)``                      colab/test_minbmm.ipynb:2131-2132
           output shapes                                     minbmm.py:116-121
* topk_bmm ``torch.bmm(A, B).topk(k, dim=-1)`` for dim=2 and
           ``torch.bmm(B^T, A^T).topk(k, dim=-1)`` for dim=1 colab/test_topkbmm.ipynb:2673-2677
           (k is always the last output axis)                topkbmm.py:119-127

Pinning status
--------------
The reference ships no golden vectors, no seeds and no known-answer tests
(its inputs are unseeded ``torch.randn``), and its own kernels need CuPy plus a GPU, so
they cannot be executed where this oracle is built. The oracle is therefore pinned to
the reference's *test expressions* above (which run here, on CPU torch), and to
exact-arithmetic fixtures under ``tests/golden/`` whose answers do not depend on
rounding. Index choice between values closer than the tolerance is UNPINNED: the
reference kernels are racy there (kernels/minbmm.cu:76-79). This oracle and the CUDA
path both take the lowest index for min (``torch.min`` on CPU does the same).
"""
from __future__ import annotations

import math
import os
import time

import torch

RTOL = 1e-5
ATOL = 1e-4

# --------------------------------------------------------------------------------------
# the four ops
# --------------------------------------------------------------------------------------


def _as3d(A, B):
    if A.dim() == 2 and B.dim() == 2:
        return A[None], B[None], True
    if A.dim() == 3 and B.dim() == 3:
        return A, B, False
    raise ValueError("A and B need to be 2d or 3d")


def bmm(A: torch.Tensor, B: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """colab/test_bmm.ipynb:2121 -- C[l,m,n] = A[l,m,k] @ B[l,k,n]."""
    A3, B3, two_d = _as3d(A, B)
    C = torch.bmm(A3.to(dtype), B3.to(dtype))
    return C[0] if two_d else C


def make_masks(mask: torch.Tensor):
    """bool keep-mask [l,m,n] or [m,n] -> (block_mask, thread_mask, element_mask), uint8.

    colab/test_mbmm.ipynb:1295-1313: thread_mask holds the COUNT of kept elements in each
    8x8 tile, block_mask is 1 where a 128x128 tile keeps anything, element_mask is the mask.
    Shapes that are not multiples of 8 / 128 are padded with zeros first (the notebook
    only uses multiples)."""
    shared = mask.dim() == 2
    mk = mask[None] if shared else mask
    l, m, n = mk.shape
    m8, n8 = math.ceil(m / 8), math.ceil(n / 8)
    m128, n128 = math.ceil(m / 128), math.ceil(n / 128)
    pad = torch.zeros(l, m128 * 128, n128 * 128, dtype=torch.int32)
    pad[:, :m, :n] = mk.to(torch.int32)
    thread = pad.view(l, m128 * 16, 8, n128 * 16, 8).sum(dim=(2, 4))[:, :m8, :n8]
    block = pad.view(l, m128, 128, n128, 128).sum(dim=(2, 4)) > 0
    block_mask = block.to(torch.uint8)
    thread_mask = thread.to(torch.uint8)
    element_mask = mk.to(torch.uint8)
    if shared:
        return block_mask[0], thread_mask[0], element_mask[0]
    return block_mask, thread_mask, element_mask


def effective_keep(block_mask, thread_mask, element_mask, m, n):
    """Element-level keep mask the reference kernel realises from its three masks
    (kernels/mbmm.cu:251-255 block exit, :360-363 thread-tile skip, :111-133 multiply)."""
    bm = (block_mask != 0).repeat_interleave(128, dim=-2).repeat_interleave(128, dim=-1)[..., :m, :n]
    tm = (thread_mask != 0).repeat_interleave(8, dim=-2).repeat_interleave(8, dim=-1)[..., :m, :n]
    return bm & tm, element_mask


def mbmm(A, B, block_mask, thread_mask, element_mask, share_mask=False, dtype=torch.float32):
    """colab/test_mbmm.ipynb:1342-1343 restated with the kernel's three-level masks.

    Result = (A @ B) * element_mask, forced to 0 wherever the block mask or the 8x8
    thread mask is 0. (The kernel multiplies by the element-mask byte, so values other
    than 0/1 scale; kernels/mbmm.cu:127-128.)"""
    A3, B3, two_d = _as3d(A, B)
    l, m, _ = A3.shape
    n = B3.shape[2]
    if two_d and not share_mask:
        block_mask, thread_mask, element_mask = block_mask[None], thread_mask[None], element_mask[None]
    keep, em = effective_keep(block_mask, thread_mask, element_mask, m, n)
    C = torch.bmm(A3.to(dtype), B3.to(dtype))
    C = C * em.to(dtype)
    C = torch.where(keep.expand_as(C), C, torch.zeros((), dtype=dtype))
    return C[0] if two_d else C


def mbmm_softmax(A, B, block_mask, thread_mask, element_mask, share_mask=False, scale=1.0, dtype=torch.float64):
    """Softmax over the kept entries of each row of scale * (A @ B): the masked product of
    colab/test_mbmm.ipynb:1342-1343 with -inf instead of 0 at the masked entries, then
    torch.softmax along the last axis. Rows that keep nothing are all zeros. The keep set is
    the one the three masks define together (kernels/mbmm.cu:251-255,360-363,111-133)."""
    A3, B3, two_d = _as3d(A, B)
    l, m, _ = A3.shape
    n = B3.shape[2]
    bm, tm, em = (x[None] if x.dim() == 2 else x for x in (block_mask, thread_mask, element_mask))
    tiles, em = effective_keep(bm, tm, em, m, n)
    keep = (tiles & (em != 0)).expand(l, m, n)
    S = torch.bmm(A3.to(dtype), B3.to(dtype)) * scale
    S = S.masked_fill(~keep, float("-inf"))
    P = torch.softmax(S, dim=-1)
    P = torch.where(keep, P, torch.zeros_like(P))
    P = torch.nan_to_num(P, nan=0.0)
    return P[0] if two_d else P


def product(A3, B3, distance="inner", dtype=torch.float32):
    """The [l,m,n] matrix the epilogues reduce: the products (madd,
    kernels/bmm_helpers.cu:20-26) or, for distance "l2"/"euclidean", the squared distances
    sum_k (A[m,k] - B[k,n])^2 (squared_l2, kernels/bmm_helpers.cu:28-35; selected in
    minbmm.py:14-15 and topkbmm.py:17-18), computed directly, not through norms."""
    A3, B3 = A3.to(dtype), B3.to(dtype)
    if distance == "inner":
        return torch.bmm(A3, B3)
    if distance in ("l2", "euclidean"):
        out = torch.empty(A3.shape[0], A3.shape[1], B3.shape[2], dtype=dtype)
        step = max(1, (1 << 24) // max(1, A3.shape[2] * B3.shape[2]))  # bound the broadcast temporary
        Bt = B3.transpose(1, 2)  # [l, n, k]
        for r0 in range(0, A3.shape[1], step):
            d = A3[:, r0:r0 + step, None, :] - Bt[:, None, :, :]
            out[:, r0:r0 + step] = (d * d).sum(-1)
        return out
    if distance in ("l1", "manhattan"):  # l1, kernels/bmm_helpers.cu:46-52 (minbmm.py:16-17)
        out = torch.empty(A3.shape[0], A3.shape[1], B3.shape[2], dtype=dtype)
        step = max(1, (1 << 24) // max(1, A3.shape[2] * B3.shape[2]))
        Bt = B3.transpose(1, 2)
        for r0 in range(0, A3.shape[1], step):
            out[:, r0:r0 + step] = (A3[:, r0:r0 + step, None, :] - Bt[:, None, :, :]).abs().sum(-1)
        return out
    raise ValueError(f"distance {distance!r} is not restated")


def min_bmm(A, B, dim=1, dtype=torch.float32, distance="inner"):
    """colab/test_minbmm.ipynb:2131-2132; dim counted on the 3-D product, 2-D inputs bump
    dim by one first (minbmm.py:86-90). Returns (values fp32-ish, indices int64)."""
    A3, B3, two_d = _as3d(A, B)
    if two_d:
        dim += 1
    assert dim in (1, 2)
    C = product(A3, B3, distance, dtype)
    v, i = C.min(dim=dim)
    return (v[0], i[0]) if two_d else (v, i)


def topk_bmm(A, B, k=128, dim=1, dtype=torch.float32, distance="inner"):
    """colab/test_topkbmm.ipynb:2673-2677; output [l, R, k] with R = n (dim 1) or m (dim 2),
    largest first (topkbmm.py:119-127, kernels/topkbmm.cu:170-176)."""
    A3, B3, two_d = _as3d(A, B)
    if two_d:
        dim += 1
    assert dim in (1, 2)
    C = product(A3, B3, distance, dtype)
    if dim == 1:
        C = C.transpose(1, 2)
    kk = min(k, C.shape[-1])
    v, i = C.topk(kk, dim=-1)
    if kk < k:  # fewer candidates than k: pad -inf / -1 (kernels/topkbmm.cu:277-278)
        padv = torch.full(C.shape[:-1] + (k - kk,), float("-inf"), dtype=v.dtype)
        padi = torch.full(C.shape[:-1] + (k - kk,), -1, dtype=i.dtype)
        v, i = torch.cat([v, padv], -1), torch.cat([i, padi], -1)
    return (v[0], i[0]) if two_d else (v, i)


# --------------------------------------------------------------------------------------
# comparators (tolerance: rel 1e-5 / abs 1e-4; indices exact unless values compete
# within that tolerance)
# --------------------------------------------------------------------------------------


def values_close(got, want, rtol=RTOL, atol=ATOL):
    got = got.detach().cpu().double()
    want = want.detach().cpu().double()
    both_inf = torch.isinf(got) & torch.isinf(want) & (torch.sign(got) == torch.sign(want))
    err = (got - want).abs()
    ok = (err <= atol + rtol * want.abs()) | both_inf
    return bool(ok.all()), float(torch.where(both_inf, torch.zeros_like(err), err).max()) if err.numel() else 0.0


def check_min(got_v, got_i, A, B, dim, rtol=RTOL, atol=ATOL, distance="inner"):
    """Values within tolerance of the oracle; each returned index must point at an entry of
    the oracle product that is within tolerance of the oracle minimum. Returns a dict of
    counts; raises AssertionError on failure."""
    A3, B3, two_d = _as3d(A.cpu(), B.cpu())
    d = dim + 1 if two_d else dim
    C = product(A3, B3, distance, torch.float64)
    wv, wi = C.min(dim=d)
    gv = (got_v[None] if two_d else got_v).cpu().double()
    gi = (got_i[None] if two_d else got_i).cpu()
    assert gv.shape == wv.shape, (gv.shape, wv.shape)
    assert gi.dtype == torch.int64
    tol = atol + rtol * wv.abs()
    verr = (gv - wv).abs()
    assert bool((verr <= tol).all()), f"min values off: max err {float(verr.max()):.3e}"
    assert bool(((gi >= 0) & (gi < C.shape[d])).all()), "index out of range"
    at = torch.gather(C, d, gi.unsqueeze(d)).squeeze(d)
    assert bool(((at - wv).abs() <= tol).all()), "an index does not point at a (near-)minimum"
    return {"max_val_err": float(verr.max()), "idx_mismatch": int((gi != wi).sum())}


def check_topk(got_v, got_i, A, B, k, dim, rtol=RTOL, atol=ATOL, distance="inner"):
    """Values (descending) within tolerance of the oracle's; every index in range, unique per
    row, and pointing at a product entry within tolerance of the value reported for it."""
    A3, B3, two_d = _as3d(A.cpu(), B.cpu())
    d = dim + 1 if two_d else dim
    C = product(A3, B3, distance, torch.float64)
    if d == 1:
        C = C.transpose(1, 2).contiguous()
    kk = min(k, C.shape[-1])
    wv, wi = C.topk(kk, dim=-1)
    gv = (got_v[None] if two_d else got_v).cpu().double()
    gi = (got_i[None] if two_d else got_i).cpu()
    assert gv.shape == C.shape[:-1] + (k,), (gv.shape, C.shape, k)
    assert gi.dtype == torch.int64
    if kk < k:
        assert bool(torch.isneginf(gv[..., kk:]).all()) and bool((gi[..., kk:] == -1).all())
        gv, gi = gv[..., :kk], gi[..., :kk]
    tol = atol + rtol * wv.abs()
    verr = (gv - wv).abs()
    assert bool((verr <= tol).all()), f"top-k values off: max err {float(verr.max()):.3e}"
    assert bool((gv[..., :-1] >= gv[..., 1:]).all()), "values not descending"
    assert bool(((gi >= 0) & (gi < C.shape[-1])).all()), "index out of range"
    srt = gi.sort(dim=-1).values
    assert bool((srt[..., 1:] != srt[..., :-1]).all()), "duplicate index in a row"
    at = torch.gather(C, 2, gi)
    assert bool(((at - gv).abs() <= atol + rtol * at.abs()).all()), "an index does not match its value"
    return {"max_val_err": float(verr.max()), "idx_mismatch": int((gi != wi).sum())}


# --------------------------------------------------------------------------------------
# seeded inputs: the five benchmark configurations and small shapes
# --------------------------------------------------------------------------------------

CONFIG_SEEDS = {"c1": 1001, "c2": 1002, "c3": 1003, "c4": 1004, "c5": 1005}
CONFIG_SHAPES = {  # (l, m, k, n)
    "c1": (1, 16384, 64, 16384),
    "c2": (128, 1024, 128, 1024),
    "c3": (128, 1024, 64, 1024),
    "c4": (1, 1048576, 128, 65536),
    "c5": (1, 1048576, 256, 1048576),
}


def flops(l, m, k, n):
    """FLOP model of the reference harness, colab/test_bmm.ipynb:2104."""
    return 2.0 * l * m * n * k


def make_inputs(name: str, rows: int | None = None, cols: int | None = None, batches: int | None = None):
    """Seeded CPU tensors for configuration `name`. `rows`/`cols`/`batches` cut the
    problem down (leading rows of A, leading columns of B, leading batches) AFTER the
    generator position is fixed by the shape actually generated, so a cut-down problem is
    its own seeded problem, not a slice of the full one."""
    l, m, k, n = CONFIG_SHAPES[name]
    if rows is not None:
        m = rows
    if cols is not None:
        n = cols
    if batches is not None:
        l = batches
    g = torch.Generator().manual_seed(CONFIG_SEEDS[name])
    if name == "c2":
        A = torch.rand(l, m, k, generator=g) * 2 - 1
        B = torch.rand(l, k, n, generator=g) * 2 - 1
        return {"A": A, "B": B}
    A = torch.randn(l, m, k, generator=g)
    B = torch.randn(l, k, n, generator=g)
    out = {"A": A, "B": B}
    if name == "c3":
        half = l // 2
        mask = torch.zeros(l, m, n, dtype=torch.bool)
        mask[:half] = torch.tril(torch.ones(m, n, dtype=torch.bool))
        tiles = torch.rand(l - half, math.ceil(m / 64), math.ceil(n / 64), generator=g) < 0.3
        mask[half:] = tiles.repeat_interleave(64, 1).repeat_interleave(64, 2)[:, :m, :n]
        out["mask"] = mask
    if name == "c5":
        out["k"] = 64
    return out


def exact_inputs(l, m, k, n, seed, lo=-8, hi=8):
    """Small-integer-valued fp32 operands: every product and partial sum is exactly
    representable, so any correct implementation returns bit-identical values."""
    g = torch.Generator().manual_seed(seed)
    A = torch.randint(lo, hi + 1, (l, m, k), generator=g).float()
    B = torch.randint(lo, hi + 1, (l, k, n), generator=g).float()
    return A, B


# --------------------------------------------------------------------------------------
# k-means step (the consumer of min_bmm with the l2 distance)
# --------------------------------------------------------------------------------------


def kmeans_assign(X, centroids):
    """Nearest centroid by squared Euclidean distance, lowest index on ties: what
    MinBMMCUDA(distance="l2") returns for points X [n,d] against centroids [k,d]."""
    d2 = ((X.double()[:, None, :] - centroids.double()[None, :, :]) ** 2).sum(-1)
    v, i = d2.min(dim=1)
    return v, i


def kmeans_update(X, assignment, centroids):
    """Mean of the points of every cluster (fp64 sums); empty clusters keep their centroid."""
    k, d = centroids.shape
    sums = torch.zeros(k, d, dtype=torch.float64)
    sums.index_add_(0, assignment, X.double())
    counts = torch.bincount(assignment, minlength=k).double()
    out = centroids.double().clone()
    live = counts > 0
    out[live] = sums[live] / counts[live, None]
    return out, counts


# --------------------------------------------------------------------------------------
# timed CPU arm (reference semantics on the host cores)
# --------------------------------------------------------------------------------------


def cpu_time(fn, repeat=1):
    fn()
    best = float("inf")
    for _ in range(repeat):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


def cpu_min_bmm_rows_per_s(A, B, repeat=1):
    torch.set_num_threads(os.cpu_count() or 1)
    t = cpu_time(lambda: torch.bmm(A, B).min(dim=-1), repeat)
    return A.shape[0] * A.shape[1] / t, t


def cpu_topk_bmm_chunked(A, B, k, chunk=131072):
    """Running top-k over column chunks of B (the full product would not fit in RAM)."""
    best_v = best_i = None
    n = B.shape[2]
    for c0 in range(0, n, chunk):
        C = torch.bmm(A, B[:, :, c0:c0 + chunk])
        v, i = C.topk(min(k, C.shape[-1]), dim=-1)
        i = i + c0
        if best_v is None:
            best_v, best_i = v, i
        else:
            cv, ci = torch.cat([best_v, v], -1), torch.cat([best_i, i], -1)
            best_v, sel = cv.topk(k, dim=-1)
            best_i = torch.gather(ci, -1, sel)
    return best_v, best_i
