"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header
declares, validates arguments before touching a device, and answers workspace queries."""
import ctypes
import os
import re

import pytest
import torch

from conftest import ROOT
from custom_matmul_kernels_b200 import custom_kernel as ck

HEADER = os.path.join(ROOT, "include", "fbmm.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fbmm_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib):
    syms = declared_symbols()
    assert len(syms) >= 10
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/fbmm.h but not exported"
        assert s in ck.SIGNATURES, f"{s} has no ctypes signature"
    assert sorted(ck.SIGNATURES) == syms


def test_header_cites_reference_for_every_entry_point():
    text = open(HEADER).read()
    for cite in ("kernels/bmm.cu:185", "kernels/mbmm.cu:209", "kernels/minbmm.cu:348", "kernels/topkbmm.cu:500",
                 "kernels/bitonic_sort.cu:183", "custom_kernel.py:12"):
        assert cite in text


def test_version_and_error_string(lib):
    assert lib.fbmm_version() >= 1000
    assert isinstance(lib.fbmm_last_error(), bytes)


def _call_bmm(lib, A=64, lda=4, B=64, ldb=4, C=64, l=1, m=4, n=4, k=4, la=ord("n"), lb=ord("n")):
    return lib.fbmm_bmm_f32(None, A, la, lda, m * k, B, lb, ldb, k * n, C, n, m * n, l, m, n, k)


def test_argument_validation_needs_no_device(lib):
    # every one of these returns before any CUDA call
    assert _call_bmm(lib, m=0) == ck.FBMM_ERR_INVALID
    assert b"positive" in lib.fbmm_last_error()
    assert _call_bmm(lib, C=None) == ck.FBMM_ERR_INVALID
    assert _call_bmm(lib, la=ord("x")) == ck.FBMM_ERR_INVALID
    assert _call_bmm(lib, A=None) == ck.FBMM_ERR_INVALID
    assert _call_bmm(lib, A=68) == ck.FBMM_ERR_ALIGN          # base not 16-byte aligned
    assert _call_bmm(lib, lda=6, k=6, ldb=4) == ck.FBMM_ERR_ALIGN   # pitch not a multiple of 4
    assert _call_bmm(lib, lda=2) == ck.FBMM_ERR_INVALID       # pitch shorter than a row
    with pytest.raises(ValueError):
        ck.check(_call_bmm(lib, m=-1))


def test_topk_and_min_validation(lib):
    rc = lib.fbmm_topk_bmm_f32(None, 64, ord("n"), 4, 16, 64, ord("n"), 4, 16, 64, 64, 1, 4, 4, 4, 129, 2, 0, 0, None, 0)
    assert rc == ck.FBMM_ERR_INVALID and b"1..128" in lib.fbmm_last_error()
    rc = lib.fbmm_topk_bmm_f32(None, 64, ord("n"), 4, 16, 64, ord("n"), 4, 16, 64, 64, 1, 4, 4, 4, 8, 3, 0, 0, None, 0)
    assert rc == ck.FBMM_ERR_INVALID and b"dim" in lib.fbmm_last_error()
    rc = lib.fbmm_min_bmm_f32(None, 64, ord("n"), 4, 16, 64, ord("n"), 4, 16, 64, 64, 1, 4, 4, 4, 2, 0, None, 0)
    assert rc == ck.FBMM_ERR_WORKSPACE
    rc = lib.fbmm_min_bmm_f32(None, 64, ord("n"), 4, 16, 64, ord("n"), 4, 16, 64, 64, 1, 4, 4, 4, 2, 7, None, 0)
    assert rc == ck.FBMM_ERR_INVALID and b"distance" in lib.fbmm_last_error()
    # FBMM_DIST_L1 (2) is an fp32 mode: the 16-bit entries refuse it before touching anything
    rc = lib.fbmm_min_bmm_x16(None, 64, 8, 32, 64, 8, 32, 1, 64, 64, 1, 4, 4, 8, 2, 2, None, 0)
    assert rc == ck.FBMM_ERR_UNSUPPORTED and b"fp32" in lib.fbmm_last_error()
    rc = lib.fbmm_topk_merge_f32(None, 64, 64, 0, 4, 8, 64, 64)
    assert rc == ck.FBMM_ERR_INVALID


def test_workspace_queries(lib):
    assert lib.fbmm_min_bmm_workspace_bytes(1, 16384, 16384, 64, 2, 0) == 16384 * 8
    assert lib.fbmm_min_bmm_workspace_bytes(2, 100, 300, 64, 1, 0) == 2 * 300 * 8
    # l2 distance adds room for the squared norms of both operands
    assert lib.fbmm_min_bmm_workspace_bytes(1, 256, 512, 64, 2, 1) == 256 * 8 + 256 * 4 + 512 * 4
    # many row blocks: one column chunk; the running lists of the units in flight (per SM
    # 128 rows x 64 or 128 list slots x 8 bytes) and a few KB of sweep-pacing counters
    sms = 148  # assumed by the library without a device; a B200 has as many
    w64 = lib.fbmm_topk_bmm_workspace_bytes(1, 1 << 20, 1 << 20, 256, 64, 2, 0)
    w128 = lib.fbmm_topk_bmm_workspace_bytes(1, 1 << 20, 1 << 20, 256, 100, 2, 0)
    lists64 = sms * 128 * 64 * 8
    assert lists64 < w64 < lists64 + (1 << 20) and w128 - w64 == lists64
    # few row blocks: per-chunk candidate lists on top
    assert lib.fbmm_topk_bmm_workspace_bytes(1, 128, 1 << 16, 64, 64, 2, 0) > w64


def test_presplit_query_follows_dim(lib):
    """dim = 1 swaps the operands' roles; its scratch is that of the dim = 2 call on (B^T, A^T)."""
    l, m, n, k = 1, 4096, 65536, 256
    # A [m,k] row-major ('n'), B [k,n] row-major ('n'): as row problem of dim 1, rows come from B
    # (stored [k][n], i.e. the 't' layout of a row operand) and columns from A (stored [m][k], the 't'
    # layout of a column operand)
    q1 = lib.fbmm_presplit_workspace_bytes(l, m, n, k, 1, ord("n"), k, m * k, ord("n"), n, k * n)
    q2 = lib.fbmm_presplit_workspace_bytes(l, n, m, k, 2, ord("t"), n, k * n, ord("t"), k, m * k)
    assert q1 == q2 > 0
    assert q1 != lib.fbmm_presplit_workspace_bytes(l, m, n, k, 2, ord("n"), k, m * k, ord("n"), n, k * n)
    assert lib.fbmm_presplit_workspace_bytes(l, m, n, k, 3, ord("n"), k, m * k, ord("n"), n, k * n) == 0


def test_sharded_and_packed_validation(lib):
    rc = lib.fbmm_topk_bmm_packed_f32(None, 64, ord("n"), 4, 16, 64, ord("n"), 4, 16, None, 1, 4, 4, 4, 8, 2, 0, None, 0)
    assert rc == ck.FBMM_ERR_INVALID and b"candidates" in lib.fbmm_last_error()
    rc = lib.fbmm_topk_bmm_packed_f32(None, 64, ord("n"), 4, 16, 64, ord("n"), 4, 16, 68, 1, 4, 4, 4, 8, 2, 0, None, 0)
    assert rc == ck.FBMM_ERR_ALIGN
    rc = lib.fbmm_topk_merge_packed_f32(None, 64, 0, 4, 8, 128, 64, 64)
    assert rc == ck.FBMM_ERR_INVALID
    rc = lib.fbmm_topk_merge_packed_f32(None, 64, 2, 4, 8, -1, 64, 64)
    assert rc == ck.FBMM_ERR_INVALID
    # rank out of range, null communicator, missing workspace: all before any CUDA or NCCL call
    args = lambda comm, world, rank, ws, wsb: lib.fbmm_topk_bmm_sharded_f32(  # noqa: E731
        None, comm, world, rank, 64, ord("n"), 4, 64, ord("n"), 4, 4, 64, 64, 4, 4, 4, 2, 0, 1, ws, wsb)
    assert args(1, 2, 2, None, 0) == ck.FBMM_ERR_INVALID
    assert args(None, 2, 0, None, 0) == ck.FBMM_ERR_INVALID
    assert args(1, 2, 0, None, 0) == ck.FBMM_ERR_WORKSPACE
    need = lib.fbmm_topk_bmm_sharded_workspace_bytes(8, 1 << 20, 1 << 17, 256, 64, 0, ord("n"), 256, ord("n"), 1 << 17)
    # send + 8 received lists of 2^20 x 64 entries of 8 bytes, plus the local step's scratch
    assert need > 9 * (1 << 20) * 64 * 8
    assert lib.fbmm_comm_init_rank(None, 2, 0, None) == ck.FBMM_ERR_INVALID


def test_wrappers_reject_bad_inputs_on_cpu():
    from custom_matmul_kernels_b200 import BMMCUDA, MBMMCUDA, MinBMMCUDA, TopkBMMCUDA
    A, B = torch.zeros(2, 4, 8), torch.zeros(2, 8, 4)
    for op in (BMMCUDA(), MinBMMCUDA(), TopkBMMCUDA()):
        with pytest.raises(ValueError):
            op(A, B)  # not CUDA tensors
        with pytest.raises(ValueError):
            op(A, torch.zeros(2, 7, 4))
        with pytest.raises(TypeError):
            op(A.double(), B.double())
        with pytest.raises(TypeError):
            op(A.half(), B)  # dtypes differ
        with pytest.raises(ValueError):
            op(A[0], B)
    assert MinBMMCUDA(distance="l1")._distance_code == 2 and TopkBMMCUDA(distance="manhattan")._distance_code == 2
    assert MinBMMCUDA(distance="euclidean")._distance_code == 1 and TopkBMMCUDA(distance="l2")._distance_code == 1
    with pytest.raises(ValueError):
        TopkBMMCUDA(distance="cosine")
    assert BMMCUDA().get_mode(A, B.transpose(1, 2).contiguous().transpose(1, 2)) == "nt"
    assert MBMMCUDA(share_mask=True).share_mask is True


def test_operand_x16_descriptor_logic():
    """`operand_x16` passes k-contiguous, 8-element-aligned storage through and repacks the rest."""
    from custom_matmul_kernels_b200.custom_kernel import operand_x16
    X = torch.zeros(2, 5, 16, dtype=torch.float16)
    keep, ld, st = operand_x16(X)
    assert keep is X and (ld, st) == (16, 80)
    keep, ld, st = operand_x16(torch.zeros(2, 16, 5, dtype=torch.float16).transpose(1, 2))  # k not contiguous
    assert keep.shape == (2, 5, 16) and keep.is_contiguous() and (ld, st) == (16, 80)
    keep, ld, st = operand_x16(torch.ones(1, 3, 12, dtype=torch.bfloat16))  # pitch 12 is not a multiple of 8
    assert keep.shape == (1, 3, 16) and (ld, st) == (16, 48) and float(keep[0, 0, 11]) == 1 and float(keep[0, 0, 12]) == 0


def test_operand_descriptor_logic():
    """`operand` passes TMA-addressable storage through and repacks the rest."""
    X = torch.zeros(2, 8, 12)
    keep, t, ld, bs = ck.operand(X)
    assert keep is X and not t and ld == 12 and bs == 96
    Xt = torch.zeros(2, 12, 8).transpose(1, 2)          # stored [l][12][8], logical [l][8][12]
    keep, t, ld, bs = ck.operand(Xt)
    assert keep is Xt and t and ld == 8
    odd = torch.arange(2 * 5 * 7, dtype=torch.float32).view(2, 5, 7)   # pitch 7: not addressable
    keep, t, ld, bs = ck.operand(odd)
    assert keep is not odd and not t and ld == 8 and bs == 40
    assert torch.equal(keep[:, :, :7], odd) and bool((keep[:, :, 7:] == 0).all())
    off = torch.zeros(2 * 8 * 12 + 1)[1:].view(2, 8, 12)               # base off by 4 bytes
    keep, _, _, _ = ck.operand(off)
    assert keep.data_ptr() % 16 == 0
    bc = torch.zeros(1, 8, 12).expand(3, 8, 12)                        # broadcast batch: passed through
    keep, _, _, bs = ck.operand(bc)
    assert keep is bc and bs == 0


def test_make_masks_matches_oracle():
    from custom_matmul_kernels_b200 import make_masks
    from oracle import ref_semantics as R
    g = torch.Generator().manual_seed(1)
    mask = torch.rand(2, 200, 136, generator=g) < 0.2
    mask[0, :128, :128] = False
    for a, b in zip(make_masks(mask), R.make_masks(mask)):
        assert torch.equal(a, b)
    for a, b in zip(make_masks(mask[0]), R.make_masks(mask[0])):
        assert torch.equal(a, b)
