"""Masked batched matmul (drop-in for mbmm.py:7 MBMMCUDA)."""
from __future__ import annotations

import math

import torch

from .custom_kernel import CustomKernel, check, dtype_code_x16, layout_letter, operand, operand_x16


def make_masks(mask: torch.Tensor):
    """bool keep-mask [l,m,n] or [m,n] -> (block_mask, thread_mask, element_mask), uint8,
    built the way the reference's notebook builds them (colab/test_mbmm.ipynb:1295-1313):
    thread_mask counts the kept elements of each 8x8 tile, block_mask flags 128x128 tiles
    that keep anything, element_mask is the mask itself. Edge tiles are padded with zeros."""
    shared = mask.dim() == 2
    mk = mask[None] if shared else mask
    l, m, n = mk.shape
    m128, n128 = math.ceil(m / 128), math.ceil(n / 128)
    pad = torch.zeros((l, m128 * 128, n128 * 128), dtype=torch.int32, device=mask.device)
    pad[:, :m, :n] = mk.to(torch.int32)
    thread = pad.view(l, m128 * 16, 8, n128 * 16, 8).sum(dim=(2, 4))[:, :math.ceil(m / 8), :math.ceil(n / 8)]
    block = pad.view(l, m128, 128, n128, 128).sum(dim=(2, 4)) > 0
    out = (block.to(torch.uint8).contiguous(), thread.to(torch.uint8).contiguous(), mk.to(torch.uint8).contiguous())
    return tuple(t[0] for t in out) if shared else out


class MBMMCUDA(CustomKernel):
    """``MBMMCUDA(patch_m, patch_n, share_mask)(A, B, block_mask, thread_mask,
    element_mask, mode="nn") -> C`` (mbmm.py:8-12,109-196).

    C = (A @ B) * element_mask, and 0 wherever block_mask (128x128 tiles) or thread_mask
    (8x8 tiles) is 0; tiles whose block_mask byte is 0 are neither loaded nor multiplied.
    A mask byte of 1 KEEPS (colab/test_mbmm.ipynb:1295-1313; the docstring at
    mbmm.py:130-148 words it the other way round). Masks are uint8 with shapes
    [l,ceil(m/128),ceil(n/128)], [l,ceil(m/8),ceil(n/8)], [l,m,n], or without the batch
    axis when share_mask=True (mbmm.py:62-72). As in the reference only mode "nn" exists
    and inputs are made contiguous (mbmm.py:100-107,171-172). The reference cannot even be
    constructed (it opens kernels/mbmm_kernel.cu, mbmm.py:18); this class can."""

    def __init__(self, patch_m=4, patch_n=4, share_mask=False):
        super().__init__()
        self.patch_m = patch_m
        self.patch_n = patch_n
        self.share_mask = share_mask

    def _call_nn(self, A, B, block_mask, thread_mask, element_mask):
        l, m, k = A.shape
        n = B.shape[2]
        for name, t in (("block_mask", block_mask), ("thread_mask", thread_mask), ("element_mask", element_mask)):
            if t.dtype != torch.uint8:
                raise TypeError(f"{name} must be uint8")
            if t.device != A.device:
                raise ValueError(f"{name} must be on the same device as A")
        lead = () if self.share_mask else (l,)
        want = {
            "block_mask": lead + (math.ceil(m / 128), math.ceil(n / 128)),
            "thread_mask": lead + (math.ceil(m / 8), math.ceil(n / 8)),
            "element_mask": lead + (m, n),
        }
        got = {"block_mask": block_mask, "thread_mask": thread_mask, "element_mask": element_mask}
        for name, shape in want.items():
            if tuple(got[name].shape) != shape:
                raise ValueError(f"{name} has shape {tuple(got[name].shape)}, expected {shape}")
        C = torch.empty((l, m, n), device=A.device, dtype=A.dtype)
        if l == 0 or m == 0 or n == 0:
            return C
        if k == 0:
            return C.zero_()
        bm, tm, em = block_mask.contiguous(), thread_mask.contiguous(), element_mask.contiguous()
        if A.dtype in (torch.float16, torch.bfloat16):
            # fp16 / bf16 go to the tensor cores as they are; C comes back in their type
            a_keep, lda, sa = operand_x16(A)
            b_keep, ldb, sb = operand_x16(B.transpose(1, 2))
            with torch.cuda.device(A.device):
                check(self.lib.fbmm_mbmm_x16(
                    self.stream_ptr(A.device), a_keep.data_ptr(), lda, sa, b_keep.data_ptr(), ldb, sb,
                    dtype_code_x16(A.dtype), C.data_ptr(), n, m * n,
                    bm.data_ptr(), tm.data_ptr(), em.data_ptr(), 1 if self.share_mask else 0, l, m, n, k))
            return C
        a_keep, a_t, lda, sa = operand(A)
        b_keep, b_t, ldb, sb = operand(B)
        with torch.cuda.device(A.device):
            check(self.lib.fbmm_mbmm_f32(
                self.stream_ptr(A.device),
                a_keep.data_ptr(), layout_letter(a_t, False), lda, sa,
                b_keep.data_ptr(), layout_letter(b_t, True), ldb, sb,
                C.data_ptr(), n, m * n,
                bm.data_ptr(), tm.data_ptr(), em.data_ptr(), 1 if self.share_mask else 0,
                l, m, n, k))
        return C

    def _call_tt(self, A, B, block_mask, thread_mask, element_mask):
        raise NotImplementedError

    def _call_tn(self, A, B, block_mask, thread_mask, element_mask):
        raise NotImplementedError

    def _call_nt(self, A, B, block_mask, thread_mask, element_mask):
        raise NotImplementedError

    def __call__(self, A, B, block_mask, thread_mask, element_mask, mode="nn"):
        A3, B3, two_d = self.check_inputs(A, B, (torch.float32, torch.float16, torch.bfloat16))
        A3 = A3.contiguous()
        B3 = B3.contiguous()
        if two_d and not self.share_mask:
            block_mask, thread_mask, element_mask = block_mask[None], thread_mask[None], element_mask[None]
        if mode == "nn":
            C = self._call_nn(A3, B3, block_mask, thread_mask, element_mask)
        elif mode == "tt":
            C = self._call_tt(A3, B3, block_mask, thread_mask, element_mask)
        elif mode == "tn":
            C = self._call_tn(A3, B3, block_mask, thread_mask, element_mask)
        elif mode == "nt":
            C = self._call_nt(A3, B3, block_mask, thread_mask, element_mask)
        else:
            raise ValueError(f"unknown mode {mode!r}")
        return C[0] if two_d else C


class MBMMSoftmaxCUDA(MBMMCUDA):
    """``MBMMSoftmaxCUDA(share_mask=False)(A, B, block_mask, thread_mask, element_mask, scale=1.0) -> P``:
    the masked product followed by a softmax over the kept entries of every row,
    ``softmax(scale * (A @ B) with masked entries at -inf, dim=-1)``, without the scores
    ever being written out. This is the step that callers of the reference's masked bmm
    (mbmm.py:109-196) run next when the mask is an attention mask; the reference itself has
    no such op. Masked entries are 0 in P, and a row that keeps nothing is all zeros (torch
    gives NaN there). Masks as for MBMMCUDA, read as keep (non-zero) / drop; fp32 only."""

    def __call__(self, A, B, block_mask, thread_mask, element_mask, scale=1.0):
        A3, B3, two_d = self.check_inputs(A, B, (torch.float32,))
        if two_d and not self.share_mask:
            block_mask, thread_mask, element_mask = block_mask[None], thread_mask[None], element_mask[None]
        l, m, k = A3.shape
        n = B3.shape[2]
        lead = () if self.share_mask else (l,)
        want = {"block_mask": lead + (math.ceil(m / 128), math.ceil(n / 128)),
                "thread_mask": lead + (math.ceil(m / 8), math.ceil(n / 8)), "element_mask": lead + (m, n)}
        got = {"block_mask": block_mask, "thread_mask": thread_mask, "element_mask": element_mask}
        for name, shape in want.items():
            if got[name].dtype != torch.uint8:
                raise TypeError(f"{name} must be uint8")
            if got[name].device != A3.device:
                raise ValueError(f"{name} must be on the same device as A")
            if tuple(got[name].shape) != shape:
                raise ValueError(f"{name} has shape {tuple(got[name].shape)}, expected {shape}")
        P = torch.empty((l, m, n), device=A3.device, dtype=torch.float32)
        if l == 0 or m == 0 or n == 0:
            return P[0] if two_d else P
        if k == 0:
            raise ValueError("k must be positive")
        bm, tm, em = block_mask.contiguous(), thread_mask.contiguous(), element_mask.contiguous()
        a_keep, a_t, lda, sa = operand(A3)
        b_keep, b_t, ldb, sb = operand(B3)
        with torch.cuda.device(A3.device):
            check(self.lib.fbmm_mbmm_softmax_f32(
                self.stream_ptr(A3.device),
                a_keep.data_ptr(), layout_letter(a_t, False), lda, sa,
                b_keep.data_ptr(), layout_letter(b_t, True), ldb, sb,
                P.data_ptr(), n, m * n, bm.data_ptr(), tm.data_ptr(), em.data_ptr(), 1 if self.share_mask else 0,
                float(scale), l, m, n, k))
        return P[0] if two_d else P
