"""Plain batched fp32 matmul on the B200 tensor cores (drop-in for bmm.py:7 BMMCUDA)."""
from __future__ import annotations

import torch

from .custom_kernel import CustomKernel, check, dtype_code_x16, layout_letter, operand, operand_x16

_X16 = (torch.float16, torch.bfloat16)


class BMMCUDA(CustomKernel):
    """``BMMCUDA(patch_m, patch_n)(A, B) -> C`` with A [l,m,k] (or [m,k]) and B [l,k,n]
    (or [k,n]), fp32 (bmm.py:8,68-129); fp16 / bf16 operands are accepted too (the reference
    admits torch.half, bmm.py:89, but its kernel takes float* only) and give C in their type.

    `patch_m` / `patch_n` sized the reference's CTA raster patch (bmm.py:19-21); they are
    accepted and stored but never change results. Unlike the reference, which launched
    its "nn" kernel for every stride layout (bmm.py:115), transposed views are honoured,
    and the result lives on A's device rather than on cuda:0 (bmm.py:106)."""

    def __init__(self, patch_m=4, patch_n=4):
        super().__init__()
        self.patch_m = patch_m
        self.patch_n = patch_n

    def __call__(self, A, B):
        A3, B3, two_d = self.check_inputs(A, B, (torch.float32,) + _X16)
        l, m, k = A3.shape
        n = B3.shape[2]
        C = torch.empty((l, m, n), device=A3.device, dtype=A3.dtype)  # the reference's C has A's type (bmm.py:106)
        if l == 0 or m == 0 or n == 0:
            return C[0] if two_d else C
        if k == 0:
            C.zero_()
            return C[0] if two_d else C
        if A3.dtype in _X16:
            # fp16 / bf16 go to the tensor cores as they are (fp32 accumulation, C rounded to nearest)
            a_keep, lda, sa = operand_x16(A3)
            b_keep, ldb, sb = operand_x16(B3.transpose(1, 2))
            with torch.cuda.device(A3.device):
                check(self.lib.fbmm_bmm_x16(
                    self.stream_ptr(A3.device), a_keep.data_ptr(), lda, sa, b_keep.data_ptr(), ldb, sb,
                    dtype_code_x16(A3.dtype), C.data_ptr(), n, m * n, l, m, n, k))
            return C[0] if two_d else C
        a_keep, a_t, lda, sa = operand(A3)
        b_keep, b_t, ldb, sb = operand(B3)
        with torch.cuda.device(A3.device):
            check(self.lib.fbmm_bmm_f32(
                self.stream_ptr(A3.device),
                a_keep.data_ptr(), layout_letter(a_t, False), lda, sa,
                b_keep.data_ptr(), layout_letter(b_t, True), ldb, sb,
                C.data_ptr(), n, m * n, l, m, n, k))
        return C[0] if two_d else C
