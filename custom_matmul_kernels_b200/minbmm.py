"""Fused matmul + min/argmin (drop-in for minbmm.py:7 MinBMMCUDA)."""
from __future__ import annotations

import torch

from .custom_kernel import (FBMM_DIST_L1, CustomKernel, check, distance_code, dtype_code_x16, layout_letter, operand,
                            operand_x16)

_X16 = (torch.float16, torch.bfloat16)


class MinBMMCUDA(CustomKernel):
    """``MinBMMCUDA(patch_m, patch_n, distance)(A, B, dim) -> (values, indices)``.

    A [l,m,k] @ B [l,k,n] is reduced with min/argmin along `dim` of the 3-D product
    without ever being written out: dim=1 gives [l,n], dim=2 gives [l,m]
    (minbmm.py:116-121); for 2-D inputs `dim` is bumped by one first (minbmm.py:86-90).
    values are fp32, indices int64. Ties resolve to the lowest index (the reference is
    racy there, kernels/minbmm.cu:76-79). distance="inner" reduces the products,
    distance="l2"/"euclidean" the squared distances sum_k (A[m,k] - B[k,n])^2
    (minbmm.py:12-19), distance="l1"/"manhattan" the sums sum_k |A[m,k] - B[k,n]|
    (minbmm.py:16-17; fp32 tensors only: a SIMT kernel, the tensor cores cannot form |a - b|)."""

    def __init__(self, patch_m=4, patch_n=4, distance="inner"):
        super().__init__()
        self.patch_m = patch_m
        self.patch_n = patch_n
        self._distance_code = distance_code(distance)
        self.distance = distance

    def __call__(self, A, B, dim=1):
        A3, B3, two_d = self.check_inputs(A, B, (torch.float32,) + _X16)
        if two_d:
            dim += 1
        if dim not in (1, 2):
            raise ValueError("dim must be 1 or 2 on the 3-D product (0 or 1 for 2-D inputs)")
        l, m, k = A3.shape
        n = B3.shape[2]
        if min(l, m, n, k) <= 0:
            raise ValueError(f"empty problem: l={l} m={m} n={n} k={k}")
        rows = n if dim == 1 else m
        values = torch.empty((l, rows), device=A3.device, dtype=torch.float32)
        indices = torch.empty((l, rows), device=A3.device, dtype=torch.int64)
        if A3.dtype in _X16:
            if self._distance_code == FBMM_DIST_L1:
                raise NotImplementedError("distance='l1' takes fp32 tensors only")
            # fp16 / bf16 go to the tensor cores as they are; values come back in fp32
            a_keep, lda, sa = operand_x16(A3)
            b_keep, ldb, sb = operand_x16(B3.transpose(1, 2))
            ws_bytes = self.lib.fbmm_min_bmm_workspace_bytes(l, m, n, k, dim, self._distance_code)
            ws = torch.empty(max(ws_bytes, 256), device=A3.device, dtype=torch.uint8)
            with torch.cuda.device(A3.device):
                check(self.lib.fbmm_min_bmm_x16(
                    self.stream_ptr(A3.device), a_keep.data_ptr(), lda, sa, b_keep.data_ptr(), ldb, sb,
                    dtype_code_x16(A3.dtype), values.data_ptr(), indices.data_ptr(), l, m, n, k, dim,
                    self._distance_code, ws.data_ptr(), ws_bytes))
            return (values[0], indices[0]) if two_d else (values, indices)
        a_keep, a_t, lda, sa = operand(A3)
        b_keep, b_t, ldb, sb = operand(B3)
        # own scratch (packed keys) plus, for large problems, room for pre-split lo planes
        ws_bytes = (self.lib.fbmm_min_bmm_workspace_bytes(l, m, n, k, dim, self._distance_code) + 255) // 256 * 256
        ws_bytes += self.lib.fbmm_presplit_workspace_bytes(l, m, n, k, dim, layout_letter(a_t, False), lda, sa,
                                                           layout_letter(b_t, True), ldb, sb)
        ws = torch.empty(max(ws_bytes, 256), device=A3.device, dtype=torch.uint8)
        with torch.cuda.device(A3.device):
            check(self.lib.fbmm_min_bmm_f32(
                self.stream_ptr(A3.device),
                a_keep.data_ptr(), layout_letter(a_t, False), lda, sa,
                b_keep.data_ptr(), layout_letter(b_t, True), ldb, sb,
                values.data_ptr(), indices.data_ptr(), l, m, n, k, dim, self._distance_code,
                ws.data_ptr(), ws_bytes))
        if two_d:
            return values[0], indices[0]
        return values, indices
