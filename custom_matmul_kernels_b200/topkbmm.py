"""Fused matmul + top-k (drop-in for topkbmm.py:7 TopkBMMCUDA)."""
from __future__ import annotations

import torch

from .custom_kernel import (FBMM_DIST_L1, CustomKernel, check, distance_code, dtype_code_x16, layout_letter, operand,
                            operand_x16)

_X16 = (torch.float16, torch.bfloat16)


class TopkBMMCUDA(CustomKernel):
    """``TopkBMMCUDA(patch_m, patch_n, distance)(A, B, k, dim) -> (values, indices)``.

    The k largest entries, descending, along `dim` of A [l,m,k] @ B [l,k,n], never
    writing the product out. k is always the LAST output axis: dim=1 gives [l,n,k], dim=2
    gives [l,m,k] (topkbmm.py:119-127) -- not torch.topk's layout for dim=1. 0 < k <= 128
    (topkbmm.py:104). Outputs are contiguous (the reference returns [:,:,:k] views of
    128-wide buffers, topkbmm.py:150-151). Any m and n are handled; where fewer than k
    entries exist the tail is -inf / -1. distance="l2" ranks the squared distances
    sum_k (A[m,k] - B[k,n])^2 (largest first, as the reference does, topkbmm.py:17-18),
    distance="l1" the sums sum_k |A[m,k] - B[k,n]| (topkbmm.py:19-20; fp32 tensors only: a SIMT
    kernel, the tensor cores cannot form |a - b|)."""

    def __init__(self, patch_m=4, patch_n=4, distance="inner"):
        super().__init__()
        self.patch_m = patch_m
        self.patch_n = patch_n
        self._distance_code = distance_code(distance)
        self.distance = distance

    def __call__(self, A, B, k=128, dim=1, index_offset=0):
        A3, B3, two_d = self.check_inputs(A, B, (torch.float32,) + _X16)
        if two_d:
            dim += 1
        if dim not in (1, 2):
            raise ValueError("dim must be 1 or 2 on the 3-D product (0 or 1 for 2-D inputs)")
        if not 0 < k <= 128:
            raise ValueError("k must be in 1..128")
        l, m, d = A3.shape
        n = B3.shape[2]
        if min(l, m, n, d) <= 0:
            raise ValueError(f"empty problem: l={l} m={m} n={n} k={d}")
        rows = n if dim == 1 else m
        values = torch.empty((l, rows, k), device=A3.device, dtype=torch.float32)
        indices = torch.empty((l, rows, k), device=A3.device, dtype=torch.int64)
        if A3.dtype in _X16:
            if self._distance_code == FBMM_DIST_L1:
                raise NotImplementedError("distance='l1' takes fp32 tensors only")
            # fp16 / bf16 go to the tensor cores as they are; values come back in fp32
            a_keep, lda, sa = operand_x16(A3)
            b_keep, ldb, sb = operand_x16(B3.transpose(1, 2))
            with torch.cuda.device(A3.device):
                ws_bytes = (self.lib.fbmm_topk_bmm_workspace_bytes(l, m, n, d, k, dim, self._distance_code)
                            + 255) // 256 * 256
                ws = torch.empty(max(ws_bytes, 256), device=A3.device, dtype=torch.uint8)
                check(self.lib.fbmm_topk_bmm_x16(
                    self.stream_ptr(A3.device), a_keep.data_ptr(), lda, sa, b_keep.data_ptr(), ldb, sb,
                    dtype_code_x16(A3.dtype), values.data_ptr(), indices.data_ptr(), l, m, n, d, k, dim,
                    self._distance_code, index_offset, ws.data_ptr(), ws_bytes))
            return (values[0], indices[0]) if two_d else (values, indices)
        a_keep, a_t, lda, sa = operand(A3)
        b_keep, b_t, ldb, sb = operand(B3)
        with torch.cuda.device(A3.device):
            # own scratch (per-chunk lists) plus, for large problems, room for pre-split lo planes
            ws_bytes = (self.lib.fbmm_topk_bmm_workspace_bytes(l, m, n, d, k, dim, self._distance_code) + 255) // 256 * 256
            ws_bytes += self.lib.fbmm_presplit_workspace_bytes(l, m, n, d, dim, layout_letter(a_t, False), lda, sa,
                                                               layout_letter(b_t, True), ldb, sb)
            ws = torch.empty(max(ws_bytes, 256), device=A3.device, dtype=torch.uint8)
            check(self.lib.fbmm_topk_bmm_f32(
                self.stream_ptr(A3.device),
                a_keep.data_ptr(), layout_letter(a_t, False), lda, sa,
                b_keep.data_ptr(), layout_letter(b_t, True), ldb, sb,
                values.data_ptr(), indices.data_ptr(), l, m, n, d, k, dim, self._distance_code, index_offset,
                ws.data_ptr(), ws_bytes))
        if two_d:
            return values[0], indices[0]
        return values, indices

    def packed(self, A, B, k=128, dim=1):
        """The same top-k in wire format: one int64 per entry whose low half holds the fp32
        value's bits and whose high half holds the int32 index (-1 = empty), indices being
        plain positions along `dim` of THIS call's operands. A rank that owns a column shard
        of B hands this tensor to one all-gather as it is (sharding.topk_bmm_column_sharded);
        sharding.unpack_candidates splits it again. fp32 operands only. Shape [l, rows, k]
        ([rows, k] for 2-D inputs)."""
        A3, B3, two_d = self.check_inputs(A, B, (torch.float32,))
        if two_d:
            dim += 1
        if dim not in (1, 2):
            raise ValueError("dim must be 1 or 2 on the 3-D product (0 or 1 for 2-D inputs)")
        if not 0 < k <= 128:
            raise ValueError("k must be in 1..128")
        l, m, d = A3.shape
        n = B3.shape[2]
        if min(l, m, n, d) <= 0:
            raise ValueError(f"empty problem: l={l} m={m} n={n} k={d}")
        rows = n if dim == 1 else m
        out = torch.empty((l, rows, k), device=A3.device, dtype=torch.int64)
        a_keep, a_t, lda, sa = operand(A3)
        b_keep, b_t, ldb, sb = operand(B3)
        with torch.cuda.device(A3.device):
            ws_bytes = (self.lib.fbmm_topk_bmm_workspace_bytes(l, m, n, d, k, dim, self._distance_code) + 255) // 256 * 256
            ws_bytes += self.lib.fbmm_presplit_workspace_bytes(l, m, n, d, dim, layout_letter(a_t, False), lda, sa,
                                                               layout_letter(b_t, True), ldb, sb)
            ws = torch.empty(max(ws_bytes, 256), device=A3.device, dtype=torch.uint8)
            check(self.lib.fbmm_topk_bmm_packed_f32(
                self.stream_ptr(A3.device),
                a_keep.data_ptr(), layout_letter(a_t, False), lda, sa,
                b_keep.data_ptr(), layout_letter(b_t, True), ldb, sb,
                out.data_ptr(), l, m, n, d, k, dim, self._distance_code, ws.data_ptr(), ws_bytes))
        return out[0] if two_d else out
