"""k-means on top of the fused min_bmm: the caller-side loop the reference's min_bmm was
written for (its README motivates `MinBMMCUDA` with nearest-centroid search), with the
distance matrix never written to memory.

One iteration is two library calls: `MinBMMCUDA(distance="l2")` assigns every point to
its nearest centroid (squared distances on the tensor cores, argmin in the epilogue), and
`fbmm_kmeans_update_f32` moves every centroid to the mean of its points.
"""
from __future__ import annotations

import torch

from .custom_kernel import CustomKernel, check
from .minbmm import MinBMMCUDA


class KMeansCUDA(CustomKernel):
    """``KMeansCUDA().fit(X, centroids, iters) -> (centroids, assignment, distances)``.

    X is [n, d] fp32, centroids [k, d] fp32 (the starting positions; not modified).
    `assign` and `update` are the two halves of an iteration and can be called on their
    own. A centroid that no point chose stays where it is."""

    def __init__(self):
        super().__init__()
        self._min = MinBMMCUDA(distance="l2")

    def assign(self, X: torch.Tensor, centroids: torch.Tensor):
        """Nearest centroid of every point: (squared distances [n] fp32, indices [n] int64)."""
        self._check(X, centroids)
        # rows of X against columns of centroids^T: the transposed view is the 't' layout
        dist, idx = self._min(X, centroids.t(), dim=1)
        return dist, idx

    def update(self, X: torch.Tensor, assignment: torch.Tensor, centroids: torch.Tensor):
        """New centroids [k, d] (a fresh tensor) and cluster sizes [k] fp32."""
        self._check(X, centroids)
        n, d = X.shape
        k = centroids.shape[0]
        if assignment.shape != (n,) or assignment.dtype != torch.int64 or assignment.device != X.device:
            raise ValueError("assignment must be an int64 tensor of shape [n] on X's device")
        Xc = X if X.stride(1) == 1 else X.contiguous()
        assignment = assignment.contiguous()
        out = centroids.contiguous().clone()
        counts = torch.empty(k, device=X.device, dtype=torch.float32)
        ws_bytes = self.lib.fbmm_kmeans_update_workspace_bytes(k, d)
        ws = torch.empty(ws_bytes, device=X.device, dtype=torch.uint8)
        with torch.cuda.device(X.device):
            check(self.lib.fbmm_kmeans_update_f32(
                self.stream_ptr(X.device), Xc.data_ptr(), Xc.stride(0), assignment.data_ptr(), n, d, k,
                out.data_ptr(), out.stride(0), counts.data_ptr(), ws.data_ptr(), ws_bytes))
        return out, counts

    def fit(self, X: torch.Tensor, centroids: torch.Tensor, iters: int = 10):
        """`iters` rounds of assign + update, then a last assignment against the final
        centroids."""
        c = centroids
        for _ in range(iters):
            _, idx = self.assign(X, c)
            c, _ = self.update(X, idx, c)
        dist, idx = self.assign(X, c)
        return c, idx, dist

    @staticmethod
    def _check(X, centroids):
        if X.dim() != 2 or centroids.dim() != 2 or X.shape[1] != centroids.shape[1]:
            raise ValueError("X must be [n, d] and centroids [k, d]")
        if X.dtype != torch.float32 or centroids.dtype != torch.float32:
            raise TypeError("X and centroids must be float32")
        if X.device.type != "cuda" or centroids.device != X.device:
            raise ValueError("X and centroids must be CUDA tensors on one device")
