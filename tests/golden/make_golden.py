"""Generates the golden fixtures in this folder from the CPU oracle.

    python tests/golden/make_golden.py

The reference (DeMoriarty/custom_matmul_kernels) ships no known-answer vectors and its
kernels need CuPy + a GPU, so these fixtures come from the reference's own TEST
EXPRESSIONS (torch on CPU, restated in oracle/ref_semantics.py). Two kinds:

* exact_*  small-integer operands: every product and partial sum is exactly representable
           in fp32 (and in tf32 pieces), so values are bit-exact for ANY correct
           implementation and planted ties pin the lowest-index rule of min.
* randn_*  seeded normal operands with the oracle's fp32 answers, compared within
           rel 1e-5 / abs 1e-4.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import ref_semantics as R  # noqa: E402


def save(name, **arrays):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **arrays)
    print(f"{name}: {os.path.getsize(path)} bytes")


def main():
    torch.manual_seed(0)
    # ---- exact bmm, odd shape (no multiple of 128 / 32 / 4 anywhere)
    A, B = R.exact_inputs(2, 45, 19, 53, seed=11)
    save("exact_bmm", A=A.numpy().astype(np.int8), B=B.numpy().astype(np.int8),
         C=R.bmm(A, B).numpy().astype(np.int32))

    # ---- exact min with planted ties: duplicate columns of B (dim=2 ties) and duplicate
    # rows of A (dim=1 ties); answers must name the LOWEST index.
    A, B = R.exact_inputs(2, 150, 16, 300, seed=12, lo=-3, hi=3)
    B[:, :, 200:300] = B[:, :, 0:100]      # columns 200.. repeat columns 0..
    B[:, :, 129] = B[:, :, 127]            # a tie across the 128-column tile edge
    A[:, 140:150] = A[:, 0:10]
    v2, i2 = R.min_bmm(A, B, dim=2)
    v1, i1 = R.min_bmm(A, B, dim=1)
    save("exact_min", A=A.numpy().astype(np.int8), B=B.numpy().astype(np.int8),
         v_dim2=v2.numpy().astype(np.int32), i_dim2=i2.numpy(), v_dim1=v1.numpy().astype(np.int32), i_dim1=i1.numpy())

    # ---- exact top-k (values pinned exactly; indices checked for consistency by the tests)
    A, B = R.exact_inputs(1, 70, 24, 520, seed=13)
    v2, i2 = R.topk_bmm(A, B, k=20, dim=2)
    v1, i1 = R.topk_bmm(A, B, k=20, dim=1)
    save("exact_topk", A=A.numpy().astype(np.int8), B=B.numpy().astype(np.int8), k=np.int32(20),
         v_dim2=v2.numpy().astype(np.int32), v_dim1=v1.numpy().astype(np.int32))

    # ---- exact top-k with fewer candidates than k (tail must be -inf / -1)
    A, B = R.exact_inputs(1, 9, 8, 5, seed=14)
    v2, i2 = R.topk_bmm(A, B, k=8, dim=2)
    save("exact_topk_short", A=A.numpy().astype(np.int8), B=B.numpy().astype(np.int8), k=np.int32(8),
         v_dim2=v2.numpy(), i_dim2=i2.numpy())

    # ---- exact masked bmm: m = n = 264 gives 3x3 block tiles with ragged edges. Tiles:
    # (0,0) causal, (0,1) all masked, (0,2) all kept, (1,0) one element kept,
    # (1,1) random, (1,2) masked, (2,*) random / kept / masked.
    l, m, k, n = 2, 264, 12, 264
    A, B = R.exact_inputs(l, m, k, n, seed=15, lo=-4, hi=4)
    g = torch.Generator().manual_seed(16)
    mask = torch.zeros(l, m, n, dtype=torch.bool)
    mask[:, :128, :128] = torch.tril(torch.ones(128, 128, dtype=torch.bool))
    mask[:, :128, 256:] = True
    mask[:, 200, 77] = True
    mask[:, 128:256, 128:256] = torch.rand(l, 128, 128, generator=g) < 0.3
    mask[:, 256:, :128] = torch.rand(l, 8, 128, generator=g) < 0.5
    mask[:, 256:, 128:256] = True
    bm, tm, em = R.make_masks(mask)
    C = R.mbmm(A, B, bm, tm, em)
    assert torch.equal(C, torch.bmm(A, B).masked_fill_(~mask, 0))  # colab/test_mbmm.ipynb:1342-1343
    save("exact_mbmm", A=A.numpy().astype(np.int8), B=B.numpy().astype(np.int8),
         mask=np.packbits(mask.numpy(), axis=-1), C=C.numpy().astype(np.int16))

    # ---- seeded normal operands, fp32 oracle answers
    g = torch.Generator().manual_seed(21)
    A = torch.randn(2, 60, 40, generator=g)
    B = torch.randn(2, 40, 72, generator=g)
    v2, i2 = R.min_bmm(A, B, dim=2)
    v1, i1 = R.min_bmm(A, B, dim=1)
    t2v, t2i = R.topk_bmm(A, B, k=7, dim=2)
    t1v, t1i = R.topk_bmm(A, B, k=7, dim=1)
    save("randn_small", A=A.numpy(), B=B.numpy(), C=R.bmm(A, B).numpy(), min_v2=v2.numpy(), min_i2=i2.numpy(),
         min_v1=v1.numpy(), min_i1=i1.numpy(), topk_v2=t2v.numpy(), topk_i2=t2i.numpy(), topk_v1=t1v.numpy(),
         topk_i1=t1i.numpy(), k=np.int32(7))


if __name__ == "__main__":
    main()
