"""ctypes wrapper of oracle/fbmm_oracle.c (test infrastructure only)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def build() -> str:
    src = os.path.join(HERE, "fbmm_oracle.c")
    if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "liboracle.so"], check=True, capture_output=True)
    return LIB


def _lib():
    return ctypes.CDLL(build())


_DIST = {"inner": 0, "l2": 1, "euclidean": 1, "l1": 2, "manhattan": 2}


def _f(t):
    return np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.float32)


def _p(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def bmm(A, B):
    a, b = _f(A), _f(B)
    l, m, k = a.shape
    n = b.shape[2]
    c = np.empty((l, m, n), np.float32)
    _lib().oracle_bmm(_p(a), _p(b), _p(c), l, m, n, k)
    return torch.from_numpy(c)


def mbmm(A, B, block_mask, thread_mask, element_mask, share_mask=False):
    a, b = _f(A), _f(B)
    l, m, k = a.shape
    n = b.shape[2]
    bm, tm, em = (np.ascontiguousarray(t.cpu().numpy(), dtype=np.uint8) for t in (block_mask, thread_mask, element_mask))
    c = np.empty((l, m, n), np.float32)
    _lib().oracle_mbmm(_p(a), _p(b), _p(c), _p(bm), _p(tm), _p(em), int(share_mask), l, m, n, k)
    return torch.from_numpy(c)


def min_bmm(A, B, dim, distance="inner"):
    a, b = _f(A), _f(B)
    l, m, k = a.shape
    n = b.shape[2]
    r = m if dim == 2 else n
    v = np.empty((l, r), np.float32)
    i = np.empty((l, r), np.int64)
    _lib().oracle_min_bmm(_p(a), _p(b), _p(v), _p(i), l, m, n, k, dim, _DIST[distance])
    return torch.from_numpy(v), torch.from_numpy(i)


def topk_bmm(A, B, topk, dim, distance="inner"):
    a, b = _f(A), _f(B)
    l, m, k = a.shape
    n = b.shape[2]
    r = m if dim == 2 else n
    v = np.empty((l, r, topk), np.float32)
    i = np.empty((l, r, topk), np.int64)
    _lib().oracle_topk_bmm(_p(a), _p(b), _p(v), _p(i), l, m, n, k, topk, dim, _DIST[distance])
    return torch.from_numpy(v), torch.from_numpy(i)
