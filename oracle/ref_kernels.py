"""Launches the reference's own kernels, prebuilt by oracle/build_ref.py (TEST INFRASTRUCTURE ONLY).

The cubins under oracle/_ref/ are the reference's kernel text compiled as its wrappers
compile it; this module plays the part of CuPy's ``RawKernel.__call__`` with the CUDA driver
API: same grid, block and argument lists as the reference's launches (bmm.py:108-125,
mbmm.py:76-97, minbmm.py:116-143). Nothing in the shipped package imports it; the tests use it
to pin the CPU oracle and libfbmm.so to outputs of the reference itself.

Shapes: the reference's block-mask read runs one byte past a mask row for CTAs that start
exactly at the right edge (kernels/mbmm.cu:231-233,251), and its early-exit test lets such
CTAs through (kernels/bmm.cu:206); with m and n multiples of 512 (128 x the patch size of 4) no
such CTA exists, so the helpers below insist on that.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import build_ref

PATCH = 4


def available() -> bool:
    return build_ref.is_built()


_modules = {}


_cuda = None


def _driver():
    """libcuda through ctypes: cuModuleLoadData / cuModuleGetFunction / cuLaunchKernel."""
    global _cuda
    if _cuda is None:
        _cuda = ctypes.CDLL("libcuda.so.1")
        _cuda.cuModuleLoadData.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_char_p]
        _cuda.cuModuleGetFunction.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p, ctypes.c_char_p]
        _cuda.cuLaunchKernel.argtypes = [ctypes.c_void_p] + [ctypes.c_uint] * 6 + [ctypes.c_uint, ctypes.c_void_p,
                                                                                   ctypes.c_void_p, ctypes.c_void_p]
    return _cuda


def _check(err, what):
    if err != 0:
        raise RuntimeError(f"{what} failed with CUresult {err}")


def _function(cubin: str, name: str):
    drv = _driver()
    torch.zeros(1, device="cuda")  # makes torch's primary context current in this thread
    key = (cubin, torch.cuda.current_device())
    if key not in _modules:
        with open(os.path.join(build_ref.OUT_DIR, cubin), "rb") as f:
            image = f.read()
        mod = ctypes.c_void_p()
        _check(drv.cuModuleLoadData(ctypes.byref(mod), image), "cuModuleLoadData")
        _modules[key] = mod
    fn = ctypes.c_void_p()
    _check(drv.cuModuleGetFunction(ctypes.byref(fn), _modules[key], name.encode()), f"cuModuleGetFunction({name})")
    return fn


def _launch(fn, grid, args):
    """args: list of (ctypes type, value). Block is 256 threads as in the reference."""
    holders = [t(v) for t, v in args]
    ptrs = (ctypes.c_void_p * len(holders))(*[ctypes.addressof(h) for h in holders])
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    _check(_driver().cuLaunchKernel(fn, grid[0], grid[1], grid[2], 256, 1, 1, 0, stream, ptrs, None), "cuLaunchKernel")


def _grid(l, m, n):
    if m % (128 * PATCH) or n % (128 * PATCH):
        raise ValueError("reference kernels are only launched on m, n that are multiples of 512 here")
    gy = math.ceil(n / (128 * PATCH)) * math.ceil(m / (128 * PATCH))
    if gy > 65535:
        raise ValueError("the reference's grid overflows gridDim.y for this shape")
    return (PATCH * PATCH, gy, l)


def _stored(X: torch.Tensor, transposed: bool) -> torch.Tensor:
    """Contiguous storage of logical [l, r, c] as the 'n' ([l][r][c]) or 't' ([l][c][r]) kernels index it."""
    return X.transpose(1, 2).contiguous() if transposed else X.contiguous()


_P, _I = ctypes.c_void_p, ctypes.c_int


def bmm(A: torch.Tensor, B: torch.Tensor, mode: str = "nn") -> torch.Tensor:
    """bmm_{mode} of kernels/bmm.cu on logical A [l,m,k], B [l,k,n] (CUDA fp32); C pre-zeroed as bmm.py:106."""
    l, m, k = A.shape
    n = B.shape[2]
    a, b = _stored(A, mode[0] == "t"), _stored(B, mode[1] == "t")
    C = torch.zeros((l, m, n), device=A.device, dtype=torch.float32)
    _launch(_function("ref_bmm.cubin", f"bmm_{mode}"), _grid(l, m, n),
            [(_P, a.data_ptr()), (_P, b.data_ptr()), (_P, C.data_ptr()), (_I, m), (_I, n), (_I, k)])
    torch.cuda.synchronize()
    return C


def mbmm(A, B, block_mask, thread_mask, element_mask, share_mask=False) -> torch.Tensor:
    """mbmm_nn of kernels/mbmm.cu; C pre-zeroed as mbmm.py:74."""
    l, m, k = A.shape
    n = B.shape[2]
    a, b = A.contiguous(), B.contiguous()
    bm, tm, em = (t.contiguous() for t in (block_mask, thread_mask, element_mask))
    C = torch.zeros((l, m, n), device=A.device, dtype=torch.float32)
    cubin = "ref_mbmm_shared.cubin" if share_mask else "ref_mbmm.cubin"
    _launch(_function(cubin, "mbmm_nn"), _grid(l, m, n),
            [(_P, a.data_ptr()), (_P, b.data_ptr()), (_P, C.data_ptr()), (_P, bm.data_ptr()), (_P, tm.data_ptr()),
             (_P, em.data_ptr()), (_I, m), (_I, n), (_I, k)])
    torch.cuda.synchronize()
    return C


def min_bmm(A, B, dim: int, mode: str = "nn", distance: str = "inner"):
    """min_bmm_{mode} of kernels/minbmm.cu; values pre-filled with +inf as minbmm.py:116-122.
    Indices start at -1 (the reference leaves them uninitialised)."""
    l, m, k = A.shape
    n = B.shape[2]
    a, b = _stored(A, mode[0] == "t"), _stored(B, mode[1] == "t")
    rows = n if dim == 1 else m
    values = torch.full((l, rows), float("inf"), device=A.device, dtype=torch.float32)
    indices = torch.full((l, rows), -1, device=A.device, dtype=torch.int64)
    cubin = {"inner": "ref_minbmm_inner.cubin", "l2": "ref_minbmm_l2.cubin", "l1": "ref_minbmm_l1.cubin"}[distance]
    _launch(_function(cubin, f"min_bmm_{mode}"), _grid(l, m, n),
            [(_P, a.data_ptr()), (_P, b.data_ptr()), (_P, values.data_ptr()), (_P, indices.data_ptr()), (_I, m),
             (_I, n), (_I, k), (_I, dim)])
    torch.cuda.synchronize()
    return values, indices
