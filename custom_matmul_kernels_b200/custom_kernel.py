"""ctypes loader for libfbmm.so.

Takes the place of the reference's ``custom_kernel.py`` (custom_kernel.py:12-43), whose
``CustomKernel`` base class wired CuPy to torch's allocator and captured a stream once.
Here the base class hands its subclasses the C-ABI library and the stream that is current
at call time; there is no JIT step and no CPU fallback: if the library is not built the
import of an op fails loudly.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfbmm.so")

FBMM_OK = 0
FBMM_ERR_INVALID = -1
FBMM_ERR_ALIGN = -2
FBMM_ERR_WORKSPACE = -3
FBMM_ERR_CUDA = -4
FBMM_ERR_DEVICE = -5
FBMM_ERR_UNSUPPORTED = -6
FBMM_ERR_PEER = -7
FBMM_ERR_COMM = -8
FBMM_DIST_INNER = 0
FBMM_DIST_L2 = 1
FBMM_DIST_L1 = 2


def distance_code(distance: str) -> int:
    """The reference's `distance` strings (minbmm.py:12-19). inner and l2 run on the tensor
    cores; l1 has no matrix-product form and runs as a SIMT kernel (fp32 operands only);
    anything else is an error (the reference builds that ValueError but never raises it,
    minbmm.py:19)."""
    if distance == "inner":
        return FBMM_DIST_INNER
    if distance in ("l2", "euclidean"):
        return FBMM_DIST_L2
    if distance in ("l1", "manhattan"):
        return FBMM_DIST_L1
    raise ValueError("Unrecognized distance type")

_c_ll = ctypes.c_longlong
_c_int = ctypes.c_int
_c_ptr = ctypes.c_void_p
_c_size = ctypes.c_size_t

_OPERANDS = [_c_ptr, _c_int, _c_ll, _c_ll, _c_ptr, _c_int, _c_ll, _c_ll]  # A.., B..

# name -> (restype, argtypes); every symbol include/fbmm.h declares
SIGNATURES = {
    "fbmm_version": (_c_int, []),
    "fbmm_last_error": (ctypes.c_char_p, []),
    "fbmm_check": (_c_int, [_c_ptr]),
    "fbmm_bmm_f32": (_c_int, [_c_ptr] + _OPERANDS + [_c_ptr, _c_ll, _c_ll, _c_int, _c_int, _c_int, _c_int]),
    "fbmm_mbmm_f32": (_c_int, [_c_ptr] + _OPERANDS + [_c_ptr, _c_ll, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                                      _c_int, _c_int, _c_int, _c_int]),
    "fbmm_mbmm_softmax_f32": (_c_int, [_c_ptr] + _OPERANDS + [_c_ptr, _c_ll, _c_ll, _c_ptr, _c_ptr, _c_ptr, _c_int,
                                                              ctypes.c_float, _c_int, _c_int, _c_int, _c_int]),
    "fbmm_min_bmm_workspace_bytes": (_c_size, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int]),
    "fbmm_min_bmm_f32": (_c_int, [_c_ptr] + _OPERANDS + [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                         _c_int, _c_ptr, _c_size]),
    "fbmm_min_bmm_f32_noalloc": (_c_int, [_c_ptr] + _OPERANDS + [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int,
                                                                 _c_int]),
    "fbmm_presplit_workspace_bytes": (_c_size, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ll, _c_int,
                                                _c_ll, _c_ll]),
    "fbmm_topk_bmm_workspace_bytes": (_c_size, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int]),
    "fbmm_topk_bmm_f32": (_c_int, [_c_ptr] + _OPERANDS + [_c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                          _c_int, _c_int, _c_ll, _c_ptr, _c_size]),
    "fbmm_topk_merge_f32": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_ptr, _c_ptr]),
    "fbmm_topk_bmm_packed_f32": (_c_int, [_c_ptr] + _OPERANDS + [_c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                                                                 _c_int, _c_ptr, _c_size]),
    "fbmm_topk_merge_packed_f32": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_ll, _c_int, _c_ll, _c_ptr, _c_ptr]),
    "fbmm_comm_get_unique_id": (_c_int, [_c_ptr]),
    "fbmm_comm_init_rank": (_c_int, [ctypes.POINTER(_c_ptr), _c_int, _c_int, _c_ptr]),
    "fbmm_comm_destroy": (_c_int, [_c_ptr]),
    "fbmm_topk_bmm_sharded_workspace_bytes": (_c_size, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll,
                                                        _c_int, _c_ll]),
    "fbmm_topk_bmm_sharded_f32": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_int, _c_ptr, _c_int, _c_ll, _c_ptr, _c_int, _c_ll,
                                           _c_ll, _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr,
                                           _c_size]),
    "fbmm_selftest_wait_expiry": (_c_int, [_c_ptr]),
    "fbmm_bmm_x16": (_c_int, [_c_ptr, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_ll, _c_int, _c_ptr, _c_ll, _c_ll, _c_int,
                              _c_int, _c_int, _c_int]),
    "fbmm_mbmm_x16": (_c_int, [_c_ptr, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_ll, _c_int, _c_ptr, _c_ll, _c_ll, _c_ptr,
                               _c_ptr, _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int]),
    "fbmm_min_bmm_x16": (_c_int, [_c_ptr, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_ll, _c_int, _c_ptr, _c_ptr, _c_int,
                                  _c_int, _c_int, _c_int, _c_int, _c_int, _c_ptr, _c_size]),
    "fbmm_topk_bmm_x16": (_c_int, [_c_ptr, _c_ptr, _c_ll, _c_ll, _c_ptr, _c_ll, _c_ll, _c_int, _c_ptr, _c_ptr, _c_int,
                                   _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_ll, _c_ptr, _c_size]),
    "fbmm_kmeans_update_workspace_bytes": (_c_size, [_c_int, _c_int]),
    "fbmm_kmeans_update_f32": (_c_int, [_c_ptr, _c_ptr, _c_ll, _c_ptr, _c_ll, _c_int, _c_int, _c_ptr, _c_ll, _c_ptr,
                                        _c_ptr, _c_size]),
}

_lib = None
_lock = threading.Lock()


def load_library() -> ctypes.CDLL:
    """Loads libfbmm.so once and declares every entry point's signature."""
    global _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise ImportError(
                    f"{LIB_PATH} is missing: build it with `python -m custom_matmul_kernels_b200.build` "
                    "(needs nvcc). There is no fallback path.")
            lib = ctypes.CDLL(LIB_PATH)
            for name, (restype, argtypes) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype = restype
                fn.argtypes = argtypes
            _lib = lib
    return _lib


class FbmmError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"libfbmm error {code}: {message}")
        self.code = code


def check(rc: int) -> None:
    """Turns a negative status into the exception the reference's asserts would raise."""
    if rc == FBMM_OK:
        return
    msg = load_library().fbmm_last_error().decode()
    if rc in (FBMM_ERR_INVALID, FBMM_ERR_ALIGN):
        raise ValueError(f"libfbmm error {rc}: {msg}")
    raise FbmmError(rc, msg)


def operand(X: torch.Tensor):
    """Describes a [l, r, c] fp32 CUDA tensor to the C ABI.

    Returns (tensor_to_keep_alive, transposed, pitch, batch_stride): `transposed` is True
    when the storage runs along r (the reference's "t" stride layout, bmm.py:56-66).
    Storage the TMA engine cannot address (unaligned base, pitch or batch stride not a
    multiple of 4 elements, neither of the last two strides equal to 1) is repacked into a
    row-major buffer whose pitch is rounded up to 4 elements. A batch stride of 0 (one matrix
    expanded over the batch axis) is passed through as it is: the library reads the one
    matrix for every batch."""
    l, r, c = X.shape
    sl, sr, sc = X.stride()

    def addressable(ld, inner):
        return (X.data_ptr() % 16 == 0 and ld % 4 == 0 and ld >= inner
                and (l == 1 or (sl % 4 == 0 and sl >= 0)))

    if sc == 1 and addressable(sr, c):
        return X, False, sr, sl
    if sr == 1 and addressable(sc, r):
        return X, True, sc, sl
    cp = (c + 3) // 4 * 4
    buf = torch.zeros((l, r, cp), dtype=X.dtype, device=X.device) if cp != c else torch.empty_like(
        X, memory_format=torch.contiguous_format)
    buf[:, :, :c] = X
    return buf, False, cp, r * cp


FBMM_F16, FBMM_BF16 = 1, 2


def dtype_code_x16(dtype: torch.dtype) -> int:
    return FBMM_F16 if dtype == torch.float16 else FBMM_BF16


def operand_x16(X: torch.Tensor):
    """Describes a 16-bit [l, r, k] CUDA tensor to the *_x16 entry points, which take
    k-contiguous storage only. Returns (tensor_to_keep_alive, pitch, batch_stride) in
    elements. Anything else (k not contiguous, pitch or batch stride not a multiple of 8
    elements, unaligned base) is copied into a row-major buffer with the pitch rounded up
    to 8 elements."""
    l, r, k = X.shape
    sl, sr, sk = X.stride()
    if (sk == 1 and X.data_ptr() % 16 == 0 and sr % 8 == 0 and sr >= k
            and (l == 1 or (sl % 8 == 0 and sl > 0))):
        return X, sr, sl
    kp = (k + 7) // 8 * 8
    buf = torch.zeros((l, r, kp), dtype=X.dtype, device=X.device) if kp != k else torch.empty(
        (l, r, k), dtype=X.dtype, device=X.device)
    buf[:, :, :k] = X
    return buf, kp, r * kp


def layout_letter(transposed: bool, is_b: bool) -> int:
    """'n'/'t' as the reference kernel suffixes use them: a row-major [m,k] A is 'n', a
    row-major [k,n] B is 'n' (bmm.py:56-66)."""
    return ord("t") if transposed else ord("n")


class CustomKernel:
    """Base of the four op wrappers (same name and role as custom_kernel.py:12)."""

    def __init__(self):
        self.lib = load_library()

    def get_mode(self, A, B):
        """Stride layout of the last two dims of A and B, 'n' or 't' each, as the reference's
        wrappers detect it (bmm.py:56-66); '?' where neither stride is 1."""
        mode = [None, None]
        for i, X in enumerate((A, B)):
            if X.stride()[-1] == 1:
                mode[i] = "n"
            elif X.stride()[-2] == 1:
                mode[i] = "t"
        return "".join(m or "?" for m in mode)

    @staticmethod
    def stream_ptr(device: torch.device) -> int:
        # The reference captured the stream once at construction (custom_kernel.py:15);
        # the stream current at call time is what callers of torch ops expect.
        return torch.cuda.current_stream(device).cuda_stream

    @staticmethod
    def check_inputs(A: torch.Tensor, B: torch.Tensor, dtypes=(torch.float32,)):
        """Shared argument checks of the wrappers (bmm.py:75-90, minbmm.py:84-99)."""
        if A.dim() != B.dim():
            raise ValueError("A and B need the same number of dimensions")
        if A.dim() == 2:
            A3, B3, two_d = A[None], B[None], True
        elif A.dim() == 3:
            A3, B3, two_d = A, B, False
        else:
            raise ValueError("A and B need to be 2d or 3d")
        if A3.shape[0] != B3.shape[0]:
            raise ValueError(f"batch sizes differ: {A3.shape[0]} vs {B3.shape[0]}")
        if A3.shape[2] != B3.shape[1]:
            raise ValueError(f"inner dimensions differ: A {tuple(A3.shape)} B {tuple(B3.shape)}")
        if A3.dtype != B3.dtype:
            raise TypeError("A and B need the same dtype")
        if A3.dtype not in dtypes:
            raise TypeError(f"dtype {A3.dtype} is not implemented for this op (the reference kernels take float* "
                            f"only); accepted: {', '.join(str(d) for d in dtypes)}")
        if A3.device.type != "cuda" or B3.device.type != "cuda":
            raise ValueError("A and B must be CUDA tensors")
        if A3.device != B3.device:
            raise ValueError("A and B must be on the same device")
        return A3, B3, two_d
