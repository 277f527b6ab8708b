"""B200-native fused fp32 batched matmul: bmm, masked bmm, min/argmin bmm, top-k bmm.

The four callable classes keep the names and call signatures of the reference's
``bmm.py``, ``mbmm.py``, ``minbmm.py`` and ``topkbmm.py``; the work is done by hand-written
sm_100a kernels in ``libfbmm.so`` (see ``include/fbmm.h`` for the C ABI).
"""
from .bmm import BMMCUDA
from .mbmm import MBMMCUDA, MBMMSoftmaxCUDA, make_masks
from .minbmm import MinBMMCUDA
from .topkbmm import TopkBMMCUDA
from .kmeans import KMeansCUDA

__all__ = ["BMMCUDA", "MBMMCUDA", "MBMMSoftmaxCUDA", "MinBMMCUDA", "TopkBMMCUDA", "KMeansCUDA", "make_masks"]
