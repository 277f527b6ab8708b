"""Compiles the reference's own CUDA kernels into oracle/_ref/ (TEST INFRASTRUCTURE ONLY).

    python -m oracle.build_ref [reference_root]        (default: the REFERENCE_ROOT
                                                        environment variable)

The reference (DeMoriarty/custom_matmul_kernels) has no build system: its wrappers read
kernel text, substitute placeholders and hand the result to CuPy's RawKernel with
``backend='nvcc'`` (bmm.py:13-54, mbmm.py:18-50, minbmm.py:23-64). This script does the same
three steps without CuPy, from the sources where they lie:

* text = kernels/bmm_helpers.cu + kernels/{bmm,minbmm}.cu, or kernels/mbmm.cu on its own
  (bmm.py:13-17, minbmm.py:23-27; mbmm.cu carries its own helper copies);
* ``_PM_``/``_PN_`` -> 4 (the wrappers' default patch size), ``__DISTANCE_FN__`` ->
  madd / squared_l2 / l1 (bmm.py:19-23, minbmm.py:12-19,29-33), ``__MASK_BID__`` -> bid or 0
  (mbmm.py:24);
* nvcc with the wrappers' options ``--maxrregcount=128 --use_fast_math`` (bmm.py:29), to a
  cubin for sm_100.

Only the cubins are written, into oracle/_ref/ (git-ignored; they travel to the GPU box like
any other built file). The substituted text lives in a temporary directory outside the
repository and is deleted; no reference source is copied into the tree.
kernels/topkbmm.cu and kernels/bitonic_sort.cu are left out on purpose: they take a global
spin mutex (kernels/topkbmm.cu:13-47), which is not something to run on a shared GPU.

tests/test_gpu_reference_kernels.py launches these cubins through the CUDA driver API and
compares them with the CPU oracle and with libfbmm.so.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")

# cubin name -> (kernel files concatenated in this order, placeholder substitutions)
VARIANTS = {
    "ref_bmm.cubin": (("bmm_helpers.cu", "bmm.cu"), {"__DISTANCE_FN__": "madd"}),
    "ref_minbmm_inner.cubin": (("bmm_helpers.cu", "minbmm.cu"), {"__DISTANCE_FN__": "madd"}),
    "ref_minbmm_l2.cubin": (("bmm_helpers.cu", "minbmm.cu"), {"__DISTANCE_FN__": "squared_l2"}),
    "ref_minbmm_l1.cubin": (("bmm_helpers.cu", "minbmm.cu"), {"__DISTANCE_FN__": "l1"}),
    "ref_mbmm.cubin": (("mbmm.cu",), {"__MASK_BID__": "bid"}),
    "ref_mbmm_shared.cubin": (("mbmm.cu",), {"__MASK_BID__": "0"}),
}
PATCH = {"_PM_": "4", "_PN_": "4"}
NVCC_FLAGS = ["-cubin", "-arch=sm_100", "--maxrregcount=128", "--use_fast_math", "-w"]


def reference_root(argv=None) -> str | None:
    argv = [a for a in (sys.argv[1:] if argv is None else argv) if not a.startswith("--")]
    root = argv[0] if argv else os.environ.get("REFERENCE_ROOT")
    if root and os.path.isdir(os.path.join(root, "kernels")):
        return root
    return None


def is_built() -> bool:
    return all(os.path.exists(os.path.join(OUT_DIR, name)) for name in VARIANTS)


def build(root: str | None = None, force: bool = False) -> bool:
    """Builds every cubin that is missing (all of them with `force`). Returns False, and
    leaves what is there untouched, when the reference tree or nvcc is not available."""
    root = root or reference_root([])
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if root is None or not os.path.exists(nvcc):
        return False
    os.makedirs(OUT_DIR, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="fbmm_ref_") as tmp:
        for name, (files, subs) in VARIANTS.items():
            out = os.path.join(OUT_DIR, name)
            if os.path.exists(out) and not force:
                continue
            text = ""
            for f in files:
                with open(os.path.join(root, "kernels", f)) as fh:
                    text += fh.read()
            for key, val in {**PATCH, **subs}.items():
                text = text.replace(key, val)
            src = os.path.join(tmp, name.replace(".cubin", ".cu"))
            with open(src, "w") as fh:
                fh.write(text)
            proc = subprocess.run([nvcc] + NVCC_FLAGS + ["-o", out, src], capture_output=True, text=True)
            if proc.returncode != 0:
                raise RuntimeError(f"nvcc failed on the reference's {'+'.join(files)}:\n{proc.stderr}")
    return True


if __name__ == "__main__":
    ok = build(reference_root(), force="--force" in sys.argv)
    print("built" if ok else "reference tree or nvcc not found; nothing built", OUT_DIR)
