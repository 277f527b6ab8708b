"""fbmm_min_bmm_f32_noalloc: min_bmm for hosts that may not allocate.

A caller that embeds libfbmm.so through the C ABI in a loop with a frozen memory budget (or
a plugin host that gets nothing but input and output buffers) cannot hand over a workspace
and cannot call cudaMalloc. This entry point keeps its scratch in a device array inside
the library. The test calls it through the C ABI twice in a row, with different operands,
and requires the same bits as the workspace-taking entry point each time: the second call
proves that keys left behind by the first one are cleared. It lives in a file of its own,
collected last, so that a run stopping at the first failure has already run everything
else."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_pair(lib, A, B, dim):
    """(values, indices) from the no-alloc entry point and from fbmm_min_bmm_f32."""
    l, m, k = A.shape
    n = B.shape[2]
    rows = m if dim == 2 else n
    stream = torch.cuda.current_stream().cuda_stream
    out = []
    for noalloc in (True, False):
        v = torch.full((l, rows), float("nan"), device=A.device)
        i = torch.full((l, rows), -7, device=A.device, dtype=torch.int64)
        common = (stream, A.data_ptr(), ord("n"), k, m * k, B.data_ptr(), ord("n"), n, k * n, v.data_ptr(),
                  i.data_ptr(), l, m, n, k, dim)
        if noalloc:
            rc = lib.fbmm_min_bmm_f32_noalloc(*common)
        else:
            nbytes = lib.fbmm_min_bmm_workspace_bytes(l, m, n, k, dim, 0)
            ws = torch.empty(nbytes, device=A.device, dtype=torch.uint8)
            rc = lib.fbmm_min_bmm_f32(*common, 0, ws.data_ptr(), nbytes)
        assert rc == 0, lib.fbmm_last_error()
        out.append((v, i))
    torch.cuda.synchronize()
    return out


def test_noalloc_matches_workspace_entry_point_twice_in_a_row(dev, lib):
    from oracle import ref_semantics as R
    g = torch.Generator().manual_seed(77)
    # first call: many rows, large values
    A1 = (torch.randn(2, 700, 96, generator=g) * 3).to(dev)
    B1 = torch.randn(2, 96, 1500, generator=g).to(dev)
    (v_na, i_na), (v_ws, i_ws) = _call_pair(lib, A1, B1, 2)
    assert torch.equal(v_na, v_ws) and torch.equal(i_na, i_ws)
    R.check_min(v_na, i_na, A1.cpu(), B1.cpu(), 2)
    # second call right after: fewer rows, every product far ABOVE the first call's minima,
    # so a key left over from call one would win the atomicMin if it were not cleared
    A2 = (torch.rand(1, 300, 64, generator=g) + 1).to(dev)
    B2 = (torch.rand(1, 64, 900, generator=g) + 1).to(dev)
    for dim in (2, 1):
        (v_na, i_na), (v_ws, i_ws) = _call_pair(lib, A2, B2, dim)
        assert torch.equal(v_na, v_ws) and torch.equal(i_na, i_ws)
        assert float(v_na.min()) > 0
        R.check_min(v_na, i_na, A2.cpu(), B2.cpu(), dim)
    assert lib.fbmm_check(None) == 0, lib.fbmm_last_error()


def test_noalloc_rejects_more_rows_than_its_array_holds(dev, lib):
    from custom_matmul_kernels_b200 import custom_kernel as ck
    A = torch.zeros(1, 128, 32, device=dev)
    B = torch.zeros(1, 32, 128, device=dev)
    v = torch.empty(8, device=dev)
    i = torch.empty(8, device=dev, dtype=torch.int64)
    # 262145 rows declared: rejected from the sizes alone, before anything is launched
    rc = lib.fbmm_min_bmm_f32_noalloc(None, A.data_ptr(), ord("n"), 32, 0, B.data_ptr(), ord("n"), 128, 0,
                                      v.data_ptr(), i.data_ptr(), 1, 262145, 128, 32, 2)
    assert rc == ck.FBMM_ERR_WORKSPACE
    assert b"262144" in lib.fbmm_last_error()
