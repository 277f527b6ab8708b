"""Two-GPU tests of the column-sharded top-k over real NCCL (skipped on a one-GPU box):
the Python path (TopkBMMCUDA.packed -> one all_gather_into_tensor -> packed merge), the C-ABI
path (fbmm_comm_init_rank + fbmm_topk_bmm_sharded_f32, NCCL reached through dlopen), and the
agreement step that keeps a rank from entering the all-gather when a peer's local step
failed. The failing rank fails on the host, before it launches anything (a misaligned
operand is rejected by argument validation); no rank exits with work in flight."""
import os
import socket
from datetime import timedelta

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev, timeout=timedelta(seconds=120))
    problems = []

    def expect(cond, what):
        # collected, not raised: every rank walks through every collective whatever it finds
        if not cond:
            problems.append(what)

    try:
        import ctypes
        from custom_matmul_kernels_b200 import TopkBMMCUDA
        from custom_matmul_kernels_b200 import custom_kernel as ck
        from custom_matmul_kernels_b200 import sharding as S
        from oracle import ref_semantics as R
        lib = ck.load_library()
        op = TopkBMMCUDA()
        g = torch.Generator().manual_seed(21)
        m, k, n, kk = 4096, 64, 20000, 64       # 20000 columns: the last rank's shard is ragged
        A = torch.randn(1, m, k, generator=g).to(dev)
        B = torch.randn(1, k, n, generator=g).to(dev)
        want_v, want_i = op(A, B, k=kk, dim=2)   # the unsharded answer, computed on every rank
        B_loc, off = S.column_shard(B)
        B_loc = B_loc.contiguous()
        stride = S.shard_stride(n, world, 128)
        expect(off == rank * stride, "shard offset")

        # Python path
        v, i = S.topk_bmm_column_sharded(A, B_loc, stride, kk, lambda a, b, q: op.packed(a, b, k=q, dim=2))
        expect(torch.equal(v, want_v) and torch.equal(i, want_i), "python path differs from the unsharded answer")

        # a rank whose local step raises: its peers get PeerFailure, nobody merges
        def failing(a, b, q):
            if rank == 1:
                raise RuntimeError("local top-k failed on purpose")
            return op.packed(a, b, k=q, dim=2)

        try:
            S.topk_bmm_column_sharded(A, B_loc, stride, kk, failing)
            expect(False, "the failure was not reported")
        except S.PeerFailure:
            expect(rank != 1, "PeerFailure on the failing rank")
        except RuntimeError as e:
            expect(rank == 1 and "on purpose" in str(e), f"unexpected error {e!r}")

        # C-ABI path: communicator made through the library, id handed round by the host
        idbuf = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            expect(lib.fbmm_comm_get_unique_id(idbuf.data_ptr()) == 0, f"unique id: {lib.fbmm_last_error()}")
        idd = idbuf.to(dev)
        dist.broadcast(idd, 0)
        idbuf = idd.cpu()
        comm = ctypes.c_void_p()
        rc = lib.fbmm_comm_init_rank(ctypes.byref(comm), world, rank, idbuf.data_ptr())
        if rc != 0:
            raise RuntimeError(f"fbmm_comm_init_rank: {lib.fbmm_last_error()}")
        n_loc = B_loc.shape[2]
        ws_bytes = lib.fbmm_topk_bmm_sharded_workspace_bytes(world, m, n_loc, k, kk, 0, ord("n"), k, ord("n"), n_loc)
        ws = torch.empty(ws_bytes, device=dev, dtype=torch.uint8)
        cv = torch.empty(m, kk, device=dev)
        ci = torch.empty(m, kk, device=dev, dtype=torch.int64)
        stream = torch.cuda.current_stream().cuda_stream

        def sharded(b_ptr, check_peers):
            return lib.fbmm_topk_bmm_sharded_f32(stream, comm, world, rank, A.data_ptr(), ord("n"), k, b_ptr, ord("n"),
                                                 n_loc, stride, cv.data_ptr(), ci.data_ptr(), m, n_loc, k, kk, 0,
                                                 check_peers, ws.data_ptr(), ws_bytes)

        for check_peers in (1, 0):
            cv.zero_()
            expect(sharded(B_loc.data_ptr(), check_peers) == 0, f"sharded call: {lib.fbmm_last_error()}")
            expect(torch.equal(cv, want_v[0]) and torch.equal(ci, want_i[0]), "C-ABI path differs from the unsharded answer")
        try:
            R.check_topk(cv[None, :256], ci[None, :256], A[:, :256], B, kk, 2)
        except AssertionError as e:
            expect(False, f"oracle check: {e}")

        # rank 1 hands in a misaligned operand: it gets its own error, rank 0 FBMM_ERR_PEER
        rc = sharded(B_loc.data_ptr() + (4 if rank == 1 else 0), 1)
        expect(rc == (ck.FBMM_ERR_ALIGN if rank == 1 else ck.FBMM_ERR_PEER), f"failure exchange gave {rc}: {lib.fbmm_last_error()}")
        # and the communicator still works
        expect(sharded(B_loc.data_ptr(), 1) == 0, f"call after a failure: {lib.fbmm_last_error()}")
        expect(torch.equal(cv, want_v[0]), "result after a failure")
        torch.cuda.synchronize()
        expect(lib.fbmm_comm_destroy(comm) == 0, "comm destroy")
        expect(lib.fbmm_check(None) == 0, "device status")
        dist.barrier()
        out.put(f"rank {rank}: " + ("ok" if not problems else "; ".join(problems)))
    except Exception as e:  # surface the failure to the parent
        out.put(f"rank {rank}: fail {e!r}")
        raise
    finally:
        dist.destroy_process_group()


def test_column_sharded_topk_on_two_gpus(dev):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    codes = [p.exitcode for p in procs]
    for p in procs:
        if p.is_alive():
            p.terminate()
    msgs = []
    while not out.empty():
        msgs.append(out.get())
    assert codes == [0, 0] and sorted(msgs) == ["rank 0: ok", "rank 1: ok"], (codes, msgs)
