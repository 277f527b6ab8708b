"""CPU tests of the multi-GPU partition / exchange logic: two gloo ranks, oracle compute."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from custom_matmul_kernels_b200 import sharding as S
from oracle import ref_semantics as R


def test_shard_range_covers_everything_once():
    for total, world, gran in [(1048576, 8, 128), (1000, 3, 128), (5, 8, 1), (128, 2, 128), (0, 2, 1)]:
        seen = []
        for r in range(world):
            b, e = S.shard_range(total, world, r, gran)
            assert 0 <= b <= e <= total
            if b < e:
                assert b % gran == 0
            seen += list(range(b, e))
        assert seen == list(range(total))
    with pytest.raises(ValueError):
        S.shard_range(10, 2, 2)


def test_merge_candidates_torch_handles_empty_slots():
    v = torch.tensor([[[5., 3., float("-inf")]], [[4., 4., 1.]]])
    i = torch.tensor([[[7, 2, -1]], [[9, 11, 30]]])
    mv, mi = S.merge_candidates_torch(v, i, 3)
    assert mv.tolist() == [[5., 4., 4.]] and sorted(mi[0].tolist()) == [7, 9, 11]


def test_pack_unpack_candidates_round_trip():
    v = torch.tensor([[1.5, -2.0, float("-inf")], [0.0, -0.0, 3.25]])
    i = torch.tensor([[7, 123456, -1], [0, 2147483646, 5]])
    p = S.pack_candidates(v, i)
    assert p.dtype == torch.int64
    vv, ii = S.unpack_candidates(p)
    assert torch.equal(vv.view(torch.int32), v.view(torch.int32)) and torch.equal(ii, i)
    # in memory an entry is { float value; int index; }
    raw = p.numpy().view("<i4").reshape(2, 3, 2)
    assert raw[0, 1, 1] == 123456 and raw[0, 2, 1] == -1
    mv, mi = S.merge_packed_torch(torch.stack([p, p]), 2, 1000)
    assert mv[0].tolist() == [1.5, 1.5] and sorted(mi[0].tolist()) == [7, 1007]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        A = torch.randn(1, 300, 24, generator=g)
        B = torch.randn(1, 24, 1000, generator=g)
        k = 9

        def local_packed(a, b, kk):
            v, i = R.topk_bmm(a, b, k=kk, dim=2)   # shard-local columns, -1 in empty slots
            return S.pack_candidates(v, i)

        # column shards + ONE all-gather of packed candidates + merge
        B_loc, off = S.column_shard(B)
        stride = S.shard_stride(B.shape[2], world, 128)
        assert off == rank * stride
        v, i = S.topk_bmm_column_sharded(A, B_loc.contiguous(), stride, k, local_packed, merge=S.merge_packed_torch)
        R.check_topk(v, i, A, B, k, 2)
        wv, _ = R.topk_bmm(A, B, k=k, dim=2)
        assert torch.equal(v, wv)

        # a rank whose local step fails: nobody enters the all-gather, nobody merges
        merges = []

        def failing(a, b, kk):
            if rank == 1:
                raise RuntimeError("local top-k failed on purpose")
            return local_packed(a, b, kk)

        def counting_merge(*args):
            merges.append(1)
            return S.merge_packed_torch(*args)

        try:
            S.topk_bmm_column_sharded(A, B_loc.contiguous(), stride, k, failing, merge=counting_merge)
            raise AssertionError("the failure was not reported")
        except S.PeerFailure:
            assert rank == 0
        except RuntimeError as e:
            assert rank == 1 and "on purpose" in str(e)
        assert not merges
        # the group is still usable afterwards
        v2, _ = S.topk_bmm_column_sharded(A, B_loc.contiguous(), stride, k, local_packed, merge=S.merge_packed_torch)
        assert torch.equal(v2, wv)

        # row shards: no communication, concatenation of rank outputs is the full answer
        A_loc, r0 = S.row_shard(A)
        mv, mi = R.min_bmm(A_loc, B, dim=2)
        gathered = [None] * world
        dist.all_gather_object(gathered, (r0, mv, mi))
        full_v = torch.cat([x[1] for x in sorted(gathered, key=lambda x: x[0])], dim=1)
        full_i = torch.cat([x[2] for x in sorted(gathered, key=lambda x: x[0])], dim=1)
        ov, oi = R.min_bmm(A, B, dim=2)
        assert torch.equal(full_v, ov) and torch.equal(full_i, oi)

        # batch shards
        Ab = torch.randn(5, 8, 4, generator=g)
        sl = S.batch_shard(Ab)
        counts = [None] * world
        dist.all_gather_object(counts, sl.shape[0])
        assert sum(counts) == 5
        if rank == 0:
            out.put("ok")
    except Exception as e:  # surface the failure to the parent
        if rank == 0:
            out.put(f"fail: {e!r}")
        raise
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_partitions_match_single_device():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get() == "ok"


def test_topk_grid_shapes():
    assert S.topk_grid(1) == (1, 1)
    assert S.topk_grid(2) == (1, 2)
    assert S.topk_grid(4) == (2, 2)
    assert S.topk_grid(8) == (4, 2)
    assert S.topk_grid(3) == (3, 1)          # no way to cut 3 ranks into column pairs
    assert S.topk_grid(8, max_column_shards=8) == (1, 8)


def _grid_worker(rank, world, port, out):
    """Four ranks as a 2 x 2 grid: columns of B cut two ways inside each row group (packed
    all-gather + merge within the group), rows of A cut across the two groups."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(9)
        A = torch.randn(1, 512, 24, generator=g)
        B = torch.randn(1, 24, 1000, generator=g)
        k = 11
        rg, cs = S.topk_grid(world)
        assert (rg, cs) == (2, 2)
        group = S.make_column_groups(world, cs, rank)
        r0, r1 = S.shard_range(A.shape[1], rg, rank // cs, 256)
        c0, c1 = S.shard_range(B.shape[2], cs, rank % cs, 128)
        stride = S.shard_stride(B.shape[2], cs, 128)

        def local_packed(a, b, kk):
            v, i = R.topk_bmm(a, b, k=kk, dim=2)
            return S.pack_candidates(v, i)

        v, i = S.topk_bmm_column_sharded(A[:, r0:r1].contiguous(), B[:, :, c0:c1].contiguous(), stride, k, local_packed,
                                         merge=S.merge_packed_torch, group=group)
        wv, wi = R.topk_bmm(A, B, k=k, dim=2)
        assert torch.equal(v, wv[:, r0:r1])
        R.check_topk(v, i, A[:, r0:r1], B, k, 2)
        gathered = [None] * world
        dist.all_gather_object(gathered, (rank, r0, v))
        if rank == 0:
            # one rank of every row group: together they hold every row once
            rows = torch.cat([x[2] for x in sorted(gathered) if x[0] % cs == 0], dim=1)
            assert torch.equal(rows, wv)
            out.put("ok")
    except Exception as e:
        if rank == 0:
            out.put(f"fail: {e!r}")
        raise
    finally:
        dist.destroy_process_group()


def test_four_rank_gloo_grid_matches_single_device():
    ctx = mp.get_context("spawn")
    out = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_grid_worker, args=(r, 4, port, out)) for r in range(4)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert out.get() == "ok"
