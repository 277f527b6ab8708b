"""Multi-GPU partitioning of the fused-BMM ops: one process per GPU, torch.distributed.

The reference is single-GPU (outputs hard-wired to cuda:0, bmm.py:106), so there is no
reference behaviour to match beyond "same answer as one device". Three partitions:

* by batch        bmm / mbmm: contiguous batch ranges, no communication;
* by A rows       min / top-k with one batch: each rank owns M/G rows and the whole B, no
                  communication;
* by B columns    top-k against a very wide B: each rank owns N/G columns and the whole A,
                  writes its local top-k as packed 8-byte candidates {fp32 value, int32
                  shard-local column} straight into the send buffer, then ONE all-gather and a
                  merge kernel on every rank that adds each shard's first column and widens
                  the indices to int64.

The compute callables are injected so that the partition / exchange logic can be tested
with CPU tensors over the gloo backend.
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist


class PeerFailure(RuntimeError):
    """Another rank failed in its local step; this rank skipped the exchange and the merge."""


def shard_range(total: int, world: int, rank: int, granule: int = 1) -> Tuple[int, int]:
    """[begin, end) of `rank`'s contiguous share of `total` items, split in multiples of
    `granule` (the last ranks may get less, or nothing)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    stride = shard_stride(total, world, granule)
    b = min(total, rank * stride)
    e = min(total, (rank + 1) * stride)
    return b, e


def shard_stride(total: int, world: int, granule: int = 1) -> int:
    """Items between the first items of consecutive ranks' shares (see shard_range)."""
    blocks = (total + granule - 1) // granule
    return (blocks + world - 1) // world * granule


def world_info(group=None) -> Tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


def batch_shard(x: torch.Tensor, group=None) -> torch.Tensor:
    """This rank's contiguous slice of the batch axis (bmm / mbmm operands and masks)."""
    rank, world = world_info(group)
    b, e = shard_range(x.shape[0], world, rank)
    return x[b:e]


def row_shard(A: torch.Tensor, group=None) -> Tuple[torch.Tensor, int]:
    """This rank's rows of A [l, m, k] (multiples of the 128-row tile) and their offset."""
    rank, world = world_info(group)
    b, e = shard_range(A.shape[1], world, rank, granule=128)
    return A[:, b:e], b


def column_shard(B: torch.Tensor, group=None) -> Tuple[torch.Tensor, int]:
    """This rank's columns of B [l, k, n] (multiples of the 128-column tile) and their offset."""
    rank, world = world_info(group)
    b, e = shard_range(B.shape[2], world, rank, granule=128)
    return B[:, :, b:e], b


# ---------------------------------------------------------------------------------------
# wire format of the candidate exchange: one int64 per entry, low half = fp32 value bits,
# high half = int32 shard-local column (-1 = empty slot). In memory (little endian) that is
# { float value; int index; }, what fbmm_topk_bmm_packed_f32 writes.
# ---------------------------------------------------------------------------------------
# Column shards cost the top-k kernel efficiency as they get narrower (every row block restarts
# its running lists, and the merges of the first tiles of a sweep hold up the MMAs: measured on one
# B200, 1 048 576 rows, K = 256, k = 64: 231 TFLOP/s at 1 048 576 columns, 229 at 524 288, 217 at
# 262 144, 206 at 131 072), and the exchange grows with the number of shards. So beyond
# MAX_COLUMN_SHARDS ranks the ranks form a grid: columns of B are cut MAX_COLUMN_SHARDS ways (the
# packed all-gather + merge stay in the data path, inside each group of ranks that share rows), and
# the rows of A are cut across the groups, which need no communication at all.
MAX_COLUMN_SHARDS = 2


def topk_grid(world: int, max_column_shards: int = MAX_COLUMN_SHARDS) -> Tuple[int, int]:
    """(row_groups, column_shards) of the rank grid for column-sharded top-k; rank r sits in row
    group r // column_shards and holds column shard r % column_shards."""
    c = max(1, min(world, max_column_shards))
    while world % c:
        c -= 1
    return world // c, c


def make_column_groups(world: int, column_shards: int, rank: int):
    """One process group per row group (the ranks that hold the column shards of the same rows);
    every rank has to call this, since creating a group is collective. Returns this rank's group
    (None when a single group spans the world)."""
    if column_shards == world:
        return None
    mine = None
    for g in range(world // column_shards):
        ranks = list(range(g * column_shards, (g + 1) * column_shards))
        grp = dist.new_group(ranks=ranks)
        if rank in ranks:
            mine = grp
    return mine


def pack_candidates(values: torch.Tensor, local_indices: torch.Tensor) -> torch.Tensor:
    bits = values.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return (local_indices.to(torch.int64) << 32) | bits


def unpack_candidates(packed: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    low_halves = packed.contiguous().view(torch.int32)[..., 0::2]  # little endian: the value comes first
    return low_halves.contiguous().view(torch.float32), packed >> 32


def merge_candidates_torch(cand_v: torch.Tensor, cand_i: torch.Tensor, k: int):
    """Reference merge of [groups, rows, k] candidate lists with torch ops (CPU tests)."""
    g, rows, kk = cand_v.shape
    v = cand_v.permute(1, 0, 2).reshape(rows, g * kk)
    i = cand_i.permute(1, 0, 2).reshape(rows, g * kk)
    v = torch.where(i < 0, torch.full_like(v, float("-inf")), v)
    top_v, sel = v.topk(k, dim=-1)
    return top_v, torch.gather(i, 1, sel)


def merge_packed_torch(packed: torch.Tensor, k: int, group_index_stride: int):
    """Torch statement of fbmm_topk_merge_packed_f32 for [groups, rows, k] packed lists (CPU tests)."""
    v, i = unpack_candidates(packed)
    offs = (torch.arange(packed.shape[0], device=packed.device, dtype=torch.int64) * group_index_stride)[:, None, None]
    return merge_candidates_torch(v, torch.where(i >= 0, i + offs, i), k)


def merge_candidates_cuda(cand_v: torch.Tensor, cand_i: torch.Tensor, k: int):
    """[groups, rows, k] candidates -> ([rows, k], [rows, k]) through fbmm_topk_merge_f32."""
    from .custom_kernel import check, load_library
    lib = load_library()
    g, rows, kk = cand_v.shape
    assert kk == k and cand_v.is_contiguous() and cand_i.is_contiguous()
    out_v = torch.empty((rows, k), device=cand_v.device, dtype=torch.float32)
    out_i = torch.empty((rows, k), device=cand_v.device, dtype=torch.int64)
    with torch.cuda.device(cand_v.device):
        check(lib.fbmm_topk_merge_f32(torch.cuda.current_stream(cand_v.device).cuda_stream, cand_v.data_ptr(),
                                      cand_i.data_ptr(), g, rows, k, out_v.data_ptr(), out_i.data_ptr()))
    return out_v, out_i


def merge_packed_cuda(packed: torch.Tensor, k: int, group_index_stride: int):
    """[groups, rows, k] packed candidates -> ([rows, k] fp32, [rows, k] int64 global indices)
    through fbmm_topk_merge_packed_f32, read in place from the gathered buffer."""
    from .custom_kernel import check, load_library
    lib = load_library()
    g, rows, kk = packed.shape
    assert kk == k and packed.is_contiguous() and packed.dtype == torch.int64
    out_v = torch.empty((rows, k), device=packed.device, dtype=torch.float32)
    out_i = torch.empty((rows, k), device=packed.device, dtype=torch.int64)
    with torch.cuda.device(packed.device):
        check(lib.fbmm_topk_merge_packed_f32(torch.cuda.current_stream(packed.device).cuda_stream, packed.data_ptr(), g,
                                             rows, k, group_index_stride, out_v.data_ptr(), out_i.data_ptr()))
    return out_v, out_i


def topk_bmm_column_sharded(A: torch.Tensor, B_local: torch.Tensor, cols_per_rank: int, k: int,
                            local_packed: Callable, merge: Callable = merge_packed_cuda, group=None,
                            check_peers: bool = True, timings: dict | None = None):
    """Top-k of A @ [B_0 | B_1 | ...] where this rank holds B_local, the columns
    [rank * cols_per_rank, ...) of B, and all of A [1, m, d].

    local_packed(A, B_local, k) -> int64 [1, m, k] packed candidates with shard-local
    columns (TopkBMMCUDA.packed); a rank whose shard is empty contributes empty slots. The
    candidates are exchanged with ONE all_gather and merged on every rank by
    merge(gathered [world, m, k], k, cols_per_rank). Returns (values [1,m,k], indices [1,m,k]).

    With check_peers the ranks first agree, through a 4-byte all-reduce, that every local
    step succeeded: if one raised, that rank re-raises, the others raise PeerFailure, and
    nobody enters the all-gather or runs the merge. `timings` (CUDA only), when given,
    receives the events around the three phases."""
    rank, world = world_info(group)
    m = A.shape[1]
    cuda = A.device.type == "cuda"
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if (timings is not None and cuda) else None
    if ev:
        ev[0].record()
    err = None
    packed = None
    try:
        if B_local.shape[2] > 0:
            packed = local_packed(A, B_local, k).reshape(m, k)
        else:
            packed = pack_candidates(torch.full((m, k), float("-inf"), device=A.device),
                                     torch.full((m, k), -1, device=A.device, dtype=torch.int64))
    except Exception as e:  # noqa: BLE001 -- reported to the peers below, then re-raised
        err = e
    if ev:
        ev[1].record()
    if world > 1 and check_peers:
        flag = torch.tensor([0 if err is None else 1], device=A.device, dtype=torch.int32)
        dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
        if int(flag.item()) != 0:
            if err is not None:
                raise err
            raise PeerFailure("another rank failed in its local top-k; the exchange and the merge were skipped")
    elif err is not None:
        raise err
    if world == 1:
        gathered = packed.reshape(1, m, k)
    else:
        gathered = torch.empty((world, m, k), device=A.device, dtype=torch.int64)
        dist.all_gather_into_tensor(gathered, packed.reshape(1, m, k).contiguous(), group=group)
    if ev:
        ev[2].record()
    mv, mi = merge(gathered, k, cols_per_rank)
    if ev:
        ev[3].record()
        timings["events"] = ev
    return mv[None], mi[None]
