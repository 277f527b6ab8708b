"""Multi-GPU partitioning of the fused-BMM ops: one process per GPU, torch.distributed.

The reference is single-GPU (outputs hard-wired to cuda:0, bmm.py:106), so there is no
reference behaviour to match beyond "same answer as one device". Three partitions:

* by batch        bmm / mbmm: contiguous batch ranges, no communication;
* by A rows       min / top-k with one batch: each rank owns M/G rows and the whole B, no
                  communication;
* by B columns    top-k against a very wide B: each rank owns N/G columns and the whole A,
                  produces its local top-k with GLOBAL column indices, then ONE all-gather
                  of the (value, index) candidates and a merge kernel on every rank.

The compute callables are injected so that the partition / exchange logic can be tested
with CPU tensors over the gloo backend.
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int, granule: int = 1) -> Tuple[int, int]:
    """[begin, end) of `rank`'s contiguous share of `total` items, split in multiples of
    `granule` (the last ranks may get less, or nothing)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} / world {world}")
    blocks = (total + granule - 1) // granule
    per = (blocks + world - 1) // world
    b = min(total, rank * per * granule)
    e = min(total, (rank + 1) * per * granule)
    return b, e


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


def merge_candidates_torch(cand_v: torch.Tensor, cand_i: torch.Tensor, k: int):
    """Reference merge of [groups, rows, k] candidate lists with torch ops (CPU tests)."""
    g, rows, kk = cand_v.shape
    v = cand_v.permute(1, 0, 2).reshape(rows, g * kk)
    i = cand_i.permute(1, 0, 2).reshape(rows, g * kk)
    v = torch.where(i < 0, torch.full_like(v, float("-inf")), v)
    top_v, sel = v.topk(k, dim=-1)
    return top_v, torch.gather(i, 1, sel)


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


def topk_bmm_column_sharded(A: torch.Tensor, B_local: torch.Tensor, col_offset: int, k: int,
                            local_topk: Callable, merge: Callable = merge_candidates_cuda, group=None):
    """Top-k of A @ [B_0 | B_1 | ...] where this rank holds B_local (columns starting at
    `col_offset`) and all of A [1, m, d].

    local_topk(A, B_local, k, index_offset) -> (values [1,m,k], indices [1,m,k]) with
    global column indices; ranks whose shard is empty contribute -inf / -1. The
    candidates are exchanged with ONE all_gather per tensor and merged on every rank.
    Returns (values [1,m,k], indices [1,m,k])."""
    rank, world = world_info(group)
    m = A.shape[1]
    if B_local.shape[2] > 0:
        v, i = local_topk(A, B_local, k, col_offset)
    else:
        v = torch.full((1, m, k), float("-inf"), device=A.device, dtype=torch.float32)
        i = torch.full((1, m, k), -1, device=A.device, dtype=torch.int64)
    if world == 1:
        return v, i
    all_v = torch.empty((world, m, k), device=A.device, dtype=torch.float32)
    all_i = torch.empty((world, m, k), device=A.device, dtype=torch.int64)
    dist.all_gather_into_tensor(all_v, v.reshape(1, m, k).contiguous(), group=group)
    dist.all_gather_into_tensor(all_i, i.reshape(1, m, k).contiguous(), group=group)
    mv, mi = merge(all_v, all_i, k)
    return mv[None], mi[None]
