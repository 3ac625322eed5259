"""N-sharded dense / FP8 / sparse GEMM over several GPUs (one process per GPU).

The GEMMs of this library shard along N with no data-path collective: every
rank owns a contiguous slab of ``rhs`` rows (= output columns), ``lhs`` is
replicated, and each rank writes its ``[M, N_local]`` output slab, visiting its
own ``tiles_m x tiles_n_local`` grid in Hilbert order. Slabs are aligned to 256
columns (one CTA-pair tile; also a whole number of 128-row ``scale_rhs`` blocks),
so no tile and no scale block straddles two ranks.

A replicated output is assembled only when the caller asks for it, with one
``all_gather`` (NCCL on GPUs, gloo in the CPU tests): either of the row-major
``[M, N]`` matrix through a ``[world, M, N_max]`` staging buffer, or — with the
transposed store of ``croq_matmul_ex`` — of ``output^T [N, M]``, whose slabs are
contiguous row blocks and need no staging when all slabs have the same width.

The reference has no multi-GPU code; this module defines the behaviour.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

SLAB_ALIGN = 256


def shard_range(n_global: int, world: int, rank: int, align: int = SLAB_ALIGN) -> tuple[int, int]:
    """[lo, hi) of the output columns rank `rank` owns: whole `align`-wide blocks,
    dealt out contiguously, the last rank taking the ragged rest (possibly nothing)."""
    blocks = -(-n_global // align)
    per = -(-blocks // world)
    lo = min(n_global, rank * per * align)
    hi = min(n_global, (rank + 1) * per * align)
    return lo, hi


class CudaBackend:
    """The library's kernels."""

    def matmul(self, lhs, rhs_shard, transposed=False):
        from . import api
        from .schedule import hilbert_schedule
        m, n_loc = lhs.shape[0], rhs_shard.shape[0]
        sm, sn = hilbert_schedule(-(-m // 256), -(-n_loc // 256))
        dev = lhs.device
        return api.matmul_ex(lhs, rhs_shard, None, torch.from_numpy(sm).to(dev), torch.from_numpy(sn).to(dev),
                             256, 256, transposed=transposed)

    def blockscale(self, lhs, scale_lhs, rhs_shard, scale_rhs_shard):
        from . import api
        return api.blockscale_gemm_e4m3(lhs, scale_lhs, rhs_shard, scale_rhs_shard)


def _all_gather_rows(staging: torch.Tensor, mine: torch.Tensor, group) -> None:
    """staging[r] = rank r's `mine` (list form of all_gather: also available on gloo)."""
    dist.all_gather(list(staging.unbind(0)), mine.contiguous(), group=group)


def _gather_row_major(local: torch.Tensor, n_global: int, group) -> torch.Tensor:
    """[M, N_local] slabs of all ranks -> replicated [M, N]."""
    world = dist.get_world_size(group)
    bounds = [shard_range(n_global, world, r) for r in range(world)]
    widest = max(hi - lo for lo, hi in bounds)
    m = local.shape[0]
    mine = local
    if local.shape[1] != widest:                      # ragged last slab: pad to the common width
        mine = local.new_zeros((m, widest))
        mine[:, : local.shape[1]] = local
    staging = local.new_empty((world, m, widest))
    _all_gather_rows(staging, mine, group)
    out = local.new_empty((m, n_global))
    for r, (lo, hi) in enumerate(bounds):
        if hi > lo:
            out[:, lo:hi] = staging[r, :, : hi - lo]
    return out


def _gather_transposed(local_t: torch.Tensor, n_global: int, group) -> torch.Tensor:
    """[N_local, M] slabs (transposed store) of all ranks -> replicated output^T [N, M]."""
    world = dist.get_world_size(group)
    bounds = [shard_range(n_global, world, r) for r in range(world)]
    widths = [hi - lo for lo, hi in bounds]
    m = local_t.shape[1]
    if len(set(widths)) == 1:                          # equal slabs: gather straight into place
        out = local_t.new_empty((n_global, m))
        _all_gather_rows(out.view(world, widths[0], m), local_t, group)
        return out
    widest = max(widths)
    mine = local_t.new_zeros((widest, m))
    mine[: local_t.shape[0]] = local_t
    staging = local_t.new_empty((world, widest, m))
    _all_gather_rows(staging, mine, group)
    return torch.cat([staging[r, :w] for r, w in enumerate(widths) if w > 0], dim=0)


def matmul_nsharded(lhs: torch.Tensor, rhs_shard: torch.Tensor, n_global: int, *,
                    gather_output: str | None = None, group=None, backend=None) -> torch.Tensor:
    """output[:, lo:hi] = lhs @ rhs_shard^T for this rank's slab (``shard_range``).

    gather_output: None -> this rank's [M, N_local] slab (no collective);
    "row_major" -> the replicated [M, N]; "transposed" -> the replicated output^T [N, M]
    (the slabs are computed with the transposed store)."""
    backend = backend or CudaBackend()
    if gather_output not in (None, "row_major", "transposed"):
        raise ValueError("gather_output is None, 'row_major' or 'transposed'")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    lo, hi = shard_range(n_global, world, rank)
    if rhs_shard.shape[0] != hi - lo:
        raise ValueError(f"rank {rank} owns columns [{lo},{hi}) but got {rhs_shard.shape[0]} rhs rows")
    if gather_output == "transposed":
        local_t = (backend.matmul(lhs, rhs_shard, transposed=True) if hi > lo
                   else lhs.new_empty((0, lhs.shape[0])))
        return _gather_transposed(local_t, n_global, group) if world > 1 else local_t
    local = backend.matmul(lhs, rhs_shard) if hi > lo else lhs.new_empty((lhs.shape[0], 0))
    if gather_output is None or world == 1:
        return local
    return _gather_row_major(local, n_global, group)


def blockscale_nsharded(lhs: torch.Tensor, scale_lhs: torch.Tensor, rhs_shard: torch.Tensor,
                        scale_rhs_shard: torch.Tensor, n_global: int, *,
                        gather_output: bool = False, group=None, backend=None) -> torch.Tensor:
    """FP8 block-scaled GEMM on this rank's slab: ``rhs_shard`` e4m3 [N_local, K] with its
    ``scale_rhs`` rows [N_local/128, K/128]; ``lhs`` and ``scale_lhs`` replicated."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    lo, hi = shard_range(n_global, world, rank)
    if rhs_shard.shape[0] != hi - lo or scale_rhs_shard.shape[0] != -(-(hi - lo) // 128):
        raise ValueError(f"rank {rank} owns columns [{lo},{hi}): rhs / scale_rhs rows do not match")
    local = (backend.blockscale(lhs, scale_lhs, rhs_shard, scale_rhs_shard) if hi > lo
             else torch.empty((lhs.shape[0], 0), dtype=torch.bfloat16, device=lhs.device))
    if not gather_output or world == 1:
        return local
    return _gather_row_major(local, n_global, group)
