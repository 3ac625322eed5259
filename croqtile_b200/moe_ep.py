"""Expert-parallel MoE layer over one process per GPU.

Tokens are data-parallel (every rank routes its own T/world tokens over all E
experts), experts are owner-partitioned (rank r holds experts
[r*E/world, (r+1)*E/world)). One exchange step on each side of the expert
GEMMs, as an all-to-all-v over NCCL (NVLink/NVSwitch):

  route -> permute + quantise (rows come out expert-sorted, hence already
  grouped by destination rank) -> counts all-gather -> dispatch all-to-all of
  e4m3 rows and their f32 scales -> local regroup by expert -> gate/up grouped
  GEMM with SwiGLU -> re-quantise -> down grouped GEMM -> inverse regroup ->
  combine all-to-all of bf16 rows -> weighted unpermute.

The reference has no MoE and no multi-GPU code; this module defines the
behaviour. Per-row results do not depend on where a row is computed, so the
output equals the single-GPU ``api.moe_forward`` bit for bit.

The arithmetic goes through a backend object (default: the CUDA kernels of
``croqtile_b200.api``); the exchange logic itself is device-agnostic, which is
what the CPU multi-process tests exercise.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist


class CudaBackend:
    """The library's kernels (``croqtile_b200.api``)."""

    def __init__(self):
        from . import api
        self.api = api

    def route(self, logits, k):
        return self.api.moe_route_topk(logits, k)

    def permute_quant(self, x, perm_to_src, k):
        q, s = self.api.quant_rows_e4m3(x)      # once per token, then gather e4m3 rows
        return self.api.moe_permute_q_e4m3(q, s, perm_to_src, k)

    def quant_rows(self, x):
        return self.api.quant_rows_e4m3(x)

    def grouped_gemm(self, x, xs, w, ws, offsets, swiglu):
        return self.api.moe_grouped_gemm_e4m3(x, xs, w, ws, offsets, swiglu=swiglu)

    def gather_rows(self, src, index):
        """dst[i,:] = src[index[i],:] for any 2-D tensor whose row is a whole number of 16-bit words."""
        words = src.contiguous().view(torch.uint8).view(torch.bfloat16)   # bytes as 16-bit words
        out = self.api.moe_permute(words, index, 1)
        return out.view(torch.uint8).view(src.dtype).view(index.shape[0], src.shape[1])

    def unpermute(self, y, src_to_perm, topk_w):
        return self.api.moe_unpermute(y, src_to_perm, topk_w)


def regroup_index(recv_counts: np.ndarray) -> np.ndarray:
    """Rows arrive ordered [source rank][local expert][row]; the grouped GEMM
    wants [local expert][source rank][row]. Returns ``index`` with
    ``sorted[i] = received[index[i]]``. recv_counts is [world, E_local]."""
    counts = np.asarray(recv_counts, np.int64)
    flat = counts.ravel()                                   # received segment order (src, e)
    seg_start = np.concatenate([[0], np.cumsum(flat)[:-1]]).reshape(counts.shape)
    order_starts = seg_start.T.ravel()                      # segments in (e, src) order
    order_counts = counts.T.ravel()
    total = int(flat.sum())
    if total == 0:
        return np.zeros(0, np.int32)
    seg_of_row = np.repeat(np.arange(order_counts.size), order_counts)
    dst_start = np.concatenate([[0], np.cumsum(order_counts)[:-1]])
    within = np.arange(total) - dst_start[seg_of_row]
    return (order_starts[seg_of_row] + within).astype(np.int32)


def _as_bytes(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8)


def _all_to_all_rows(rows: torch.Tensor, send_rows, recv_rows, group) -> torch.Tensor:
    """all-to-all-v of whole rows (any dtype, moved as bytes)."""
    row_bytes = rows.shape[1] * rows.element_size()
    src = _as_bytes(rows).view(-1)
    out = torch.empty((int(sum(recv_rows)) * row_bytes,), dtype=torch.uint8, device=rows.device)
    dist.all_to_all_single(out, src, [int(r) * row_bytes for r in recv_rows],
                           [int(s) * row_bytes for s in send_rows], group=group)
    return out.view(int(sum(recv_rows)), row_bytes).view(rows.dtype).view(int(sum(recv_rows)), rows.shape[1])


def plan_exchange(expert_counts: torch.Tensor, world: int, rank: int, group=None):
    """Exchanges the per-expert row counts and derives the split sizes.
    Returns (send_rows [world], recv_counts [world, E_local] as numpy)."""
    E = expert_counts.shape[0]
    e_loc = E // world
    gathered = [torch.empty_like(expert_counts) for _ in range(world)]
    dist.all_gather(gathered, expert_counts.contiguous(), group=group)
    all_counts = torch.stack(gathered).cpu().numpy().astype(np.int64)      # [src, E]
    send_rows = all_counts[rank].reshape(world, e_loc).sum(1)
    recv_counts = all_counts[:, rank * e_loc:(rank + 1) * e_loc]
    return send_rows, recv_counts


def moe_forward_ep(x, logits, w13, w13_scale, w2, w2_scale, k: int = 8, group=None, backend=None,
                   timers=None):
    """x [T_local,H] bf16, logits [T_local,E] f32; w13 [E_local,2I,H], w2 [E_local,H,I]
    e4m3 with 128x128 block scales (this rank's experts). Returns [T_local,H] bf16."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    E = logits.shape[1]
    if E % world != 0 or w13.shape[0] != E // world:
        raise ValueError("experts must divide evenly over ranks and w13/w2 hold this rank's experts")
    dev = x.device

    def mark(name):
        """Records a device timestamp for the phase that just ended (timers is a
        list of (name, torch.cuda.Event) pairs supplied by the caller)."""
        if timers is not None and x.is_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            timers.append((name, ev))

    mark("start")
    r = backend.route(logits, k)
    xq, xs = backend.permute_quant(x, r["perm_to_src"], k)
    mark("route+permute_quant")
    if world == 1:
        offsets = r["expert_offsets"]
        g = backend.grouped_gemm(xq, xs, w13, w13_scale, offsets, True)
        gq, gs = backend.quant_rows(g)
        y = backend.grouped_gemm(gq, gs, w2, w2_scale, offsets, False)
        mark("expert_gemms")
        out = backend.unpermute(y, r["src_to_perm"], r["topk_w"])
        mark("unpermute")
        return out

    send_rows, recv_counts = plan_exchange(r["expert_counts"], world, rank, group)
    recv_rows = recv_counts.sum(1)
    mark("count_exchange")
    xq_in = _all_to_all_rows(xq, send_rows, recv_rows, group)
    xs_in = _all_to_all_rows(xs, send_rows, recv_rows, group)
    mark("dispatch_all_to_all")

    index_np = regroup_index(recv_counts)
    index = torch.from_numpy(index_np).to(dev)
    inverse = torch.empty_like(index)
    inverse[index.long()] = torch.arange(index.shape[0], dtype=index.dtype, device=dev)
    offsets = torch.from_numpy(
        np.concatenate([[0], np.cumsum(recv_counts.sum(0))]).astype(np.int32)).to(dev)

    xq_sorted = backend.gather_rows(xq_in, index)
    xs_sorted = backend.gather_rows(xs_in, index)
    mark("regroup")
    g = backend.grouped_gemm(xq_sorted, xs_sorted, w13, w13_scale, offsets, True)
    gq, gs = backend.quant_rows(g)
    y = backend.grouped_gemm(gq, gs, w2, w2_scale, offsets, False)
    mark("expert_gemms")
    y_out = backend.gather_rows(y, inverse)                    # back to arrival order
    mark("inverse_regroup")
    y_home = _all_to_all_rows(y_out, recv_rows, send_rows, group)
    mark("combine_all_to_all")
    out = backend.unpermute(y_home, r["src_to_perm"], r["topk_w"])
    mark("unpermute")
    return out
