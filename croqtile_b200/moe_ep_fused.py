"""Expert-parallel MoE layer with the token exchange fused into the row kernels.

Same layer and same results as ``croqtile_b200.moe_ep.moe_forward_ep``, but no
library all-to-all and no regroup pass: every rank keeps three receive buffers
in symmetric (peer-mapped) memory and

  * the dispatch kernel (gather + e4m3 quantiser) stores each row directly at
    its final expert-sorted position in the owner's buffer over NVLink,
  * the expert GEMMs run on the owner's buffer in place (tile table from the
    device-side offsets, so no host synchronisation anywhere in the step),
  * the combine kernel loads each expert output row from the owner's buffer.

The only collectives left are an 8 KB all-gather of the per-expert counts and
three stream-ordered barriers per step (after dispatch, before combine, after
combine). One process per GPU, ``torch.distributed`` (NCCL) for the plumbing.
The reference has no MoE and no multi-GPU code; this module defines the
behaviour.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, api
from ._lib import View1, View2


def _v1(t):
    return ctypes.byref(View1(t.data_ptr(), (ctypes.c_size_t * 1)(t.shape[0])))


def _v2(t):
    return ctypes.byref(View2(t.data_ptr(), (ctypes.c_size_t * 2)(t.shape[0], t.shape[1])))


class FusedExpertParallel:
    """Owns the symmetric receive buffers of one rank; call ``forward`` per step.

    capacity_rows: rows each receive buffer can hold. The expected load is
    ``tokens_per_rank * k`` rows; routing imbalance needs head-room (default 2x).
    A row that does not fit is reported as CROQ_ERR_INDEX by ``api.synchronize``.
    """

    def __init__(self, hidden: int, intermediate: int, num_experts: int, tokens_per_rank: int, k: int,
                 group=None, capacity_factor: float = 2.0):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if num_experts % self.world != 0:
            raise ValueError("experts must divide evenly over ranks")
        self.E, self.e_loc, self.k = num_experts, num_experts // self.world, k
        self.H, self.I = hidden, intermediate
        self.capacity = int(tokens_per_rank * k * capacity_factor + 127) // 128 * 128
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        # symmetric buffers: e4m3 rows (as bytes), their scales, bf16 expert outputs
        self.q_buf = symm_mem.empty((self.capacity, hidden), dtype=torch.uint8, device=dev)
        self.s_buf = symm_mem.empty((self.capacity, hidden // 128), dtype=torch.float32, device=dev)
        self.y_buf = symm_mem.empty((self.capacity, hidden), dtype=torch.bfloat16, device=dev)
        name = self.group.group_name
        self._handles = [symm_mem.rendezvous(b, name) for b in (self.q_buf, self.s_buf, self.y_buf)]
        ptrs = [torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=dev)
                for h in self._handles]
        self.peer_q, self.peer_s, self.peer_y = ptrs
        self._flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self._lib = _lib.load()

    def _route(self, logits):
        """Routing through the allocation-free entry point when the problem fits its
        built-in scratch (no allocator traffic inside the step)."""
        T = logits.shape[0]
        if ((T + 63) // 64) * self.E > 65536:
            return api.moe_route_topk(logits, self.k)
        k, E, dev = self.k, self.E, self.dev
        out = dict(
            topk_idx=torch.empty((T, k), dtype=torch.int32, device=dev),
            topk_w=torch.empty((T, k), dtype=torch.float32, device=dev),
            expert_counts=torch.empty((E,), dtype=torch.int32, device=dev),
            expert_offsets=torch.empty((E + 1,), dtype=torch.int32, device=dev),
            perm_to_src=torch.empty((T * k,), dtype=torch.int32, device=dev),
            src_to_perm=torch.empty((T * k,), dtype=torch.int32, device=dev),
        )
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc = self._lib.croq_moe_route_topk_noalloc(
            _v2(logits), k, 1, _v2(out["topk_idx"]), _v2(out["topk_w"]), _v1(out["expert_counts"]),
            _v1(out["expert_offsets"]), _v1(out["perm_to_src"]), _v1(out["src_to_perm"]), stream)
        _lib.check(rc, "croq_moe_route_topk_noalloc")
        return out

    def _barrier(self):
        """Stream-ordered barrier: every rank's earlier kernels are complete
        before any rank's later kernels start."""
        dist.all_reduce(self._flag, group=self.group)

    def forward(self, x, logits, w13, w13_scale, w2, w2_scale, timers=None):
        """x bf16 [T_local,H]; logits f32 [T_local,E]; this rank's expert weights."""
        lib, k, E = self._lib, self.k, self.E
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

        def mark(name):
            if timers is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                timers.append((name, ev))

        mark("start")
        r = self._route(logits)
        mark("route")
        # counts of every rank -> placement of my rows in the owners' buffers (all on the device)
        counts = torch.empty((self.world, E), dtype=torch.int32, device=self.dev)
        dist.all_gather_into_tensor(counts, r["expert_counts"], group=self.group)
        total = counts.sum(0, dtype=torch.int32)                                  # rows per expert, all sources
        per_owner = total.view(self.world, self.e_loc)
        expert_start = (per_owner.cumsum(1, dtype=torch.int32) - per_owner).reshape(-1)   # inside the owner
        before_me = counts[: self.rank].sum(0, dtype=torch.int32)                 # rows of lower source ranks
        dest_base = (expert_start + before_me).contiguous()
        mine = total[self.rank * self.e_loc:(self.rank + 1) * self.e_loc]
        offsets = torch.zeros(self.e_loc + 1, dtype=torch.int32, device=self.dev)
        offsets[1:] = mine.cumsum(0, dtype=torch.int32)
        mark("counts+placement")

        # quantise the local tokens once, then send e4m3 rows (each token goes to k owners)
        xq0, xs0 = api.quant_rows_e4m3(x)
        rc = lib.croq_moe_dispatch_rows_q_e4m3(_v2(xq0), _v2(xs0), _v1(r["perm_to_src"]),
                                               _v2(r["topk_idx"]), _v1(r["expert_offsets"]),
                                               _v1(dest_base), _v1(self.peer_q), _v1(self.peer_s),
                                               self.e_loc, self.capacity, stream)
        _lib.check(rc, "croq_moe_dispatch_rows_q_e4m3")
        self._barrier()                      # all rows addressed to me have landed
        mark("dispatch")

        xq = self.q_buf.view(torch.float8_e4m3fn)
        g = api.moe_grouped_gemm_e4m3(xq, self.s_buf, w13, w13_scale, offsets, swiglu=True)
        gq = torch.empty((self.capacity, self.I), dtype=torch.float8_e4m3fn, device=self.dev)
        gs = torch.empty((self.capacity, self.I // 128), dtype=torch.float32, device=self.dev)
        rc = lib.croq_quant_rows_e4m3_n(_v2(g), _v2(gq), _v2(gs), _v1(offsets[self.e_loc:]), stream)
        _lib.check(rc, "croq_quant_rows_e4m3_n")
        api.moe_grouped_gemm_e4m3(gq, gs, w2, w2_scale, offsets, swiglu=False, out=self.y_buf)
        self._barrier()                      # every owner's outputs are complete
        mark("expert_gemms")

        out = torch.empty((x.shape[0], self.H), dtype=torch.bfloat16, device=self.dev)
        rc = lib.croq_moe_combine_remote(_v1(self.peer_y), _v2(r["topk_idx"]), _v1(r["src_to_perm"]),
                                         _v1(r["expert_offsets"]), _v1(dest_base), _v2(r["topk_w"]),
                                         _v2(out), self.e_loc, self.capacity, stream)
        _lib.check(rc, "croq_moe_combine_remote")
        self._barrier()                      # peers are done reading my buffers: next step may overwrite
        mark("combine")
        return out
