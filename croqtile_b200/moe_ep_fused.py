"""Expert-parallel MoE layer with the token exchange fused into the kernels.

Same layer and same results as ``croqtile_b200.moe_ep.moe_forward_ep``, but no
library all-to-all and no regroup pass: every rank keeps its receive buffers in
symmetric (peer-mapped) memory and

  * the dispatch kernel copies each quantised row, its scales and its return
    address directly to its final expert-sorted position in the owner's buffers
    over NVLink (the local tokens are quantised once beforehand),
  * the expert GEMMs run on the owner's buffer in place (tile table from the
    device-side offsets, so no host synchronisation anywhere in the step),
  * the combine kernel loads each expert output row from the owner's buffer
    (default), or the down projection's epilogue stores every result row
    straight into the home rank's buffer at row t*k+j and the combine becomes a
    local weighted sum (``push_results=True``).

The only collectives left are an 8 KB all-gather of the per-expert counts and
three (two with pushed results) stream-ordered barriers per step. One process
per GPU, ``torch.distributed`` (NCCL) for the plumbing; only plain loads and
stores cross the link. The reference has no MoE and no multi-GPU code; this
module defines the behaviour.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import _lib, api
from ._lib import View1, View2, View3


def _v1(t):
    return ctypes.byref(View1(t.data_ptr(), (ctypes.c_size_t * 1)(t.shape[0])))


def _v2(t):
    return ctypes.byref(View2(t.data_ptr(), (ctypes.c_size_t * 2)(t.shape[0], t.shape[1])))


def _v3(t):
    return ctypes.byref(View3(t.data_ptr(), (ctypes.c_size_t * 3)(*t.shape)))


class FusedExpertParallel:
    """Owns the symmetric receive buffers of one rank; call ``forward`` per step.

    capacity_rows: rows each receive buffer can hold. The expected load is
    ``tokens_per_rank * k`` rows; routing imbalance needs head-room (default 2x).
    A row that does not fit is reported as CROQ_ERR_INDEX by ``api.synchronize``.

    push_results: False (default) keeps the expert outputs on the owner and lets the
    combine kernel load them over NVLink. True lets the down projection's epilogue store
    each result row into the home rank's buffer instead (one barrier less per step, same
    bits). The pushed form is not the default: on two GPUs it ended most benchmark runs
    with "unspecified launch failure" on one rank after several back-to-back steps, and the
    cause has not been found; do not enable it outside single-GPU tests.
    """

    def __init__(self, hidden: int, intermediate: int, num_experts: int, tokens_per_rank: int, k: int,
                 group=None, capacity_factor: float = 2.0, push_results: bool = False):
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
        # symmetric buffers. Received on the expert owner: e4m3 rows (as bytes), their
        # scales and each row's return address. Received on the token's home rank: the
        # expert outputs, one row per (token, pick) in t*k+j order.
        self.home_rows = tokens_per_rank * k
        self.q_buf = symm_mem.empty((self.capacity, hidden), dtype=torch.uint8, device=dev)
        self.s_buf = symm_mem.empty((self.capacity, hidden // 128), dtype=torch.float32, device=dev)
        self.ret_buf = symm_mem.empty((self.capacity,), dtype=torch.int64, device=dev)
        self.push_results = push_results
        y_rows = self.home_rows if push_results else self.capacity
        self.y_home = symm_mem.empty((y_rows, hidden), dtype=torch.bfloat16, device=dev)
        name = self.group.group_name
        self._handles = [symm_mem.rendezvous(b, name)
                         for b in (self.q_buf, self.s_buf, self.ret_buf, self.y_home)]
        ptrs = [torch.tensor([int(p) for p in h.buffer_ptrs], dtype=torch.int64, device=dev)
                for h in self._handles]
        self.peer_q, self.peer_s, self.peer_ret, self.peer_y = ptrs
        self._identity = torch.arange(self.home_rows, dtype=torch.int32, device=dev)
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
        dest_base = torch.empty((E,), dtype=torch.int32, device=self.dev)
        offsets = torch.empty((self.e_loc + 1,), dtype=torch.int32, device=self.dev)
        rc = lib.croq_moe_ep_placement(_v2(counts), self.rank, _v1(dest_base), _v1(offsets), stream)
        _lib.check(rc, "croq_moe_ep_placement")
        mark("counts+placement")

        # quantise the local tokens once, then send e4m3 rows (each token goes to k owners)
        # together with the address their result has to come back to
        if x.shape[0] * k > self.home_rows:
            raise ValueError("more tokens than the buffers were sized for")
        xq0, xs0 = api.quant_rows_e4m3(x)
        rc = lib.croq_moe_dispatch_rows_q_e4m3(_v2(xq0), _v2(xs0), _v1(r["perm_to_src"]),
                                               _v2(r["topk_idx"]), _v1(r["expert_offsets"]),
                                               _v1(dest_base), _v1(self.peer_q), _v1(self.peer_s),
                                               _v1(self.peer_ret), self.rank,
                                               self.e_loc, self.capacity, stream)
        _lib.check(rc, "croq_moe_dispatch_rows_q_e4m3")
        # All rows addressed to me have landed. It also orders this step after every
        # rank's combine of the previous step, so peers may overwrite y_home again.
        self._barrier()
        mark("dispatch")

        xq = self.q_buf.view(torch.float8_e4m3fn)
        g = api.moe_grouped_gemm_e4m3(xq, self.s_buf, w13, w13_scale, offsets, swiglu=True)
        gq = torch.empty((self.capacity, self.I), dtype=torch.float8_e4m3fn, device=self.dev)
        gs = torch.empty((self.capacity, self.I // 128), dtype=torch.float32, device=self.dev)
        rc = lib.croq_quant_rows_e4m3_n(_v2(g), _v2(gq), _v2(gs), _v1(offsets[self.e_loc:]), stream)
        _lib.check(rc, "croq_quant_rows_e4m3_n")
        if not self.push_results:
            # results stay on the owner; the combine loads them over NVLink
            api.moe_grouped_gemm_e4m3(gq, gs, w2, w2_scale, offsets, swiglu=False, out=self.y_home)
            self._barrier()                  # every owner's outputs are complete
            mark("expert_gemms")
            out = torch.empty((x.shape[0], self.H), dtype=torch.bfloat16, device=self.dev)
            rc = lib.croq_moe_combine_remote(_v1(self.peer_y), _v2(r["topk_idx"]), _v1(r["src_to_perm"]),
                                             _v1(r["expert_offsets"]), _v1(dest_base), _v2(r["topk_w"]),
                                             _v2(out), self.e_loc, self.capacity, stream)
            _lib.check(rc, "croq_moe_combine_remote")
            self._barrier()                  # peers are done reading my buffer: next step may overwrite
            mark("combine")
            return out
        # down projection; its epilogue stores every result row at its return address in
        # the home rank's y_home (over NVLink, while the next tiles' main loops run)
        rc = lib.croq_moe_grouped_gemm_e4m3_scatter(_v2(gq), _v2(gs), _v3(w2), _v3(w2_scale), _v1(offsets),
                                                    _v1(self.ret_buf), _v1(self.peer_y), self.home_rows,
                                                    stream)
        _lib.check(rc, "croq_moe_grouped_gemm_e4m3_scatter")
        self._barrier()                      # every owner has delivered my rows
        mark("expert_gemms")

        # rows of token t sit at y_home[t*k .. t*k+k-1]: a local weighted sum in ascending j
        rows = x.shape[0] * k
        out = api.moe_unpermute(self.y_home[:rows], self._identity[:rows], r["topk_w"])
        mark("combine")
        return out
