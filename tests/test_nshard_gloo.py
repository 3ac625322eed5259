"""N-sharded GEMM assembly as gloo ranks on CPU (world sizes 2 and 3): slab bounds,
the row-major and the transposed all-gather of the output, ragged last slabs and ranks
that own nothing. The arithmetic is the oracle's row-by-row GEMM; what is under test is
croqtile_b200.nshard (partitioning, padding, gather, reassembly)."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


class OracleGemm:
    """Backend over the CPU oracle (fp32 operands, fp32 result)."""

    def matmul(self, lhs, rhs_shard, transposed=False):
        from oracle import oracle as o
        out = torch.from_numpy(o.gemm_row_row(lhs.numpy(), rhs_shard.numpy()))
        return out.t().contiguous() if transposed else out


def problem(n):
    rng = np.random.default_rng(n)
    lhs = rng.integers(-4, 5, (40, 64)).astype(np.float32)        # exact in fp32: bit-exact compare
    rhs = rng.integers(-4, 5, (n, 64)).astype(np.float32)
    return torch.from_numpy(lhs), torch.from_numpy(rhs)


def worker(rank, world, port, n, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from croqtile_b200.nshard import matmul_nsharded, shard_range
    lhs, rhs = problem(n)
    lo, hi = shard_range(n, world, rank)
    shard = rhs[lo:hi].contiguous()
    be = OracleGemm()
    local = matmul_nsharded(lhs, shard, n, backend=be)
    full = matmul_nsharded(lhs, shard, n, gather_output="row_major", backend=be)
    full_t = matmul_nsharded(lhs, shard, n, gather_output="transposed", backend=be)
    np.savez(Path(out_dir) / f"r{rank}.npz", local=local.numpy(), full=full.numpy(), full_t=full_t.numpy(),
             lo=lo, hi=hi)
    dist.barrier()
    dist.destroy_process_group()


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_ranges_cover_n_in_aligned_slabs():
    from croqtile_b200.nshard import shard_range
    for n in (256, 1000, 8192, 7168, 300, 1):
        for world in (1, 2, 3, 8):
            bounds = [shard_range(n, world, r) for r in range(world)]
            assert bounds[0][0] == 0 and bounds[-1][1] == n
            for (lo, hi), (lo2, _) in zip(bounds, bounds[1:]):
                assert hi == lo2 and (lo % 256 == 0 or lo == n)   # contiguous, 256-aligned starts
            assert all(hi >= lo for lo, hi in bounds)
    assert [shard_range(8192, 8, r) for r in (0, 7)] == [(0, 1024), (7168, 8192)]
    assert shard_range(300, 3, 2) == (300, 300)              # a rank may own nothing


@pytest.mark.parametrize("world,n", [(2, 512), (2, 1000), (3, 600)])
def test_gathered_output_equals_the_unsharded_product(tmp_path, world, n):
    from oracle import oracle as o
    mp.spawn(worker, args=(world, free_port(), n, str(tmp_path)), nprocs=world, join=True)
    lhs, rhs = problem(n)
    want = o.gemm_row_row(lhs.numpy(), rhs.numpy())
    for r in range(world):
        got = np.load(tmp_path / f"r{r}.npz")
        np.testing.assert_array_equal(got["local"], want[:, int(got["lo"]):int(got["hi"])])
        np.testing.assert_array_equal(got["full"], want)
        np.testing.assert_array_equal(got["full_t"], want.T)
