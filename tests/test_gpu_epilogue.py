"""GPU parity of the dense GEMM's store variants (croq_matmul_ex) against the CPU
oracle, through the C ABI: f32 output (tests/gpu/end2end/wgmma_ss.co:5-28),
transposed store (wgmma_ss.co:146-166), masked store on ragged extents
(wgmma_ss.co:169-194, the 70x130 case) and scalar bias (ampere_mma.co:79-104)."""
import numpy as np
import pytest
import torch

from croqtile_b200 import api
from croqtile_b200._lib import CroqError
from tests.gpu_util import bits_of, max_rel_err, to_dev_16
from tests.test_oracle_golden import kat1_inputs

pytestmark = pytest.mark.gpu
TORCH = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}


def result_f32(oracle, t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.float32:
        return t.cpu().numpy()
    return oracle.decode(bits_of(t), "f16" if t.dtype == torch.float16 else "bf16")


def expected(oracle, ref_f32: np.ndarray, out: str, transposed: bool) -> np.ndarray:
    e = ref_f32.T if transposed else ref_f32
    e = np.ascontiguousarray(e, np.float32)
    return e if out == "f32" else oracle.decode(oracle.round_to(e, out), out)


@pytest.mark.parametrize("tile", [(256, 256), (64, 128)])          # CTA-pair / single-CTA kernel
@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_kat1_every_variant_is_bit_exact(oracle, dtype, tile):
    """The mod-3 pattern (wgmma_ss.co:324-344) has exactly representable results,
    so every output type, orientation and bias must match bit for bit."""
    lhs, rhs = kat1_inputs()
    lb, rb = oracle.round_to(lhs, dtype), oracle.round_to(rhs, dtype)
    ref = oracle.gemm_row_row(oracle.decode(lb, dtype), oracle.decode(rb, dtype))
    a, b = to_dev_16(lb, dtype), to_dev_16(rb, dtype)
    for out in ("f16", "bf16", "f32"):
        for transposed in (False, True):
            for bias in (0.0, 0.75):
                shape = ref.T.shape if transposed else ref.shape
                buf = torch.full(shape, float("nan"), dtype=TORCH[out], device="cuda")
                api.matmul_ex(a, b, buf, None, None, tile[0], tile[1], transposed=transposed, bias=bias)
                api.synchronize()
                want = expected(oracle, ref + np.float32(bias), out, transposed)
                np.testing.assert_array_equal(result_f32(oracle, buf), want,
                                              err_msg=f"{dtype}->{out} transposed={transposed} bias={bias}")


@pytest.mark.parametrize("shape", [(70, 130, 72), (1000, 776, 264), (129, 257, 8), (515, 300, 1032)])
@pytest.mark.parametrize("out,transposed", [("f32", False), ("f32", True), ("f16", True), ("bf16", False)])
def test_ragged_extents(oracle, shape, out, transposed):
    """Masked store: extents that are no multiple of any tile, unaligned rows."""
    m, n, k = shape
    rng = np.random.default_rng(m * 31 + n)
    lhs = (rng.random((m, k)) * 2 - 1).astype(np.float32)
    rhs = (rng.random((n, k)) * 2 - 1).astype(np.float32)
    lb, rb = oracle.round_to(lhs, "f16"), oracle.round_to(rhs, "f16")
    ref = oracle.gemm_row_row(oracle.decode(lb, "f16"), oracle.decode(rb, "f16")) + np.float32(0.125)
    # guard band around the output: the store must not touch anything outside it
    rows, cols = (n, m) if transposed else (m, n)
    slab = torch.full((rows + 2, cols), -77.0, dtype=TORCH[out], device="cuda")
    buf = slab[1:rows + 1]
    api.matmul_ex(to_dev_16(lb, "f16"), to_dev_16(rb, "f16"), buf, transposed=transposed, bias=0.125)
    api.synchronize()
    want = ref.T if transposed else ref
    # f32 output: only the accumulation differs from the oracle's sequential fp32 sum (the
    # tensor core adds aligned products in groups), which stays far below 16-bit rounding
    tol = 1e-4 if out == "f32" else 5e-3
    err = max_rel_err(result_f32(oracle, buf), want, floor=0.05 * np.sqrt(k))
    assert err <= tol, f"max relative error {err:.3e}"
    assert (slab[0].float() == -77.0).all() and (slab[-1].float() == -77.0).all()


def test_empty_k_gives_the_bias(oracle):
    a = torch.empty((64, 0), dtype=torch.float16, device="cuda")
    b = torch.empty((32, 0), dtype=torch.float16, device="cuda")
    out = api.matmul_ex(a, b, out_dtype=torch.float32, bias=1.5)
    api.synchronize()
    assert out.shape == (64, 32) and (out == 1.5).all()
    out = api.matmul_ex(a, b, transposed=True)
    api.synchronize()
    assert out.shape == (32, 64) and (out == 0).all()


def test_argument_errors():
    a = torch.zeros((64, 64), dtype=torch.float16, device="cuda")
    with pytest.raises(CroqError):     # transposed output must be [N, M]
        api.matmul_ex(a, a[:32].contiguous(), torch.empty((64, 32), dtype=torch.float16, device="cuda"),
                      transposed=True)
