"""The C-ABI boundary without a GPU: the library loads, exports every symbol
the header declares, and rejects bad arguments before touching CUDA."""
import ctypes
import re
from pathlib import Path

import pytest

from croqtile_b200 import _lib
from croqtile_b200._lib import View1, View2

ROOT = Path(__file__).resolve().parents[1]
HEADER = (ROOT / "include" / "croq_b200.h").read_text()


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(croq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("croq_matmul_f16", "croq_matmul_bf16", "croq_blockscale_gemm_e4m3",
                 "croq_gemm_sp_f16", "croq_moe_route_topk", "croq_moe_permute",
                 "croq_moe_unpermute", "croq_moe_grouped_gemm_e4m3", "croq_synchronize",
                 "croq_status_string"):
        assert must in names


def test_library_exports_every_declared_symbol(croq):
    for name in declared_symbols():
        assert hasattr(croq, name), f"{name} declared in croq_b200.h but not exported"
    assert set(declared_symbols()) == set(_lib.SIGNATURES), "ctypes table and header disagree"


def test_view_layout_matches_spanned_view():
    # choreo::spanned_view<T,R> is {T* ptr; size_t dims[R];} (runtime/choreo.h:761-762)
    assert ctypes.sizeof(View1) == 16 and ctypes.sizeof(View2) == 24
    assert View2.ptr.offset == 0 and View2.dims.offset == 8


def test_status_strings(croq):
    assert croq.croq_status_string(0) == b"ok"
    assert b"align" in croq.croq_status_string(3)
    assert croq.croq_version().count(b".") == 2


def v2(ptr, r, c):
    return ctypes.byref(View2(ptr, (ctypes.c_size_t * 2)(r, c)))


def v1(ptr, n):
    return ctypes.byref(View1(ptr, (ctypes.c_size_t * 1)(n)))


def test_argument_checks_run_before_any_cuda_call(croq):
    """Mirrors the reference wrapper's runtime_check list
    (lib/Target/GPU/cute_codegen.cpp:9939-9961): equal-named dims must agree."""
    P = 0x1000  # fake, 16-byte aligned, never dereferenced: checks fail first
    mm = croq.croq_matmul_f16
    assert mm(None, None, None, None, None, 256, 256, None) == 1          # NULL
    assert mm(v2(0, 8, 8), v2(P, 8, 8), v2(P, 8, 8), None, None, 256, 256, None) == 1
    assert mm(v2(P, 64, 32), v2(P, 64, 48), v2(P, 64, 64), None, None, 256, 256, None) == 2   # K differs
    assert mm(v2(P, 64, 32), v2(P, 64, 32), v2(P, 64, 32), None, None, 256, 256, None) == 2   # out N
    assert mm(v2(P, 64, 32), v2(P, 64, 32), v2(P, 64, 64), None, None, 0, 256, None) == 2
    assert mm(v2(P, 64, 32), v2(P, 64, 32), v2(P, 64, 64), v1(P, 1), None, 64, 64, None) == 1  # one schedule only
    assert mm(v2(P, 512, 32), v2(P, 512, 32), v2(P, 512, 512), v1(P, 3), v1(P, 3), 256, 256, None) == 2  # T < tiles
    assert mm(v2(P, 512, 32), v2(P, 512, 32), v2(P, 512, 512), v1(P, 4), v1(P, 5), 256, 256, None) == 2
    assert mm(v2(P + 2, 64, 32), v2(P, 64, 32), v2(P, 64, 64), None, None, 256, 256, None) == 3  # base
    assert mm(v2(P, 64, 20), v2(P, 64, 20), v2(P, 64, 64), None, None, 256, 256, None) == 3      # pitch
    bs = croq.croq_blockscale_gemm_e4m3
    ok = (v2(P, 128, 256), v2(P, 128, 2), v2(P, 256, 256), v2(P, 2, 2), v2(P, 128, 256))
    assert bs(ok[0], v2(P, 128, 3), ok[2], ok[3], ok[4], 1, None) == 2     # scale_lhs [M, K/128]
    assert bs(ok[0], ok[1], ok[2], v2(P, 3, 2), ok[4], 1, None) == 2       # scale_rhs [N/128, K/128]
    assert bs(ok[0], ok[1], ok[2], ok[3], ok[4], 7, None) == 8             # out dtype
    assert bs(ok[0], ok[1], ok[2], ok[3], None, 1, None) == 1


def test_loader_fails_loudly_when_library_is_missing(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libcroq_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()


def test_package_does_not_import_the_oracle():
    import subprocess, sys
    code = ("import sys; import croqtile_b200, croqtile_b200.api; "
            "assert not any(m.startswith('oracle') for m in sys.modules), 'oracle imported'")
    subprocess.run([sys.executable, "-c", code], check=True, cwd=ROOT)
    for f in (ROOT / "croqtile_b200").rglob("*"):
        if f.suffix in (".py", ".cu", ".cuh", ".h", ".cpp") and f.is_file():
            assert "oracle" not in f.read_text().lower(), f"{f} mentions the oracle"
