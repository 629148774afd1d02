"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/flashrt_b200.h declares (no compute calls here)."""
import re

import pytest
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "flashrt-hf-kernels_b200" / "torch-ext"))


def declared_symbols():
    text = (ROOT / "include" / "flashrt_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(frt_[a-z0-9_]+)\s*\(", text)))


def test_header_and_ctypes_table_agree():
    from flashrt_b200_core import capi
    assert sorted(capi.SIGNATURES) == declared_symbols()


def test_library_exports_every_declared_symbol():
    from flashrt_b200_core import capi
    lib = capi.lib()
    for name in declared_symbols():
        assert getattr(lib, name) is not None


def test_library_exports_nothing_beyond_the_header():
    """every extern "C" frt_* symbol of the shipped library is declared in the header: no undeclared
    debug or experiment entry points"""
    import shutil
    import subprocess
    from flashrt_b200_core import capi
    nm = shutil.which("nm")
    if nm is None:
        pytest.skip("no nm")
    out = subprocess.run([nm, "-D", "--defined-only", str(capi.LIB_PATH)], check=True, capture_output=True,
                         text=True).stdout
    exported = sorted({line.split()[-1] for line in out.splitlines() if line.split()[-1].startswith("frt_")})
    assert exported == declared_symbols()


def test_gemm_plan_query():
    """the host-side configuration query: prefill shapes take the CTA-pair kernel, token counts <= 64 the
    weight-streaming form, and the Qwen3-8B o / down projections at 33..64 tokens the cluster split-K"""
    import ctypes as C
    from flashrt_b200_core import capi
    lib = capi.lib()

    def plan(m, n, k):
        cfg, split = C.c_int(0), C.c_int(0)
        assert lib.frt_nvfp4_gemm_plan(m, n, k, C.byref(cfg), C.byref(split)) == 0
        return cfg.value, split.value

    assert plan(4096, 6144, 4096) == (4, 1)
    assert plan(8192, 57344, 8192) == (4, 1)
    assert plan(1, 4096, 4096)[0] == 11 and plan(16, 4096, 4096)[0] == 11
    assert plan(17, 4096, 4096)[0] == 12 and plan(64, 24576, 4096) == (13, 1)
    assert plan(64, 4096, 4096) == (13, 8) and plan(64, 4096, 12288) == (13, 8)
    assert plan(64, 6144, 4096) == (13, 4)
    assert lib.frt_nvfp4_gemm_plan(4, 100, 64, None, None) == -1


def test_host_only_entry_points():
    from flashrt_b200_core import capi
    lib = capi.lib()
    assert lib.frt_nvfp4_sf_swizzled_bytes(129, 4096) == 65536
    assert lib.frt_nvfp4_sf_swizzled_bytes(1, 1024) == 8192
    assert lib.frt_nvfp4_sf_swizzled_bytes(16, 12288) == 98304
    from oracle import nvfp4_oracle as O
    offs = O.sf_offsets(300, 704)
    for r, kb in [(0, 0), (31, 3), (32, 4), (127, 43), (128, 0), (299, 43), (133, 17)]:
        assert lib.frt_nvfp4_sf_offset(r, kb * 16, 704) == offs[r, kb]
    assert lib.frt_error_string(0) == b"ok"
    assert lib.frt_launch_count() >= 0


def test_header_is_plain_c(tmp_path):
    """the boundary is a C ABI: the header must compile as C99 with no C++ or torch types"""
    import shutil
    import subprocess
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "use_header.c"
    src.write_text('#include "flashrt_b200.h"\nint main(void) { return frt_error_string(0) == 0; }\n')
    root = Path(__file__).resolve().parent.parent
    subprocess.run([cc, "-std=c99", "-Wall", "-Werror", f"-I{root / 'include'}", "-fsyntax-only", str(src)], check=True)


def test_host_side_checks_of_the_newer_entry_points():
    """argument checks that return before any device work: workspace size formula, option round trip, the
    exchange producer's null / shape / rank checks, the interleaved layout's shape rule"""
    import ctypes as C
    from flashrt_b200_core import capi
    lib = capi.lib()
    assert lib.frt_nvfp4_grouped_gemm_workspace_bytes(4096, 128) == 16 + 32 * (4096 // 16 + 2 * 128 + 8)
    assert lib.frt_nvfp4_grouped_gemm_workspace_bytes(0, 4) == 0
    for key, value in ((5, 2), (6, 0), (7, 4), (8, 3), (10, 2)):
        prev = lib.frt_set_option(key, value)
        assert lib.frt_set_option(key, prev) == value
    assert lib.frt_set_option(9, 5) == 31 and lib.frt_set_option(9, 31) == 20      # clamped to its floor
    assert lib.frt_set_option(3, 1) == -1                                          # no such key in the shipped library
    nul = (C.c_void_p * 8)()
    one = C.c_void_p(256)
    some = (C.c_void_p * 8)(*([256] * 8))
    f = lib.frt_norm_quant_nvfp4_bcast
    assert f(None, None, None, 1e-6, 1.0, None, None, some, some, 2, 0, 128, 1024, 0, one, some, 2, 0, 1, None) == -1
    assert f(None, one, None, 1e-6, 1.0, one, None, some, some, 2, 0, 128, 1024, 0, one, some, 2, 0, 1, None) == -1
    assert f(None, one, None, 1e-6, 1.0, None, None, some, some, 2, 0, 128, 1000, 0, one, some, 2, 0, 1, None) == -2
    assert f(None, one, None, 1e-6, 1.0, None, None, some, some, 2, 0, 128, 1024, 0, one, some, 9, 0, 1, None) == -4
    assert f(None, one, None, 1e-6, 1.0, None, None, some, some, 2, 0, 128, 1024, 0, one, some, 2, 2, 1, None) == -4
    assert f(None, one, None, 1e-6, 1.0, None, None, nul, some, 2, 0, 128, 1024, 0, one, some, 2, 0, 1, None) == -1
    assert lib.frt_peer_wait(None, 2, 1, None) == -1 and lib.frt_peer_wait(one, 9, 1, None) == -4
    assert lib.frt_nvfp4_repack_interleaved(one, one, 12, 64, None) == -2          # N % 8
    assert lib.frt_nvfp4_repack_interleaved(one, one, 16, 96, None) == -2          # K % 64
