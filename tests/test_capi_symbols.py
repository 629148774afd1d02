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
