"""The C-ABI library loads without a GPU and exports every function include/geoweave_b200.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "geoweave_b200.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gw_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from geoweave_b200 import build as gw_build
    from geoweave_b200 import _lib

    gw_build.build()
    return _lib.load()


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("gw_indexer_topk_fused", "gw_indexer_scores", "gw_topk_exact", "gw_merge_two_topk", "gw_sparse_attn_fwd",
                 "gw_indexer_topk_workspace_bytes", "gw_strerror"):
        assert must in names


def test_every_declared_symbol_is_exported(lib):
    raw = ctypes.CDLL(lib._name)
    for name in declared_functions():
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header(lib):
    from geoweave_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_functions()


def test_no_compute_calls_needed_for_metadata(lib):
    assert lib.gw_abi_version() >= 1
    assert b"unsupported" in lib.gw_strerror(-2)
    assert lib.gw_indexer_topk_workspace_bytes(1, 4164, 4164, 4, 64, 1024) > 0
    assert lib.gw_indexer_topk_workspace_bytes(1, 0, 10, 4, 64, 4) == 0


def test_argument_validation_happens_before_any_launch(lib):
    # null pointers / bad sizes are refused on the host, so this is safe without a device
    assert lib.gw_topk_exact(None, 0, 1, 8, 8, 4, None, None, None, None) == -1
    assert lib.gw_merge_two_topk(None, None, 4, None, None, 4, 0, 0, 1, 4, None, None, None) == -1
    assert lib.gw_indexer_topk_fused(None, None, None, 1, 1, 8, 8, 4, 64, 0.125, 4, None, None, None, 0, None, None) == -1


def test_product_package_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "geoweave_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in src.replace("the oracle", ""), f"{f} refers to the oracle"


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 on its own, and a C program that takes the address of an
    entry point must link against the library."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler here")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "use_header.c"
    src.write_text('#include "geoweave_b200.h"\n'
                   "int main(void) { return gw_abi_version() > 0 && gw_strerror(0) != 0 ? 0 : 1; }\n")
    res = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-I", os.path.join(root, "include"), "-fsyntax-only", str(src)],
                         capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    lib_dir = os.path.join(root, "geoweave_b200")
    exe = tmp_path / "use_header"
    res = subprocess.run([gcc, "-std=c99", "-I", os.path.join(root, "include"), str(src), "-o", str(exe), "-L", lib_dir,
                          "-lgeoweave_b200", f"-Wl,-rpath,{lib_dir}"], capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    assert subprocess.run([str(exe)]).returncode == 0   # metadata calls only: no GPU needed
