"""The C-ABI library builds for sm_100a, loads, and exports every declared symbol (no GPU needed)."""

import ctypes
import re
from pathlib import Path

from nano_vllm_jax_b200 import _lib, build

ROOT = Path(__file__).resolve().parents[1]


def _declared():
    text = (ROOT / "include" / "nvj_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nvj_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = build.build()
    lib = ctypes.CDLL(str(path))
    names = _declared()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} declared in nvj_b200.h but not exported"


def test_ctypes_signatures_cover_the_header():
    assert sorted(_lib.SIGNATURES) == _declared()


def test_header_is_plain_c_and_a_c_program_links_against_the_library(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 with nothing but the standard headers, and a C program
    that names an entry point of every group links against the shared library (no CUDA or torch types involved)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:  # pragma: no cover
        import pytest
        pytest.skip("gcc not available")
    so = build.build()
    src = tmp_path / "use_abi.c"
    src.write_text(
        '#include "nvj_b200.h"\n'
        "int main(void) {\n"
        "  int (*fns[])() = {(int (*)())nvj_kv_append, (int (*)())nvj_paged_decode_fused_append,\n"
        "                    (int (*)())nvj_paged_prefill_packed, (int (*)())nvj_hybrid_snapshot,\n"
        "                    (int (*)())nvj_qk_norm_rope_kv_append, (int (*)())nvj_p2p_allgather_i32};\n"
        "  return nvj_abi_version() == 1 && sizeof(fns) > 0 && nvj_kv_append(0, 0, 0, 0, 0, 0, 0, 0, -1, 1, 0, 0, 0, 16, 2, 256, 0, 0) == NVJ_ERR_INVALID_ARGUMENT ? 0 : 1;\n"
        "}\n")
    exe = tmp_path / "use_abi"
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-Wno-strict-prototypes", "-I", str(ROOT / "include"),
                        str(src), "-o", str(exe), str(so), f"-Wl,-rpath,{so.parent}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_status_strings_and_version():
    lib = _lib.load()
    assert lib.nvj_abi_version() == 1
    assert lib.nvj_status_string(0) == b"ok"
    assert b"workspace" in lib.nvj_status_string(-4)


def test_argument_checks_run_before_any_launch():
    lib = _lib.load()
    # negative sizes / null pointers are rejected on the host, no device needed
    assert lib.nvj_kv_append(None, None, 0, None, None, None, 0, 0, -1, 1, None, None, 0, 16, 2, 256, None, None) == -1
    assert lib.nvj_kv_append(None, None, 0, None, None, None, 0, 0, 2, 2, None, None, 0, 16, 2, 256, None, None) == -1
    assert lib.nvj_kv_append(None, None, 7, None, None, None, 0, 0, 2, 2, None, None, 0, 16, 2, 256, None, None) == -2
    assert lib.nvj_row_argmax(None, 0, 8, None, None) == 0
    assert lib.nvj_copy_blocks(None, None, 1, 4, 64, 256, None, None, 0, None, None) == 0
    assert lib.nvj_paged_decode_workspace_init(None, 0, None) == -4


def test_no_product_module_imports_the_oracle():
    for p in (ROOT / "nano_vllm_jax_b200").rglob("*.py"):
        assert "oracle" not in p.read_text(), f"{p} mentions the oracle"
