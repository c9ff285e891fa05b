"""The recipe that builds the reference's own FP32 CUDA kernels as a checker (oracle/build_ref.py)."""

import ctypes

import pytest

from oracle import build_ref as B


def test_extract_function_takes_exactly_one_definition():
    text = "int a() { return 1; }\n__global__ void Foo(\n int x) {\n  if (x) { x = 2; }\n}\nint b() { return 3; }\n"
    got = B.extract_function(text, r"__global__\s+void\s+Foo\s*\(")
    assert got.startswith("__global__ void Foo(") and got.endswith("\n}") and "int b" not in got and "int a" not in got
    assert got.count("{") == got.count("}")
    with pytest.raises(RuntimeError):
        B.extract_function(text, r"void\s+Missing\s*\(")


def test_generated_source_holds_the_three_reference_functions_and_the_launchers():
    if not B.reference_source().exists():
        pytest.skip("no reference checkout on this machine")
    src = B.generated_source()
    for name, _ in B.WANTED:
        assert src.count(name) >= 1
    assert "extern \"C\" int ref_fp32_kv_append" in src and "extern \"C\" int ref_fp32_paged_decode" in src
    assert "XLA_FFI" not in src  # only the kernels are taken, none of the handler code
    assert src.count("{") == src.count("}")


def test_checker_library_builds_and_exports_its_entry_points():
    path = B.build()
    if path is None:
        pytest.skip("no reference checkout and no library built earlier")
    lib = ctypes.CDLL(str(path))
    assert hasattr(lib, "ref_fp32_kv_append") and hasattr(lib, "ref_fp32_paged_decode")
