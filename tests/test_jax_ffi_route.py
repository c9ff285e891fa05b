"""The jax.ffi route (kernels/jax_ffi.py + csrc/xla_ffi): what can be checked without JAX.

JAX and the XLA FFI headers are not installed where this library is built, so the adapter is not compiled and
these checks are structural: the Python module imports and fails the way the reference's optional routes do, every
target it registers has a handler in the adapter source, and the adapter calls only entry points that
include/nvj_b200.h declares.
"""

import importlib.util
import re
from pathlib import Path

import pytest

from nano_vllm_jax_b200.kernels import jax_ffi

ROOT = Path(__file__).resolve().parents[1]
HANDLERS = (ROOT / "nano_vllm_jax_b200" / "csrc" / "xla_ffi" / "handlers.cc").read_text()
HEADER = (ROOT / "include" / "nvj_b200.h").read_text()


def test_every_registered_target_has_a_handler_and_the_other_way_round():
    defined = set(re.findall(r'extern "C" XLA_FFI_Error\* (\w+)\(XLA_FFI_CallFrame\* frame\)', HANDLERS))
    assert defined == set(jax_ffi.TARGETS.values())
    assert len(set(jax_ffi.TARGETS)) == len(jax_ffi.TARGETS)


def test_adapter_calls_only_declared_entry_points_with_the_declared_number_of_arguments():
    header = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    declared = {}
    for m in re.finditer(r"\b(nvj_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", header, flags=re.S):
        args = m.group(2).strip()
        declared[m.group(1)] = 0 if args in ("", "void") else args.count(",") + 1
    body = re.sub(r"//[^\n]*", "", HANDLERS)
    used = set(re.findall(r"\b(nvj_[a-z0-9_]+)\s*\(", body))
    assert used and used <= set(declared), used - set(declared)
    for name in used:
        for m in re.finditer(r"\b" + name + r"\s*\(", body):
            depth, i, commas = 1, m.end(), 0
            while depth:  # walk to the call's closing parenthesis, counting the commas at its own level
                ch = body[i]
                if ch == "(":
                    depth += 1
                elif ch == ")":
                    depth -= 1
                elif ch == "," and depth == 1:
                    commas += 1
                i += 1
            assert commas + 1 == declared[name], f"{name}: {commas + 1} arguments passed, {declared[name]} declared"


def test_without_jax_the_route_reports_itself_unavailable():
    if importlib.util.find_spec("jax") is not None:
        pytest.skip("JAX is installed here: the route is exercised by its own tests")
    with pytest.raises(jax_ffi.KernelBackendUnavailable, match="needs JAX"):
        jax_ffi.row_argmax([[1.0, 2.0]])
    with pytest.raises(jax_ffi.KernelBackendUnavailable):
        jax_ffi.build_xla_ffi_library()
