"""Builds the reference project's own FP32 CUDA kernels as a checker library.  TEST INFRASTRUCTURE ONLY.

The reference ships two hand-written CUDA kernels for this path,
`Fp32KvAppendKernel` and `Fp32PagedDecodeAttentionKernel`
(nanovllm_jax/kernels/csrc/fp32_kv_append.cu:801-841, 843-957, with the helper
`MultiplyLikeXlaDot` at :29-31).  They are plain `__global__` functions; only the
XLA-FFI handlers around them need a header that is not installed here.  This
recipe reads the three function bodies out of the reference checkout at build
time, puts them between a few includes and the small launcher below (same launch
geometry as the reference handlers, fp32_kv_append.cu:1601-1603 and 1667-1673),
compiles the result with nvcc for sm_100a into `oracle/_ref/libref_fp32.so`, and
deletes the generated source again.  No reference text is stored in this
repository; `oracle/_ref/` is not tracked.

The library is the pin for the floating-point part of the oracle: the tests hold
`oracle.kv_cache_ref.paged_decode_attention_gqa_nhd(mode="fp32")`,
`oracle.kv_cache_ref.kv_append_paged_nhd` and this project's kernels to the
reference kernels at the reference's own tolerance
(tests/test_cuda_fp32_ffi.py:197-290 of the reference: 2e-5, append exact).

    python -m oracle.build_ref            # build if the reference checkout is present
"""

from __future__ import annotations

import os
import re
import shutil
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
LIB_PATH = OUT_DIR / "libref_fp32.so"
SOURCE_IN_REFERENCE = Path("nanovllm_jax/kernels/csrc/fp32_kv_append.cu")

WANTED = (
    ("MultiplyLikeXlaDot", r"__device__\s+inline\s+float\s+MultiplyLikeXlaDot\s*\("),
    ("Fp32KvAppendKernel", r"__global__\s+void\s+Fp32KvAppendKernel\s*\("),
    ("Fp32PagedDecodeAttentionKernel", r"__global__\s+void\s+Fp32PagedDecodeAttentionKernel\s*\("),
)

PROLOGUE = """// GENERATED at build time; not tracked.  Kernel bodies come from the reference checkout.
#include <cfloat>
#include <cmath>
#include <cstdint>
#include <cuda_runtime_api.h>
namespace {
"""

# The launchers repeat what the reference handlers do around the kernels: 256 threads, one thread per
# appended element; one CTA per (row, query head) with (max_kv_len + 256) floats of dynamic shared memory.
LAUNCHER = """
}  // namespace

extern "C" int ref_fp32_kv_append(const float* append_key, const float* append_value, const int32_t* batch_indices,
                                  const int32_t* positions, float* k_cache, float* v_cache, const int32_t* kv_indices,
                                  const int32_t* kv_indptr, const int32_t* valid_mask, int64_t nnz_tokens,
                                  int64_t page_size, int64_t num_kv_heads, int64_t head_dim, void* stream) {
  const int64_t total = nnz_tokens * num_kv_heads * head_dim;
  if (total == 0) return 0;
  const int threads = 256;
  const int blocks = static_cast<int>((total + threads - 1) / threads);
  Fp32KvAppendKernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      append_key, append_value, batch_indices, positions, k_cache, v_cache, kv_indices, kv_indptr, valid_mask,
      nnz_tokens, page_size, num_kv_heads, head_dim);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int ref_fp32_paged_decode(const float* q, const float* k_cache, const float* v_cache, const int32_t* kv_indptr,
                                     const int32_t* kv_indices, const int32_t* kv_last_page_len, const int32_t* seq_lens,
                                     const float* softmax_scale, float* out, int64_t batch, int64_t num_q_heads,
                                     int64_t num_pages, int64_t page_size, int64_t num_kv_heads, int64_t head_dim,
                                     int64_t total_page_entries, void* stream) {
  if (batch <= 0) return 0;
  const int64_t max_pages_per_sequence = total_page_entries / batch;
  const int64_t max_kv_len = max_pages_per_sequence * page_size;
  const int threads = 256;
  const size_t shared_bytes = static_cast<size_t>(max_kv_len + threads) * sizeof(float);
  if (shared_bytes > 48 * 1024) return -1;  // the reference asks for no opt-in: longer tables cannot launch
  Fp32PagedDecodeAttentionKernel<<<static_cast<int>(batch * num_q_heads), threads, shared_bytes,
                                   static_cast<cudaStream_t>(stream)>>>(
      q, k_cache, v_cache, kv_indptr, kv_indices, kv_last_page_len, seq_lens, softmax_scale, out, batch, num_q_heads,
      num_pages, page_size, num_kv_heads, head_dim, max_pages_per_sequence, max_kv_len);
  return static_cast<int>(cudaGetLastError());
}
"""


def reference_root() -> Path:
    return Path(os.environ.get("NVJ_REFERENCE_ROOT", "/root/reference"))


def reference_source() -> Path:
    return reference_root() / SOURCE_IN_REFERENCE


def extract_function(text: str, start_pattern: str) -> str:
    """The text of one function definition: from the match of `start_pattern` to its closing brace."""
    m = re.search(start_pattern, text)
    if m is None:
        raise RuntimeError(f"pattern {start_pattern!r} not found in the reference source")
    i = text.index("{", m.end())
    depth = 0
    for j in range(i, len(text)):
        if text[j] == "{":
            depth += 1
        elif text[j] == "}":
            depth -= 1
            if depth == 0:
                return text[m.start():j + 1]
    raise RuntimeError("unbalanced braces in the reference source")


def generated_source() -> str:
    text = reference_source().read_text()
    parts = [extract_function(text, pattern) for _, pattern in WANTED]
    return PROLOGUE + "\n\n".join(parts) + "\n" + LAUNCHER


def build(force: bool = False) -> Path | None:
    """Compile the checker library; returns its path, or None when there is no reference checkout to build from
    (a library built earlier is then used as it is)."""
    src = reference_source()
    if not src.exists():
        return LIB_PATH if LIB_PATH.exists() else None
    if (not force and LIB_PATH.exists() and LIB_PATH.stat().st_mtime > src.stat().st_mtime
            and LIB_PATH.stat().st_mtime > Path(__file__).stat().st_mtime):
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    OUT_DIR.mkdir(exist_ok=True)
    gen = OUT_DIR / "ref_fp32_kernels.cu"
    gen.write_text(generated_source())
    try:
        proc = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-shared",
                               "-Xcompiler", "-fPIC", "-o", str(LIB_PATH), str(gen)], capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed on the reference kernels:\n" + proc.stdout + proc.stderr)
    finally:
        gen.unlink(missing_ok=True)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force=True))
