"""Pins the floating-point oracle, and this library's kernels, to the reference project's own CUDA kernels.

`oracle/_ref/libref_fp32.so` holds the reference's `Fp32KvAppendKernel` and
`Fp32PagedDecodeAttentionKernel` (nanovllm_jax/kernels/csrc/fp32_kv_append.cu:801-957) compiled
unchanged by `oracle/build_ref.py`.  The reference's tests hold those kernels to its pure-JAX
functions at rtol = atol = 2e-5 for attention and exactly for the append
(tests/test_cuda_fp32_ffi.py:197-290 and :120-193 of the reference); the same bounds are used here
between the reference kernels and (a) the NumPy oracle, (b) this library's kernels, on the inputs
of those reference tests and on seeded random ones.
"""

import ctypes
import os

import numpy as np
import pytest
import torch

from helpers import BS, SCALE, bits, decode_case, to_numpy, to_torch
from oracle import kv_cache_ref as R
from oracle.build_ref import LIB_PATH

pytestmark = pytest.mark.gpu

REF_TOL = 2e-5  # the reference's own bound between its kernel and its pure-JAX function


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(LIB_PATH):
        pytest.skip("oracle/_ref/libref_fp32.so has not been built (python -m oracle.build_ref needs the reference checkout)")
    lib = ctypes.CDLL(str(LIB_PATH))
    p, i64 = ctypes.c_void_p, ctypes.c_int64
    lib.ref_fp32_kv_append.argtypes = [p] * 9 + [i64] * 4 + [p]
    lib.ref_fp32_kv_append.restype = ctypes.c_int
    lib.ref_fp32_paged_decode.argtypes = [p] * 9 + [i64] * 7 + [p]
    lib.ref_fp32_paged_decode.restype = ctypes.c_int
    return lib


def _stream():
    return torch.cuda.current_stream().cuda_stream


def ref_decode(lib, q, k, v, indptr, indices, last, lens, scale):
    """The reference kernel on fp32 CUDA tensors: q [B, Hq, D] -> [B, Hq, D]."""
    out = torch.full_like(q, float("nan"))
    sc = torch.tensor([scale], dtype=torch.float32, device=q.device)
    rc = lib.ref_fp32_paged_decode(q.data_ptr(), k.data_ptr(), v.data_ptr(), indptr.data_ptr(), indices.data_ptr(),
                                   last.data_ptr(), lens.data_ptr(), sc.data_ptr(), out.data_ptr(), q.shape[0], q.shape[1],
                                   k.shape[0], k.shape[1], k.shape[2], k.shape[3], indices.numel(), _stream())
    assert rc == 0, f"reference decode kernel launch failed ({rc})"
    torch.cuda.synchronize()
    return out


def _linspace_case(page_size, width, hq, hkv, d):
    """Inputs of the reference's own decode test (tests/test_cuda_fp32_ffi.py:212-246 of the reference)."""
    batch = 2
    pages = width * batch + 1
    n = pages * page_size * hkv * d
    lens = np.array([page_size + 1, width * page_size - 1], np.int32)
    tables = np.array([[pages - 1, 1, 2][:width], [0, 3, 4][:width]], np.int32)
    k = np.linspace(-0.3, 0.4, n, dtype=np.float32).reshape(pages, page_size, hkv, d)
    v = np.linspace(0.2, 0.9, n, dtype=np.float32).reshape(pages, page_size, hkv, d)
    q = np.linspace(-0.5, 0.5, batch * hq * d, dtype=np.float32).reshape(batch, hq, d)
    return q, k, v, tables, lens, float(1.0 / np.sqrt(d))


def _random_case(seed, pages, page_size, hq, hkv, d, lens):
    rng = np.random.default_rng(seed)
    lens = np.asarray(lens, np.int32)
    need = -(-lens // page_size)
    width = int(need.max())
    perm = rng.permutation(pages)
    tables = np.zeros((len(lens), width), np.int32)
    o = 0
    for b in range(len(lens)):
        tables[b, :need[b]] = perm[o:o + need[b]]
        o += need[b]
    k = rng.standard_normal((pages, page_size, hkv, d), dtype=np.float32)
    v = rng.standard_normal((pages, page_size, hkv, d), dtype=np.float32)
    q = rng.standard_normal((len(lens), hq, d), dtype=np.float32)
    return q, k, v, tables, lens, float(1.0 / np.sqrt(d))


CASES = [
    ("reference test, P4 W3 Hq4 Hkv2 D8", lambda: _linspace_case(4, 3, 4, 2, 8)),
    ("reference test, P16 W2 Hq8 Hkv2 D256", lambda: _linspace_case(16, 2, 8, 2, 256)),
    ("random, model shape, lens 1..2000", lambda: _random_case(31, 700, 16, 8, 2, 256, [1, 15, 16, 17, 700, 1999, 2000, 333])),
    ("random, P8 Hq6 Hkv3 D64", lambda: _random_case(32, 300, 8, 6, 3, 64, [5, 64, 777, 1200])),
]


@pytest.mark.parametrize("name,make", CASES, ids=[c[0] for c in CASES])
def test_decode_oracle_and_library_match_the_reference_kernel(ref, name, make):
    from nano_vllm_jax_b200.kernels import paged_kv as K
    q, k, v, tables, lens, scale = make()
    indices, indptr = R.dense_block_tables_to_kv_indptr(tables)
    last = R.kv_last_page_len_from_seq_lens(lens, k.shape[1])
    tq, tk, tv = to_torch(q), to_torch(k), to_torch(v)
    t_indices, t_indptr, t_last, t_lens = to_torch(indices), to_torch(indptr), to_torch(last), to_torch(lens)
    want = to_numpy(ref_decode(ref, tq, tk, tv, t_indptr, t_indices, t_last, t_lens, scale))
    assert not np.isnan(want).any()
    # (a) the NumPy restatement of the reference's pure function, fp32 mode
    oracle = R.paged_decode_attention_gqa_nhd(q, k, v, indptr, indices, last, lens, scale, mode="fp32")
    np.testing.assert_allclose(oracle, want, rtol=REF_TOL, atol=REF_TOL)
    # (b) this library's kernel on the same fp32 cache (the generic kernel serves fp32 caches)
    got = to_numpy(K.paged_decode_attention_gqa_nhd(tq, tk, tv, t_indptr, t_indices, t_last, t_lens, scale))
    np.testing.assert_allclose(got, want, rtol=REF_TOL, atol=REF_TOL)
    # the dense block-table entry point as well
    got2 = to_numpy(K.paged_decode_attention(tq, tk, tv, to_torch(tables), t_lens, scale))
    np.testing.assert_allclose(got2, want, rtol=REF_TOL, atol=REF_TOL)


@pytest.mark.parametrize("variant", [2, 3])
def test_bf16_streaming_kernels_against_the_reference_kernel_on_the_same_values(ref, variant):
    """The bf16 decode kernels (CUDA-core pipelined, tensor-core TMA) against the reference kernel fed the same
    numbers widened to fp32: what differs is only the arithmetic, and it must stay inside 2e-3 (contract 2e-2)."""
    from nano_vllm_jax_b200.kernels import paged_kv as K
    c = decode_case(33, 1200, 12, 1, 2040, empty_rows=(4,))
    k32 = np.asarray(c["k_cache"][0]).astype(np.float32)
    v32 = np.asarray(c["v_cache"][0]).astype(np.float32)
    q32 = np.asarray(c["q"][:, 0]).astype(np.float32)
    lens = c["seq_lens"]
    indices, indptr = R.dense_block_tables_to_kv_indptr(c["tables"])
    last = R.kv_last_page_len_from_seq_lens(lens, BS)
    want = to_numpy(ref_decode(ref, to_torch(q32), to_torch(k32), to_torch(v32), to_torch(indptr), to_torch(indices),
                               to_torch(last), to_torch(lens), SCALE))
    got = to_numpy(K.paged_decode_attention(to_torch(c["q"][:, 0]).contiguous(), to_torch(c["k_cache"][0]),
                                            to_torch(c["v_cache"][0]), to_torch(c["tables"]), to_torch(lens), SCALE,
                                            variant=variant))
    active = lens > 0
    assert np.abs(got[active] - want[active]).max() <= 2e-3
    assert not got[~active].any()


def test_append_oracle_and_library_match_the_reference_kernel_exactly(ref):
    from nano_vllm_jax_b200.kernels import paged_kv as K
    rng = np.random.default_rng(34)
    pages, P, hkv, d, batch, width = 40, 16, 2, 256, 5, 6
    k0 = rng.standard_normal((pages, P, hkv, d), dtype=np.float32)
    v0 = rng.standard_normal((pages, P, hkv, d), dtype=np.float32)
    tables = rng.permutation(pages)[: batch * width].reshape(batch, width).astype(np.int32)
    # ragged rows of 1..7 new tokens at arbitrary start positions, a few of them masked out
    rows, pos = [], []
    for b in range(batch):
        start, n = int(rng.integers(0, 60)), int(rng.integers(1, 8))
        rows += [b] * n
        pos += list(range(start, start + n))
    rows, pos = np.array(rows, np.int32), np.array(pos, np.int32)
    nnz = len(rows)
    mask = (rng.random(nnz) > 0.2).astype(np.int32)
    ak = rng.standard_normal((nnz, hkv, d), dtype=np.float32)
    av = rng.standard_normal((nnz, hkv, d), dtype=np.float32)
    indices, indptr = R.dense_block_tables_to_kv_indptr(tables)
    last = np.full(batch, P, np.int32)
    for vm in (None, mask):
        rk, rv = to_torch(k0), to_torch(v0)
        t = [to_torch(x) for x in (ak, av, rows, pos, indices, indptr)]
        tm = None if vm is None else to_torch(vm)
        rc = ref.ref_fp32_kv_append(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), rk.data_ptr(),
                                    rv.data_ptr(), t[4].data_ptr(), t[5].data_ptr(), None if tm is None else tm.data_ptr(),
                                    nnz, P, hkv, d, _stream())
        assert rc == 0
        torch.cuda.synchronize()
        ok, ov = R.kv_append_paged_nhd(ak, av, rows, pos, k0, v0, indices, indptr, last, valid_mask=vm)
        np.testing.assert_array_equal(bits(ok), bits(to_numpy(rk)))
        np.testing.assert_array_equal(bits(ov), bits(to_numpy(rv)))
        lk, lv = to_torch(k0), to_torch(v0)
        K.kv_append_paged_nhd(t[0], t[1], t[2], t[3], lk, lv, t[4], t[5], to_torch(last), valid_mask=tm)
        torch.cuda.synchronize()
        assert torch.equal(lk, rk) and torch.equal(lv, rv)
