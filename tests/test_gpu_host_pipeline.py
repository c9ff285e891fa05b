"""Decode steps submitted from host tensors through the three-stream pipeline equal the same steps run one by one,
with the compute stage launched eagerly and replayed from a CUDA graph per slot."""

import numpy as np
import pytest
import torch

from helpers import BS, SCALE, bits, decode_case, to_numpy, to_torch
from oracle import kv_cache_ref as R

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("capture", [False, True])
def test_pipelined_host_steps_equal_serial_steps_and_the_oracle(capture):
    from nano_vllm_jax_b200.backends import B200Backend
    from nano_vllm_jax_b200.host_pipeline import HostDecodePipeline
    from nano_vllm_jax_b200.kv_cache import KVCacheStorage

    steps, rows = 5, 24
    c = decode_case(31, 2048, rows, 300, 900)  # its tables cover the lengths of the LAST step
    rng = np.random.default_rng(5)
    k0, v0 = to_torch(c["k_cache"]), to_torch(c["v_cache"])
    backend = B200Backend()
    piped = KVCacheStorage(k0.clone(), v0.clone())
    serial = KVCacheStorage(k0.clone(), v0.clone())
    lens0 = c["seq_lens"].astype(np.int32) - (steps - 1)  # lengths after the first step's append
    host = []
    for s in range(steps):
        q = torch.from_numpy(rng.standard_normal((rows, 1, 8, 256), dtype=np.float32)).to(torch.bfloat16).pin_memory()
        nk = torch.from_numpy(rng.standard_normal((rows, 1, 2, 256), dtype=np.float32)).to(torch.bfloat16).pin_memory()
        nv = torch.from_numpy(rng.standard_normal((rows, 1, 2, 256), dtype=np.float32)).to(torch.bfloat16).pin_memory()
        lens = torch.from_numpy(lens0 + s).pin_memory()
        pos = torch.from_numpy((lens0 + s - 1).astype(np.int32)).pin_memory()
        host.append((q, nk, nv, pos, lens))
    tables = torch.from_numpy(c["tables"]).pin_memory()

    pipe = HostDecodePipeline(backend, piped, rows, tables.shape[1], BS, SCALE, 4, depth=2, capture=capture)
    assert pipe.h2d_bytes_per_step == rows * (8 + 2 + 2) * 256 * 2 + tables.numel() * 4 + rows * 8
    outs = []
    for s, (q, nk, nv, pos, lens) in enumerate(host):
        if s == 2:  # pageable operands of another integer width are converted on the host and copied all the same
            pos, lens = pos.to(torch.int64), lens.to(torch.int64)
        t = pipe.submit(0, q, nk, nv, tables, pos, lens)
        if s >= 1:  # read a result while the next step is in flight
            outs.append(pipe.result(t - 1).clone())
    outs.append(pipe.result(steps - 1).clone())
    with pytest.raises(ValueError):
        pipe.result(0)  # its slot has been reused
    pipe.drain()
    torch.cuda.synchronize()

    d_tab = tables.cuda()
    for s, (q, nk, nv, pos, lens) in enumerate(host):
        md = backend.build_attention_metadata(pos.cuda().view(rows, 1), d_tab, lens.cuda(), BS, False)
        _, ref = backend.write_kv_and_attention(0, q.cuda(), nk.cuda(), nv.cuda(), serial, md, BS, SCALE, 4, False)
        assert torch.equal(outs[s], ref.cpu()), f"step {s}: pipelined result differs from the serial one"
    np.testing.assert_array_equal(bits(to_numpy(piped.k_cache)), bits(to_numpy(serial.k_cache)))
    np.testing.assert_array_equal(bits(to_numpy(piped.v_cache)), bits(to_numpy(serial.v_cache)))

    # and the last step against the oracle on the final cache
    q, nk, nv, pos, lens = host[-1]
    want = R.paged_attention_decode(to_numpy(q), to_numpy(serial.k_cache), to_numpy(serial.v_cache), c["tables"],
                                    lens.numpy(), BS, SCALE, 4, positions=pos.numpy().reshape(rows, 1))
    assert np.abs(outs[-1].numpy().reshape(want.shape) - want).max() <= 2e-3
