"""`paged_kv.CopyList` on the host: the checks it makes before anything reaches the library."""

import pytest
import torch

from nano_vllm_jax_b200.kernels.paged_kv import CopyList


def test_sizes_dtypes_and_layouts_are_checked_when_the_list_is_built():
    a, b = torch.zeros(8, dtype=torch.int32), torch.zeros(8, dtype=torch.int32)
    lst = CopyList([a], [b])
    assert lst.n == 1
    with pytest.raises(ValueError):
        CopyList([a], [torch.zeros(4, dtype=torch.int32)])            # another size
    with pytest.raises(ValueError):
        CopyList([a], [torch.zeros(8, dtype=torch.float32)])          # same bytes, another dtype
    with pytest.raises(ValueError):
        CopyList([a], [torch.zeros((8, 2), dtype=torch.int32)[:, 0]])  # strided source
    with pytest.raises(ValueError):
        CopyList([a, a], [b])


def test_a_replaced_source_must_match_the_slot_it_replaces():
    a, b = torch.zeros((4, 2), dtype=torch.bfloat16), torch.ones((4, 2), dtype=torch.bfloat16)
    lst = CopyList([a], [a])
    lst.set_source(0, b)
    lst.set_source(0, b.view(8))          # the byte count is what counts
    with pytest.raises(ValueError):
        lst.set_source(0, torch.ones(7, dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        lst.set_source(0, torch.ones((8, 2), dtype=torch.bfloat16)[:, 0])
