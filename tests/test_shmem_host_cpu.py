"""Argument checks of the host-side put / get wrappers, on emulated CPU ranks (no copy is issued: both calls
must refuse before touching memory)."""
import pytest
import torch

from triton_distributed_b200.runtime import LocalWorld
from triton_distributed_b200.runtime import shmem_host as SH


def _symm(n):
    lw = LocalWorld(2, torch.device("cpu"))
    return lw.heap(0).empty((n,), torch.float32)


def test_getmem_rejects_destination_larger_than_symmetric_source():
    src = _symm(16)
    with pytest.raises(ValueError, match="larger than the symmetric source"):
        SH.getmem_on_stream(torch.empty(32), src, 1)


def test_getmem_rejects_non_contiguous_destination():
    src = _symm(16)
    dst = torch.empty(8, 4)[:, :2]
    assert not dst.is_contiguous()
    with pytest.raises(ValueError, match="contiguous destination"):
        SH.getmem_on_stream(dst, src, 1)


def test_putmem_rejects_source_larger_than_symmetric_destination():
    dst = _symm(16)
    with pytest.raises(ValueError, match="larger than the symmetric destination"):
        SH.putmem_on_stream(dst, torch.empty(32), 1)
    # a non-contiguous source is measured by its own element count, not by its storage
    with pytest.raises(ValueError, match="larger than the symmetric destination"):
        SH.putmem_on_stream(dst, torch.empty(64, 2)[:, 0], 1)
