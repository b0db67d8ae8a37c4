"""The VMM heap's set-up on CPU ranks (gloo) against a fake of the native library: one rank's map call fails.
Every rank must then run the same sequence of collectives (no rank is left inside one the others never enter)
and all of them must give the segment up together, with what they built released."""
import json
import sys

import torch
import torch.distributed as dist

from triton_distributed_b200 import _lib
from triton_distributed_b200.runtime import heap as H
from triton_distributed_b200.runtime import initialize_distributed


class FakeLib:
    """Answers the symmetric-heap entry points without a GPU; `fail_map_on` makes tdist_symm_map fail there."""

    def __init__(self, rank, fail_map_on):
        self.rank, self.fail_map_on = rank, fail_map_on
        self.released, self.unmapped, self.freed = [], [], []
        self._next = 100 * (rank + 1)

    def _set(self, ref, value):
        ref._obj.value = value
        return 0

    def tdist_symm_caps(self, dev, caps):
        return self._set(caps, 3)

    def tdist_symm_round_size(self, dev, nbytes, world, out):
        return self._set(out, (nbytes.value + 4095) // 4096 * 4096)

    def tdist_symm_create(self, dev, nbytes, handle, fd):
        self._next += 1
        self._set(handle, self._next)
        return self._set(fd, 3)

    def tdist_symm_import(self, fd, handle):
        self._next += 1
        return self._set(handle, self._next)

    def tdist_symm_reserve(self, nbytes, va):
        return self._set(va, 1 << 40)

    def tdist_symm_map(self, va, nbytes, handle, dev):
        return 1 if self.rank == self.fail_map_on else 0

    def tdist_symm_unmap(self, va, nbytes):
        self.unmapped.append(va.value)
        return 0

    def tdist_symm_address_free(self, va, nbytes):
        self.freed.append(va.value)
        return 0

    def tdist_symm_release(self, handle):
        self.released.append(handle.value)
        return 0

    def tdist_last_error(self):
        return b"fake map failure"


def main():
    group = initialize_distributed(seed=0)
    rank, world = dist.get_rank(), dist.get_world_size()
    fake = FakeLib(rank, fail_map_on=world - 1)
    _lib.lib = lambda: fake
    H.exchange_fds = lambda group, fds: [[7] for _ in range(world)]
    H.close_fds = lambda fds: None
    calls = []
    real_all_reduce, real_gather = dist.all_reduce, dist.all_gather_object

    def logged_all_reduce(t, *a, **k):
        calls.append("all_reduce")
        return real_all_reduce(t, *a, **k)

    def logged_gather(*a, **k):
        calls.append("all_gather_object")
        return real_gather(*a, **k)

    dist.all_reduce, dist.all_gather_object = logged_all_reduce, logged_gather
    heap = object.__new__(H.SymmetricHeap)
    heap.group, heap.rank, heap.world = group, rank, world
    heap.device, heap.backend, heap.use_nvls = torch.device("cpu"), "auto", True
    seg, err = heap._try_vmm(1 << 20)
    dist.all_reduce, dist.all_gather_object = real_all_reduce, real_gather
    mine = {"none": seg is None, "err": err, "calls": calls, "released": len(fake.released), "freed": len(fake.freed),
            "unmapped": len(fake.unmapped)}
    everyone = [None] * world
    dist.all_gather_object(everyone, mine, group=group)
    if rank == 0:
        print("RESULT " + json.dumps(everyone), flush=True)
    dist.barrier(group)
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
