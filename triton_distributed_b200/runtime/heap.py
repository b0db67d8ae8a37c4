"""Symmetric heap: the same allocation at the same offset on every rank, with every peer's copy
mapped into this process.

Three backings share one interface:

``vmm``    cuMemCreate segments exported as POSIX descriptors and mapped back to back into one
           reserved address range (native part: ``csrc/runtime/symm_heap.cc``); optional NVLS
           multicast mapping over the same memory (``TDIST_NVLS=1``).
``ipc``    cudaMalloc + cudaIpc handles, for systems that refuse descriptor export.
``local``  all ranks emulated inside one process on one device (``LocalWorld``): used to run a
           single rank's fused kernel against prepared peer buffers on a single GPU, and by the
           CPU tests (plain host tensors).

It stands in for the reference's NVSHMEM symmetric heap and its Python shim
(reference shmem/nvshmem_bind/pynvshmem/python/pynvshmem/__init__.py:93-171:
``nvshmem_create_tensor``, ``nvshmem_create_tensor_list_intra_node``, ``symm_tensor``).
"""
from __future__ import annotations

import atexit
import ctypes as C
import math
import os
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _lib
from .fd_exchange import close_fds, exchange_fds

ALIGN = 1024  # every symmetric object starts on a 1 KiB boundary (TMA swizzle atoms, 16 B bulk copies)


def _default_segment_bytes() -> int:
    return int(os.environ.get("TDIST_SYMM_HEAP_BYTES", str(1 << 30)))


class _RawCudaBuffer:
    """Minimal ``__cuda_array_interface__`` carrier so torch can wrap a mapped address range."""

    def __init__(self, ptr: int, nbytes: int, keepalive=None):
        self._keepalive = keepalive
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None,
        }


def tensor_from_ptr(ptr: int, nbytes: int, device: torch.device, keepalive=None) -> torch.Tensor:
    """uint8 tensor over ``nbytes`` of device memory at ``ptr`` (no copy, no ownership)."""
    return torch.as_tensor(_RawCudaBuffer(ptr, nbytes, keepalive), device=device)


@dataclass
class SymmTensor:
    """One symmetric object: ``local`` is this rank's copy, ``peers[r]`` rank r's copy as mapped
    here (``peers[rank] is local``), ``mc`` the NVLS multicast alias when the heap has one."""

    local: torch.Tensor
    peers: List[torch.Tensor]
    rank: int
    mc: Optional[torch.Tensor] = None

    @property
    def world(self) -> int:
        return len(self.peers)

    @property
    def ptrs(self) -> List[int]:
        return [t.data_ptr() for t in self.peers]

    def ptr_array(self):
        return _lib.ptr_array(self.ptrs)

    def half_ptr_arrays(self):
        """For a symmetric object whose leading dimension is the call parity (size 2): the two ctypes
        pointer arrays (one per parity) of every rank's half, built once and cached — slicing tensors
        and boxing pointers on every launch costs tens of microseconds."""
        cached = getattr(self, "_half_arrays", None)
        if cached is None:
            cached = tuple(_lib.ptr_array([t[h].data_ptr() for t in self.peers]) for h in range(2))
            object.__setattr__(self, "_half_arrays", cached)
        return cached

    def cached_ptr_array(self):
        cached = getattr(self, "_ptr_array", None)
        if cached is None:
            cached = _lib.ptr_array(self.ptrs)
            object.__setattr__(self, "_ptr_array", cached)
        return cached

    def symm_at(self, peer: int) -> torch.Tensor:
        return self.peers[peer]

    def view_as(self, shape: Sequence[int], dtype: torch.dtype, offset_bytes: int = 0) -> "SymmTensor":
        """Reinterpret a prefix of the object (all copies alike)."""
        nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()

        def cut(t: torch.Tensor) -> torch.Tensor:
            if t.numel() == 0:  # host heap: copies of other processes are not mapped
                return torch.empty(0, dtype=dtype)
            flat = t.reshape(-1).view(torch.uint8)
            return flat[offset_bytes: offset_bytes + nbytes].view(dtype).view(*shape)

        local = cut(self.local)
        return SymmTensor(local, [local if t is self.local else cut(t) for t in self.peers], self.rank,
                          None if self.mc is None else cut(self.mc))


class _Segment:
    def __init__(self, nbytes: int, local_u8: torch.Tensor, peer_u8: List[torch.Tensor], mc_u8=None, cleanup=None):
        self.nbytes = nbytes
        self.local_u8 = local_u8
        self.peer_u8 = peer_u8
        self.mc_u8 = mc_u8
        self.offset = 0
        self.cleanup = cleanup

    def take(self, nbytes: int) -> Optional[int]:
        start = (self.offset + ALIGN - 1) // ALIGN * ALIGN
        if start + nbytes > self.nbytes:
            return None
        self.offset = start + nbytes
        return start


class SymmetricHeap:
    """Collective allocator of symmetric tensors for one process group.

    Every rank must call :meth:`empty` / :meth:`zeros` in the same order with the same sizes.
    """

    def __init__(self, group=None, device: Optional[torch.device] = None, segment_bytes: Optional[int] = None,
                 backend: Optional[str] = None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self.segment_bytes = segment_bytes or _default_segment_bytes()
        if backend is None:
            backend = os.environ.get("TDIST_HEAP_BACKEND", "auto")
        if self.device.type == "cpu":
            backend = "host"
        self.backend = backend
        self.use_nvls = os.environ.get("TDIST_NVLS", "0") == "1"
        self._segments: List[_Segment] = []
        self._closed = False
        atexit.register(self.close)

    # ------------------------------------------------------------------ allocation
    def empty(self, shape: Sequence[int], dtype: torch.dtype) -> SymmTensor:
        shape = tuple(int(s) for s in shape)
        if self.backend == "host":
            # Host memory of another process is not mapped: only the local copy exists and the CPU
            # paths of the ops go through torch.distributed collectives instead of peer pointers.
            local = torch.empty(shape, dtype=dtype)
            peers = [local if r == self.rank else torch.empty(0, dtype=dtype) for r in range(self.world)]
            return SymmTensor(local, peers, self.rank)
        esize = torch.empty((), dtype=dtype).element_size()
        nbytes = max(1, math.prod(shape)) * esize
        seg, off = None, None
        for s in self._segments:
            off = s.take(nbytes)
            if off is not None:
                seg = s
                break
        if seg is None:
            seg = self._new_segment(max(self.segment_bytes, nbytes + ALIGN))
            self._segments.append(seg)
            off = seg.take(nbytes)
            assert off is not None

        def cut(u8: torch.Tensor) -> torch.Tensor:
            return u8[off: off + math.prod(shape) * esize].view(dtype).view(*shape)

        peers = [cut(u8) for u8 in seg.peer_u8]
        local = cut(seg.local_u8)
        peers[self.rank] = local
        return SymmTensor(local, peers, self.rank, None if seg.mc_u8 is None else cut(seg.mc_u8))

    def zeros(self, shape: Sequence[int], dtype: torch.dtype) -> SymmTensor:
        """Like :meth:`empty` but zero-filled, with a barrier so no peer sees stale contents."""
        t = self.empty(shape, dtype)
        t.local.zero_()
        self.barrier()
        return t

    def barrier(self) -> None:
        """Host barrier: everything this rank enqueued before is complete on every rank after."""
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)
        if self.world > 1:
            dist.barrier(self.group)

    # ------------------------------------------------------------------ segment creation
    def _new_segment(self, nbytes: int) -> _Segment:
        if self.backend == "host":
            return self._new_segment_host(nbytes)
        if self.world == 1 and self.backend in ("auto", "ipc"):
            buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            return _Segment(nbytes, buf, [buf])
        if self.backend in ("auto", "vmm"):
            seg, err = self._try_vmm(nbytes)
            ok = torch.tensor([1 if seg is not None else 0], device=self.device, dtype=torch.int32)
            if self.world > 1:
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            if int(ok.item()) == 1:
                return seg
            if seg is not None and seg.cleanup:
                seg.cleanup()
            if self.backend == "vmm":
                raise _lib.TdistError(f"VMM symmetric heap failed on some rank (this rank: {err})")
            if self.rank == 0:
                print(f"[tdist] VMM heap unavailable ({err}); falling back to cudaIpc", flush=True)
        return self._new_segment_ipc(nbytes)

    def _new_segment_host(self, nbytes: int) -> _Segment:
        buf = torch.empty(nbytes, dtype=torch.uint8)
        # Host memory of another process is not mapped: only the local copy exists, CPU ops go
        # through torch.distributed collectives instead of peer pointers.
        return _Segment(nbytes, buf, [buf if r == self.rank else torch.empty(0, dtype=torch.uint8) for r in range(self.world)])

    def _try_vmm(self, nbytes: int):
        lib = _lib.lib()
        dev = self.device.index if self.device.index is not None else (torch.cuda.current_device() if self.device.type == "cuda" else 0)
        stage = "caps"
        handles: List[int] = [0] * self.world
        va = C.c_uint64(0)
        mapped: List[int] = []
        seg_bytes = 0
        try:
            caps = C.c_int(0)
            _lib.check(lib.tdist_symm_caps(dev, C.byref(caps)), "tdist_symm_caps")
            if not (caps.value & 1):
                raise _lib.TdistError("device lacks VMM / POSIX descriptor export")
            rounded = C.c_size_t(0)
            _lib.check(lib.tdist_symm_round_size(dev, C.c_size_t(nbytes), self.world if self.use_nvls else 0, C.byref(rounded)), "round")
            seg_bytes = rounded.value
            stage = "create"
            h = C.c_uint64(0)
            fd = C.c_int(-1)
            _lib.check(lib.tdist_symm_create(dev, C.c_size_t(seg_bytes), C.byref(h), C.byref(fd)), "tdist_symm_create")
            handles[self.rank] = h.value
        except Exception as e:  # noqa: BLE001 - every rank must reach the agreement step
            if self.world > 1:
                bad = torch.zeros(1, device=self.device, dtype=torch.int32)
                dist.all_reduce(bad, op=dist.ReduceOp.MIN, group=self.group)
            return None, f"{stage}: {e}"
        # Agree before the descriptor exchange (a collective): a rank that could not create its
        # segment must not leave the others waiting on its socket.
        if self.world > 1:
            ok = torch.ones(1, device=self.device, dtype=torch.int32)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=self.group)
            if int(ok.item()) == 0:
                lib.tdist_symm_release(C.c_uint64(handles[self.rank]))
                os.close(fd.value)
                return None, "another rank could not create its segment"
        try:
            stage = "exchange"
            all_fds = exchange_fds(self.group, [fd.value])
            stage = "import"
            for r in range(self.world):
                if r == self.rank:
                    continue
                hh = C.c_uint64(0)
                _lib.check(lib.tdist_symm_import(all_fds[r][0], C.byref(hh)), "tdist_symm_import")
                handles[r] = hh.value
            close_fds([f for fl in all_fds for f in fl])
            stage = "map"
            _lib.check(lib.tdist_symm_reserve(C.c_size_t(seg_bytes * self.world), C.byref(va)), "reserve")
            for r in range(self.world):
                _lib.check(lib.tdist_symm_map(C.c_uint64(va.value + r * seg_bytes), C.c_size_t(seg_bytes), C.c_uint64(handles[r]), dev), "map")
                mapped.append(r)
        except Exception as e:  # noqa: BLE001 - every rank must reach the agreement step
            map_err = f"{stage}: {e}"
        else:
            map_err = ""
        # Agree again after exchange / import / map: a rank that failed here must not go on to the fallback's
        # collectives while the others enter the multicast set-up's. Every rank runs this one all-reduce; if any
        # rank failed, all of them undo what they built and return None together.
        all_mapped = not map_err
        if self.world > 1:
            t = torch.tensor([1 if all_mapped else 0], device=self.device, dtype=torch.int32)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
            all_mapped = int(t.item()) == 1
        if not all_mapped:
            for r in mapped:
                lib.tdist_symm_unmap(C.c_uint64(va.value + r * seg_bytes), C.c_size_t(seg_bytes))
            if va.value:
                lib.tdist_symm_address_free(C.c_uint64(va.value), C.c_size_t(seg_bytes * self.world))
            for hdl in handles:
                if hdl:
                    lib.tdist_symm_release(C.c_uint64(hdl))
            return None, map_err or "another rank could not exchange, import or map the segments"

        # Optional NVLS alias: rank 0 creates a multicast object, every rank adds its device and binds its
        # own segment, then maps the object. Every step is followed by an agreement so that a rank that
        # failed never leaves the others inside a collective.
        mc_va, mc_handle = 0, 0
        if self.use_nvls and self.world > 1:
            def agree(flag: bool) -> bool:
                t = torch.tensor([1 if flag else 0], device=self.device, dtype=torch.int32)
                dist.all_reduce(t, op=dist.ReduceOp.MIN, group=self.group)
                return int(t.item()) == 1

            mc_err = ""
            mch, mfd = C.c_uint64(0), C.c_int(-1)
            good = bool(caps.value & 2)
            if good and self.rank == 0:
                good = lib.tdist_mc_create(self.world, C.c_size_t(seg_bytes), C.byref(mch), C.byref(mfd)) == 0
            if agree(good):
                mine = [mfd.value] if self.rank == 0 else [os.open(os.devnull, os.O_RDONLY)]
                got = exchange_fds(self.group, mine)
                if self.rank != 0:
                    good = lib.tdist_symm_import(got[0][0], C.byref(mch)) == 0
                close_fds([f for fl in got for f in fl])
                good = good and lib.tdist_mc_add_device(C.c_uint64(mch.value), dev) == 0
                if agree(good):          # every device is added before any rank binds
                    good = lib.tdist_mc_bind(C.c_uint64(mch.value), C.c_uint64(handles[self.rank]), C.c_size_t(seg_bytes)) == 0
                    if good:
                        mva = C.c_uint64(0)
                        good = (lib.tdist_symm_reserve(C.c_size_t(seg_bytes), C.byref(mva)) == 0 and
                                lib.tdist_symm_map(C.c_uint64(mva.value), C.c_size_t(seg_bytes), C.c_uint64(mch.value), dev) == 0)
                        if good:
                            mc_va, mc_handle = mva.value, mch.value
                    if not agree(good):
                        mc_err = "bind / map failed on some rank"
                else:
                    mc_err = "import / add-device failed on some rank"
            else:
                mc_err = "device without multicast support, or cuMulticastCreate failed"
            if mc_err:
                mc_va = 0
                if self.rank == 0:
                    print(f"[tdist] NVLS multicast unavailable ({mc_err}); multimem ops will refuse to run", flush=True)

        def cleanup(va=va.value, seg_bytes=seg_bytes, handles=list(handles), mapped=list(mapped), mc_va=mc_va, mc_handle=mc_handle):
            if mc_va:
                lib.tdist_symm_unmap(C.c_uint64(mc_va), C.c_size_t(seg_bytes))
                lib.tdist_symm_address_free(C.c_uint64(mc_va), C.c_size_t(seg_bytes))
                lib.tdist_mc_unbind(C.c_uint64(mc_handle), dev, C.c_size_t(seg_bytes))
                lib.tdist_symm_release(C.c_uint64(mc_handle))
            for r in mapped:
                lib.tdist_symm_unmap(C.c_uint64(va + r * seg_bytes), C.c_size_t(seg_bytes))
            if va:
                lib.tdist_symm_address_free(C.c_uint64(va), C.c_size_t(seg_bytes * self.world))
            for hdl in handles:
                if hdl:
                    lib.tdist_symm_release(C.c_uint64(hdl))

        peer_u8 = [tensor_from_ptr(va.value + r * seg_bytes, seg_bytes, self.device) for r in range(self.world)]
        mc_u8 = tensor_from_ptr(mc_va, seg_bytes, self.device) if mc_va else None
        seg = _Segment(seg_bytes, peer_u8[self.rank], peer_u8, mc_u8, cleanup)
        seg.base_va = va.value
        seg.handles = handles
        return seg, ""

    def _new_segment_ipc(self, nbytes: int) -> _Segment:
        lib = _lib.lib()
        ptr = C.c_void_p()
        handle = (C.c_char * 64)()
        _lib.check(lib.tdist_ipc_alloc(C.c_size_t(nbytes), C.byref(ptr), handle), "tdist_ipc_alloc")
        mine = bytes(handle.raw)
        gathered: List[Optional[bytes]] = [None] * self.world
        dist.all_gather_object(gathered, mine, group=self.group)
        ptrs = []
        for r in range(self.world):
            if r == self.rank:
                ptrs.append(ptr.value)
            else:
                p = C.c_void_p()
                buf = (C.c_char * 64).from_buffer_copy(gathered[r])
                _lib.check(lib.tdist_ipc_open(buf, C.byref(p)), "tdist_ipc_open")
                ptrs.append(p.value)
        peer_u8 = [tensor_from_ptr(p, nbytes, self.device) for p in ptrs]

        def cleanup(ptrs=list(ptrs), rank=self.rank):
            for r, p in enumerate(ptrs):
                if r == rank:
                    lib.tdist_ipc_free(C.c_void_p(p))
                else:
                    lib.tdist_ipc_close(C.c_void_p(p))

        return _Segment(nbytes, peer_u8[self.rank], peer_u8, None, cleanup)

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        segs, self._segments = self._segments, []
        if not segs:
            return
        try:
            if self.device.type == "cuda" and torch.cuda.is_available():
                torch.cuda.synchronize(self.device)
        except Exception:  # noqa: BLE001 - best effort at interpreter exit
            pass
        for s in segs:
            if s.cleanup is not None:
                try:
                    s.cleanup()
                except Exception:  # noqa: BLE001
                    pass


# ---------------------------------------------------------------------- single-process emulation
class LocalWorld:
    """``world`` ranks emulated in one process on one device.

    ``heap(r)`` is rank r's allocator; the k-th allocation of every rank's heap refers to the same
    symmetric object, so per-rank contexts built one after the other line up as they would across
    processes. Kernels of different emulated ranks must never wait on each other: tests launch one
    rank's kernel at a time against flags and buffers they prepared beforehand.
    """

    def __init__(self, world: int, device=None):
        self.world = world
        if device is None:
            device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = torch.device(device)
        self._objects: List[List[torch.Tensor]] = []
        self._heaps = [_LocalHeap(self, r) for r in range(world)]

    def heap(self, rank: int) -> "_LocalHeap":
        return self._heaps[rank]

    def _object(self, index: int, shape, dtype) -> List[torch.Tensor]:
        while len(self._objects) <= index:
            self._objects.append([])
        if not self._objects[index]:
            self._objects[index] = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(self.world)]
        objs = self._objects[index]
        if tuple(objs[0].shape) != tuple(shape) or objs[0].dtype != dtype:
            raise ValueError("emulated ranks allocated different symmetric objects at the same position")
        return objs


class _LocalHeap:
    backend = "local"
    group = None

    def __init__(self, world: LocalWorld, rank: int):
        self._world = world
        self.rank = rank
        self.world = world.world
        self.device = world.device
        self._count = 0

    def empty(self, shape, dtype) -> SymmTensor:
        objs = self._world._object(self._count, tuple(int(s) for s in shape), dtype)
        self._count += 1
        return SymmTensor(objs[self.rank], list(objs), self.rank)

    zeros = empty

    def barrier(self) -> None:
        if self.device.type == "cuda":
            torch.cuda.synchronize(self.device)

    def close(self) -> None:
        pass
