"""Passing file descriptors between the ranks of one node.

A cuMem allocation is shared with another process as a POSIX file descriptor, and a descriptor
only crosses a process boundary as ``SCM_RIGHTS`` ancillary data on a Unix-domain socket. Each
rank listens on an abstract-namespace socket whose name carries a job token agreed through the
process group, serves its descriptors to the ``world - 1`` peers that connect, and fetches theirs.

The reference never needs this step: NVSHMEM does its own bootstrap from a unique id broadcast
over NCCL (reference shmem/nvshmem_bind/pynvshmem/python/pynvshmem/__init__.py:157-171).
"""
from __future__ import annotations

import array
import os
import secrets
import socket
import threading
from typing import List, Sequence

import torch.distributed as dist


def global_rank(group, group_rank: int) -> int:
    """Rank in the default group of member ``group_rank`` of ``group``."""
    if group is None or group is dist.group.WORLD:
        return group_rank
    return dist.get_global_rank(group, group_rank)


def _sock_name(token: str, rank: int) -> bytes:
    return b"\0tdist-" + token.encode() + b"-" + str(rank).encode()


def _send_fds(conn: socket.socket, fds: Sequence[int]) -> None:
    conn.sendmsg([b"F"], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", fds).tobytes())])


def _recv_fds(conn: socket.socket, n: int) -> List[int]:
    fds = array.array("i")
    msg, ancdata, _flags, _addr = conn.recvmsg(1, socket.CMSG_LEN(n * fds.itemsize))
    if msg != b"F":
        raise RuntimeError("descriptor exchange: unexpected payload from peer")
    for level, ctype, data in ancdata:
        if level == socket.SOL_SOCKET and ctype == socket.SCM_RIGHTS:
            fds.frombytes(data[: len(data) - (len(data) % fds.itemsize)])
    if len(fds) != n:
        raise RuntimeError(f"descriptor exchange: expected {n} descriptors, got {len(fds)}")
    return list(fds)


def exchange_fds(group, fds: Sequence[int], timeout_s: float = 60.0) -> List[List[int]]:
    """All-gather of file descriptors inside ``group`` (all ranks on one host).

    Returns ``out[r]`` = rank r's descriptors as valid descriptors of *this* process
    (``out[rank]`` are the caller's own, not duplicated). The caller closes what it receives.
    """
    rank = dist.get_rank(group)
    world = dist.get_world_size(group)
    if world == 1:
        return [list(fds)]
    box = [secrets.token_hex(8) if rank == 0 else None]
    dist.broadcast_object_list(box, src=global_rank(group, 0), group=group)
    token = box[0]

    server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    server.bind(_sock_name(token, rank))
    server.listen(world)
    server.settimeout(timeout_s)
    errors: List[BaseException] = []

    def serve():
        try:
            for _ in range(world - 1):
                conn, _ = server.accept()
                with conn:
                    _send_fds(conn, fds)
                    conn.recv(1)  # the peer acknowledges before we drop the connection
        except BaseException as e:  # noqa: BLE001 - reported to the caller below
            errors.append(e)

    th = threading.Thread(target=serve, name="tdist-fd-server", daemon=True)
    th.start()
    dist.barrier(group)  # every rank is listening

    out: List[List[int]] = [[] for _ in range(world)]
    out[rank] = list(fds)
    try:
        for step in range(1, world):
            peer = (rank + step) % world
            with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                c.settimeout(timeout_s)
                c.connect(_sock_name(token, peer))
                out[peer] = _recv_fds(c, len(fds))
                c.send(b"K")
    finally:
        th.join(timeout_s)
        server.close()
    if errors:
        raise RuntimeError(f"descriptor exchange failed on rank {rank}: {errors[0]!r}")
    dist.barrier(group)
    return out


def close_fds(fds: Sequence[int]) -> None:
    for fd in fds:
        try:
            os.close(fd)
        except OSError:
            pass
