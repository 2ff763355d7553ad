"""One process per GPU: the ranks of a model cut across GPUs (`lc_dist_*` of the C ABI).

    rank 0:  ident = dist.unique_id()        -> hand the 128 bytes to the other ranks (a file, a socket, torch.distributed ...)
    all:     dist.init(rank, world, ident)   -> with the rank's device current, before any Engine is created
             Engine(...)                     -> tp_size / tp_rank default to the world and rank of init
             dist.finalize()
"""
from __future__ import annotations

import ctypes as C

from ._capi import check, load


def unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    check(load().lc_dist_unique_id(buf))
    return buf.raw


def init(rank: int, world: int, ident: bytes, peer_memory: bool | None = None) -> None:
    """peer_memory: True asks for the sums as one kernel over the peers' mapped buffers, False for NCCL; None keeps the
    library's default (peer memory where every buffer could be mapped, else NCCL)."""
    if len(ident) != 128:
        raise ValueError("the identifier of lc_dist_unique_id is 128 bytes")
    check(load().lc_dist_init(rank, world, C.create_string_buffer(ident, 128)))
    if peer_memory is not None:
        check(load().lc_dist_set_backend(1 if peer_memory else 0))


def finalize() -> None:
    check(load().lc_dist_finalize())


def time_allreduce(count: int, iters: int = 50) -> float:
    """Microseconds per sum of `count` floats over the ranks (every rank must call it)."""
    us = C.c_float()
    check(load().lc_dist_time_allreduce(count, iters, C.byref(us)))
    return float(us.value)


def info() -> dict:
    """rank, world and whether the sums run over mapped peer buffers (known once a model was finalized or a sum timed)."""
    r, w, p = C.c_int32(), C.c_int32(), C.c_int32()
    check(load().lc_dist_info(C.byref(r), C.byref(w), C.byref(p)))
    return {"rank": r.value, "world": w.value, "peer_memory": bool(p.value)}


def debug() -> list:
    """The record of the first wait of a sum that ran out (all zero when none did); reading clears it."""
    buf = (C.c_uint32 * 8)()
    check(load().lc_dist_debug(buf))
    return list(buf)
