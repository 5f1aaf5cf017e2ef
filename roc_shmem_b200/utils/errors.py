"""Status codes of the native runtime as Python exceptions.

The reference aborts the process on any failure (``NET_CHECK`` → ``abort()``,
gpu_ib/backend_ib.cpp:42-48) and its device waits spin for ever
(context_tmpl_device.hpp:202-203).  Here every native call returns a status and
every wait is bounded, so failures surface as exceptions the caller can handle.
"""
from __future__ import annotations

OK, ERR_INVALID, ERR_NOMEM, ERR_TIMEOUT, ERR_RANGE, ERR_STATE, ERR_LIMIT, ERR_CUDA, ERR_UNSUPPORTED, \
    ERR_ABORTED, ERR_PEER_DEAD = range(11)

_NAMES = {
    OK: "ok", ERR_INVALID: "invalid argument", ERR_NOMEM: "symmetric heap exhausted",
    ERR_TIMEOUT: "wait timed out", ERR_RANGE: "address outside the symmetric heap",
    ERR_STATE: "runtime not initialised", ERR_LIMIT: "out of team or context slots",
    ERR_CUDA: "CUDA error", ERR_UNSUPPORTED: "unsupported", ERR_ABORTED: "job aborted by global_exit",
    ERR_PEER_DEAD: "peer marked failed",
}


class ShmemError(RuntimeError):
    """A native call returned a non-zero status."""

    def __init__(self, status: int, detail: str = ""):
        self.status = status
        self.detail = detail
        msg = _NAMES.get(status, f"status {status}")
        super().__init__(f"{msg}: {detail}" if detail else msg)


class ShmemTimeout(ShmemError):
    """A bounded wait (wait_until, barrier, signal, proxy completion) ran out."""


class ShmemAborted(ShmemError):
    """Another PE called global_exit, or a peer was marked failed."""


def raise_for_status(status: int, detail: str = "") -> None:
    if status == OK:
        return
    if status == ERR_TIMEOUT:
        raise ShmemTimeout(status, detail)
    if status in (ERR_ABORTED, ERR_PEER_DEAD):
        raise ShmemAborted(status, detail)
    raise ShmemError(status, detail)
