"""Cross-GPU batch-norm statistics with the sum inside the kernel (peer memory over NVLink).

    ex = BnExchange(channels)            # one per process, after torch.distributed is initialised
    ops_a, ops_b = ops.Upsample(...), ops.BnStats(...)
    ex.run_pair(ops_a, ops_b)            # ONE launch; ops_b.mean / invstd are global statistics

The handles travel through `torch.distributed.all_gather_object`; with a world of one (or
without torch.distributed) the exchange degenerates to the local buffer, which is how the
single-GPU tests exercise the same kernel code.
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from .ops import _stream_ptr


class BnExchange:
    def __init__(self, channels: int, group=None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.channels = int(channels)
        L = _lib.lib()
        self._h = C.c_void_p()
        # Every rank walks through the same collectives even when a local step failed, and all
        # ranks raise together: nobody is left waiting inside a gather.
        rc = L.hfuse_exchange_create(self.world, self.rank, self.channels, C.byref(self._h))
        if self.world > 1:
            buf = C.create_string_buffer(64)
            if rc == 0:
                rc = L.hfuse_exchange_local_handle(self._h, buf)
            gathered = [None] * self.world
            dist.all_gather_object(gathered, (rc, buf.raw), group=group)
            if all(g[0] == 0 for g in gathered):
                rc = L.hfuse_exchange_connect(self._h, b"".join(g[1] for g in gathered))
            else:
                rc = rc or -5          # a peer failed (HFUSE_ERR_LAUNCH)
            # doubles as the barrier that says "every rank has mapped every buffer"
            status = [None] * self.world
            dist.all_gather_object(status, rc, group=group)
            bad = [(r, c) for r, c in enumerate(status) if c != 0]
            if bad:
                self.close()
                raise _lib.HfuseError(bad[0][1], f"peer-memory exchange set-up failed on rank {bad[0][0]}")
        else:
            _lib.check(rc, "hfuse_exchange_create")

    @classmethod
    def local_ranks(cls, channels: int, devices) -> list["BnExchange"]:
        """Exchange objects for ONE process that drives several ranks: rank r lives on devices[r]
        (peer access between different devices must already be enabled).  Connected through raw
        device pointers, no IPC and no torch.distributed."""
        L = _lib.lib()
        world = len(devices)
        out = []
        for r, d in enumerate(devices):
            ex = cls.__new__(cls)
            ex.world, ex.rank, ex.channels, ex._h = world, r, int(channels), C.c_void_p()
            with torch.cuda.device(d):
                _lib.check(L.hfuse_exchange_create(world, r, ex.channels, C.byref(ex._h)), "hfuse_exchange_create")
            out.append(ex)
        ptrs = (C.c_void_p * world)()
        for r, ex in enumerate(out):
            p = C.c_void_p()
            _lib.check(L.hfuse_exchange_local_pointer(ex._h, C.byref(p)), "hfuse_exchange_local_pointer")
            ptrs[r] = p.value
        for ex in out:
            _lib.check(L.hfuse_exchange_connect_pointers(ex._h, ptrs), "hfuse_exchange_connect_pointers")
        return out

    def set_timeout(self, seconds: float) -> None:
        """Limit of the in-kernel wait for the other ranks (default 5 s)."""
        _lib.check(_lib.lib().hfuse_exchange_set_timeout(self._h, int(seconds * 1e9)), "hfuse_exchange_set_timeout")

    def run(self, bn, stream=None):
        """Standalone statistics kernel with the in-kernel all-reduce."""
        _lib.check(_lib.lib().hfuse_bnstats_allreduce_f32(*bn.c_args(), self._h, _stream_ptr(stream)),
                   "hfuse_bnstats_allreduce_f32")
        return bn.result()

    def run_pair(self, up, bn, stream=None):
        """Fused upsample + statistics + in-kernel all-reduce: one launch."""
        _lib.check(_lib.lib().hfuse_upsample_bnstats_allreduce_f32(*up.c_args(), *bn.c_args(), self._h,
                                                                   _stream_ptr(stream)),
                   "hfuse_upsample_bnstats_allreduce_f32")
        return up.result(), bn.result()

    def timed_out(self) -> bool:
        flag = C.c_int(0)
        _lib.check(_lib.lib().hfuse_exchange_status(self._h, C.byref(flag)), "hfuse_exchange_status")
        return bool(flag.value)

    def clear_status(self, stream=None) -> None:
        """Lower the timed-out flag again (it stays raised once a wait has run out)."""
        _lib.check(_lib.lib().hfuse_exchange_clear_status(self._h, _stream_ptr(stream)), "hfuse_exchange_clear_status")

    def close(self):
        if self._h:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            _lib.lib().hfuse_exchange_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
