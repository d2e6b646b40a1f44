"""One-shot all-reduce over peer-mapped buffers for decode-sized tensors.

``RowParallelLinear.forward`` and ``MoE.forward`` of the reference sum their partial outputs with
``dist.all_reduce`` (model.py:263-264, 691-692): 181 collectives of 14 KB - 1 MB per decode step at TP = 8, all
bound by latency.  ``P2PAllReduce`` keeps one exported buffer per rank (CUDA IPC) and sums with one small kernel per
rank that reads the peers' partial sums with ordinary loads (``csrc/allreduce.cu``); larger tensors stay on NCCL.

    ar = dsv3_b200.P2PAllReduce(group=None, max_bytes=2 << 20)     # collective: every rank of the group calls it
    ar.all_reduce(y)                                               # in place, same order and shapes on all ranks
    ...
    ar.close()                                                     # collective: after every rank's last use

``install_all_reduce(model_module, ar)`` points the name ``dist`` that ``model.py`` looks up at call time to a proxy
whose ``all_reduce`` takes this path for small bf16 tensors and defers to ``torch.distributed`` otherwise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from ._lib import lib
from .ops import _stream


class P2PAllReduce:
    def __init__(self, group=None, max_bytes: int = 2 << 20, limit_ns: int = 0):
        import torch.distributed as dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.max_bytes = int(max_bytes)
        self.limit_ns = int(limit_ns)
        self.device = torch.device("cuda", torch.cuda.current_device())
        hb = lib.dsv3_p2p_handle_bytes()
        handle = ctypes.create_string_buffer(hb)
        comm = ctypes.c_void_p()
        _lib.check(lib.dsv3_p2p_create(self.rank, self.world, self.max_bytes, ctypes.byref(comm), handle))
        self._comm = comm
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        blob = ctypes.create_string_buffer(b"".join(handles), hb * self.world)
        _lib.check(lib.dsv3_p2p_connect(self._comm, blob))
        dist.barrier(group=group)

    def fits(self, t: torch.Tensor) -> bool:
        return (t.is_cuda and t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() * 2 <= self.max_bytes
                and t.data_ptr() % 16 == 0)

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """Sum ``t`` over the ranks in place (bf16, contiguous, at most ``max_bytes``)."""
        if not self.fits(t):
            raise ValueError("P2PAllReduce.all_reduce takes a contiguous bfloat16 CUDA tensor of at most max_bytes")
        with torch.cuda.device(t.device):
            _lib.check(lib.dsv3_allreduce_oneshot(self._comm, t.data_ptr(), t.data_ptr(), t.numel(), self.limit_ns, _stream()))
        return t

    def close(self) -> None:
        import torch.distributed as dist
        if self._comm is not None:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)          # no rank unmaps while a peer may still read
            lib.dsv3_p2p_destroy(self._comm)
            self._comm = None


class _DistProxy:
    """Stands in for the ``torch.distributed`` module inside model.py: ``all_reduce`` of a small bf16 tensor with the
    default SUM over the default group goes through ``P2PAllReduce``; everything else is passed through."""

    def __init__(self, real, ar: P2PAllReduce):
        self._real, self._ar = real, ar

    def all_reduce(self, tensor, *args, **kwargs):
        if not args and not kwargs and self._ar.fits(tensor):
            return self._ar.all_reduce(tensor)
        return self._real.all_reduce(tensor, *args, **kwargs)

    def __getattr__(self, name):
        return getattr(self._real, name)


def install_all_reduce(model_module, ar: Optional[P2PAllReduce]) -> None:
    """model.py calls ``dist.all_reduce(y)`` through its module-level name ``dist`` (model.py:9, 127, 264, 692)."""
    import torch.distributed as dist
    model_module.dist = _DistProxy(dist, ar) if ar is not None else dist
