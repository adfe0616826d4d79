"""Peer-memory plumbing for the tensor-parallel decode step: symmetric receive areas on every rank and the call into
``xl_peer_reduce_add_rmsnorm`` (all-reduce of partial sums + residual add + RMSNorm in one kernel over NVLink).

PyTorch is used for what it is here for: device memory that every rank can address (``torch.distributed._symmetric_memory``)
and the rendezvous that exchanges the addresses.  The kernel itself only issues plain loads and stores on those addresses
(no multicast, no library call on peer memory)."""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import ops
from ._lib import PeerReduceParams, check, lib

_DTYPES = {torch.float32: 0, torch.bfloat16: 1}


class PeerReducer:
    """Receive areas for `rows_max` rows of `D` values of `dtype` from every rank of `group`, double buffered."""

    def __init__(self, group, device, rows_max: int, D: int, dtype):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device, self.rows_max, self.D, self.dtype = torch.device(device), rows_max, D, dtype
        if self.world > 8:
            raise ValueError("the peer reduction kernel covers up to 8 ranks")
        name = self.group.group_name
        if hasattr(symm, "enable_symm_mem_for_group") and not symm.is_symm_mem_enabled_for_group(name):
            symm.enable_symm_mem_for_group(name)
        self.recv = symm.empty(2 * self.world * rows_max * D, dtype=dtype, device=self.device)
        self.flags = symm.empty(2 * self.world * rows_max, dtype=torch.int32, device=self.device)
        hr, hf = symm.rendezvous(self.recv, name), symm.rendezvous(self.flags, name)
        self.recv.zero_()
        self.flags.zero_()
        self.epoch = torch.zeros(rows_max, dtype=torch.int32, device=self.device)
        self._handles = (hr, hf)   # keep the mappings alive
        self.peer_recv = torch.tensor([int(x) for x in hr.buffer_ptrs], dtype=torch.int64, device=self.device)
        self.peer_flags = torch.tensor([int(x) for x in hf.buffer_ptrs], dtype=torch.int64, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)   # every rank's areas are zeroed before anybody pushes

    @classmethod
    def create(cls, group, device, rows_max: int, D: int, dtype):
        """The reducer, or (None, reason) when symmetric memory cannot be set up on this machine."""
        try:
            return cls(group, device, rows_max, D, dtype), None
        except Exception as e:   # no symmetric-memory support, no peer access, ...
            return None, f"{type(e).__name__}: {str(e)[:300]}"

    def reduce_add_rmsnorm(self, partial, x, weight, eps: float):
        """``x_new = x + sum_ranks(partial)`` and ``RMSNorm(x_new) * weight``; every rank must call this with the same
        number of rows, in the same order.  Returns (x_new, normed) shaped like ``x``; x is updated in place."""
        D = x.shape[-1]
        p2, x2 = partial.reshape(-1, D), x.reshape(-1, D)
        rows = x2.shape[0]
        if rows > self.rows_max or D != self.D or x.dtype != self.dtype or p2.shape != x2.shape:
            raise ValueError("reduce_add_rmsnorm: shape or dtype does not match the receive areas")
        if p2.stride(-1) != 1:
            p2 = p2.contiguous()
        if x2.stride(-1) != 1:
            raise ValueError("reduce_add_rmsnorm: x must have contiguous rows")
        normed = torch.empty((rows, D), dtype=x.dtype, device=x.device)
        p = PeerReduceParams()
        p.partial, p.peer_recv, p.recv_local = p2.data_ptr(), self.peer_recv.data_ptr(), self.recv.data_ptr()
        p.peer_flags, p.flags_local, p.epoch = self.peer_flags.data_ptr(), self.flags.data_ptr(), self.epoch.data_ptr()
        p.x, p.weight, p.x_out, p.normed = x2.data_ptr(), weight.data_ptr(), x2.data_ptr(), normed.data_ptr()
        p.status = ops.status_word(x.device).data_ptr()
        p.rank, p.world, p.rows, p.D, p.rows_max = self.rank, self.world, rows, D, self.rows_max
        p.partial_sr, p.x_sr, p.xo_sr, p.n_sr = p2.stride(0), x2.stride(0), x2.stride(0), D
        p.eps, p.dtype = eps, _DTYPES[x.dtype]
        with torch.cuda.device(x.device):
            check(lib().xl_peer_reduce_add_rmsnorm(C.byref(p), torch.cuda.current_stream(x.device).cuda_stream), "xl_peer_reduce_add_rmsnorm")
        return x, normed.reshape(x.shape)
