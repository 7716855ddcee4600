"""The exchange step of the tensor-parallel decode: sum of the row-parallel projections' partial outputs.

`OneShotAllReduce` runs the library's one-launch all-reduce over peer memory (`nf4_b200_tp_allreduce`); its
buffers are symmetric memory of `torch.distributed._symmetric_memory` (every rank maps every rank's buffer;
PyTorch is plumbing here -- the kernel only gets the raw addresses).  The NCCL all-reduce stays available as
the fallback and as the checker (thunder/executors/torchex.py:2058-2078 is the reference's call).
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import _lib


class OneShotAllReduce:
    """y = sum over ranks of `partial` (+ residual) for bf16 tiles of at most `max_numel` elements."""

    def __init__(self, group, device, max_numel: int):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm_mem

        # plain peer mappings are all the kernel needs; keep the buffers out of any NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        self.lib = _lib.load()
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device)
        self.nbytes = int(self.lib.nf4_b200_tp_allreduce_buffer_bytes(int(max_numel)))
        self.max_numel = int(max_numel)
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        self.handle = symm_mem.rendezvous(self.buf, group)
        ptrs = list(self.handle.buffer_ptrs)
        assert len(ptrs) == self.world and ptrs[self.rank] == self.buf.data_ptr()
        self.ptrs = (ctypes.c_uint64 * self.world)(*ptrs)
        dist.barrier(group)          # every rank has zeroed its flags before anybody's first store arrives

    def __call__(self, partial: torch.Tensor, residual=None, out=None, pdl: bool = False) -> torch.Tensor:
        n = partial.numel()
        if partial.dtype != torch.bfloat16 or not partial.is_contiguous() or n > self.max_numel or n % 8:
            raise ValueError(f"OneShotAllReduce: contiguous bf16 tiles of up to {self.max_numel} elements (multiple of 8)")
        if out is None:
            out = torch.empty_like(partial)
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(self.lib.nf4_b200_tp_allreduce(partial.data_ptr(), residual.data_ptr() if residual is not None else None,
                                                  out.data_ptr(), n, self.ptrs, self.nbytes, self.rank, self.world, 1 if pdl else 0, st),
                   "nf4_b200_tp_allreduce")
        return out
