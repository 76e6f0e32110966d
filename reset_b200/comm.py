"""One-shot all-reduce over NVLink peer memory for the row-parallel linears of a tensor-parallel
decode step (``nvfp4r_peer_allreduce_bf16``): host-side set-up and the per-call wrapper.

Every rank allocates its receive memory through the C ABI, the 64-byte IPC handles travel
through ``torch.distributed`` (any backend: they are plain bytes), every rank maps the others'
memory, and from then on an all-reduce is ONE kernel launch per rank on the caller's stream
(CUDA-graph capturable; no NCCL call). In the reference's deployment this exchange is vLLM's
all-reduce inside ``RowParallelLinear``; the reference has no code for it.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib as L


class PeerAllReduce:
    """Sum-all-reduce of bf16 tensors of at most ``max_elems`` elements among the ranks of
    ``group`` (one process per GPU, one node). All ranks must call :meth:`all_reduce_` in the
    same order with the same sizes."""

    def __init__(self, device, max_elems: int, group=None):
        import torch.distributed as dist

        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if self.world > L.PEER_MAX_WORLD:
            raise ValueError(f"PeerAllReduce: at most {L.PEER_MAX_WORLD} ranks")
        self.max_elems = int(max_elems) + (int(max_elems) & 1)
        self._own = C.c_void_p()
        self._peers: list = []
        self.comm = None
        if self.world == 1:
            return
        lib = L.lib()
        with torch.cuda.device(self.device):
            nbytes = lib.nvfp4r_peer_buffer_bytes(self.world, self.max_elems)
            handle = C.create_string_buffer(64)
            L.check(lib.nvfp4r_peer_alloc(nbytes, C.byref(self._own), handle), "nvfp4r_peer_alloc")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            comm = L.PeerComm()
            comm.world, comm.rank, comm.max_elems = self.world, self.rank, self.max_elems
            for r in range(self.world):
                if r == self.rank:
                    comm.base[r] = self._own.value
                    continue
                ptr = C.c_void_p()
                L.check(lib.nvfp4r_peer_open(C.create_string_buffer(handles[r], 64), C.byref(ptr)),
                        "nvfp4r_peer_open")
                self._peers.append(ptr)
                comm.base[r] = ptr.value
            self.comm = comm
            torch.cuda.synchronize(self.device)
        dist.barrier(group=group)              # nobody pushes before everybody has mapped and zeroed

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """In place; ``t`` bf16, contiguous, even element count."""
        if self.world == 1:
            return t
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or t.numel() % 2 or t.numel() > self.max_elems:
            raise ValueError("PeerAllReduce: contiguous bf16 tensor of even size <= max_elems expected")
        with torch.cuda.device(t.device):
            st = L.lib().nvfp4r_peer_allreduce_bf16(C.byref(self.comm), t.data_ptr(), t.data_ptr(), t.numel(),
                                                   L.PEER_ALLREDUCE, torch.cuda.current_stream().cuda_stream)
        L.check(st, "nvfp4r_peer_allreduce_bf16")
        return t

    def gather_(self, t: torch.Tensor) -> torch.Tensor:
        """Second half only: the contributions were pushed by the epilogue of the linear that
        produced ``t`` (``nvfp4r_linear_packed_ex`` with ``push_to``); sums them into ``t``."""
        if self.world == 1:
            return t
        with torch.cuda.device(t.device):
            st = L.lib().nvfp4r_peer_allreduce_bf16(C.byref(self.comm), t.data_ptr(), t.data_ptr(), t.numel(),
                                                   L.PEER_GATHER, torch.cuda.current_stream().cuda_stream)
        L.check(st, "nvfp4r_peer_allreduce_bf16")
        return t

    def close(self) -> None:
        """Unmap the peers and free the receive memory (after a barrier of the caller's)."""
        lib = L.lib()
        for p in self._peers:
            lib.nvfp4r_peer_close(p)
        self._peers = []
        if self._own.value:
            lib.nvfp4r_peer_free(self._own)
            self._own = C.c_void_p()
        self.comm = None
