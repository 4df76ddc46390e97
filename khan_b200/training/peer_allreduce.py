"""Mean of the flat gradient buffer over the GPUs of one node through peer memory.

The reference averages the towers' gradients variable by variable on the CPU
(``khan/training/trainer_multi_tower.py:137-179``).  With one process per GPU the same average is
ONE kernel launch per rank (``ani_peer_mean_f32`` of the C library): every rank copies its
gradients into a staging buffer that the other ranks have mapped with CUDA IPC, tells them, waits
(bounded) until all have done the same, and sums the staging buffers over NVLink -- every rank in
the same order, so all ranks hold the same mean bit for bit.  Unlike a library collective it can be
captured into the CUDA graph of the training step.

The 64-byte handles travel through ``torch.distributed`` (any backend); nothing else of the
exchange touches the host.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _lib


# Measured on the 296,464-value gradient buffer of the training step (ms per step, peer kernel / NCCL
# all-reduce): 2 GPUs 0.230 / 0.237, 4 GPUs 0.243 / 0.246, 8 GPUs 0.274 / 0.263 -- with every rank summing
# all staging buffers a rank pulls 8.3 MB per step over NVLink on 8 GPUs, and NCCL reduces inside the
# switch there.  The two-halves form (slice means + exchange of the slices) moves a quarter of the bytes
# but pays a second round of flags: on 4 GPUs 0.253 against 0.243.  So the callers get the peer kernel
# for up to four ranks and the library all-reduce above.
PEER_MAX_RANKS = 4


class PeerAllReduce:
    """``mean_(flat)`` replaces ``dist.all_reduce(flat); flat /= world`` for float32 CUDA buffers of at
    most ``n_floats`` values (a multiple of 4, 16-byte aligned).  Every rank must construct it and call
    ``mean_`` the same number of times, on one stream per rank."""

    def __init__(self, n_floats: int, device, group=None, two_halves=None):
        """``two_halves``: True = every rank forms the mean of its slice and the slices are exchanged, False =
        every rank sums everything, None = the library's choice (two halves above four ranks).  The
        environment variable KHAN_B200_PEER_FORM ("two_halves" / "one") overrides it, for measurements."""
        import os
        import torch.distributed as dist
        form = os.environ.get("KHAN_B200_PEER_FORM")
        if form in ("two_halves", "one"):
            two_halves = form == "two_halves"
        self.device = torch.device(device)
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.n_floats = int(n_floats)
        self._ptr = ctypes.c_void_p()
        L = _lib.lib()
        with torch.cuda.device(self.device):
            status = L.ani_peer_create(self.rank, self.world, self.n_floats, ctypes.byref(self._ptr))
            mine = (ctypes.c_ubyte * 64)()
            if status == 0 and two_halves is not None:
                status = L.ani_peer_set_two_halves(self._ptr, int(bool(two_halves)))
            if status == 0:
                status = L.ani_peer_handle(self._ptr, mine)
            handles = [None] * self.world
            dist.all_gather_object(handles, (status, bytes(mine)), group=group)
            if status == 0 and all(h[0] == 0 for h in handles):
                for q, (_, raw) in enumerate(handles):
                    if q != self.rank and status == 0:
                        buf = (ctypes.c_ubyte * 64).from_buffer_copy(raw)
                        status = L.ani_peer_connect(self._ptr, q, buf)
            # all ranks use the peer path, or none does
            ok = torch.tensor([1 if status == 0 and all(h[0] == 0 for h in handles) else 0], device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self.close()
                raise RuntimeError("peer memory between the GPUs of this process group is not available "
                                   f"(rank {self.rank}: {_lib.lib().ani_status_string(status).decode()})")

    def mean_(self, flat: torch.Tensor, stream=None) -> torch.Tensor:
        """In place: ``flat`` becomes its mean over the ranks (enqueued on ``stream`` or the current stream)."""
        if flat.dtype != torch.float32 or not flat.is_contiguous():
            raise ValueError("PeerAllReduce.mean_ takes a contiguous float32 buffer")
        _lib.same_device(self.device, flat, where="PeerAllReduce.mean_")
        if stream is None:
            stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        _lib.check(_lib.lib().ani_peer_mean_f32(self._ptr, flat.data_ptr(), flat.numel(), stream),
                   "ani_peer_mean_f32")
        return flat

    def close(self) -> None:
        if self._ptr:
            with torch.cuda.device(self.device):
                _lib.lib().ani_peer_destroy(self._ptr)
            self._ptr = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def try_peer_allreduce(n_floats: int, device, group=None):
    """A ``PeerAllReduce`` when the process group has several ranks on GPUs that can map each other's
    memory, else ``None`` (the callers then use the library all-reduce).  Collective: every rank calls it."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return None
    if dist.get_world_size(group) > PEER_MAX_RANKS:
        return None
    try:
        return PeerAllReduce(n_floats, device, group)
    except RuntimeError:
        return None
