"""Peer-buffer registry: symmetric staging memory over NVLink for the in-kernel collectives.

``PeerGroup`` is the B200 equivalent of the reference's device mesh (``glm_tpu/distributed/mesh.py:31-57``,
``parallel_state.py:23-78``): it owns this rank's staging/flag buffers, exchanges CUDA IPC handles with the other
ranks through ``torch.distributed`` (any backend: the handles are 128 opaque bytes), maps the peers' buffers and
hands the kernels a ``PeerComm`` table.  It also carves named regions out of the staging buffer (the same
offsets on every rank) and exposes them as torch tensors.

With ``world == 1`` no buffers are exchanged and kernels skip every wait.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from glm_tpu_b200.exceptions import DeviceStatusError
from glm_tpu_b200.ops import native


class _RawCudaBuffer:
    """Expose a raw device pointer to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 2,
        }


@dataclass
class Region:
    name: str
    offset: int
    nbytes: int


class PeerGroup:
    def __init__(self, world: int = 1, rank: int = 0, *, staging_bytes: int = 0, wait_limit: int = 2_000_000, group=None,
                 device=None):
        self.world, self.rank, self.group = world, rank, group
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.wait_limit = wait_limit
        self._lib = native.lib()
        self._ar_bytes = int(self._lib.glmb_peer_ar_bytes())
        self._total = self._ar_bytes + _align(staging_bytes, 4096)
        self._cursor = self._ar_bytes
        self.regions: dict[str, Region] = {}
        self._handle = C.c_void_p()
        with torch.cuda.device(self.device):
            code = self._lib.glmb_peer_create(world, rank, C.c_size_t(self._total), C.byref(self._handle))
        if code != 0:
            raise RuntimeError(f"peer registry allocation failed (cuda error {code})")
        self._base = int(self._lib.glmb_peer_data(self._handle))
        self._bytes = torch.as_tensor(_RawCudaBuffer(self._base, self._total), device=self.device)
        self.status_ptr = int(self._lib.glmb_peer_status_ptr(self._handle))
        self.comm = native.PeerComm()
        if world > 1:
            self._exchange()
        code = self._lib.glmb_peer_comm(self._handle, C.c_uint32(wait_limit), C.byref(self.comm))
        if code != 0:
            raise RuntimeError("peer table is incomplete")

    # ------------------------------------------------------------------ set-up
    def _exchange(self) -> None:
        import torch.distributed as dist

        mine = (C.c_ubyte * 128)()
        code = self._lib.glmb_peer_export(self._handle, mine)
        if code != 0:
            raise RuntimeError(f"cudaIpcGetMemHandle failed ({code})")
        gathered: list = [None] * self.world
        dist.all_gather_object(gathered, bytes(mine), group=self.group)
        for peer, blob in enumerate(gathered):
            if peer == self.rank:
                continue
            buf = (C.c_ubyte * 128).from_buffer_copy(blob)
            with torch.cuda.device(self.device):
                code = self._lib.glmb_peer_import(self._handle, peer, buf)
            if code != 0:
                raise RuntimeError(f"cudaIpcOpenMemHandle for rank {peer} failed ({code})")
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ regions
    def region(self, name: str, nbytes: int) -> Region:
        """Reserve ``nbytes`` of staging (same call order on every rank gives the same offsets)."""
        if name in self.regions:
            if self.regions[name].nbytes < nbytes:
                raise ValueError(f"region {name!r} already exists with a smaller size")
            return self.regions[name]
        nbytes = _align(nbytes, 256)
        if self._cursor + nbytes + GUARD_BYTES > self._total:
            raise MemoryError(f"staging buffer exhausted while reserving {name!r}")
        reg = Region(name, self._cursor, nbytes)
        self._cursor += nbytes + GUARD_BYTES
        self.regions[name] = reg
        # canary words behind the region: peers push into this memory, so an overrun by a kernel of ANY rank lands here
        self._bytes[reg.offset + nbytes : reg.offset + nbytes + GUARD_BYTES].fill_(GUARD_PATTERN)
        return reg

    def check_canaries(self) -> None:
        """Raise if a guard band behind any region was overwritten (synchronizes; call between steps, not per step)."""
        bad = []
        for reg in self.regions.values():
            guard = self._bytes[reg.offset + reg.nbytes : reg.offset + reg.nbytes + GUARD_BYTES]
            if not bool((guard == GUARD_PATTERN).all()):
                bad.append(reg.name)
        if bad:
            raise DeviceStatusError(f"staging regions overrun: {bad}", 0)

    def tensor(self, region: Region, shape, dtype) -> torch.Tensor:
        count = 1
        for n in shape:
            count *= n
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        if nbytes > region.nbytes:
            raise ValueError(f"tensor of {nbytes} bytes does not fit region {region.name!r}")
        return self._bytes[region.offset : region.offset + nbytes].view(dtype).view(*shape)

    # ------------------------------------------------------------------ status
    @property
    def kernel_comm(self):
        """What a kernel wrapper takes as ``comm``: ``None`` for a single GPU."""
        return self.comm if self.world > 1 else None

    def read_status(self, clear: bool = True) -> int:
        value = C.c_uint32(0)
        stream = C.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        code = self._lib.glmb_peer_read_status(self._handle, int(clear), stream, C.byref(value))
        if code != 0:
            raise RuntimeError(f"reading the status word failed ({code})")
        return int(value.value)

    def check_status(self) -> None:
        value = self.read_status()
        if value:
            names = [n for bit, n in ((1, "wait timeout"), (2, "index clamped"), (4, "non-finite value"), (8, "bad shape")) if value & bit]
            raise DeviceStatusError("device status: " + ", ".join(names), value)

    def close(self) -> None:
        if self._handle:
            self._bytes = None
            self._lib.glmb_peer_destroy(self._handle)
            self._handle = C.c_void_p()


GUARD_BYTES = 256
GUARD_PATTERN = 0xA5


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a
