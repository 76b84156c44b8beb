"""Python side of the NVLink peer-memory runtime (``csrc/comm.cu``).

A ``PeerGroup`` is the set of ranks of one NVSwitch domain (one process per GPU).  Each rank allocates
named *symmetric buffers* (same name and size on every rank), the 64-byte CUDA IPC handles are exchanged
ONCE over a host side channel (``torch.distributed.all_gather_object``), and from then on kernels address a
peer's buffer through ``group.ptrs(name)[peer]``.  Only scalars (fitness values, pairing decisions, status
words) ever cross the host.  This replaces the reference's gloo barriers, TCP sockets and shared-filesystem
coordination (gossip/network_utils.py, gossip/evolutionary_node.py:392-725).

``LocalTransport`` wires several ranks that live in ONE process on ONE GPU (pointers are shared directly);
it exists so the multi-rank logic can be tested on a single GPU by running the ranks one after another.
"""
from __future__ import annotations

import ctypes as C

import torch

from ..ops import _lib as L

MAX_RANKS = 8
DEFAULT_TIMEOUT_NS = 20_000_000_000   # bounded device-side wait: 20 s, then the status word is set

_P = C.c_void_p
_SIGS = {
    "grb_comm_malloc": [C.c_size_t, C.POINTER(C.c_void_p), C.c_char_p],
    "grb_comm_free": [_P],
    "grb_comm_open": [C.c_char_p, C.POINTER(C.c_void_p)],
    "grb_comm_close": [_P],
    "grb_comm_signal": [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_ulonglong, _P],
    "grb_comm_wait": [_P, C.c_int, C.c_ulonglong, C.c_ulonglong, _P, _P],
    "grb_push_add_ranges": [_P, C.POINTER(C.c_void_p), C.c_int, C.c_int, _P, C.c_int, C.c_longlong, _P],
    "grb_bcast_ranges": [_P, C.POINTER(C.c_void_p), C.c_int, C.c_int, _P, C.c_int, C.c_longlong, _P],
    "grb_sfadamw_shard_step": [_P, _P, _P, _P, C.POINTER(C.c_void_p), C.c_int, C.c_int64, C.c_int64] +
                              [C.c_float] * 8 + [C.c_int, _P, _P],
}
_bound = False


def _lib():
    global _bound
    lib = L.lib()
    if not _bound:
        for name, sig in _SIGS.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = sig, C.c_int
        _bound = True
    return lib


def ptr_array(ptrs):
    arr = (C.c_void_p * len(ptrs))()
    for i, p in enumerate(ptrs):
        arr[i] = p
    return arr


_TYPESTR = {torch.float32: "<f4", torch.uint8: "|u1", torch.int64: "<i8", torch.int32: "<i4", torch.bfloat16: "<u2"}


class _CudaArray:
    def __init__(self, ptr, numel, typestr, keep):
        self.__cuda_array_interface__ = {"shape": (numel,), "typestr": typestr, "data": (ptr, False), "version": 2}
        self._keep = keep


class SymBuffer:
    """One rank's instance of a symmetric buffer: a zero-filled cudaMalloc allocation and its IPC handle."""

    def __init__(self, nbytes: int, device: torch.device):
        self.nbytes, self.device = nbytes, device
        p = C.c_void_p()
        h = C.create_string_buffer(64)
        with torch.cuda.device(device):
            L.check(_lib().grb_comm_malloc(nbytes, C.byref(p), h), "grb_comm_malloc")
        self.ptr, self.handle = p.value, h.raw
        self._freed = False

    def tensor(self, dtype: torch.dtype, numel: int | None = None) -> torch.Tensor:
        """A torch view of the buffer (no copy; the buffer outlives the tensor only while this object is alive)."""
        item = torch.empty(0, dtype=dtype).element_size()
        numel = self.nbytes // item if numel is None else numel
        t = torch.as_tensor(_CudaArray(self.ptr, numel, _TYPESTR[dtype], self), device=self.device)
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t

    def free(self):
        if not self._freed:
            _lib().grb_comm_free(self.ptr)
            self._freed = True


class TorchDistTransport:
    """Exchanges IPC handles over torch.distributed (host control plane) and maps the peers' buffers."""

    def __init__(self, rank, world, process_group=None):
        self.rank, self.world, self.pg = rank, world, process_group

    def exchange(self, name: str, buf: SymBuffer):
        import torch.distributed as dist
        handles = [None] * self.world
        dist.all_gather_object(handles, (name, buf.handle, buf.nbytes), group=self.pg)
        ptrs = []
        for r, (n, h, nb) in enumerate(handles):
            if n != name or nb != buf.nbytes:
                raise RuntimeError(f"symmetric buffer mismatch: rank {r} sent {n!r} ({nb} B), expected {name!r} ({buf.nbytes} B)")
            if r == self.rank:
                ptrs.append(buf.ptr)
            else:
                p = C.c_void_p()
                with torch.cuda.device(buf.device):
                    L.check(_lib().grb_comm_open(h, C.byref(p)), f"grb_comm_open(rank {r}, {name})")
                ptrs.append(p.value)
        return ptrs

    def host_barrier(self):
        import torch.distributed as dist
        dist.barrier(group=self.pg)


class LocalTransport:
    """All ranks in one process on one GPU: every rank registers its buffer, pointers are shared as they are."""

    def __init__(self, world):
        self.world = world
        self.table: dict[str, dict[int, SymBuffer]] = {}

    def for_rank(self, rank):
        return _LocalEndpoint(self, rank)


class _LocalEndpoint:
    def __init__(self, hub: LocalTransport, rank: int):
        self.hub, self.rank, self.world = hub, rank, hub.world
        self.pending = []

    def exchange(self, name, buf):
        self.hub.table.setdefault(name, {})[self.rank] = buf
        self.pending.append(name)
        return None      # resolved by PeerGroup.finish_local_connect once every rank has registered

    def host_barrier(self):
        pass


class PeerGroup:
    def __init__(self, rank: int, world: int, device, transport=None):
        if world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks per NVSwitch domain")
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.transport = transport if transport is not None else TorchDistTransport(rank, world)
        self.local: dict[str, SymBuffer] = {}
        self._ptrs: dict[str, list[int]] = {}
        self.step = 0
        self.flags = self.alloc("__flags__", 8 * MAX_RANKS)
        self.timeout_ns = DEFAULT_TIMEOUT_NS

    def alloc(self, name: str, nbytes: int) -> SymBuffer:
        """Collective: every rank calls it with the same name and size."""
        nbytes = (nbytes + 255) // 256 * 256
        buf = SymBuffer(nbytes, self.device)
        self.local[name] = buf
        ptrs = self.transport.exchange(name, buf)
        if ptrs is not None:
            self._ptrs[name] = ptrs
        return buf

    def finish_local_connect(self):
        hub = self.transport.hub
        for name, per_rank in hub.table.items():
            if len(per_rank) == self.world:
                self._ptrs[name] = [per_rank[r].ptr for r in range(self.world)]

    def ptrs(self, name: str) -> list[int]:
        """Device addresses of buffer `name` on every rank (index = rank; own entry is the local pointer)."""
        return self._ptrs[name]

    def device_barrier(self) -> None:
        """Stream-ordered barrier across the group: kernels launched after it on any rank see every peer-memory
        write issued before it on every rank.  The wait is bounded; expiry sets the device status word."""
        self.step += 1
        lib = _lib()
        st = L.stream()
        L.check(lib.grb_comm_signal(ptr_array(self.ptrs("__flags__")), self.world, self.rank, self.step, st), "grb_comm_signal")
        L.check(lib.grb_comm_wait(self.flags.ptr, self.world, self.step, self.timeout_ns,
                                  L.err_flag(self.device).data_ptr(), st), "grb_comm_wait")

    def signal_only(self) -> None:
        self.step += 1
        L.check(_lib().grb_comm_signal(ptr_array(self.ptrs("__flags__")), self.world, self.rank, self.step, L.stream()),
                "grb_comm_signal")

    def wait_only(self, value: int | None = None, timeout_ns: int | None = None) -> None:
        L.check(_lib().grb_comm_wait(self.flags.ptr, self.world, self.step if value is None else value,
                                     self.timeout_ns if timeout_ns is None else timeout_ns,
                                     L.err_flag(self.device).data_ptr(), L.stream()), "grb_comm_wait")

    def close(self):
        for name, ptrs in self._ptrs.items():
            if isinstance(self.transport, TorchDistTransport):
                for r, p in enumerate(ptrs):
                    if r != self.rank:
                        _lib().grb_comm_close(p)
        self._ptrs.clear()
        for b in self.local.values():
            b.free()
        self.local.clear()
