"""NVSwitch multicast (NVLS) buffers: one allocation per rank, all bound to ONE multicast object.

A store to the multicast address (``multimem.st`` from a kernel) is replicated by the switch into every rank's copy
of the buffer: the data leaves the writing GPU once instead of once per peer.  The data-parallel mode uses it for the
bf16 weight mirror: the owner of a parameter writes the new bf16 value once and all replicas receive it
(``csrc/optim.cu``, the ``mc16`` argument of the sharded Schedule-Free AdamW kernels).  Opt-in (``GRB_NVLS=1``): a
rank that dies while its memory is bound to a multicast object can disturb its peers' GPUs, so failure-handling
tests and unattended runs keep to plain peer stores.

Set-up (once per buffer, host side, CUDA driver API through cuda-python):
  rank 0   cuMulticastCreate(size, world devices) -> export as a POSIX file descriptor -> sent to the other ranks of
           the box over a Unix-domain socket (SCM_RIGHTS), the only way a descriptor can cross processes
  all      cuMulticastAddDevice; host barrier; cuMemCreate (own physical memory) ; cuMulticastBindMem;
           map the own memory at one address (ordinary loads / stores / TMA) and the multicast object at another

The reference has nothing comparable (its transport is TCP, gossip/network_utils.py); this belongs to the NVLink
data plane that replaces it.
"""
from __future__ import annotations

import array
import os
import socket
import time

import torch

try:
    from cuda.bindings import driver as cu
except ImportError:      # older cuda-python
    from cuda import cuda as cu


class NvlsUnavailable(RuntimeError):
    pass


def _ck(res, what: str):
    err = res[0]
    if int(err) != 0:
        raise NvlsUnavailable(f"{what}: CUDA driver error {int(err)} ({err})")
    return res[1] if len(res) == 2 else res[1:]


def supported(device_index: int) -> bool:
    """Whether the driver reports multicast support for this device (False on any error)."""
    try:
        _ck(cu.cuInit(0), "cuInit")
        dev = _ck(cu.cuDeviceGet(device_index), "cuDeviceGet")
        return bool(_ck(cu.cuDeviceGetAttribute(cu.CUdevice_attribute.CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev),
                        "cuDeviceGetAttribute"))
    except Exception:
        return False


def _send_fd(path: str, fd: int, n_peers: int, timeout: float = 60.0) -> None:
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    try:
        if os.path.exists(path):
            os.unlink(path)
        srv.bind(path)
        srv.listen(n_peers)
        srv.settimeout(timeout)
        for _ in range(n_peers):
            conn, _ = srv.accept()
            with conn:
                conn.sendmsg([b"F"], [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))])
    finally:
        srv.close()
        if os.path.exists(path):
            os.unlink(path)


def _recv_fd(path: str, timeout: float = 60.0) -> int:
    t0 = time.time()
    while True:
        s = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        try:
            s.connect(path)
            break
        except OSError:
            s.close()
            if time.time() - t0 > timeout:
                raise NvlsUnavailable(f"no multicast handle arrived on {path} within {timeout} s")
            time.sleep(0.05)
    with s:
        fds = array.array("i")
        msg, anc, _, _ = s.recvmsg(1, socket.CMSG_LEN(fds.itemsize))
        for level, typ, data in anc:
            if level == socket.SOL_SOCKET and typ == socket.SCM_RIGHTS:
                fds.frombytes(data[:fds.itemsize])
    if not fds:
        raise NvlsUnavailable("the multicast handle message carried no descriptor")
    return fds[0]


class MulticastBuffer:
    """``nbytes`` of device memory on this rank, bound with the same buffer of every other rank to one multicast
    object.  ``ptr`` addresses the local copy, ``mc_ptr`` all copies at once (stores only)."""

    def __init__(self, name: str, nbytes: int, rank: int, world: int, device: torch.device, host_barrier, sock_dir: str = "/tmp"):
        self.name, self.rank, self.world, self.device = name, rank, world, torch.device(device)
        idx = self.device.index if self.device.index is not None else torch.cuda.current_device()
        torch.cuda.set_device(idx)
        torch.zeros(1, device=self.device)          # makes sure the primary context exists and is current
        if not supported(idx):
            raise NvlsUnavailable("the driver reports no multicast support on this device")
        dev = _ck(cu.cuDeviceGet(idx), "cuDeviceGet")
        fd_type = cu.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR
        mprop = cu.CUmulticastObjectProp()
        mprop.numDevices = world
        mprop.handleTypes = fd_type
        mprop.flags = 0
        mprop.size = nbytes
        gran = _ck(cu.cuMulticastGetGranularity(mprop, cu.CUmulticastGranularity_flags.CU_MULTICAST_GRANULARITY_RECOMMENDED),
                   "cuMulticastGetGranularity")
        aprop = cu.CUmemAllocationProp()
        aprop.type = cu.CUmemAllocationType.CU_MEM_ALLOCATION_TYPE_PINNED
        aprop.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
        aprop.location.id = idx
        aprop.requestedHandleTypes = fd_type
        agran = _ck(cu.cuMemGetAllocationGranularity(aprop, cu.CUmemAllocationGranularity_flags.CU_MEM_ALLOC_GRANULARITY_RECOMMENDED),
                    "cuMemGetAllocationGranularity")
        g = max(int(gran), int(agran))
        self.nbytes = (nbytes + g - 1) // g * g
        mprop.size = self.nbytes
        path = os.path.join(sock_dir, f"grb_nvls_{os.environ.get('MASTER_PORT', '0')}_{name}.sock")
        if rank == 0:
            self.mc = _ck(cu.cuMulticastCreate(mprop), "cuMulticastCreate")
            fd = _ck(cu.cuMemExportToShareableHandle(self.mc, fd_type, 0), "cuMemExportToShareableHandle")
            try:
                _send_fd(path, int(fd), world - 1)
            finally:
                os.close(int(fd))
        else:
            fd = _recv_fd(path)
            try:
                self.mc = _ck(cu.cuMemImportFromShareableHandle(fd, fd_type), "cuMemImportFromShareableHandle")
            finally:
                os.close(fd)
        _ck(cu.cuMulticastAddDevice(self.mc, dev), "cuMulticastAddDevice")
        host_barrier()                               # every device has joined before anybody binds memory
        self.mem = _ck(cu.cuMemCreate(self.nbytes, aprop, 0), "cuMemCreate")
        _ck(cu.cuMulticastBindMem(self.mc, 0, self.mem, 0, self.nbytes, 0), "cuMulticastBindMem")
        acc = cu.CUmemAccessDesc()
        acc.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
        acc.location.id = idx
        acc.flags = cu.CUmemAccess_flags.CU_MEM_ACCESS_FLAGS_PROT_READWRITE
        self.ptr = int(_ck(cu.cuMemAddressReserve(self.nbytes, g, 0, 0), "cuMemAddressReserve"))
        _ck(cu.cuMemMap(self.ptr, self.nbytes, 0, self.mem, 0), "cuMemMap (local)")
        _ck(cu.cuMemSetAccess(self.ptr, self.nbytes, [acc], 1), "cuMemSetAccess (local)")
        self.mc_ptr = int(_ck(cu.cuMemAddressReserve(self.nbytes, g, 0, 0), "cuMemAddressReserve"))
        _ck(cu.cuMemMap(self.mc_ptr, self.nbytes, 0, self.mc, 0), "cuMemMap (multicast)")
        _ck(cu.cuMemSetAccess(self.mc_ptr, self.nbytes, [acc], 1), "cuMemSetAccess (multicast)")
        host_barrier()                               # every rank's memory is bound before the first multicast store
        self.tensor(torch.uint8, self.nbytes).zero_()
        torch.cuda.synchronize(self.device)

    def tensor(self, dtype: torch.dtype, numel: int | None = None) -> torch.Tensor:
        """Torch view of the LOCAL copy (ordinary memory: kernels, TMA and torch ops may read and write it)."""
        from .comm import _CudaArray, _TYPESTR
        item = torch.empty(0, dtype=dtype).element_size()
        n = self.nbytes // item if numel is None else numel
        t = torch.as_tensor(_CudaArray(self.ptr, n, _TYPESTR[dtype], self), device=self.device)
        return t.view(torch.bfloat16) if dtype == torch.bfloat16 else t
