"""Multicast (NVSwitch) output buffer for the N-sharded product, one process per GPU.

`MulticastBuffer` builds what `btm_gemm_nshard_mc` needs: a full-size C on every rank, all bound to one multicast
object. The rank that creates the object gets a POSIX file descriptor for it; a descriptor is only meaningful inside
its own process, so it travels to the other ranks as ancillary data (SCM_RIGHTS) over a Unix-domain socket whose path
is agreed through the process group. Everything else is the C ABI (btm_mc_*).

All ranks must call `release()` (it barriers first): on NVSwitch systems a process must not disappear while its memory
is still bound to a multicast object that other ranks use.
"""
from __future__ import annotations

import ctypes as C
import os
import socket
import tempfile

from . import _lib


def supported(device: int) -> bool:
    return bool(_lib.lib().btm_mc_supported(device))


class MulticastBuffer:
    def __init__(self, dist, device: int, rank: int, world: int, nbytes: int):
        L = _lib.lib()
        self.L, self.dist, self.device, self.rank, self.world = L, dist, device, rank, world
        self.handle = C.c_void_p()
        self.local_ptr = None
        self.mc_ptr = None
        # Every rank says whether its device can take part; one refusal and nobody tries.
        votes = [None] * world
        dist.all_gather_object(votes, supported(device))
        if not all(votes):
            raise NotImplementedError("multicast objects are not supported on every rank's device")
        path = [None]
        server = None
        if rank == 0:
            path[0] = os.path.join(tempfile.mkdtemp(prefix="btm_mc_"), "fd.sock")
            server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
            server.bind(path[0])
            server.listen(world)
            server.settimeout(120)
        dist.broadcast_object_list(path, src=0)
        status = 0
        try:
            if rank == 0:
                fd = C.c_int(-1)
                status = L.btm_mc_create(device, world, nbytes, C.byref(self.handle), C.byref(fd))
                if status:
                    self.error = _lib.last_error()
                for _ in range(world - 1):
                    conn, _addr = server.accept()
                    with conn:
                        if status == 0:
                            socket.send_fds(conn, [b"ok"], [fd.value])
                        else:
                            conn.sendall(b"no")
                if status == 0:
                    os.close(fd.value)
            else:
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as c:
                    c.settimeout(120)
                    c.connect(path[0])
                    msg, fds, _flags, _addr = socket.recv_fds(c, 16, 1)
                if msg == b"ok" and fds:
                    status = L.btm_mc_import(device, world, nbytes, fds[0], C.byref(self.handle))
                    if status:
                        self.error = _lib.last_error()
                    os.close(fds[0])
                else:
                    status = _lib.ERR_UNSUPPORTED
                    self.error = "the creating rank could not make the multicast object"
        finally:
            if server is not None:
                server.close()
                try:
                    os.unlink(path[0])
                    os.rmdir(os.path.dirname(path[0]))
                except OSError:
                    pass
        # All ranks go on or none does: a bind waits until every rank of the team has added its device.
        codes = [None] * world
        dist.all_gather_object(codes, int(status))
        if any(codes):
            self._drop()
            raise NotImplementedError("multicast object could not be created or opened on every rank: " + getattr(self, "error", "another rank failed"))
        status = L.btm_mc_add_device(self.handle)
        err = _lib.last_error() if status else ""
        dist.all_gather_object(codes, int(status))
        if any(codes):
            self.release(barrier=True)
            raise NotImplementedError("a device could not be added to the multicast object: " + (err or "another rank failed"))
        local, mc = C.c_void_p(), C.c_void_p()
        status = L.btm_mc_bind(self.handle, C.byref(local), C.byref(mc))
        err = _lib.last_error() if status else ""
        dist.all_gather_object(codes, int(status))
        if any(codes):
            self.release(barrier=True)
            raise NotImplementedError("multicast memory could not be bound on every rank: " + (err or "another rank failed"))
        self.local_ptr, self.mc_ptr = local.value, mc.value

    def _drop(self):
        if self.handle:
            self.L.btm_mc_release(self.handle)
            self.handle = C.c_void_p()

    def release(self, barrier: bool = True):
        """Unmap, unbind and free on every rank, while all ranks are still here."""
        import torch
        if barrier:
            torch.cuda.synchronize()
            self.dist.barrier()
        self._drop()
        if barrier:
            self.dist.barrier()
