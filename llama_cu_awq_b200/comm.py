"""Process-per-GPU set-up of the peer-memory communicator (q4_comm_*): every rank creates its inbox, the
64-byte IPC handles are exchanged through torch.distributed, and every rank maps its peers' inboxes."""
import ctypes as C

from . import _lib
from ._lib import check


class ProcessComm:
    def __init__(self, rank, world, dist):
        L = _lib.lib()
        self._L = L
        self.handle = C.c_void_p()
        check(L.q4_comm_create_local(C.byref(self.handle), world, rank), "comm_create_local")
        buf = C.create_string_buffer(64)
        check(L.q4_comm_export(self.handle, buf), "comm_export")
        handles = [None] * world
        dist.all_gather_object(handles, bytes(buf.raw))
        for peer, h in enumerate(handles):
            if peer != rank:
                check(L.q4_comm_import(self.handle, peer, h), "comm_import")
        dist.barrier()

    def status(self):
        return self._L.q4_comm_status(self.handle)

    def close(self):
        if self.handle:
            self._L.q4_comm_destroy(self.handle)
            self.handle = C.c_void_p()
