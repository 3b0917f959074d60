"""Process-per-GPU set-up of the peer-memory communicator (q4_comm_*): every rank creates its inbox, the
64-byte IPC handles are exchanged through torch.distributed, and every rank maps its peers' inboxes."""
import ctypes as C

from . import _lib
from ._lib import check


class ProcessComm:
    def __init__(self, rank, world, dist, lib=None):
        L = lib or _lib.lib()
        self._L = L
        self.rank, self.world = rank, world
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

    def attach_nccl(self, dist):
        """Creates an NCCL communicator beside the peer-memory one (rank 0's id is broadcast through torch.distributed)."""
        L = self._L
        if not L.q4_comm_nccl_available():
            raise RuntimeError("libnccl.so.2 cannot be opened")
        buf = C.create_string_buffer(128)
        if self.rank == 0:
            check(L.q4_comm_nccl_unique_id(buf), "nccl_unique_id")
        ids = [bytes(buf.raw)]
        dist.broadcast_object_list(ids, src=0)
        buf = C.create_string_buffer(ids[0], 128)
        check(L.q4_comm_nccl_init(self.handle, buf), "nccl_init")

    def set_backend(self, backend):
        check(self._L.q4_comm_set_backend(self.handle, backend), "set_backend")

    def status(self):
        return self._L.q4_comm_status(self.handle)

    def close(self):
        if self.handle:
            self._L.q4_comm_destroy(self.handle)
            self.handle = C.c_void_p()
