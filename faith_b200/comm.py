"""Python handle of the library's communicator (fb_comm): NCCL bound at run time, plus the optional one-shot
all-reduce over NVLink.  One process per GPU; the 128-byte NCCL id travels through an existing torch.distributed
process group (any backend) or is passed in by the caller."""
import ctypes

import torch

from . import _lib
from ._lib import check, load

ALGO_NCCL, ALGO_ONESHOT = 0, 1
SUM, MAX = 0, 1


class Comm:
    def __init__(self, handle, rank, world, oneshot_floats):
        self._h = handle
        self.rank, self.world, self.oneshot_floats = rank, world, oneshot_floats

    @staticmethod
    def unique_id():
        buf = ctypes.create_string_buffer(128)
        check(load().fb_comm_unique_id(buf), "fb_comm_unique_id")
        return buf.raw

    @classmethod
    def create(cls, unique_id, rank, world, oneshot_floats=0):
        """The current CUDA device is the communicator's device."""
        h = ctypes.c_void_p()
        check(load().fb_comm_create(ctypes.byref(h), ctypes.c_char_p(unique_id), rank, world, oneshot_floats),
              "fb_comm_create")
        return cls(h, rank, world, oneshot_floats)

    @classmethod
    def from_process_group(cls, group=None, oneshot_floats=0):
        """Builds the communicator over the ranks of a torch.distributed group: rank 0 makes the id, a broadcast of one
        Python object carries it."""
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        box = [cls.unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls.create(box[0], rank, world, oneshot_floats)

    def all_reduce(self, buf, op=SUM, algo=ALGO_NCCL):
        if buf.dtype != torch.float32 or not buf.is_cuda or not buf.is_contiguous():
            raise _lib.FaithError("all_reduce needs a contiguous float32 CUDA tensor")
        with torch.cuda.device(buf.device):
            check(load().fb_allreduce_f32(self._h, buf.data_ptr(), buf.numel(), op, algo,
                                          torch.cuda.current_stream().cuda_stream), "fb_allreduce_f32")
        return buf

    def check(self, sync=False):
        check(load().fb_comm_check(self._h, 1 if sync else 0), "fb_comm_check")

    def set_wait_ns(self, ns):
        check(load().fb_comm_set_wait_ns(self._h, ns), "fb_comm_set_wait_ns")

    def abort(self):
        check(load().fb_comm_abort(self._h), "fb_comm_abort")

    def destroy(self):
        if self._h is not None:
            h, self._h = self._h, None
            check(load().fb_comm_destroy(h), "fb_comm_destroy")
