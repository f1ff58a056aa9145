"""Carries the tensor-parallel group's rendezvous bytes between the test processes over a
torch.distributed (gloo) group: the library makes and consumes the bytes, the launcher moves them."""
import torch.distributed as dist

from doppler_b200 import tp


def init_group(dev, rank: int, world: int):
    box = [tp.make_unique_id(dev) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    tp.init_group(dev, rank, world, box[0])


def setup_exchange(dev, rank: int, world: int):
    handles = [None] * world
    dist.all_gather_object(handles, tp.export_exchange(dev))
    tp.attach_exchange(dev, handles)
    dist.barrier()  # nobody pushes before every rank has mapped every area
