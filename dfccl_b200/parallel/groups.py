"""Process-group plumbing: one process per GPU, ``torch.distributed`` only for rendezvous
(and for pipeline send / recv); every collective on the data path goes through the daemon."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional

import torch

from .. import native as nv


@dataclass
class Dist:
    rank: int
    world: int
    local_rank: int
    device: torch.device
    comm: nv.Comm
    torch_dist: bool

    def barrier(self) -> None:
        if self.torch_dist:
            import torch.distributed as dist
            dist.barrier()

    def destroy(self) -> None:
        self.comm.destroy()
        if self.torch_dist:
            import torch.distributed as dist
            dist.destroy_process_group()


def init_distributed(backend: Optional[str] = None) -> Dist:
    """Read RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* from the environment, bind the GPU and
    create the world communicator of this library (its unique id travels over
    ``torch.distributed``).  With WORLD_SIZE unset this is a single-rank job."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available() and backend != "host"
    if cuda:
        torch.cuda.set_device(local)
        nv.set_backend("cuda")
        device = torch.device("cuda", local)
    else:
        nv.set_backend("host")
        device = torch.device("cpu")
    if world == 1:
        (comm,) = nv.Comm.init_loopback(1, local if cuda else 0)
        return Dist(0, 1, local, device, comm, False)
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo", rank=rank, world_size=world,
                                device_id=device if cuda else None)
    box = [nv.get_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    comm = nv.Comm.init_rank(world, box[0], rank)
    return Dist(rank, world, local, device, comm, True)
