"""Process-group bootstrap and the (dp, tp) device mesh
(reference: train/infra.py:115-137, train/train_qwen.py:79-86)."""
from __future__ import annotations

import datetime
import os

import torch
import torch.distributed as dist


def init_distributed(backend: str = "auto", device: str = "auto", timeout_s: int = 1800):
    """Initialise torch.distributed from the torchrun environment (RANK / WORLD_SIZE /
    LOCAL_RANK / MASTER_*); a no-op for single-process runs.  Returns (rank, world, device)."""
    timeout_s = int(os.environ.get("VLMT_PG_TIMEOUT_S", timeout_s))  # short in tests: a lost rank ends the job quickly
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if device == "auto":
        device = "cuda" if torch.cuda.is_available() else "cpu"
    if device == "cuda":
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        if backend == "auto":
            backend = "nccl" if dev.type == "cuda" else "gloo"
        kwargs = {"device_id": dev} if dev.type == "cuda" else {}
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, world, dev


class Mesh:
    """2-D (dp, tp) mesh: TP ranks are adjacent (``rank = dp_rank * tp + tp_rank``) so a
    tensor-parallel group stays inside one NVSwitch domain."""

    def __init__(self, world: int, tp: int, device: torch.device):
        if world % tp:
            raise ValueError(f"world size {world} is not divisible by tp_size {tp}")
        self.world, self.tp, self.dp = world, tp, world // tp
        self.device = device
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.tp_rank, self.dp_rank = self.rank % tp, self.rank // tp
        self.tp_group = self.dp_group = self.world_group = None
        self.mesh = None
        if dist.is_initialized() and world > 1:
            from torch.distributed.device_mesh import init_device_mesh

            self.mesh = init_device_mesh(device.type, (self.dp, tp), mesh_dim_names=("dp", "tp"))
            self.tp_group = self.mesh.get_group("tp")
            self.dp_group = self.mesh.get_group("dp")
            self.world_group = dist.group.WORLD

    def __repr__(self):
        return f"Mesh(world={self.world}, dp={self.dp}, tp={self.tp}, rank={self.rank})"


def get_mesh(tp_size: int, device: torch.device) -> Mesh:
    world = dist.get_world_size() if dist.is_initialized() else 1
    return Mesh(world, tp_size, device)


def get_tp_group(mesh: Mesh):
    return mesh.tp_group


def get_dp_group(mesh: Mesh):
    return mesh.dp_group
