"""DeviceMesh composition and ``ParallelDims`` (reference: parallel.py:42-349).

Mesh order is ``(pp, dp | dp_replicate, dp_shard, [ep], [cp], [tp])`` with tp innermost, so TP peers
are adjacent ranks; size-1 ep/cp/tp dims are omitted, pp and dp are always present. On one NVSwitch
box every dimension has the same all-to-all bandwidth, so the order only fixes rank numbering.
``build_world_mesh`` keeps a process-wide mesh like the reference but may be called again with
``replace=True`` (the reference raises on any second call).
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import List, Optional

import torch.distributed as dist
from torch.distributed.device_mesh import DeviceMesh, init_device_mesh

log = logging.getLogger(__name__)


class MeshDimName:
    dp = "dp"
    dp_replicate = "dp_replicate"
    dp_shard = "dp_shard"
    tp = "tp"
    cp = "cp"
    pp = "pp"
    ep = "ep"


_WORLD_MESH: Optional[DeviceMesh] = None


def get_world_mesh() -> Optional[DeviceMesh]:
    return _WORLD_MESH


def reset_world_mesh() -> None:
    global _WORLD_MESH
    _WORLD_MESH = None


def mesh_layout(world_size: int, *, dp_size: Optional[int] = None, tp_size: int = 1, pp_size: int = 1,
                cp_size: int = 1, ep_size: int = 1, dp_shard: Optional[int] = None,
                dp_replicate: Optional[int] = None) -> tuple[list[int], list[str]]:
    """Shape and dim names of the mesh (pure function; used by tests and by ``ParallelDims``)."""
    if dp_shard is not None and dp_replicate is not None:
        dp_size = dp_shard * dp_replicate
    if dp_size is None:
        denom = tp_size * pp_size * cp_size * ep_size
        if world_size % denom:
            raise ValueError(f"world_size ({world_size}) is not divisible by tp*pp*cp*ep ({denom})")
        dp_size = world_size // denom
    if world_size != tp_size * pp_size * cp_size * dp_size * ep_size:
        raise ValueError(f"world_size ({world_size}) must equal tp ({tp_size}) * pp ({pp_size}) * cp ({cp_size})"
                         f" * dp ({dp_size}) * ep ({ep_size})")
    shape, names = [pp_size], [MeshDimName.pp]
    if dp_shard is not None and dp_replicate is not None:
        shape += [dp_replicate, dp_shard]
        names += [MeshDimName.dp_replicate, MeshDimName.dp_shard]
    else:
        shape.append(dp_size)
        names.append(MeshDimName.dp)
    for size, name in ((ep_size, MeshDimName.ep), (cp_size, MeshDimName.cp), (tp_size, MeshDimName.tp)):
        if size > 1:
            shape.append(size)
            names.append(name)
    return shape, names


def build_world_mesh(*, world_size: Optional[int] = None, dp_size: Optional[int] = None, tp_size: int = 1,
                     pp_size: int = 1, cp_size: int = 1, ep_size: int = 1, dp_shard: Optional[int] = None,
                     dp_replicate: Optional[int] = None, device_type: str = "cpu",
                     replace: bool = False) -> DeviceMesh:
    global _WORLD_MESH
    if _WORLD_MESH is not None and not replace:
        raise RuntimeError("World mesh already exists!")
    if world_size is None:
        world_size = dist.get_world_size() if dist.is_initialized() else 1
    shape, names = mesh_layout(world_size, dp_size=dp_size, tp_size=tp_size, pp_size=pp_size, cp_size=cp_size,
                               ep_size=ep_size, dp_shard=dp_shard, dp_replicate=dp_replicate)
    mesh = init_device_mesh(device_type, tuple(shape), mesh_dim_names=tuple(names))
    log.info("Built device mesh: %s = %s", names, shape)
    _WORLD_MESH = mesh
    return mesh


def _names(mesh: DeviceMesh) -> tuple:
    return tuple(mesh.mesh_dim_names or ())


def _sub(mesh: DeviceMesh, name: str) -> Optional[DeviceMesh]:
    return mesh[name] if name in _names(mesh) else None


def get_dp_model_mesh(world_mesh: Optional[DeviceMesh] = None, device_mesh: Optional[DeviceMesh] = None) -> Optional[DeviceMesh]:
    """The mesh FSDP shards over: the dp dims (both of them under HSDP), never cp/tp/pp."""
    mesh = world_mesh or device_mesh or _WORLD_MESH   # ``device_mesh``: the reference's name for the argument
    if mesh is None:
        return None
    names = _names(mesh)
    if MeshDimName.dp_replicate in names and MeshDimName.dp_shard in names:
        return mesh[MeshDimName.dp_replicate, MeshDimName.dp_shard]
    return _sub(mesh, MeshDimName.dp)


def get_dp_mesh(world_mesh: Optional[DeviceMesh] = None, device_mesh: Optional[DeviceMesh] = None) -> Optional[DeviceMesh]:
    """The mesh the data loader shards over (CP/TP peers of one dp index read the same batch)."""
    mesh = world_mesh or device_mesh or _WORLD_MESH   # ``device_mesh``: the reference's name for the argument
    if mesh is None:
        return None
    names = _names(mesh)
    if MeshDimName.dp in names:
        return mesh[MeshDimName.dp]
    if MeshDimName.dp_shard in names:
        return mesh[MeshDimName.dp_replicate, MeshDimName.dp_shard]
    return None


def get_tp_mesh(world_mesh: Optional[DeviceMesh] = None, device_mesh: Optional[DeviceMesh] = None):
    mesh = world_mesh or device_mesh or _WORLD_MESH   # ``device_mesh``: the reference's name for the argument
    return None if mesh is None else _sub(mesh, MeshDimName.tp)


def get_cp_mesh(world_mesh: Optional[DeviceMesh] = None, device_mesh: Optional[DeviceMesh] = None):
    mesh = world_mesh or device_mesh or _WORLD_MESH   # ``device_mesh``: the reference's name for the argument
    return None if mesh is None else _sub(mesh, MeshDimName.cp)


def get_pp_mesh(world_mesh: Optional[DeviceMesh] = None, device_mesh: Optional[DeviceMesh] = None):
    mesh = world_mesh or device_mesh or _WORLD_MESH   # ``device_mesh``: the reference's name for the argument
    return None if mesh is None else _sub(mesh, MeshDimName.pp)


def get_ep_mesh(world_mesh: Optional[DeviceMesh] = None, device_mesh: Optional[DeviceMesh] = None):
    """The ep dim; without one, experts are spread over dp_shard (then dp), as in the reference."""
    mesh = world_mesh or device_mesh or _WORLD_MESH   # ``device_mesh``: the reference's name for the argument
    if mesh is None:
        return None
    for n in (MeshDimName.ep, MeshDimName.dp_shard, MeshDimName.dp):
        if n in _names(mesh):
            return mesh[n]
    return None


def get_expert_replica_group(world_mesh: Optional[DeviceMesh] = None):
    """Process group of the ranks that hold the *same expert shard* as this rank and see different tokens: the data-
    parallel dims that expert parallelism does not use, times cp. With an explicit ep dim those are all dp dims (eight
    ranks with ``ep_size=2`` keep four copies of every expert, whose gradients have to be summed); without one the
    experts are spread over dp_shard (or dp) itself and only dp_replicate / cp are left. ``None`` when that product
    is 1. Collective over the mesh."""
    mesh = world_mesh or _WORLD_MESH
    if mesh is None:
        return None
    names = _names(mesh)
    dp_dims = [n for n in names if n in (MeshDimName.dp, MeshDimName.dp_replicate, MeshDimName.dp_shard)]
    if MeshDimName.ep not in names:
        for n in (MeshDimName.dp_shard, MeshDimName.dp):     # the dim get_ep_mesh hands to the experts
            if n in dp_dims:
                dp_dims.remove(n)
                break
    rep = [n for n in dp_dims + ([MeshDimName.cp] if MeshDimName.cp in names else []) if mesh[n].size() > 1]
    if not rep:
        return None
    if len(rep) == 1:
        return mesh[rep[0]].get_group()
    return mesh[tuple(n for n in names if n in rep)]._flatten("expert_replica").get_group()


def get_hsdp_groups(world_mesh: Optional[DeviceMesh] = None):
    """``(shard_group, replicate_group)`` when the mesh has ``dp_replicate`` and ``dp_shard`` dims (hybrid sharding):
    state is sharded over dp_shard (x ep x cp) and replicated over dp_replicate. ``(None, None)`` otherwise."""
    mesh = world_mesh or _WORLD_MESH
    if mesh is None:
        return None, None
    names = _names(mesh)
    if MeshDimName.dp_replicate not in names or MeshDimName.dp_shard not in names:
        return None, None
    if mesh[MeshDimName.dp_replicate].size() <= 1:
        return None, None
    inner = [n for n in names if n in (MeshDimName.dp_shard, MeshDimName.ep, MeshDimName.cp) and mesh[n].size() > 1]
    if not inner:
        shard = None
    elif len(inner) == 1:
        shard = mesh[inner[0]].get_group()
    else:
        shard = mesh[tuple(inner)]._flatten("hsdp_shard").get_group()
    return shard, mesh[MeshDimName.dp_replicate].get_group()


def get_replica_group(world_mesh: Optional[DeviceMesh] = None):
    """Process group of the ranks that hold the *same* (non-expert) parameters as this rank and see different
    tokens: the product of the dp (or dp_replicate x dp_shard), ep and cp dims. Gradients of replicated parameters
    are averaged over exactly this group; tensor- and pipeline-parallel peers hold other shards / stages and stay
    out. ``None`` when that product is 1; the world group when it is the whole world. Collective over the mesh."""
    mesh = world_mesh or _WORLD_MESH
    if mesh is None:
        return None
    rep = [n for n in _names(mesh) if n in (MeshDimName.dp, MeshDimName.dp_replicate, MeshDimName.dp_shard,
                                             MeshDimName.ep, MeshDimName.cp)]
    size = 1
    for n in rep:
        size *= mesh[n].size()
    if size <= 1:
        return None
    if size == mesh.size():
        return dist.group.WORLD
    if len(rep) == 1:
        return mesh[rep[0]].get_group()
    return mesh[tuple(rep)]._flatten("replica").get_group()


def data_parallel_coords(world_mesh: Optional[DeviceMesh] = None) -> tuple[int, int]:
    """(index, count) of this rank among the ranks that read *different* batches: dp x ep.
    EP peers process different tokens for the dense layers, so they count as data-parallel here."""
    mesh = world_mesh or _WORLD_MESH
    if mesh is None:
        return 0, 1
    idx, cnt = 0, 1
    for n in _names(mesh):
        if n in (MeshDimName.dp, MeshDimName.dp_replicate, MeshDimName.dp_shard, MeshDimName.ep):
            size = mesh[n].size()
            idx = idx * size + mesh[n].get_local_rank()
            cnt *= size
    return idx, cnt


@dataclass
class ParallelDims:
    dp_shard: int = 1
    dp_replicate: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    _world_size: Optional[int] = field(default=None, repr=False)
    _mesh: Optional[DeviceMesh] = field(default=None, repr=False)

    def __post_init__(self):
        self._validate()

    def _validate(self):
        for n in ("dp_replicate", "tp", "pp", "cp", "ep"):
            if getattr(self, n) < 1:
                raise ValueError(f"{n} must be >= 1")
        if self.dp_shard < 1 and self.dp_shard != -1:
            raise ValueError("dp_shard must be >= 1, or -1 to be inferred from the world size")

    @property
    def dp(self) -> int:
        return self.dp_shard * self.dp_replicate

    @property
    def world_size(self) -> int:
        return self.dp_replicate * max(self.dp_shard, 1) * self.tp * self.pp * self.cp * self.ep

    def set_world_size(self, world_size: int) -> "ParallelDims":
        """Infer ``dp_shard`` (if -1) or ``dp_replicate`` so the product matches ``world_size``."""
        rest = self.tp * self.pp * self.cp * self.ep
        if world_size % rest:
            raise ValueError(f"world_size {world_size} not divisible by tp*pp*cp*ep = {rest}")
        dp = world_size // rest
        self._world_size = world_size
        if self.dp_shard == -1:
            if dp % self.dp_replicate:
                raise ValueError("dp_replicate does not divide the data-parallel size")
            self.dp_shard = dp // self.dp_replicate
        elif self.dp_replicate == 1:
            if dp % self.dp_shard:
                raise ValueError("dp_shard does not divide the data-parallel size")
            self.dp_replicate = dp // self.dp_shard
        elif self.world_size != world_size:
            # both data-parallel factors were given: they have to fit (reference: parallel.py:273-297)
            raise ValueError(f"parallel dims multiply to {self.world_size}, world_size is {world_size}")
        return self

    @property
    def dp_enabled(self) -> bool:
        return self.dp > 1

    def layout(self) -> tuple[list[int], list[str]]:
        hsdp = self.dp_replicate > 1 and self.dp_shard > 1
        return mesh_layout(self.world_size, dp_size=None if hsdp else self.dp, tp_size=self.tp, pp_size=self.pp,
                           cp_size=self.cp, ep_size=self.ep, dp_shard=self.dp_shard if hsdp else None,
                           dp_replicate=self.dp_replicate if hsdp else None)

    def build_mesh(self, device_type: str = "cpu") -> DeviceMesh:
        hsdp = self.dp_replicate > 1 and self.dp_shard > 1
        self._mesh = build_world_mesh(world_size=self.world_size, dp_size=None if hsdp else self.dp,
                                      tp_size=self.tp, pp_size=self.pp, cp_size=self.cp, ep_size=self.ep,
                                      dp_shard=self.dp_shard if hsdp else None,
                                      dp_replicate=self.dp_replicate if hsdp else None, device_type=device_type,
                                      replace=True)
        return self._mesh

    @property
    def mesh(self) -> Optional[DeviceMesh]:
        return self._mesh
