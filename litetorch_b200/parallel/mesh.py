"""N-dimensional device mesh, placements and DTensor (`lt.distributed.DeviceMesh / Placement / DTensor`).

The reference ships these as data holders whose `get_rank` returns 0 and whose `redistribute` returns null
(include/litetorch/device_mesh.h:10-22, dtensor.h:12-36), and an unused `ncclCommSplit` plan
(src/distributed/distributed.cpp:907-936).  Here a mesh owns one process group per axis (e.g.
dp x pp x cp x tp), and `DTensor.redistribute` really moves data between Shard / Replicate / Partial
placements with all-gather, reduce-scatter, all-reduce or a local slice.
"""
from __future__ import annotations

import enum
import itertools
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from ..core import Tensor, _unwrap


class DeviceMesh:
    def __init__(self, shape: Sequence[int], dim_names="", rank: Optional[int] = None, create_groups: bool = True):
        self.shape = [int(s) for s in shape]
        if isinstance(dim_names, str):
            dim_names = [n for n in dim_names.replace(",", " ").split() if n] or ["dim%d" % i for i in range(len(self.shape))]
        self.dim_names = list(dim_names)
        assert len(self.dim_names) == len(self.shape)
        self.world = 1
        for s in self.shape:
            self.world *= s
        self._rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        self._groups: Dict[str, object] = {}
        self._group_ranks: Dict[str, List[int]] = {}
        for name in self.dim_names:
            self._group_ranks[name] = self.ranks_along(name)
        if create_groups and dist.is_initialized() and dist.get_world_size() == self.world and self.world > 1:
            for ax, name in enumerate(self.dim_names):
                # every rank must create every group, in the same order
                others = [range(s) for i, s in enumerate(self.shape) if i != ax]
                for fixed in itertools.product(*others):
                    ranks = []
                    for k in range(self.shape[ax]):
                        c = list(fixed)
                        c.insert(ax, k)
                        ranks.append(self.rank_of(c))
                    g = dist.new_group(ranks)
                    if self._rank in ranks:
                        self._groups[name] = g

    # row-major rank <-> coordinates
    def coords_of(self, rank: int) -> List[int]:
        c = []
        for s in reversed(self.shape):
            c.append(rank % s)
            rank //= s
        return list(reversed(c))

    def rank_of(self, coords: Sequence[int]) -> int:
        r = 0
        for c, s in zip(coords, self.shape):
            r = r * s + c
        return r

    def get_rank(self, coords: Optional[Sequence[int]] = None) -> int:
        """This process's rank, or with `coords` the rank at those mesh coordinates (the reference's signature,
        src/bindings/python_bindings.cpp:743; its implementation returns 0 for every input)."""
        return self._rank if coords is None else self.rank_of(coords)

    # the reference's field names (include/litetorch/device_mesh.h:12-14)
    @property
    def mesh_shape(self) -> List[int]:
        return self.shape

    @property
    def mesh_dim_names(self) -> str:
        return ",".join(self.dim_names)

    @property
    def mesh_topology(self) -> List[int]:
        return list(range(self.world))

    def get_coordinate(self) -> List[int]:
        return self.coords_of(self._rank)

    def get_local_rank(self, dim) -> int:
        ax = self.dim_names.index(dim) if isinstance(dim, str) else dim
        return self.get_coordinate()[ax]

    def size(self, dim) -> int:
        ax = self.dim_names.index(dim) if isinstance(dim, str) else dim
        return self.shape[ax]

    def ranks_along(self, dim) -> List[int]:
        ax = self.dim_names.index(dim) if isinstance(dim, str) else dim
        c = self.get_coordinate()
        out = []
        for k in range(self.shape[ax]):
            cc = list(c)
            cc[ax] = k
            out.append(self.rank_of(cc))
        return out

    def get_group(self, dim):
        name = dim if isinstance(dim, str) else self.dim_names[dim]
        return self._groups.get(name)


class PlacementType(enum.IntEnum):
    REPLICATE = 0
    SHARD = 1
    PARTIAL = 2


class Placement:
    def __init__(self, type: PlacementType = PlacementType.REPLICATE, dim: int = 0):
        self.type, self.dim = PlacementType(type), dim

    @staticmethod
    def replicate():
        return Placement(PlacementType.REPLICATE)

    @staticmethod
    def shard(dim: int):
        return Placement(PlacementType.SHARD, dim)

    @staticmethod
    def partial():
        return Placement(PlacementType.PARTIAL)

    def __eq__(self, o):
        return isinstance(o, Placement) and o.type == self.type and (self.type != PlacementType.SHARD or o.dim == self.dim)

    def __repr__(self):
        return {0: "Replicate()", 1: "Shard(%d)" % self.dim, 2: "Partial()"}[int(self.type)]


class DTensor:
    """A local shard plus how it relates to the global tensor along every mesh axis."""

    def __init__(self, local_tensor: Tensor, mesh: DeviceMesh, placements: Sequence[Placement]):
        self.local_tensor, self.mesh, self.placements = local_tensor, mesh, list(placements)
        # fewer placements than mesh axes (the reference's guide builds a DTensor on a 2-D mesh from one): the rest replicate
        self.placements += [Placement.replicate() for _ in range(len(mesh.shape) - len(self.placements))]
        assert len(self.placements) == len(mesh.shape)

    @property
    def device_mesh(self) -> DeviceMesh:
        return self.mesh

    def to_local(self) -> Tensor:
        return self.local_tensor

    def full_tensor(self) -> Tensor:
        return self.redistribute([Placement.replicate()] * len(self.placements)).local_tensor

    def redistribute(self, new_mesh=None, new_placements: Optional[Sequence[Placement]] = None, placements=None) -> "DTensor":
        """`redistribute(placements)` or, with the reference's arguments, `redistribute(new_mesh, new_placements)`
        (src/bindings/python_bindings.cpp:762); the mesh must be the tensor's own mesh (same shape)."""
        if placements is None:
            if new_placements is not None:
                placements = new_placements
            elif new_mesh is not None and not isinstance(new_mesh, DeviceMesh):
                placements, new_mesh = new_mesh, None
        if isinstance(new_mesh, DeviceMesh) and list(new_mesh.shape) != list(self.mesh.shape):
            raise ValueError("redistribute onto a mesh of another shape is not supported: %s vs %s" % (new_mesh.shape, self.mesh.shape))
        if placements is None:
            raise TypeError("redistribute needs the new placements")
        t = _unwrap(self.local_tensor)
        cur = list(self.placements)
        for ax, (src, dst) in enumerate(zip(cur, placements)):
            if src == dst:
                continue
            n = self.mesh.shape[ax]
            g = self.mesh.get_group(ax)
            live = dist.is_initialized() and n > 1 and g is not None
            k = self.mesh.get_local_rank(ax)
            if src.type == PlacementType.SHARD and dst.type == PlacementType.REPLICATE:
                if live:
                    parts = [torch.empty_like(t) for _ in range(n)]
                    dist.all_gather(parts, t.contiguous(), group=g)
                    t = torch.cat(parts, src.dim)
            elif src.type == PlacementType.REPLICATE and dst.type == PlacementType.SHARD:
                t = t.chunk(n, dst.dim)[k].contiguous()
            elif src.type == PlacementType.PARTIAL and dst.type == PlacementType.REPLICATE:
                if live:
                    t = t.clone()
                    dist.all_reduce(t, group=g)
            elif src.type == PlacementType.PARTIAL and dst.type == PlacementType.SHARD:
                if live:
                    t = t.clone()
                    dist.all_reduce(t, group=g)
                t = t.chunk(n, dst.dim)[k].contiguous()
            elif src.type == PlacementType.SHARD and dst.type == PlacementType.SHARD:
                if live:
                    parts = [torch.empty_like(t) for _ in range(n)]
                    dist.all_gather(parts, t.contiguous(), group=g)
                    t = torch.cat(parts, src.dim)
                t = t.chunk(n, dst.dim)[k].contiguous()
            elif src.type == PlacementType.REPLICATE and dst.type == PlacementType.PARTIAL:
                t = t if k == 0 else torch.zeros_like(t)
            cur[ax] = dst
        return DTensor(Tensor(t), self.mesh, cur)


def distribute_tensor(tensor: Tensor, mesh: DeviceMesh, placements: Sequence[Placement]) -> DTensor:
    return DTensor(tensor, mesh, [Placement.replicate()] * len(mesh.shape)).redistribute(placements)
