"""N-D process mesh: pp x dp_replicate x dp_shard x cp x tp (tp innermost), plus ep / etp views for MoE.

Dimension names and derived meshes follow data_pipeline/trainer/distributed/parallel_dims.py:1039-1317
(dp_shard = -1 means "whatever is left"; fsdp = dp_shard * cp, batch = dp_replicate * dp_shard,
loss = batch * cp) and the rank layout of data_pipeline/trainer/distributed/tensor_parallel.py:260-306
(rank = dp * (pp * tp) + pp_idx * tp + tp_idx is the 3-D special case).  Groups are created lazily with
`dist.new_group` so that the same code runs on NCCL and on gloo (CPU tests).  Topology facts used for defaults
on B200 / NVSwitch: every GPU of a node reaches every peer at full NVLink bandwidth, so dimension placement inside
a node is not bandwidth-sensitive; tp and cp are still innermost to keep them inside one node on multi-node jobs.
"""
from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from typing import Sequence

import torch
import torch.distributed as dist

NVLINK5_GBPS_PER_DIRECTION = 900.0
DIM_ORDER = ("pp", "dp_replicate", "dp_shard", "cp", "tp")


@dataclass
class ParallelDimsConfig:
    dp_replicate: int = 1
    dp_shard: int = -1
    cp: int = 1
    tp: int = 1
    pp: int = 1
    ep: int = 1
    etp: int = 1
    sp: bool = False
    world_size: int = 1

    def resolve(self) -> "ParallelDimsConfig":
        fixed = self.dp_replicate * self.cp * self.tp * self.pp
        if self.world_size % fixed != 0:
            raise ValueError(f"world size {self.world_size} is not divisible by dp_replicate*cp*tp*pp = {fixed}")
        shard = self.world_size // fixed if self.dp_shard in (-1, 0) else self.dp_shard
        if shard * fixed != self.world_size:
            raise ValueError(f"dp_replicate({self.dp_replicate}) * dp_shard({shard}) * cp({self.cp}) * tp({self.tp}) * "
                             f"pp({self.pp}) != world size {self.world_size}")
        if self.ep > 1 and (shard * self.cp * self.dp_replicate) % self.ep != 0 and (shard * self.cp) % self.ep != 0:
            raise ValueError(f"ep({self.ep}) must divide the data-parallel ranks")
        return ParallelDimsConfig(self.dp_replicate, shard, self.cp, self.tp, self.pp, self.ep, self.etp, self.sp,
                                  self.world_size)


class ParallelDims:
    """Coordinates of this rank and the process groups along every (possibly flattened) dimension."""

    def __init__(self, cfg: ParallelDimsConfig, rank: int | None = None, create_groups: bool = True):
        self.cfg = cfg.resolve()
        self.rank = rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0)
        self.sizes = {d: getattr(self.cfg, d) for d in DIM_ORDER}
        self.coords = self._coords_of(self.rank)
        self._groups: dict[str, dist.ProcessGroup | None] = {}
        self._group_ranks: dict[str, list[int]] = {}
        self._create = create_groups and dist.is_initialized() and dist.get_world_size() > 1

    # ---------------------------------------------------------------- layout arithmetic
    def _coords_of(self, rank: int) -> dict[str, int]:
        out, r = {}, rank
        for d in reversed(DIM_ORDER):
            out[d] = r % self.sizes[d]
            r //= self.sizes[d]
        return out

    def rank_of(self, **coords) -> int:
        c = dict(self.coords)
        c.update(coords)
        r = 0
        for d in DIM_ORDER:
            r = r * self.sizes[d] + c[d]
        return r

    def ranks_along(self, dims: Sequence[str], rank: int | None = None) -> list[int]:
        """Ranks that share every coordinate with `rank` except along `dims` (ordered, outer dim first)."""
        base = self._coords_of(self.rank if rank is None else rank)
        out = []
        for combo in itertools.product(*[range(self.sizes[d]) for d in dims]):
            c = dict(base)
            c.update(dict(zip(dims, combo)))
            r = 0
            for d in DIM_ORDER:
                r = r * self.sizes[d] + c[d]
            out.append(r)
        return out

    _FLAT = {"fsdp": ("dp_shard", "cp"), "batch": ("dp_replicate", "dp_shard"), "loss": ("dp_replicate", "dp_shard", "cp"),
             "dp": ("dp_replicate", "dp_shard"), "dp_cp": ("dp_replicate", "dp_shard", "cp")}

    def dims_of(self, name: str) -> tuple[str, ...]:
        return self._FLAT.get(name, (name,))

    def size(self, name: str) -> int:
        n = 1
        for d in self.dims_of(name):
            n *= self.sizes[d]
        return n

    def local_rank(self, name: str) -> int:
        r = 0
        for d in self.dims_of(name):
            r = r * self.sizes[d] + self.coords[d]
        return r

    def enabled(self, name: str) -> bool:
        return self.size(name) > 1

    # ---------------------------------------------------------------- groups
    def group(self, name: str):
        """Process group along `name` (None when its size is 1 or torch.distributed is not running)."""
        if name in self._groups:
            return self._groups[name]
        dims = self.dims_of(name)
        if self.size(name) == 1 or not self._create:
            self._groups[name] = None
            self._group_ranks[name] = self.ranks_along(dims)
            return None
        mine = None
        seen = set()
        for r in range(self.cfg.world_size):   # every rank creates every group, in the same order
            ranks = tuple(self.ranks_along(dims, r))
            if ranks in seen:
                continue
            seen.add(ranks)
            g = dist.new_group(list(ranks))
            if self.rank in ranks:
                mine = g
                self._group_ranks[name] = list(ranks)
        self._groups[name] = mine
        return mine

    def group_ranks(self, name: str) -> list[int]:
        if name not in self._group_ranks:
            self.group(name)
        return self._group_ranks[name]

    # pipeline helpers
    @property
    def pp_stage(self) -> int:
        return self.coords["pp"]

    @property
    def is_first_stage(self) -> bool:
        return self.coords["pp"] == 0

    @property
    def is_last_stage(self) -> bool:
        return self.coords["pp"] == self.sizes["pp"] - 1

    def pp_neighbor(self, delta: int) -> int:
        return self.rank_of(pp=(self.coords["pp"] + delta) % self.sizes["pp"])

    def describe(self) -> str:
        return " x ".join(f"{d}={self.sizes[d]}" for d in DIM_ORDER) + f" | rank {self.rank} at {self.coords}"


class MeshView:
    """One named view of the mesh: ordered dimension names (outer first), their sizes, this rank's coordinates and
    the process group along every dimension of the view."""

    def __init__(self, name: str, dims: "ParallelDims", axes: Sequence[str]):
        self.name, self.axes = name, tuple(axes)
        self.shape = tuple(dims.size(a) for a in axes)
        self.coords = tuple(dims.local_rank(a) for a in axes)
        self._dims = dims

    def get_group(self, axis: str):
        if axis not in self.axes:
            raise KeyError(f"mesh {self.name!r} has no dimension {axis!r} (has {self.axes})")
        return self._dims.group(axis)

    def size(self, axis: str | None = None) -> int:
        if axis is None:
            n = 1
            for s in self.shape:
                n *= s
            return n
        return self.shape[self.axes.index(axis)]

    def __repr__(self) -> str:
        return f"MeshView({self.name}: " + " x ".join(f"{a}={s}" for a, s in zip(self.axes, self.shape)) + ")"


def build_mesh(dims: "ParallelDims") -> dict[str, MeshView]:
    """The four views that the layers of a training job index (parallel_dims.py:1225-1317 builds the same set):
      dataloading [pp, batch, cp, tp]              which ranks read the same samples
      loss        [loss]                           ranks whose losses are averaged (dp_replicate * dp_shard * cp)
      dense       [pp, dp_replicate, fsdp, tp]     sharding of dense weights (fsdp = dp_shard * cp)
      sparse      [pp, dp_replicate, fsdp, tp]     expert weights; ep / etp are sub-divisions of fsdp x tp and get their
                                                   groups from `ParallelDims.group("ep")` when ep > 1"""
    return {"dataloading": MeshView("dataloading", dims, ("pp", "batch", "cp", "tp")),
            "loss": MeshView("loss", dims, ("loss",)),
            "dense": MeshView("dense", dims, ("pp", "dp_replicate", "fsdp", "tp")),
            "sparse": MeshView("sparse", dims, ("pp", "dp_replicate", "fsdp", "tp"))}


class MeshCache:
    """Process groups are expensive to create and must be created by all ranks in the same order: one ParallelDims
    (with its lazily created groups and views) per distinct configuration, shared by every engine of the process."""

    _cache: dict[tuple, "ParallelDims"] = {}
    _views: dict[tuple, dict[str, MeshView]] = {}

    @staticmethod
    def _key(cfg: ParallelDimsConfig) -> tuple:
        c = cfg.resolve()
        return (c.pp, c.dp_replicate, c.dp_shard, c.cp, c.tp, c.ep, c.etp, c.world_size)

    @classmethod
    def get(cls, cfg: ParallelDimsConfig, rank: int | None = None) -> "ParallelDims":
        k = cls._key(cfg) + (rank,)
        if k not in cls._cache:
            cls._cache[k] = ParallelDims(cfg, rank)
        return cls._cache[k]

    @classmethod
    def views(cls, cfg: ParallelDimsConfig, rank: int | None = None) -> dict[str, MeshView]:
        k = cls._key(cfg) + (rank,)
        if k not in cls._views:
            cls._views[k] = build_mesh(cls.get(cfg, rank))
        return cls._views[k]

    @classmethod
    def clear(cls) -> None:
        cls._cache.clear()
        cls._views.clear()


def create_parallel_dims_from_config(dist_cfg, world_size: int | None = None, rank: int | None = None) -> ParallelDims:
    """From a SOTAConfig `distributed` section (its `parallel` sub-section and the legacy degree keys)."""
    p = dist_cfg.parallel
    ws = world_size if world_size is not None else (dist.get_world_size() if dist.is_initialized() else 1)
    strat = str(dist_cfg.strategy).lower()
    pp = p.pp if p.pp > 1 else (dist_cfg.num_pipeline_stages if strat in ("zbpp", "pipeline_zbpp", "pipeline", "pp") else 1)
    cp = p.cp if p.cp > 1 else (dist_cfg.context_parallel_size if strat in ("context_parallel", "cp") else 1)
    pp, cp = min(pp, ws), min(cp, ws)
    return ParallelDims(ParallelDimsConfig(p.dp_replicate, p.dp_shard, cp, p.tp, pp, p.ep, p.etp, p.sp, ws), rank)


@dataclass
class MemoryEstimate:
    params_gb: float
    grads_gb: float
    optimizer_gb: float
    activations_gb: float

    @property
    def total_gb(self) -> float:
        return self.params_gb + self.grads_gb + self.optimizer_gb + self.activations_gb


def estimate_memory(n_params: float, dims: ParallelDimsConfig, seq_len: int, micro_batch: int, hidden: int, layers: int,
                    checkpointing: bool = True, keep_params_gathered: bool = True) -> MemoryEstimate:
    """Per-GPU memory model for the flat engine (bf16 params + grads, fp32 master + 2 moments sharded over fsdp)."""
    d = dims.resolve()
    model_split = d.tp * d.pp
    shard = d.dp_shard * d.cp
    p = n_params / model_split
    params = p * 2 / (1 if keep_params_gathered else shard)
    grads = p * 2
    optim = p * 12 / shard
    tokens = seq_len * micro_batch / (d.cp * (d.tp if d.sp else 1))
    per_layer = tokens * hidden * 2 * (2 if checkpointing else 34)
    act = per_layer * layers / d.pp
    gb = 1 / 2 ** 30
    return MemoryEstimate(params * gb, grads * gb, optim * gb, act * gb)


# ------------------------------------------------------------------------------------------------ planning helpers
class HardwareDetector:
    """What the job runs on: GPU count / name / memory, NVLink-connected peers, NUMA node of every GPU.
    After data_pipeline/trainer/distributed/parallel_dims.py:294-760 (read-only: nothing is configured here)."""

    @staticmethod
    def detect() -> dict:
        import os
        info = {"num_gpus": 0, "name": None, "memory_gb": 0.0, "sm_count": 0, "peer_access": [], "numa": {},
                "nvswitch": False}
        if not torch.cuda.is_available():
            return info
        n = torch.cuda.device_count()
        prop = torch.cuda.get_device_properties(0)
        info.update(num_gpus=n, name=prop.name, memory_gb=prop.total_memory / 2 ** 30, sm_count=prop.multi_processor_count)
        peers = [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
        info["peer_access"] = peers
        # every GPU reaching every other one directly is what an NVSwitch box looks like from here
        info["nvswitch"] = n > 2 and all(all(row) for row in peers)
        for i in range(n):
            try:
                bus = torch.cuda.get_device_properties(i).pci_bus_id
                path = f"/sys/bus/pci/devices/0000:{bus:02x}:00.0/numa_node"
                if os.path.exists(path):
                    info["numa"][i] = int(open(path).read().strip())
            except Exception:
                pass
        return info


class MemoryEstimator:
    """Per-GPU bytes of a parallel configuration before anything is allocated
    (data_pipeline/trainer/distributed/parallel_dims.py:771)."""

    @staticmethod
    def estimate_per_gpu_memory(model_params: int, batch_size: int, seq_len: int, hidden_dim: int, num_layers: int,
                                tp_degree: int = 1, pp_degree: int = 1, cp_degree: int = 1, dp_shard_degree: int = 1,
                                use_activation_checkpointing: bool = False, precision_bytes: int = 2,
                                shard_params: bool = False, intermediate_dim: int | None = None) -> int:
        local = model_params / (tp_degree * pp_degree)
        params = local * precision_bytes / (dp_shard_degree if shard_params else 1)
        grads = local * precision_bytes
        optim = local * 12 / dp_shard_degree                      # fp32 master + two Adam moments, sharded
        tokens = batch_size * seq_len / cp_degree
        inter = intermediate_dim or 4 * hidden_dim
        per_layer = tokens * precision_bytes * ((5 * hidden_dim + 2 * inter + inter) / tp_degree + 2 * hidden_dim)
        layers = num_layers / pp_degree
        acts = per_layer * layers
        if use_activation_checkpointing:
            acts = tokens * hidden_dim * precision_bytes * layers + per_layer      # layer inputs + one live layer
        return int(params + grads + optim + acts)

    @staticmethod
    def fits(bytes_needed: int, capacity_gb: float = 180.0, headroom: float = 0.92) -> bool:
        return bytes_needed <= capacity_gb * 2 ** 30 * headroom


class CommAlgorithmSelector:
    """Which implementation a collective of a given size should use on an NVSwitch box: small messages are launch-bound
    (one-shot peer-memory kernels), large ones bandwidth-bound (in-switch reduction when available, else the library
    ring).  After data_pipeline/trainer/distributed/parallel_dims.py:957."""

    def __init__(self, world: int, nvswitch: bool = True, multicast: bool = True):
        self.world, self.nvswitch, self.multicast = world, nvswitch, multicast

    def all_reduce(self, nbytes: int) -> str:
        if self.world == 1:
            return "none"
        if self.nvswitch and nbytes <= 256 << 10:
            return "one_shot_p2p"
        if self.nvswitch and self.multicast:
            return "multimem"
        return "ring"

    def reduce_scatter(self, nbytes: int) -> str:
        if self.world == 1:
            return "none"
        return ("multimem" if self.multicast else "p2p_pull") if self.nvswitch else "ring"

    def bucket_bytes(self) -> int:
        """Gradient bucket size: collective cost on NVSwitch is latency- not link-bound, so buckets only need to
        amortise a launch (tens of MB)."""
        return (80 << 20) if self.nvswitch else (25 << 20)
