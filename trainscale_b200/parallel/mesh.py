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

from ..utils.refargs import ANY, reference_kwargs

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

    @reference_kwargs(config="cfg")
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

    # ---------------------------------------------------------------- the reference's accessors
    # (data_pipeline/trainer/distributed/parallel_dims.py:1168-1640).  Meshes are `MeshView`s (names, sizes, this rank's
    # coordinates, process groups created on demand) instead of torch DeviceMesh objects.
    @classmethod
    def create(cls, world_size: int, dp_replicate: int = 1, dp_shard: int = -1, cp: int = 1, tp: int = 1, pp: int = 1,
               ep: int = 1, etp: int = 1, sp: int = 1, **kwargs):
        return create_parallel_dims(world_size, dp_replicate, dp_shard, cp, tp, pp, ep, etp, sp, **kwargs)

    @property
    def config(self) -> ParallelDimsConfig:
        return self.cfg

    def build_mesh(self):
        """Ok({view name: MeshView}) for the dataloading / loss / dense / sparse views (built once)."""
        from ..core.types import Err, Ok
        import time
        try:
            if getattr(self, "_views", None) is None:
                t0 = time.perf_counter_ns()
                self._views = build_mesh(self)
                self.metrics.mesh_build_ns += time.perf_counter_ns() - t0
            return Ok(self._views)
        except (RuntimeError, ValueError) as e:
            return Err(e)

    def get_optional_mesh(self, dims):
        """`MeshView` over one dimension name or a list of them; None when every named dimension has size 1."""
        names = [dims] if isinstance(dims, str) else list(dims)
        valid = set(DIM_ORDER) | set(self._FLAT) | {"ep", "etp"}
        for n in names:
            if n not in valid:
                raise ValueError(f"invalid mesh dim {n!r}; valid: {sorted(valid)}")
        m = self.metrics
        m.num_mesh_accesses += 1
        key = tuple(names)
        cache = self.__dict__.setdefault("_mesh_cache", {})
        if key in cache:
            m.num_cache_hits += 1
            return cache[key]
        m.num_cache_misses += 1
        sized = {n: (getattr(self.cfg, n) if n in ("ep", "etp") else self.size(n)) for n in names}
        view = None if all(v == 1 for v in sized.values()) else MeshView("x".join(names), self, [n for n in names])
        cache[key] = view
        return view

    def get_mesh(self, dims):
        view = self.get_optional_mesh(dims)
        if view is None:
            raise ValueError(f"mesh {dims!r} is not available (every named dimension has size 1)")
        return view

    def get_all_1d_meshes(self) -> dict:
        out = {}
        for n in ("pp", "dp_replicate", "dp_shard", "cp", "tp"):
            if self.sizes[n] > 1:
                out[n] = self.get_mesh(n)
        return out

    @property
    def world_mesh(self) -> "MeshView":
        return MeshView("world", self, DIM_ORDER)

    dp_replicate_enabled = property(lambda self: self.cfg.dp_replicate > 1)
    dp_shard_enabled = property(lambda self: self.cfg.dp_shard > 1)
    dp_enabled = property(lambda self: self.cfg.dp_replicate > 1 or self.cfg.dp_shard > 1)
    fsdp_enabled = property(lambda self: self.cfg.dp_shard > 1 or self.cfg.cp > 1)
    cp_enabled = property(lambda self: self.cfg.cp > 1)
    tp_enabled = property(lambda self: self.cfg.tp > 1)
    pp_enabled = property(lambda self: self.cfg.pp > 1)
    ep_enabled = property(lambda self: self.cfg.ep > 1)
    etp_enabled = property(lambda self: self.cfg.etp > 1)
    sp_enabled = property(lambda self: bool(self.cfg.sp))
    fsdp_gradient_divide_factor = property(lambda self: self.cfg.dp_replicate * self.cfg.dp_shard * self.cfg.cp)
    non_data_parallel_size = property(lambda self: self.cfg.cp * self.cfg.tp * self.cfg.pp)
    # tokens per sequence must divide by tp (sequence parallelism) and by 2 * cp (head-tail balanced context shards)
    seq_len_divisor = property(lambda self: self.cfg.tp * self.cfg.cp * 2)
    device_type = property(lambda self: "cuda" if torch.cuda.is_available() else "cpu")
    hardware_vendor = property(lambda self: HardwareDetector.detect_vendor())
    architecture = property(lambda self: HardwareDetector.detect_architecture())
    intra_node_interconnect = property(lambda self: HardwareDetector.detect_intra_node_interconnect())

    @property
    def metrics(self) -> "ParallelDimsMetrics":
        if "_metrics" not in self.__dict__:
            self.__dict__["_metrics"] = ParallelDimsMetrics()
        return self.__dict__["_metrics"]

    def get_communication_algorithm(self, message_size_bytes: int, dim_name: str = "dp_shard") -> "CommunicationAlgorithm":
        """What an all-reduce of that size along `dim_name` should use.  On an NVSwitch node every peer is one hop away,
        so small messages go through one-shot peer kernels and large ones through the in-switch reduction; both are
        reported as NCCL_AUTO / TREE / RING in the reference's vocabulary."""
        n = self.size(dim_name) if dim_name in set(DIM_ORDER) | set(self._FLAT) else 1
        if n <= 1:
            return CommunicationAlgorithm.NCCL_AUTO
        kind = CommAlgorithmSelector(n, nvswitch=HardwareDetector.detect().get("nvswitch", False)).all_reduce(
            message_size_bytes)
        return {"one_shot_p2p": CommunicationAlgorithm.TREE, "multimem": CommunicationAlgorithm.NCCL_AUTO,
                "ring": CommunicationAlgorithm.RING}.get(kind, CommunicationAlgorithm.NCCL_AUTO)

    def estimate_memory_per_gpu(self, model_params: int, batch_size: int, seq_len: int, hidden_dim: int, num_layers: int,
                                use_activation_checkpointing: bool = False, precision_bytes: int = 2) -> int:
        c = self.cfg
        return MemoryEstimator.estimate_per_gpu_memory(
            model_params, max(1, batch_size // max(1, c.dp_replicate * c.dp_shard)), seq_len, hidden_dim, num_layers,
            c.tp, c.pp, c.cp, c.dp_shard * c.dp_replicate, use_activation_checkpointing, precision_bytes)


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


class ParallelDimsMetricsLite:
    """Access counters of `MeshCache` (the full record, `ParallelDimsMetrics`, is defined further down)."""

    def __init__(self):
        self.num_mesh_accesses = self.num_cache_hits = self.num_cache_misses = 0


class MeshCache:
    """Process groups are expensive to create and must be created by all ranks in the same order: one ParallelDims
    (with its lazily created groups and views) per distinct configuration, shared by every engine of the process."""

    _cache: dict[tuple, "ParallelDims"] = {}
    _views: dict[tuple, dict[str, MeshView]] = {}
    metrics = ParallelDimsMetricsLite()

    @staticmethod
    def _key(cfg: ParallelDimsConfig) -> tuple:
        c = cfg.resolve()
        return (c.pp, c.dp_replicate, c.dp_shard, c.cp, c.tp, c.ep, c.etp, c.world_size)

    @classmethod
    def get(cls, cfg: "ParallelDimsConfig | str | None" = None, rank: int | None = None, *, name: str | None = None):
        """`get(cfg, rank)` -> the cached `ParallelDims` of that layout; `get(name)` -> the mesh stored under a
        dimension name by `set` (None when absent)."""
        if name is not None or isinstance(cfg, str):
            return cls.get_named(name if name is not None else cfg)
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
        cls._named.clear()
        cls.metrics = ParallelDimsMetricsLite()

    # name -> mesh store of the reference (parallel_dims.py:600-700): 1-D meshes by dimension name, the flattened
    # "global" meshes (dataloading / dense / sparse) and the world mesh
    _named: dict = {}

    @classmethod
    def set(cls, name: str, mesh) -> None:
        cls._named[("dim", name)] = mesh

    @classmethod
    def set_global(cls, name: str, mesh) -> None:
        cls._named[("global", name)] = mesh

    @classmethod
    def get_global(cls, name: str):
        return cls._lookup(("global", name))

    @classmethod
    def set_world(cls, mesh) -> None:
        cls._named[("world", "")] = mesh

    @classmethod
    def get_world(cls):
        return cls._lookup(("world", ""))

    @classmethod
    def get_named(cls, name: str):
        return cls._lookup(("dim", name))

    @classmethod
    def _lookup(cls, key):
        cls.metrics.num_mesh_accesses += 1
        hit = key in cls._named
        cls.metrics.num_cache_hits += hit
        cls.metrics.num_cache_misses += not hit
        return cls._named.get(key)


@reference_kwargs(config="dist_cfg")
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


def _hd_cc(device: int = 0) -> tuple:
    return torch.cuda.get_device_capability(device) if torch.cuda.is_available() else (0, 0)


def _hd_install():
    """Typed single-fact probes of the reference (parallel_dims.py:294-700) as static methods of `HardwareDetector`,
    all derived from `detect()` / `detect_node_topology()`."""
    H = HardwareDetector
    H.detect_vendor = staticmethod(lambda: HardwareVendor.NVIDIA if torch.cuda.is_available() else HardwareVendor.CPU)
    H.detect_compute_capability = staticmethod(_hd_cc)
    H.detect_architecture = staticmethod(lambda device=0: GPUArchitecture.from_compute_capability(_hd_cc(device))
                                         if torch.cuda.is_available() else GPUArchitecture.UNKNOWN)
    H.detect_node_topology = staticmethod(lambda: detect_node_topology())
    H.detect_numa_topology = staticmethod(lambda: detect_node_topology().numa_topology)
    H.detect_intra_node_interconnect = staticmethod(lambda: detect_node_topology().intra_node_interconnect)
    H.detect_inter_node_interconnect = staticmethod(lambda: detect_cluster_topology().inter_node_interconnect)
    H.detect_nvlink_topology = staticmethod(lambda: {g.index: list(g.nvlink_connected)
                                                     for g in detect_node_topology().gpu_info})

    def get_optimal_device_order() -> list:
        """GPU indices ordered so that neighbours in the list are neighbours in hardware: grouped by NUMA node, inside
        a node by index.  With a switch every order is equally good and the natural order is returned."""
        node = detect_node_topology()
        if node.has_nvswitch or node.numa_topology is None:
            return list(range(node.num_gpus))
        return [g for grp in node.numa_topology.gpus_per_node for g in sorted(grp)]
    H.get_optimal_device_order = staticmethod(get_optimal_device_order)


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

    @staticmethod
    def check_memory_fit(available_memory_bytes: int, estimated_memory_bytes: int, safety_margin: float = 0.9):
        """Ok(None) when the estimate fits `safety_margin` of the available bytes, else Err(MemoryError) with both."""
        from ..core.types import Err, Ok
        usable = int(available_memory_bytes * safety_margin)
        if estimated_memory_bytes > usable:
            return Err(MemoryError(f"estimated {estimated_memory_bytes / 2 ** 30:.2f} GiB exceeds the usable "
                                   f"{usable / 2 ** 30:.2f} GiB"))
        return Ok(None)


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

    # ---- library-level choice (data_pipeline/trainer/distributed/parallel_dims.py:969-1040).  Nothing is set here:
    # `get_nccl_env_vars` RETURNS the variables a launcher may export before the process group is created.
    @staticmethod
    def select_allreduce_algorithm(message_size_bytes: int, num_devices: int, interconnect=None,
                                   has_nvswitch: bool = False) -> "CommunicationAlgorithm":
        """Behind a switch the library's own choice stands (it reduces inside the switch when it can, which beats any
        ring or tree).  Without one: a tree for latency-bound messages (< 256 KiB) or many devices, a ring for
        bandwidth-bound ones (> 4 MiB), the library's choice in between."""
        if num_devices <= 1:
            return CommunicationAlgorithm.AUTO
        if has_nvswitch:
            return CommunicationAlgorithm.NCCL_AUTO
        if message_size_bytes < 256 * 1024:
            return CommunicationAlgorithm.TREE
        if message_size_bytes > 4 * 1024 * 1024:
            return CommunicationAlgorithm.RING
        return CommunicationAlgorithm.NCCL_AUTO

    @staticmethod
    def get_nccl_env_vars(algorithm: "CommunicationAlgorithm", interconnect=None) -> dict:
        env: dict[str, str] = {}
        if interconnect in (InterconnectType.NVLINK3, InterconnectType.NVLINK4, InterconnectType.NVLINK5):
            env["NCCL_P2P_LEVEL"] = "NVL"
        if interconnect in (InterconnectType.INFINIBAND_HDR, InterconnectType.INFINIBAND_NDR):
            env["NCCL_IB_DISABLE"] = "0"
            env["NCCL_NET_GDR_LEVEL"] = "5"
        if algorithm == CommunicationAlgorithm.RING:
            env["NCCL_ALGO"] = "Ring"
        elif algorithm == CommunicationAlgorithm.TREE:
            env["NCCL_ALGO"] = "Tree"
        return env


# ------------------------------------------------------------------------------------------------ typed topology records
from enum import IntEnum  # noqa: E402
from typing import NamedTuple  # noqa: E402


class HardwareVendor(IntEnum):
    UNKNOWN = 0
    NVIDIA = 1
    AMD = 2
    INTEL = 3
    CPU = 4


class InterconnectType(IntEnum):
    UNKNOWN = 0
    PCIE = 1
    NVLINK3 = 2
    NVLINK4 = 3
    NVLINK5 = 4
    INFINITY_FABRIC = 5
    INTEL_FABRIC = 6
    INFINIBAND_HDR = 7
    INFINIBAND_NDR = 8
    ROCE_V2 = 9
    ETHERNET = 10


class GPUArchitecture(IntEnum):
    UNKNOWN = 0
    AMPERE = 1
    ADA = 2
    HOPPER = 3
    BLACKWELL = 4
    CDNA2 = 10
    CDNA3 = 11
    CDNA4 = 12
    GAUDI2 = 20
    GAUDI3 = 21

    @classmethod
    def from_compute_capability(cls, cc: tuple) -> "GPUArchitecture":
        return {(8, 0): cls.AMPERE, (8, 6): cls.AMPERE, (8, 9): cls.ADA, (9, 0): cls.HOPPER}.get(
            tuple(cc), cls.BLACKWELL if cc[0] in (10, 12) else cls.UNKNOWN)


class ParallelDimType(IntEnum):
    DATA = 0
    TENSOR = 1
    PIPELINE = 2
    CONTEXT = 3
    EXPERT = 4
    SEQUENCE = 5


class CommunicationAlgorithm(IntEnum):
    AUTO = 0
    RING = 1
    TREE = 2
    RECURSIVE_HALVING = 3
    BUCKET = 4
    NCCL_AUTO = 5


class NUMATopology(NamedTuple):
    num_nodes: int
    gpus_per_node: list          # NUMA node -> GPU indices
    cpu_affinity: dict           # GPU index -> CPU cores


class GPUInfo(NamedTuple):
    index: int
    name: str
    vendor: HardwareVendor
    architecture: GPUArchitecture
    compute_capability: tuple
    memory_bytes: int
    nvlink_connected: list
    pcie_bus_id: str
    numa_node: int


class NodeTopology(NamedTuple):
    hostname: str
    num_gpus: int
    gpu_info: list
    intra_node_interconnect: InterconnectType
    numa_topology: NUMATopology | None
    has_nvswitch: bool


class ClusterTopology(NamedTuple):
    num_nodes: int
    gpus_per_node: int
    total_gpus: int
    inter_node_interconnect: InterconnectType
    nodes: list
    is_homogeneous: bool


_NVLINK_BY_ARCH = {GPUArchitecture.AMPERE: InterconnectType.NVLINK3, GPUArchitecture.HOPPER: InterconnectType.NVLINK4,
                   GPUArchitecture.BLACKWELL: InterconnectType.NVLINK5}


def detect_node_topology() -> NodeTopology:
    """This node as typed records (data_pipeline/trainer/distributed/parallel_dims.py:258-292), from the same probes
    as `HardwareDetector.detect()`: a GPU that can reach peers directly is taken to be NVLink-connected to them, all-to-all
    reachability on more than two GPUs to mean a switch."""
    import socket
    raw = HardwareDetector.detect()
    n = raw["num_gpus"]
    gpus = []
    for i in range(n):
        p = torch.cuda.get_device_properties(i)
        cc = (p.major, p.minor)
        peers = [j for j in range(n) if j != i and raw["peer_access"][i][j]]
        gpus.append(GPUInfo(i, p.name, HardwareVendor.NVIDIA, GPUArchitecture.from_compute_capability(cc), cc,
                            p.total_memory, peers, str(getattr(p, "pci_bus_id", "")), raw["numa"].get(i, -1)))
    numa = None
    if raw["numa"]:
        nodes = sorted(set(raw["numa"].values()))
        numa = NUMATopology(len(nodes), [[g for g, nd in raw["numa"].items() if nd == k] for k in nodes], {})
    if n == 0:
        link = InterconnectType.UNKNOWN
    elif any(g.nvlink_connected for g in gpus):
        link = _NVLINK_BY_ARCH.get(gpus[0].architecture, InterconnectType.UNKNOWN)
    else:
        link = InterconnectType.PCIE
    return NodeTopology(socket.gethostname(), n, gpus, link, numa, bool(raw["nvswitch"]))


def detect_cluster_topology(num_nodes: int | None = None) -> ClusterTopology:
    """One node probed, the others assumed alike (the world size tells how many there are); the fabric between nodes
    cannot be seen from a process and is reported as UNKNOWN unless there is a single node."""
    node = detect_node_topology()
    world = dist.get_world_size() if dist.is_initialized() else max(node.num_gpus, 1)
    nodes = num_nodes or max(1, world // max(node.num_gpus, 1))
    return ClusterTopology(nodes, node.num_gpus, nodes * node.num_gpus,
                           InterconnectType.UNKNOWN if nodes > 1 else node.intra_node_interconnect, [node] * nodes, True)


@dataclass
class ParallelDimsMetrics:
    mesh_build_ns: int = 0
    mesh_slice_ns: int = 0
    topology_detect_ns: int = 0
    num_mesh_accesses: int = 0
    num_cache_hits: int = 0
    num_cache_misses: int = 0

    def compute_cache_hit_rate(self) -> float:
        total = self.num_cache_hits + self.num_cache_misses
        return self.num_cache_hits / total if total else 0.0

    def to_dict(self) -> dict:
        return {"mesh_build_ms": self.mesh_build_ns / 1e6, "mesh_slice_us": self.mesh_slice_ns / 1e3,
                "topology_detect_ms": self.topology_detect_ns / 1e6, "cache_hit_rate": self.compute_cache_hit_rate(),
                "total_mesh_accesses": self.num_mesh_accesses}


_DIM_TYPES = {"dp_replicate": ParallelDimType.DATA, "dp_shard": ParallelDimType.DATA, "cp": ParallelDimType.CONTEXT,
              "tp": ParallelDimType.TENSOR, "pp": ParallelDimType.PIPELINE, "ep": ParallelDimType.EXPERT,
              "etp": ParallelDimType.EXPERT, "sp": ParallelDimType.SEQUENCE}


@dataclass(frozen=True)
class DimensionSpec:
    """One mesh dimension: name, degree (>= 1), kind, whether it communicates and whether it shards data or weights."""
    name: str
    degree: int
    dim_type: ParallelDimType
    requires_comm: bool = True
    is_sharding: bool = False

    def __post_init__(self):
        if self.degree < 1:
            raise ValueError(f"dimension {self.name} degree must be >= 1, got {self.degree}")
        if self.name not in _DIM_TYPES:
            raise ValueError(f"unknown dimension name: {self.name}")

    @classmethod
    def of(cls, cfg: ParallelDimsConfig) -> list["DimensionSpec"]:
        c = cfg.resolve()
        return [cls(n, int(getattr(c, n)), _DIM_TYPES[n], int(getattr(c, n)) > 1, n in ("dp_shard", "tp", "cp", "ep", "etp"))
                for n in ("pp", "dp_replicate", "dp_shard", "cp", "tp", "ep", "etp")]


def create_parallel_dims(world_size: int, dp_replicate: int = 1, dp_shard: int = -1, cp: int = 1, tp: int = 1,
                         pp: int = 1, ep: int = 1, etp: int = 1, sp: int = 1, rank: int | None = None,
                         create_groups: bool | None = None):
    """Validated `ParallelDims` as a Result (data_pipeline/trainer/distributed/parallel_dims.py:1640-1678): Ok(dims) or
    Err(ValueError) when the degrees do not multiply to the world size.  Process groups are created only when a
    process group of that world size is initialised (or `create_groups` says so)."""
    from ..core.types import Err, Ok
    try:
        cfg = ParallelDimsConfig(dp_replicate, dp_shard, cp, tp, pp, ep, etp, bool(sp and sp > 1), world_size).resolve()
        if create_groups is None:
            create_groups = dist.is_initialized() and dist.get_world_size() == world_size
        return Ok(ParallelDims(cfg, rank=rank if rank is not None else (dist.get_rank() if dist.is_initialized() else 0),
                               create_groups=create_groups))
    except ValueError as e:
        return Err(e)


_hd_install()
