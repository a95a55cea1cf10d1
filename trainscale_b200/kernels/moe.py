"""Mixture-of-experts layer API under the names of data_pipeline/trainer/kernels/moe_kernels.py (:95-117 device queries,
:168-191 autotune space, :900-1190 grouped-GEMM functionals, :1342 autograd function, :1428-1616 router, :1618-1800
expert / block modules, :1800-1900 factories and benchmark).

The block (`SparseMoEBlock`) runs on the device-side path of `ops/moe.py`: router soft-max + top-k kernel, routing plan,
permute into 128-row-aligned expert segments, two grouped tcgen05 GEMM launches, weighted combine - no host
synchronisation on expert counts.  The `moe_grouped_gemm_*` functionals keep the reference's calling convention
(cumulative `expert_offsets` + `gather_indices` of an argsort by expert); they serve code written against that
convention and run one framework GEMM per non-empty expert segment, which needs the offsets on the host.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import activation as _act
from ..ops import gemm as _gemm
from ..ops import moe as _moe
from .compat import _FunctionPair


# ------------------------------------------------------------------------------------------------ device queries
def _props(device_id: int = 0):
    return torch.cuda.get_device_properties(device_id) if torch.cuda.is_available() else None


def get_num_sms(device_id: int = 0) -> int:
    p = _props(device_id)
    return p.multi_processor_count if p is not None else 1


def get_max_shared_memory(device_id: int = 0) -> int:
    """Largest shared-memory allocation a block may opt into, in bytes (227 KB on sm_100; 48 KB without a GPU)."""
    p = _props(device_id)
    if p is None:
        return 49152
    return int(getattr(p, "shared_memory_per_block_optin", 0) or getattr(p, "max_shared_memory_per_block", 49152))


def get_l2_cache_size(device_id: int = 0) -> int:
    p = _props(device_id)
    return int(getattr(p, "L2_cache_size", 0) or getattr(p, "l2_cache_size", 0)) if p is not None else 0


@dataclass
class MoEAutotuneConfig:
    """Search space of the reference's Triton grouped GEMM.  The tcgen05 grouped GEMM has one tile shape (128 x 256 x 64
    per CTA, pairs of CTAs on 256-row tiles), chosen at build time, so `generate_configs()` has a single entry."""
    block_m_range: tuple = (128,)
    block_n_range: tuple = (256,)
    block_k_range: tuple = (64,)
    num_warps_range: tuple = (8,)
    num_stages_range: tuple = (6,)

    def generate_configs(self) -> list:
        from . import MoEKernelConfig
        return [MoEKernelConfig() for _ in self.block_m_range for _ in self.block_n_range for _ in self.block_k_range
                for _ in self.num_warps_range for _ in self.num_stages_range]


# ------------------------------------------------------------------------------------------------ router
@dataclass
class RouterConfig:
    num_experts: int = 8
    top_k: int = 2
    capacity_factor: float = 1.25
    aux_loss_coef: float = 0.01
    z_loss_coef: float = 0.001
    noise_std: float = 0.1
    epsilon_greedy: float = 0.0
    normalize_weights: bool = True
    jitter_noise: bool = True


class MoERouter(nn.Module):
    """Soft-max top-k router with the usual regularisers: Switch-style balance loss E * sum_e f_e * P_e, z-loss on the
    log-partition of the logits, Gaussian jitter on the logits and epsilon-greedy expert replacement while training.
    Returns the reference's five values (routing_weights [T * k], selected_experts [T, k], expert_offsets [E]
    cumulative, gather_indices [T * k] = slots sorted by expert, aux_losses)."""

    def __init__(self, hidden_size: int, config: RouterConfig | None = None):
        super().__init__()
        self.config = config or RouterConfig()
        self.hidden_size = hidden_size
        self.gate = nn.Linear(hidden_size, self.config.num_experts, bias=False)
        nn.init.normal_(self.gate.weight, std=0.02)
        self._aux_loss = torch.zeros(())
        self._z_loss = torch.zeros(())
        self._load_balance_stats: dict = {}

    def route(self, hidden_flat: torch.Tensor, expert_mask: torch.Tensor | None = None):
        """(weights [T, k] fp32, experts [T, k] int64, probs [T, E], logits) for flattened tokens."""
        c = self.config
        logits = self.gate(hidden_flat).float()
        if expert_mask is not None:
            logits = logits.masked_fill(~expert_mask.bool(), float("-inf"))
        if self.training and c.jitter_noise and c.noise_std > 0:
            logits = logits + torch.randn_like(logits) * c.noise_std
        explore = self.training and c.epsilon_greedy > 0
        if explore or expert_mask is not None:
            probs = torch.softmax(logits, dim=-1)
            w, idx = probs.topk(c.top_k, dim=-1)
            if explore:
                T = hidden_flat.shape[0]
                swap = torch.rand(T, device=logits.device) < c.epsilon_greedy
                rnd = torch.randint(0, c.num_experts, (T, c.top_k), device=logits.device)
                idx = torch.where(swap[:, None], rnd, idx)
                w = probs.gather(-1, idx)
            if c.normalize_weights:
                w = w / (w.sum(-1, keepdim=True) + 1e-8)
        else:
            w, idx, probs = _moe.topk_softmax(logits, c.top_k, c.normalize_weights)
        return w, idx, probs, logits

    def losses(self, idx, probs, logits) -> dict:
        c = self.config
        zero = logits.new_zeros(())
        aux = z = zero
        if self.training and c.z_loss_coef > 0:
            z = c.z_loss_coef * torch.logsumexp(logits, dim=-1).pow(2).mean()
        if self.training and c.aux_loss_coef > 0:
            frac = torch.zeros(c.num_experts, device=logits.device).index_add_(
                0, idx.reshape(-1), torch.ones(idx.numel(), device=logits.device)) / idx.numel()
            aux = c.aux_loss_coef * c.num_experts * (frac * probs.mean(0)).sum()
            self._load_balance_stats = {"expert_fraction": frac.detach(), "router_prob": probs.mean(0).detach()}
        self._aux_loss, self._z_loss = aux, z
        return {"aux_loss": aux, "z_loss": z, "total_loss": aux + z}

    def forward(self, hidden_states: torch.Tensor, expert_mask: torch.Tensor | None = None):
        flat = hidden_states.reshape(-1, hidden_states.shape[-1])
        w, idx, probs, logits = self.route(flat, expert_mask)
        aux = self.losses(idx, probs, logits)
        slots = idx.reshape(-1)
        gather_indices = slots.argsort(stable=True)
        counts = torch.zeros(self.config.num_experts, dtype=torch.long, device=slots.device).index_add_(
            0, slots, torch.ones_like(slots))
        return w.reshape(-1), idx, counts.cumsum(0), gather_indices, aux

    def get_aux_loss(self) -> torch.Tensor:
        return self._aux_loss + self._z_loss

    def get_load_stats(self) -> dict:
        return self._load_balance_stats


# ------------------------------------------------------------------------------------------------ experts / block
class ExpertMLPLayer(nn.Module):
    """One gated expert: down(act(gate(x)) * up(x)) on the framework GEMM and GLU kernels."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False):
        super().__init__()
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.gate_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.up_proj = nn.Linear(hidden_size, intermediate_size, bias=bias)
        self.down_proj = nn.Linear(intermediate_size, hidden_size, bias=bias)

    def forward(self, x):
        gu = torch.cat((_gemm.linear(x, self.gate_proj.weight, self.gate_proj.bias),
                        _gemm.linear(x, self.up_proj.weight, self.up_proj.bias)), dim=-1)
        return _gemm.linear(_act.glu(gu, self.activation), self.down_proj.weight, self.down_proj.bias)


class SparseMoEBlock(nn.Module):
    """Router + E gated experts with packed weights (`gate_up_proj` [E, 2I, H], `down_proj` [E, H, I]);
    forward(hidden [B, S, H]) -> (output [B, S, H], aux_losses)."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int = 8, top_k: int = 2,
                 capacity_factor: float = 1.25, aux_loss_coef: float = 0.01, z_loss_coef: float = 0.001,
                 activation: str = "silu", bias: bool = False):
        super().__init__()
        if bias:
            raise ValueError("expert biases are not supported by the grouped GEMM path")
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.num_experts, self.top_k, self.activation = num_experts, top_k, activation
        self.router = MoERouter(hidden_size, RouterConfig(num_experts, top_k, capacity_factor, aux_loss_coef,
                                                          z_loss_coef))
        self.gate_up_proj = nn.Parameter(torch.empty(num_experts, 2 * intermediate_size, hidden_size))
        self.down_proj = nn.Parameter(torch.empty(num_experts, hidden_size, intermediate_size))
        for p in (self.gate_up_proj, self.down_proj):
            nn.init.kaiming_uniform_(p, a=math.sqrt(5))

    def forward(self, hidden_states: torch.Tensor):
        shape = hidden_states.shape
        flat = hidden_states.reshape(-1, shape[-1])
        w, idx, probs, logits = self.router.route(flat)
        aux = self.router.losses(idx, probs, logits)
        from . import moe_grouped_gemm
        out = moe_grouped_gemm(flat, idx, w.to(flat.dtype), self.gate_up_proj, self.down_proj, self.activation)
        return out.view(shape), aux

    def get_aux_loss(self) -> torch.Tensor:
        return self.router.get_aux_loss()


def create_moe_block(hidden_size: int, intermediate_size: int, num_experts: int = 8, top_k: int = 2,
                     **kwargs) -> SparseMoEBlock:
    return SparseMoEBlock(hidden_size, intermediate_size, num_experts, top_k, **kwargs)


def moe_forward(hidden_states: torch.Tensor, expert_weights, router: MoERouter, activation="silu"):
    """Functional block: expert_weights = (gate_up_proj [E, 2I, H], down_proj [E, H, I]) -> (output, aux loss)."""
    gate_up, down = expert_weights
    act = activation if isinstance(activation, str) else {F.silu: "silu", F.gelu: "gelu", F.relu: "relu"}.get(
        activation, "silu")
    shape = hidden_states.shape
    flat = hidden_states.reshape(-1, shape[-1])
    w, idx, probs, logits = router.route(flat)
    aux = router.losses(idx, probs, logits)
    from . import moe_grouped_gemm
    return moe_grouped_gemm(flat, idx, w.to(flat.dtype), gate_up, down, act).view(shape), aux["total_loss"]


# ------------------------------------------------------------------------------------------------ functional grouped GEMM
def _segments(expert_offsets: torch.Tensor) -> list[tuple[int, int, int]]:
    ends = [int(v) for v in expert_offsets.tolist()]
    return [(e, (ends[e - 1] if e else 0), ends[e]) for e in range(len(ends)) if ends[e] > (ends[e - 1] if e else 0)]


def moe_grouped_gemm_forward(X, W, topk: int, expert_offsets, gather_indices=None, topk_weights=None,
                             permute_x: bool = False, permute_y: bool = False, fuse_topk_weights: bool = False,
                             config=None) -> torch.Tensor:
    """Y = X_sorted @ W[e]^T per expert segment; W [E, N, K].  `gather_indices[r]` is the slot (token * topk + choice)
    sitting at sorted row r and `expert_offsets` the cumulative rows per expert.  permute_x: X is [tokens, K] and is
    gathered into sorted order here; permute_y: the result goes back to slot order; fuse_topk_weights: every row is
    multiplied by its routing weight (`topk_weights` in slot order).  Differentiable."""
    total = X.shape[0] * topk if permute_x else X.shape[0]
    if gather_indices is None:
        gather_indices = torch.arange(total, device=X.device)
    xs = X[gather_indices // topk] if permute_x else X
    parts = [xs.new_zeros(0, W.shape[1])]
    for e, a, b in _segments(expert_offsets):
        parts.append(_gemm.linear(xs[a:b], W[e]))
    y = torch.cat(parts)
    if fuse_topk_weights and topk_weights is not None:
        y = y * topk_weights.reshape(-1)[gather_indices].to(y.dtype).unsqueeze(1)
    if permute_y:
        y = torch.zeros_like(y).index_copy(0, gather_indices, y)
    return y


def moe_grouped_gemm_backward_dx(dY, W, topk: int, expert_offsets, gather_indices=None, topk_weights=None,
                                 permute_x: bool = False, permute_y: bool = False, fuse_topk_weights: bool = False,
                                 num_tokens: int | None = None, config=None) -> torch.Tensor:
    """dX of `moe_grouped_gemm_forward`: dY (slot order if permute_y, else sorted) @ W[e] per segment; with permute_x
    the k slot gradients of a token are summed into [num_tokens, K]."""
    total = dY.shape[0]
    if gather_indices is None:
        gather_indices = torch.arange(total, device=dY.device)
    g = dY[gather_indices] if permute_y else dY
    if fuse_topk_weights and topk_weights is not None:
        g = g * topk_weights.reshape(-1)[gather_indices].to(g.dtype).unsqueeze(1)
    parts = [g.new_zeros(0, W.shape[2])]
    for e, a, b in _segments(expert_offsets):
        parts.append(_gemm.linear(g[a:b], W[e].t()))
    dxs = torch.cat(parts)
    if not permute_x:
        return dxs
    T = num_tokens if num_tokens is not None else total // topk
    return torch.zeros(T, W.shape[2], dtype=dxs.dtype, device=dxs.device).index_add_(0, gather_indices // topk, dxs)


def moe_grouped_gemm_backward_dw(X, dY, topk: int, expert_offsets, gather_indices=None, topk_weights=None,
                                 permute_x: bool = False, permute_y: bool = False, fuse_topk_weights: bool = False,
                                 num_experts: int | None = None, config=None) -> torch.Tensor:
    """dW [E, N, K] of `moe_grouped_gemm_forward`: dY_seg^T @ X_seg per expert."""
    total = dY.shape[0]
    if gather_indices is None:
        gather_indices = torch.arange(total, device=dY.device)
    xs = X[gather_indices // topk] if permute_x else X
    g = dY[gather_indices] if permute_y else dY
    if fuse_topk_weights and topk_weights is not None:
        g = g * topk_weights.reshape(-1)[gather_indices].to(g.dtype).unsqueeze(1)
    E = num_experts if num_experts is not None else expert_offsets.numel()
    dW = torch.zeros(E, g.shape[1], xs.shape[1], dtype=torch.float32, device=g.device)
    for e, a, b in _segments(expert_offsets):
        dW[e] = g[a:b].float().t() @ xs[a:b].float()
    return dW.to(X.dtype)


class MoEGroupedGEMMFunction(_FunctionPair):
    """`apply(X, W, topk, expert_offsets, gather_indices, topk_weights, permute_x, permute_y, fuse_topk_weights,
    fwd_config=None, bwd_config=None)`: the reference's autograd-function entry point.  The forward functional is built
    from differentiable framework ops, so autograd derives the backward; the two explicit backward functionals above
    exist for callers that want them and are what the tests compare autograd against."""

    @staticmethod
    def apply(X, W, topk, expert_offsets, gather_indices=None, topk_weights=None, permute_x=False, permute_y=False,
              fuse_topk_weights=False, fwd_config=None, bwd_config=None):
        return moe_grouped_gemm_forward(X, W, topk, expert_offsets, gather_indices, topk_weights, permute_x, permute_y,
                                        fuse_topk_weights, fwd_config)


def benchmark_moe_kernel(batch_size: int = 4, seq_len: int = 2048, hidden_size: int = 4096,
                         intermediate_size: int = 14336, num_experts: int = 8, top_k: int = 2, num_warmup: int = 10,
                         num_iters: int = 100, dtype: torch.dtype = torch.bfloat16) -> dict:
    """CUDA-event timing of a `SparseMoEBlock` forward: mean ms, tokens/s and expert-GEMM TFLOP/s."""
    if not torch.cuda.is_available():
        raise RuntimeError("benchmark_moe_kernel needs a CUDA device")
    dev = torch.device("cuda")
    blk = SparseMoEBlock(hidden_size, intermediate_size, num_experts, top_k).to(dev, dtype).eval()
    x = torch.randn(batch_size, seq_len, hidden_size, device=dev, dtype=dtype)
    with torch.no_grad():
        for _ in range(num_warmup):
            blk(x)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(num_iters):
            blk(x)
        b.record()
        torch.cuda.synchronize()
    ms = a.elapsed_time(b) / num_iters
    tokens = batch_size * seq_len
    flops = tokens * top_k * 3 * 2 * hidden_size * intermediate_size
    return {"mean_ms": ms, "tokens_per_second": tokens / ms * 1e3, "tflops": flops / ms / 1e9}
