"""Optimizer zoo behind `create_optimizer` (torch.optim.Optimizer subclasses).

Covers the reference's list (data_pipeline/trainer/optimizers/{base,adamw,lamb,adafactor,sota_optimizers}.py):
AdamW / FusedAdamW (the sm_100a flat kernel per tensor), Adam8bit (block-wise 8-bit moment storage), Lion, LAMB,
AdaFactor (factored second moment), CAME, SophiaG (Hutchinson / GNB Hessian EMA), Prodigy, ScheduleFreeAdamW, Muon
(Newton-Schulz orthogonalised momentum), ADOPT, plus `clip_grad_norm_` with the reference's coefficient
`max_norm / (norm + 1e-6)` clamped to 1 (data_pipeline/trainer/distributed/sota_utils.py:1294-1299).
The sharded hot path does not go through these classes: the flat engine owns its AdamW / Lion state
(parallel/flat_engine.py); these serve non-sharded models, LoRA adapters and the remaining optimizer types.
"""
from __future__ import annotations

import math
from typing import Iterable

import torch
from torch.optim import Optimizer

from ..ops import optim as K
from ..utils.refargs import ANY, reference_kwargs

_IMPL_OPTIONS = {"use_triton": ANY, "fused_foreach": ANY, "enable_metrics": ANY}     # implementation switches of
# the reference's optimizers (Triton / foreach paths, metric collection): accepted, no effect on the kernels used here


@torch.no_grad()
def clip_grad_norm_(parameters: Iterable[torch.Tensor], max_norm: float, norm_type: float = 2.0,
                    error_if_nonfinite: bool = False) -> torch.Tensor:
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return torch.zeros(())
    if norm_type == float("inf"):
        total = torch.stack([g.abs().max() for g in grads]).max()
    else:
        total = torch.stack([torch.linalg.vector_norm(g.float(), norm_type) for g in grads]).norm(norm_type)
    if error_if_nonfinite and not bool(torch.isfinite(total)):
        raise RuntimeError(f"the total gradient norm is {float(total)}: gradients are not clipped")
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for g in grads:
        g.mul_(coef.to(g.dtype))
    return total


class AdamW(Optimizer):
    """Decoupled AdamW. CUDA fp32 tensors with bf16/fp32 grads use the fused flat kernel (one launch per tensor)."""

    @reference_kwargs(_IMPL_OPTIONS)
    def __init__(self, params, lr=2e-5, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, amsgrad=False, fused=True,
                 max_grad_norm: float | None = None, grad_accumulation_steps: int = 1):
        """`max_grad_norm`: clip the global gradient norm before every update.  `grad_accumulation_steps` = n: the
        update happens on every n-th `step()` call, on the MEAN of the gradients seen since the last update (the caller
        must not zero the gradients in between); data_pipeline/trainer/optimizers/adamw.py:1010-1030."""
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad, fused=fused))
        self.max_grad_norm, self.grad_accumulation_steps = max_grad_norm, max(1, int(grad_accumulation_steps))
        self._micro = 0

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        n = getattr(self, "grad_accumulation_steps", 1)
        if n > 1:
            self._micro += 1
            if self._micro % n:
                return loss
            for g in self.param_groups:
                for p in g["params"]:
                    if p.grad is not None:
                        p.grad.div_(n)
        if getattr(self, "max_grad_norm", None):
            clip_grad_norm_([p for g in self.param_groups for p in g["params"]], self.max_grad_norm)
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    if g["amsgrad"]:
                        st["max_exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    if p.dtype != torch.float32:
                        st["master"] = p.detach().float().clone()
                st["step"] += 1
                master = st.get("master", p)
                grad = p.grad
                if g["fused"] and p.is_cuda and not g["amsgrad"] and grad.dtype in (torch.float32, torch.bfloat16) \
                        and master.is_contiguous() and grad.is_contiguous():
                    low = p.view(-1) if p.dtype == torch.bfloat16 else None
                    K.adamw_flat_(master.view(-1), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1), grad.view(-1), low,
                                  lr=g["lr"], beta1=b1, beta2=b2, eps=g["eps"], weight_decay=g["weight_decay"],
                                  step=st["step"])
                    if "master" in st and low is None:
                        p.copy_(master)
                    continue
                gf = grad.float()
                st["exp_avg"].mul_(b1).add_(gf, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                v = st["exp_avg_sq"]
                if g["amsgrad"]:
                    torch.maximum(st["max_exp_avg_sq"], v, out=st["max_exp_avg_sq"])
                    v = st["max_exp_avg_sq"]
                master.mul_(1 - g["lr"] * g["weight_decay"])
                master.addcdiv_(st["exp_avg"] / bc1, (v / bc2).sqrt().add_(g["eps"]), value=-g["lr"])
                if master is not p:
                    p.copy_(master)
        return loss


FusedAdamW = AdamW


def _quantize_blockwise(x: torch.Tensor, block: int = 256):
    flat = x.reshape(-1)
    pad = (-flat.numel()) % block
    if pad:
        flat = torch.cat((flat, flat.new_zeros(pad)))
    b = flat.view(-1, block)
    scale = b.abs().amax(dim=1, keepdim=True).clamp(min=1e-12)
    q = torch.round(b / scale * 127).to(torch.int8)
    return q, scale.squeeze(1)


def _dequantize_blockwise(q: torch.Tensor, scale: torch.Tensor, shape, numel: int):
    return (q.float() * (scale.unsqueeze(1) / 127)).reshape(-1)[:numel].view(shape)


class Adam8bit(Optimizer):
    """AdamW whose moments are stored as block-wise int8 (+ one fp32 scale per 256 values); the second moment is
    stored as sqrt(v) to keep its dynamic range inside 8 bits."""

    @reference_kwargs({"percentile_clipping": (100, 100.0, None), "stochastic_rounding": (False, None)})
    def __init__(self, params, lr=2e-5, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, block_size=256,
                 min_8bit_size=4096):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, block_size=block_size,
                                      min_8bit_size=min_8bit_size))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                small = p.numel() < g["min_8bit_size"]
                if not st:
                    st["step"] = 0
                    z = torch.zeros_like(p, dtype=torch.float32)
                    if small:
                        st["m"], st["v"] = z, z.clone()
                    else:
                        st["m_q"], st["m_s"] = _quantize_blockwise(z, g["block_size"])
                        st["v_q"], st["v_s"] = _quantize_blockwise(z, g["block_size"])
                st["step"] += 1
                if not small and g["block_size"] in K.QUANT_BLOCKS and K.native_ok(p, p.grad):
                    K.adam8bit_(p, p.grad, st["m_q"], st["m_s"], st["v_q"], st["v_s"], lr=g["lr"], beta1=b1, beta2=b2,
                                eps=g["eps"], weight_decay=g["weight_decay"], step=st["step"])
                    continue
                gf = p.grad.float()
                if small:
                    m, v = st["m"], st["v"]
                else:
                    m = _dequantize_blockwise(st["m_q"], st["m_s"], p.shape, p.numel())
                    v = _dequantize_blockwise(st["v_q"], st["v_s"], p.shape, p.numel()).pow(2)
                m = m.mul(b1).add(gf, alpha=1 - b1)
                v = v.mul(b2).addcmul(gf, gf, value=1 - b2)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                pf = p.float().mul_(1 - g["lr"] * g["weight_decay"])
                pf.addcdiv_(m / bc1, (v / bc2).sqrt().add_(g["eps"]), value=-g["lr"])
                p.copy_(pf)
                if small:
                    st["m"], st["v"] = m, v
                else:
                    st["m_q"], st["m_s"] = _quantize_blockwise(m, g["block_size"])
                    st["v_q"], st["v_s"] = _quantize_blockwise(v.sqrt(), g["block_size"])
        return loss

    def state_bytes(self) -> int:
        n = 0
        for st in self.state.values():
            for v in st.values():
                if torch.is_tensor(v):
                    n += v.numel() * v.element_size()
        return n


class Lion(Optimizer):
    def __init__(self, params, lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                gf = p.grad.float()
                u = (st["exp_avg"] * b1 + gf * (1 - b1)).sign_()
                pf = p.float().mul_(1 - g["lr"] * g["weight_decay"]).add_(u, alpha=-g["lr"])
                p.copy_(pf)
                st["exp_avg"].mul_(b2).add_(gf, alpha=1 - b2)
        return loss


class LAMB(Optimizer):
    @reference_kwargs({"use_triton": ANY, "always_adapt": (False, None)})
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01, clamp_trust=(0.0, 10.0),
                 trust_ratio_clip: float | None = None):
        """`trust_ratio_clip`: upper bound of the layer-wise trust ratio (the reference's name; `clamp_trust` gives
        both bounds)."""
        if trust_ratio_clip is not None:
            clamp_trust = (clamp_trust[0], float(trust_ratio_clip))
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, clamp_trust=clamp_trust))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"], st["m"], st["v"] = 0, torch.zeros_like(p, dtype=torch.float32), torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                if K.native_ok(p, p.grad):
                    if "upd" not in st:
                        st["upd"], st["norms"] = torch.empty_like(st["m"]), torch.zeros(2, device=p.device)
                    K.lamb_(p, p.grad, st["m"], st["v"], st["upd"], st["norms"], lr=g["lr"], beta1=b1, beta2=b2,
                            eps=g["eps"], weight_decay=g["weight_decay"], step=st["step"],
                            trust_lo=g["clamp_trust"][0], trust_hi=g["clamp_trust"][1])
                    continue
                gf = p.grad.float()
                st["m"].mul_(b1).add_(gf, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
                mh, vh = st["m"] / (1 - b1 ** st["step"]), st["v"] / (1 - b2 ** st["step"])
                pf = p.float()
                upd = mh / (vh.sqrt() + g["eps"]) + g["weight_decay"] * pf
                wn, un = pf.norm(), upd.norm()
                trust = torch.where((wn > 0) & (un > 0), wn / un, torch.ones_like(wn)).clamp(*g["clamp_trust"])
                p.copy_(pf - g["lr"] * trust * upd)
        return loss


class AdaFactor(Optimizer):
    """Factored second moments for matrices (row / column EMA), update clipping by RMS, optional relative step."""

    @reference_kwargs(_IMPL_OPTIONS)
    def __init__(self, params, lr=None, eps=(1e-30, 1e-3), clip_threshold=1.0, decay_rate=-0.8, beta1=None,
                 weight_decay=0.0, scale_parameter=True, relative_step=True, warmup_init=False):
        super().__init__(params, dict(lr=lr, eps=eps, clip_threshold=clip_threshold, decay_rate=decay_rate, beta1=beta1,
                                      weight_decay=weight_decay, scale_parameter=scale_parameter,
                                      relative_step=relative_step and lr is None, warmup_init=warmup_init))

    @staticmethod
    def _rms(x):
        return x.norm() / math.sqrt(max(1, x.numel()))

    def memory_footprint(self) -> dict:
        """Bytes held per kind: `state_bytes` (second moments, factored or full, and first moments) and `buffer_bytes`
        (work buffers of the device path); data_pipeline/trainer/optimizers/adafactor.py:1420-1440."""
        state = buf = 0
        for st in self.state.values():
            for k, v in st.items():
                if torch.is_tensor(v):
                    nb = v.numel() * v.element_size()
                    if k in ("u", "sums", "col_tmp"):
                        buf += nb
                    else:
                        state += nb
        return {"state_bytes": state, "buffer_bytes": buf, "total_bytes": state + buf}

    @property
    def profiling_stats(self) -> "ProfilingStats":
        """Counts since construction: steps' wall time, how many parameters use factored / full second moments, how
        many updates ran as one device kernel."""
        ps = self.__dict__.get("_prof")
        if ps is None:
            ps = self.__dict__["_prof"] = ProfilingStats()
        ps.num_factorized_params = sum(1 for st in self.state.values() if "row" in st)
        ps.num_full_params = sum(1 for st in self.state.values() if "v" in st)
        ps.memory_allocated_bytes = self.memory_footprint()["total_bytes"]
        ps.memory_peak_bytes = max(ps.memory_peak_bytes, ps.memory_allocated_bytes)
        return ps

    @torch.no_grad()
    def step(self, closure=None):
        import time as _time
        t0 = _time.perf_counter_ns()
        try:
            return self._step(closure)
        finally:
            ps = self.__dict__.get("_prof")
            if ps is None:
                ps = self.__dict__["_prof"] = ProfilingStats()
            ps.total_step_time_ns += _time.perf_counter_ns() - t0

    def _step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                factored = p.dim() >= 2
                if not st:
                    st["step"] = 0
                    if factored:
                        st["row"] = torch.zeros(p.shape[:-1], device=p.device)
                        st["col"] = torch.zeros(p.shape[:-2] + p.shape[-1:], device=p.device)
                    else:
                        st["v"] = torch.zeros_like(p, dtype=torch.float32)
                    if g["beta1"] is not None:
                        st["m"] = torch.zeros_like(p, dtype=torch.float32)
                    st["rms"] = 0.0
                st["step"] += 1
                if g["relative_step"]:
                    min_step = 1e-6 * st["step"] if g["warmup_init"] else 1e-2
                    lr = min(min_step, 1.0 / math.sqrt(st["step"]))
                else:
                    lr = g["lr"]
                beta2 = 1.0 - st["step"] ** g["decay_rate"]
                if K.native_ok(p, p.grad) and p.dim() <= 2 and p.numel() < 2 ** 31:
                    # device path: parameter RMS, update RMS and the clip stay on the device
                    if "u" not in st:
                        st["u"] = torch.empty_like(p, dtype=torch.float32)
                        st["sums"] = torch.zeros(2, device=p.device)
                        if factored:
                            st["col_tmp"] = torch.zeros_like(st["col"])
                    K.adafactor_(p, p.grad, st, lr=lr, beta2=beta2, eps0=g["eps"][0], eps1=g["eps"][1],
                                 clip=g["clip_threshold"], scale_parameter=g["scale_parameter"], beta1=g["beta1"],
                                 weight_decay=g["weight_decay"])
                    self.__dict__.setdefault("_prof", ProfilingStats()).fused_updates += 1
                    continue
                gf = p.grad.float()
                pf = p.float()
                st["rms"] = float(self._rms(pf))
                if g["scale_parameter"]:
                    lr = lr * max(g["eps"][1], st["rms"])
                upd = gf * gf + g["eps"][0]
                if factored:
                    st["row"].mul_(beta2).add_(upd.mean(-1), alpha=1 - beta2)
                    st["col"].mul_(beta2).add_(upd.mean(-2), alpha=1 - beta2)
                    r = (st["row"] / st["row"].mean(-1, keepdim=True)).rsqrt().unsqueeze(-1)
                    c = st["col"].unsqueeze(-2).rsqrt()
                    u = gf * r * c
                else:
                    st["v"].mul_(beta2).add_(upd, alpha=1 - beta2)
                    u = gf * st["v"].rsqrt()
                u.div_(max(1.0, float(self._rms(u)) / g["clip_threshold"]))
                u.mul_(lr)
                if g["beta1"] is not None:
                    st["m"].mul_(g["beta1"]).add_(u, alpha=1 - g["beta1"])
                    u = st["m"]
                if g["weight_decay"]:
                    pf.mul_(1 - g["weight_decay"] * lr)
                p.copy_(pf - u)
        return loss


class DistributedAdaFactor(AdaFactor):
    """AdaFactor for matrices that are row-sharded over a process group (tensor-parallel column-parallel weights,
    ZeRO shards that keep whole rows): the row statistics are local, the column statistics and the row-mean / RMS
    scalars are all-reduced so that every shard applies exactly the update of the unsharded matrix
    (data_pipeline/trainer/optimizers/adafactor.py:1561 has the same role)."""

    def __init__(self, params, group=None, **kw):
        super().__init__(params, **kw)
        self.group = group

    def _world(self) -> int:
        import torch.distributed as dist
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def _sum(self, t: torch.Tensor) -> torch.Tensor:
        import torch.distributed as dist
        if self._world() > 1:
            dist.all_reduce(t, group=self.group)
        return t

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        W = self._world()
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                gf, pf = p.grad.float(), p.float()
                st = self.state[p]
                factored = gf.dim() >= 2
                if not st:
                    st["step"] = 0
                    if factored:
                        st["row"] = torch.zeros(gf.shape[:-1], device=gf.device)
                        st["col"] = torch.zeros(gf.shape[:-2] + gf.shape[-1:], device=gf.device)
                    else:
                        st["v"] = torch.zeros_like(gf)
                    if g["beta1"] is not None:
                        st["m"] = torch.zeros_like(gf)
                st["step"] += 1
                n_global = self._sum(torch.tensor(float(pf.numel()), device=pf.device))
                rms_p = float((self._sum(pf.pow(2).sum()) / n_global).sqrt())
                if g["relative_step"]:
                    min_step = 1e-6 * st["step"] if g["warmup_init"] else 1e-2
                    lr = min(min_step, 1.0 / math.sqrt(st["step"]))
                else:
                    lr = g["lr"]
                if g["scale_parameter"]:
                    lr = lr * max(g["eps"][1], rms_p)
                beta2 = 1.0 - st["step"] ** g["decay_rate"]
                upd = gf * gf + g["eps"][0]
                if factored:
                    st["row"].mul_(beta2).add_(upd.mean(-1), alpha=1 - beta2)
                    col_mean = self._sum(upd.sum(-2)) / (gf.shape[-2] * W)       # mean over ALL rows of the matrix
                    st["col"].mul_(beta2).add_(col_mean, alpha=1 - beta2)
                    row_mean = self._sum(st["row"].sum(-1, keepdim=True)) / (gf.shape[-2] * W)
                    u = gf * (st["row"] / row_mean).rsqrt().unsqueeze(-1) * st["col"].unsqueeze(-2).rsqrt()
                else:
                    st["v"].mul_(beta2).add_(upd, alpha=1 - beta2)
                    u = gf * st["v"].rsqrt()
                rms_u = float((self._sum(u.pow(2).sum()) / n_global).sqrt())
                u.div_(max(1.0, rms_u / g["clip_threshold"]))
                u.mul_(lr)
                if g["beta1"] is not None:
                    st["m"].mul_(g["beta1"]).add_(u, alpha=1 - g["beta1"])
                    u = st["m"]
                if g["weight_decay"]:
                    pf.mul_(1 - g["weight_decay"] * lr)
                p.copy_(pf - u)
        return loss


class CAME(Optimizer):
    """Confidence-guided AdaFactor: a second factored EMA of the update's instability rescales the step."""

    @reference_kwargs({"confidence_threshold": ANY})    # the confidence term is always on: it is what CAME is
    def __init__(self, params, lr=2e-4, eps=(1e-30, 1e-16), clip_threshold=1.0, betas=(0.9, 0.999, 0.9999), weight_decay=0.0):
        super().__init__(params, dict(lr=lr, eps=eps, clip_threshold=clip_threshold, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2, b3 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                gf = p.grad.float()
                st = self.state[p]
                fac = gf.dim() >= 2
                if not st:
                    st["m"] = torch.zeros_like(gf)
                    if fac:
                        st["row"], st["col"] = torch.zeros(gf.shape[:-1], device=gf.device), torch.zeros(gf.shape[:-2] + gf.shape[-1:], device=gf.device)
                        st["rrow"], st["rcol"] = st["row"].clone(), st["col"].clone()
                    else:
                        st["v"] = torch.zeros_like(gf)
                upd = gf * gf + g["eps"][0]
                if fac:
                    st["row"].mul_(b2).add_(upd.mean(-1), alpha=1 - b2)
                    st["col"].mul_(b2).add_(upd.mean(-2), alpha=1 - b2)
                    u = gf * (st["row"] / st["row"].mean(-1, keepdim=True)).rsqrt().unsqueeze(-1) * st["col"].unsqueeze(-2).rsqrt()
                else:
                    st["v"].mul_(b2).add_(upd, alpha=1 - b2)
                    u = gf * st["v"].rsqrt()
                u.div_((u.norm() / (math.sqrt(u.numel()) * g["clip_threshold"])).clamp_(min=1.0))   # stays on the device
                st["m"].mul_(b1).add_(u, alpha=1 - b1)
                if fac:
                    res = (u - st["m"]) ** 2 + g["eps"][1]
                    st["rrow"].mul_(b3).add_(res.mean(-1), alpha=1 - b3)
                    st["rcol"].mul_(b3).add_(res.mean(-2), alpha=1 - b3)
                    step_ = st["m"] * (st["rrow"] / st["rrow"].mean(-1, keepdim=True)).rsqrt().unsqueeze(-1) * st["rcol"].unsqueeze(-2).rsqrt()
                else:
                    step_ = st["m"]
                pf = p.float()
                if g["weight_decay"]:
                    pf.mul_(1 - g["lr"] * g["weight_decay"])
                p.copy_(pf - g["lr"] * step_)
        return loss


class SophiaG(Optimizer):
    """Clipped second-order step: p -= lr * clip(m / max(rho * h, eps), 1). Call `update_hessian()` every k steps
    after a backward on sampled labels (Gauss-Newton-Bartlett) or with `hutchinson=True` grads."""

    @reference_kwargs({"maximize": (False, None)})
    def __init__(self, params, lr=1e-4, betas=(0.965, 0.99), rho=0.04, weight_decay=0.1, eps=1e-15,
                 hessian_update_interval: int = 10):
        """`hessian_update_interval`: how often the caller is expected to refresh the curvature estimate; kept as an
        attribute for the training loop (`step_count % optimizer.hessian_update_interval == 0` -> `update_hessian`)."""
        super().__init__(params, dict(lr=lr, betas=betas, rho=rho, weight_decay=weight_decay, eps=eps))
        self.hessian_update_interval = int(hessian_update_interval)

    @torch.no_grad()
    def update_hessian(self, batch_size: int = 1):
        for g in self.param_groups:
            b2 = g["betas"][1]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "h" not in st:
                    st["h"] = torch.zeros_like(p, dtype=torch.float32)
                if K.native_ok(st["h"], p.grad):
                    K.sophia_hessian_(p.grad, st["h"], beta2=b2, scale=(1 - b2) * batch_size)
                    continue
                st["h"].mul_(b2).addcmul_(p.grad.float(), p.grad.float(), value=(1 - b2) * batch_size)

    def update_hessian_hutchinson(self, loss: torch.Tensor, generator: torch.Generator | None = None) -> None:
        """Hutchinson estimate of the Hessian diagonal: h <- b2 h + (1 - b2) u * (H u) with Rademacher u, from one
        Hessian-vector product (a second backward through `loss`, which must have been built from operators that
        support double differentiation - the framework's fused kernels do not; use the Gauss-Newton-Bartlett form
        `update_hessian` with them)."""
        params = [p for g in self.param_groups for p in g["params"] if p.requires_grad]
        grads = torch.autograd.grad(loss, params, create_graph=True, allow_unused=True)
        pairs = [(p, gr) for p, gr in zip(params, grads) if gr is not None]
        us = [(torch.randint(0, 2, p.shape, generator=generator, device="cpu").to(p.device) * 2 - 1).to(gr.dtype)
              for p, gr in pairs]
        hvs = torch.autograd.grad([gr for _, gr in pairs], [p for p, _ in pairs], us, allow_unused=True)
        with torch.no_grad():
            for g in self.param_groups:
                b2 = g["betas"][1]
                ids = {id(p) for p in g["params"]}
                for (p, _), u, hv in zip(pairs, us, hvs):
                    if id(p) not in ids or hv is None:
                        continue
                    st = self.state[p]
                    if "h" not in st:
                        st["h"] = torch.zeros_like(p, dtype=torch.float32)
                    st["h"].mul_(b2).add_((u * hv).float(), alpha=1 - b2)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1 = g["betas"][0]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if "m" not in st:
                    st["m"] = torch.zeros_like(p, dtype=torch.float32)
                if "h" not in st:
                    st["h"] = torch.zeros_like(p, dtype=torch.float32)
                if K.native_ok(p, p.grad):
                    K.sophia_step_(p, p.grad, st["m"], st["h"], lr=g["lr"], beta1=b1, rho=g["rho"],
                                   weight_decay=g["weight_decay"], eps=g["eps"])
                    continue
                st["m"].mul_(b1).add_(p.grad.float(), alpha=1 - b1)
                pf = p.float().mul_(1 - g["lr"] * g["weight_decay"])
                ratio = (st["m"].abs() / (g["rho"] * st["h"] + g["eps"])).clamp(max=1.0)
                p.copy_(pf - g["lr"] * st["m"].sign() * ratio)
        return loss


class Prodigy(Optimizer):
    """Parameter-free AdamW: the step size scale d is estimated from <g, x0 - x> / ||s||_1."""

    @reference_kwargs({"decouple": (True, None), "use_bias_correction": (False, None), "safeguard_warmup": (False, None),
                       "beta3": (None,)})
    def __init__(self, params, lr=1.0, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, d0=1e-6, d_coef=1.0, growth_rate=float("inf")):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, d=d0, d0=d0, d_coef=d_coef,
                                      growth_rate=growth_rate, k=0, d_numerator=0.0))

    @property
    def d(self) -> float:
        """Current estimate of the step-size scale D."""
        return float(self.param_groups[0]["d"])

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        g0 = self.param_groups[0]
        b1, b2 = g0["betas"]
        b3 = math.sqrt(b2)
        d, lr = g0["d"], g0["lr"]
        dlr = d * lr
        nums, dens = [], []            # 0-d device tensors: one host read per step, not two per tensor
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                gf = p.grad.float()
                st = self.state[p]
                if not st:
                    st["s"] = torch.zeros_like(gf)
                    st["p0"] = p.detach().float().clone()
                    st["m"], st["v"] = torch.zeros_like(gf), torch.zeros_like(gf)
                nums.append(torch.dot(gf.reshape(-1), (st["p0"] - p.float()).reshape(-1)))
                st["m"].mul_(b1).add_(gf, alpha=d * (1 - b1))
                st["v"].mul_(b2).addcmul_(gf, gf, value=d * d * (1 - b2))
                st["s"].mul_(b3).add_(gf, alpha=(d / g0["d0"]) * dlr)
                dens.append(st["s"].abs().sum())
        num, denom = g0["d_numerator"] * b3, 0.0
        if nums:
            dev = nums[0].device
            both = torch.stack([torch.stack([t.to(dev) for t in nums]).sum(), torch.stack([t.to(dev) for t in dens]).sum()]).tolist()
            num, denom = num + (d / g0["d0"]) * dlr * both[0], both[1]
        if denom > 0:
            d_hat = g0["d_coef"] * num / denom
            d = max(d, min(d_hat, d * g0["growth_rate"]))
        for g in self.param_groups:
            g["d"], g["d_numerator"], g["k"] = d, num, g["k"] + 1
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                pf = p.float()
                if g["weight_decay"]:
                    pf.mul_(1 - g["weight_decay"] * dlr)
                p.copy_(pf - dlr * st["m"] / (st["v"].sqrt() + d * g["eps"]))
        return loss


class ScheduleFreeAdamW(Optimizer):
    """Schedule-free AdamW (interpolated iterate y for gradients, averaged iterate x for evaluation).
    Call `.train()` before training steps and `.eval()` before evaluation / checkpointing."""

    def __init__(self, params, lr=2.5e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, warmup_steps=0, r=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, warmup_steps=warmup_steps,
                                      r=r, k=0, train_mode=True, weight_sum=0.0))

    @torch.no_grad()
    def _swap(self, to_train: bool):
        for g in self.param_groups:
            if g["train_mode"] == to_train:
                continue
            b1 = g["betas"][0]
            for p in g["params"]:
                st = self.state.get(p)
                if st and "z" in st:
                    w = (1 - b1) if to_train else (1 - 1 / b1)
                    p.copy_(torch.lerp(p.float(), st["z"], w))
            g["train_mode"] = to_train

    def train(self):
        self._swap(True)

    def eval(self):
        self._swap(False)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            k = g["k"] + 1
            sched = min(1.0, k / g["warmup_steps"]) if g["warmup_steps"] > 0 else 1.0
            lr = g["lr"] * sched * math.sqrt(1 - b2 ** k)
            w = (lr ** 2) * (k ** g["r"])
            g["weight_sum"] += w
            c = w / g["weight_sum"] if g["weight_sum"] > 0 else 0.0
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["z"] = p.detach().float().clone()
                    st["v"] = torch.zeros_like(p, dtype=torch.float32)
                if K.native_ok(p, p.grad):
                    K.schedule_free_(p, p.grad, st["z"], st["v"], lr=lr, beta1=b1, beta2=b2, eps=g["eps"],
                                     weight_decay=g["weight_decay"], c=c)
                    continue
                gf = p.grad.float()
                st["v"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
                gn = gf / (st["v"].sqrt() + g["eps"])
                y = p.float()
                if g["weight_decay"]:
                    gn = gn + g["weight_decay"] * y
                y = torch.lerp(y, st["z"], c)
                y.add_(gn, alpha=lr * (b1 * (1 - c) - 1))
                st["z"].sub_(gn, alpha=lr)
                p.copy_(y)
            g["k"] = k
        return loss


def _newton_schulz_bf16(G: torch.Tensor, steps: int) -> torch.Tensor:
    """The quintic iteration in bf16 on the tcgen05 GEMM (three GEMMs per step, the polynomial's additions folded
    into the GEMMs' alpha / accumulate epilogues).  Returns bf16."""
    from ..ops import gemm
    a, b, c = 3.4445, -4.7750, 2.0315
    t = G.shape[0] > G.shape[1]
    X = G.float().t() if t else G.float()
    X = (X / (X.norm() + 1e-7)).to(torch.bfloat16).contiguous()
    for _ in range(steps):
        A = gemm.matmul_nt(X, X)                                # A = X X^T (symmetric)
        B = A * b
        gemm.matmul_nt(A, A, out=B, accumulate=True, alpha=c)   # B = b A + c A A   (A^T = A)
        Xn = X * a
        gemm.matmul_nn(B, X, out=Xn, accumulate=True)           # X <- a X + B X
        X = Xn
    return X.t() if t else X


def newton_schulz_orthogonalize(G: torch.Tensor, steps: int = 5) -> torch.Tensor:
    a, b, c = 3.4445, -4.7750, 2.0315
    if G.is_cuda and G.dim() == 2 and G.shape[0] % 8 == 0 and G.shape[1] % 8 == 0:
        return _newton_schulz_bf16(G, steps)
    X = G.float()
    t = X.shape[-2] > X.shape[-1]
    if t:
        X = X.transpose(-1, -2)
    X = X / (X.norm(dim=(-2, -1), keepdim=True) + 1e-7)
    for _ in range(steps):
        A = X @ X.transpose(-1, -2)
        X = a * X + (b * A + c * A @ A) @ X
    return X.transpose(-1, -2) if t else X


class Muon(Optimizer):
    """Momentum + Newton-Schulz orthogonalisation for 2-D weights; AdamW for everything else."""

    def __init__(self, params, lr=0.02, momentum=0.95, nesterov=True, ns_steps=5, weight_decay=0.0,
                 adamw_lr=3e-4, adamw_betas=(0.9, 0.95), adamw_eps=1e-8):
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, ns_steps=ns_steps,
                                      weight_decay=weight_decay, adamw_lr=adamw_lr, adamw_betas=adamw_betas, adamw_eps=adamw_eps))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            for p in g["params"]:
                if p.grad is None:
                    continue
                gf = p.grad.float()
                st = self.state[p]
                pf = p.float()
                if gf.dim() == 2 and min(gf.shape) > 1:
                    if not st:
                        st["buf"] = torch.zeros_like(gf)
                    st["buf"].mul_(g["momentum"]).add_(gf)
                    u = gf.add(st["buf"], alpha=g["momentum"]) if g["nesterov"] else st["buf"]
                    u = newton_schulz_orthogonalize(u, g["ns_steps"]) * max(1.0, gf.shape[0] / gf.shape[1]) ** 0.5
                    pf.mul_(1 - g["lr"] * g["weight_decay"]).add_(u, alpha=-g["lr"])
                else:
                    if not st:
                        st["step"], st["m"], st["v"] = 0, torch.zeros_like(gf), torch.zeros_like(gf)
                    st["step"] += 1
                    b1, b2 = g["adamw_betas"]
                    st["m"].mul_(b1).add_(gf, alpha=1 - b1)
                    st["v"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
                    pf.addcdiv_(st["m"] / (1 - b1 ** st["step"]), (st["v"] / (1 - b2 ** st["step"])).sqrt() + g["adamw_eps"],
                                value=-g["adamw_lr"])
                p.copy_(pf)
        return loss


class ADOPT(Optimizer):
    """Adam with the second moment of the PREVIOUS step in the normaliser (converges for any beta2)."""

    @reference_kwargs({"decouple": (True, None)})       # weight decay is always the decoupled (AdamW) form here
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.9999), eps=1e-6, weight_decay=0.0, clip_lambda=lambda k: k ** 0.25):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, clip_lambda=clip_lambda))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    gf = p.grad.float()
                    st["step"], st["m"], st["v"] = 1, torch.zeros_like(gf), gf * gf
                    continue
                st["step"] += 1
                if K.native_ok(p, p.grad):
                    clip = g["clip_lambda"](st["step"]) if g["clip_lambda"] is not None else None
                    K.adopt_(p, p.grad, st["m"], st["v"], lr=g["lr"], beta1=b1, beta2=b2, eps=g["eps"],
                             weight_decay=g["weight_decay"], clip=clip)
                    continue
                gf = p.grad.float()
                n = gf / torch.clamp(st["v"].sqrt(), min=g["eps"])
                if g["clip_lambda"] is not None:
                    c = g["clip_lambda"](st["step"])
                    n.clamp_(-c, c)
                st["m"].mul_(b1).add_(n, alpha=1 - b1)
                pf = p.float().mul_(1 - g["lr"] * g["weight_decay"])
                p.copy_(pf - g["lr"] * st["m"])
                st["v"].mul_(b2).addcmul_(gf, gf, value=1 - b2)
        return loss


_OPTIMIZERS = {"adamw": AdamW, "fused_adamw": AdamW, "adam8bit": Adam8bit, "adamw_8bit": Adam8bit, "lion": Lion,
               "lamb": LAMB, "adafactor": AdaFactor, "distributed_adafactor": DistributedAdaFactor, "came": CAME, "sophia": SophiaG, "sophiag": SophiaG,
               "prodigy": Prodigy, "schedule_free": ScheduleFreeAdamW, "schedulefree": ScheduleFreeAdamW, "muon": Muon,
               "adopt": ADOPT}


def create_optimizer(params, config=None, name: str | None = None, *extra, **kw) -> Optimizer:
    """From a SOTAConfig `optimizer` section (or a name + keyword arguments).  The reference's
    `create_optimizer(name, params, lr, weight_decay, **kwargs)` (a string first) is taken as well
    (data_pipeline/trainer/optimizers/sota_optimizers.py create_optimizer)."""
    if isinstance(params, str):                               # (name, params, lr, weight_decay)
        ref_name, params, lr = params, config, name
        if lr is not None:
            kw.setdefault("lr", lr)
        if extra:
            kw.setdefault("weight_decay", extra[0])
        config, name, extra = None, ref_name, extra[1:]
    if extra:
        raise TypeError("create_optimizer() got too many positional arguments")
    params = [p for p in params if p.requires_grad] if not isinstance(params, list) or (params and torch.is_tensor(params[0])) else params
    if config is not None:
        name = name or getattr(config.type, "value", config.type)
        base = dict(lr=config.learning_rate, weight_decay=config.weight_decay)
        if name in ("adamw", "fused_adamw", "adam8bit", "lamb", "adopt", "schedule_free", "prodigy"):
            base["betas"] = tuple(config.betas)
            base["eps"] = config.eps
        if name == "lion":
            base["betas"] = tuple(config.lion_betas)
        if name == "adafactor":
            base = dict(lr=config.learning_rate, weight_decay=config.weight_decay, relative_step=False)
        if name in ("came",):
            base = dict(lr=config.learning_rate, weight_decay=config.weight_decay)
        if name in ("sophia", "sophiag", "muon"):
            base = dict(lr=config.learning_rate, weight_decay=config.weight_decay)
        base.update(kw)
        kw = base
    name = (name or "adamw").lower()
    if name not in _OPTIMIZERS:
        raise ValueError(f"unknown optimizer {name!r}; choose from {sorted(_OPTIMIZERS)}")
    return _OPTIMIZERS[name](params, **kw)


# ------------------------------------------------------------------------------------------------ reference surface
import math as _math  # noqa: E402
from dataclasses import dataclass as _dataclass, field as _field  # noqa: E402
from enum import Enum as _Enum, IntEnum as _IntEnum  # noqa: E402
from typing import NamedTuple as _NamedTuple  # noqa: E402


class FactorizationMode(_IntEnum):
    NONE = 1
    ROW_COL = 2
    BLOCK = 3


class QuantizationMode(_Enum):
    NONE = "none"
    DYNAMIC_8BIT = "dynamic_8bit"
    BLOCK_WISE_8BIT = "block_wise_8bit"
    STOCHASTIC_8BIT = "stochastic_8bit"


class OptimizerState(_Enum):
    UNINITIALIZED = "uninitialized"
    INITIALIZED = "initialized"
    STEPPED = "stepped"
    CLOSED = "closed"


@_dataclass(frozen=True)
class AdaFactorConfig:
    """Hyper-parameters of `AdaFactor` as one immutable record (data_pipeline/trainer/optimizers/adafactor.py:117);
    `build(params)` makes the optimizer."""
    lr: float | None = None
    eps1: float = 1e-30
    eps2: float = 1e-3
    clip_threshold: float = 1.0
    decay_rate: float = -0.8
    beta1: float | None = None
    weight_decay: float = 0.0
    scale_parameter: bool = True
    relative_step: bool = True
    warmup_init: bool = False
    warmup_steps: int = 10000
    min_lr: float = 1e-6
    max_lr: float = 1.0
    factorization_threshold: int = 128

    def build(self, params) -> "AdaFactor":
        return AdaFactor(params, lr=self.lr, eps=(self.eps1, self.eps2), clip_threshold=self.clip_threshold,
                         decay_rate=self.decay_rate, beta1=self.beta1, weight_decay=self.weight_decay,
                         scale_parameter=self.scale_parameter, relative_step=self.relative_step,
                         warmup_init=self.warmup_init)


class ParamState(_NamedTuple):
    step: int
    factored: bool
    exp_avg: torch.Tensor | None
    exp_avg_sq: torch.Tensor | None
    exp_avg_sq_row: torch.Tensor | None
    exp_avg_sq_col: torch.Tensor | None
    kahan_comp: torch.Tensor | None = None


class AdaFactorState:
    """State of one parameter, allocated on first use: factored row / column second moments for matrices, a full
    second moment otherwise, optional first moment and Kahan compensation.  `snapshot()` gives a `ParamState`."""

    def __init__(self, shape, device, dtype, factored: bool, use_momentum: bool, use_kahan: bool = False):
        self.step, self.factored, self.shape, self.device, self.dtype = 0, factored and len(shape) >= 2, tuple(shape), device, dtype
        self.use_momentum, self.use_kahan = use_momentum, use_kahan
        self.exp_avg = self.exp_avg_sq = self.exp_avg_sq_row = self.exp_avg_sq_col = self.kahan_comp = None
        self.is_initialized = False

    def initialize(self) -> "AdaFactorState":
        z = lambda s: torch.zeros(s, device=self.device, dtype=torch.float32)      # noqa: E731
        if self.factored:
            self.exp_avg_sq_row, self.exp_avg_sq_col = z(self.shape[:-1]), z(self.shape[:-2] + self.shape[-1:])
        else:
            self.exp_avg_sq = z(self.shape)
        if self.use_momentum:
            self.exp_avg = z(self.shape)
        if self.use_kahan:
            self.kahan_comp = z(self.shape)
        self.is_initialized = True
        return self

    def memory_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.exp_avg, self.exp_avg_sq, self.exp_avg_sq_row,
                                                          self.exp_avg_sq_col, self.kahan_comp) if t is not None)

    def snapshot(self) -> ParamState:
        return ParamState(self.step, self.factored, self.exp_avg, self.exp_avg_sq, self.exp_avg_sq_row,
                          self.exp_avg_sq_col, self.kahan_comp)

    memory_footprint = memory_bytes

    _TENSORS = ("exp_avg", "exp_avg_sq", "exp_avg_sq_row", "exp_avg_sq_col", "kahan_comp")

    def to_dict(self) -> dict:
        """Plain-dict form for a checkpoint: the step, the layout flags and clones of the tensors that exist."""
        d = {"step": self.step, "factored": self.factored, "shape": list(self.shape), "dtype": str(self.dtype),
             "use_momentum": self.use_momentum, "use_kahan": self.use_kahan}
        for k in self._TENSORS:
            t = getattr(self, k)
            if t is not None:
                d[k] = t.detach().clone()
        return d

    @classmethod
    @reference_kwargs(state_dict="d")
    def from_dict(cls, d: dict, device=None, *, shape=None, dtype=None, use_momentum: bool | None = None) -> "AdaFactorState":
        """`shape`, `dtype` and `use_momentum` fill in what a dictionary written elsewhere does not carry."""
        d = dict(d)
        if shape is not None:
            d.setdefault("shape", list(shape))
        if dtype is not None:
            d.setdefault("dtype", str(dtype))
        if use_momentum is not None:
            d.setdefault("use_momentum", use_momentum)
        d.setdefault("factored", "exp_avg_sq_row" in d)
        dtype = getattr(torch, str(d.get("dtype", "torch.float32")).replace("torch.", ""))
        st = cls(tuple(d["shape"]), device, dtype, bool(d["factored"]), bool(d.get("use_momentum", "exp_avg" in d)),
                 bool(d.get("use_kahan", "kahan_comp" in d)))
        st.step = int(d.get("step", 0))
        for k in cls._TENSORS:
            if k in d:
                setattr(st, k, d[k].to(device) if device is not None else d[k].clone())
        st.is_initialized = any(k in d for k in cls._TENSORS)
        return st


@_dataclass
class ProfilingStats:
    total_step_time_ns: int = 0
    kernel_time_ns: int = 0
    memory_allocated_bytes: int = 0
    memory_peak_bytes: int = 0
    num_factorized_params: int = 0
    num_full_params: int = 0
    triton_kernel_calls: int = 0
    fused_updates: int = 0


@_dataclass
class OptimizerMetrics:
    total_steps: int = 0
    total_params: int = 0
    kernel_time_ns: int = 0
    memory_allocated_bytes: int = 0
    grad_norm_history: list = _field(default_factory=list)

    def record_step(self, grad_norm: float, kernel_time_ns: int = 0) -> None:
        self.total_steps += 1
        self.kernel_time_ns += kernel_time_ns
        if len(self.grad_norm_history) < 1000:
            self.grad_norm_history.append(float(grad_norm))


def compute_rms_jit(tensor: torch.Tensor, eps: float = 1e-30) -> float:
    return float(torch.sqrt(tensor.float().pow(2).mean().clamp(min=eps)))


def compute_rho_jit(step: int, decay_rate: float, max_rho: float = 0.999) -> float:
    """Second-moment decay of AdaFactor at `step`: min(1 - (step + 1)^decay_rate, max_rho)."""
    return min(1.0 - _math.pow(float(step + 1), decay_rate), max_rho)


def determine_factorization(shape, threshold: int = 128) -> FactorizationMode:
    """NONE for vectors and for matrices with a side below `threshold`; ROW_COL for matrices; BLOCK above 10M values."""
    if len(shape) < 2 or shape[-1] < threshold or shape[-2] < threshold:
        return FactorizationMode.NONE
    return FactorizationMode.BLOCK if _math.prod(shape) > 10_000_000 else FactorizationMode.ROW_COL


def get_triton_block_config(numel: int, dtype=None) -> tuple[int, int, int]:
    """(block, warps, stages) the reference's Triton update kernels would pick; informational (the CUDA update kernels
    here use fixed 256-thread blocks with 16-byte accesses)."""
    return (256, 2, 2) if numel < 1024 else (512, 4, 2) if numel < 16384 else (1024, 8, 3) if numel < 131072 else (2048, 8, 4)


def get_triton_version():
    """Triton is not used by this framework."""
    return None


def create_adamw(params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01,
                 amsgrad: bool = False, max_grad_norm: float | None = None, use_triton: bool = True) -> AdamW:
    opt = AdamW(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad, fused=True)
    opt.max_grad_norm = max_grad_norm
    return opt


def create_lion(params, lr: float = 1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0, use_triton: bool = True) -> Lion:
    return Lion(params, lr=lr, betas=betas, weight_decay=weight_decay)


def create_lamb(params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-6, weight_decay: float = 0.01,
                max_trust_ratio: float = 10.0) -> LAMB:
    return LAMB(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, clamp_trust=(0.0, max_trust_ratio))


def create_adafactor(params, lr: float | None = None, eps=(1e-30, 1e-3), clip_threshold: float = 1.0,
                     decay_rate: float = -0.8, beta1: float | None = None, weight_decay: float = 0.0,
                     scale_parameter: bool = True, relative_step: bool = True, warmup_init: bool = False,
                     **_ignored) -> AdaFactor:
    return AdaFactor(params, lr=lr, eps=eps, clip_threshold=clip_threshold, decay_rate=decay_rate, beta1=beta1,
                     weight_decay=weight_decay, scale_parameter=scale_parameter, relative_step=relative_step,
                     warmup_init=warmup_init)


_ADAFACTOR_BY_SIZE = {"1b": dict(clip_threshold=1.0), "7b": dict(clip_threshold=1.0), "13b": dict(clip_threshold=0.8),
                      "70b": dict(clip_threshold=0.5), "175b": dict(clip_threshold=0.3)}


def create_adafactor_for_llm(params, model_size: str = "7b", **kwargs) -> AdaFactor:
    """AdaFactor with relative step, parameter scaling and warm-up initialisation, and an update clip that tightens with
    model size (1.0 up to 7B, 0.8 at 13B, 0.5 at 70B, 0.3 at 175B)."""
    cfg = dict(_ADAFACTOR_BY_SIZE.get(model_size.lower(), _ADAFACTOR_BY_SIZE["7b"]))
    cfg.update(kwargs)
    return create_adafactor(params, lr=None, relative_step=True, scale_parameter=True, warmup_init=True, **cfg)


class KahanAccumulator:
    """Compensated running sum of floats."""
    __slots__ = ("_sum", "_compensation")

    def __init__(self, initial: float = 0.0):
        self._sum, self._compensation = float(initial), 0.0

    def add(self, value: float) -> None:
        y = value - self._compensation
        t = self._sum + y
        self._compensation = (t - self._sum) - y
        self._sum = t

    @property
    def value(self) -> float:
        return self._sum

    def reset(self, initial: float = 0.0) -> None:
        self._sum, self._compensation = float(initial), 0.0


def stable_softmax(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    e = torch.exp(x - x.max(dim=dim, keepdim=True).values)
    return e / e.sum(dim=dim, keepdim=True)


def safe_sqrt(x: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    return torch.sqrt(x + eps)


def rms_norm(x: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    return torch.sqrt(torch.mean(x * x) + eps)


class GradScalerProtocol:
    """What an optimizer expects of a loss scaler: `get_scale()` and `update(new_scale=None)`
    (`parallel.dist_utils.GradScaler` and `torch.amp.GradScaler` both qualify)."""

    def get_scale(self) -> float: ...
    def update(self, new_scale: float | None = None) -> None: ...


class BaseOptimizer(Optimizer):
    """Base for optimizers written as one `_update(p, grad, state, group)` rule: lazy per-parameter state, optional
    global-norm clipping before the update (`max_grad_norm` in the defaults), step metrics.
    (data_pipeline/trainer/optimizers/base.py:248, sota_optimizers.py:539)"""

    @reference_kwargs({"use_triton": ANY, "fused": ANY})
    def __init__(self, params, defaults: dict, *, foreach=None, differentiable: bool = False):
        defaults = dict(defaults)
        defaults.setdefault("max_grad_norm", None)
        super().__init__(params, defaults)
        self.metrics = OptimizerMetrics(total_params=sum(p.numel() for g in self.param_groups for p in g["params"]))
        self.lifecycle = OptimizerState.INITIALIZED
        self._grad_scale = 1.0
        self._step_count = 0

    # ---- data_pipeline/trainer/optimizers/adamw.py:1001-1152, sota_optimizers.py:600-640
    @property
    def step_count(self) -> int:
        return self._step_count

    def set_grad_scale(self, scale: float) -> None:
        """The factor the loss was multiplied by (fp16 loss scaling): gradients are divided by it before the update."""
        if not scale > 0:
            raise ValueError("grad scale must be positive")
        self._grad_scale = float(scale)

    def get_grad_scale(self) -> float:
        return self._grad_scale

    def get_metrics(self) -> "OptimizerMetrics":
        return self.metrics

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float, norm_type: float = 2.0, error_if_nonfinite: bool = False) -> torch.Tensor:
        """Clip over ALL parameter groups together; returns the norm before clipping."""
        ps = [p for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not ps:
            return torch.zeros(())
        return torch.nn.utils.clip_grad_norm_(ps, max_norm, norm_type, error_if_nonfinite=error_if_nonfinite)

    def close(self) -> None:
        """Drop the per-parameter state (frees its memory); the optimizer takes no further steps."""
        self.state.clear()
        self.lifecycle = OptimizerState.CLOSED

    def _init_state(self, p: torch.Tensor, group: dict) -> dict:
        return {"step": 0}

    def _update(self, p: torch.Tensor, grad: torch.Tensor, state: dict, group: dict) -> None:
        raise NotImplementedError

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        if self.lifecycle is OptimizerState.CLOSED:
            raise RuntimeError("step() on a closed optimizer")
        norm = 0.0
        for g in self.param_groups:
            ps = [p for p in g["params"] if p.grad is not None]
            if self._grad_scale != 1.0:
                torch._foreach_div_([p.grad for p in ps], self._grad_scale)
            if g.get("max_grad_norm"):
                norm = float(clip_grad_norm_(ps, g["max_grad_norm"]))
            for p in ps:
                st = self.state[p]
                if not st:
                    st.update(self._init_state(p, g))
                st["step"] = st.get("step", 0) + 1
                self._update(p, p.grad, st, g)
        self.metrics.record_step(norm)
        self.lifecycle = OptimizerState.STEPPED
        self._step_count += 1
        return loss


BaseApexOptimizer = BaseOptimizer


def compute_grad_norm(parameters, norm_type: float = 2.0) -> tuple[float, float, float]:
    """(global norm, largest per-parameter norm, smallest per-parameter norm) of the gradients present."""
    norms = [torch.linalg.vector_norm(p.grad.detach().float(), norm_type) for p in parameters if p.grad is not None]
    if not norms:
        return 0.0, 0.0, 0.0
    stacked = torch.stack(norms)
    total = stacked.max() if norm_type == float("inf") else torch.linalg.vector_norm(stacked, norm_type)
    return float(total), float(stacked.max()), float(stacked.min())


def clip_grad_value_(parameters, clip_value: float):
    """Clamp every gradient element to [-clip_value, clip_value] in place; returns `core.types.GradientInfo` with the
    norms BEFORE clamping."""
    from ..core.types import GradientInfo
    ps = [p for p in parameters if p.grad is not None]
    total, mx, mn = compute_grad_norm(ps)
    clipped = any(bool((p.grad.abs() > clip_value).any()) for p in ps)
    overflow = any(not bool(torch.isfinite(p.grad).all()) for p in ps)
    for p in ps:
        p.grad.clamp_(-clip_value, clip_value)
    return GradientInfo(total, mx, mn, clipped, overflow)


def get_optimizer_memory_footprint(optimizer: Optimizer, param_bytes: int = 4) -> dict:
    """Bytes held in optimizer state, per state key, and the ratio to the two fp32 moments of plain Adam."""
    by_key: dict[str, int] = {}
    n_params = 0
    for g in optimizer.param_groups:
        for p in g["params"]:
            n_params += p.numel()
            for k, v in optimizer.state.get(p, {}).items():
                if torch.is_tensor(v):
                    by_key[k] = by_key.get(k, 0) + v.numel() * v.element_size()
    total = sum(by_key.values())
    return {"total_bytes": total, "state_bytes": by_key, "param_bytes": n_params * param_bytes,
            "compression_ratio": (2 * 4 * n_params) / total if total else float("inf")}


def check_optimizer_compatibility(optimizer: Optimizer, model) -> dict:
    """Things that make an optimizer / model pair fail or waste memory: sparse or meta parameters, trainable parameters
    the optimizer does not hold, parameters it holds that the model does not have, half-precision parameters without
    fp32 masters."""
    warnings, recommendations = [], []
    held = {id(p) for g in optimizer.param_groups for p in g["params"]}
    own = {id(p): n for n, p in model.named_parameters()}
    for n, p in model.named_parameters():
        if p.is_sparse:
            warnings.append(f"sparse parameter: {n}")
        if p.device.type == "meta":
            warnings.append(f"meta-device parameter: {n}")
        if p.requires_grad and id(p) not in held:
            warnings.append(f"trainable parameter not in the optimizer: {n}")
    stray = len([i for i in held if i not in own])
    if stray:
        warnings.append(f"{stray} optimizer parameter(s) do not belong to the model")
    if any(p.dtype in (torch.float16, torch.bfloat16) and p.requires_grad for p in model.parameters()):
        recommendations.append("half-precision trainable parameters: use the sharded engine (fp32 master shards) or "
                               "keep fp32 master weights")
    blocking = [w for w in warnings if w.startswith(("meta", "trainable", "sparse"))]
    return {"is_compatible": not blocking, "warnings": warnings, "recommendations": recommendations}


# ---- type aliases and tuning constants of data_pipeline/trainer/optimizers/{base,adamw,adafactor}.py.  The block
# sizes describe the reference's Triton kernels; the kernels of csrc/optim.cu choose their own launch shapes.
from typing import Any as _Any, Dict as _Dict, TypeVar as _TypeVar  # noqa: E402

ParamGroup = _Dict[str, _Any]
StateDict = _Dict[str, _Any]
ParamT = _TypeVar("ParamT", bound=torch.Tensor)
StateT = _TypeVar("StateT", bound=_Dict[str, _Any])
CACHE_LINE_SIZE, CACHE_LINE_ELEMENTS_FP32, CACHE_LINE_ELEMENTS_FP16 = 64, 16, 32
EPS_FP32, EPS_FP16, EPS_BF16 = 1e-30, 1e-7, 1e-7
DEFAULT_BLOCK_SIZE, MAX_BLOCK_SIZE, MIN_ELEMENTS_FOR_TRITON = 1024, 4096, 8192
TRITON_BLOCK_SIZE, TRITON_NUM_WARPS, TRITON_NUM_STAGES = 1024, 8, 3
MULTI_TENSOR_THRESHOLD, MAX_TENSORS_PER_KERNEL = 4 * 1024 * 1024, 64
