"""Learning-rate schedules.

Formulas follow data_pipeline/trainer/schedulers/sota_schedulers.py:64-159 (warm-up factor (step+1)/warmup, then
min_lr + (base - min_lr) * decay(progress); WSD stable/decay phases with cosine | linear | sqrt decay),
data_pipeline/trainer/schedulers/__init__.py:108-141,258-271 (warm-up kinds, cosine) and the REX / one-cycle /
polynomial / inverse-sqrt / cosine-restart variants of :166-447.  A scheduler drives any object with
`param_groups` (torch optimizers and this framework's flat engine alike) and is a pure function of the step,
so resuming only needs `last_step`.
"""
from __future__ import annotations

import math
from typing import Callable

from ..utils.refargs import ANY, reference_kwargs


def warmup_factor(step: int, warmup_steps: int, kind: str = "linear") -> float:
    if warmup_steps <= 0 or step >= warmup_steps:
        return 1.0
    p = (step + 1) / warmup_steps
    if kind == "exponential":
        return math.exp(-5.0 * (1.0 - p))
    if kind == "constant":
        return 1.0 / max(warmup_steps, 1) if False else 0.1
    return p


class BaseScheduler:
    """lr(step) = base_lr * factor(step). Subclasses implement `decay(progress_step)` in [0, 1]."""

    def __init__(self, optimizer, num_training_steps: int, warmup_steps: int = 0, min_lr_ratio: float = 0.0,
                 warmup_type: str = "linear", last_step: int = -1, *, warmup_ratio: float = 0.0,
                 warmup_start_lr: float | None = None, min_lr: float | None = None, last_epoch: int | None = None):
        """`warmup_ratio` gives the warm-up length as a fraction of the run when `warmup_steps` is 0; `warmup_start_lr`
        is the absolute rate the warm-up starts from (default 0, i.e. the pure ramp); `min_lr` is the floor as an absolute
        rate (`min_lr_ratio` as a fraction of the base rate; the larger of the two holds); `last_epoch` is torch's name
        for `last_step`.  (data_pipeline/trainer/schedulers: BaseScheduler / BaseEnhancedScheduler constructors.)"""
        self.optimizer = optimizer
        self.num_training_steps = max(1, int(num_training_steps))
        self.warmup_steps = int(warmup_steps) if warmup_steps else int(warmup_ratio * self.num_training_steps)
        self.min_lr_ratio = float(min_lr_ratio)
        self.warmup_type = getattr(warmup_type, "value", warmup_type)
        self.base_lrs = [g.get("initial_lr", g["lr"]) for g in optimizer.param_groups]
        for g, b in zip(optimizer.param_groups, self.base_lrs):
            g.setdefault("initial_lr", b)
        ref = max(self.base_lrs[0], 1e-30)
        if min_lr is not None:
            self.min_lr_ratio = max(self.min_lr_ratio, float(min_lr) / ref)
        self.warmup_start_ratio = 0.0 if warmup_start_lr is None else float(warmup_start_lr) / ref
        self.last_step = last_step if last_epoch is None else last_epoch
        self.step()

    def decay(self, s: int) -> float:   # s = steps after warm-up
        return 1.0

    def factor(self, step: int) -> float:
        if step < self.warmup_steps:
            w = warmup_factor(step, self.warmup_steps, self.warmup_type)
            return self.warmup_start_ratio + (1.0 - self.warmup_start_ratio) * w
        d = self.decay(step - self.warmup_steps)
        return self.min_lr_ratio + (1.0 - self.min_lr_ratio) * d

    def get_lr(self, step: int | None = None) -> list[float]:
        step = self.last_step if step is None else step
        f = self.factor(max(step, 0))
        return [b * f for b in self.base_lrs]

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for g in self.optimizer.param_groups]

    def step(self, step: int | None = None) -> None:
        """Advance by one, or jump to `step`."""
        self.last_step = self.last_step + 1 if step is None else int(step)
        for g, lr in zip(self.optimizer.param_groups, self.get_lr()):
            g["lr"] = lr

    def state_dict(self) -> dict:
        return {"last_step": self.last_step, "base_lrs": list(self.base_lrs)}

    @reference_kwargs(state_dict="sd")
    def load_state_dict(self, sd: dict) -> None:
        self.last_step = sd["last_step"] - 1
        self.base_lrs = list(sd.get("base_lrs", self.base_lrs))
        self.step()


class ConstantScheduler(BaseScheduler):
    pass


class CosineScheduler(BaseScheduler):
    def __init__(self, optimizer, num_training_steps, warmup_steps=0, min_lr_ratio=0.0, num_cycles: float = 0.5, **kw):
        self.num_cycles = num_cycles
        super().__init__(optimizer, num_training_steps, warmup_steps, min_lr_ratio, **kw)

    def decay(self, s):
        total = max(1, self.num_training_steps - self.warmup_steps)
        p = min(1.0, s / total)
        return 0.5 * (1.0 + math.cos(math.pi * 2.0 * self.num_cycles * p))


class LinearScheduler(BaseScheduler):
    def decay(self, s):
        total = max(1, self.num_training_steps - self.warmup_steps)
        return max(0.0, 1.0 - s / total)


class PolynomialDecayScheduler(BaseScheduler):
    def __init__(self, optimizer, num_training_steps, warmup_steps=0, min_lr_ratio=0.0, power: float = 1.0, **kw):
        self.power = power
        super().__init__(optimizer, num_training_steps, warmup_steps, min_lr_ratio, **kw)

    def decay(self, s):
        total = max(1, self.num_training_steps - self.warmup_steps)
        return max(0.0, 1.0 - min(1.0, s / total)) ** self.power


class InverseSquareRootScheduler(BaseScheduler):
    @reference_kwargs(warmup_init_lr="warmup_start_lr")
    def __init__(self, optimizer, num_training_steps: int, warmup_steps: int = 0, min_lr_ratio: float = 0.0, **kw):
        super().__init__(optimizer, num_training_steps, warmup_steps, min_lr_ratio, **kw)

    def decay(self, s):
        w = max(1, self.warmup_steps)
        return math.sqrt(w / (w + s))


class WSDScheduler(BaseScheduler):
    """Warm-up / stable / decay."""

    def __init__(self, optimizer, num_training_steps, warmup_steps=0, min_lr_ratio=0.0, stable_ratio: float = 0.8,
                 stable_steps: int | None = None, decay_type: str = "cosine", **kw):
        rest = max(0, int(num_training_steps) - int(warmup_steps))
        self.stable_steps = int(stable_steps) if stable_steps is not None else int(rest * stable_ratio)
        self.decay_steps = max(1, rest - self.stable_steps)
        self.decay_type = decay_type
        super().__init__(optimizer, num_training_steps, warmup_steps, min_lr_ratio, **kw)

    def decay(self, s):
        if s < self.stable_steps:
            return 1.0
        p = min(1.0, (s - self.stable_steps) / self.decay_steps)
        if self.decay_type == "linear":
            return 1.0 - p
        if self.decay_type == "sqrt":
            return 1.0 - math.sqrt(p)
        return 0.5 * (1.0 + math.cos(math.pi * p))


class REXScheduler(BaseScheduler):
    """Reflected exponential: (1 - p) / ((1 - gamma) + gamma (1 - p)), gamma = 0.5 in the paper."""

    def __init__(self, optimizer, num_training_steps: int, warmup_steps: int = 0, min_lr_ratio: float = 0.0,
                 gamma: float = 0.5, **kw):
        self.gamma = float(gamma)
        super().__init__(optimizer, num_training_steps, warmup_steps, min_lr_ratio, **kw)

    def decay(self, s):
        total = max(1, self.num_training_steps - self.warmup_steps)
        p = min(1.0, s / total)
        return (1.0 - p) / ((1.0 - self.gamma) + self.gamma * (1.0 - p))


class CosineRestartScheduler(BaseScheduler):
    def __init__(self, optimizer, num_training_steps, warmup_steps=0, min_lr_ratio=0.0, cycle_steps: int | None = None,
                 cycle_mult: float = 1.0, restart_decay: float = 1.0, **kw):
        self.cycle_steps = cycle_steps or max(1, (int(num_training_steps) - int(warmup_steps)) // 4)
        self.cycle_mult, self.restart_decay = cycle_mult, restart_decay
        super().__init__(optimizer, num_training_steps, warmup_steps, min_lr_ratio, **kw)

    def decay(self, s):
        length, amp = self.cycle_steps, 1.0
        while s >= length:
            s -= length
            length = max(1, int(length * self.cycle_mult))
            amp *= self.restart_decay
        return amp * 0.5 * (1.0 + math.cos(math.pi * s / length))


class OneCycleScheduler(BaseScheduler):
    """Rise from base/div to base*max_lr_ratio over pct_start, anneal to base/final_div (cosine)."""

    def __init__(self, optimizer, num_training_steps, max_lr_ratio: float = 10.0, pct_start: float = 0.3,
                 div_factor: float = 25.0, final_div_factor: float = 1e4, **kw):
        self.max_lr_ratio, self.pct_start = max_lr_ratio, pct_start
        self.div_factor, self.final_div_factor = div_factor, final_div_factor
        kw.pop("warmup_steps", None)
        kw.pop("min_lr_ratio", None)
        super().__init__(optimizer, num_training_steps, 0, 0.0, **kw)

    def factor(self, step):
        up = max(1, int(self.num_training_steps * self.pct_start))
        hi, lo, fin = self.max_lr_ratio, self.max_lr_ratio / self.div_factor, self.max_lr_ratio / self.final_div_factor
        if step < up:
            p = step / up
            return lo + (hi - lo) * 0.5 * (1 - math.cos(math.pi * p))
        p = min(1.0, (step - up) / max(1, self.num_training_steps - up))
        return fin + (hi - fin) * 0.5 * (1 + math.cos(math.pi * p))


class CosineRestartsScheduler(BaseScheduler):
    """Cosine annealing with warm restarts, parameterised by the NUMBER of cycles over the decay span
    (data_pipeline/trainer/schedulers/__init__.py:274-320): cycle c starts at base * cycle_decay^c and anneals to the
    floor; `restart_warmup_steps` ramps linearly into every cycle after the first.  `CosineRestartScheduler` is the
    form parameterised by cycle length."""

    def __init__(self, optimizer, num_training_steps, warmup_steps=0, min_lr_ratio=0.0, num_cycles: float = 1.0,
                 cycle_decay: float = 1.0, restart_warmup_steps: int = 0, **kw):
        self.num_cycles, self.cycle_decay, self.restart_warmup_steps = num_cycles, cycle_decay, restart_warmup_steps
        super().__init__(optimizer, num_training_steps, warmup_steps, min_lr_ratio, **kw)

    def decay(self, s):
        total = max(1, self.num_training_steps - self.warmup_steps)
        if s >= total:
            return 0.0
        x = s / total * self.num_cycles
        cycle = math.floor(x)
        amp = self.cycle_decay ** cycle * 0.5 * (1.0 + math.cos(math.pi * (x - cycle)))
        if cycle > 0 and self.restart_warmup_steps > 0:
            into = s - cycle * total / self.num_cycles            # steps since this cycle began
            amp *= min(1.0, (into + 1) / self.restart_warmup_steps)
        return amp


# names of the reference's first-generation schedulers (data_pipeline/trainer/schedulers/__init__.py:348,390) and the
# base class of its second generation (sota_schedulers.py:26)
PolynomialScheduler = PolynomialDecayScheduler
InverseSqrtScheduler = InverseSquareRootScheduler
BaseEnhancedScheduler = BaseScheduler


def get_cosine_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int,
                                    min_lr_ratio: float = 0.0) -> CosineScheduler:
    """Linear warm-up, cosine decay to min_lr_ratio * base (data_pipeline/trainer/schedulers/__init__.py:579)."""
    return CosineScheduler(optimizer, num_training_steps, warmup_steps=num_warmup_steps, min_lr_ratio=min_lr_ratio)


def get_linear_schedule_with_warmup(optimizer, num_warmup_steps: int, num_training_steps: int) -> LinearScheduler:
    """Linear warm-up, linear decay to zero (data_pipeline/trainer/schedulers/__init__.py:599)."""
    return LinearScheduler(optimizer, num_training_steps, warmup_steps=num_warmup_steps, min_lr_ratio=0.0)


_REGISTRY: dict[str, Callable] = {
    "cosine": CosineScheduler, "linear": LinearScheduler, "constant": ConstantScheduler, "wsd": WSDScheduler,
    "polynomial": PolynomialDecayScheduler, "inverse_sqrt": InverseSquareRootScheduler, "rex": REXScheduler,
    "cosine_restart": CosineRestartScheduler, "cosine_restarts": CosineRestartScheduler,
    "cosine_with_restarts": CosineRestartsScheduler, "onecycle": OneCycleScheduler,
    "one_cycle": OneCycleScheduler,
}


def create_scheduler(optimizer, scheduler_type: str = "cosine", num_training_steps: int = 1000, warmup_steps: int = 0,
                     warmup_ratio: float = 0.0, min_lr_ratio: float = 0.0, **kw) -> BaseScheduler:
    """warm-up = warmup_steps, else int(warmup_ratio * N) (data_pipeline/trainer/trainers/sota_trainer.py:1814-1818).
    `create_scheduler(name, optimizer, ...)`, the order of data_pipeline/trainer/schedulers/sota_schedulers.py, is taken
    as well (a string or scheduler-type enum first)."""
    if isinstance(optimizer, str) or hasattr(optimizer, "value"):
        optimizer, scheduler_type = scheduler_type, optimizer
    name = getattr(scheduler_type, "value", scheduler_type).lower()
    if name not in _REGISTRY:
        raise ValueError(f"unknown scheduler {name!r}; choose from {sorted(_REGISTRY)}")
    if warmup_steps <= 0 and warmup_ratio > 0:
        warmup_steps = int(warmup_ratio * num_training_steps)
    cls = _REGISTRY[name]
    import inspect
    accepted = set(inspect.signature(cls.__init__).parameters) | set(inspect.signature(BaseScheduler.__init__).parameters)
    kw = {k: v for k, v in kw.items() if k in accepted}
    return cls(optimizer, num_training_steps=num_training_steps, warmup_steps=warmup_steps, min_lr_ratio=min_lr_ratio,
               **kw)


create_sota_scheduler = create_scheduler


OneCycleSchedulerEnhanced = OneCycleScheduler     # alias exported by data_pipeline/trainer/schedulers/__init__.py
