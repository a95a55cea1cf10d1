"""`backward` for modules whose gradient normally comes from autograd.

The reference writes several of its fused blocks (LoRA MLP / QKV, cross-entropy, vocabulary-parallel cross-entropy) as
`torch.autograd.Function`s with hand-written `backward` statics (data_pipeline/trainer/kernels/fast_lora_mlp.py,
triton_kernels.py:330, distributed/tensor_parallel.py).  Here those blocks are `nn.Module`s over differentiable framework
ops, so autograd supplies the backward pass.  For callers that drive gradients by hand (custom pipeline schedules,
gradient checks) this mixin offers the explicit form.
"""
from __future__ import annotations

import torch


class ExplicitBackward:
    def backward(self, *inputs, grad_output: torch.Tensor | None = None, accumulate: bool = False):
        """Gradients of `self(*inputs)`.  Floating-point tensor inputs are treated as leaves.  `grad_output` defaults to
        ones (a scalar output needs none).  Returns (one gradient or None per input, {parameter name: gradient}) for the
        parameters that require gradients; with `accumulate=True` the parameter gradients are also added to `.grad`."""
        leaves = [a.detach().requires_grad_(True) if torch.is_tensor(a) and a.is_floating_point() else a for a in inputs]
        with torch.enable_grad():
            out = self(*leaves)
        out = out[0] if isinstance(out, (tuple, list)) else out
        params = {n: p for n, p in self.named_parameters() if p.requires_grad}
        wanted = [a for a in leaves if torch.is_tensor(a) and a.requires_grad] + list(params.values())
        go = grad_output if grad_output is not None else torch.ones_like(out)
        grads = list(torch.autograd.grad(out, wanted, go, allow_unused=True)) if wanted else []
        it = iter(grads)
        in_grads = tuple(next(it) if torch.is_tensor(a) and a.requires_grad else None for a in leaves)
        p_grads = {n: g for n, g in zip(params, it)}
        if accumulate:
            for n, g in p_grads.items():
                if g is not None:
                    p = params[n]
                    p.grad = g if p.grad is None else p.grad + g
        return in_grads, p_grads
