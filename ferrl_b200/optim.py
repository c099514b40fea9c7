"""AdamW over the trainable adapter tensors.

Update rule (reference ``crates/ferrl/src/optim.rs:257-296``): decoupled weight
decay, epsilon added outside the square root, bias correction by step count::

    m <- b1 m + (1-b1) g;  v <- b2 v + (1-b2) g^2
    p <- p (1 - lr*wd) - lr * (m / (1-b1^t)) / (sqrt(v / (1-b2^t)) + eps)

``state()`` / ``load_state()`` export and restore the moments and the step
counter for checkpoints (``optim.rs:146-224``).

On GPUs ``step`` is one multi-tensor kernel launch over all adapters; in a
data-parallel run ``FusedDpStep`` (``ferrl_b200.parallel.dp``) goes further and
folds the gradient all-reduce over NVLink peer memory, the 1/(accum*world)
scale, the global-norm clip and this update into the same pass.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from . import ops


@dataclass
class AdamWParams:
    lr: float = 1e-3
    beta1: float = 0.9
    beta2: float = 0.999
    eps: float = 1e-8
    weight_decay: float = 0.0


@dataclass
class OptimizerState:
    step: int
    m: list
    v: list


def beta_to_step(beta: float, step: int) -> float:
    return beta ** step


class FerrlAdamW:
    def __init__(self, params: Sequence[torch.nn.Parameter], hp: Optional[AdamWParams] = None):
        self.params = list(params)
        for p in self.params:
            if p.dtype not in (torch.float32, torch.float64):
                raise ValueError("trainable tensors must be float32/float64 masters")
        self.hp = hp or AdamWParams()
        self.m = [torch.zeros_like(p, memory_format=torch.contiguous_format) for p in self.params]
        self.v = [torch.zeros_like(p, memory_format=torch.contiguous_format) for p in self.params]
        self.step_t = 0

    def set_learning_rate(self, lr: float):
        self.hp.lr = lr

    @torch.no_grad()
    def step(self, grads: Sequence[Optional[torch.Tensor]], grad_scale: float = 1.0):
        """Apply one update. ``grads[i]`` of ``None`` leaves tensor ``i`` untouched."""
        if len(grads) != len(self.params):
            raise ValueError("gradient list does not match the parameter list")
        self.step_t += 1
        idx = [i for i, g in enumerate(grads) if g is not None]
        ops.adamw_step([self.params[i].data for i in idx], [grads[i] for i in idx],
                       [self.m[i] for i in idx], [self.v[i] for i in idx],
                       lr=self.hp.lr, beta1=self.hp.beta1, beta2=self.hp.beta2, eps=self.hp.eps,
                       weight_decay=self.hp.weight_decay, step=self.step_t, grad_scale=grad_scale)

    def state(self) -> OptimizerState:
        return OptimizerState(self.step_t, [t.detach().clone() for t in self.m],
                              [t.detach().clone() for t in self.v])

    @torch.no_grad()
    def load_state(self, st: OptimizerState):
        if len(st.m) != len(self.params) or len(st.v) != len(self.params):
            raise ValueError("optimizer state has a different number of tensors")
        for p, m, v in zip(self.params, st.m, st.v):
            if tuple(m.shape) != tuple(p.shape) or tuple(v.shape) != tuple(p.shape):
                raise ValueError("optimizer state shape mismatch")
        if st.step < 0:
            raise ValueError("optimizer step counter must be >= 0")
        for dst, src in zip(self.m, st.m):
            dst.copy_(src)
        for dst, src in zip(self.v, st.v):
            dst.copy_(src)
        self.step_t = int(st.step)

    def schema(self) -> list:
        return [(tuple(p.shape), str(p.dtype)) for p in self.params]
