"""Whole-model-on-device trainer: the degenerate plan in which nothing spills.

It runs the same stage functions, gradient creation/accumulation rules and fused
AdamW as the planned executor, with every tensor resident. It is the numerical
twin used by tests (planned execution must reproduce it bit for bit on the same
device, because the kernels and their order are identical) and the smallest
end-to-end path of the package.
"""
from __future__ import annotations

import torch

from ..models.config import DecoderConfig
from ..models.decoder import BatchMeta, HeadLossStage, build_stages
from ..ops import functional as F


class ResidentTrainer:
    def __init__(self, cfg: DecoderConfig, device: str | torch.device = "cuda",
                 dtype: torch.dtype = torch.bfloat16, seed: int = 0,
                 grad_dtype: torch.dtype | None = None, lr: float = 1e-3, beta1: float = 0.9,
                 beta2: float = 0.95, eps: float = 1e-8, weight_decay: float = 0.0,
                 stochastic_rounding: bool = True, objective=None, lora=None, rule: str = "adamw"):
        self.cfg = cfg
        self.rule = rule
        self.device = torch.device(device)
        self.dtype = dtype
        self.grad_dtype = grad_dtype or dtype
        self.hyper = dict(lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay)
        self.sr = stochastic_rounding and dtype == torch.bfloat16
        self.seed = seed
        self.stages = build_stages(cfg, objective, lora)
        self.step_count = 0
        self.P, self.G, self.M, self.V = [], [], [], []
        self._flat = []
        gen = torch.Generator().manual_seed(seed)
        for st in self.stages:
            _, pbytes = st.layout(dtype)
            _, gbytes = st.layout(self.grad_dtype, torch.float32, trainable_only=True)
            _, obytes = st.layout(dtype, trainable_only=True)
            host = torch.zeros(pbytes, dtype=torch.uint8)
            st.init_(st.views(host, dtype), gen)
            pf = host.to(self.device)
            gf = torch.zeros(gbytes, dtype=torch.uint8, device=self.device)
            mf = torch.zeros(obytes, dtype=torch.uint8, device=self.device)
            vf = torch.zeros(obytes, dtype=torch.uint8, device=self.device)
            self._flat.append((pf, gf, mf, vf))
            self.P.append(st.views(pf, dtype))
            self.G.append(st.views(gf, self.grad_dtype, torch.float32, True))
            self.M.append(st.views(mf, dtype, trainable_only=True))
            self.V.append(st.views(vf, dtype, trainable_only=True))
        self.loss_sum = torch.zeros(1, dtype=torch.float32, device=self.device)
        self._accum = 0

    # ------------------------------------------------------------------ passes
    def forward_backward(self, meta: BatchMeta, train: bool = True) -> None:
        """One microbatch; gradients are created by the first microbatch after an
        optimizer step and accumulated by the following ones."""
        first = self._accum == 0
        xs = [None]
        x = None
        body = self.stages[:-1]
        for i, st in enumerate(body):
            x, _ = st.forward(self.P[i], x, meta, ())
            xs.append(x)
        head: HeadLossStage = self.stages[-1]
        tied = ({"params": self.P[0], "grads": self.G[0] if train else None, "first": first}
                if self.cfg.tied_embeddings else None)
        dx = head.loss_and_backward(self.P[-1], self.G[-1], x, meta, self.loss_sum, first,
                                    train=train, tied=tied)
        if not train:
            return
        for i in range(len(body) - 1, -1, -1):
            st = body[i]
            if i == 0 and not st.has_trainable:
                break
            # with tied embeddings the head has already started the embedding's gradient
            create = first and not (i == 0 and self.cfg.tied_embeddings)
            dx = st.backward(self.P[i], self.G[i], xs[i], dx, meta, {}, create)
        self._accum += 1

    def optim_step(self, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        offset = 0
        for si, st in enumerate(self.stages):
            for p in st.params:
                if not p.trainable:
                    offset += (p.numel + 7) // 8 * 8
                    continue
                pt, gt = self.P[si][p.name], self.G[si][p.name]
                if self.rule != "adamw":
                    from ..ops import reference
                    reference.update_rule_(self.rule, pt.view(-1), gt.view(-1), self.M[si][p.name].view(-1),
                                           self.V[si][p.name].view(-1), step=self.step_count,
                                           grad_scale=grad_scale, **self.hyper)
                    offset += (p.numel + 7) // 8 * 8
                    continue
                F.adamw_(pt.view(-1), gt.view(-1), self.M[si][p.name].view(-1),
                         self.V[si][p.name].view(-1), step=self.step_count,
                         grad_scale=grad_scale, seed=self.seed, offset=offset,
                         stochastic_param=self.sr, stochastic_state=self.sr, **self.hyper)
                offset += (p.numel + 7) // 8 * 8
        self._accum = 0

    def step(self, microbatches: list[BatchMeta]) -> float:
        self.loss_sum.zero_()
        for mb in microbatches:
            self.forward_backward(mb)
        self.optim_step()
        return float(self.loss_sum.item())

    def evaluate(self, microbatches: list[BatchMeta]) -> float:
        self.loss_sum.zero_()
        for mb in microbatches:
            self.forward_backward(mb, train=False)
        return float(self.loss_sum.item())

    def state_dict(self) -> dict[str, torch.Tensor]:
        out = {}
        for si, st in enumerate(self.stages):
            for p in st.params:
                out[f"{st.name}.{p.name}"] = self.P[si][p.name]
        return out
