"""The small non-text family: ``Linear(16, 32) -> SiLU -> Linear(32, 8)`` in fp32 with a
weighted squared-error objective.

It exists to show that nothing in capture, planning, the runtime or the service is tied
to token sequences: a "microbatch" is ``T`` sample rows, the model input ``value`` and the
regression ``target_values`` travel as wide per-row batch fields, and the two linear maps
are the two stages of the program (there are no layers in between). The reference keeps
the same model for the same purpose
(packages/workloads/src/shadowspill_workloads/models/regression/model.py:8-16; objective
``weighted_squared_error``, models/regression/training.py:58-70: the loss is
``sum_i weights_i * ||prediction_i - targets_i||^2`` over valid rows).

The architecture record is a ``DecoderConfig`` of family ``regression`` whose fields are
read as: ``d_ff`` = input width, ``d_model`` = hidden width, ``vocab_size`` = output width.
"""
from __future__ import annotations

import torch

from .config import DecoderConfig
from .decoder import BatchMeta, ParamSpec, Stage

INPUT_FIELD = "value"
TARGET_FIELD = "target_values"


def regression_config(inputs: int = 16, hidden: int = 32, outputs: int = 8) -> DecoderConfig:
    return DecoderConfig("regression", 0, hidden, 1, 1, 1, inputs, outputs, initializer_range=0.25)


def batch_fields(cfg: DecoderConfig) -> tuple[str, ...]:
    """Wide batch fields (``name:width``) a regression run carries per row."""
    return (f"{INPUT_FIELD}:{cfg.d_ff}", f"{TARGET_FIELD}:{cfg.vocab_size}")


class RegressionInputStage(Stage):
    """``y = silu(value @ W1^T + b1)``; nothing is saved, the backward recomputes."""
    kind = "layer"

    def __init__(self, name: str, cfg: DecoderConfig):
        super().__init__(name, cfg)
        std = cfg.d_ff ** -0.5
        self.params = [ParamSpec("w1", (cfg.d_model, cfg.d_ff), std=std),
                       ParamSpec("b1", (cfg.d_model,), init="zeros")]

    def _pre(self, P, meta: BatchMeta) -> torch.Tensor:
        value = meta.extras[INPUT_FIELD].to(P["w1"].dtype)
        return torch.addmm(P["b1"], value, P["w1"].t())

    def forward(self, P, x, meta: BatchMeta, keep=None, out=None, saved_out=None):
        y = torch.nn.functional.silu(self._pre(P, meta))
        if out is not None:
            out.copy_(y)
            y = out
        return y, {}

    def backward(self, P, G, x, dy, meta: BatchMeta, saved, first: bool):
        pre = self._pre(P, meta)
        s = torch.sigmoid(pre)
        dpre = dy.to(pre.dtype) * (s * (1.0 + pre * (1.0 - s)))
        value = meta.extras[INPUT_FIELD].to(pre.dtype)
        gw, gb = dpre.t() @ value, dpre.sum(0)
        if first:
            G["w1"].copy_(gw); G["b1"].copy_(gb)
        else:
            G["w1"].add_(gw); G["b1"].add_(gb)
        return None

    def workspace_bytes(self, T: int, itemsize: int = 4) -> int:
        return 6 * T * self.cfg.d_model * 4 + (1 << 16)

    def flops(self, T: int, mean_seqlen: float) -> float:
        return 2.0 * T * self.cfg.d_ff * self.cfg.d_model


class RegressionHeadStage(Stage):
    """``prediction = x @ W2^T + b2`` and the weighted squared error against ``target_values``.
    Rows with weight zero are padding and contribute nothing."""
    kind = "head"

    def __init__(self, name: str, cfg: DecoderConfig):
        super().__init__(name, cfg)
        std = cfg.d_model ** -0.5
        self.params = [ParamSpec("w2", (cfg.vocab_size, cfg.d_model), std=std),
                       ParamSpec("b2", (cfg.vocab_size,), init="zeros")]

    @property
    def output_width(self) -> int:
        return self.cfg.vocab_size        # a forward-only program returns every row's prediction

    def predict(self, P, x) -> torch.Tensor:
        return torch.addmm(P["b2"], x.to(P["w2"].dtype), P["w2"].t())

    def outputs(self, P, x, meta: BatchMeta, tied=None) -> torch.Tensor:
        return self.predict(P, x)

    def loss_and_backward(self, P, G, x, meta: BatchMeta, loss_sum: torch.Tensor, first: bool,
                          dx=None, train: bool = True, grad_scale: float = 1.0, tied=None):
        pred = self.predict(P, x)
        w = meta.weights.to(pred.dtype)
        valid = (w > 0).unsqueeze(1)
        diff = torch.where(valid, pred - meta.extras[TARGET_FIELD].to(pred.dtype), torch.zeros_like(pred))
        loss_sum += (diff.square().sum(1) * w).sum().float()
        if not train:
            return None
        dpred = 2.0 * grad_scale * diff * w.unsqueeze(1)
        if G:
            gw, gb = dpred.t() @ x.to(pred.dtype), dpred.sum(0)
            if first:
                G["w2"].copy_(gw); G["b2"].copy_(gb)
            else:
                G["w2"].add_(gw); G["b2"].add_(gb)
        out = dpred @ P["w2"]
        if dx is not None:
            dx.copy_(out)
            out = dx
        return out

    def workspace_bytes(self, T: int, itemsize: int = 4) -> int:
        return 6 * T * max(self.cfg.d_model, self.cfg.vocab_size) * 4 + (1 << 16)

    def flops(self, T: int, mean_seqlen: float) -> float:
        return 2.0 * T * self.cfg.d_model * self.cfg.vocab_size


def build_regression_stages(cfg: DecoderConfig) -> list[Stage]:
    return [RegressionInputStage("input", cfg), RegressionHeadStage("head", cfg)]


def reference_module(cfg: DecoderConfig) -> torch.nn.Module:
    """The same network as a plain ``torch.nn`` module (tests compare against it)."""
    return torch.nn.Sequential(torch.nn.Linear(cfg.d_ff, cfg.d_model), torch.nn.SiLU(),
                               torch.nn.Linear(cfg.d_model, cfg.vocab_size))
