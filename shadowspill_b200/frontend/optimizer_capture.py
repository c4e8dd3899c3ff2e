"""Capture the update of any traceable ``torch.optim.Optimizer`` as a graph over flat tensors.

``capture_optimizer_update(lambda params: torch.optim.Adagrad(params, lr=1e-2))`` builds the
optimizer on one small parameter, lets it take a step so that its state exists, and then traces one
``optimizer.step()`` with ``make_fx``: the inputs are the parameter, its gradient, the optimizer's
per-parameter state tensors, the step counter and the learning rate (as tensors, so the graph holds
for every step and schedule); the outputs are the new parameter and the new state. Optimizers
update elementwise, so the graph, traced on eight elements, applies to a flat range of any length.
The planned executor runs it as its update rule: per parameter (or per owned shard under sharded
storage) on fp32 copies, results rounded into the stored dtypes. Up to two state tensors are
carried, in the two moment objects every trainable parameter already has.

The hyperparameters the optimizer was constructed with are constants of the graph, except ``lr``,
which follows the run's schedule. Not captured: optimizers that are not elementwise (LBFGS, Muon's
orthogonalisation), that keep more than two state tensors per parameter, or that need a closure.

Reference: packages/engine/src/shadowspill/pytorch/optimizer/trace.py:44
(``capture_optimizer_update``), packages/engine/src/shadowspill/build/optimizer.py:49
(``capture_update`` and the ``optimizer_group.N.*`` bindings).
"""
from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Callable

import torch
from torch import fx
from torch.fx.experimental.proxy_tensor import make_fx


class OptimizerNotCapturable(ValueError):
    pass


@contextlib.contextmanager
def _tracing_scope():
    """Optimizers relax their "capturable needs a CUDA tensor" assertion while a graph is being
    made (torch/optim/*.py test ``torch.compiler.is_compiling()``); capture is such a time."""
    import torch.compiler as tc
    before = tc._is_compiling_flag
    tc._is_compiling_flag = True
    try:
        yield
    finally:
        tc._is_compiling_flag = before


@dataclass
class CapturedUpdate:
    name: str
    factory: Callable[[list], torch.optim.Optimizer]
    state_names: tuple[str, ...]              # the optimizer's own names, in moment-object order
    defaults: dict = field(default_factory=dict)
    counts_steps: bool = True                 # the optimizer keeps a step counter in its state
    # True: step and learning rate are tensor inputs of one graph (the optimizer has a capturable
    # form). False: the optimizer reads them as Python numbers, so a graph holds for one
    # (step, learning rate) pair and is made again when they change: once per update, shared by
    # every parameter of that update.
    tensor_scalars: bool = True
    graph: fx.GraphModule | None = None
    _cache: dict = field(default_factory=dict, repr=False)

    def __str__(self) -> str:
        return f"captured:{self.name}"

    def graph_for(self, step: int, lr: float) -> fx.GraphModule:
        if self.tensor_scalars:
            return self.graph
        key = (int(step), float(lr))
        g = self._cache.get(key)
        if g is None:
            if len(self._cache) >= 8:
                self._cache.clear()
            g = self._cache[key] = _trace(self.factory, self.state_names, self.counts_steps, False,
                                          step=step, lr=lr)
        return g

    def apply(self, p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float,
              step: int, grad_scale: float = 1.0, **_unused) -> None:
        """One update in place. ``step`` is the 1-based number of this update."""
        dev = p.device
        states = [t.float() for t in (m, v)[:len(self.state_names)]]
        graph = self.graph_for(step, lr)
        if self.tensor_scalars:
            outs = graph(p.float(), g.float() * grad_scale, torch.tensor(float(step - 1), device=dev),
                         torch.tensor(float(lr), device=dev), *states)
        else:
            outs = graph(p.float(), g.float() * grad_scale, *states)
        p.copy_(outs[0].to(p.dtype))
        for dst, new in zip((m, v), outs[1:]):
            dst.copy_(new.to(dst.dtype))


def _trace(factory, tensor_names, counts, tensor_scalars: bool, step: int = 1, lr: float = 1e-3):
    """One ``optimizer.step()`` as a graph. With ``tensor_scalars`` the inputs are
    (p, g, step, lr, *states); otherwise (p, g, *states) for the given step and learning rate."""
    def run(p, g, step_value, lr_value, states):
        q = p.clone().requires_grad_(True)
        q.grad = g
        inner = _configured(factory([q]), tensor_scalars)
        st = {n: s.clone() for n, s in zip(tensor_names, states)}
        if counts:
            st["step"] = step_value
        inner.state[q] = st
        for group in inner.param_groups:
            group["lr"] = lr_value
        inner.step()
        return (q.detach(), *[inner.state[q][n] for n in tensor_names])
    zeros = [torch.zeros(8) for _ in tensor_names]
    with _tracing_scope():
        if tensor_scalars:
            return make_fx(lambda p, g, step_t, lr_t, *states: run(p, g, step_t.clone(), lr_t, states),
                           tracing_mode="real")(torch.zeros(8), torch.zeros(8), torch.tensor(1.0),
                                                torch.tensor(1e-3), *zeros)
        return make_fx(lambda p, g, *states: run(p, g, torch.tensor(float(step - 1)), float(lr), states),
                       tracing_mode="real")(torch.zeros(8), torch.zeros(8), *zeros)


def capture_optimizer_update(factory: Callable[[list], torch.optim.Optimizer], name: str | None = None
                             ) -> CapturedUpdate:
    probe = torch.nn.Parameter(torch.linspace(-1.0, 1.0, 8))
    probe.grad = torch.linspace(0.5, -0.5, 8)
    opt = _configured(factory([probe]), False)
    try:
        opt.step()                                          # creates the state
    except TypeError as exc:
        raise OptimizerNotCapturable(f"{type(opt).__name__}.step() needs arguments ({exc}); optimizers that "
                                     "re-evaluate the loss through a closure are not captured") from exc
    state = opt.state[probe]
    tensor_names = tuple(k for k, t in state.items() if torch.is_tensor(t) and t.shape == probe.shape)
    scalar_names = tuple(k for k, t in state.items() if k not in tensor_names)
    if len(tensor_names) > 2:
        raise OptimizerNotCapturable(f"{type(opt).__name__} keeps {len(tensor_names)} state tensors per "
                                     f"parameter ({tensor_names}); two moment objects are available")
    unknown = [k for k in scalar_names if k != "step"]
    if unknown:
        raise OptimizerNotCapturable(f"{type(opt).__name__} keeps per-parameter state {unknown} that is "
                                     "neither a tensor of the parameter's shape nor a step counter")
    counts = "step" in scalar_names
    defaults = {k: v for k, v in opt.param_groups[0].items() if k != "params" and not torch.is_tensor(v)}
    what = type(opt).__name__
    captured = None
    if "capturable" in opt.param_groups[0]:
        try:
            graph = _trace(factory, tensor_names, counts, True)
            captured = CapturedUpdate(name or what.lower(), factory, tensor_names, defaults, counts, True, graph)
        except Exception:  # noqa: BLE001  (falls back to the per-update form below)
            captured = None
    if captured is None:
        try:
            _trace(factory, tensor_names, counts, False)
        except Exception as exc:  # noqa: BLE001
            raise OptimizerNotCapturable(f"{what}.step() cannot be traced: {type(exc).__name__}: {exc}") from exc
        captured = CapturedUpdate(name or what.lower(), factory, tensor_names, defaults, counts, False)
    _check_elementwise(captured.graph_for(1, 1e-3), what)
    _verify(captured)          # the trace must reproduce the optimizer on other data
    return captured


def _configured(opt: torch.optim.Optimizer, capturable: bool = True) -> torch.optim.Optimizer:
    """Single-tensor form; with ``capturable`` the step counter and learning rate may be tensors."""
    for group in opt.param_groups:
        if "foreach" in group:
            group["foreach"] = False
        if "fused" in group:
            group["fused"] = False
        if "capturable" in group:
            group["capturable"] = bool(capturable)
    return opt


_SHAPE_BOUND = ("aten.view", "aten.reshape", "aten.expand", "aten.zeros.", "aten.ones.", "aten.full.",
                "aten.empty.", "aten.sum", "aten.mean", "aten.norm", "aten.linalg", "aten.mm", "aten.matmul")


def _check_elementwise(graph: fx.GraphModule, what: str) -> None:
    for n in graph.graph.nodes:
        if n.op == "call_function" and any(str(n.target).startswith(s) for s in _SHAPE_BOUND):
            raise OptimizerNotCapturable(f"{what}: the update uses {n.target}, which ties the graph to the "
                                         "probe's shape or mixes elements; only elementwise updates are captured")


def _verify(captured: CapturedUpdate) -> None:
    gen = torch.Generator().manual_seed(0)
    p = torch.nn.Parameter(torch.randn(37, generator=gen))
    opt = _configured(captured.factory([p]), False)
    m, v = torch.zeros(37), torch.zeros(37)
    mine = p.detach().clone()
    for k in range(3):
        g = torch.randn(37, generator=gen)
        p.grad = g.clone()
        opt.step()
        captured.apply(mine, g, m, v, lr=float(opt.param_groups[0]["lr"]), step=k + 1)
        if not torch.allclose(mine, p.detach(), rtol=1e-5, atol=1e-6):
            raise OptimizerNotCapturable(
                f"the captured graph of {type(opt).__name__} does not reproduce its step {k + 1} (largest "
                f"difference {float((mine - p.detach()).abs().max()):.3g}): its first step may depend on state "
                "that starts at zero here")
