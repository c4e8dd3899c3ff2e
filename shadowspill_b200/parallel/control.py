"""Host-side agreement between ranks before they enter ordered collectives.

A rank that fails on the host (a batch that does not fit the plan, an exception while staging
inputs, a different operation selected) must not leave its peers waiting inside a collective
for a kernel that never comes. ``coordinated`` runs the host-side preparation of an invocation
on every rank, then exchanges the outcomes over a CPU (gloo) group: if any rank failed, every
rank raises, and none launches. ``check_invocation`` makes sure the ranks chose the same
operation and accumulation mode.

Reference: packages/engine/src/shadowspill/execution/distributed/checks.py:11-41 (``coordinated``,
``check_invocation``); the control group is gloo there too
(packages/engine/src/shadowspill/communication/binding/groups.py:38).
"""
from __future__ import annotations

from datetime import timedelta
from typing import Callable, TypeVar

import torch.distributed as dist

T = TypeVar("T")
_control = None


class CoordinatedFailure(RuntimeError):
    """Raised on EVERY rank when the host-side step of at least one rank failed."""

    def __init__(self, failures: dict[int, str]):
        self.failures = dict(failures)
        first = min(failures)
        more = f" (and {len(failures) - 1} more ranks)" if len(failures) > 1 else ""
        super().__init__(f"rank {first} failed before the collectives{more}: {failures[first]}")


def control_group(timeout_seconds: float = 120.0):
    """The CPU group used for agreement (created once; the default group when that is gloo)."""
    global _control
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    if _control is None:
        if dist.get_backend() == "gloo":
            _control = dist.group.WORLD
        else:
            _control = dist.new_group(backend="gloo", timeout=timedelta(seconds=timeout_seconds))
    return _control


def gather(value, group=None) -> list:
    """``value`` of every rank, in rank order (host objects, CPU group)."""
    group = group if group is not None else control_group()
    if group is None:
        return [value]
    out: list = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, value, group=group)
    return out


def coordinated(function: Callable[[], T], group=None) -> T:
    """Runs ``function`` (host-side work only), then agrees with the other ranks on the outcome.
    Returns its result when every rank succeeded; raises ``CoordinatedFailure`` on every rank
    when any rank raised."""
    group = group if group is not None else control_group()
    if group is None:
        return function()
    result, failure = None, None
    try:
        result = function()
    except Exception as error:  # noqa: BLE001  (reported to the peers, re-raised below)
        failure = error
    outcomes = gather(None if failure is None else f"{type(failure).__name__}: {failure}", group)
    failures = {r: msg for r, msg in enumerate(outcomes) if msg is not None}
    if failures:
        raise CoordinatedFailure(failures) from failure
    return result


def check_invocation(operation: str, accumulated: int, extra=None, group=None) -> None:
    """Every rank must be about to run the same operation in the same accumulation state."""
    choice = (operation, int(accumulated), extra)
    choices = gather(choice, group)
    if any(c != choice for c in choices):
        raise ValueError(f"ranks selected different operations or accumulation states: {choices}")
