"""Client-side packing strategies, atomic groups, the coverage bound and the command table."""
import concurrent.futures as cf
import io
import random
from types import SimpleNamespace

import numpy as np
import pytest

from shadowspill_b200.client import (BatchError, BatchStatistics, CommandTable, CoverageBound, LengthStatistics,
                                     assign_bins, pack_batch, text_batch, text_batch_statistics)


def test_strategies_run_in_order_and_say_which_one_worked():
    # tightest-fit strands the last 3 (bins 12/12 -> 6+5 | 4+3+3 leaves 3 homeless); spreading fits
    found = assign_bins([6, 5, 4, 3, 3, 3], 12, 2, 8)
    assert found.strategy == "balanced" and sorted(i for b in found.bins for i in b) == list(range(6))
    assert all(sum([6, 5, 4, 3, 3, 3][i] for i in b) <= 12 for b in found.bins)
    assert assign_bins([7, 6, 5, 4, 4, 3, 3], 16, 2, 8).strategy == "best_fit"
    # four sequence slots per microbatch as well: whichever strategy answers, both limits hold
    lengths = [7, 6, 5, 4, 4, 3, 3]
    exact = assign_bins(lengths, 16, 2, 4)
    assert sorted(i for b in exact.bins for i in b) == list(range(7))
    assert all(sum(lengths[i] for i in b) <= 16 and len(b) <= 4 for b in exact.bins)
    with pytest.raises(BatchError, match="repair spent"):
        assign_bins([9, 9, 9], 16, 2, 8)
    with pytest.raises(BatchError, match="unknown packing policy"):
        assign_bins([1], 4, 1, 1, policy="random")


def test_repair_finds_what_both_greedy_passes_miss():
    rng = random.Random(3)
    seen = 0
    for _ in range(3000):
        cap, bins, seqs = rng.choice([20, 30]), rng.randint(2, 3), rng.randint(2, 5)
        lengths = [rng.randint(1, cap // 2) for _ in range(rng.randint(4, 9))]
        try:
            found = assign_bins(lengths, cap, bins, seqs)
        except BatchError:
            continue
        assert sorted(i for b in found.bins for i in b) == list(range(len(lengths)))
        assert all(sum(lengths[i] for i in b) <= cap and len(b) <= seqs for b in found.bins)
        seen += found.strategy == "repair"
    assert seen > 0


def test_atomic_groups_share_a_microbatch():
    found = assign_bins([3, 3, 2, 2], 6, 2, 8, groups=[[0, 2], [1], [3]])
    assert any({0, 2} <= set(b) for b in found.bins)
    with pytest.raises(BatchError, match="exactly once"):
        assign_bins([3, 3], 6, 2, 8, groups=[[0], [0, 1]])
    with pytest.raises(BatchError, match="needs 8 tokens"):
        assign_bins([4, 4], 6, 2, 8, groups=[[0, 1]])
    datums = text_batch([np.arange(40) % 50, np.arange(30) % 50, np.arange(20) % 50])
    placement: list = []
    mbs = pack_batch(datums, microbatch_tokens=64, microbatches=2, slots=8, placement=placement, groups=[[1, 2], [0]])
    assert placement[1][0] == placement[2][0] != placement[0][0] and len(mbs) == 2


def test_the_coverage_bound_never_admits_a_batch_that_a_greedy_pass_cannot_pack():
    rng = random.Random(0)
    admitted = 0
    for _ in range(6000):
        cap, bins, seqs = rng.choice([16, 32, 64]), rng.randint(1, 4), rng.randint(1, 6)
        lengths = [rng.randint(1, cap) for _ in range(rng.randint(1, 12))]
        if CoverageBound(cap, bins, seqs).admits(lengths):
            admitted += 1
            for policy in ("best_fit", "balanced"):
                assign_bins(lengths, cap, bins, seqs, policy=policy)       # raises if the bound lied
    assert admitted > 500
    assert not CoverageBound(16, 2, 4).admits([17]) and not CoverageBound(16, 2, 4).admits([])


def test_length_statistics_and_the_command_table():
    stats = LengthStatistics.from_lengths([345, 3507, 1126, 1013])
    assert (stats.count, stats.total, stats.minimum, stats.maximum) == (4, 5991, 345, 3507)
    assert stats.summary() == "345/3,507 1,498/1,070"
    with pytest.raises(ValueError):
        LengthStatistics.from_lengths([])
    with pytest.raises(ValueError):
        LengthStatistics.from_lengths([3, -1])
    with pytest.raises(ValueError, match="fit inside"):
        BatchStatistics.from_lengths([4, 5], supervised=[5, 5])
    datums = text_batch([np.arange(12) % 7, np.arange(30) % 7])
    both = text_batch_statistics(datums)
    assert both.lengths.total == sum(len(d) for d in datums) and both.supervised.total <= both.lengths.total

    out = io.StringIO()
    table = CommandTable(stream=out)
    ok, bad = cf.Future(), cf.Future()
    assert table.track("step", ok, batch=both, planned_seconds=0.5) is ok
    table.track("optim_step", bad)
    ok.set_result(SimpleNamespace(loss=2.5, execution_seconds=0.25, completed_updates=1))
    bad.set_exception(RuntimeError("worker lost"))
    text = out.getvalue().splitlines()
    assert text[0].startswith("Client clock:") and "Tokens/s" in text[1]
    rows = [ln for ln in text if "step()" in ln]
    assert len(rows) == 4 and "pending" in rows[0] and " done " in rows[2] and "failed" in rows[3]
    assert f"{both.lengths.total / 0.25:,.0f}" in rows[2] and "2.5000" in rows[2] and "0.50s" in rows[2]
    with pytest.raises(ValueError):
        table.track("save", cf.Future())
    with pytest.raises(ValueError):
        table.track("optim_step", cf.Future(), batch=both)
    with pytest.raises(ValueError):
        table.track("step", cf.Future(), planned_seconds=-1)

    class Broken(io.StringIO):
        def write(self, _):
            raise OSError("closed pipe")
    silent = CommandTable(stream=Broken())
    fut = cf.Future()
    silent.track("forward", fut)
    fut.set_result(SimpleNamespace(loss=1.0, execution_seconds=1.0))
    assert isinstance(silent.error, OSError) and fut.result().loss == 1.0     # the call is untouched
