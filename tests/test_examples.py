"""The example scripts run as written (CPU paths)."""
import importlib.util
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _load(name):
    spec = importlib.util.spec_from_file_location(name, ROOT / "examples" / f"{name}.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_train_budgeted_example(tmp_path):
    loss = _load("train_budgeted").main(["--steps", "2", "--out", str(tmp_path)])
    assert loss > 0
    assert (tmp_path / "index.html").exists() and (tmp_path / "runtime.html").exists()


def test_train_budgeted_example_with_a_file_spill_pool(tmp_path):
    plain = _load("train_budgeted").main(["--steps", "2"])
    filed = _load("train_budgeted").main(["--steps", "2", "--spill-pool", "file", "--spill-dir", str(tmp_path)])
    assert filed == plain


def test_service_quickstart_example():
    losses = _load("service_quickstart").main()
    assert len(losses) == 4 and losses[-1] < losses[0]


def test_regression_example():
    losses = _load("regression_training").main(["--steps", "8"])
    assert len(losses) == 8 and losses[-1] < losses[0]


def test_regression_example_on_two_ranks():
    losses = _load("regression_training").main(["--steps", "6", "--ranks", "2"])
    assert len(losses) == 6 and losses[-1] < losses[0]


def test_policy_example():
    history = _load("policy_training").main(["--iterations", "2"])
    assert len(history) == 4
    # with old log-probabilities taken from the current weights the first surrogate of every
    # iteration is -mean(advantage) over response tokens = 0 up to rounding; steps lower it
    assert abs(history[0]) < 1e-4 and abs(history[2]) < 1e-4
    assert history[1] < history[0] and history[3] < history[2]


def test_offline_sweep_example(tmp_path):
    """Planning inputs exported from a prepared session are planned again, elsewhere, for other
    budgets and link rates; every feasible cell gets its plan report."""
    mod = _load("offline_sweep")
    exported = tmp_path / "measurements.zip"
    mod.main(["--export", str(exported)])
    sweep = mod.main([str(exported), "--output", str(tmp_path / "sweep.html"), "--device-gib", "0.2", "0.53", "1.0",
                      "--transfer-scale", "0.5", "2"])
    rows = sweep.table()
    assert len(rows) == 6 and sum(r["feasible"] for r in rows) >= 4
    fits = [r for r in rows if r["feasible"]]
    # a faster link never makes the same budget slower; more memory never makes the same link slower
    by = {(r["device_gib"], r["transfer_scale"]): r["seconds"] for r in fits}
    for (d, x), s in by.items():
        if (d, 2.0) in by and x == 0.5:
            assert by[(d, 2.0)] <= s + 1e-9
    page = (tmp_path / "sweep.html").read_text()
    assert page.count("<tr>") == 7 and "plan</a>" in page
    linked = next((tmp_path / "sweep").iterdir())
    assert (linked / "index.html").exists() and (linked / "tasks.csv").exists()


def test_saved_plan_example():
    out = _load("saved_plan").main(steps=2)
    assert out["skipped_preparation"] and len(out["losses"]) == 2 and out["prepared_seconds"] > 0


def test_lora_long_context_example():
    losses = _load("lora_long_context").main(["--steps", "3"])
    assert len(losses) == 3 and losses[-1] < losses[0]
