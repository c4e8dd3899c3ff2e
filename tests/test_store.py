"""Content-addressed store: addressing, modes, atomic writes."""
from shadowspill_b200.store import ContentStore, StoreMode


def test_round_trip_and_modes(tmp_path):
    s = ContentStore(tmp_path)
    key = {"device": "B200", "task": "llama3:layer:fwd:T8192", "kernels": "abc"}
    assert s.get("task_profile", key) is None and s.misses == 1
    assert s.put("task_profile", key, {"seconds": 0.004, "workspace_bytes": 123})
    assert s.get("task_profile", key) == {"seconds": 0.004, "workspace_bytes": 123}
    assert s.get("task_profile", {**key, "kernels": "other"}) is None      # another library: another entry
    assert s.get("calibration", key) is None                                # kinds do not mix
    ro = ContentStore(tmp_path, StoreMode.READ)
    assert ro.get("task_profile", key) is not None and not ro.put("task_profile", key, {})
    fresh = ContentStore(tmp_path, "refresh")
    assert fresh.get("task_profile", key) is None and fresh.put("task_profile", key, {"seconds": 1.0})
    assert s.get("task_profile", key) == {"seconds": 1.0}
    assert ContentStore(tmp_path, "off").get("task_profile", key) is None
    assert not list(tmp_path.rglob("*.tmp"))


def test_damaged_entry_reads_as_absent(tmp_path):
    s = ContentStore(tmp_path)
    s.put("k", {"a": 1}, [1, 2, 3])
    path = next(tmp_path.rglob("*.json"))
    path.write_text("{not json")
    assert s.get("k", {"a": 1}) is None
