"""The runtime's threads under ThreadSanitizer, and the filter that reads its reports."""
import pytest

from shadowspill_b200.qualification import races

FOREIGN = """WARNING: ThreadSanitizer: data race (pid=1)
  Write of size 8 at 0x7b0400000000 by thread T9:
    #0 c10::SmallVectorImpl<long>::operator= <null> (libtorch_cpu.so+0x1a1e83a)
    #1 gomp_thread_start <null> (libgomp.so.1+0x1baf2)

  Previous read of size 8 at 0x7b0400000000 by main thread:
    #0 at::TensorIteratorBase::reorder_dimensions() <null> (libtorch_cpu.so+0x1a20585)
    #1 wait_flag shadowspill_b200/csrc/src/runtime.cpp:385 (libss_core.so+0x352e6)

SUMMARY: ThreadSanitizer: data race (libtorch_cpu.so+0x1a1e83a)
"""
OURS = """WARNING: ThreadSanitizer: data race (pid=1)
  Write of size 4 at 0x7b0400000010 by thread T3:
    #0 ssc::StagedLane::pump() shadowspill_b200/csrc/src/staged_lane.cpp:201 (libss_core.so+0x4100)
    #1 worker_main shadowspill_b200/csrc/src/runtime.cpp:360 (libss_core.so+0x3000)

  Previous read of size 4 at 0x7b0400000010 by thread T5:
    #0 ssc::StagedLane::disk_main() shadowspill_b200/csrc/src/staged_lane.cpp:158 (libss_core.so+0x4000)

SUMMARY: ThreadSanitizer: data race staged_lane.cpp:201
"""


def test_only_reports_with_a_racing_access_in_the_core_count():
    assert races.core_reports(FOREIGN) == []          # a core frame deeper in the stack is not a racing access
    got = races.core_reports(FOREIGN + OURS + FOREIGN)
    assert len(got) == 1 and "StagedLane::pump" in got[0]
    assert races.core_reports("") == []


def test_runtime_threads_are_race_free_under_thread_sanitizer():
    res = races.run()
    if not res["available"]:
        pytest.skip(res["reason"])
    assert res["workload_ok"], res["stderr_tail"]
    assert res["core_reports"] == [], res["core_reports"][0][:3000]
