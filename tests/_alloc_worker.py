"""Child process of the allocation-adapter GPU test: a FRESH process, because the adapter has to
become the CUDA allocator before anything allocates."""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch

from shadowspill_b200.runtime import allocator as al


def main():
    mode = sys.argv[1]
    adapter = al.install()
    assert al.installed() is adapter
    from shadowspill_b200.data.synthetic import make_batch
    from shadowspill_b200.models.config import DecoderConfig
    from shadowspill_b200.training.session import TrainingSession, TrainingSetup
    cfg = DecoderConfig("llama3", 2, 512, 4, 2, 128, 1024, 4096)
    setup = TrainingSetup(model=cfg, device_gib=1.0, spill_gib=0.5, tokens_per_step=2048, microbatch_tokens=1024,
                          lr=1e-3, calibrate=False, calibrate_overlap=False, allocator="planned",
                          frontend="graph" if mode == "graph" else "stages",
                          candidate_selections=("0:save_attention",))
    session = TrainingSession(setup)
    ex = session.executor
    assert ex.allocator is adapter and ex.workspace_bytes > 0
    contracts = [t for t in ex.program.tasks if t.allocations]
    assert contracts, "profiling recorded no allocation contracts"
    batch = make_batch(0, vocab=cfg.vocab_size, tokens_per_step=2048, microbatch_tokens=1024, median=200,
                       min_len=16, max_len=1024, slots=session.slots)
    if mode in ("run", "graph"):
        losses = [session.step(batch).loss]            # the first step warms what lives outside tasks
        before = adapter.stats()
        losses += [session.step(batch).loss for _ in range(2)]
        after = adapter.stats()
        assert losses[-1] < losses[0], losses
        assert after["slice_allocations"] > before["slice_allocations"]        # tasks used the slice
        assert after["driver_allocations"] == before["driver_allocations"]     # and nothing else, once warm
        assert 0 < after["peak"] <= ex.workspace_bytes
        print(f"OK ran: {after['slice_allocations']} slice allocations, peak {after['peak']} of {ex.workspace_bytes}")
    elif mode == "violate":
        victim = next(t for t in ex.program.tasks if t.kind == "backward" and t.allocations)
        victim.allocations = victim.allocations[:-1] + [victim.allocations[-1] + 512]
        try:
            session.step(batch)
        except al.AllocationContractViolation as exc:
            assert victim.name in str(exc), exc
            print(f"OK violation: {exc}")
        else:
            raise SystemExit("the changed contract went unnoticed")
    elif mode == "oom":
        adapter.configure(ex.rt.device_base + ex.planned_device_bytes, 1 << 20, ex.stream.cuda_stream)
        try:
            session.step(batch)
        except torch.OutOfMemoryError as exc:
            assert "workspace exhausted" in str(exc) and "task " in str(exc), exc
            print(f"OK oom: {exc}")
        else:
            raise SystemExit("a one-megabyte workspace did not run out")
    torch.cuda.synchronize()
    session.close()


if __name__ == "__main__":
    main()
