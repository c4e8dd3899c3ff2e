"""Plan and run a few budgeted training steps in process, then write both reports.

    python examples/train_budgeted.py                 # tiny model on CPU (mock device backend)
    python examples/train_budgeted.py --device cuda --model llama3-1b --device-gib 8 --spill-gib 32 \
        --tokens 32768 --microbatch 8192
    python examples/train_budgeted.py --spill-pool file --spill-dir /tmp     # spill to a direct-I/O file
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from shadowspill_b200.data.synthetic import make_batch
from shadowspill_b200.planning.plan import SearchOptions
from shadowspill_b200.training.session import TrainingSession, TrainingSetup


def main(argv=None) -> float:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3-tiny")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--device-gib", type=float, default=0.53)
    ap.add_argument("--spill-gib", type=float, default=0.25)
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--microbatch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--out", default="")
    ap.add_argument("--spill-pool", default="host", choices=["host", "file", "remote"])
    ap.add_argument("--spill-dir", default="", help="directory of the file spill pool")
    ap.add_argument("--spill-address", default="", help="host:port of an ss_memory_daemon")
    a = ap.parse_args(argv)
    cpu = a.device == "cpu"
    setup = TrainingSetup(model=a.model, device_gib=a.device_gib, spill_gib=a.spill_gib,
                          tokens_per_step=a.tokens, microbatch_tokens=a.microbatch, lr=3e-3,
                          device=a.device, dtype="float32" if cpu else "bfloat16",
                          profile=not cpu, calibrate=not cpu, trace_capacity=1 << 14,
                          spill_pool=a.spill_pool, spill_directory=a.spill_dir, spill_address=a.spill_address,
                          search=SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=2))
    session = TrainingSession(setup, log=print)
    s = session.plan.summary
    print(f"plan: {s.fetch_bytes / 2**20:.1f} MiB fetched, {s.evict_bytes / 2**20:.1f} MiB evicted per step; "
          f"device pool {session.plan.device_bytes / 2**20:.1f} MiB")
    loss = 0.0
    for i in range(a.steps):
        batch = make_batch(i, vocab=session.cfg.vocab_size, tokens_per_step=a.tokens,
                           microbatch_tokens=a.microbatch, median=60 if cpu else 1200,
                           min_len=8, max_len=min(a.microbatch, 8192), slots=session.slots)
        loss = session.step(batch).loss
        print(f"step {i}: loss {loss:.4f}")
    if a.out:
        session.write_plan_report(a.out)
        batch = make_batch(99, vocab=session.cfg.vocab_size, tokens_per_step=a.tokens,
                           microbatch_tokens=a.microbatch, median=60 if cpu else 1200,
                           min_len=8, max_len=min(a.microbatch, 8192), slots=session.slots)
        _, diag = session.traced_step(batch, a.out)
        print(f"traced step: {diag.makespan_s * 1e3:.1f} ms measured, "
              f"{diag.simulated_makespan_s * 1e3:.1f} ms simulated -> {a.out}/runtime.html")
    session.close()
    return loss


if __name__ == "__main__":
    main()
