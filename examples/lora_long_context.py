"""Low-rank adapters on a frozen base, one long sequence per step, token-local work in row chunks.

    python examples/lora_long_context.py                                   # CPU, tiny hybrid model
    python examples/lora_long_context.py --device cuda --model qwen35-9b --tokens 32768 --rows 8192

Three things combine here. The adapters: only the factors train, so the frozen base owns no
gradient, no moments and no update. The graph frontend: the adapted layers are exported and
differentiated like any other, so the planner may keep activations instead of recomputing. Axis
chunks: projections, norms and the feed-forward run ``--rows`` tokens at a time, so a step's
temporaries follow the chunk, not the sequence; attention and the delta rule still see the whole
sequence.
"""
import argparse
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))


def main(argv=None) -> list[float]:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="qwen35-tiny")
    ap.add_argument("--device", default="cpu", choices=["cpu", "cuda"])
    ap.add_argument("--tokens", type=int, default=512, help="length of the one sequence of every step")
    ap.add_argument("--rows", type=int, default=128, help="row-chunk size of the token-local operators")
    ap.add_argument("--rank", type=int, default=8)
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args(argv)
    from shadowspill_b200.data.synthetic import make_batch
    from shadowspill_b200.planning.plan import SearchOptions
    from shadowspill_b200.training.session import TrainingSession, TrainingSetup
    cpu = a.device == "cpu"
    setup = TrainingSetup(model=a.model, device=a.device, dtype="float32" if cpu else "bfloat16",
                          device_gib=0.6 if cpu else 24.0, spill_gib=0.5 if cpu else 128.0,
                          tokens_per_step=a.tokens, microbatch_tokens=a.tokens, slots=4, mean_seqlen=float(a.tokens),
                          frontend="graph", axis_chunk_rows=a.rows, lr=1e-2 if cpu else 1e-4,
                          profile=not cpu, calibrate=not cpu, stochastic_rounding=not cpu,
                          profile_sequence_tokens=0 if cpu else a.tokens,
                          lora={"rank": a.rank, "alpha": 2.0 * a.rank, "routed_experts": True, "train_base": False,
                                "targets": ["wq", "wk", "wv", "wo", "w13", "w2", "w_qkvz", "w_out"]},
                          recompute_shares=(100, 0), saved_variant="save_attention",
                          search=SearchOptions(minimum_object_bytes_evict_eligible=1024 if cpu else 1 << 20, workers=2))
    session = TrainingSession(setup, log=lambda m: print("[prepare]", m))
    trainable = sum(p.numel for st in session.executor.stages for p in st.params if p.trainable)
    total = sum(p.numel for st in session.executor.stages for p in st.params)
    print(f"{trainable:,} of {total:,} parameters train; layer stages are {type(session.executor.stages[1]).__name__}; "
          f"plan keeps: {session.plan.summary.selection or 'nothing (recompute)'}")
    losses = []
    try:
        for step in range(a.steps):
            batch = make_batch(step % 2, vocab=session.cfg.vocab_size, tokens_per_step=a.tokens,
                               microbatch_tokens=a.tokens, fixed_len=a.tokens, slots=session.slots)
            losses.append(session.step(batch).loss)
            print(f"step {step}: loss {losses[-1]:.4f}")
    finally:
        session.close()
    return losses


if __name__ == "__main__":
    main()
