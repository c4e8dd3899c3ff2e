"""Child process of the host-agreement test: a gloo rank that may raise before the collectives."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch.distributed as dist

from shadowspill_b200.parallel import control


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    bad = int(sys.argv[1])                       # the rank that fails on the host (-1: nobody)
    dist.init_process_group("gloo")
    entered_collective = False

    def prepare():
        if rank == bad:
            raise ValueError(f"microbatch 1: 300 tokens, plan expects 256")
        return rank * 10
    try:
        got = control.coordinated(prepare)
        # only now would a rank enqueue its collectives
        entered_collective = True
        dist.barrier()
        assert got == rank * 10
        control.check_invocation("step", 0)
        try:
            control.check_invocation("step" if rank else "forward_backward", 0)
            print(f"rank {rank} MISSED mismatch", flush=True)
            sys.exit(1)
        except ValueError:
            pass
        print(f"rank {rank} OK ran", flush=True)
    except control.CoordinatedFailure as exc:
        assert bad in exc.failures and "plan expects 256" in exc.failures[bad]
        assert not entered_collective
        print(f"rank {rank} OK refused ({sorted(exc.failures)})", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
