"""Child process of the data-parallel tests: one rank of a 2+-rank job."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist

from shadowspill_b200.communication.info import CommunicationInfo
from shadowspill_b200.data.synthetic import make_batch, to_device
from shadowspill_b200.execution.executor import Executor, Hyperparameters
from shadowspill_b200.execution.resident import ResidentTrainer
from shadowspill_b200.frontend.capture import BatchGeometry, StepDataOrdering, build_step
from shadowspill_b200.models.config import DecoderConfig, preset
from shadowspill_b200.planning.plan import MemoryBudgets, SearchOptions, plan_program


def main():
    device = sys.argv[1]                      # cpu | cuda
    arm = sys.argv[2] if len(sys.argv) > 2 else "auto"
    expert_parallel = arm == "ep"         # routed model, experts split over the ranks
    if expert_parallel:
        arm = "peer"
    pretrained = arm.startswith("pretrained-")   # start from whole-parameter weights of another seed
    if pretrained:
        arm = arm.split("-", 1)[1]
    master = arm.startswith("master-")    # fp32 master shards beside the model-dtype shards
    if master:
        arm = arm.split("-", 1)[1]
    tied = arm.startswith("tied-")        # the head reads, and adds to the gradient of, the embedding
    if tied:
        arm = arm.split("-", 1)[1]
    graph = arm.startswith("graph-")      # stages exported and differentiated by the graph frontend
    if graph:
        arm = arm.split("-", 1)[1]
    groups = 1
    if arm.startswith("groups-"):         # microbatches in two sweeps; gradients meet in fp32 shard sums
        groups, arm = 2, arm.split("-", 1)[1]
    rule = "adamw"
    if arm.startswith("lion-"):           # the unfused update path: all-reduce, then the rule
        rule, arm = "lion", arm.split("-", 1)[1]
    # "small-<arm>": tensors under 64 KiB stay whole on every rank (the norm vectors and, in the
    # tiny model, the attention projections), everything larger is cut into shards
    min_shard = 0
    if arm.startswith("small-"):
        min_shard, arm = 64 << 10, arm.split("-", 1)[1]
    fused = arm.startswith("fused-")      # forward weight gather inside the consuming GEMM
    if fused:
        arm = arm.split("-", 1)[1]
    replicas = 1
    if arm.startswith("replicas-"):       # e.g. replicas-dist / replicas-peer on 4 ranks: 2 x 2
        replicas, arm = 2, arm.split("-", 1)[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    cuda = device == "cuda"
    if cuda:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{rank}"))
    else:
        dist.init_process_group("gloo")
    dtype = torch.bfloat16 if cuda else torch.float32
    # the sm_100a attention kernels need head widths of 64/128/256
    cfg = DecoderConfig("llama3", 2, 256, 4, 2, 64, 512, 1024) if cuda else preset("llama3-tiny")
    if expert_parallel:
        from dataclasses import replace
        cfg = replace(preset("olmoe-tiny"), d_model=256, head_dim=64, vocab_size=1024)
    if tied:
        from dataclasses import replace
        cfg = replace(cfg, tied_embeddings=True)
    T, n_mb = 256, 2 * groups
    if fused:
        # matrices large enough for several 256-row tiles and 64-multiple contraction lengths
        cfg = DecoderConfig("llama3", 2, 512, 8, 2, 64, 1024, 1024)
        T = 512
    geo = BatchGeometry(T, n_mb, slots=16, mean_seqlen=64)
    shard_world = world // replicas
    prog, desc = build_step(cfg, geo, StepDataOrdering(microbatch_groups=groups), dtype=dtype, world_size=shard_world, rank=rank,
                            expert_parallel=expert_parallel, replicas=replicas,
                            min_shard_bytes=min_shard, master_weights=master, fused_gather=fused,
                            frontend="graph" if graph else "stages")
    total = sum(o.bytes for o in prog.objects)
    plan = plan_program(prog, MemoryBudgets(total, 64 << 20, headroom_bytes=0), CommunicationInfo(),
                        SearchOptions(minimum_object_bytes_evict_eligible=1024, workers=1,
                                      deterministic=True))
    lr = 3e-4 if cuda else 3e-3
    ex = Executor(plan, desc, device=device, device_index=rank if cuda else 0, seed=5,
                  hyper=Hyperparameters(lr=lr, rule=rule), stochastic_rounding=False, collectives=arm)
    ex.initialize(on_device=False)
    ref = ResidentTrainer(cfg, device=f"cuda:{rank}" if cuda else "cpu", dtype=dtype,
                          seed=9 if pretrained else 5, lr=lr, stochastic_rounding=False, rule=rule)
    if pretrained:
        # every rank keeps its slice of each whole tensor; moments stay at zero on both sides
        whole = {k: v.cpu() for k, v in ref.state_dict().items() if not k.startswith("exp_avg")}
        ex.load_full_state_dict(whole)
    ok = True
    for step in range(2):
        # the global batch: every rank's microbatches, weights normalised over all of them
        parts = [make_batch(100 * step + r, vocab=cfg.vocab_size, tokens_per_step=T * n_mb,
                            microbatch_tokens=T, median=60, min_len=8, max_len=128, slots=16)
                 for r in range(world)]
        for part in parts:
            for mb in part:
                mb.weights /= world
        res = ex.run(parts[rank])
        loss = torch.tensor([res.loss], dtype=torch.float64, device="cuda" if cuda else "cpu")
        dist.all_reduce(loss)
        want = ref.step([to_device(m, ref.device) for part in parts for m in part])
        tol = 2e-2 if cuda else 1e-5
        if abs(float(loss) - want) > tol * max(1.0, abs(want)):
            print(f"rank {rank} step {step}: loss {float(loss)} != {want}", flush=True)
            ok = False
    if fused:
        from shadowspill_b200.ops import functional as F
        # 2 layers x 4 matrices x 2 steps, each gathered by the first GEMM that read it
        if F.fused_gather_launches != 16:
            print(f"rank {rank}: {F.fused_gather_launches} fused gathers, expected 16", flush=True)
            ok = False
    # owned slices must equal the matching slices of the resident model
    refs = ref.state_dict()
    # gradient summation order differs (per-rank partial sums), hence a few ulps in fp32
    rtol, atol = (5e-2, 2e-3) if cuda else (1e-4, 5e-5)
    banks = {f"{st.name}.{p.name}": p for st in ex.stages for p in st.params if p.expert_sharded}
    for name, shard in ex.named_tensors():
        if name.startswith("exp_avg"):
            continue
        key = name[len("master."):] if name.startswith("master.") else name   # masters mirror the weights
        full = refs[key].reshape(-1).cpu()
        if key in banks:                  # this rank's experts, stored whole
            p = banks[key]
            per = p.numel // p.shape[0]
            lo, hi = p.expert_lo * per, (p.expert_lo + p.shape[0]) * per
        else:
            lo = (rank % shard_world) * shard.numel()
            hi = min(full.numel(), lo + shard.numel())
        if hi <= lo:
            continue
        a, b = shard[:hi - lo].float(), full[lo:hi].float()
        if cuda:
            # bf16: Adam turns the sign of a near-zero gradient into a 2*lr difference, so
            # compare as a numerical gate does (relative L2 and cosine), not elementwise
            rel = float((a - b).norm() / (b.norm() + 1e-12))
            cos = float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-12))
            lim = 6e-2 if expert_parallel else 2.5e-2      # routing ties flip a few tokens in bf16
            good = (rel < lim and cos > 0.998) or float((a - b).abs().max()) < 1e-6
        else:
            good = torch.allclose(a, b, rtol=rtol, atol=atol)
        if not good:
            print(f"rank {rank}: {name} differs by {float((a - b).abs().max())}", flush=True)
            ok = False
    if cuda:
        from shadowspill_b200.ops import _lib
        _lib.check_status()
    ex.close()
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank} {'OK' if ok else 'FAILED'} arm={ex.collectives.name}", flush=True)
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
