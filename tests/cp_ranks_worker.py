"""One rank of the 2-GPU context-parallel parity check (launched by tests/test_gpu_cp_ranks.py through
torch.distributed.run).  Every rank draws the same seeded full-length inputs on the CPU, takes its token shard, runs
`context_parallel_prefill` over NCCL (one all-gather of the per-rank state maps; no peer-memory operands) and compares
its output rows and the final state with the fp64 recurrence.  Exits non-zero on any mismatch."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT / "eat-kernels_b200", ROOT / "oracle", ROOT / "tests"):
    sys.path.insert(0, str(p))

import kda_oracle as ko  # noqa: E402
from kda_testlib import gold_raw, slow_gates_  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from kda_b200 import parallel
    failures = []
    for case, (H, T, slow, balanced) in enumerate([(4, 2048, False, False), (4, 2272, True, True), (3, 1000, False, True)]):
        inputs = ko.make_inputs_raw(H, [T], 900 + case)
        if slow:
            slow_gates_(inputs, 900 + case)
        gold_o, gold_s, _ = gold_raw(inputs, [T])
        shards = parallel.balanced_shards(T, world, H) if balanced else [T // world] * (world - 1) + [T - (T // world) * (world - 1)]
        t0 = sum(shards[:rank])
        sl = slice(t0, t0 + shards[rank])
        q, k, v, g, beta, A_log, dt_bias, scale, init, _ = inputs
        mine = [t[:, sl].contiguous().to(dev) for t in (q, k, v, g, beta)]
        out, fin = parallel.context_parallel_prefill(*mine, A_log.to(dev), dt_bias.to(dev), scale,
                                                     init.to(dev) if rank == 0 else None)
        torch.cuda.synchronize()
        tag = f"rank {rank} case {case} H={H} T={T} shards={shards}"
        try:
            ko.check_close(out.cpu(), gold_o[:, sl], tag + " output")
            ko.check_close(fin.cpu(), gold_s, tag + " final state")
        except AssertionError as e:
            failures.append(str(e))
    flag = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(flag)
    dist.destroy_process_group()
    for f in failures:
        print("MISMATCH:", f, flush=True)
    if int(flag.item()):
        sys.exit(1)
    print(f"rank {rank}: context-parallel parity ok", flush=True)


if __name__ == "__main__":
    main()
