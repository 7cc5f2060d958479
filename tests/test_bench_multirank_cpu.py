"""CPU: the N > 1 path of bench.py (independent replicas, no data-path collective) -- the cross-rank
reduction of the timings and the aggregate throughput, on two gloo ranks."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import bench

    # replica r measured (10 + 5 r) ms for the device loop and (20 - 3 r) ms end to end
    ms, e2e = bench.max_over_ranks([10.0 + 5 * rank, 20.0 - 3 * rank], world)
    tok = bench.aggregate_throughput(world, batch=1, steps=100, ms_max=ms)
    Path(out_dir, f"rank{rank}.txt").write_text(f"{ms} {e2e} {tok}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_replicas_reduce_to_the_slowest_rank(tmp_path):
    port = 29600 + os.getpid() % 300
    mp.spawn(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        ms, e2e, tok = map(float, (tmp_path / f"rank{rank}.txt").read_text().split())
        assert ms == 15.0 and e2e == 20.0                 # max over ranks of each timing
        assert abs(tok - 2 * 100 / 0.015) < 1e-6            # whole-job tokens/s = sum over replicas


def test_single_rank_is_identity():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.max_over_ranks([3.0, 4.0], 1) == [3.0, 4.0]
    assert bench.aggregate_throughput(1, 4, 10, 2.0) == 4 * 10 / 2e-3
    assert bench.algorithmic_bytes(__import__("prime_kernels_b200.decode", fromlist=["x"]).SMOLLM2_360M, 1, 0) == 723642240
    assert bench.algorithmic_bytes(__import__("prime_kernels_b200.decode", fromlist=["x"]).SMOLLM2_135M, 1, 1) == 269030016 + 23040
