"""World-size-2 `gloo` coverage (CPU) of the multi-GPU logic of bench.py: the path shards by
sequence with no data-path collective, so what ranks share is the seed-by-rank input sharding,
the MAX reduction of the timings and the rule that only rank 0 reports."""
from __future__ import annotations

import io
import os
import sys
from contextlib import redirect_stdout
from pathlib import Path
from types import SimpleNamespace

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "relation-lm_b200"))
    import bench

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = SimpleNamespace(max_context=32, vocab_size=16000, boundary_vocab_size=256)
        tokens, bounds = bench.rank_inputs(cfg, 1002, 4, rank)
        # the slowest rank defines every reported time
        mine = [10.0 + rank, 5.0 - rank, 1.0]
        reduced = bench.max_over_ranks(mine, world, torch.device("cpu"))
        # the reference arm runs on rank 0 only: other ranks return without work or output
        printed = ""
        if rank != 0:
            buf = io.StringIO()
            with redirect_stdout(buf):
                bench.run_reference(SimpleNamespace(workload="cfg2", batch=8, steps=1, warmup=3, gpus=world))
            printed = buf.getvalue()
        torch.save({"tokens": tokens, "bounds": bounds, "reduced": reduced, "printed": printed},
                   os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_shard_inputs_and_reduce_timings(tmp_path):
    world, port = 2, 29541 + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    r0, r1 = (torch.load(tmp_path / f"rank{r}.pt") for r in range(world))
    assert r0["tokens"].shape == r1["tokens"].shape == (4, 32)
    assert not torch.equal(r0["tokens"], r1["tokens"])          # different sequences per rank
    assert not torch.equal(r0["bounds"], r1["bounds"])
    assert int(r0["tokens"].max()) < 16000 and int(r0["bounds"].max()) < 256
    assert r0["reduced"] == r1["reduced"] == [11.0, 5.0, 1.0]   # element-wise maximum over ranks
    assert r1["printed"] == ""


def test_job_rate_counts_every_rank():
    sys.path.insert(0, str(ROOT))
    import bench

    assert bench.job_rate(1, 8, 64, 20.0) == 8 * 64 / 0.02
    assert bench.job_rate(8, 8, 64, 20.0) == 8 * bench.job_rate(1, 8, 64, 20.0)
    one = bench.workload_config("cfg2", 8, 1)
    eight = bench.workload_config("cfg2", 8, 8)
    assert one["batch_per_gpu"] == eight["batch_per_gpu"] == 8 and eight["global_batch"] == 64
