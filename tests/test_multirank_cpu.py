"""CPU, world_size 2 over gloo: the host side of the multi-GPU benchmark path -- how work
is split over ranks (independent shards, no data exchange), and how the whole-job number is
formed (max time over ranks)."""

import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import bench

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        assert bench._dist_env() == (rank, world, rank)
        # matmul: a rank's A block depends on the rank, B does not (replicated by seed)
        wl = bench.MatmulWorkload(small=True)
        wl.M, wl.N, wl.K = 64, 32, 48
        a, b = wl.host_inputs(rank, world)
        sums = torch.tensor([a.float().sum().item(), b.float().sum().item()], dtype=torch.float64)
        gathered = [torch.zeros(2, dtype=torch.float64) for _ in range(world)]
        dist.all_gather(gathered, sums)
        assert gathered[0][0] != gathered[1][0], "ranks must own different row blocks of A"
        assert gathered[0][1] == gathered[1][1], "B must be identical on every rank"
        # attention: the 512 (batch, head) pairs are split evenly, shards differ
        at = bench.AttentionWorkload(small=True)
        at.B, at.H, at.S, at.D = 1, 4, 8, 64
        q, k, v = at.host_inputs(rank, world)
        assert q.shape == (2, 8, 64) and at.units_per_step() == 4 * 2 * 8 * 8 * 64 // 2
        # the job is as slow as its slowest rank
        total_ms, e2e_ms = bench.max_over_ranks([10.0 + rank, 5.0 - rank], world, "cpu")
        assert (total_ms, e2e_ms) == (11.0, 5.0)
        value = bench.job_throughput(2 * 8192 ** 3, world, 10, 10 * total_ms, "TFLOP/s")
        assert abs(value - 2 * 8192 ** 3 * 2 * 10 / 0.110 / 1e12) < 1e-6
        with open(os.path.join(out_dir, f"ok{rank}"), "w") as f:
            f.write("ok")
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_gloo(tmp_path):
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def test_reference_arm_runs_only_on_rank_zero(monkeypatch, capsys):
    sys.path.insert(0, ROOT)
    import bench

    monkeypatch.setenv("RANK", "1")
    monkeypatch.setenv("WORLD_SIZE", "2")
    args = type("A", (), {"gpus": 2, "steps": 1, "warmup": 1})()
    bench.run_reference(args, bench.SoftmaxWorkload())
    assert capsys.readouterr().out == ""
