"""The N > 1 host logic of bench.py on CPU: two gloo ranks on 127.0.0.1 check the batch sharding of the
long-context sweep (disjoint, complete), the whole-job reduction (time = max over ranks, work = sum), and that the
reference arm runs on rank 0 only."""
import json
import os
import socket
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    import bench
    from tests import workloads as W
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b_total = 1024
        seq_all = W.seqlens_lognormal(b_total, 8192, 1.0, 256, 131072, seed=0)
        begin, end = bench.shard_of_rank(b_total, world, rank)
        mine = torch.zeros(b_total, dtype=torch.int64)
        mine[begin:end] = 1
        cover = mine.clone()
        dist.all_reduce(cover, op=dist.ReduceOp.SUM)
        assert bool((cover == 1).all()), "every request belongs to exactly one rank"
        tokens = float(seq_all[begin:end].sum())
        # rank r pretends to have needed (10 + r) ms for the device leg and (20 - r) ms end to end
        res = bench.reduce_over_ranks(10.0 + rank, 20.0 - rank, float(end - begin), tokens, 2.0 * tokens, 3.0 * tokens, dist, "cpu")
        if rank == 0:
            with open(os.path.join(out_dir, "reduced.json"), "w") as f:
                json.dump({"res": res, "tokens_all": float(seq_all.sum()), "world": world}, f)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_reduce(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = json.load(open(tmp_path / "reduced.json"))
    ms_total, ms_e2e, units, tokens, flops, nbytes = r["res"]
    assert ms_total == 10.0 + (world - 1) and ms_e2e == 20.0           # maxima over the ranks
    assert units == 1024.0 and tokens == r["tokens_all"]              # sums over the ranks
    assert flops == 2.0 * tokens and nbytes == 3.0 * tokens


def test_single_process_reduction_is_identity():
    sys.path.insert(0, ROOT)
    import bench
    assert bench.reduce_over_ranks(1.0, 2.0, 3.0, 4.0, 5.0, 6.0, None, "cpu") == (1.0, 2.0, 3.0, 4.0, 5.0, 6.0)
    assert bench.shard_of_rank(1024, 8, 3) == (384, 512)


def test_token_balanced_shards():
    """The long-context sweep's router: disjoint shards of equal request count whose token sums differ by little."""
    sys.path.insert(0, ROOT)
    import bench
    from tests import workloads as W
    seq_all = W.seqlens_lognormal(1024, 8192, 1.0, 256, 131072, seed=0)
    for world in (1, 2, 4, 8):
        shards = [bench.balanced_shard(seq_all, world, r) for r in range(world)]
        assert all(s.numel() == 1024 // world for s in shards)
        assert torch.equal(torch.sort(torch.cat(shards)).values, torch.arange(1024))
        tokens = torch.tensor([int(seq_all[s].sum()) for s in shards], dtype=torch.float64)
        assert float(tokens.max() / tokens.mean()) < 1.02, tokens
    # (contiguous slices of the same batch: the fullest rank is 8 % above the mean at 4 ranks, 18 % at 8)


def test_reference_arm_is_rank0_only():
    """Under torchrun every rank starts `bench.py --impl reference`; all but rank 0 leave at once, silently."""
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0"],
                       env=env, capture_output=True, text=True, timeout=300)
    assert p.returncode == 0 and p.stdout.strip() == ""
