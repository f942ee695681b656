"""KV-sharded decode: every rank attends over its part of each request's cache, the partials are all-gathered and
merged like split-KV partials.  On CPU two gloo ranks check the gather + split-layout logic against the oracle with a
torch statement of the merge; on two GPUs the real path (NCCL all_gather + mla_combine) is checked end to end."""
import math
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _case(seed=0, b=3, h_q=16, lens=(300, 64, 1000)):
    """Full problem plus, per rank of 2, a paged cache holding that rank's part (request 1 lives on rank 0 only)."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, 1, h_q, 576, generator=g).to(torch.bfloat16)
    kv = [torch.randn(n, 576, generator=g).to(torch.bfloat16) for n in lens]
    cut = [150, 64, 400]                                    # tokens [0, cut) on rank 0, the rest on rank 1
    return q, kv, cut


def _paged(parts):
    """List of [n_i, 576] -> (blocked cache [nb, 64, 1, 576], block_table [b, max_blocks], seqlens [b])."""
    nblk = [max((p.size(0) + 63) // 64, 1) for p in parts]
    cache = torch.zeros(sum(nblk), 64, 1, 576, dtype=torch.bfloat16)
    table = torch.zeros(len(parts), max(nblk), dtype=torch.int32)
    at = 0
    for i, p in enumerate(parts):
        flat = cache[at:at + nblk[i]].view(-1, 576)
        flat[:p.size(0)] = p
        table[i, :nblk[i]] = torch.arange(at, at + nblk[i], dtype=torch.int32)
        at += nblk[i]
    return cache, table, torch.tensor([p.size(0) for p in parts], dtype=torch.int32)


def _merge_ref(o_accum, lse_accum, num_splits, b):
    """Torch statement of the combine step (base-2 LSEs, normalised partial outputs)."""
    outs, lses = [], []
    for i in range(b):
        lo, hi = int(num_splits[i]), int(num_splits[i + 1])
        l2 = lse_accum[lo:hi]                                               # [n, s_q, h_q]
        m = l2.max(dim=0).values
        wgt = torch.exp2(l2 - torch.where(torch.isinf(m), torch.zeros_like(m), m))
        den = wgt.sum(0)
        o = (wgt.unsqueeze(-1) * o_accum[lo:hi]).sum(0) / torch.where(den > 0, den, torch.ones_like(den)).unsqueeze(-1)
        outs.append(o)
        lses.append(torch.where(den > 0, (torch.log2(den) + m) / 1.4426950408889634, torch.full_like(den, math.inf)))
    return torch.stack(outs), torch.stack(lses).transpose(1, 2)              # [b, s_q, h_q, d_v], [b, h_q, s_q]


def _full_reference(q, kv):
    from oracle import attention
    cache, table, lens = _paged(kv)
    return attention.dense_decode(q, cache, table, lens, 512, False)


def _cpu_rank(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    from oracle import attention
    from flashmla_b200.context_parallel import partials_to_split_layout
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, kv, cut = _case()
        mine = [k[:c] if rank == 0 else k[c:] for k, c in zip(kv, cut)]
        cache, table, lens = _paged(mine)
        out_r, lse_r = attention.dense_decode(q, cache, table, lens, 512, False)     # this rank's partial (oracle on CPU)
        outs = [torch.empty_like(out_r) for _ in range(world)]
        lses = [torch.empty_like(lse_r) for _ in range(world)]
        dist.all_gather(outs, out_r.contiguous())
        dist.all_gather(lses, lse_r.contiguous())
        o_accum, lse_accum, num_splits = partials_to_split_layout(torch.stack(outs), torch.stack(lses))
        assert num_splits.tolist() == [0, 2, 4, 6]
        assert lse_accum[3].eq(-math.inf).all(), "request 1 has nothing on rank 1"
        out, lse = _merge_ref(o_accum, lse_accum, num_splits, q.size(0))
        ref_out, ref_lse = _full_reference(q, kv)
        assert (out - ref_out.float()).abs().max() <= 2e-2
        assert (lse - ref_lse).abs().max() <= 1e-3
    finally:
        dist.destroy_process_group()


def test_kv_sharded_layout_two_gloo_ranks():
    mp.spawn(_cpu_rank, args=(2, _free_port()), nprocs=2, join=True)


def _gpu_rank(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, ROOT)
    import flashmla_b200 as fm
    from flashmla_b200.context_parallel import flash_mla_decode_kv_sharded
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        q, kv, cut = _case(seed=1, b=3, h_q=128, lens=(5000, 64, 9000))
        cut = [2500, 64, 1000]
        mine = [k[:c] if rank == 0 else k[c:] for k, c in zip(kv, cut)]
        cache, table, lens = _paged(mine)
        out, lse = flash_mla_decode_kv_sharded(q.to(dev), cache.to(dev), table.to(dev), lens.to(dev), 512)
        torch.cuda.synchronize()
        fm.check_status()
        ref_out, ref_lse = _full_reference(q, kv)
        assert (out.cpu().float() - ref_out.float()).abs().max() <= 2e-2
        assert (lse.cpu() - ref_lse).abs().max() <= 1e-3
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_kv_shard_merge_on_one_gpu():
    """Everything of the KV-sharded path except the all_gather, on ONE GPU: the two shards' partials are computed one
    after the other through the ordinary decode API, stacked as the gather would deliver them, and merged by the
    library's combine kernel (merge_kv_shard_partials, the function the multi-rank path calls after its all_gather)."""
    sys.path.insert(0, ROOT)
    import flashmla_b200 as fm
    from flashmla_b200.context_parallel import merge_kv_shard_partials
    dev = torch.device("cuda", 0)
    q, kv, _ = _case(seed=1, b=3, h_q=128, lens=(5000, 64, 9000))
    cut = [2500, 64, 1000]
    outs, lses = [], []
    for rank in range(2):
        mine = [k[:c] if rank == 0 else k[c:] for k, c in zip(kv, cut)]
        cache, table, lens = _paged(mine)
        meta, _ = fm.get_mla_metadata()
        o, l = fm.flash_mla_with_kvcache(q.to(dev), cache.to(dev), table.to(dev), lens.to(dev), 512, meta, None, None, False)
        outs.append(o)
        lses.append(l)
    out, lse = merge_kv_shard_partials(torch.stack(outs), torch.stack(lses))
    torch.cuda.synchronize()
    fm.check_status()
    ref_out, ref_lse = _full_reference(q, kv)
    assert (out.cpu().float() - ref_out.float()).abs().max() <= 2e-2
    assert (lse.cpu() - ref_lse).abs().max() <= 1e-3


@pytest.mark.gpu
def test_kv_sharded_decode_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_gpu_rank, args=(2, _free_port()), nprocs=2, join=True)
