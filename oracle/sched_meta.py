"""Tile-scheduler metadata: CPU restatement of
csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu:11-107.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).  No golden vector exists
upstream; this restatement is pinned against the reference's own kernel, built
unmodified by oracle/build_ref.py and run beside it in
tests/test_gpu_sched_reference.py, and by the known answers in
tests/golden/sched_meta_known_answers.json, which were derived by hand from the
CUDA source (and which the reference kernel reproduces).

Output layout (csrc/params.h:10-17): one row of 8 int32 per SM partition
  [begin_req_idx, end_req_idx (inclusive), begin_block_idx,
   end_block_idx (exclusive), begin_split_idx, is_first_req_splitted,
   is_last_req_splitted, <pad, never written>]
and num_splits[b+1], the exclusive prefix sum of the number of splits of
every request.
"""
from typing import Optional, Sequence, Tuple

import numpy as np

META_INTS = 8          # csrc/params.h:10-17 (7 used ints + 1 pad)
META_USED_INTS = 7


def effective_seqlens(
    b: int,
    block_size_n: int,
    seqlens_k: Optional[Sequence[int]] = None,
    topk: int = -1,
    extra_topk: int = -1,
    topk_length: Optional[Sequence[int]] = None,
    extra_topk_length: Optional[Sequence[int]] = None,
) -> np.ndarray:
    """Per-request length the scheduler balances on
    (get_decoding_sched_meta.cu:29-42)."""
    out = np.zeros(b, dtype=np.int64)
    for i in range(b):
        if topk == -1:
            s = int(seqlens_k[i])                      # :33
        else:
            s = int(topk_length[i]) if topk_length is not None else topk   # :36
            if s == 0:
                s = 1                                   # :37
            if extra_topk > 0:                          # :38 (extra_topk "truthy"; -1 means disabled in callers -> guarded there)
                s = (s + block_size_n - 1) // block_size_n * block_size_n   # :39
                s += int(extra_topk_length[i]) if extra_topk_length is not None else extra_topk  # :40
        out[i] = s
    return out


def get_sched_meta(
    b: int,
    num_sm_parts: int,
    block_size_n: int = 64,
    fixed_overhead_num_blocks: int = 5,
    seqlens_k: Optional[Sequence[int]] = None,
    topk: int = -1,
    extra_topk: int = -1,
    topk_length: Optional[Sequence[int]] = None,
    extra_topk_length: Optional[Sequence[int]] = None,
) -> Tuple[np.ndarray, np.ndarray]:
    """Return (meta[int32, num_sm_parts x 8], num_splits[int32, b+1]).

    Column 7 of meta is returned as 0; the reference never writes it
    (get_decoding_sched_meta.cu:66-98), so comparisons use columns 0..6.
    """
    F = fixed_overhead_num_blocks
    seq = effective_seqlens(b, block_size_n, seqlens_k, topk, extra_topk, topk_length, extra_topk_length)

    # :43-53  -- a zero-length request still counts one block
    first_blk = np.zeros(b, dtype=np.int64)
    last_blk = np.maximum(seq - 1, 0) // block_size_n
    nblk = last_blk - first_blk + 1
    total = int((nblk + F).sum())

    payload = -(-total // num_sm_parts) + F            # :62

    meta = np.zeros((num_sm_parts, META_INTS), dtype=np.int32)
    num_splits = np.zeros(b + 1, dtype=np.int32)

    def first_block_idx_shared(i: int) -> int:
        # The shared-memory arrays are adjacent (:21-26): reading
        # first_block_idx_shared[b] lands on last_block_idx_shared[0].
        return int(first_blk[i]) if i < b else int(last_blk[0])

    now_req, now_block, now_split, cum = 0, 0, 0, 0
    for p in range(num_sm_parts):
        begin_req = now_req                                          # :67
        begin_block = now_block + first_block_idx_shared(now_req)    # :68
        begin_split = now_split                                      # :69
        first_split = int(now_block != 0)                            # :70
        remain = payload
        while now_req < b:                                           # :72
            rest = int(nblk[now_req]) - now_block
            if remain >= rest + F:                                   # :75
                cum += now_split + 1
                num_splits[now_req + 1] = cum
                remain -= rest + F
                now_req += 1
                now_block = 0
                now_split = 0
            else:
                if remain - F > 0:                                   # :83
                    now_block += remain - F
                    now_split += 1
                    remain = 0
                break
        end_req = now_req if now_block > 0 else now_req - 1          # :92
        if now_block > 0:                                            # :93
            end_block = now_block + first_block_idx_shared(now_req)
        else:
            end_block = 0 if seq[now_req - 1] == 0 else int(last_blk[now_req - 1]) + 1
        last_split = int(end_block != int(last_blk[end_req]) + 1 and seq[end_req] != 0)   # :94
        if begin_req == end_req:                                     # :95-97
            first_split = last_split = int(bool(first_split) or bool(last_split))
        meta[p, :META_USED_INTS] = [begin_req, end_req, begin_block, end_block, begin_split, first_split, last_split]
    # :100 -- the device assert of the reference
    assert now_req == b and now_block == 0 and now_split == 0, "scheduler did not consume every request"
    return meta, num_splits


def splits_of_partition(meta_row, num_splits, b):
    """Enumerate (request, begin_block, end_block, split_slot_or_-1) for one
    partition, the way the decode kernels walk it
    (csrc/sm90/decode/dense/splitkv_mla.cuh:1021-1033,1242 and
    csrc/sm100/decode/head64/kernel.cuh:97-112).  split_slot == -1 means the
    request is not split and the kernel writes the final output directly."""
    begin_req, end_req, begin_block, end_block, begin_split, first_split, last_split = [int(x) for x in meta_row[:7]]
    out = []
    if begin_req >= b:
        return out
    for r in range(begin_req, end_req + 1):
        sb = begin_block if r == begin_req else 0
        eb = end_block if r == end_req else None     # None = to the request's last block
        is_split = (first_split if r == begin_req else 0) or (last_split if r == end_req else 0)
        slot = -1
        if is_split:
            slot = int(num_splits[r]) + (begin_split if r == begin_req else 0)
        out.append((r, sb, eb, slot))
    return out
