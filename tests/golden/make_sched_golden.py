"""Generate tests/golden/sched_meta_reference.json: tile-scheduler metadata produced by the reference's OWN CUDA kernel
(csrc/smxx/decode/get_decoding_sched_meta/get_decoding_sched_meta.cu, built unmodified into oracle/_ref/ by
oracle/build_ref.py) on seeded dense and sparse cases.  Needs a GPU and that library.

Usage:  python tests/golden/make_sched_golden.py [output.json]

Every case is first run through the CPU restatement, which asserts the reference's closing device assert on the host, so
that the reference kernel is only launched on inputs it accepts."""
import ctypes
import json
import os
import random
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import sched_meta as osm  # noqa: E402


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "sched_meta_reference.json")
    lib = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libref_sched_meta.so"))
    lib.ref_get_decoding_sched_meta.restype = ctypes.c_int
    lib.ref_get_decoding_sched_meta.argtypes = [ctypes.c_int] * 6 + [ctypes.c_void_p] * 5 + [ctypes.c_int, ctypes.c_void_p]
    dev = torch.device("cuda:0")
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    ten = lambda x: None if x is None else torch.tensor(x, dtype=torch.int32, device=dev)
    rng = random.Random(2024)
    specs = []
    for _ in range(40):                                    # dense
        b = rng.randint(1, 24)
        kind = rng.random()
        seq = [0 if rng.random() < 0.12 else (rng.randint(1, 300) if kind < 0.4 else rng.randint(1, 9000)) for _ in range(b)]
        specs.append(dict(seqlens=seq, num_sm_parts=rng.choice([1, 2, 3, 5, 8, 13]), fixed_overhead=rng.choice([5, 5, 3, 0])))
    specs.append(dict(seqlens=[4096] * 16 + [8192], num_sm_parts=74, fixed_overhead=5))
    for _ in range(30):                                    # sparse
        b = rng.randint(1, 20)
        topk = rng.choice([64, 100, 128, 2048, 1])
        extra_topk = rng.choice([0, 0, 64, 192])
        specs.append(dict(b=b, topk=topk, extra_topk=extra_topk,
                          topk_length=[rng.randint(0, topk) for _ in range(b)] if rng.random() < 0.6 else None,
                          extra_topk_length=[rng.randint(0, extra_topk) for _ in range(b)] if extra_topk and rng.random() < 0.6 else None,
                          num_sm_parts=rng.choice([1, 2, 4, 7, 12]), fixed_overhead=rng.choice([5, 5, 3])))
    cases = []
    for s in specs:
        dense = "seqlens" in s
        b = len(s["seqlens"]) if dense else s["b"]
        P, F = s["num_sm_parts"], s["fixed_overhead"]
        kw = dict(seqlens_k=s["seqlens"]) if dense else dict(topk=s["topk"], extra_topk=s["extra_topk"], topk_length=s["topk_length"],
                                                             extra_topk_length=s["extra_topk_length"])
        osm.get_sched_meta(b, P, 64, F, **kw)              # raises where the reference's device assert would fire
        meta = torch.full((P, 8), -7, dtype=torch.int32, device=dev)
        ns = torch.full((b + 1,), -7, dtype=torch.int32, device=dev)
        # (the input tensors stay referenced until the kernel has run)
        tl_t = None if dense else ten(s["topk_length"])
        etl_t = None if dense else ten(s["extra_topk_length"])
        seq_t = ten(s["seqlens"]) if dense else None
        rc = lib.ref_get_decoding_sched_meta(b, 1, 64, F, -1 if dense else s["topk"], 0 if dense else s["extra_topk"],
                                             ptr(tl_t), ptr(etl_t), ptr(seq_t), ptr(meta), ptr(ns), P, None)
        torch.cuda.synchronize()
        assert rc == 0
        cases.append(dict(s, block_size_n=64, meta=meta[:, :7].cpu().tolist(), num_splits=ns.cpu().tolist()))
    with open(out_path, "w") as f:
        f.write('{\n "_comment": "Produced by the reference kernel itself (tests/golden/make_sched_golden.py). Columns: begin_req, end_req, '
                'begin_block, end_block, begin_split, first_split, last_split.",\n "cases": [\n')
        f.write(",\n".join("  " + json.dumps(c) for c in cases))
        f.write("\n ]\n}\n")
    print(len(cases), "cases ->", out_path)


if __name__ == "__main__":
    main()
