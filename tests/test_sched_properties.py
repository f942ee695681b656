"""Properties of the tile scheduler's CPU restatement (oracle/sched_meta.py), checked with hypothesis, and the
hand-derived known answers for the sparse modes.  The same property checker runs on the CUDA kernel's output in
tests/test_gpu_sched_combine.py.  The reference holds no golden vector for the scheduler, so these properties (which
follow from how the decode kernels consume the metadata) and the hand-derived vectors are what pins it."""
import json
import os

from hypothesis import given, settings, strategies as st

from oracle import sched_meta
from tests.helpers import check_schedule_properties


@settings(max_examples=300, deadline=None)
@given(seqlens=st.lists(st.one_of(st.just(0), st.integers(1, 300), st.integers(1, 40000)), min_size=1, max_size=200),
       P=st.sampled_from([1, 2, 3, 5, 37, 74, 148, 300]), F=st.sampled_from([0, 3, 5]), bs=st.sampled_from([64, 32]))
def test_dense_schedule_properties(seqlens, P, F, bs):
    meta, ns = sched_meta.get_sched_meta(len(seqlens), P, bs, F, seqlens_k=seqlens)
    check_schedule_properties(meta, ns, seqlens, P, bs, F)


@settings(max_examples=300, deadline=None)
@given(data=st.data(), b=st.integers(1, 150), P=st.sampled_from([1, 3, 64, 74, 148]), topk=st.sampled_from([64, 100, 128, 2048]),
       extra_topk=st.sampled_from([0, 64, 192]), F=st.sampled_from([3, 5]))
def test_sparse_schedule_properties(data, b, P, topk, extra_topk, F):
    tl = data.draw(st.one_of(st.none(), st.lists(st.integers(0, topk), min_size=b, max_size=b)))
    etl = None
    if extra_topk:
        etl = data.draw(st.one_of(st.none(), st.lists(st.integers(0, extra_topk), min_size=b, max_size=b)))
    meta, ns = sched_meta.get_sched_meta(b, P, 64, F, topk=topk, extra_topk=extra_topk, topk_length=tl, extra_topk_length=etl)
    eff = sched_meta.effective_seqlens(b, 64, None, topk, extra_topk, tl, etl)
    check_schedule_properties(meta, ns, eff, P, 64, F)


def test_known_answers_all_modes(golden_dir):
    cases = json.load(open(os.path.join(golden_dir, "sched_meta_known_answers.json")))["cases"]
    assert len(cases) >= 8
    for c in cases:
        if "seqlens" in c:
            b = len(c["seqlens"])
            kw = dict(seqlens_k=c["seqlens"])
            eff = c["seqlens"]
        else:
            b = c.get("b") or len(c["topk_length"])
            kw = dict(topk=c["topk"], extra_topk=c["extra_topk"], topk_length=c.get("topk_length"),
                      extra_topk_length=c.get("extra_topk_length"))
            eff = sched_meta.effective_seqlens(b, c["block_size_n"], None, c["topk"], c["extra_topk"], c.get("topk_length"),
                                               c.get("extra_topk_length"))
        meta, ns = sched_meta.get_sched_meta(b, c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"], **kw)
        assert meta[:, :7].tolist() == c["meta"], c
        assert ns.tolist() == c["num_splits"], c
        # the hand-derived vectors themselves satisfy the properties
        check_schedule_properties(c["meta"], c["num_splits"], eff, c["num_sm_parts"], c["block_size_n"], c["fixed_overhead"])
