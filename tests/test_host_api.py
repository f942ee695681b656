"""CPU-only checks: the C-ABI library loads and exports every declared symbol, the header and the ctypes
structures agree, and the host-side API mirror enforces the reference's misuse checks."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header():
    return open(os.path.join(ROOT, "include", "flashmla_b200.h")).read()


def test_library_exports_every_declared_symbol():
    from flashmla_b200 import _capi
    declared = set(re.findall(r"^\s*(?:const char\*|int|size_t)\s+(mla_\w+)\s*\(", _header(), flags=re.M))
    assert declared, "no declarations found in the header"
    assert declared == set(_capi.SYMBOLS), (declared, set(_capi.SYMBOLS))
    lib = _capi.lib()
    for name in declared:
        assert hasattr(lib, name), f"{name} not exported"
    assert lib.mla_abi_version() == 2
    assert lib.mla_last_error() == b""


def _struct_fields(name):
    text = _header()
    end = text.index("} " + name + ";")
    body = text[text.rindex("typedef struct {", 0, end) + len("typedef struct {"):end]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for stmt in body.split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        typ, names = re.match(r"((?:const\s+)?\w+\s*\*?)\s*(.*)", stmt).groups()
        for n in names.split(","):
            n = n.strip()
            is_ptr = "*" in typ or n.startswith("*")
            fields.append((n.lstrip("* "), "ptr" if is_ptr else typ.strip()))
    return fields


@pytest.mark.parametrize("cname,pyname", [
    ("mla_sched_meta_args_t", "SchedMetaArgs"), ("mla_dense_decode_args_t", "DenseDecodeArgs"),
    ("mla_sparse_decode_args_t", "SparseDecodeArgs"), ("mla_combine_args_t", "CombineArgs"),
    ("mla_sparse_prefill_args_t", "SparsePrefillArgs"),
])
def test_ctypes_structs_match_header(cname, pyname):
    from flashmla_b200 import _capi
    cfields = _struct_fields(cname)
    pyfields = getattr(_capi, pyname)._fields_
    assert [f[0] for f in cfields] == [f[0] for f in pyfields]
    cmap = {"int32_t": ctypes.c_int32, "int64_t": ctypes.c_int64, "float": ctypes.c_float, "ptr": ctypes.c_void_p}
    for (n, ct), (_, pt) in zip(cfields, pyfields):
        assert cmap[ct] is pt, (n, ct, pt)


def test_invalid_arguments_are_reported_without_a_gpu():
    from flashmla_b200 import _capi
    lib = _capi.lib()
    a = _capi.SchedMetaArgs(b=0, num_sm_parts=4, block_size_n=64, fixed_overhead_num_blocks=5, topk=-1)
    assert lib.mla_get_sched_meta(a) == 1
    assert b"batch size" in lib.mla_last_error()
    c = _capi.CombineArgs(b=1, s_q=1, h_q=1, d_v=256)
    assert lib.mla_combine(c) == 1 and b"d_v" in lib.mla_last_error()
    d = _capi.DenseDecodeArgs(b=1, s_q=1, h_q=8, h_kv=1, d_qk=512, d_v=512)
    assert lib.mla_dense_decode_fwd(d) == 1 and b"576" in lib.mla_last_error()
    assert lib.mla_dense_decode_fwd(None) == 1


def test_api_mirrors_reference_misuse_checks():
    import flashmla_b200 as fm
    meta, none = fm.get_mla_metadata(torch.zeros(3), 128, 1)      # old-style positional arguments are ignored
    assert isinstance(meta, fm.FlashMLASchedMeta) and none is None and not meta.have_initialized
    q = torch.zeros(2, 1, 8, 576, dtype=torch.bfloat16)
    k = torch.zeros(4, 64, 1, 576, dtype=torch.bfloat16)
    bt = torch.zeros(2, 2, dtype=torch.int32)
    sl = torch.zeros(2, dtype=torch.int32)
    with pytest.raises(AssertionError, match="must be of type FlashMLASchedMeta"):
        fm.flash_mla_with_kvcache(q, k, bt, sl, 512, None)
    with pytest.raises(AssertionError, match="num_splits must be None"):
        fm.flash_mla_with_kvcache(q, k, bt, sl, 512, meta, torch.zeros(1))
    with pytest.raises(AssertionError, match="causal must be False"):
        fm.flash_mla_with_kvcache(q, k, None, None, 512, fm.get_mla_metadata()[0], None, None, True, True,
                                  torch.zeros(2, 1, 64, dtype=torch.int32))
    with pytest.raises(AssertionError, match="is_fp8_kvcache must be True"):
        fm.flash_mla_with_kvcache(q, k, None, None, 512, fm.get_mla_metadata()[0], None, None, False, False,
                                  torch.zeros(2, 1, 64, dtype=torch.int32))
    with pytest.raises(AssertionError, match="block_table and cache_seqlens must be provided"):
        fm.flash_mla_with_kvcache(q, k, None, None, 512, fm.get_mla_metadata()[0])
    # no CPU path: CPU tensors are refused loudly
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fm.flash_mla_with_kvcache(q, k, bt, sl, 512, fm.get_mla_metadata()[0])
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        fm.flash_mla_sparse_fwd(torch.zeros(2, 8, 576, dtype=torch.bfloat16), torch.zeros(9, 1, 576, dtype=torch.bfloat16),
                                torch.zeros(2, 1, 64, dtype=torch.int32), 0.1)
    # re-using a sched_meta with a different shape trips the reference's consistency assertion
    m = fm.get_mla_metadata()[0]
    m.have_initialized = True
    m.config = fm.FlashMLASchedMeta.Config(3, 1, 8, 64, 1, False, False, None, None, None)
    with pytest.raises(AssertionError, match="sched_meta.config.b must be equal to batch_size"):
        fm.flash_mla_with_kvcache(q, k, bt, sl, 512, m)


def test_workspace_bytes():
    """Host-only sizing of the split-KV scratch (no device is touched)."""
    from flashmla_b200 import _capi
    lib = _capi.lib()
    off = ctypes.c_size_t(0)
    total = lib.mla_workspace_bytes(128, 1, 128, 512, 74, ctypes.byref(off))
    rows = (128 + 74) * 128
    assert off.value == rows * 512 * 4 and off.value % 256 == 0
    assert total == off.value + rows * 4
    total = lib.mla_workspace_bytes(3, 2, 5, 512, 7, ctypes.byref(off))       # an odd row count: the LSE part stays 256-byte aligned
    rows = (3 + 7) * 2 * 5
    assert off.value >= rows * 512 * 4 and off.value % 256 == 0 and total == off.value + rows * 4
    assert lib.mla_workspace_bytes(0, 1, 128, 512, 74, None) == 0 and b"positive" in lib.mla_last_error()
