#!/usr/bin/env python
"""Benchmark of the MLA decode / sparse-prefill path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" is one pass of the public API call over one batch of synthetic input.  The default workload is
dense BF16 MLA decode at the DeepSeek-V3 serving shape (batch 128 per GPU, h_q 128, mean sequence length
4096, s_q 1); rank 0 prints ONE JSON line.  For N > 1 launch with torch.distributed.run: every rank runs its
own batch on its own GPU (batch-sharded replicas, no collective on the data path), time is the maximum
over ranks and `value` the aggregate over all GPUs.

A pass takes a fraction of a millisecond, so every one of the K timed steps replays the pass R times back to back
(R chosen so that a step lasts about 20 ms) between one pair of CUDA events and reports elapsed / R.

--impl reference times the reference's torch attention on the host cores on a bounded sample of the same workload:
the CPU restatement under oracle/, or the unmodified function of a FlashMLA checkout when FLASHMLA_REFERENCE_DIR
names one.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

D_QK, D_V = 576, 512
# acceptance bounds of the benchmark specification (the same numbers as tests/helpers.py)
OUT_COS_TOL, OUT_ABS_TOL, LSE_TOL = 1e-5, 2e-2, 1e-3
TARGET_STEP_MS = 20.0
L2_NOTE = "KV cache (> L2) streamed once per pass; q/out may stay in L2 between replays, see ms_per_step_cold_l2"


# ------------------------------------------------------------------------------------------------------
# workloads: inputs + algorithmic bytes / flops (conventions of the reference's own test scripts:
# tests/test_flash_mla_dense_decoding.py:174-190, tests/lib.py:345-402)
# ------------------------------------------------------------------------------------------------------
def shard_of_rank(n_total, world, rank):
    """Requests [begin, end) of the batch-sharded sweep that `rank` of `world` serves (equal shares, no overlap)."""
    per = n_total // world
    return rank * per, (rank + 1) * per


def balanced_shard(seqlens, world, rank):
    """Indices of the requests `rank` of `world` serves when the router balances KV tokens: requests sorted by length are
    dealt to the ranks in serpentine order (0..world-1, world-1..0, ...), so every rank gets the same number of requests
    and nearly the same number of tokens, whatever the length distribution."""
    order = torch.argsort(seqlens.to(torch.int64), descending=True, stable=True)
    pos = torch.arange(order.numel())
    lap, k = pos // world, pos % world
    owner = torch.where(lap % 2 == 0, k, world - 1 - k)
    return torch.sort(order[owner == rank]).values


def reduce_over_ranks(ms_total, ms_e2e_total, units, tokens, flops, nbytes, dist, device):
    """Whole-job figures from per-rank ones: times are the MAXIMUM over ranks (the job is as slow as its slowest
    rank), work is the SUM.  `dist` is torch.distributed (any backend) or None for a single process."""
    if dist is None:
        return ms_total, ms_e2e_total, units, tokens, flops, nbytes
    stats = torch.tensor([ms_total, ms_e2e_total, units, tokens, flops, nbytes], dtype=torch.float64, device=device)
    mx = stats.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = stats.clone()
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    return float(mx[0]), float(mx[1]), float(sm[2]), float(sm[3]), float(sm[4]), float(sm[5])


def max_over_ranks(values, dist, device):
    if dist is None:
        return list(values)
    t = torch.tensor(list(values), dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t]


def make_workload(name, device, seed, prefill_sq=4096):
    from tests import workloads as W
    if name in ("dense", "dense_sq2"):
        s_q = 2 if name == "dense_sq2" else 1
        b, h_q = 128, 128
        seq = W.seqlens_normal(b, 4096, 512, 1, 8192, True, seed)
        d = W.dense_decode_inputs(seq, s_q, h_q, 1, seed=seed, device=device, data_on_device=True)
        S = int(seq.sum())
        return dict(kind="dense", inputs=d, s_q=s_q, b=b, h_q=h_q, tokens=S,
                    bytes=S * D_QK * 2 + b * s_q * h_q * D_QK * 2 + b * s_q * h_q * D_V * 2,
                    flops=2.0 * h_q * s_q * S * (D_QK + D_V),
                    desc=f"dense bf16 MLA decode b={b} h_q={h_q} h_kv=1 s_q={s_q} seqlens~N(4096,512^2) clip[1,8192] one=8192 causal paged(64)")
    if name == "longctx":
        b_total, h_q = 1024, 128
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        seq_all = W.seqlens_lognormal(b_total, 8192, 1.0, 256, 131072, seed=0)
        mine = balanced_shard(seq_all, world, rank)
        per = mine.numel()
        seq = seq_all[mine].contiguous()
        d = W.dense_decode_inputs(seq, 1, h_q, 1, seed=seed, device=device, data_on_device=True)
        S = int(seq.sum())
        return dict(kind="dense", inputs=d, s_q=1, b=per, h_q=h_q, tokens=S,
                    bytes=S * D_QK * 2 + per * h_q * D_QK * 2 + per * h_q * D_V * 2,
                    flops=2.0 * h_q * S * (D_QK + D_V),
                    desc=f"dense bf16 MLA decode b={b_total} total (batch-sharded, token-balanced) h_q=128 s_q=1 seqlens lognormal(median 8192, sigma 1) clip[256,131072]")
    if name in ("sparse_decode", "sparse_decode_m1"):
        # (_m1: the 512-wide "MODEL1" form - 584-byte records with e8m0 scales, d_qk = 512 - a side measurement)
        m1 = name == "sparse_decode_m1"
        d_qk, rec = (512, 584) if m1 else (D_QK, 656)
        b, h_q, s_kv, topk = 64, 128, 32768, 2048
        d = W.sparse_decode_inputs(b, 1, h_q, s_kv, topk, seed=seed, device=device, data_on_device=True, model1=m1)
        valid = b * d["n_valid"]
        return dict(kind="sparse_decode", inputs=d, s_q=1, b=b, h_q=h_q, tokens=valid, d_qk=d_qk,
                    bytes=valid * rec + b * h_q * d_qk * 2 + b * h_q * D_V * 2,
                    flops=2.0 * h_q * valid * (d_qk + D_V),
                    flops_padded=2.0 * h_q * b * topk * (d_qk + D_V),      # the reference's convention counts the -1 slots too
                    desc=f"sparse fp8 MLA decode b={b} h_q={h_q} s_kv={s_kv} topk={topk} (5% padded -1) " +
                         ("584B records (d_qk 512) e8m0 scales" if m1 else "656B records scale=amax/448"))
    if name == "sparse_prefill":
        s_q, h_q, s_kv, topk = prefill_sq, 128, 32768, 2048
        d = W.sparse_prefill_inputs(s_q, h_q, s_kv, topk, causal_base=28672, seed=seed, device=device, data_on_device=True)
        valid = s_q * topk
        return dict(kind="sparse_prefill", inputs=d, s_q=s_q, b=1, h_q=h_q, tokens=valid,
                    bytes=s_kv * D_QK * 2 + 4 * s_q * topk + s_q * h_q * (D_QK + D_V) * 2,
                    flops=2.0 * valid * h_q * (D_QK + D_V),
                    desc=f"token-sparse MLA prefill s_q={s_q} h_q={h_q} s_kv={s_kv} topk={topk} causal-valid indices")
    raise SystemExit(f"unknown workload {name}")


def config_of(w):
    """The `config` object of the JSON line: what is measured, identical for both arms."""
    return {"workload": w["desc"], "per_gpu_batch": w["b"], "l2": L2_NOTE}


def run_step(w, sm_scale=None):
    """One pass through the public API on device-resident inputs."""
    import flashmla_b200 as fm
    d = w["inputs"]
    if sm_scale is None:
        sm_scale = w.get("d_qk", D_QK) ** -0.5
    if w["kind"] == "dense":
        out, lse = fm.flash_mla_with_kvcache(d["q"], d["blocked_k"], d["block_table"], d["cache_seqlens"], D_V, w["meta"], None, sm_scale, True)
    elif w["kind"] == "sparse_decode":
        out, lse = fm.flash_mla_with_kvcache(d["q"], d["kv_fp8"], None, None, D_V, w["meta"], None, sm_scale, False, True, d["indices"])
    else:
        out, _, lse = fm.flash_mla_sparse_fwd(d["q"], d["kv"], d["indices"], sm_scale)
    return out, lse


def make_host_buffers(w):
    d = w["inputs"]
    pin = lambda t: t.detach().cpu().contiguous().pin_memory()
    host = {"q": pin(d["q"])}
    if w["kind"] == "dense":
        host["block_table"] = pin(d["block_table"])
        host["cache_seqlens"] = pin(d["cache_seqlens"])
    else:
        host["indices"] = pin(d["indices"])
    out, lse = run_step(w)
    torch.cuda.synchronize()
    host["out"] = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    host["lse"] = torch.empty(lse.shape, dtype=lse.dtype).pin_memory()
    h2d = sum(v.numel() * v.element_size() for k, v in host.items() if k not in ("out", "lse"))
    d2h = host["out"].numel() * host["out"].element_size() + host["lse"].numel() * host["lse"].element_size()
    return host, h2d, d2h


class E2EPipeline:
    """End-to-end passes through the public API with host buffers: every pass copies its inputs from pinned host memory
    to the device, runs the API call (for dense decode including a new schedule: the sequence lengths are new) and
    reads its result back into pinned host memory.  Consecutive passes are independent, so SLOTS of them are in flight
    at once, each on its own stream with its own device input and host output buffers: the copy engines of both
    directions and the SMs work at the same time, as in a serving loop that prepares the next batch while the current
    one runs.  One pass per slot is captured in a CUDA graph (copies, schedule, kernels) so that the host thread's
    per-call overhead stays off the clock; if capture is not possible the same sequence is issued call by call.
    With compute=False only the copies run (the same bytes, no kernel): the ceiling the host link sets for this figure."""
    SLOTS = 3

    def __init__(self, w, host, compute=True):
        self.w, self.host, self.compute = w, host, compute
        dev = w["inputs"]["q"].device
        self.streams = [torch.cuda.Stream(dev) for _ in range(self.SLOTS)]
        self.keys = [k for k in host if k not in ("out", "lse")]
        self.dev_in = [{k: torch.empty_like(host[k], device=dev) for k in self.keys} for _ in range(self.SLOTS)]
        self.host_out = [{k: torch.empty_like(host[k]).pin_memory() for k in ("out", "lse")} for _ in range(self.SLOTS)]
        self.dev_out = {k: torch.empty_like(host[k], device=dev) for k in ("out", "lse")} if not compute else None
        self.done = [None] * self.SLOTS
        self.keep = [None] * self.SLOTS
        self.graphs = None
        self.mode = "call by call"
        try:
            graphs = []
            for slot in range(self.SLOTS):
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self.streams[slot]):
                    self.keep[slot] = self._one_pass(slot)
                graphs.append(g)
            self.graphs = graphs
            self.mode = "one CUDA graph per slot (copies + schedule + kernels)"
        except Exception as exc:
            print(f"bench.py: end-to-end leg issued call by call ({exc})", file=sys.stderr)
            torch.cuda.synchronize()

    def _one_pass(self, slot):
        """host -> device, API call, device -> host; on the current stream."""
        import flashmla_b200 as fm
        w, d, x = self.w, self.w["inputs"], self.dev_in[slot]
        for k in self.keys:
            x[k].copy_(self.host[k], non_blocking=True)
        if not self.compute:
            out, lse = self.dev_out["out"], self.dev_out["lse"]
        elif w["kind"] == "dense":
            meta, _ = fm.get_mla_metadata()                    # the sequence lengths are new: the schedule is recomputed
            out, lse = fm.flash_mla_with_kvcache(x["q"], d["blocked_k"], x["block_table"], x["cache_seqlens"], D_V, meta,
                                                 None, D_QK ** -0.5, True)
        elif w["kind"] == "sparse_decode":
            out, lse = fm.flash_mla_with_kvcache(x["q"], d["kv_fp8"], None, None, D_V, w["meta"], None, w.get("d_qk", D_QK) ** -0.5,
                                                 False, True, x["indices"])
        else:
            out, _, lse = fm.flash_mla_sparse_fwd(x["q"], d["kv"], x["indices"], D_QK ** -0.5)
        self.host_out[slot]["out"].copy_(out, non_blocking=True)
        self.host_out[slot]["lse"].copy_(lse, non_blocking=True)
        return out, lse

    def step(self, i):
        slot = i % self.SLOTS
        if self.done[slot] is not None:
            self.done[slot].synchronize()          # the host has the result of pass i - SLOTS before its buffers are reused
        with torch.cuda.stream(self.streams[slot]):
            if self.graphs is not None:
                self.graphs[slot].replay()
            else:
                self.keep[slot] = self._one_pass(slot)
            self.done[slot] = torch.cuda.Event()
            self.done[slot].record()

    def run(self, steps):
        cur = torch.cuda.current_stream()
        for st in self.streams:
            st.wait_stream(cur)
        for i in range(steps):
            self.step(i)
        for st in self.streams:
            cur.wait_stream(st)

    def timed(self, steps, reps, barrier):
        """K steps, each `reps` pipelined passes between one event pair; returns the mean milliseconds per pass."""
        self.run(2 * self.SLOTS)
        barrier()
        total = 0.0
        for _ in range(steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            self.run(reps)
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1) / reps
        barrier()
        return total / steps


class KernelTimer:
    """Records a CUDA event pair around every kernel launch of the API (on the launching stream)."""

    def __init__(self):
        self.pairs = {}
        self._open = {}

    def start(self, name):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self._open[name] = e

    def stop(self, name):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pairs.setdefault(name, []).append((self._open.pop(name), e))

    def mean_ms(self):
        return {k: sum(a.elapsed_time(b) for a, b in v) / len(v) for k, v in self.pairs.items()}

    def launches(self):
        return sum(len(v) for v in self.pairs.values())


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=float(p["hbm_gbs"]), tflops=float(p["bf16_tflops"]), tflops_sustained=float(p["bf16_tflops_sustained"]),
                    source="measured")
    return dict(hbm=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def captured_traffic(workload):
    """DRAM bytes per launch of the workload's main kernel from the ncu capture summarised under profiles/
    (dram__bytes_read.sum + dram__bytes_write.sum); the small JSON beside the summary names the commit it was taken at."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    try:
        rec = json.load(open(path)).get(workload)
    except (OSError, ValueError):
        return None, None
    if not rec:
        return None, None
    return float(rec["dram_bytes_per_launch"]), rec.get("captured_at_commit")


def bind_to_gpu_numa_node(gpu_index):
    """Pins this process (and, by first touch, its pinned host buffers) to the cores nvidia-smi lists as closest to the
    GPU.  Read-only query; returns a short description for the JSON line."""
    try:
        txt = subprocess.run(["nvidia-smi", "topo", "-m"], capture_output=True, text=True, timeout=20).stdout
    except Exception as exc:
        return f"unbound ({type(exc).__name__})"
    header = None
    for ln in txt.splitlines():
        cols = [c.strip() for c in ln.split("\t") if c.strip() != ""]
        if not cols:
            continue
        if header is None and any("CPU Affinity" in c for c in cols):
            header = cols
            continue
        if header is not None and cols[0] == f"GPU{gpu_index}":
            # the row has one more leading cell (its own name) than the header has GPU/NIC columns
            try:
                aff = cols[1 + header.index("CPU Affinity")] if header[0] != "" else cols[header.index("CPU Affinity")]
            except (ValueError, IndexError):
                return "unbound (no affinity column)"
            cores = set()
            for part in aff.split(","):
                part = part.strip()
                if "-" in part:
                    a, b = part.split("-")
                    cores.update(range(int(a), int(b) + 1))
                elif part.isdigit():
                    cores.add(int(part))
            allowed = cores & set(os.sched_getaffinity(0))
            if not allowed:
                return f"unbound (affinity {aff} not available to this process)"
            os.sched_setaffinity(0, allowed)
            return f"cores {aff}"
    return "unbound (GPU row not found)"


# ------------------------------------------------------------------------------------------------------
# CPU arm: the reference's torch attention on the host cores, bounded sample.  Returns the checker's outputs too, so
# that the timed GPU result can be compared with them.
# ------------------------------------------------------------------------------------------------------
def _reference_dense_fn():
    """(function, kind): the unmodified reference_torch of a FlashMLA checkout named by FLASHMLA_REFERENCE_DIR
    (its tests/test_flash_mla_dense_decoding.py:73-141), else the restatement under oracle/."""
    ref_dir = os.environ.get("FLASHMLA_REFERENCE_DIR")
    if ref_dir and os.path.exists(os.path.join(ref_dir, "tests", "test_flash_mla_dense_decoding.py")):
        try:
            import types
            sys.modules.setdefault("flash_mla", types.ModuleType("flash_mla"))
            sys.path.insert(0, os.path.join(ref_dir, "tests"))
            import test_flash_mla_dense_decoding as ref_mod
            return (lambda q, kc, bt, sl, dv, causal: ref_mod.reference_torch(sl, bt, q, kc, dv, causal)), "reference"
        except Exception as exc:
            print(f"bench.py: FLASHMLA_REFERENCE_DIR is set but its test module does not import ({exc}); using oracle/", file=sys.stderr)
    from oracle import attention
    return attention.dense_decode, "port"


def cpu_baseline(w, budget_s=15.0, keep_outputs=False):
    from oracle import attention, quant
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    d = w["inputs"]
    outs = {}
    kind = "port"
    if w["kind"] == "dense":
        dense_fn, kind = _reference_dense_fn()
        b = w["b"]
        q, bt, sl = d["q"].cpu(), d["block_table"].cpu(), d["cache_seqlens"].cpu()
        done_tokens, t_used, n_req = 0, 0.0, 0
        for i in range(b):
            pages = bt[i, :(int(sl[i]) + 63) // 64].long()
            kv_i = d["blocked_k"][pages.to(d["blocked_k"].device)].cpu()
            bt_i = torch.arange(pages.numel(), dtype=torch.int32).view(1, -1)
            t0 = time.perf_counter()
            o, l = dense_fn(q[i:i + 1], kv_i, bt_i, sl[i:i + 1], D_V, True)
            t_used += time.perf_counter() - t0
            if keep_outputs:
                outs[i] = (o, l)
            done_tokens += int(sl[i])
            n_req += 1
            if t_used > budget_s:
                break
        frac = done_tokens / w["tokens"]
        name = "reference_torch of the FlashMLA checkout" if kind == "reference" else "oracle.attention.dense_decode"
        sample = f"{n_req} of {b} requests ({done_tokens} of {w['tokens']} KV tokens), {name}"
    elif w["kind"] == "sparse_decode":
        b = w["b"]
        t_used, n_req = 0.0, 0
        for i in range(b):
            idx = d["indices"][i:i + 1].cpu()
            pages = torch.unique(idx[idx >= 0] // 64)
            remap = torch.full((d["kv_fp8"].size(0),), -1, dtype=torch.int64)
            remap[pages.long()] = torch.arange(pages.numel())
            kv_raw = d["kv_fp8"][pages.to(d["kv_fp8"].device).long()].cpu().contiguous()
            idx_s = torch.where(idx >= 0, (remap[(idx.clamp_min(0) // 64).long()] * 64 + idx % 64).to(torch.int32), idx)
            qi = d["q"][i:i + 1].cpu()
            t0 = time.perf_counter()
            kv_deq = quant.dequantize_model1(kv_raw) if w.get("d_qk") == 512 else quant.dequantize_v32(kv_raw)
            o, l = attention.sparse_decode(qi, kv_deq, idx_s, w.get("d_qk", D_QK) ** -0.5, D_V)
            t_used += time.perf_counter() - t0
            if keep_outputs:
                outs[i] = (o, l)
            n_req += 1
            if t_used > budget_s:
                break
        frac = n_req / b
        sample = f"{n_req} of {b} requests, oracle.quant.dequantize_v32 (touched pages) + oracle.attention.sparse_decode"
    else:
        rows = 0
        t_used = 0.0
        q, kv, idx = d["q"], d["kv"].cpu(), d["indices"]
        while t_used < budget_s and rows < w["s_q"]:
            r1 = min(rows + 16, w["s_q"])
            qi, ii = q[rows:r1].cpu(), idx[rows:r1].cpu()
            t0 = time.perf_counter()
            o, _, l = attention.sparse_prefill(qi, kv, ii, D_QK ** -0.5, D_V, row_chunk=16)
            t_used += time.perf_counter() - t0
            if keep_outputs:
                for r in range(rows, r1):
                    outs[r] = (o[r - rows:r - rows + 1], l[r - rows:r - rows + 1])
            rows = r1
        frac = rows / w["s_q"]
        sample = f"{rows} of {w['s_q']} query rows, oracle.attention.sparse_prefill"
    return dict(seconds=t_used, frac=frac, cores=cores, sample=sample, kind=kind, outputs=outs)


def check_against_oracle(w, out, lse, oracle_outputs):
    """Compares the TIMED result (the output of the replayed graph) with the checker's outputs, unit by unit (request /
    query row); raises on the first unit outside the acceptance bounds.  Returns the number of units checked."""
    from oracle.compare import cos_diff, max_abs_err
    out_c, lse_c = out.detach().cpu(), lse.detach().cpu()
    for i, (o_ref, l_ref) in oracle_outputs.items():
        o, l = out_c[i:i + 1], lse_c[i:i + 1]
        cd = abs(cos_diff(o.float(), o_ref.float()))
        mae = max_abs_err(o, o_ref)
        fin = torch.isfinite(l_ref)
        le = float((l[fin] - l_ref[fin]).abs().max()) if fin.any() else 0.0
        if not (cd <= OUT_COS_TOL and mae <= OUT_ABS_TOL and le <= LSE_TOL and torch.equal(torch.isinf(l), torch.isinf(l_ref))):
            raise SystemExit(f"bench.py: the timed result of unit {i} is outside the acceptance bounds "
                             f"(cosine deficit {cd:.2e}, max abs {mae:.2e}, lse {le:.2e})")
    return len(oracle_outputs)


def metric_of(w):
    if w["kind"] == "sparse_prefill":
        return "mla_sparse_prefill_tflops", "TFLOP/s", w["flops"] / 1e12
    if w["kind"] == "sparse_decode":
        return "mla_sparse_decode_tflops", "TFLOP/s", w["flops"] / 1e12
    return "mla_dense_decode_hbm_gbs", "GB/s", w["bytes"] / 1e9


def side_measurements(dev):
    """The path's other workloads in short form (CUDA-graph replays of one pass: 6 cold-L2 passes first, while the part is
    not yet at its power limit, then 3 steps of about 20 ms), so that one default run carries a figure for every kernel of
    the path.  Parity of these workloads is the job of the GPU tests and of `--workload <name>` runs, which check the
    timed result against the oracle."""
    import flashmla_b200 as fm
    out = {}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for name in ("dense_sq2", "sparse_decode", "sparse_prefill"):
        w = make_workload(name, dev, seed=0)
        w["meta"] = fm.get_mla_metadata()[0]
        for _ in range(3):
            run_step(w)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            keep = run_step(w)
        for _ in range(3):
            graph.replay()
        scrub = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        cold = 0.0
        for i in range(7):                         # the first pass only warms the scrub buffer's own mapping
            scrub.fill_(1)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            if i:
                cold += e0.elapsed_time(e1)
        e0.record()
        for _ in range(5):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        reps = max(1, min(400, int(round(TARGET_STEP_MS / max(e0.elapsed_time(e1) / 5, 1e-3)))))
        total = 0.0
        for _ in range(3):
            e0.record()
            for _ in range(reps):
                graph.replay()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1) / reps
        ms = total / 3
        metric, unit, units = metric_of(w)
        out[name] = {"metric": metric, "value": units / (ms / 1e3), "unit": unit, "ms_per_step": ms, "ms_per_step_cold_l2": cold / 6,
                     "replays_per_step": reps, "tflops": w["flops"] / 1e12 / (ms / 1e3), "workload": w["desc"]}
        if "flops_padded" in w:
            out[name]["tflops_reference_convention"] = w["flops_padded"] / 1e12 / (ms / 1e3)
        del graph, keep, scrub, w
        torch.cuda.empty_cache()
    return out


def bench_quantize(args):
    """The cache-write kernel (bf16 token rows -> 656-byte FP8 records) on --quant-blocks (default 32768) blocks of 64 random rows: a side
    measurement of the step before sparse decode, one JSON line of its own."""
    from flashmla_b200.kvcache import quantize_fp8_kvcache, BYTES_PER_TOKEN
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    blocks = args.quant_blocks
    x = torch.randn(blocks, 64, 1, D_QK, device="cuda", dtype=torch.bfloat16)
    for _ in range(max(args.warmup, 3)):
        quantize_fp8_kvcache(x)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(args.steps):
        quantize_fp8_kvcache(x)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    ntok = blocks * 64
    peaks = measured_peaks()
    gbs = ntok * (2 * D_QK + BYTES_PER_TOKEN) / ms / 1e6
    print(json.dumps({"metric": "mla_quantize_fp8_kvcache_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16->e4m3", "data": "synthetic",
                      "config": {"workload": f"FP8 cache writer, {ntok} tokens of 576 bf16 -> 656-byte records (read + written bytes, > L2)"},
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"],
                                   "traffic": None, "peak_source": peaks["source"]}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense", choices=["dense", "dense_sq2", "longctx", "sparse_decode", "sparse_decode_m1", "sparse_prefill", "quantize"])
    ap.add_argument("--kernel", type=int, default=0, help="0 auto, 1 portable kernel, 2 tcgen05 kernel")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-side", action="store_true", help="leave out the short measurements of the other workloads (default workload, one GPU)")
    ap.add_argument("--replays", type=int, default=0, help="passes per timed step (0: as many as make a step last about 20 ms)")
    ap.add_argument("--quant-blocks", type=int, default=32768, help="64-token blocks of the quantize workload (smaller for profiler captures)")
    ap.add_argument("--prefill-sq", type=int, default=4096, help="query tokens of the sparse_prefill workload (smaller for profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.workload == "quantize":
        bench_quantize(args)
        return
    if args.impl == "reference":
        if rank != 0:
            return
        dev = "cuda:0" if torch.cuda.is_available() else "cpu"
        w = make_workload(args.workload, dev, seed=0, prefill_sq=args.prefill_sq)
        metric, unit, units_per_step = metric_of(w)
        # each "step" is one bounded sample of the workload on all host cores
        vals = []
        for i in range(args.warmup + args.steps):
            r = cpu_baseline(w, budget_s=6.0)
            if i >= args.warmup:
                vals.append(units_per_step * r["frac"] / r["seconds"])
        v = sum(vals) / len(vals)
        line = {"impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": 1e3 * units_per_step / v, "higher_is_better": True,
                "scaling": "strong" if args.workload == "longctx" else "weak",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config_of(w),
                "note": "the reference's torch attention on the host cores, bounded sample, extrapolated to a full step",
                "cpu_baseline": {"value": v, "unit": unit, "cores": r["cores"], "kind": r["kind"], "sample": r["sample"]},
                "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    import flashmla_b200 as fm
    from flashmla_b200 import flash_mla_interface as fmi
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = bind_to_gpu_numa_node(local_rank)          # before any pinned buffer is allocated
    os.environ.setdefault("OMP_NUM_THREADS", str(len(os.sched_getaffinity(0))))
    torch.set_num_threads(len(os.sched_getaffinity(0)))
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    fm.set_impl(args.kernel)

    w = make_workload(args.workload, dev, seed=rank, prefill_sq=args.prefill_sq)
    w["meta"] = fm.get_mla_metadata()[0]
    metric, unit, units_per_step = metric_of(w)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up, and how many passes make a step of about 20 ms (the same R on every rank) ----------------
    for _ in range(args.warmup):
        run_step(w)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        run_step(w)
    e1.record()
    torch.cuda.synchronize()
    est_ms = max_over_ranks([e0.elapsed_time(e1) / 5], dist, dev)[0]
    reps = args.replays if args.replays > 0 else max(1, min(400, int(round(TARGET_STEP_MS / max(est_ms, 1e-3)))))

    # ---- eager launches: K steps of R passes, with an event pair around every kernel of the first pass of a step ------
    timer = KernelTimer()
    barrier()
    ms_eager = 0.0
    with ClockSampler(local_rank) as clocks_eager:
        for _ in range(args.steps):
            fmi.set_kernel_timer(timer)
            run_step(w)                                            # per-kernel times (not part of the step's own clock)
            fmi.set_kernel_timer(None)
            e0.record()
            for _ in range(reps):
                run_step(w)
            e1.record()
            torch.cuda.synchronize()
            ms_eager += e0.elapsed_time(e1) / reps
        barrier()
    ms_eager /= args.steps
    kernel_ms = timer.mean_ms()
    launches_per_pass = timer.launches() // args.steps
    clocks = clocks_eager

    # ---- the same pass as a CUDA graph: captured once and replayed (a decode loop is launch-bound between its kernels;
    # the API neither allocates outside torch's allocator nor synchronises, so it can be captured) ----------------------
    ms_step, launch_mode = ms_eager, "eager launches"
    ms_cold = None
    kernel_ms_isolated = None
    g_out = g_lse = None
    try:
        eager_out, eager_lse = run_step(w)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            g_out, g_lse = run_step(w)
        for _ in range(3):
            graph.replay()
        barrier()
        total = 0.0
        with ClockSampler(local_rank) as clocks_graph:
            for _ in range(args.steps):
                e0.record()
                for _ in range(reps):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize()
                total += e0.elapsed_time(e1) / reps
            barrier()
        if not (torch.equal(g_out.view(torch.int16), eager_out.view(torch.int16)) and torch.equal(g_lse, eager_lse)):
            raise RuntimeError("graph replay and eager launch disagree")
        ms_step, launch_mode, clocks = total / args.steps, "CUDA graph replay of one pass", clocks_graph
        # the same pass with a cold L2: 512 MB are overwritten before every single timed replay (the method of the
        # reference's tests/kernelkit/bench.py:166-205)
        scrub = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        total = 0.0
        for _ in range(args.steps):
            scrub.fill_(1)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        ms_cold = total / args.steps
        # ... and every kernel of an isolated, cold-L2 pass on its own (eager launches with an event pair around each):
        # what the kernels take when the part is not yet held back by its power limit
        timer_iso = KernelTimer()
        for _ in range(args.steps):
            scrub.fill_(1)
            fmi.set_kernel_timer(timer_iso)
            run_step(w)
            fmi.set_kernel_timer(None)
            torch.cuda.synchronize()
        kernel_ms_isolated = timer_iso.mean_ms()
        del scrub
    except Exception as exc:                      # capture is an optimisation of the launch path, never a requirement
        print(f"bench.py: CUDA graph capture not used ({exc})", file=sys.stderr)
        g_out, g_lse = run_step(w)
        torch.cuda.synchronize()

    # ---- end-to-end timing: host buffers in, result out; and the copies alone ---------------------------------
    host, h2d, d2h = make_host_buffers(w)
    reps_e2e = max(1, min(reps, int(round(TARGET_STEP_MS / max(3 * est_ms, 1e-3)))))
    pipe = E2EPipeline(w, host)
    solo_ms = None
    if dist is not None:
        # rank 0 alone first (the others wait): what one GPU reaches when it has the host to itself
        if rank == 0:
            solo_ms = pipe.timed(max(3, args.steps // 4), reps_e2e, lambda: torch.cuda.synchronize())
        barrier()
    ms_e2e = pipe.timed(args.steps, reps_e2e, barrier)
    out_chk, lse_chk = run_step(w)                                  # the pipelined path returns the same result
    torch.cuda.synchronize()
    last = pipe.host_out[(reps_e2e - 1) % pipe.SLOTS]
    if not (torch.equal(last["out"].view(torch.int16), out_chk.cpu().view(torch.int16)) and torch.equal(last["lse"], lse_chk.cpu())):
        raise SystemExit("bench.py: the end-to-end leg returned a different result than the device-resident leg")
    ms_copy = E2EPipeline(w, host, compute=False).timed(max(3, args.steps // 2), reps_e2e, barrier)

    # ---- reduce over ranks ---------------------------------------------------------------------------------
    ms_step_all, ms_e2e_all, units_all, tokens_all, flops_all, bytes_all = reduce_over_ranks(
        ms_step, ms_e2e, units_per_step, float(w["tokens"]), w["flops"], float(w["bytes"]), dist, dev)
    ms_eager_all, ms_copy_all, ms_cold_all = max_over_ranks([ms_eager, ms_copy, ms_cold if ms_cold is not None else -1.0], dist, dev)
    if rank != 0:
        dist.destroy_process_group()
        return

    peaks = measured_peaks()
    main_kernel = {"dense": "mla_dense_decode_fwd", "sparse_decode": "mla_sparse_decode_fwd",
                   "sparse_prefill": "mla_sparse_prefill_fwd"}[w["kind"]]
    k_ms = kernel_ms[main_kernel]
    if w["kind"] == "dense":
        roof = {"bound": "hbm", "achieved": w["bytes"] / 1e9 / (k_ms / 1e3), "peak": peaks["hbm"], "unit": "GB/s"}
    else:
        roof = {"bound": "tensor", "achieved": w["flops"] / 1e12 / (k_ms / 1e3), "peak": peaks["tflops"], "unit": "TFLOP/s"}
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["timed"] = "inside the timed region: back-to-back passes, clocks as sampled (see clocks)"
    if kernel_ms_isolated is not None:
        # the same kernel launched alone after an L2 scrub (burst clocks): comparable with the burst peak figures
        k_iso = kernel_ms_isolated[main_kernel]
        ach = (w["bytes"] / 1e9 if w["kind"] == "dense" else w["flops"] / 1e12) / (k_iso / 1e3)
        roof["isolated"] = {"kernel_ms": k_iso, "achieved": ach, "frac": ach / roof["peak"]}
    if w["kind"] == "dense":
        # dense decode with 128 heads sits at the ridge: its arithmetic intensity is about 242 FLOP per cache byte, so the
        # tensor pipe's SUSTAINED peak (power-capped) bounds it at nearly the same point as the HBM peak does
        roof["tensor_frac_of_sustained_peak"] = (w["flops"] / 1e12 / (k_ms / 1e3)) / peaks["tflops_sustained"]
    traffic, traffic_commit = captured_traffic(args.workload) if world == 1 else (None, None)
    roof["traffic"] = traffic
    roof["traffic_captured_at_commit"] = traffic_commit
    roof["kernel"] = main_kernel
    roof["kernel_ms"] = k_ms
    roof["peak_source"] = peaks["source"]

    clk = clocks.summary()
    e2e = {"value": units_all / (ms_e2e_all / 1e3), "unit": unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": ms_e2e_all, "replays_per_step": reps_e2e,
           "pipelining": f"{E2EPipeline.SLOTS} passes in flight, each on its own stream with its own buffers; {pipe.mode}",
           "host_binding": numa,
           "copy_only": {"ms_per_step": ms_copy_all, "per_rank_gbs": (h2d + d2h) / 1e9 / (ms_copy_all / 1e3),
                         "aggregate_gbs": world * (h2d + d2h) / 1e9 / (ms_copy_all / 1e3),
                         "what": "the same host<->device copies with no kernel between them: the host link's ceiling for this figure"}}
    if solo_ms is not None:
        e2e["ms_per_step_rank0_alone"] = solo_ms
        e2e["e2e_efficiency_vs_n1"] = solo_ms / ms_e2e_all
    line = {
        "metric": metric, "value": units_all / (ms_step_all / 1e3), "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step_all, "higher_is_better": True,
        "scaling": "strong" if args.workload == "longctx" else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": config_of(w),
        "kernel": {0: "auto", 1: "portable", 2: "tcgen05"}[args.kernel], "launch": launch_mode, "replays_per_step": reps,
        "ms_per_step_eager": ms_eager_all,
        "ms_per_step_cold_l2": ms_cold_all if ms_cold_all >= 0 else None,
        "ms_x_sm_ghz": ms_step_all * clk["sm_mhz"] / 1e3 if clk["sm_mhz"] else None,
        "tflops": flops_all / 1e12 / (ms_step_all / 1e3), "hbm_gbs": bytes_all / 1e9 / (ms_step_all / 1e3),
        "kv_tokens_per_s": tokens_all / (ms_step_all / 1e3),
        "kernel_ms": kernel_ms, "kernel_ms_isolated_cold_l2": kernel_ms_isolated,
        "gpu_launches": launches_per_pass * reps * args.steps,
        "roofline": roof, "clocks": clk, "e2e": e2e,
    }
    if "flops_padded" in w:
        line["tflops_reference_convention"] = world * w["flops_padded"] / 1e12 / (ms_step_all / 1e3)
    if not args.no_cpu_baseline and world == 1:
        r = cpu_baseline(w, budget_s=12.0, keep_outputs=True)
        line["cpu_baseline"] = {"value": units_per_step * r["frac"] / r["seconds"], "unit": unit, "cores": r["cores"],
                                "kind": r["kind"], "sample": r["sample"]}
        # the result that was timed (the replayed graph's output) against the checker, unit by unit
        line["parity_checked"] = check_against_oracle(w, g_out, g_lse, r["outputs"])
        line["parity_bounds"] = {"out_cos_deficit": OUT_COS_TOL, "out_max_abs": OUT_ABS_TOL, "lse_abs": LSE_TOL}
    # (not with a forced replay count: that is how profiler captures keep the run short)
    if world == 1 and args.workload == "dense" and args.kernel == 0 and args.replays == 0 and not args.no_side:
        del g_out, g_lse
        w.clear()
        torch.cuda.empty_cache()
        try:
            line["side_workloads"] = side_measurements(dev)
        except Exception as exc:                  # a side measurement never takes the headline line with it
            line["side_workloads"] = {"error": str(exc)}
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
