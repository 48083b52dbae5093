#!/usr/bin/env python
"""Benchmark of the paged-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of the operator over one batch of seeded synthetic input
with the shape of a benchmark configuration.  The headline workload is the
chunked-prefill configuration (``cfg2``: Qwen3-8B shape, 4 sequences, cached
prefix U{0..4096} + a 512-token chunk, causal), reported in TFLOP/s; the same
JSON line carries the long-context decode configuration (``cfg5a``) in GB/s
under ``"decode"``.  Under torchrun every rank runs its own batch (weak
scaling, sharding by request: no collective on the data path); ``e2e`` at
N > 1 adds the NCCL all-gather that reassembles the outputs.

``value``       kernel-only throughput, inputs resident in HBM, CUDA events per step,
                L2 flushed between steps; max over ranks of the summed time.
``e2e``         the same metric through ``AttnBackend.forward`` with HOST buffers:
                pinned host -> device copies of q/k/v and metadata, K/V store,
                attention, device -> pinned host copy of the output, all timed.
``roofline``    algorithmic flops (or bytes) / mean kernel time against the measured peak.
``cpu_baseline``the CPU restatement (gather pages, fp32 SDPA) timed on the host cores.

``--impl reference`` times that CPU path alone (the reference's Metal kernels
need macOS and its MLX CPU path needs the ``mlx`` package, neither is
available here).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "paged decode HBM GB/s + prefill TFLOP/s vs roofline at 1/2/4/8 B200"
L2_FLUSH_BYTES = 256 << 20
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes per launch of the dominant kernel divided by the workload's algorithmic bytes, each
# from an ncu capture of that workload summarised under profiles/ (cfg4 and cfg5a were captured at a
# reduced batch and scale with the tokens read).  A workload without a capture reports no traffic.
TRAFFIC_PER_ALGORITHMIC_BYTE = {
    "cfg1": (1.00, "profiles/dram_traffic_cfg1_cfg3.md"),
    "cfg2": (0.83, "profiles/prefill_tc_kernel_cfg2.md"),
    "cfg3": (1.03, "profiles/dram_traffic_cfg1_cfg3.md"),
    "cfg4": (1.02, "profiles/prefill_tc_kernel_cfg4_batch8.md"),
    "cfg5a": (1.005, "profiles/decode_partial_kernel_cfg5a_batch16.md"),
}


def traffic_of(w):
    """(bytes per launch, source) from the capture of this workload, or (None, None)."""
    key = w.name.split("_")[0]
    if key not in TRAFFIC_PER_ALGORITHMIC_BYTE or INDEX != "page":
        return None, None
    ratio, source = TRAFFIC_PER_ALGORITHMIC_BYTE[key]
    return ratio * w.algorithmic_bytes(), source


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ----------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    _NAMES = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
              0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in self._NAMES.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ----------------------------------------------------------------------------- workloads
BATCH_OVERRIDE = None  # --batch: smaller batch of the same configuration (profiling captures)
INDEX = "page"         # --index: "page" = one id per 16-token page (the *_p16 operators, K/V tiles
                       # fetched as TMA boxes); "token" = the reference's per-token slot ids


def make_workload(name: str, device, rank: int):
    w = _make_workload(name, device, rank)
    w.index = INDEX
    if INDEX == "page":
        w.page_indptr, w.page_indices, w.kv_lens_dev = w.page_csr()
    return w


def _make_workload(name: str, device, rank: int):
    from mini_sglang_mlx_b200 import synthetic as S
    seed_shift = 0 * rank  # every rank runs the same batch shape and lengths: fixed work per GPU
    kw = {} if BATCH_OVERRIDE is None else {"batch": BATCH_OVERRIDE}
    if name == "cfg1":
        from mini_sglang_mlx_b200.attention import compute_num_kv_splits
        w = S.cfg1_decode(seed=101 + seed_shift, device=device, **kw)
        splits = compute_num_kv_splits(w.kv_lens, w.hkv)
        w.num_kv_splits = torch.tensor(splits, dtype=torch.int32, device=device)
        w.max_kv_splits = max(splits)      # the launch grid: no more split slots than any sequence uses
        return w
    if name == "cfg2":
        return S.cfg2_prefill(seed=202 + seed_shift, device=device, **kw)
    if name == "cfg3":
        return S.cfg3_window_block(seed=303 + seed_shift, device=device, **kw)
    if name == "cfg4":
        return S.cfg4_verify(seed=404 + seed_shift, device=device, **kw)
    if name == "cfg5a":
        from mini_sglang_mlx_b200.attention import compute_num_kv_splits
        w = S.cfg5a_decode(seed=505 + seed_shift, device=device, **kw)
        splits = compute_num_kv_splits(w.kv_lens, w.hkv)
        w.num_kv_splits = torch.tensor(splits, dtype=torch.int32, device=device)
        w.max_kv_splits = max(splits)
        return w
    if name.startswith("cfg5b"):
        _, c, p = name.split("_")
        return S.cfg5b_prefill_point(int(c), int(p), seed=606 + seed_shift, device=device)
    if name.startswith("d256p_"):   # head_dim 256 prefill: d256p_<kv heads>_<q heads>_<q len>[_<prefix>]
        f = [int(x) for x in name.split("_")[1:]]
        return S.d256_prefill_point(f[0], f[1], f[2], f[3] if len(f) > 3 else 0, device=device)
    if name.startswith("d256d_"):   # head_dim 256 decode: d256d_<kv heads>_<q heads>_<kv len>[_<batch>]
        from mini_sglang_mlx_b200.attention import compute_num_kv_splits
        f = [int(x) for x in name.split("_")[1:]]
        w = S.d256_decode_point(f[0], f[1], f[2], f[3] if len(f) > 3 else 1, device=device)
        splits = compute_num_kv_splits(w.kv_lens, w.hkv)
        w.num_kv_splits = torch.tensor(splits, dtype=torch.int32, device=device)
        w.max_kv_splits = max(splits)
        return w
    raise SystemExit(f"unknown workload {name}")


def run_op(w):
    from mini_sglang_mlx_b200 import (paged_decode_attention, paged_decode_attention_p16,
                                      paged_prefill_attention, paged_prefill_attention_p16)
    if w.index == "page":
        if w.kind == "decode":
            return paged_decode_attention_p16(w.q, w.k_cache, w.v_cache, w.page_indptr, w.page_indices,
                                              w.kv_lens_dev, w.num_kv_splits, w.sm_scale, w.max_kv_splits)
        return paged_prefill_attention_p16(w.q, w.k_cache, w.v_cache, w.qo_indptr, w.page_indptr,
                                           w.page_indices, w.kv_lens_dev, w.prefix_lens, w.sm_scale,
                                           w.max_len_extend, is_cross_attention=w.is_cross_attention,
                                           sliding_window_size=w.sliding_window_size)
    if w.kind == "decode":
        return paged_decode_attention(w.q, w.k_cache, w.v_cache, w.kv_indptr, w.kv_indices,
                                      w.num_kv_splits, w.sm_scale, w.max_kv_splits)
    return paged_prefill_attention(w.q, w.k_cache, w.v_cache, w.qo_indptr, w.kv_indptr, w.kv_indices,
                                   w.prefix_lens, w.sm_scale, w.max_len_extend,
                                   is_cross_attention=w.is_cross_attention,
                                   sliding_window_size=w.sliding_window_size)


def launches_per_step(w) -> int:
    """Kernels of this library per operator call.  Decode: one (its key-range splits are merged
    by the CTA that finishes last).  Prefill: one, or two when the splits of a large (sequence,
    query tile, head) unit are merged by a second, dependent launch; the library says which."""
    if w.kind == "decode":
        return 1
    from mini_sglang_mlx_b200 import _lib
    return int(_lib.lib().msgl_prefill_launch_count(
        w.batch, int(w.q.shape[0]), int(sum(w.kv_lens)), w.hq, w.hkv, w.head_dim,
        int(w.max_len_extend), int(w.sliding_window_size), 1 if w.index == "page" else 0))


def barrier(dist_on: bool):
    if dist_on:
        torch.distributed.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, dist_on: bool) -> float:
    if not dist_on:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
    return float(t.item())


GRAPH_REPLAY = False  # --graph: the operator call captured once in a CUDA graph, steps replay it


def time_kernel_steps(w, steps: int, warmup: int, dist_on: bool, flush):
    """Sum of per-step device times (ms) of `steps` operator calls, L2 flushed before each."""
    call = lambda: run_op(w)  # noqa: E731
    if GRAPH_REPLAY:
        # warm the op (workspace, attributes) on a side stream, then capture one call; a replay
        # puts the op's launches on the stream without the host-side launch path
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                run_op(w)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            run_op(w)
        call = graph.replay
    return _time_calls(call, steps, warmup, dist_on, flush)


def _time_calls(run, steps: int, warmup: int, dist_on: bool, flush):
    for _ in range(warmup):
        flush.zero_()
        run()
    barrier(dist_on)
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps)]
    for i in range(steps):
        flush.zero_()
        starts[i].record()
        run()
        ends[i].record()
    barrier(dist_on)
    per = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    return sum(per), per


# ----------------------------------------------------------------------------- end to end
class _ModelCfg:
    def __init__(self, w):
        self.head_dim, self.num_kv_heads, self.num_qo_heads = w.head_dim, w.hkv, w.hq


def build_e2e(w, device):
    """A one-layer pool holding the workload's KV, a per-token slot table, the requests, and
    pinned host buffers with this step's q/k/v."""
    from mini_sglang_mlx_b200.attention import AttnBackend
    from mini_sglang_mlx_b200.core import Batch, BatchPhase, Req
    from mini_sglang_mlx_b200.kvcache import MHAKVCache
    num_slots = w.k_cache.shape[0]
    pool = MHAKVCache.__new__(MHAKVCache)
    # adopt the workload's tensors as layer 0 of the pool (no second copy of a 38 GB pool)
    pool._num_layers, pool._dtype = 1, w.k_cache.dtype
    pool._storage_shape = tuple(w.k_cache.shape)
    pool._k_buffer, pool._v_buffer = [w.k_cache], [w.v_cache]
    max_len = max(w.kv_lens)
    table = torch.zeros((w.batch, max_len), dtype=torch.int32, device=device)
    indptr = w.kv_indptr.tolist()
    for b in range(w.batch):
        table[b, : w.kv_lens[b]] = w.kv_indices[indptr[b]:indptr[b + 1]]
    be = AttnBackend(_ModelCfg(w), pool, table, page_size=16 if INDEX == "page" else 1)
    if w.kind == "decode":
        reqs = [Req(table_idx=b, cached_len=w.kv_lens[b] - 1, device_len=w.kv_lens[b]) for b in range(w.batch)]
        phase = BatchPhase.DECODE
    else:
        reqs = [Req(table_idx=b, cached_len=w.kv_lens[b] - w.q_lens[b], device_len=w.kv_lens[b])
                for b in range(w.batch)]
        phase = BatchPhase.PREFILL
    out_loc = torch.cat([table[r.table_idx, r.cached_len:r.device_len] for r in reqs]).contiguous()
    n = out_loc.numel()
    # q, k, v and the slot ids of a step sit back to back in ONE pinned staging buffer (and one
    # device buffer per pipeline stage), so a step's inputs cross PCIe as a single copy: four
    # separate copies of the same bytes took 0.73 ms against 0.53 ms on this hardware.
    parts = dict(q=w.q, k=w.k_cache[out_loc.long()], v=w.v_cache[out_loc.long()], out_loc=out_loc)
    offs, total = {}, 0
    for key, t in parts.items():
        offs[key] = total
        total += (t.numel() * t.element_size() + 255) // 256 * 256

    def views(buf):
        return {key: buf[offs[key]: offs[key] + t.numel() * t.element_size()].view(t.dtype).view(t.shape)
                for key, t in parts.items()}

    staging = torch.empty(total, dtype=torch.uint8).pin_memory()
    host = views(staging)
    for key, t in parts.items():
        host[key].copy_(t.cpu())
    host["staging"] = staging
    host["out"] = [torch.empty(w.q.shape, dtype=w.q.dtype).pin_memory() for _ in range(2)]
    dev = []
    for _ in range(2):
        buf = torch.empty(total, dtype=torch.uint8, device=device)
        d = views(buf)
        d["staging"] = buf
        dev.append(d)
    batch = Batch(reqs=reqs, phase=phase)
    return be, batch, host, dev


def e2e_bytes(w, host, batch):
    md = 4 * (3 * (w.batch + 1) + 2 * w.batch)  # pointer arrays, table ids, prefix lens / splits
    bi = sum(host[k].numel() * host[k].element_size() for k in ("q", "k", "v", "out_loc")) + md
    bo = host["out"][0].numel() * host["out"][0].element_size()
    return bi, bo


class E2EPipeline:
    """The serving-side call pattern: every step copies its q/k/v and slot ids from pinned host
    memory, runs ``AttnBackend.prepare_metadata`` + ``forward`` (K/V store, attention) and copies
    the output back to pinned host memory.  Copies and compute of neighbouring steps overlap on
    three streams with double-buffered device inputs and host outputs; the caller takes the
    result of step i-1 (a host-side wait) before it submits step i+1."""

    def __init__(self, w, be, batch, host, dev, gather):
        self.w, self.be, self.batch, self.host, self.dev, self.gather = w, be, batch, host, dev, gather
        self.s_in, self.s_run, self.s_out, self.s_gather = (torch.cuda.Stream() for _ in range(4))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]
        self.ev_run = [torch.cuda.Event() for _ in range(2)]
        self.ev_gather = [torch.cuda.Event() for _ in range(2)]
        self.ev_out = [torch.cuda.Event() for _ in range(2)]
        self.i = 0

    def step(self):
        w, k = self.w, self.i % 2
        if self.i >= 2:
            self.ev_out[k].synchronize()          # the caller has read the result of step i-2
        with torch.cuda.stream(self.s_in):
            if self.i >= 2:
                self.s_in.wait_event(self.ev_run[k])   # step i-2 no longer reads these inputs
            self.dev[k]["staging"].copy_(self.host["staging"], non_blocking=True)   # q, k, v, slot ids
            self.ev_in[k].record(self.s_in)
        with torch.cuda.stream(self.s_run):
            self.s_run.wait_event(self.ev_in[k])
            self.batch.out_loc = self.dev[k]["out_loc"]
            self.be.prepare_metadata(self.batch)
            out = self.be.forward(self.dev[k]["q"], self.dev[k]["k"], self.dev[k]["v"], 0, self.batch,
                                  is_cross_attention=w.is_cross_attention,
                                  sliding_window_size=w.sliding_window_size)
            self.ev_run[k].record(self.s_run)
        if self.gather is not None:
            # the reassembly of the ranks' outputs runs on a stream of its own, so that the next
            # step's store and attention do not queue behind the collective
            with torch.cuda.stream(self.s_gather):
                self.s_gather.wait_event(self.ev_run[k])
                out.record_stream(self.s_gather)
                out = self.gather(out)
                self.ev_gather[k].record(self.s_gather)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.ev_gather[k] if self.gather is not None else self.ev_run[k])
            out.record_stream(self.s_out)
            self.host["out"][k].copy_(out[: self.host["out"][k].shape[0]], non_blocking=True)
            self.ev_out[k].record(self.s_out)
        self.i += 1

    def drain(self):
        for s in (self.s_in, self.s_run, self.s_gather, self.s_out):
            s.synchronize()

    def copy_floor_ms(self, steps: int, dist_on: bool) -> float:
        """Per-step time of the bare staging copies alone (this step's inputs host -> device, the
        output device -> host, on their two streams, nothing else running), all ranks at once:
        what the end-to-end step cannot go below on this host."""
        out_dev = torch.empty_like(self.host["out"][0], device=self.dev[0]["staging"].device)
        barrier(dist_on)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record(self.s_in)
        self.s_out.wait_event(start)
        for i in range(steps):
            with torch.cuda.stream(self.s_in):
                self.dev[i % 2]["staging"].copy_(self.host["staging"], non_blocking=True)
            with torch.cuda.stream(self.s_out):
                self.host["out"][i % 2].copy_(out_dev, non_blocking=True)
        self.s_in.wait_stream(self.s_out)
        end.record(self.s_in)
        self.drain()
        barrier(dist_on)
        return start.elapsed_time(end) / steps


def bind_near_gpu(index: int):
    """Restrict this process to the CPUs NVML names as local to GPU `index` (those among the
    CPUs it may use), so that the pinned staging buffers allocated next are placed on the
    GPU's NUMA node.  Returns (previous affinity, note); the caller restores the affinity."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        allowed = os.sched_getaffinity(0)
        words = pynvml.nvmlDeviceGetCpuAffinity(handle, (max(allowed) + 64) // 64)
        near = {64 * i + b for i, word in enumerate(words) for b in range(64) if (int(word) >> b) & 1}
        cpus = near & allowed
        if not cpus or cpus == allowed:
            return None, "all usable CPUs are equally near" if cpus else "no usable CPU near the GPU"
        os.sched_setaffinity(0, cpus)
        return allowed, f"{len(cpus)} of {len(allowed)} CPUs"
    except Exception as e:  # noqa: BLE001
        return None, f"unavailable ({type(e).__name__})"


NUMA_NOTE = None


def time_e2e(w, device, steps, warmup, dist_on, world):
    global NUMA_NOTE
    previous, NUMA_NOTE = bind_near_gpu(device.index)
    try:
        return _time_e2e(w, device, steps, warmup, dist_on, world)
    finally:
        if previous is not None:
            os.sched_setaffinity(0, previous)


def _time_e2e(w, device, steps, warmup, dist_on, world):
    be, batch, host, dev = build_e2e(w, device)
    gather = None
    if dist_on and world > 1:
        def gather(out):
            full = out.new_empty((world * out.shape[0], *out.shape[1:]))
            torch.distributed.all_gather_into_tensor(full, out.contiguous())
            return full
    pipe = E2EPipeline(w, be, batch, host, dev, gather)
    for _ in range(warmup):
        pipe.step()
    pipe.drain()
    barrier(dist_on)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(pipe.s_in)
    for _ in range(steps):
        pipe.step()
    pipe.drain()
    end.record(pipe.s_out)
    barrier(dist_on)
    ms = start.elapsed_time(end)
    bi, bo = e2e_bytes(w, host, batch)
    floor = pipe.copy_floor_ms(steps, dist_on)
    return ms, bi, bo, floor


# ----------------------------------------------------------------------------- CPU baseline
def cpu_units(w):
    """(sequence, kv head) pairs: the unit the CPU path is sampled in."""
    return [(b, h) for b in range(w.batch) for h in range(w.hkv)]


def cpu_run_units(wc, units):
    """The CPU restatement (gather pages -> fp32 SDPA with the explicit mask) on some units.
    Returns the flops it performed."""
    from oracle import paged_attention_oracle as O
    g = wc.hq // wc.hkv
    flops = 0
    W = wc.sliding_window_size
    for (b, h) in units:
        s, e = int(wc.kv_indptr[b]), int(wc.kv_indptr[b + 1])
        rows = wc.kv_indices[s:e].long()
        k = wc.k_cache[rows, h:h + 1]
        v = wc.v_cache[rows, h:h + 1]
        L = e - s
        if wc.kind == "decode":
            q = wc.q[b:b + 1, h * g:(h + 1) * g]
            O._attend(q.float(), k.float(), v.float(), wc.sm_scale, None)
            flops += 4 * wc.head_dim * g * L
        else:
            qs, qe = int(wc.qo_indptr[b]), int(wc.qo_indptr[b + 1])
            pre = int(wc.prefix_lens[b])
            for q0 in range(qs, qe, 1024):
                q1 = min(qe, q0 + 1024)
                mask = O.visibility_mask(q1 - q0, L, pre, is_cross_attention=wc.is_cross_attention,
                                         sliding_window_size=W, q_offset=q0 - qs)
                O._attend(wc.q[q0:q1, h * g:(h + 1) * g].float(), k.float(), v.float(), wc.sm_scale, mask)
                flops += 4 * wc.head_dim * g * int(mask.sum())
    return flops


def cpu_copy_of(w):
    """Host copy of a workload holding only the slots it touches (re-indexed densely)."""
    import copy
    wc = copy.copy(w)
    idx = w.kv_indices.long()
    uniq, inv = torch.unique(idx, return_inverse=True)
    wc.k_cache = w.k_cache[uniq].cpu()
    wc.v_cache = w.v_cache[uniq].cpu()
    wc.kv_indices = inv.to(torch.int32).cpu()
    for name in ("q", "kv_indptr", "qo_indptr", "prefix_lens"):
        t = getattr(w, name)
        if t is not None:
            setattr(wc, name, t.cpu())
    return wc


def unit_of(w):
    return ("TFLOP/s", 1e12) if w.kind == "prefill" else ("GB/s", 1e9)


def cpu_work(w, units, flops):
    if w.kind == "prefill":
        return flops
    g = w.hq // w.hkv
    return sum(2 * w.kv_lens[b] * w.head_dim * 2 + 4 * w.kv_lens[b] + 2 * g * w.head_dim * 2 for b, _ in units)


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use every core it may."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_baseline(w, budget_s: float = 12.0):
    wc = cpu_copy_of(w)
    units = cpu_units(wc)
    cores = use_all_host_threads()
    cpu_run_units(wc, units[:1])  # warm-up
    t0 = time.perf_counter()
    done, work = 0, 0.0
    while time.perf_counter() - t0 < budget_s:
        u = units[done % len(units)]
        fl = cpu_run_units(wc, [u])
        work += cpu_work(wc, [u], fl)
        done += 1
    dt = time.perf_counter() - t0
    unit, div = unit_of(w)
    return {"value": work / dt / div, "unit": unit, "cores": cores, "kind": "port",
            "sample": f"{done} (sequence, kv-head) units of {w.name} (the batch has {len(units)}; "
                      f"cycled), gather pages then fp32 SDPA on torch CPU, {dt:.1f} s"}


# ----------------------------------------------------------------------------- arms
def measure(name, device, rank, world, steps, warmup, dist_on, flush, peaks, peak_kind, with_e2e=True):
    w = make_workload(name, device, rank)
    unit, div = unit_of(w)
    work = w.algorithmic_flops() if w.kind == "prefill" else w.algorithmic_bytes()
    big = w.kind == "decode" and w.algorithmic_bytes() > 4 * L2_FLUSH_BYTES
    fl = torch.empty(1, dtype=torch.uint8, device=device) if big else flush
    total_ms, per = time_kernel_steps(w, steps, warmup, dist_on, fl)
    total_ms = max_over_ranks(total_ms, dist_on)
    work_all = work
    if dist_on:
        t = torch.tensor([float(work)], dtype=torch.float64, device=device)
        torch.distributed.all_reduce(t)
        work_all = float(t.item())
    value = work_all * steps / (total_ms * 1e-3) / div
    own = work * steps / (sum(per) * 1e-3) / div
    # which roofline binds: arithmetic intensity against the ridge of the measured peaks
    step_s = sum(per) * 1e-3 / steps
    intensity = w.algorithmic_flops() / max(1, w.algorithmic_bytes())
    ridge = peaks["bf16_tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
    if w.kind == "prefill" and intensity >= ridge:
        peak = peaks["bf16_tflops"]
        ach = w.algorithmic_flops() / step_s / 1e12
        roof = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                "frac": ach / peak, "traffic": traffic_of(w)[0], "traffic_source": traffic_of(w)[1],
                "peak_source": f"{peak_kind} burst bf16"}
    else:
        peak = peaks["hbm_gbs"]
        ach = w.algorithmic_bytes() / step_s / 1e9
        roof = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                "traffic": traffic_of(w)[0], "traffic_source": traffic_of(w)[1],
                "peak_source": f"{peak_kind} copy bandwidth",
                "flop_per_byte": intensity, "ridge_flop_per_byte": ridge}
    res = {"workload": w.name, "value": value, "unit": unit, "ms_per_step": total_ms / steps,
           "median_ms": statistics.median(per), "min_ms": min(per), "roofline": roof,
           "algorithmic_bytes": w.algorithmic_bytes(), "algorithmic_flops": w.algorithmic_flops(),
           "gpu_launches": launches_per_step(w) * steps,
           "l2": "inputs larger than L2" if big else "flushed between steps (256 MiB write)"}
    if GRAPH_REPLAY:
        res["cuda_graph"] = "each step replays one captured operator call"
    if with_e2e:
        e_steps = max(3, min(steps, 50))
        ms, bi, bo, floor = time_e2e(w, device, e_steps, min(warmup, 5), dist_on, world)
        ms = max_over_ranks(ms, dist_on)
        floor = max_over_ranks(floor, dist_on)
        res["e2e"] = {"value": work_all * e_steps / (ms * 1e-3) / div, "unit": unit,
                      "h2d_bytes_per_step": bi, "d2h_bytes_per_step": bo, "steps": e_steps,
                      "ms_per_step": ms / e_steps, "copy_floor_ms": floor, "cpu_binding": NUMA_NOTE,
                      "pipelining": "copies and compute of neighbouring steps overlap "
                                    "(copy-in, compute, gather, copy-out streams, 2 buffers); one "
                                    "host wait per step; copy_floor_ms = the bare staging copies of "
                                    "all ranks at once, no compute"}
    return w, res


# ----------------------------------------------------------------------------- strong scaling
LAST_STEP_STATS = {}


def _timed_steps(call, steps, dist_on):
    """Device time (ms) per call over `steps` calls in a row: the MEDIAN step of each rank, max
    over ranks.  The mean and the slowest single step (each the max over ranks) are left in
    LAST_STEP_STATS: with eight processes on a shared host a rank now and then stalls for tens of
    milliseconds between two launches (seen: one 26 ms step among twenty of 0.67 ms), which the
    mean of a 20-step run of a sub-millisecond step shows and the median does not."""
    for _ in range(3):
        call()
    barrier(dist_on)
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    marks[0].record()
    for i in range(steps):
        out = call()
        marks[i + 1].record()
    barrier(dist_on)
    per = sorted(marks[i].elapsed_time(marks[i + 1]) for i in range(steps))
    LAST_STEP_STATS.clear()
    LAST_STEP_STATS.update(timing="median step of each rank, max over ranks",
                           mean_ms=max_over_ranks(marks[0].elapsed_time(marks[steps]), dist_on) / steps,
                           slowest_step_ms=max_over_ranks(per[-1], dist_on))
    return max_over_ranks(per[len(per) // 2], dist_on), out


def sharded_decode(device, rank, world, steps):
    """ONE global long-context decode batch (cfg5a) split over the ranks by request
    (`parallel.assign_requests`: longest first onto the least loaded rank).  A rank's pool holds the
    pages of its own sequences only (same values as in the global pool, freshly permuted), with its
    own page index and lengths; the outputs are reassembled with `parallel.gather_request_outputs`
    (one NCCL all-gather); rank 0 also runs the unsharded batch and compares bit for bit."""
    from mini_sglang_mlx_b200 import paged_decode_attention_p16, parallel as P, synthetic as S
    from mini_sglang_mlx_b200.attention import compute_num_kv_splits
    w = S.cfg5a_decode(seed=505, device=device)
    w.index = "page"
    splits_all = compute_num_kv_splits(w.kv_lens, w.hkv)
    shards = P.assign_requests(w.kv_lens, world)
    mine = shards[rank]
    need = [(w.kv_lens[b] + S.PAGE_SIZE - 1) // S.PAGE_SIZE for b in mine]
    src_pages = torch.cat([w.page_table[b, :n] for b, n in zip(mine, need)]).long()
    n_local = int(src_pages.numel())
    g = torch.Generator().manual_seed(9000 + rank)
    place = torch.randperm(n_local + 16, generator=g)[:n_local].to(device)      # where each page goes
    shape = (w.k_cache.shape[0] // S.PAGE_SIZE, S.PAGE_SIZE, w.hkv, w.head_dim)
    pools = []
    for full in (w.k_cache, w.v_cache):
        local = torch.zeros((n_local + 16, *shape[1:]), dtype=full.dtype, device=device)
        local[place] = full.view(shape)[src_pages]
        pools.append(local.view(-1, w.hkv, w.head_dim))
    kc, vc = pools
    q = w.q[mine].contiguous()
    pip = S._indptr(need).to(device)
    pidx = place.to(torch.int32)
    lens = torch.tensor([w.kv_lens[b] for b in mine], dtype=torch.int32, device=device)
    splits = torch.tensor([splits_all[b] for b in mine], dtype=torch.int32, device=device)
    reference = None
    if rank == 0:
        gp, gi, gl = w.page_csr()
        reference = paged_decode_attention_p16(w.q, w.k_cache, w.v_cache, gp, gi, gl,
                                               torch.tensor(splits_all, dtype=torch.int32, device=device),
                                               w.sm_scale, w.max_kv_splits)
        torch.cuda.synchronize()
    total_bytes = w.algorithmic_bytes()
    per_token = 2 * w.hkv * w.head_dim * 2
    rank_bytes = [sum(w.kv_lens[b] for b in s) * per_token for s in shards]
    kv_lens, batch, name = list(w.kv_lens), w.batch, w.name
    del w, full, local, pools
    torch.cuda.empty_cache()

    call = lambda: paged_decode_attention_p16(q, kc, vc, pip, pidx, lens, splits, 1 / math.sqrt(128), 32)  # noqa: E731
    ms, out_local = _timed_steps(call, steps, True)
    step_stats = dict(LAST_STEP_STATS)
    plan = P.GatherPlan(shards, [1] * batch, device)
    gather = lambda: P.gather_request_outputs(out_local, plan)  # noqa: E731
    gms, full_out = _timed_steps(gather, 3, True)
    exact = bool(torch.equal(full_out, reference)) if rank == 0 else None
    return {"workload": name, "split": "by request: parallel.assign_requests, longest first onto the "
                                       "least loaded rank; per-rank pool, page index and lengths",
            "scaling": "strong", "value": total_bytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
            "ms_per_step": ms, **step_stats, "reassembly_ms": gms,
            "value_with_reassembly": total_bytes / ((ms + gms) * 1e-3) / 1e9,
            "load_imbalance_max_over_mean": max(rank_bytes) / (sum(rank_bytes) / world),
            "sequences_per_rank": [len(s) for s in shards],
            "matches_unsharded_bit_for_bit": exact, "steps": steps}


def sharded_by_head(device, rank, world, steps):
    """The batch-1 fallback: one prefill grid point (chunk 2048 after a 8192-token prefix) split
    by KV-head group (`parallel.head_slices`); each rank holds the K/V heads of its group for all
    tokens; `parallel.gather_head_outputs` concatenates along the head axis.  Rank 0 compares with
    the unsharded op (same rows and heads; the key-range split may differ, so within the parity
    tolerance rather than bit for bit)."""
    from mini_sglang_mlx_b200 import paged_prefill_attention_p16, parallel as P, synthetic as S
    w = S.cfg5b_prefill_point(2048, 8192, device=device)
    if w.hkv % world != 0:
        return {"workload": w.name, "skipped": f"{w.hkv} KV heads do not split over {world} ranks"}
    qs, ks = P.head_slices(w.hq, w.hkv, world)[rank]
    q = w.q[:, qs].contiguous()
    kc, vc = w.k_cache[:, ks].contiguous(), w.v_cache[:, ks].contiguous()
    pip, pidx, lens = w.page_csr()

    def run(q_, kc_, vc_):
        return paged_prefill_attention_p16(q_, kc_, vc_, w.qo_indptr, pip, pidx, lens, w.prefix_lens,
                                           w.sm_scale, w.max_len_extend)
    ms, out_local = _timed_steps(lambda: run(q, kc, vc), steps, True)
    step_stats = dict(LAST_STEP_STATS)
    gms, full_out = _timed_steps(lambda: P.gather_head_outputs(out_local), 3, True)
    err = None
    if rank == 0:
        err = float((full_out.float() - run(w.q, w.k_cache, w.v_cache).float()).abs().max())
    flops = w.algorithmic_flops()
    return {"workload": w.name, "split": "by KV-head group: parallel.head_slices", "scaling": "strong",
            "value": flops / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, **step_stats,
            "reassembly_ms": gms, "value_with_reassembly": flops / ((ms + gms) * 1e-3) / 1e12,
            "max_abs_diff_to_unsharded": err, "tolerance": 2e-2, "steps": steps}


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist_on = world > 1
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if dist_on:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=device)
    peaks, peak_kind = load_peaks()
    flush = torch.empty(L2_FLUSH_BYTES, dtype=torch.uint8, device=device)

    with ClockSampler(local) as clocks:
        w, main = measure(args.workload, device, rank, world, args.steps, args.warmup, dist_on, flush,
                          peaks, peak_kind, with_e2e=not args.no_e2e)
        extra = {}
        if args.workload == "cfg2" and not args.no_decode:
            del w
            torch.cuda.empty_cache()
            dsteps = max(3, min(args.steps, 20))
            w2, dec = measure("cfg5a", device, rank, world, dsteps, 3, dist_on, flush, peaks, peak_kind,
                              with_e2e=False)
            dec["steps"] = dsteps
            extra["decode"] = dec
            del w2
            torch.cuda.empty_cache()

    if dist_on and not args.no_sharded:
        torch.cuda.empty_cache()
        ssteps = max(3, min(args.steps, 20))
        extra["sharded"] = {"decode": sharded_decode(device, rank, world, ssteps),
                            "prefill_by_head": sharded_by_head(device, rank, world, ssteps)}
        torch.cuda.empty_cache()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cpu = cpu_baseline(make_workload(args.workload, device, rank))
    if rank == 0:
        line = {
            "metric": METRIC, "value": main["value"], "unit": main["unit"], "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": main["workload"],
                       "sharding": "value/e2e: by request, one batch per GPU (weak scaling); "
                                   "\"sharded\": one global batch split over the GPUs (strong scaling)",
                       "l2": main["l2"], "page_size": 16,
                       "index_granularity": ("one id per 16-token page (TMA box loads)" if INDEX == "page"
                                             else "per-token slot ids"),
                       "median_ms": main["median_ms"], "min_ms": main["min_ms"],
                       "algorithmic_flops_per_step": main["algorithmic_flops"],
                       "algorithmic_bytes_per_step": main["algorithmic_bytes"],
                       **({"cuda_graph": main["cuda_graph"]} if "cuda_graph" in main else {})},
            "clocks": clocks.summary(), "e2e": main.get("e2e"), "gpu_launches": main["gpu_launches"],
            "roofline": main["roofline"], "cpu_baseline": cpu,
        }
        line.update(extra)
        print(json.dumps(line))
    if dist_on:
        torch.distributed.destroy_process_group()


def run_pre_attention_step(args):
    """`--workload qk_norm_rope_store`: the fused step in front of the attention op (q/k RMSNorm,
    RoPE, K/V scatter) over one prefill chunk of a Qwen3-8B-shaped layer; HBM-bound, GB/s."""
    from mini_sglang_mlx_b200 import qk_norm_rope_store
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    peaks, peak_kind = load_peaks()
    n, hq, hkv, d = args.batch or 32768, 32, 8, 128
    g = torch.Generator().manual_seed(707)
    qkv = torch.randn(n, (hq + 2 * hkv) * d, generator=g).bfloat16()
    qw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    kw = (1 + 0.1 * torch.randn(d, generator=g)).bfloat16()
    pos = torch.arange(n, dtype=torch.int32)
    num_slots = 2 * n
    loc = torch.randperm(num_slots, generator=g)[:n].int()
    qkv_d = qkv.to(device)
    q = qkv_d[:, : hq * d].view(n, hq, d)
    k = qkv_d[:, hq * d:(hq + hkv) * d].view(n, hkv, d)
    v = qkv_d[:, (hq + hkv) * d:].view(n, hkv, d)
    kc = torch.zeros(num_slots, hkv, d, dtype=torch.bfloat16, device=device)
    vc = torch.zeros_like(kc)
    args_d = (qw.to(device), kw.to(device), pos.to(device), loc.to(device), kc, vc)
    nbytes = n * (2 * hq + 4 * hkv) * d * 2          # q read+write, k and v read, k and v rows written
    # 0.8 GB per step at the default size: larger than L2.  Smaller chunks get the L2 flush of the
    # attention workloads in front of every step (which also keeps the launch queued ahead of the
    # GPU, so that the events do not time the host's launch path).
    small = nbytes < 2 * L2_FLUSH_BYTES
    flush = torch.empty(L2_FLUSH_BYTES if small else 1, dtype=torch.uint8, device=device)
    with ClockSampler(device.index) as clocks:
        for _ in range(args.warmup):
            qk_norm_rope_store(q, k, v, *args_d, rope_base=1e6)
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        for i in range(args.steps):
            if small:
                flush.zero_()
            starts[i].record()
            qk_norm_rope_store(q, k, v, *args_d, rope_base=1e6)
            ends[i].record()
        torch.cuda.synchronize()
    per = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    ms = sum(per) / len(per)
    cpu = None
    if not args.no_cpu:
        from oracle.qk_norm_rope_oracle import qk_norm_rope_store_oracle
        cores = use_all_host_threads()
        m = 2048
        qc = qkv[:m, : hq * d].view(m, hq, d)
        kc_ = qkv[:m, hq * d:(hq + hkv) * d].view(m, hkv, d)
        vc_ = qkv[:m, (hq + hkv) * d:].view(m, hkv, d)
        pool = torch.zeros(num_slots, hkv, d, dtype=torch.bfloat16)
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < 10.0:
            qk_norm_rope_store_oracle(qc, kc_, vc_, qw, kw, pos[:m], loc[:m], pool, pool.clone(),
                                      rope_base=1e6, eps=1e-6, rotary_dim=d)
            reps += 1
        dt = time.perf_counter() - t0
        cpu = {"value": reps * m * (2 * hq + 4 * hkv) * d * 2 / dt / 1e9, "unit": "GB/s", "cores": cores,
               "kind": "port", "sample": f"{m} of {n} tokens per pass, torch-CPU restatement of norm, rope, scatter"}
    ach = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "fused q/k RMSNorm + RoPE + K/V scatter, HBM GB/s", "value": ach, "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"qk_norm_rope_store, {n} tokens, Hq32/Hkv8, D128, fused qkv rows",
                   "l2": "flushed between steps (256 MiB write)" if small else "inputs larger than L2",
                   "algorithmic_bytes_per_step": nbytes},
        "clocks": clocks.summary(), "e2e": None, "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": ach / peaks["hbm_gbs"], "traffic": None,
                     "peak_source": f"{peak_kind} copy bandwidth"},
        "cpu_baseline": cpu}))


def run_store_kv(args):
    """`--workload store_kv_cache`: the K/V scatter of one prefill chunk into the paged pool
    (Qwen3-8B shape, Hkv 8, D 128), HBM-bound: rows read once, written once."""
    from mini_sglang_mlx_b200 import store_kv_cache
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    peaks, peak_kind = load_peaks()
    n, hkv, d = args.batch or 131072, 8, 128
    g = torch.Generator().manual_seed(808)
    k = torch.randn(n, hkv, d, generator=g).bfloat16().to(device)
    v = torch.randn(n, hkv, d, generator=g).bfloat16().to(device)
    num_slots = 2 * n
    loc = torch.randperm(num_slots, generator=g)[:n].int().to(device)
    kc = torch.zeros(num_slots, hkv, d, dtype=torch.bfloat16, device=device)
    vc = torch.zeros_like(kc)
    nbytes = 4 * n * hkv * d * 2 + 4 * n        # k, v read; k, v rows written; slot ids
    with ClockSampler(device.index) as clocks:
        for _ in range(args.warmup):
            store_kv_cache(kc, vc, loc, k, v)
        torch.cuda.synchronize()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        for i in range(args.steps):           # 1.07 GB per step: larger than L2
            starts[i].record()
            store_kv_cache(kc, vc, loc, k, v)
            ends[i].record()
        torch.cuda.synchronize()
    per = [s_.elapsed_time(e) for s_, e in zip(starts, ends)]
    ms = sum(per) / len(per)
    cpu = None
    if not args.no_cpu:
        from oracle.paged_attention_oracle import store_kv_cache_oracle
        cores = use_all_host_threads()
        m = 16384
        kc_h = torch.zeros(num_slots, hkv, d, dtype=torch.bfloat16)
        vc_h = torch.zeros_like(kc_h)
        k_h, v_h, loc_h = k[:m].cpu(), v[:m].cpu(), loc[:m].cpu()
        t0, reps = time.perf_counter(), 0
        while time.perf_counter() - t0 < 10.0:
            store_kv_cache_oracle(kc_h, vc_h, loc_h, k_h, v_h)
            reps += 1
        dt = time.perf_counter() - t0
        cpu = {"value": reps * (4 * m * hkv * d * 2 + 4 * m) / dt / 1e9, "unit": "GB/s", "cores": cores,
               "kind": "port", "sample": f"{m} of {n} tokens per pass, torch-CPU index_copy restatement"}
    ach = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "K/V scatter into the paged pool, HBM GB/s", "value": ach, "unit": "GB/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"store_kv_cache, {n} tokens, Hkv8, D128", "l2": "inputs larger than L2",
                   "algorithmic_bytes_per_step": nbytes},
        "clocks": clocks.summary(), "e2e": None, "gpu_launches": args.steps,
        "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": ach / peaks["hbm_gbs"], "traffic": None,
                     "peak_source": f"{peak_kind} copy bandwidth"},
        "cpu_baseline": cpu}))


def run_reference(args):
    """The CPU path the reference's own tests use as ground truth (gather pages, SDPA), as a
    torch-CPU restatement: MLX is not installable here and the Metal kernels need macOS."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    device = "cuda" if torch.cuda.is_available() else "cpu"
    from mini_sglang_mlx_b200 import synthetic as S
    if args.workload == "cfg2":
        w = S.cfg2_prefill(device=device) if device == "cuda" else S.cfg2_prefill(device="cpu")
    else:
        w = make_workload(args.workload, device, 0)
    wc = cpu_copy_of(w)
    units = cpu_units(wc)
    cores = use_all_host_threads()
    # size the per-step sample so that warmup + steps fit in about two minutes
    t0 = time.perf_counter()
    cpu_run_units(wc, units[:1])
    t_unit = time.perf_counter() - t0
    per_step = max(1, min(len(units), int(120.0 / max(1, args.steps + args.warmup) / max(t_unit, 1e-4))))
    sample = units[:per_step]
    for _ in range(args.warmup):
        cpu_run_units(wc, sample)
    t0 = time.perf_counter()
    work = 0.0
    for _ in range(args.steps):
        fl = cpu_run_units(wc, sample)
        work += cpu_work(wc, sample, fl)
    dt = time.perf_counter() - t0
    unit, div = unit_of(w)
    value = work / dt / div
    desc = (f"{per_step} of {len(units)} (sequence, kv-head) units of {w.name} per step, "
            f"gather pages then fp32 SDPA on torch CPU")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": unit,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w.name, "note": "reference Metal kernels need macOS; MLX CPU backend not "
                   "installable here; this is the torch-CPU restatement of its gather-then-SDPA path"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg2")
    ap.add_argument("--no-decode", action="store_true", help="skip the cfg5a decode measurement")
    ap.add_argument("--graph", action="store_true",
                    help="kernel timing replays a CUDA graph of one operator call (launch overhead apart)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline")
    ap.add_argument("--no-sharded", action="store_true",
                    help="N > 1: skip the strong-scaling section (one global batch split over the ranks)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end measurement")
    ap.add_argument("--index", default="page", choices=["page", "token"],
                    help="kernel-only timing through the page-granular operators (one id per 16-token "
                         "page) or the per-token ones; the end-to-end leg always runs AttnBackend")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the configuration's batch size (small profiling captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    global BATCH_OVERRIDE, GRAPH_REPLAY, INDEX
    INDEX = args.index
    BATCH_OVERRIDE = args.batch
    GRAPH_REPLAY = args.graph
    if args.workload == "qk_norm_rope_store":
        run_pre_attention_step(args)
    elif args.workload == "store_kv_cache":
        run_store_kv(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
