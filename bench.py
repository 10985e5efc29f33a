#!/usr/bin/env python
"""Benchmark of the PagedAttention decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload cfg2|cfg3|cfg4|cfg5|cfg1]

One "step" is one decode call (one new token per sequence, one layer) of
``paged_attention_v2`` over the whole synthetic batch.  The default workload is
the Llama-3-8B-shape batch-256 decode (256 sequences, 32 query / 8 KV heads,
head size 128, block size 16, bf16, lengths U{512..4096}).  Prints ONE JSON line.

value      tokens/s with every input resident in HBM (device-timed, CUDA events)
e2e        the same through the public op with HOST step inputs: pinned query,
           block tables and sequence lengths are copied in, the output copied
           back, inside the timed region (the KV cache is engine state and stays
           resident, as it does for the reference op)
roofline   algorithmic bytes / op duration against the measured HBM copy peak
cpu_baseline  the reference project's own CPU attention kernel on a bounded
           sample of the same workload, on this host's cores

``--impl reference`` times only that CPU implementation (rank 0).
Multi-GPU (torchrun, one rank per GPU): every rank decodes its own batch of the
same shape (sequences partitioned, no collective on the data path) — weak scaling.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "paged_attention decode tokens/s"
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one decode-kernel launch divided by the
# algorithmic bytes of that launch, from ncu captures of small cases of the same kernels (64
# sequences of the bf16 workload, 16 sequences of the fp8 workload; their summaries are kept with
# the other profiler summaries of this repository).  Traffic grows in proportion to tokens.
NCU_TRAFFIC_RATIO = {"cfg2": 1.010, "cfg4": 1.010, "cfg3": 1.014, "cfg5": 1.014}


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            parts = [p.strip() for p in r.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": float(max(mx)) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


class L2Flush:
    """Empties L2 between timed steps: writes a buffer twice the size of L2, then reads another
    one.  The write alone would leave L2 full of dirty lines, and the next kernel would pay for
    their write-back inside its timed interval."""

    NOTE = "flushed between timed calls: 256 MB written, then 256 MB read (no dirty lines left)"

    def __init__(self, dev):
        self.w = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.r = torch.zeros(64 << 20, dtype=torch.int32, device=dev)

    def __call__(self):
        self.w.zero_()
        self.r.sum()


def build_workload(name: str, device, world: int, rank: int, num_seqs=None):
    from vllm_b200 import workloads as W

    if num_seqs is not None:
        if name == "cfg2":
            return W.config2(device, seed=0, rank=rank, num_seqs=num_seqs), "v2", "weak"
        if name == "cfg3":
            return W.config3(device, seed=rank, num_seqs=num_seqs), "v2", "weak"
        if name == "cfg5":
            return W.config5(device, world_size=world, rank=rank, num_seqs=num_seqs), "v2", "strong"
    if name in ("cfg3w", "cfg3wf"):
        # the KV-write step of config 3 (x-layout / flash layout): 128 new tokens per sequence
        return W.config3(device, seed=rank, num_seqs=num_seqs or 128), name, "weak"
    if name == "cfg2":
        return W.config2(device, seed=0, rank=rank), "v2", "weak"
    if name == "cfg1":
        return W.config1(device, seed=rank), "v1", "weak"
    if name == "cfg3":
        return W.config3(device, seed=rank), "v2", "weak"
    if name == "cfg4":
        return W.config4(device, world_size=world, rank=rank), "v2", "strong"
    if name == "cfg5":
        return W.config5(device, world_size=world, rank=rank), "v2", "strong"
    raise SystemExit(f"unknown workload {name}")


def cpu_reference_leg(w, steps: int, warmup: int, budget_s: float = 30.0, min_s: float = 10.0):
    """Times the reference project's CPU decode attention on a bounded sample (the
    first sequences of the workload, their blocks gathered into a compact pool)."""
    from oracle import ref_cpu

    if not ref_cpu.available():
        return None
    ncores = os.cpu_count() or 1
    torch.set_num_threads(ncores)
    lens = w.seq_lens.cpu().numpy().astype(np.int64)
    # sample: as many leading sequences as fit ~64k tokens (fp8 caches are dequantised to bf16)
    take = int(max(1, min(len(lens), np.searchsorted(np.cumsum(lens), 65536) + 1)))
    B = w.block_size
    need = np.ceil(lens[:take] / B).astype(int)
    bt_old = w.block_tables[:take].cpu().numpy()
    used = np.concatenate([bt_old[s, :need[s]] for s in range(take)]) if take else np.zeros(0, int)
    uniq, inv = np.unique(used, return_inverse=True)
    bt_new = np.zeros_like(bt_old)
    off = 0
    for s in range(take):
        bt_new[s, :need[s]] = inv[off:off + need[s]]
        off += need[s]
    idx = torch.from_numpy(uniq.astype(np.int64)).to(w.key_cache.device)
    kc = w.key_cache[idx].cpu()
    vc = w.value_cache[idx].cpu()
    note = ""
    if w.kv_cache_dtype != "auto":
        from oracle import paged_oracle as O
        kc = O.dequantize_fp8(kc, float(w.k_scale), torch.bfloat16)
        vc = O.dequantize_fp8(vc, float(w.v_scale), torch.bfloat16)
        note = " (CPU stand-in: fp8 cache dequantised to bf16; the reference has no CPU fp8 KV path)"
    kf, vf = ref_cpu.x_layout_to_flash(kc, vc)
    r = ref_cpu.RefCpuDecode(w.query[:take].cpu(), kf, vf, torch.from_numpy(bt_new),
                             torch.from_numpy(lens[:take].astype(np.int32)), w.scale, None, True)
    for _ in range(max(1, warmup)):
        r.run()
    times = []
    t_all = time.perf_counter()
    # `steps` calls at least; keep going (bounded) so that the sample is ~10 s of CPU work
    while len(times) < max(1, steps) or (time.perf_counter() - t_all < min_s and len(times) < 5000):
        t0 = time.perf_counter()
        r.run()
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_all > budget_s:
            break
    t = float(np.median(times))
    return {
        "value": take / t, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "reference",
        "sample": f"first {take} of {len(lens)} sequences ({int(lens[:take].sum())} KV tokens), "
                  f"{len(times)} timed calls of cpu_attention_with_kv_cache (isa={r.isa}, KV split on)" + note,
        "ms_per_step": t * 1e3, "seqs": take,
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2",
                    choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "cfg3w", "cfg3wf"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--num-seqs", type=int, default=None,
                    help="override the batch size of cfg2/cfg3/cfg5 (small cases for profiler captures)")
    a = ap.parse_args()
    a.warmup = max(3, a.warmup)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    dist = world > 1

    if a.impl == "reference" and rank != 0:
        return 0

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (the product has no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    w, version, scaling = build_workload(a.workload, dev, world, rank, a.num_seqs)
    cfg = {
        "workload": f"{w.name}: paged_attention_{version}, num_seqs={w.num_seqs} per GPU, "
                    f"{w.num_heads} query / {w.num_kv_heads} KV heads, head_size={w.head_size}, "
                    f"block_size={w.block_size}, kv_cache_dtype={w.kv_cache_dtype}, "
                    f"{w.total_tokens()} KV tokens on rank 0",
        "partitioning": "sequences per rank, no collective" if scaling == "weak" else
                        ("kv heads per rank" if a.workload == "cfg4" else "sequences per rank"),
        "l2": "inputs larger than L2 (KV bytes per step >> 126 MB), no flush needed"
              if w.attn_bytes() > 4 * 126e6 else L2Flush.NOTE,
    }

    if a.impl == "reference":
        leg = cpu_reference_leg(w, a.steps, a.warmup, budget_s=120.0, min_s=10.0)
        if leg is None:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/_C_ref_cpu.so not built"}))
            return 0
        line = {
            "impl": "reference", "metric": METRIC, "value": leg["value"], "unit": "tokens/s",
            "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": leg["ms_per_step"],
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": cfg,
            "cpu_baseline": {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": leg["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }
        print(json.dumps(line))
        return 0

    if dist:
        import torch.distributed as td
        td.init_process_group("nccl", device_id=dev)

    from vllm_b200 import _custom_ops as ops  # noqa: F401  (fails loudly if the .so is missing)
    from vllm_b200 import capi
    from vllm_b200 import workloads as W

    is_write = version in ("cfg3w", "cfg3wf")
    if is_write:
        # KV write: new K/V [T, Hkv, D] bf16 -> fp8 cache; flash layout uses [NB, B, H, D] caches
        T = w.new_key.shape[0]
        if version == "cfg3wf":
            nb = w.key_cache.shape[0]
            kcache = torch.zeros(nb, w.block_size, w.num_kv_heads, w.head_size, dtype=torch.uint8, device=dev)
            vcache = torch.zeros_like(kcache)
            write = ops.reshape_and_cache_flash
        else:
            kcache, vcache = w.key_cache, w.value_cache
            write = ops.reshape_and_cache
        units_rank = T
        bytes_rank = w.reshape_bytes()
        metric = "reshape_and_cache tokens/s"
        kernel_name = "reshape_and_cache_flash_kernel" if version == "cfg3wf" else "reshape_and_cache_kernel"
        cfg["workload"] = (f"{w.name} KV write ({'flash' if version == 'cfg3wf' else 'x'} layout): "
                           f"{T} new tokens x {w.num_kv_heads} heads x {w.head_size}, bf16 -> fp8-e4m3, "
                           f"block_size={w.block_size}")
        flush = L2Flush(dev)
        cfg["l2"] = L2Flush.NOTE
        nk, nv, sm = w.new_key, w.new_value, w.slot_mapping

        def step():
            write(nk, nv, kcache, vcache, sm, "fp8", w.k_scale, w.v_scale)
    else:
        scratch = w.scratch()
        out = torch.empty_like(w.query)
        flush = None if w.attn_bytes() > 4 * 126e6 else L2Flush(dev)
        units_rank = w.num_seqs
        bytes_rank = w.attn_bytes()
        metric = METRIC
        kernel_name = "pa_decode_kernel (split-KV merge fused; one launch per step)"

        def step():
            W.run_attention(w, out=out, version=version, scratch=scratch)

    def barrier():
        if dist:
            td.barrier()
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        step()
    barrier()

    # ---- device-resident timing: one event pair per step (the launching stream is torch's current stream)
    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    sampler.start()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.steps)]
    capi.launch_count(reset=True)
    barrier()
    t_wall = time.perf_counter()
    for s, e in evs:
        if flush is not None:
            flush()
        s.record()
        step()
        e.record()
    barrier()
    t_wall = time.perf_counter() - t_wall
    launches = capi.launch_count()
    per_step = [s.elapsed_time(e) for s, e in evs]
    ms = float(np.mean(per_step))
    clocks = sampler.stop()

    # ---- end to end with host step inputs (pinned), one event pair per step so that the
    # L2 flush of small workloads stays outside the timed intervals
    if is_write:
        hk, hv, hs = nk.cpu().pin_memory(), nv.cpu().pin_memory(), sm.cpu().pin_memory()
        dk, dv, ds = torch.empty_like(nk), torch.empty_like(nv), torch.empty_like(sm)
        done = torch.zeros(1, dtype=torch.int32, device=dev)
        hdone = torch.zeros(1, dtype=torch.int32).pin_memory()

        def e2e_step():
            dk.copy_(hk, non_blocking=True)
            dv.copy_(hv, non_blocking=True)
            ds.copy_(hs, non_blocking=True)
            write(dk, dv, kcache, vcache, ds, "fp8", w.k_scale, w.v_scale)
            hdone.copy_(done, non_blocking=True)  # the step's result is the updated cache; read a token back

        h2d = hk.numel() * 2 + hv.numel() * 2 + hs.numel() * 8
        d2h = 4
    else:
        hq = w.query.cpu().pin_memory()
        hbt = w.block_tables.cpu().pin_memory()
        hsl = w.seq_lens.cpu().pin_memory()
        hout = torch.empty_like(hq).pin_memory()
        dq, dbt, dsl = torch.empty_like(w.query), torch.empty_like(w.block_tables), torch.empty_like(w.seq_lens)
        wq, wbt, wsl = w.query, w.block_tables, w.seq_lens

        def e2e_step():
            dq.copy_(hq, non_blocking=True)
            dbt.copy_(hbt, non_blocking=True)
            dsl.copy_(hsl, non_blocking=True)
            w.query, w.block_tables, w.seq_lens = dq, dbt, dsl
            W.run_attention(w, out=out, version=version, scratch=scratch)
            hout.copy_(out, non_blocking=True)

        h2d = hq.numel() * hq.element_size() + hbt.numel() * 4 + hsl.numel() * 4
        d2h = hout.numel() * hout.element_size()

    for _ in range(3):
        e2e_step()
    barrier()
    evs2 = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(a.steps)]
    for s_ev, e_ev in evs2:
        if flush is not None:
            flush()
        s_ev.record()
        e2e_step()
        e_ev.record()
    barrier()
    ms_e2e = float(np.mean([s_ev.elapsed_time(e_ev) for s_ev, e_ev in evs2]))
    if not is_write:
        w.query, w.block_tables, w.seq_lens = wq, wbt, wsl

    # ---- max over ranks, whole-job aggregate
    seqs_total = units_rank
    if dist:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
        td.all_reduce(t, op=td.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
        n = torch.tensor([seqs_total], dtype=torch.int64, device=dev)
        td.all_reduce(n)
        seqs_total = int(n[0])

    if rank == 0:
        peak, peak_kind = measured_peak()
        achieved = bytes_rank / (ms * 1e-3) / 1e9
        ratio = NCU_TRAFFIC_RATIO.get(a.workload)
        line = {
            "metric": metric, "value": seqs_total / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": cfg, "clocks": clocks,
            "e2e": {"value": seqs_total / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ms_per_step": ms_e2e},
            "gpu_launches": int(launches),
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                "frac_of_nominal_8TBs": achieved / 8000.0,
                "traffic": None if ratio is None else ratio * bytes_rank,
                "algorithmic_bytes_per_launch": int(bytes_rank),
                "kernel": kernel_name,
                "ms_min": float(np.min(per_step)), "ms_median": float(np.median(per_step)),
            },
            "wall_s_timed_region": t_wall,
        }
        if world == 1 and not a.no_cpu_baseline and not is_write:
            try:
                leg = cpu_reference_leg(w, steps=5, warmup=1)
            except Exception as ex:  # the baseline must never take the GPU number down with it
                leg = None
                line["cpu_baseline_error"] = repr(ex)
            if leg is not None:
                line["cpu_baseline"] = {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    if dist:
        td.barrier()
        td.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
