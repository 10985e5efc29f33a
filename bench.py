#!/usr/bin/env python
"""Benchmark of the PagedAttention decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload cfg2|cfg1|cfg3|cfg4|cfg5|cfg3w|cfg3wf] [--headline-only]
                    [--shard-of N] [--num-seqs S]

One "step" is one decode call (one new token per sequence, one layer) of
``paged_attention_v2`` over the whole synthetic batch.  The default workload is
the Llama-3-8B-shape batch-256 decode (256 sequences, 32 query / 8 KV heads,
head size 128, block size 16, bf16, lengths U{512..4096}).  Prints ONE JSON line.

value      tokens/s with every input resident in HBM (device-timed, CUDA events)
e2e        the same through the public op with HOST step inputs: pinned query,
           block tables and sequence lengths are copied in and the output is
           copied back for every step inside the timed region, on copy streams so
           that the copies of neighbouring steps run under the kernel (the KV cache
           is engine state and stays resident, as it does for the reference op)
roofline   algorithmic bytes / op duration against the measured HBM copy peak,
           and against a pure-read peak measured in the same run
cpu_baseline  the reference project's own CPU attention kernel on a bounded
           sample of the same workload, on this host's cores
configs    (default workload, 1 GPU) the other benchmark configurations - small-batch
           v1, fp8 decode and its KV write, skewed long context, large-batch fp8 -
           each with its time, achieved bandwidth and the reference project's own CUDA
           kernel timed on the same tensors (``ref_gpu_ms``)
strong_scaling  (default workload) the long-context configuration with KV heads
           sharded over the ranks and the large-batch one with sequences sharded:
           one GPU's time for the whole problem, the slowest rank's time for its
           shard, and the shards' outputs all-gathered over NCCL and compared with
           the unsharded result

``--impl reference`` times only the CPU implementation (rank 0).
Multi-GPU (torchrun, one rank per GPU): for ``value`` every rank decodes its own
batch of the same shape (sequences partitioned, no collective on the data path) -
weak scaling.
"""
from __future__ import annotations

import argparse
import gc
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
L2_BYTES = 126e6


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def ncu_traffic_ratio(name: str):
    """dram bytes (read + write) of one launch / algorithmic bytes of that launch, from the
    profiler captures of small cases of the same kernels that profiles/ncu_traffic.json records
    (with the commit they were taken at).  Traffic grows in proportion to the tokens."""
    f = ROOT / "profiles" / "ncu_traffic.json"
    try:
        return float(json.loads(f.read_text())["ratio"][name])
    except Exception:
        return None


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
    BIG = "inputs larger than L2 (KV bytes per step >> 126 MB), no flush needed"

    def __init__(self, dev):
        self.w = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.r = torch.zeros(64 << 20, dtype=torch.int32, device=dev)

    def __call__(self):
        self.w.zero_()
        self.r.sum()


def time_steps(step, steps: int, warmup: int, flush=None):
    """Per-step device times in ms: one CUDA event pair per step on the current stream, so the
    L2 flush of small workloads stays outside the timed intervals."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in evs:
        if flush is not None:
            flush()
        s.record()
        step()
        e.record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in evs]


def read_peak_gbs(dev) -> float:
    """Pure-read HBM bandwidth: sum-reduce over a 4 GiB buffer, best of 5 (CUDA events)."""
    x = torch.empty(1 << 30, dtype=torch.float32, device=dev)
    x.zero_()
    t = time_steps(lambda: x.sum(), 5, 2)
    del x
    torch.cuda.empty_cache()
    return (1 << 32) / (min(t) * 1e-3) / 1e9


def build_workload(name: str, device, world: int, rank: int, num_seqs=None):
    import workloads as W

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


# ---------------------------------------------------------------- reference CUDA kernels (timed baseline)
_REF_GPU = None


def ref_gpu_ops():
    """The reference project's own CUDA kernels, compiled unmodified for sm_100a by
    oracle/build_ref.py.  Used here only as a timed baseline on the same tensors (like the
    CPU leg); nothing of the product calls it.  None when the library was not built."""
    global _REF_GPU
    if _REF_GPU is None:
        so = ROOT / "oracle" / "_ref" / "_C_ref.so"
        if not so.exists():
            _REF_GPU = False
        else:
            try:
                torch.ops.load_library(str(so))
                _REF_GPU = (torch.ops._C_ref, torch.ops._C_ref_cache_ops)
            except Exception:
                _REF_GPU = False
    return _REF_GPU or None


def attention_case(w, version: str, steps: int, warmup: int, peaks, with_ref: bool = True):
    """Times one attention configuration (and the reference CUDA kernel on the same tensors)."""
    import workloads as W

    dev = w.query.device
    scratch = w.scratch() if version == "v2" else None
    out = torch.empty_like(w.query)
    nbytes = w.attn_bytes()
    flush = None if nbytes > 4 * L2_BYTES else L2Flush(dev)
    t = time_steps(lambda: W.run_attention(w, out=out, version=version, scratch=scratch), steps, warmup, flush)
    ms = float(np.mean(t))
    res = {
        "op": f"paged_attention_{version}", "ms": ms, "ms_min": float(np.min(t)),
        "bytes": int(nbytes), "achieved_gbs": nbytes / (ms * 1e-3) / 1e9,
        "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["copy"],
        "frac_of_read_peak": nbytes / (ms * 1e-3) / 1e9 / peaks["read"],
        "tokens_per_s": w.num_seqs / (ms * 1e-3),
        "l2": L2Flush.BIG if flush is None else "flushed between timed calls",
    }
    ref = ref_gpu_ops() if with_ref else None
    if ref is not None:
        r = torch.empty_like(w.query)
        tail = (w.query, w.key_cache, w.value_cache, w.num_kv_heads, w.scale, w.block_tables,
                w.seq_lens, w.block_size, w.max_seq_len, None, w.kv_cache_dtype, w.k_scale,
                w.v_scale, 0, 0, 0, 64, 0)
        if version == "v1":
            fn = lambda: ref[0].paged_attention_v1(r, *tail)  # noqa: E731
        else:
            e, m, tt = w.scratch()
            fn = lambda: ref[0].paged_attention_v2(r, e, m, tt, *tail)  # noqa: E731
        tr = time_steps(fn, max(3, min(10, steps)), 2, flush)
        res["ref_gpu_ms"] = float(np.mean(tr))
        res["speedup_vs_ref_gpu"] = res["ref_gpu_ms"] / ms
        res["max_abs_diff_vs_ref_gpu"] = float((r.float() - out.float()).abs().max())
    return res


def write_case(w, layout: str, kv: str, steps: int, warmup: int, peaks, tokens=None, shift: int = 0):
    """Times the KV write of config 3's shape: `layout` x|flash, cache type `kv` fp8|auto,
    `tokens` = None for the prefill-shaped write (128 new tokens per sequence, consecutive
    slots) or a count for a decode-shaped one (that many scattered slots, one per sequence);
    `shift` writes the new tokens that many positions earlier in their sequences, so that the
    chunk of each sequence starts inside a cache block (the continuation of earlier context)."""
    from vllm_b200 import _custom_ops as ops

    dev = w.query.device
    nk, nv, sm = w.new_key, w.new_value, w.slot_mapping
    if tokens is not None:
        # the last position of each sequence: one slot per sequence, scattered over the pool
        per = nk.shape[0] // w.num_seqs
        pick = torch.arange(w.num_seqs, device=dev) * per + per - 1
        reps = (tokens + w.num_seqs - 1) // w.num_seqs
        pick = pick.repeat(reps)[:tokens]
        nk, nv, sm = nk[pick].contiguous(), nv[pick].contiguous(), sm[pick].contiguous()
    if shift:
        # the same number of new tokens per sequence, `shift` positions earlier: positions
        # [len - new - shift, len - shift), through the sequence's block table
        per = nk.shape[0] // w.num_seqs
        L = int(w.seq_lens[0])
        pos = torch.arange(L - per - shift, L - shift, device=dev)
        bt = w.block_tables.long()
        sm = (bt[:, pos // w.block_size] * w.block_size + (pos % w.block_size).view(1, -1)).reshape(-1).contiguous()
    T = nk.shape[0]
    nb, B, H, D = w.key_cache.shape[0], w.block_size, w.num_kv_heads, w.head_size
    cdt = torch.uint8 if kv == "fp8" else nk.dtype
    if layout == "flash":
        kc = torch.zeros(nb, B, H, D, dtype=cdt, device=dev)
        vc = torch.zeros_like(kc)
        ours = ops.reshape_and_cache_flash
    else:
        x = 16 // (1 if kv == "fp8" else nk.element_size())
        kc = torch.zeros(nb, H, D // x, B, x, dtype=cdt, device=dev)
        vc = torch.zeros(nb, H, D, B, dtype=cdt, device=dev)
        ours = ops.reshape_and_cache
    nbytes = T * H * D * (2 * nk.element_size() + 2 * kc.element_size()) + 8 * T
    flush = L2Flush(dev)
    t = time_steps(lambda: ours(nk, nv, kc, vc, sm, kv, w.k_scale, w.v_scale), steps, warmup, flush)
    ms = float(np.mean(t))
    res = {
        "op": "reshape_and_cache" + ("_flash" if layout == "flash" else ""), "tokens": int(T),
        "kv_cache_dtype": kv, "ms": ms, "ms_min": float(np.min(t)), "bytes": int(nbytes),
        "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["copy"],
        "l2": "flushed between timed calls",
    }
    ref = ref_gpu_ops()
    if ref is not None:
        kr, vr = torch.zeros_like(kc), torch.zeros_like(vc)
        rfn = ref[1].reshape_and_cache_flash if layout == "flash" else ref[1].reshape_and_cache
        tr = time_steps(lambda: rfn(nk, nv, kr, vr, sm, kv, w.k_scale, w.v_scale), max(3, min(10, steps)), 2, flush)
        res["ref_gpu_ms"] = float(np.mean(tr))
        res["speedup_vs_ref_gpu"] = res["ref_gpu_ms"] / ms
        res["bit_equal_to_ref_gpu"] = bool(torch.equal(kr, kc) and torch.equal(vr, vc))
    return res


def _free():
    gc.collect()
    torch.cuda.empty_cache()


def extra_configs(dev, peaks, steps: int = 30, warmup: int = 5):
    """The benchmark configurations besides the headline one, on one GPU."""
    import workloads as W

    out = {}
    w = W.config1(dev)
    out["cfg1"] = dict(attention_case(w, "v1", steps, warmup, peaks), workload=w.name)
    del w
    _free()
    w = W.config3(dev)
    out["cfg3"] = dict(attention_case(w, "v2", steps, warmup, peaks), workload=w.name)
    out["cfg3w"] = write_case(w, "x", "fp8", steps, warmup, peaks)
    out["cfg3wf"] = write_case(w, "flash", "fp8", steps, warmup, peaks)
    out["cfg3w_auto"] = write_case(w, "x", "auto", steps, warmup, peaks)
    out["cfg3wf_auto"] = write_case(w, "flash", "auto", steps, warmup, peaks)
    out["cfg3w_decode"] = write_case(w, "x", "fp8", steps, warmup, peaks, tokens=256)
    out["cfg3w_decode1024"] = write_case(w, "x", "fp8", steps, warmup, peaks, tokens=1024)
    out["cfg3w_shifted"] = write_case(w, "x", "fp8", steps, warmup, peaks, shift=5)
    out["cfg3w_auto_shifted"] = write_case(w, "x", "auto", steps, warmup, peaks, shift=5)
    del w
    _free()
    w = W.config4(dev)
    out["cfg4"] = dict(attention_case(w, "v2", steps, warmup, peaks), workload=w.name)
    del w
    _free()
    w = W.config5(dev)
    out["cfg5"] = dict(attention_case(w, "v2", max(10, steps // 3), 3, peaks), workload=w.name)
    del w
    _free()
    return out


def strong_scaling(dev, world: int, rank: int, peaks, td, steps: int = 30, warmup: int = 5):
    """Strong scaling of the two sharded configurations.  Every rank builds the whole problem
    from the same seed and keeps its shard (KV heads of every block for the long-context one,
    sequences with a private block pool for the large-batch one); rank 0 also times the whole
    problem on its GPU.  No collective on the data path; after the timed region the shards'
    outputs are all-gathered over NCCL and compared with the unsharded result on rank 0."""
    import workloads as W

    assert world > 1
    res = {}
    for name, make, shard, gather_dim in (("cfg4", W.config4, W.shard_kv_heads, 1),
                                          ("cfg5", W.config5, W.shard_sequences, 0)):
        full = make(dev)
        tol = 2e-2 if full.kv_cache_dtype != "auto" else 1e-2
        n_steps = steps if name == "cfg4" else max(10, steps // 3)
        entry = {"sharding": "kv heads" if gather_dim == 1 else "sequences", "world": world,
                 "workload": full.name}
        want = None
        if rank == 0:
            one = attention_case(full, "v2", n_steps, warmup, peaks, with_ref=False)
            entry.update(t1_ms=one["ms"], t1_frac=one["frac"], bytes_total=one["bytes"])
            if world > 1:
                want = W.run_attention(full, version="v2").clone()
        mine = shard(full, world, rank)
        if rank != 0:
            del full
            _free()
        td.barrier()
        torch.cuda.synchronize()
        m = attention_case(mine, "v2", n_steps, warmup, peaks, with_ref=False)
        out = W.run_attention(mine, version="v2").contiguous()
        stats = torch.tensor([m["ms"], m["frac"], -m["frac"]], dtype=torch.float64, device=dev)
        td.all_reduce(stats, op=td.ReduceOp.MAX)
        # verification: assemble the shards over NCCL
        if gather_dim == 1:
            buf = torch.empty((world,) + tuple(out.shape), dtype=out.dtype, device=dev)
            td.all_gather_into_tensor(buf, out)
            got = buf.permute(1, 0, 2, 3).reshape(out.shape[0], -1, out.shape[2])
        else:
            got = torch.empty((out.shape[0] * world,) + tuple(out.shape[1:]), dtype=out.dtype, device=dev)
            td.all_gather_into_tensor(got, out)
        if rank == 0:
            diff = (got.float() - want.float()).abs()
            ok = bool(torch.allclose(got.float(), want.float(), atol=tol, rtol=tol))
            entry.update(tN_ms=float(stats[0]), efficiency=entry["t1_ms"] / (world * float(stats[0])),
                         shard_frac_max=float(stats[1]), shard_frac_min=float(-stats[2]),
                         shard_bytes_rank0=m["bytes"], l2=m["l2"],
                         verified=ok, max_abs_diff=float(diff.max()), tolerance=tol,
                         gathered_sequences=int(got.shape[0]))
            res[name] = entry
        del mine, out, got
        if rank == 0:
            del full, want
        _free()
    return res


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="cfg2",
                    choices=["cfg1", "cfg2", "cfg3", "cfg4", "cfg5", "cfg3w", "cfg3wf"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the other configurations and the strong-scaling section")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="cfg4 / cfg5: time rank 0's shard of an N-way sharded run on this GPU (for profiles)")
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

    if a.shard_of > 1 and world == 1:
        w, version, scaling = build_workload(a.workload, dev, a.shard_of, 0, a.num_seqs)
    else:
        w, version, scaling = build_workload(a.workload, dev, world, rank, a.num_seqs)
    cfg = {
        "workload": f"{w.name}: paged_attention_{version}, num_seqs={w.num_seqs} per GPU, "
                    f"{w.num_heads} query / {w.num_kv_heads} KV heads, head_size={w.head_size}, "
                    f"block_size={w.block_size}, kv_cache_dtype={w.kv_cache_dtype}, "
                    f"{w.total_tokens()} KV tokens on rank 0",
        "partitioning": "sequences per rank, no collective" if scaling == "weak" else
                        ("kv heads per rank" if a.workload == "cfg4" else "sequences per rank"),
        "l2": L2Flush.BIG if w.attn_bytes() > 4 * L2_BYTES else L2Flush.NOTE,
    }

    if a.impl == "reference":
        leg = cpu_reference_leg(w, a.steps, a.warmup, budget_s=120.0, min_s=10.0)
        if leg is None:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/_C_ref_cpu.so not built"}))
            return 0
        cfg["note"] = ("one host process on all cores; its throughput does not depend on --gpus "
                       "(it is the whole CPU side, whatever number of GPUs it is compared with)")
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

    td = None
    if dist:
        import datetime

        import torch.distributed as td
        td.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=600))

    from vllm_b200 import _custom_ops as ops  # noqa: F401  (fails loudly if the .so is missing)
    from vllm_b200 import capi
    import workloads as W

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
        kernel_name = "kv_write_staged_kernel (reshape_and_cache%s)" % ("_flash" if version == "cfg3wf" else "")
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
        flush = None if w.attn_bytes() > 4 * L2_BYTES else L2Flush(dev)
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

    # ---- end to end with host step inputs (pinned)
    e2e_how = "serial"
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
        ms_e2e = float(np.mean(time_steps(e2e_step, a.steps, 3, flush)))
    else:
        hq = w.query.cpu().pin_memory()
        hbt = w.block_tables.cpu().pin_memory()
        hsl = w.seq_lens.cpu().pin_memory()
        h2d = hq.numel() * hq.element_size() + hbt.numel() * 4 + hsl.numel() * 4
        d2h = hq.numel() * hq.element_size()
        wq, wbt, wsl = w.query, w.block_tables, w.seq_lens
        if flush is not None:
            # small workloads: copies and kernel in stream order, L2 flushed outside the intervals
            hout = torch.empty_like(hq).pin_memory()
            dq, dbt, dsl = torch.empty_like(wq), torch.empty_like(wbt), torch.empty_like(wsl)

            def e2e_step():
                dq.copy_(hq, non_blocking=True)
                dbt.copy_(hbt, non_blocking=True)
                dsl.copy_(hsl, non_blocking=True)
                w.query, w.block_tables, w.seq_lens = dq, dbt, dsl
                W.run_attention(w, out=out, version=version, scratch=scratch)
                hout.copy_(out, non_blocking=True)

            ms_e2e = float(np.mean(time_steps(e2e_step, a.steps, 3, flush)))
        else:
            # Every step's inputs go host -> device and its output device -> host inside the timed
            # region, double-buffered on two copy streams: the input copy of step i+1 and the
            # output copy of step i-1 run while the kernel of step i does (what an engine that
            # prepares the next step's metadata during the current one does).
            e2e_how = "copy streams: H2D of step i+1 and D2H of step i-1 overlap the kernel of step i"
            cur = torch.cuda.current_stream()
            s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
            dq = [torch.empty_like(wq) for _ in range(2)]
            dbt = [torch.empty_like(wbt) for _ in range(2)]
            dsl = [torch.empty_like(wsl) for _ in range(2)]
            douts = [torch.empty_like(wq) for _ in range(2)]
            houts = [torch.empty_like(hq).pin_memory() for _ in range(2)]
            ev_in = [torch.cuda.Event() for _ in range(2)]
            ev_k = [torch.cuda.Event() for _ in range(2)]
            ev_out = [torch.cuda.Event() for _ in range(2)]

            def run_pipeline(n):
                for i in range(n):
                    b = i & 1
                    with torch.cuda.stream(s_in):
                        if i >= 2:
                            s_in.wait_event(ev_k[b])     # the kernel of step i-2 has read these inputs
                        dq[b].copy_(hq, non_blocking=True)
                        dbt[b].copy_(hbt, non_blocking=True)
                        dsl[b].copy_(hsl, non_blocking=True)
                        ev_in[b].record(s_in)
                    cur.wait_event(ev_in[b])
                    if i >= 2:
                        cur.wait_event(ev_out[b])        # the output of step i-2 has left douts[b]
                    w.query, w.block_tables, w.seq_lens = dq[b], dbt[b], dsl[b]
                    W.run_attention(w, out=douts[b], version=version, scratch=scratch)
                    ev_k[b].record(cur)
                    with torch.cuda.stream(s_out):
                        s_out.wait_event(ev_k[b])
                        houts[b].copy_(douts[b], non_blocking=True)
                        ev_out[b].record(s_out)
                cur.wait_stream(s_out)
                cur.wait_stream(s_in)

            run_pipeline(4)
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s_in.wait_stream(cur)
            s_out.wait_stream(cur)
            e0.record(cur)
            s_in.wait_event(e0)
            run_pipeline(a.steps)
            e1.record(cur)
            barrier()
            ms_e2e = e0.elapsed_time(e1) / a.steps
            assert torch.equal(houts[(a.steps - 1) & 1], out.cpu()), "e2e output differs from the resident run"
        w.query, w.block_tables, w.seq_lens = wq, wbt, wsl
    clocks = sampler.stop()

    # ---- max over ranks, whole-job aggregate
    seqs_total = units_rank
    if dist:
        t = torch.tensor([ms, ms_e2e], dtype=torch.float64, device=dev)
        td.all_reduce(t, op=td.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])
        n = torch.tensor([seqs_total], dtype=torch.int64, device=dev)
        td.all_reduce(n)
        seqs_total = int(n[0])

    line = None
    peak, peak_kind = measured_peak()
    peaks = {"copy": peak, "read": None}
    if rank == 0:
        achieved = bytes_rank / (ms * 1e-3) / 1e9
        ratio = ncu_traffic_ratio(a.workload)
        line = {
            "metric": metric, "value": seqs_total / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": cfg, "clocks": clocks,
            "e2e": {"value": seqs_total / (ms_e2e * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                    "ms_per_step": ms_e2e, "how": e2e_how},
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
    # the headline workload's tensors are no longer needed on the device
    w_cpu_leg = w if (rank == 0 and world == 1 and not a.no_cpu_baseline and not is_write) else None
    if rank == 0 and w_cpu_leg is not None:
        try:
            leg = cpu_reference_leg(w_cpu_leg, steps=5, warmup=1)
        except Exception as ex:  # the baseline must never take the GPU number down with it
            leg = None
            line["cpu_baseline_error"] = repr(ex)
        if leg is not None:
            line["cpu_baseline"] = {k: leg[k] for k in ("value", "unit", "cores", "kind", "sample")}

    extras = a.workload == "cfg2" and not a.headline_only and a.num_seqs is None
    if extras:
        if rank == 0 and not is_write:
            ref = attention_case(w, version, 5, 2, {"copy": peak, "read": 1.0}) if ref_gpu_ops() else {}
            if "ref_gpu_ms" in ref:
                line["ref_gpu"] = {"ms": ref["ref_gpu_ms"], "speedup": ref["ref_gpu_ms"] / ms,
                                   "what": "the reference project's paged_attention_v2 CUDA kernels, built "
                                           "unmodified for sm_100a, same tensors, same event timing"}
        del w, w_cpu_leg
        if not is_write:
            del scratch, out
        _free()
        peaks["read"] = read_peak_gbs(dev)
        if rank == 0:
            line["peak_read_gbs"] = peaks["read"]
            line["roofline"]["frac_of_read_peak"] = line["roofline"]["achieved"] / peaks["read"]
        try:
            if world == 1:
                line["configs"] = extra_configs(dev, peaks)
                line["strong_scaling"] = {
                    k: {"world": 1, "t1_ms": line["configs"][k]["ms"], "tN_ms": line["configs"][k]["ms"],
                        "t1_frac": line["configs"][k]["frac"], "efficiency": 1.0, "verified": None,
                        "note": "one GPU: nothing to shard"} for k in ("cfg4", "cfg5")}
            else:
                ss = strong_scaling(dev, world, rank, peaks, td)
                if rank == 0:
                    line["strong_scaling"] = ss
        except Exception as ex:  # keep the headline even if a side measurement fails
            if rank == 0:
                line["extras_error"] = repr(ex)
            else:
                raise
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist:
        td.barrier()
        td.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
