#!/usr/bin/env python
"""Benchmark of the JSON parse + validate path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--records R] [--impl reference]

One step = one pass of the hot path (line index, validation, typed-column emission: one kernel) over one batch of
synthetic Petstore `Pet` records held as NDJSON: R = 1,000,000 records per GPU (~295 MB, the single-GPU benchmark
configuration), regenerated from a fixed seed on every run.

  value        records/s with the input already resident in HBM and the columns left in HBM
  e2e          the same through host buffers: pinned host text in, every column copied back to pinned host memory,
               both inside the timed region
  roofline     algorithmic bytes (input + every produced column) / device time of the parse kernel, against the
               measured HBM copy bandwidth
  reserialise  the reverse direction (columns -> JSON) on the parsed columns, reported beside it
  cpu_baseline the CPU restatement of the reference path (oracle/) on this box's host cores; the JVM reference
               itself cannot run here

`--impl reference` times only that CPU restatement, on all host threads, and prints the same line shape.

With N > 1 (launched under torchrun, one rank per GPU) rank 0 owns a pj_group over the N GPUs: one process, one host
thread and stream per device inside the library, shard g of the stream resident on GPU g, the head of shard g+1
copied device to device behind shard g, one ncclAllGather of the counter table. The other ranks take part in the
barriers and hold no GPU work; timing is taken on rank 0 around the synchronous group call (the per-shard kernel
times come from CUDA events inside the library). Every shard's columns are checked against the generator's values
outside the timed region.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import ctypes as C
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED = 0x5EED
SLACK = 64 * 1024
FALLBACK_HBM_GBS = 6650.0  # an earlier measurement, used only when MEASURED_PEAKS.json is absent
# dram__bytes_read.sum + dram__bytes_write.sum of the parse kernel per record, from one ncu capture per workload at
# 500 000 records (traffic grows with the record count); None = no capture of that workload
TRAFFIC_BYTES_PER_RECORD = {"pet": 413, "mixed": None, "zipf": None, "array1k": None}


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ---- CPU restatement of the reference path (oracle/) -------------------------------------------------
class CpuPort:
    """The scalar C restatement, run on T host threads over LF-aligned byte ranges of the sample."""

    def __init__(self):
        build = importlib.import_module("micronaut3-bug_b200.build")
        self.abi = importlib.import_module("micronaut3-bug_b200.abi")
        self.lib = C.CDLL(build.build_oracle())

    def parse_ranges(self, text: np.ndarray, threads: int) -> tuple[int, float]:
        abi = self.abi
        cuts = [0]
        for t in range(1, threads):
            p = text.size * t // threads
            nl = np.nonzero(text[p:p + 100000] == 10)[0]
            cuts.append(p + int(nl[0]) + 1 if nl.size else text.size)
        cuts.append(text.size)
        parts = [text[cuts[i]:cuts[i + 1]] for i in range(threads) if cuts[i + 1] > cuts[i]]
        outs = [abi.HostColumns(abi.PJ_SCHEMA_PET, abi.default_caps(abi.PJ_SCHEMA_PET, int(np.count_nonzero(p == 10)) + 2, p.size, p.size // 20)) for p in parts]

        def run(i):
            p = parts[i]
            st = self.lib.pjo_parse(C.c_uint32(abi.PJ_SCHEMA_PET), C.c_uint32(0), C.c_void_p(p.ctypes.data), C.c_uint64(p.size), C.c_uint64(0), 1, 1,
                                    C.c_uint64(0), C.byref(outs[i].raw))
            assert st == 0
            return outs[i].n_records

        t0 = time.perf_counter()
        with cf.ThreadPoolExecutor(max_workers=len(parts)) as ex:
            n = sum(ex.map(run, range(len(parts))))
        return n, time.perf_counter() - t0


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


def run_reference(args, pj, abi):
    """`--impl reference`: the CPU restatement on all host threads; each step parses a bounded sample."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    sample = args.records  # the whole workload of the GPU arm every step (1 M records: about 0.1 s on 16 threads)
    text = pj.gen_text(abi.PJ_SCHEMA_PET, SEED, 0, sample, 0)
    port = CpuPort()
    for _ in range(args.warmup):
        port.parse_ranges(text, threads)
    total_t, total_n = 0.0, 0
    for _ in range(args.steps):
        n, dt = port.parse_ranges(text, threads)
        total_t += dt; total_n += n
    rps = total_n / total_t
    line = {
        "impl": "reference", "metric": "pet_ndjson_parse_validate_records_per_s", "value": rps, "unit": "records/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total_t / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": {"workload": "1M Pet records as NDJSON, one record per line (BASELINE configs[1])", "records_per_gpu": args.records,
                   "seed": SEED, "sample_records_per_step": sample},
        "gb_per_s": rps * text.size / sample / 1e9,
        "cpu_baseline": {"value": rps, "unit": "records/s", "cores": threads, "kind": "port",
                         "sample": f"{sample} Pet records ({text.size / 1e6:.1f} MB) per step, split into {threads} LF-aligned ranges, one thread each; "
                                   "CPU restatement in C (oracle/), not the JVM reference, which cannot run on this box"},
        "e2e": {"value": rps, "unit": "records/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    _emit_line(line)


WORKLOADS = {
    "pet": "1M Pet records as NDJSON, one record per line (BASELINE configs[1])",
    "mixed": "Pet/Order/User 50/30/20 with 1% malformed records as NDJSON (BASELINE configs[2] distributions)",
    "zipf": "Pets with zipf(1.2) list lengths, 5% escaped strings, random blanks as NDJSON (BASELINE configs[3] distributions)",
    "array1k": "JSON array of 1000 Pets (BASELINE configs[0]); launch-latency bound at this size",
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--records", type=int, default=1_000_000, help="records per GPU and step")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", default="pet", choices=sorted(WORKLOADS), help="pet: 1M Pet records (the headline configuration); mixed: Pet/Order/User 50/30/20 with 1%% malformed; zipf: Pets with zipf(1.2) list lengths, 5%% escaped strings, random blanks; array1k: a JSON array of 1000 Pets (the reference's own CPU-runnable case), parse and re-serialise")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--host-piece-bytes", type=int, default=0, help="pj_options.host_piece_bytes of the end-to-end leg (0 = library default)")
    ap.add_argument("--tile-bytes", type=int, default=0, help="pj_options.tile_bytes (0 = chosen by the library)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    pj = importlib.import_module("micronaut3-bug_b200")
    abi = pj.abi
    build = importlib.import_module("micronaut3-bug_b200.build")
    build.build_generator()  # no-ops when the libraries are up to date
    if args.impl == "reference":
        return run_reference(args, pj, abi)  # maps the generator and the CPU restatement, nothing of the GPU library
    build.build_library()

    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; there is no CPU fallback for the product path (use --impl reference)")
    if world > 1:
        return run_group(args, pj, abi, world)
    return run_single(args, pj, abi)


def gen_setup(args, abi):
    mixed_wl = args.workload in ("mixed", "zipf")  # side workloads: parse only, no end-to-end or CPU leg
    array_wl = args.workload == "array1k"
    if array_wl:
        args.records = 1000
    schema = abi.PJ_SCHEMA_MIXED if args.workload == "mixed" else abi.PJ_SCHEMA_PET
    gen_flags = {"pet": 0, "mixed": abi.PJ_GEN_MALFORMED, "zipf": abi.PJ_GEN_ZIPF_LISTS | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE,
                 "array1k": abi.PJ_GEN_ARRAY}[args.workload]
    if mixed_wl or array_wl:
        args.no_e2e = True
        args.no_cpu_baseline = True
    return schema, gen_flags, mixed_wl, array_wl


def cpu_baseline(text_np, R):
    threads = host_threads()
    sample = min(R, 200_000)
    port = CpuPort()
    sample_text = text_np[: int(np.nonzero(text_np == 10)[0][sample - 1]) + 1]
    port.parse_ranges(sample_text, threads)
    reps, tot = 0, 0.0
    while tot < 10.0 and reps < 20:
        n, dt = port.parse_ranges(sample_text, threads)
        tot += dt; reps += 1
    n1, dt1 = port.parse_ranges(sample_text, 1)
    return {"value": sample * reps / tot, "unit": "records/s", "cores": threads, "kind": "port",
            "single_thread_records_per_s": n1 / dt1,
            "sample": f"{sample} Pet records ({sample_text.size / 1e6:.1f} MB) x {reps} passes, {threads} LF-aligned ranges, one thread each; "
                      "CPU restatement in C (oracle/), not the JVM reference, which cannot run on this box"}


def roofline_block(args, alg_bytes, k_ms, whole_ms, R, kernel_name):
    peak, peak_src = measured_peak()
    k_achieved = alg_bytes / (k_ms * 1e-3) / 1e9
    achieved = alg_bytes / (whole_ms * 1e-3) / 1e9
    per_rec = TRAFFIC_BYTES_PER_RECORD.get(args.workload)
    return {"bound": "hbm", "achieved": k_achieved, "peak": peak, "unit": "GB/s", "frac": k_achieved / peak,
            "traffic": per_rec * R if per_rec else None, "peak_source": peak_src + " HBM copy bandwidth", "kernel": kernel_name,
            "algorithmic_bytes_per_launch": int(alg_bytes), "kernel_ms_per_launch": k_ms,
            "note": "algorithmic bytes = input + every produced column (the 8-byte record starts included: the kernel finds them itself)",
            "whole_step": {"achieved": achieved, "frac": achieved / peak, "device_ms_per_step": whole_ms}}


def run_single(args, pj, abi):
    import torch

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    PET, gen_flags, mixed_wl, array_wl = gen_setup(args, abi)
    R = args.records
    framing = abi.PJ_FRAMING_ARRAY if array_wl else abi.PJ_FRAMING_NDJSON

    text_np = pj.gen_text(PET, SEED, 0, R, gen_flags)
    nbytes = int(text_np.size)
    h_text = torch.empty(nbytes + SLACK, dtype=torch.uint8).pin_memory()
    h_text[:nbytes].copy_(torch.from_numpy(text_np))
    d_text = torch.zeros(nbytes + SLACK, dtype=torch.uint8, device=dev)
    d_text[:nbytes].copy_(h_text[:nbytes], non_blocking=True)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device=dev)  # the library launches on this stream; the timing events are recorded on it
    torch.cuda.set_stream(stream)
    ctx = pj.Context(device=0, inclusion=abi.PJ_INCLUDE_NON_NULL, stream=stream.cuda_stream, host_piece_bytes=args.host_piece_bytes,
                     tile_bytes=args.tile_bytes)
    cols = pj.DeviceColumns.sized_for(PET, R + 16, nbytes + SLACK, max(6 * R, (nbytes + SLACK) // 12), dev)
    torch.cuda.synchronize()

    launches = 0
    stage_ms = np.zeros(8)
    for _ in range(args.warmup):
        ctx.parse(PET, d_text[:nbytes], cols, framing)
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    sampler.start()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        ctx.parse(PET, d_text[:nbytes], cols, framing)
        st = ctx.stats()
        launches += st.kernel_launches
        stage_ms += np.array(list(st.stage_ms))
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop()
    n_rec = cols.n_records
    last_stats = ctx.stats()
    alg_bytes = last_stats.algorithmic_bytes
    assert n_rec == R and (mixed_wl or cols.n_errors == 0), (n_rec, cols.n_errors)

    # ---- the reverse direction on the parsed columns ------------------------------------------------------
    d_out = torch.empty(nbytes + 64, dtype=torch.uint8, device=dev)
    w_ms, w_dev_ms, w_launch, w_alg, w_len, w_kernel_ms, w_phase = 0.0, 0.0, 0, 0, 0, 0.0, []
    wsteps = max(3, args.steps // 2)
    if not mixed_wl:
        for _ in range(3):
            ctx.write(PET, cols, d_out, framing)
        torch.cuda.synchronize()
        w0, w1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        w0.record(stream)
        for _ in range(wsteps):
            w_len = ctx.write(PET, cols, d_out, framing)
            st = ctx.stats()
            w_dev_ms += st.device_ms; w_launch += st.kernel_launches; w_alg = st.algorithmic_bytes
            w_kernel_ms += st.main_kernel_ms; w_phase = [int(x) // max(int(st.tiles), 1) for x in st.phase_cycles]
        w1.record(stream)
        torch.cuda.synchronize()
        w_ms = w0.elapsed_time(w1)
        assert w_len == nbytes and torch.equal(d_out[:nbytes], d_text[:nbytes]), "re-serialised bytes differ from the input"

    # ---- end to end through host buffers ------------------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        pin = lambda n: torch.empty(n, dtype=torch.uint8).pin_memory().numpy()
        caps = {c.id: int(cols.raw.col[c.id].bytes) for c in abi.schema_columns(PET)}
        hcols = abi.HostColumns(PET, {k: min(v, max(cols.count(k) * 8 + 64, 64)) for k, v in caps.items()}, alloc=pin)
        h_np = h_text.numpy()[:nbytes]
        for _ in range(2):
            ctx.parse(PET, h_np, hcols)
        torch.cuda.synchronize()
        esteps = max(3, args.steps // 4)
        t0 = time.perf_counter()
        for _ in range(esteps):
            ctx.parse(PET, h_np, hcols)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        st = ctx.stats()
        assert hcols.n_records == R
        e2e = {"value": R * esteps / dt, "unit": "records/s", "h2d_bytes_per_step": int(st.h2d_bytes), "d2h_bytes_per_step": int(st.d2h_bytes),
               "ms_per_step": 1e3 * dt / esteps, "steps": esteps, "pieces": int(st.pieces),
               "note": "pinned host text in, every column back to pinned host memory; the library overlaps the copies of one piece with the kernel of the next"}

    k_ms = stage_ms[2] / args.steps
    line = {
        "metric": "pet_ndjson_parse_validate_records_per_s",
        "value": n_rec * args.steps / (ms * 1e-3),
        "unit": "records/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": WORKLOADS[args.workload], "records_per_gpu": R, "seed": SEED, "input_bytes_per_gpu": nbytes,
                   "l2": "input (295 MB at 1M records) and columns are larger than the 126 MB L2; no flush between steps", "sharding": "single GPU"},
        "gb_per_s": n_rec * args.steps / (ms * 1e-3) * nbytes / R / 1e9,
        "roofline": roofline_block(args, alg_bytes, k_ms, ms / args.steps, R,
                                   "k_parse_tile over the array index (one launch per step)" if array_wl else
                                   "k_parse_stream (line index, tokenising, validation and emission of one tile per block; one launch per step)"),
        "gpu_launches": launches,
        "tile_kernel": {"threads_per_block": int(last_stats.tile_records), "blocks": int(last_stats.tiles), "fast_records": int(last_stats.fast_records),
                        "phase_cycles_per_block": [int(x) // max(int(last_stats.tiles), 1) for x in last_stats.phase_cycles],
                        "wide_records": int(last_stats.wide_records), "wide_fast_records": int(last_stats.wide_fast_records),
                        "wide_cycles_per_block": [int(x) // max(int(last_stats.tiles), 1) for x in last_stats.wide_cycles],
                        "lookback_polls": int(last_stats.lookback_polls), "lookback_rounds": int(last_stats.lookback_rounds)},
        "clocks": clocks,
        "e2e": e2e,
    }
    if w_ms:
        peak, _ = measured_peak()
        wa = w_alg / (w_dev_ms / wsteps * 1e-3) / 1e9
        line["reserialise"] = {"records_per_s": R * wsteps / (w_ms * 1e-3), "gb_per_s_out": nbytes * wsteps / (w_ms * 1e-3) / 1e9, "ms_per_step": w_ms / wsteps,
                               "steps": wsteps, "gpu_launches": w_launch, "byte_identical_to_input": True,
                               "roofline": {"bound": "hbm", "achieved": wa, "peak": peak, "unit": "GB/s", "frac": wa / peak, "traffic": None,
                                            "algorithmic_bytes_per_step": int(w_alg), "kernel": "k_write_tile", "kernel_ms_per_launch": w_kernel_ms / wsteps,
                                            "kernel_achieved": w_alg / (w_kernel_ms / wsteps * 1e-3) / 1e9,
                                            "phase_cycles_per_block": w_phase}}
    if not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(text_np, R)
    _emit_line(line)


def run_group(args, pj, abi, world):
    """N > 1: rank 0 drives all N GPUs through pj_group_*; the other ranks only keep the launcher's barriers."""
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")  # NCCL's banner must not land on stdout: one JSON line only
    dist.init_process_group("gloo")  # between the ranks only barriers travel; the GPUs' exchange is inside the library
    if rank != 0:
        dist.barrier()  # start of the timed region
        dist.barrier()  # end of it
        dist.barrier()  # rank 0 has printed
        dist.destroy_process_group()
        return
    assert torch.cuda.device_count() >= world, f"{world} ranks, {torch.cuda.device_count()} visible GPUs"
    PET, gen_flags, mixed_wl, array_wl = gen_setup(args, abi)
    assert not array_wl, "array framing does not shard"
    R = args.records
    devices = list(range(world))
    texts, bufs, lens, cols = [], [], [], []
    for g in devices:
        t = pj.gen_text(PET, SEED, g * R, R, gen_flags)  # shard g = records [gR, (g+1)R) of the stream
        texts.append(t)
        d = torch.zeros(t.size + SLACK, dtype=torch.uint8, device=f"cuda:{g}")
        d[: t.size].copy_(torch.from_numpy(t))
        bufs.append(d); lens.append(int(t.size))
        cols.append(pj.DeviceColumns.sized_for(PET, R + 16, t.size + SLACK, max(6 * R, (t.size + SLACK) // 12), f"cuda:{g}"))
    for g in devices:
        torch.cuda.synchronize(g)
    grp = pj.Group(devices, inclusion=abi.PJ_INCLUDE_NON_NULL, tile_bytes=args.tile_bytes)

    def sync_all():
        for g in devices:
            torch.cuda.synchronize(g)

    for _ in range(args.warmup):
        grp.parse(PET, bufs, lens, cols, SLACK)
    sync_all()
    dist.barrier()
    sampler = ClockSampler(0)
    sampler.start()
    kernel_ms = np.zeros(world)
    copy_ms = np.zeros(world)
    gather_ms = np.zeros(world)
    launches = 0
    prep = grp.prepare_parse(PET, bufs, lens, cols, SLACK)
    grp.parse_prepared(prep)
    sync_all()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        shards = grp.parse_prepared(prep)  # returns when every shard's kernels and the counter exchange are done
    sync_all()
    ms = 1e3 * (time.perf_counter() - t0)
    for g in devices:  # per-shard figures of the last step stand for all of them (the library keeps one call's statistics)
        st = grp.stats(g)
        kernel_ms[g] = st.stage_ms[2] * args.steps; launches += (st.kernel_launches + 1) * args.steps  # + the counter kernel of the exchange
        copy_ms[g] = shards[g].slack_copy_ms * args.steps; gather_ms[g] = shards[g].gather_ms * args.steps
    dist.barrier()
    clocks = sampler.stop()
    total_rec = sum(c.n_records for c in cols)
    assert total_rec == world * R, (total_rec, world * R)
    alg_bytes = sum(int(grp.stats(g).algorithmic_bytes) for g in devices)

    # ---- every shard's columns against the generator's values (outside the timed region) ------------------
    sharded_check = "ok"
    off = 0
    for g in devices:
        first = g * R + (1 if g else 0)                       # the record at a shard's byte 0 belongs to the shard before it
        n = R - (1 if g else 0) + (1 if g < world - 1 else 0)  # ... and a shard also takes the first record of the next one
        assert cols[g].n_records == n and (mixed_wl or cols[g].n_errors == 0), (g, cols[g].n_records, n)
        span = sum(lens) + 64
        want = pj.gen_columns(PET, SEED, first, n, gen_flags, min(span, lens[g] + (lens[g + 1] if g + 1 < world else 0) + 64))
        got = {c.name: cols[g].get(c.name) for c in abi.schema_columns(PET)}
        exp = want.as_dict()
        lf = np.nonzero(texts[g] == 10)[0]
        start0 = off + (int(lf[0]) + 1 if g else 0)           # where the shard's first own record starts in the stream
        for name, a in got.items():
            e = exp[name]
            if name == "rec_start":
                e = e - e[0] + np.uint64(start0) if e.size else e
            if a.shape != e.shape or not np.array_equal(a, e):
                sharded_check = f"shard {g}: column {name} differs"
                break
        off += lens[g]
        if sharded_check != "ok":
            break
    if sharded_check != "ok":
        raise SystemExit("bench.py: " + sharded_check)

    # ---- the reverse direction: every GPU serialises its own table ----------------------------------------
    outs = [torch.empty(lens[g] + SLACK + 64, dtype=torch.uint8, device=f"cuda:{g}") for g in devices]
    reser = None
    if not mixed_wl:
        for _ in range(3):
            grp.write(PET, cols, outs)
        sync_all()
        wsteps = max(3, args.steps // 2)
        w_kernel = np.zeros(world)
        t0 = time.perf_counter()
        for _ in range(wsteps):
            wsh = grp.write(PET, cols, outs)
            for g in devices:
                w_kernel[g] += grp.stats(g).main_kernel_ms
        sync_all()
        w_ms = 1e3 * (time.perf_counter() - t0)
        out_bytes = sum(int(s.bytes) for s in wsh)
        w_alg = sum(int(grp.stats(g).algorithmic_bytes) for g in devices)
        # shard g's text = the bytes of the records it owns
        off = 0
        for g in devices:
            lf = np.nonzero(texts[g] == 10)[0]
            lo = int(lf[0]) + 1 if g else 0
            own = texts[g][lo:]
            if g + 1 < world:
                lf2 = np.nonzero(texts[g + 1] == 10)[0]
                own = np.concatenate([own, texts[g + 1][: int(lf2[0]) + 1]])
            assert int(wsh[g].bytes) == own.size and int(wsh[g].global_offset) == off, (g, int(wsh[g].bytes), own.size)
            assert np.array_equal(outs[g][: own.size].cpu().numpy(), own), f"shard {g}: re-serialised bytes differ from the input"
            off += own.size
        peak, _ = measured_peak()
        reser = {"records_per_s": total_rec * wsteps / (w_ms * 1e-3), "gb_per_s_out": out_bytes * wsteps / (w_ms * 1e-3) / 1e9, "ms_per_step": w_ms / wsteps,
                 "steps": wsteps, "byte_identical_to_input": True, "kernel_ms_per_shard": (w_kernel / wsteps).tolist(),
                 "roofline": {"bound": "hbm", "unit": "GB/s", "peak": peak, "kernel": "k_write_tile",
                              "achieved_per_gpu": w_alg / world / (float(w_kernel.max()) / wsteps * 1e-3) / 1e9,
                              "frac": w_alg / world / (float(w_kernel.max()) / wsteps * 1e-3) / 1e9 / peak, "traffic": None}}

    # ---- end to end: pinned host text to every GPU, the group call, every column back to pinned host memory
    e2e = None
    if not args.no_e2e:
        pin = lambda nb: torch.empty(nb, dtype=torch.uint8).pin_memory().numpy()
        h_all = pin(sum(lens) + 64)  # the whole stream in one pinned buffer: the shards are ranges of it
        off = 0
        for t in texts:
            h_all[off: off + t.size] = t
            off += t.size
        hcols = [abi.HostColumns(PET, {c.id: max(cols[g].count(c.id) * np.dtype(c.dtype).itemsize + 64, 64) for c in abi.schema_columns(PET)}, alloc=pin) for g in devices]
        for _ in range(2):
            grp.parse_host(PET, h_all[: sum(lens)], lens, hcols, SLACK)
        esteps = max(3, args.steps // 4)
        t0 = time.perf_counter()
        for _ in range(esteps):
            grp.parse_host(PET, h_all[: sum(lens)], lens, hcols, SLACK)
        dt = time.perf_counter() - t0
        assert sum(h.n_records for h in hcols) == total_rec
        h2d = sum(int(grp.stats(g).h2d_bytes) for g in devices)
        d2h = sum(int(grp.stats(g).d2h_bytes) for g in devices)
        e2e = {"value": total_rec * esteps / dt, "unit": "records/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": 1e3 * dt / esteps, "steps": esteps,
               "note": "pj_group_parse_host: one pinned host stream in, every shard through the host-buffer route of its GPU side by side (pieces overlap copies and kernels), every column of every shard back to pinned host memory"}

    k_ms = float(kernel_ms.max()) / args.steps
    line = {
        "metric": "pet_ndjson_parse_validate_records_per_s",
        "value": total_rec * args.steps / (ms * 1e-3),
        "unit": "records/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": ms / args.steps,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "u8",
        "data": "synthetic",
        "config": {"workload": WORKLOADS[args.workload], "records_per_gpu": R, "seed": SEED, "input_bytes_per_gpu": lens[0],
                   "l2": "input (295 MB at 1M records) and columns are larger than the 126 MB L2; no flush between steps",
                   "sharding": f"one byte range per GPU, {SLACK // 1024} KiB slack copied from the next GPU (peer copy), counter table by ncclAllGather; "
                               "one process (rank 0) drives the GPUs through pj_group_parse, one host thread per GPU inside the library",
                   "timing": "host clock on rank 0 around the synchronous group calls, between barriers; kernel times from CUDA events inside the library"},
        "gb_per_s": total_rec * args.steps / (ms * 1e-3) * sum(lens) / total_rec / 1e9,
        "roofline": roofline_block(args, alg_bytes / world, k_ms, ms / args.steps, R,
                                   "k_parse_stream, one launch per GPU and step (slowest GPU; algorithmic bytes per GPU)"),
        "gpu_launches": launches,
        "uses_nccl": grp.uses_nccl,
        "sharded_check": sharded_check,
        "kernel_ms_per_shard": (kernel_ms / args.steps).tolist(),
        "stitch_ms_per_step": {"slack_copy": float(copy_ms.max()) / args.steps, "counter_exchange_enqueue": float(gather_ms.max()) / args.steps,
                               "host_and_launch": max(ms / args.steps - k_ms - float(copy_ms.max()) / args.steps - float(gather_ms.min()) / args.steps, 0.0)},
        "clocks": clocks,
        "e2e": e2e,
    }
    if reser:
        line["reserialise"] = reser
    _emit_line(line)
    grp.close()
    dist.barrier()
    dist.destroy_process_group()


def _emit_line(line: dict) -> None:
    """The one JSON line, written to the process's original stdout (see _quiet_stdout)."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = 1


def _quiet_stdout() -> None:
    """Native libraries (NCCL's version banner, for one) print to file descriptor 1. The contract is ONE JSON line on
    stdout, so descriptor 1 is pointed at stderr for the whole run and the line goes to a saved copy of the original."""
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)


if __name__ == "__main__":
    _quiet_stdout()
    main()
