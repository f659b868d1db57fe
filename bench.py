"""Benchmark of the hot path: the bandwidth-bound fused defn.

Workload (the second configuration of BASELINE.json): logits f32 {8192,32768}
normal(0,2) from seed 1; ONE defn that returns row max, exp(x-max), its sum,
logsumexp, softmax, argmax per row and the chain tanh(x*0.5+0.1)*sigmoid(x).
The compiler turns it into a single row kernel, so one step = one launch that
reads x once (1 GiB) and writes the three full-size outputs (3 GiB) plus four
per-row vectors.  ``value`` = those algorithmic bytes / device time.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 runs one replica per GPU (the configuration has no cross-device
exchange; "replicas only"), launched by torch.distributed.run, and reports the
aggregate.  ``--impl reference`` times the CPU restatement of the same graph
(oracle/rows_oracle.c, all host threads) on a bounded sample of rows.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

ROWS, COLS = 8192, 32768
SEED = 1
METRIC, UNIT = "fused-op HBM GB/s", "GB/s"

# DRAM bytes per launch of the row kernel measured once under ncu
# (dram__bytes_read.sum + dram__bytes_write.sum; see profiles/).  None until captured.
NCU_TRAFFIC_BYTES_PER_LAUNCH = None


def algorithmic_bytes(rows, cols):
    """Each distinct input read once + each output written once."""
    full = rows * cols * 4
    return full * 4 + rows * 4 * 4          # x, exp, softmax, chain; max, sum, lse (f32) + argmax (s32)


def fused_rows(x):
    from nx_b200 import nx
    m = nx.reduce_max(x, axes=[1], keep_axes=True)
    e = nx.exp(x - m)
    s = nx.sum(e, axes=[1], keep_axes=True)
    return (nx.squeeze(m, [1]), e, nx.squeeze(s, [1]), nx.logsumexp(x, axes=[1]), e / s,
            nx.argmax(x, axis=1), nx.tanh(x * 0.5 + 0.1) * nx.sigmoid(x))


def make_input(rows, cols, seed):
    rng = np.random.default_rng(seed)
    out = np.empty((rows, cols), dtype=np.float32)
    step = max(1, (1 << 24) // cols)
    for r in range(0, rows, step):
        out[r:r + step] = rng.standard_normal((min(step, rows - r), cols), dtype=np.float32) * 2.0
    return out


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def load_rows_oracle():
    path = os.path.join(ROOT, "oracle", "librows_oracle.so")
    if not os.path.exists(path):
        subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle")], check=True)
    lib = C.CDLL(path)
    lib.rows_oracle.restype = None
    lib.rows_oracle.argtypes = [C.c_void_p, C.c_int64, C.c_int64] + [C.c_void_p] * 7
    lib.rows_oracle_threads.restype = C.c_int
    return lib


def cpu_rows(lib, x):
    rows, cols = x.shape
    outs = [np.empty(rows, np.float32), np.empty((rows, cols), np.float32), np.empty(rows, np.float32),
            np.empty(rows, np.float32), np.empty((rows, cols), np.float32), np.empty(rows, np.int32),
            np.empty((rows, cols), np.float32)]
    t0 = time.perf_counter()
    lib.rows_oracle(x.ctypes.data, rows, cols, *[o.ctypes.data for o in outs])
    return time.perf_counter() - t0, outs


def cpu_baseline(x_sample):
    lib = load_rows_oracle()
    cpu_rows(lib, x_sample[:8])                      # page in / spin up the thread pool
    dt, _ = cpu_rows(lib, x_sample)
    gbs = algorithmic_bytes(*x_sample.shape) / dt / 1e9
    return {"value": round(gbs, 3), "unit": UNIT, "cores": lib.rows_oracle_threads(), "kind": "port",
            "sample": f"{x_sample.shape[0]} of {ROWS} rows x {COLS} cols, one pass, {dt:.2f} s"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    lib = load_rows_oracle()
    rows = 1024                                        # bounded sample: 0.5 GiB of algorithmic traffic per step
    x = make_input(rows, COLS, SEED)
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_rows(lib, x[:64])
    times = [cpu_rows(lib, x)[0] for _ in range(args.steps)]
    dt = sum(times) / len(times)
    gbs = algorithmic_bytes(rows, COLS) / dt / 1e9
    line = {"impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3 * ROWS / rows, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "fused row defn f32 {8192,32768} (max, exp, sum, logsumexp, softmax, argmax, tanh*sigmoid chain)",
                       "sample_rows": rows},
            "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": lib.rows_oracle_threads(), "kind": "port",
                             "sample": f"{rows} of {ROWS} rows per step; ms_per_step is scaled to the full {ROWS} rows"},
            "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS, help="reduced row count (profiling captures only)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank, world)
    args.warmup = max(args.warmup, 3)

    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from nx_b200 import backend, defn, nif, nx
    backend.set_default_backend("b200", local)
    lib = nif.lib()
    rows = args.rows
    x_host = make_input(rows, COLS, SEED)
    x = nx.tensor(x_host)
    step_fn = defn.compile(fused_rows, [defn.template((rows, COLS), "f32")], device=local)
    prog = step_fn.program
    outs = prog.run([x], local)                       # allocates the output buffers once
    nbytes = algorithmic_bytes(rows, COLS)

    def barrier():
        nif.check(lib.nxb200_device_synchronize(local))
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        prog.run_into([x], outs, local)
    barrier()
    sampler = ClockSampler(local)
    nif.check(lib.nxb200_timer_begin(local))
    for _ in range(args.steps):
        prog.run_into([x], outs, local)
    ms = C.c_float()
    nif.check(lib.nxb200_timer_end(local, C.byref(ms)))
    barrier()
    clocks = sampler.stop()
    elapsed_ms = ms.value
    if dist is not None:
        t = torch.tensor([elapsed_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / args.steps
    value = world * nbytes / (ms_per_step * 1e-3) / 1e9
    per_gpu = nbytes / (ms.value / args.steps * 1e-3) / 1e9

    # ---- end to end: host buffers in, host buffers out, through the same public call ----
    e2e = None
    if not args.no_e2e:
        pin_in = torch.empty(x_host.nbytes, dtype=torch.uint8, pin_memory=True)
        pin_in.numpy()[:] = x_host.reshape(-1).view(np.uint8)
        out_bytes = [o.size * 4 for o in outs]
        pin_out = [torch.empty(n, dtype=torch.uint8, pin_memory=True) for n in out_bytes]
        e2e_steps = max(2, min(args.steps, 5))

        def one():
            nif.check(lib.nxb200_buffer_write_async(x.data.handle, pin_in.data_ptr(), x_host.nbytes))
            prog.run_into([x], outs, local)
            for o, p, n in zip(outs, pin_out, out_bytes):
                nif.check(lib.nxb200_buffer_read_async(o.data.handle, p.data_ptr(), n))
            nif.check(lib.nxb200_device_synchronize(local))

        one()
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            one()
        dt = (time.perf_counter() - t0) / e2e_steps
        if dist is not None:
            t = torch.tensor([dt], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e = {"value": round(world * nbytes / dt / 1e9, 3), "unit": UNIT, "h2d_bytes_per_step": int(x_host.nbytes),
               "d2h_bytes_per_step": int(sum(out_bytes)), "ms_per_step": round(dt * 1e3, 3), "steps": e2e_steps}

    if rank == 0:
        peak, which = peaks()
        line = {"metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "fused row defn f32 {%d,32768} (max, exp, sum, logsumexp, softmax, argmax, tanh*sigmoid chain)" % rows,
                           "seed": SEED, "parallelism": "replicas only" if world > 1 else "single GPU",
                           "l2": "inputs (1 GiB) and outputs (3 GiB) per step are larger than L2 (126 MB); no flush needed"},
                "roofline": {"bound": "hbm", "achieved": round(per_gpu, 2), "peak": peak, "unit": "GB/s",
                             "frac": round(per_gpu / peak, 4), "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH,
                             "peak_source": f"of {which}", "kernel": "nxb_k0_row",
                             "algorithmic_bytes_per_launch": nbytes},
                "clocks": clocks, "gpu_launches": args.steps * prog.launch_count(), "e2e": e2e,
                "plan": prog.describe().strip().split("\n")}
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(x_host[:min(rows, 1024)])
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
