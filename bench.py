"""Benchmark of the hot path.

Headline workload (the second configuration of BASELINE.json, the one the
metric "fused-op HBM GB/s" is quoted on): logits f32 {8192,32768} normal(0,2)
from seed 1; ONE defn returning row max, exp(x-max), its sum, logsumexp,
softmax, argmax per row and the chain tanh(x*0.5+0.1)*sigmoid(x).  The compiler
turns it into a single row kernel, so one step = one launch that reads x once
(1 GiB) and writes the three full-size outputs (3 GiB) plus four per-row
vectors.  ``value`` = those algorithmic bytes / device time, whole job.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--all-configs]

N > 1 (launched by torch.distributed.run, one rank per GPU): the headline
configuration has no cross-device exchange, so it runs as independent replicas
("replicas only", weak scaling) and the aggregate is reported.  The sharded
configuration (the decoder block) is timed in the same run and reported under
``"decoder"``: batch data-parallel over N GPUs (no collective) and, for N > 1,
tensor-parallel linears with an NCCL all-reduce after each row-parallel product.

``--impl reference`` times the CPU restatement of the same graph
(oracle/rows_oracle.c, all host threads); each of its K steps runs a bounded
sample of the rows so that the run ends within a minute or so.

At N = 1 the line also carries ``"configs"``: device-time measurements of the
other configurations (MLP, dense dot, batched dot, quantised linear, integer
dot), each over at least 100 timed launches with its own clock sample and its
roofline fraction; ``--no-configs`` leaves them out.  At N > 1 the decoder
section checks every rank's sharded result against the single-GPU program's and
prints the outcome under ``"decoder": {"parity": ...}``; a mismatch aborts the
run without a line.
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
WORKLOAD = "fused row defn f32 {%d,32768} (max, exp, sum, logsumexp, softmax, argmax, tanh*sigmoid chain)"

# DRAM traffic of one launch of the row kernel, derived from an ncu capture of a 1024-row case
# (dram__bytes_read.sum = 134,252,032, dram__bytes_write.sum = 343,617,792): reads grow with the
# rows (every row is read once); writes are the algorithmic output bytes less what was still
# dirty in L2 when the kernel ended, which is a constant of the cache, not of the row count.
NCU_READ_BYTES_PER_ROW = 134_252_032 / 1024
NCU_L2_RESIDUE_BYTES = (3 * 1024 * 32768 * 4 + 1024 * 16) - 343_617_792


def row_kernel_traffic(rows, cols):
    writes = 3 * rows * cols * 4 + rows * 16
    return int(NCU_READ_BYTES_PER_ROW * rows * (cols / 32768) + max(0, writes - NCU_L2_RESIDUE_BYTES))


def workload_config(rows, world):
    """The `config` object of the line; both arms print the same one."""
    return {"workload": WORKLOAD % rows, "seed": SEED,
            "parallelism": "replicas only" if world > 1 else "single GPU",
            "l2": "input (1 GiB) and outputs (3 GiB) per step exceed L2 (126 MB); no flush needed"}


def algorithmic_bytes(rows, cols):
    """Each distinct input read once + each output written once."""
    full = rows * cols * 4
    return full * 4 + rows * 4 * 4          # x, exp, softmax, chain; max, sum, lse (f32) + argmax (s32)


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """SM clock and throttle reasons of one GPU DURING a timed region.  A thread reads them through NVML
    (what nvidia-smi itself reads; a query takes well under a millisecond, so regions of a few
    milliseconds still get samples) and stamps every sample with the host clock; `begin()` / `end()`
    mark the region, and only samples taken inside it are reported.  Without the NVML module the
    recipe's `nvidia-smi -lms` loop is used, its samples stamped on arrival."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index, period_ms=50):
        self.samples, self.proc, self.nvml, self.max_mhz = [], None, None, None
        self.t0, self.t1, self.running = None, None, True
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = None
            try:
                # the CUDA device's PCI address: NVML numbers devices without regard to CUDA_VISIBLE_DEVICES
                import torch
                pr = torch.cuda.get_device_properties(index)
                bus_id = f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
                self.handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus_id.encode())
            except Exception:
                self.handle = None
            if self.handle is None:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.nvml = pynvml
            self.period = min(period_ms, 2) / 1e3
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", str(period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while self.running:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                mask = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((time.perf_counter(), mhz, {k for k, b in self.BITS.items() if mask & b}))
            except Exception:
                pass
            time.sleep(self.period)

    def _read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            r = [c.strip() for c in line.split(",")]
            if len(r) >= 6 and r[0].replace(".", "").isdigit():
                if r[1].replace(".", "").isdigit():
                    self.max_mhz = max(self.max_mhz or 0.0, float(r[1]))
                self.samples.append((time.perf_counter(), float(r[0]), {n for n, v in zip(names, r[2:6]) if v.lower().startswith("active")}))

    def begin(self):
        self.t0 = time.perf_counter()

    def end(self):
        self.t1 = time.perf_counter()

    def stop(self):
        if self.nvml is None and not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["neither NVML nor nvidia-smi available"], "samples": 0}
        if self.t1 is None:
            self.t1 = time.perf_counter()
        if self.nvml is None:
            time.sleep(0.1)                      # the last lines of the nvidia-smi loop
        self.running = False
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        else:
            self.t.join(timeout=1)
        t0 = self.t0 if self.t0 is not None else 0.0
        inside = [s_ for s_ in self.samples if t0 <= s_[0] <= self.t1]
        sm = [s_[1] for s_ in inside]
        reasons = sorted(set().union(*[s_[2] for s_ in inside])) if inside else []
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(sm), "source": "NVML, sampled inside the timed region" if self.nvml else "nvidia-smi -lms, sampled inside the timed region"}


# ---- CPU arm -----------------------------------------------------------------------------

def load_rows_oracle():
    path = os.path.join(ROOT, "oracle", "librows_oracle.so")
    if not os.path.exists(path):
        subprocess.run(["make", "-s", "-C", os.path.join(ROOT, "oracle")], check=True)
    lib = C.CDLL(path)
    lib.rows_oracle.restype = None
    lib.rows_oracle.argtypes = [C.c_void_p, C.c_int64, C.c_int64] + [C.c_void_p] * 7
    lib.rows_oracle_threads.restype = C.c_int
    # launchers such as torch.distributed.run export OMP_NUM_THREADS=1: use the cores this process may run on
    lib.rows_oracle_set_threads(len(os.sched_getaffinity(0)))
    return lib


class CpuRows:
    """The CPU restatement with its output buffers allocated (and touched) once."""

    def __init__(self, rows, cols):
        self.lib = load_rows_oracle()
        self.outs = [np.zeros(rows, np.float32), np.zeros((rows, cols), np.float32), np.zeros(rows, np.float32),
                     np.zeros(rows, np.float32), np.zeros((rows, cols), np.float32), np.zeros(rows, np.int32),
                     np.zeros((rows, cols), np.float32)]

    def __call__(self, x):
        t0 = time.perf_counter()
        self.lib.rows_oracle(x.ctypes.data, x.shape[0], x.shape[1], *[o.ctypes.data for o in self.outs])
        return time.perf_counter() - t0


def cpu_baseline(x):
    """Oracle port on this box's host cores: the full workload, three passes (a few seconds)."""
    f = CpuRows(*x.shape)
    f(x[:64])
    times = [f(x) for _ in range(3)]
    dt = min(times)
    return {"value": round(algorithmic_bytes(*x.shape) / dt / 1e9, 3), "unit": UNIT, "cores": f.lib.rows_oracle_threads(),
            "kind": "port", "sample": f"all {x.shape[0]} rows x {x.shape[1]} cols, best of 3 passes ({sum(times):.1f} s total)"}


def run_reference(args, rank):
    """The CPU arm: K steps, each over a bounded sample of the rows (a contiguous block that
    moves through the matrix), sized from a first pass so that the K steps take about a minute."""
    if rank != 0:
        return
    from nx_b200 import configs
    x = configs.fused_rows_input(ROWS, COLS, SEED)
    f = CpuRows(ROWS, COLS)
    f(x[:256])
    per_row = f(x[:1024]) / 1024
    for _ in range(max(0, min(args.warmup, 3) - 1)):
        f(x[:1024])
    steps = max(1, args.steps)
    sample = int(60.0 / steps / per_row) // 256 * 256
    sample = max(1024, min(ROWS, sample))
    times = []
    for i in range(steps):
        r0 = (i * sample) % (ROWS - sample + 1)
        times.append(f(x[r0:r0 + sample]))
    dt = sum(times) / len(times)
    gbs = algorithmic_bytes(sample, COLS) / dt / 1e9
    cores = f.lib.rows_oracle_threads()
    what = f"{sample} of {ROWS} rows per step ({sample * COLS * 16 >> 20} MiB of traffic, beyond the host caches), {steps} steps"
    line = {"impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(ROWS, args.gpus),
            "note": "CPU restatement of the reference's evaluator path (one pass per output), all host threads",
            "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": cores, "kind": "port", "sample": what},
            "e2e": {"value": round(gbs, 3), "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


# ---- device helpers ------------------------------------------------------------------------

class Timer:
    def __init__(self, lib, device):
        self.lib, self.device = lib, device

    def time(self, fn, steps, warmup=3):
        from nx_b200 import nif
        for _ in range(warmup):
            fn()
        nif.check(self.lib.nxb200_device_synchronize(self.device))
        nif.check(self.lib.nxb200_timer_begin(self.device))
        for _ in range(steps):
            fn()
        ms = C.c_float()
        nif.check(self.lib.nxb200_timer_end(self.device, C.byref(ms)))
        return ms.value / steps


def device_inputs(inputs):
    from nx_b200 import nx
    return [nx.tensor(a, t) for a, t in inputs]


def time_program(timer, fun, inputs, device, steps=10):
    from nx_b200 import defn
    dev = device_inputs(inputs)
    prog = defn.compile(fun, [defn.template(a.shape, t) for a, t in inputs], device=device).program
    outs = prog.run(dev, device)
    return timer.time(lambda: prog.run_into(dev, outs, device), steps), prog


class StreamTimer:
    """Per-launch device times with an L2 flush before every launch: events of the library's compute
    stream (wrapped as a torch stream) bracket the launch alone, the flush sits outside them.  The
    flush READS a buffer twice the size of L2: the cache is then full of clean lines, as it is when
    other layers' weights have streamed through it.  (A flush by writes leaves 126 MB of dirty lines
    whose write-back competes with the timed kernel's reads.)"""

    def __init__(self, lib, device, torch):
        from nx_b200 import nif
        h = C.c_void_p()
        nif.check(lib.nxb200_device_stream(device, C.byref(h)))
        self.torch, self.lib, self.device = torch, lib, device
        self.stream = torch.cuda.ExternalStream(h.value, device=device)
        self.flush = torch.zeros(64 << 20, dtype=torch.int32, device=f"cuda:{device}")

    def flushed(self, fn, iters=30):
        torch = self.torch
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
        with torch.cuda.stream(self.stream):
            for a, b in evs:
                self.flush.sum()
                a.record(self.stream)
                fn()
                b.record(self.stream)
        self.stream.synchronize()
        return statistics.median(a.elapsed_time(b) for a, b in evs)


def timed_config(timer, device, fun, inputs, work, bound, peak, unit, min_iters=100, min_ms=300.0, flusher=None):
    """One configuration: at least `min_iters` timed launches lasting at least `min_ms` in total, with
    the SM clock sampled during them.  `work` is flop (tensor bound) or algorithmic bytes (hbm bound)."""
    from nx_b200 import backend, defn
    dev = device_inputs(inputs)
    prog = defn.compile(fun, [defn.template(a.shape, t) for a, t in inputs], device=device).program
    outs = prog.run(dev, device)
    run = lambda: prog.run_into(dev, outs, device)
    probe = timer.time(run, 10, warmup=5)                       # a short burst: sizes the loop
    iters = int(max(min_iters, min(20000, min_ms / max(probe, 1e-4))))
    sampler = ClockSampler(device, period_ms=20)
    ms = timer.time(run, iters, warmup=3)
    clocks = sampler.stop()
    rate = work / ms / 1e9 if bound == "tensor" else work / ms / 1e6
    res = {"ms": round(ms, 5), "iters": iters, "burst_ms": round(probe, 5), "launches": prog.launch_count(),
           "roofline": {"bound": bound, "achieved": round(rate, 1), "peak": peak, "unit": unit, "frac": round(rate / peak, 4)},
           "clocks": clocks}
    if flusher is not None:
        res["ms_l2_flushed"] = round(flusher.flushed(run), 5)
    for t_ in dev + outs:
        backend.backend_deallocate(t_)
    return res, prog


def int8_yardstick(torch, device):
    """A library integer product as the denominator for the s8 rates: torch._int_mm 8192^3 -> s32,
    best of 10 (used by the benchmark only, never by the product path)."""
    try:
        a = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=f"cuda:{device}")
        b = torch.randint(-127, 128, (8192, 8192), dtype=torch.int8, device=f"cuda:{device}").t()
        for _ in range(3):
            torch._int_mm(a, b)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        del a, b
        torch.cuda.empty_cache()
        return {"tops": round(2 * 8192 ** 3 / best / 1e9, 1), "how": "torch._int_mm s8 8192^3 -> s32, best of 10"}
    except Exception as e:   # noqa: BLE001 - the yardstick is optional
        return {"tops": None, "how": f"torch._int_mm unavailable: {type(e).__name__}"}


def other_configs(timer, device, pk, torch):
    """Device-time measurements of the other configurations, each with clocks and a roofline."""
    from nx_b200 import configs, nif
    nx_ = configs.nx
    flusher = StreamTimer(nif.lib(), device, torch)
    hbm, tf_burst, tf_sus = float(pk["hbm_gbs"]), float(pk["bf16_tflops"]), float(pk.get("bf16_tflops_sustained", pk["bf16_tflops"]))
    res = {"peaks": {"hbm_gbs": hbm, "bf16_tflops_burst": tf_burst, "bf16_tflops_sustained": tf_sus,
                     "note": "roofline.frac of the tensor-bound entries is against the burst figure; loops of 0.3 s and more "
                             "run under the power cap, where the sustained figure is the library's own ceiling"}}
    r, _ = timed_config(timer, device, configs.mlp, configs.mlp_inputs(), 2 * 64 * (784 * 128 + 128 * 10), "tensor", tf_burst, "TFLOP/s")
    r["note"] = "launch bound: four kernels replayed as one CUDA graph"
    res["mlp_f32_64x784x128x10"] = r

    def tensor_entry(name, fun, inputs, flop, peak=tf_burst, unit="TFLOP/s"):
        r, prog = timed_config(timer, device, fun, inputs, flop, "tensor", peak, unit)
        if unit == "TFLOP/s":
            r["roofline"]["frac_of_sustained"] = round(r["roofline"]["achieved"] / tf_sus, 4)
            r["burst_tflops"] = round(flop / r["burst_ms"] / 1e9, 1)
        r["plan"] = prog.describe().strip().split("\n")
        res[name] = r

    dense = configs.dense_inputs()
    tensor_entry("dense_bf16_8192^3_bias_gelu", configs.dense_bias_gelu, dense, 2 * 8192 ** 3)
    tensor_entry("dot_bf16_8192^3_kmajor", lambda a, b: nx_.dot(a, [1], b, [1]), [dense[0], dense[0]], 2 * 8192 ** 3)
    del dense
    byt = (2 * 64 * 2048 * 128 + 64 * 2048 * 2048) * 2
    r, _ = timed_config(timer, device, configs.batched_dot, configs.batched_inputs(), byt, "hbm", hbm, "GB/s")
    r["tflops"] = round(2 * 64 * 2048 * 2048 * 128 / r["ms"] / 1e9, 1)
    res["batched_bf16_64x2048x128x2048"] = r
    for m in (1, 16, 256, 4096):
        f_in, _ = configs.quantised_inputs(m=m)
        byt = 11008 * 4096 + 11008 * 4 + m * 4096 * 2 + m * 11008 * 4
        flop = 2 * m * 4096 * 11008
        if m <= 16:
            r, prog = timed_config(timer, device, configs.quantised_linear, f_in, byt, "hbm", hbm, "GB/s", flusher=flusher)
            r["roofline"]["achieved_l2_flushed"] = round(byt / r["ms_l2_flushed"] / 1e6, 1)
            r["roofline"]["frac_l2_flushed"] = round(byt / r["ms_l2_flushed"] / 1e6 / hbm, 4)
            r["note"] = "ms: back-to-back launches (W, 45 MB, stays in L2); ms_l2_flushed: median single launch after an L2 flush"
        else:
            r, prog = timed_config(timer, device, configs.quantised_linear, f_in, flop, "tensor", tf_burst, "TFLOP/s")
            r["roofline"]["frac_of_sustained"] = round(r["roofline"]["achieved"] / tf_sus, 4)
            r["gbs"] = round(byt / r["ms"] / 1e6, 1)
        r["plan"] = prog.describe().strip().split("\n")
        res[f"quantised_linear_M{m}"] = r
    # the integer-accumulate products (random s8 data) against a measured library integer product
    yard = int8_yardstick(torch, device)
    res["int8_yardstick"] = yard
    ipeak, iunit = (yard["tops"], "TOP/s") if yard["tops"] else (4500.0, "TOP/s")
    _, i_in = configs.quantised_inputs(m=4096)
    tensor_entry("s8_dot_s32_4096x11008x4096", configs.integer_linear, i_in, 2 * 4096 * 4096 * 11008, ipeak, iunit)
    rng = np.random.default_rng(7)
    sq = [(rng.integers(-127, 128, (8192, 8192)).astype(np.int8), "s8") for _ in range(2)]
    tensor_entry("s8_dot_s8_8192^3", lambda x, w: nx_.dot(x, [1], w, [1]), sq, 2 * 8192 ** 3, ipeak, iunit)
    for k in ("s8_dot_s32_4096x11008x4096", "s8_dot_s8_8192^3"):
        res[k]["roofline"]["peak_source"] = "measured yardstick (int8_yardstick)" if yard["tops"] else "nominal 4.5 POP/s"
    return res


def progress(rank, what):
    """One line per phase on stderr (rank 0): a run that stalls shows where."""
    if rank == 0:
        print(f"[bench {time.strftime('%H:%M:%S')}] {what}", file=sys.stderr, flush=True)


def decoder_section(timer, device, rank, world, dist, torch):
    """Decoder block tokens/s: single GPU, batch data-parallel, tensor-parallel and {dp, tp} meshes.
    At N > 1 every sharded result is compared with the single-GPU program's result on this rank's GPU."""
    from nx_b200 import backend as B, configs, defn, nif, nx, sharding
    import zlib
    lib = nif.lib()
    block = configs.make_decoder_block()
    batch, seq = 8, 2048
    inputs = configs.decoder_inputs(batch=batch, seq=seq)
    out = {"tokens_per_step": batch * seq, "flops_per_token": 438.4e6,
           "note": "bf16 {8,2048,4096}, 32 heads, SwiGLU 11008; FLOP count uses full (unmasked) attention"}
    parity = {}

    def sync_max(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    reference = {}

    def single_reference():
        """The single-GPU program's result for the whole batch, computed on this rank's GPU."""
        if "out" not in reference:
            dev = device_inputs(inputs)
            prog = defn.compile(block, [defn.template(a.shape, t) for a, t in inputs], device=device).program
            o, = prog.run(dev, device)
            reference["out"] = nx.to_numpy(o)
            for t_ in dev + [o]:
                B.backend_deallocate(t_)
        return reference["out"]

    def check_parity(label, got, batch_slice, replicated_over):
        """bf16 tolerance against the single-GPU result; results that are replicated over a
        tensor-parallel group must be bit-identical within it."""
        want = single_reference()[batch_slice]
        err = np.abs(got - want)
        outside = float(np.mean(err > 1e-2 + 2e-2 * np.abs(want)))
        rel = float(np.linalg.norm((got - want).ravel().astype(np.float64)) / max(1e-30, np.linalg.norm(want.ravel().astype(np.float64))))
        # Partitioned programs sum in another order (partial products, then the sum over the group), and
        # thirteen kernels round to bf16 in between: single elements may differ by a few bf16 steps.  A wrong
        # kernel or a wrong partition moves whole rows: the relative error of the result as a whole and the
        # largest single error tell the two apart (the share of elements outside rtol 2e-2 atol 1e-2 is reported).
        ok = rel <= 1e-2 and float(err.max()) <= 0.05 * float(np.abs(want).max())
        mine = {"ok": ok, "max_abs_err": float(err.max()), "rel": rel, "outside": outside,
                "bit_identical_to_single": bool(np.array_equal(got, want)),
                "crc": zlib.crc32(got.tobytes()), "group": replicated_over}
        rows = [None] * world
        dist.all_gather_object(rows, mine)
        groups = {}
        for r_ in rows:
            groups.setdefault(r_["group"], set()).add(r_["crc"])
        same = all(len(v) == 1 for v in groups.values())
        parity[label] = {"ok": all(r_["ok"] for r_ in rows), "ranks_checked": world,
                         "tolerance": "every rank's result against the single-GPU program: relative error of the whole result "
                                      "<= 1e-2 (a few bf16 roundings) and no element off by more than 5 % of the largest value",
                         "max_abs_err": max(r_["max_abs_err"] for r_ in rows),
                         "relative_error": max(r_["rel"] for r_ in rows),
                         "share_outside_elementwise_tolerance": max(r_["outside"] for r_ in rows),
                         "bit_identical_to_single_gpu": all(r_["bit_identical_to_single"] for r_ in rows),
                         "bit_identical_across_group": same}

    def run_sharded(mesh, shardings, label, check=True, batch_axis=None, group_axis=None):
        def shard(a, sh):
            for dim, axes in sh.items():
                n = mesh.shape[axes[0]]
                c = mesh.coords(rank)[axes[0]]
                step = a.shape[dim] // n
                a = np.take(a, range(c * step, (c + 1) * step), axis=dim)
            return np.ascontiguousarray(a)
        progress(rank, f"decoder {label}: partition + build")
        local = [(shard(a, sh), t) for (a, t), sh in zip(inputs, shardings)]
        blob, _, _ = sharding.partition(block, mesh, shardings, [defn.template(a.shape, t) for a, t in local], rank)
        prog = defn.Program(blob)
        dev = device_inputs(local)
        if dist is not None:
            dist.barrier()          # every rank has built its program: kernels that wait on peers are bounded
        progress(rank, f"decoder {label}: first run")
        outs = prog.run(dev, device)
        nif.check(lib.nxb200_device_synchronize(device))
        if dist is not None:
            dist.barrier()
        progress(rank, f"decoder {label}: timing")
        ms = sync_max(timer.time(lambda: prog.run_into(dev, outs, device), 5, warmup=2))
        out[label] = {"ms_per_step": round(ms, 3), "tokens_per_s": round(batch * seq / ms * 1e3),
                      "tflops": round(438.4e6 * batch * seq / ms / 1e9, 1), "launches_per_step": prog.launch_count()}
        if check and dist is not None:
            progress(rank, f"decoder {label}: parity against the single-GPU program")
            coords = mesh.coords(rank)
            if batch_axis is None:
                sl, grp = slice(0, batch), "all"
            else:
                per = batch // mesh.shape[batch_axis]
                sl = slice(coords[batch_axis] * per, (coords[batch_axis] + 1) * per)
                grp = f"dp{coords[batch_axis]}" if group_axis is not None else f"rank{rank}"
            check_parity(label, nx.to_numpy(outs[0]), sl, grp)
        for t_ in dev + outs:
            B.backend_deallocate(t_)

    def tensor_parallel(mesh, tp_axis, dp_axis, label, also_nccl):
        progress(rank, f"decoder {label}: communicator + peer memory")
        ex = sharding.torch_exchange()
        b_local = batch // (mesh.shape[dp_axis] if dp_axis is not None else 1)
        peer = sharding.init_tensor_parallel_group(mesh, tp_axis, rank, device, ex, gather=sharding.torch_gather(),
                                                   peer_elems=b_local * seq * 4096)
        # the collective alone: the sum over the group of one {b_local, seq, 4096} bf16 activation, which each
        # of the block's two row-parallel products needs (NCCL on the compute stream, device-timed)
        msg = nx.tensor(np.zeros((b_local, seq, 4096), np.float32), "bf16")
        for _ in range(2):
            nif.check(lib.nxb200_comm_all_reduce_sum(msg.data.handle))
        dist.barrier()
        ar_ms = sync_max(timer.time(lambda: nif.check(lib.nxb200_comm_all_reduce_sum(msg.data.handle)), 5, warmup=1))
        B.backend_deallocate(msg)
        xs = {0: [dp_axis]} if dp_axis is not None else {}
        col, row = {1: [tp_axis]}, {0: [tp_axis]}
        tp = [xs, col, col, col, row, col, col, row, {}, {}]
        kw = dict(batch_axis=dp_axis, group_axis=tp_axis)
        if also_nccl:
            # the two all-reduces as NCCL calls after their products, then fused into the products over peer memory
            os.environ["NXB200_FUSED_ALLREDUCE"] = "never"
            run_sharded(mesh, tp, label + "_nccl", **kw)
            del os.environ["NXB200_FUSED_ALLREDUCE"]           # automatic choice per product
        before = sharding.fused_all_reduce_launches()
        run_sharded(mesh, tp, label, **kw)
        fused = (sharding.fused_all_reduce_launches() - before) // 8 if peer else 0      # 1 + 2 + 5 runs
        out[label]["all_reduce"] = f"{fused} of 2 fused into their products over peer memory, the rest NCCL"
        nbytes_msg = b_local * seq * 4096 * 2
        n_tp = mesh.shape[tp_axis]
        out[label]["all_reduce_alone"] = {"ms": round(ar_ms, 3), "message_bytes": nbytes_msg, "ranks": n_tp,
                                          "bus_gbs": round(nbytes_msg * 2 * (n_tp - 1) / n_tp / ar_ms / 1e6, 1),
                                          "note": "two of these per block; NCCL all-reduce timed alone on the same group"}
        if fused and label in parity:
            # the fused kernel reduces every tile once, in rank order, on its owner: the copies must agree bit for bit
            parity[label]["ok"] = parity[label]["ok"] and parity[label]["bit_identical_across_group"]
        progress(rank, f"decoder {label}: releasing the communicator")
        nif.check(lib.nxb200_device_synchronize(device))
        dist.barrier()
        nif.check(lib.nxb200_comm_destroy())
        dist.barrier()

    if world == 1:
        run_sharded(sharding.Mesh("one", (1,)), [{}] * 10, "single", check=False)
    else:
        run_sharded(sharding.Mesh("dp", (world,)), [{0: [0]}] + [{}] * 9, f"dp{world}", batch_axis=0)
        tensor_parallel(sharding.Mesh("tp", (world,)), 0, None, f"tp{world}", also_nccl=True)
        for dp in (2, 4):
            tp_ = world // dp
            if tp_ >= 2 and dp * tp_ == world:
                tensor_parallel(sharding.Mesh("dp_tp", (dp, tp_)), 1, 0, f"dp{dp}xtp{tp_}", also_nccl=False)
        out["parity"] = parity
        best = min((k for k in out if isinstance(out[k], dict) and "ms_per_step" in out[k]), key=lambda k: out[k]["ms_per_step"])
        out["best"] = best
    reference.clear()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=ROWS, help="reduced row count (profiling captures only)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-decoder", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="leave out the per-configuration measurements (N = 1)")
    ap.add_argument("--all-configs", action="store_true", help="accepted for compatibility: the configurations are on by default")
    ap.add_argument("--profile-gemm", type=int, default=0, metavar="N",
                    help="run only an N^3 bf16 dense product with the fused bias+gelu epilogue (ncu captures of the tensor-core kernel)")
    ap.add_argument("--profile-batched", action="store_true",
                    help="run only the batched bf16 product {64,2048,128} x {64,128,2048} (ncu captures of the short-k tensor-core kernel)")
    ap.add_argument("--profile-decoder", type=int, default=0, metavar="B",
                    help="run only the decoder block on a batch of B sequences (ncu launch lists)")
    ap.add_argument("--profile-quantised", type=int, default=0, metavar="M",
                    help="run only the s8-weight linear {M,4096}x{11008,4096} (ncu captures of the small-batch kernels)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        return run_reference(args, rank)
    args.warmup = max(args.warmup, 3)

    # The library first: it then runs its kernels through the toolkit's runtime compiler, which its rpath
    # names.  torch ships an older copy under the same soname, and whichever is loaded first serves both.
    from nx_b200 import backend, configs, defn, nif, nx
    lib = nif.lib()
    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    backend.set_default_backend("b200", local)
    timer = Timer(lib, local)
    if args.profile_decoder:
        ms_, prog_ = time_program(timer, configs.make_decoder_block(), configs.decoder_inputs(batch=args.profile_decoder), local, steps=args.steps)
        print(json.dumps({"workload": f"decoder block bf16 {{{args.profile_decoder},2048,4096}}", "ms": round(ms_, 4),
                          "tokens_per_s": round(args.profile_decoder * 2048 / ms_ * 1e3), "plan": prog_.describe().strip().split("\n")}))
        return
    if args.profile_quantised:
        m_ = args.profile_quantised
        ms_, prog_ = time_program(timer, configs.quantised_linear, configs.quantised_inputs(m=m_)[0], local, steps=args.steps)
        print(json.dumps({"workload": f"s8-weight linear bf16 {{{m_},4096}} x s8 {{11008,4096}}", "us": round(ms_ * 1e3, 2),
                          "w_stream_gbs": round(11008 * 4096 / ms_ / 1e6), "plan": prog_.describe().strip().split("\n")}))
        return
    if args.profile_gemm:
        n = args.profile_gemm
        ms_, prog_ = time_program(timer, configs.dense_bias_gelu, configs.dense_inputs(m=n, n=n, k=n), local, steps=args.steps)
        print(json.dumps({"workload": f"dense bf16 {n}^3 + bias + gelu", "ms": round(ms_, 4), "tflops": round(2 * n ** 3 / ms_ / 1e9, 1),
                          "plan": prog_.describe().strip().split("\n")}))
        return
    if args.profile_batched:
        ms_, prog_ = time_program(timer, configs.batched_dot, configs.batched_inputs(), local, steps=args.steps)
        byt = (2 * 64 * 2048 * 128 + 64 * 2048 * 2048) * 2
        print(json.dumps({"workload": "batched bf16 {64,2048,128} x {64,128,2048}", "ms": round(ms_, 4), "gbs": round(byt / ms_ / 1e6, 1),
                          "tflops": round(2 * 64 * 2048 * 2048 * 128 / ms_ / 1e9, 1), "plan": prog_.describe().strip().split("\n")}))
        return
    rows = args.rows
    progress(rank, "headline: inputs + build")
    x_host = configs.fused_rows_input(rows, COLS, SEED)
    x = nx.tensor(x_host)
    prog = defn.compile(configs.fused_rows, [defn.template((rows, COLS), "f32")], device=local).program
    outs = prog.run([x], local)                       # allocates the output buffers once
    nbytes = algorithmic_bytes(rows, COLS)

    def barrier():
        nif.check(lib.nxb200_device_synchronize(local))
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)                     # started before the warm-up: it is polling when the timed region begins
    for _ in range(args.warmup):
        prog.run_into([x], outs, local)
    barrier()
    nif.check(lib.nxb200_timer_begin(local))
    sampler.begin()
    for _ in range(args.steps):
        prog.run_into([x], outs, local)
    ms = C.c_float()
    nif.check(lib.nxb200_timer_end(local, C.byref(ms)))
    sampler.end()
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
    progress(rank, "headline: timed; end to end")
    e2e = None
    if not args.no_e2e:
        pin_in = torch.empty(x_host.nbytes, dtype=torch.uint8, pin_memory=True)
        pin_in.numpy()[:] = x_host.reshape(-1).view(np.uint8)
        out_bytes = [o.size * 4 for o in outs]
        # two sets of pinned result buffers: the host could consume one while the other fills
        pin_out = [[torch.empty(n, dtype=torch.uint8, pin_memory=True) for n in out_bytes] for _ in range(2)]
        e2e_steps = max(2, min(args.steps, 6))

        def one(i):
            # upload on the upload stream (overlaps the previous step's downloads: the link is full
            # duplex), the program after it, the downloads after the program; the library orders the
            # next step's program after these downloads, so the device results are never overwritten early
            nif.check(lib.nxb200_buffer_write_async(x.data.handle, pin_in.data_ptr(), x_host.nbytes))
            prog.run_into([x], outs, local)
            for o, p, n in zip(outs, pin_out[i % 2], out_bytes):
                nif.check(lib.nxb200_buffer_read_async(o.data.handle, p.data_ptr(), n))

        one(0)
        nif.check(lib.nxb200_device_synchronize(local))
        barrier()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            one(i)
        nif.check(lib.nxb200_device_synchronize(local))     # every step's results are in host memory
        dt = (time.perf_counter() - t0) / e2e_steps
        if dist is not None:
            t = torch.tensor([dt], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        e2e = {"value": round(world * nbytes / dt / 1e9, 3), "unit": UNIT, "h2d_bytes_per_step": int(x_host.nbytes),
               "d2h_bytes_per_step": int(sum(out_bytes)), "ms_per_step": round(dt * 1e3, 3), "steps": e2e_steps,
               "overlap": "upload of step i+1 runs while step i's results download (separate copy streams)"}
        # what reached host memory in both result sets is what the device holds
        for k, o in enumerate(outs):
            dev_bytes = nx.to_numpy(o).reshape(-1).view(np.uint8)
            for s in range(2):
                if not np.array_equal(pin_out[s][k].numpy()[:: 4099], dev_bytes[:: 4099]):
                    raise SystemExit(f"end-to-end run: result {k} in host buffer set {s} differs from the device tensor")
        del pin_in, pin_out

    launches = args.steps * prog.launch_count()
    plan = prog.describe().strip().split("\n")
    # free the 4 GiB of the headline workload before the other sections
    for t_ in [x] + outs:
        backend.backend_deallocate(t_)

    decoder = None
    if not args.no_decoder and rows == ROWS:
        decoder = decoder_section(timer, local, rank, world, dist, torch)

    if decoder is not None and world > 1:
        bad = [k for k, v in decoder.get("parity", {}).items() if not v["ok"]]
        if bad:
            if rank == 0:
                print("sharded decoder results differ from the single-GPU program: " + json.dumps({k: decoder["parity"][k] for k in bad}),
                      file=sys.stderr)
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(3)

    if rank == 0:
        pk, which = peaks()
        peak = float(pk["hbm_gbs"])
        line = {"metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": workload_config(rows, world),
                "roofline": {"bound": "hbm", "achieved": round(per_gpu, 2), "peak": peak, "unit": "GB/s",
                             "frac": round(per_gpu / peak, 4),
                             "traffic": row_kernel_traffic(rows, COLS),
                             "traffic_source": "ncu capture of a 1024-row launch of this kernel: reads scaled by the rows, writes = "
                                               f"algorithmic output bytes less the {NCU_L2_RESIDUE_BYTES / 1e6:.1f} MB still dirty in L2 when the kernel ends",
                             "peak_source": f"of {which}", "kernel": "nxb_k0_row",
                             "algorithmic_bytes_per_launch": nbytes},
                "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "plan": plan}
        if decoder is not None:
            line["decoder"] = decoder
        if not args.no_configs and world == 1 and rows == ROWS:
            progress(rank, "other configurations")
            line["configs"] = other_configs(timer, local, pk, torch)
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(x_host)
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
