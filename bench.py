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
(oracle/rows_oracle.c, all host threads).  ``--all-configs`` adds device-time
measurements of the other configurations (MLP, dense dot, batched dot,
quantised linear) under ``"configs"``.
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

# DRAM bytes per launch of the row kernel from one ncu capture of a 1024-row case
# (dram__bytes_read.sum + dram__bytes_write.sum = 134.3 MB + 343.8 MB), scaled by the
# row count; reads match the algorithmic 128 MiB exactly, writes are below the
# algorithmic 384 MiB because the last ~59 MB were still dirty in L2 when the kernel ended.
NCU_TRAFFIC_BYTES_PER_1024_ROWS = 134_280_448 + 343_771_136


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
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "50"],
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
        time.sleep(0.1)
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
    if rank != 0:
        return
    from nx_b200 import configs
    rows = ROWS
    x = configs.fused_rows_input(rows, COLS, SEED)
    f = CpuRows(rows, COLS)
    for _ in range(max(1, min(args.warmup, 2))):
        f(x[:256])
    steps = max(1, min(args.steps, 10))             # each step is the whole workload (under a second per step)
    times = [f(x) for _ in range(steps)]
    dt = sum(times) / len(times)
    gbs = algorithmic_bytes(rows, COLS) / dt / 1e9
    cores = f.lib.rows_oracle_threads()
    line = {"impl": "reference", "metric": METRIC, "value": round(gbs, 3), "unit": UNIT, "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": round(dt * 1e3, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD % rows, "seed": SEED,
                       "note": "CPU restatement of the reference's evaluator path (one pass per output), all host threads"},
            "cpu_baseline": {"value": round(gbs, 3), "unit": UNIT, "cores": cores, "kind": "port",
                             "sample": f"whole workload per step, {steps} steps"},
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


def decoder_section(timer, device, rank, world, dist, torch):
    """Decoder block tokens/s: single GPU, batch data-parallel and tensor-parallel."""
    from nx_b200 import backend as B, configs, defn, nx, sharding
    block = configs.make_decoder_block()
    batch, seq = 8, 2048
    inputs = configs.decoder_inputs(batch=batch, seq=seq)
    out = {"tokens_per_step": batch * seq, "flops_per_token": 438.4e6,
           "note": "bf16 {8,2048,4096}, 32 heads, SwiGLU 11008; FLOP count uses full (unmasked) attention"}

    def sync_max(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run_sharded(mesh, shardings, label):
        def shard(a, sh):
            for dim, axes in sh.items():
                n = mesh.shape[axes[0]]
                c = mesh.coords(rank)[axes[0]]
                step = a.shape[dim] // n
                a = np.take(a, range(c * step, (c + 1) * step), axis=dim)
            return np.ascontiguousarray(a)
        local = [(shard(a, sh), t) for (a, t), sh in zip(inputs, shardings)]
        blob, _, _ = sharding.partition(block, mesh, shardings, [defn.template(a.shape, t) for a, t in local], rank)
        prog = defn.Program(blob)
        dev = device_inputs(local)
        if dist is not None:
            dist.barrier()          # every rank has built its program: kernels that wait on peers are bounded
        outs = prog.run(dev, device)
        if dist is not None:
            dist.barrier()
        ms = sync_max(timer.time(lambda: prog.run_into(dev, outs, device), 5, warmup=2))
        out[label] = {"ms_per_step": round(ms, 3), "tokens_per_s": round(batch * seq / ms * 1e3),
                      "tflops": round(438.4e6 * batch * seq / ms / 1e9, 1), "launches_per_step": prog.launch_count()}

    if world == 1:
        run_sharded(sharding.Mesh("one", (1,)), [{}] * 10, "single")
    else:
        run_sharded(sharding.Mesh("dp", (world,)), [{0: [0]}] + [{}] * 9, f"dp{world}")
        mesh = sharding.Mesh("tp", (world,))
        ex = sharding.torch_exchange()
        peer = sharding.init_tensor_parallel_group(mesh, 0, rank, device, ex, gather=sharding.torch_gather(),
                                                   peer_elems=batch * seq * 4096)
        tp = [{}, {1: [0]}, {1: [0]}, {1: [0]}, {0: [0]}, {1: [0]}, {1: [0]}, {0: [0]}, {}, {}]
        # the two all-reduces as NCCL calls after their products, then fused into the products over peer memory
        os.environ["NXB200_FUSED_ALLREDUCE"] = "never"
        run_sharded(mesh, tp, f"tp{world}_nccl")
        del os.environ["NXB200_FUSED_ALLREDUCE"]           # automatic choice per product
        before = sharding.fused_all_reduce_launches()
        run_sharded(mesh, tp, f"tp{world}")
        fused = (sharding.fused_all_reduce_launches() - before) // 8 if peer else 0      # 1 + 2 + 5 runs
        out[f"tp{world}"]["all_reduce"] = f"{fused} of 2 fused into their products over peer memory, the rest NCCL"
    return out


def other_configs(timer, device, pk):
    from nx_b200 import configs
    res = {}
    ms, prog = time_program(timer, configs.mlp, configs.mlp_inputs(), device, steps=50)
    res["mlp_f32_64x784x128x10"] = {"ms": round(ms, 4), "launches": prog.launch_count()}
    ms, prog = time_program(timer, configs.dense_bias_gelu, configs.dense_inputs(), device)
    tf = 2 * 8192 ** 3 / ms / 1e9
    res["dense_bf16_8192^3_bias_gelu"] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_measured_bf16_peak": round(tf / pk["bf16_tflops"], 3),
                                           "plan": prog.describe().strip().split("\n")}
    ms, prog = time_program(timer, lambda a, b: configs.nx.dot(a, [1], b, [1]), [configs.dense_inputs()[0], configs.dense_inputs()[0]], device)
    tf = 2 * 8192 ** 3 / ms / 1e9
    res["dot_bf16_8192^3_kmajor"] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_measured_bf16_peak": round(tf / pk["bf16_tflops"], 3)}
    ms, prog = time_program(timer, configs.batched_dot, configs.batched_inputs(), device)
    byt = (2 * 64 * 2048 * 128 + 64 * 2048 * 2048) * 2
    res["batched_bf16_64x2048x128x2048"] = {"ms": round(ms, 4), "tflops": round(2 * 64 * 2048 * 2048 * 128 / ms / 1e9, 1),
                                            "gbs": round(byt / ms / 1e6, 1), "frac_of_measured_hbm": round(byt / ms / 1e6 / pk["hbm_gbs"], 3)}
    for m in (1, 16, 256, 4096):
        f_in, i_in = configs.quantised_inputs(m=m)
        ms, prog = time_program(timer, configs.quantised_linear, f_in, device)
        byt = 11008 * 4096 + 11008 * 4 + m * 4096 * 2 + m * 11008 * 4
        res[f"quantised_linear_M{m}"] = {"ms": round(ms, 4), "tflops": round(2 * m * 4096 * 11008 / ms / 1e9, 2), "gbs": round(byt / ms / 1e6, 1)}
    # the integer-accumulate products (random s8 data): x {4096,4096} . W {11008,4096}^T with an s32 result, and s8 8192^3
    nx_ = configs.nx
    _, i_in = configs.quantised_inputs(m=4096)
    ms, prog = time_program(timer, configs.integer_linear, i_in, device)
    res["s8_dot_s32_4096x11008x4096"] = {"ms": round(ms, 4), "tops": round(2 * 4096 * 4096 * 11008 / ms / 1e9, 1), "plan": prog.describe().strip().split("\n")}
    rng = np.random.default_rng(7)
    sq = [(rng.integers(-127, 128, (8192, 8192)).astype(np.int8), "s8") for _ in range(2)]
    ms, prog = time_program(timer, lambda x, w: nx_.dot(x, [1], w, [1]), sq, device)
    res["s8_dot_s8_8192^3"] = {"ms": round(ms, 4), "tops": round(2 * 8192 ** 3 / ms / 1e9, 1)}
    return res


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
    ap.add_argument("--all-configs", action="store_true")
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

    import torch
    dist = None
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from nx_b200 import backend, configs, defn, nif, nx
    backend.set_default_backend("b200", local)
    lib = nif.lib()
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

    if rank == 0:
        pk, which = peaks()
        peak = float(pk["hbm_gbs"])
        line = {"metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": WORKLOAD % rows, "seed": SEED,
                           "parallelism": "replicas only" if world > 1 else "single GPU",
                           "l2": "input (1 GiB) and outputs (3 GiB) per step exceed L2 (126 MB); no flush needed"},
                "roofline": {"bound": "hbm", "achieved": round(per_gpu, 2), "peak": peak, "unit": "GB/s",
                             "frac": round(per_gpu / peak, 4),
                             "traffic": int(NCU_TRAFFIC_BYTES_PER_1024_ROWS * rows / 1024),
                             "peak_source": f"of {which}", "kernel": "nxb_k0_row",
                             "algorithmic_bytes_per_launch": nbytes},
                "clocks": clocks, "gpu_launches": launches, "e2e": e2e, "plan": plan}
        if decoder is not None:
            line["decoder"] = decoder
        if args.all_configs and world == 1:
            line["configs"] = other_configs(timer, local, pk)
        if not args.no_cpu and world == 1:
            line["cpu_baseline"] = cpu_baseline(x_host)
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
