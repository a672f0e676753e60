#!/usr/bin/env python
"""Measurement harness for the elementwise/reduction path.

    python bench.py --gpus N --steps K --warmup W            # the CUDA path (this library)
    python bench.py --impl reference --steps K --warmup W    # the CPU arm

Workload of the headline number (``config.workload``): Black-Scholes call/put
pricing of 2^26 options in float64, written exactly as examples/example_bs.py of
the reference writes it -- 26 elementwise ufunc calls and 2 copies through the
dpnp-style API.  One step = one evaluation of the chain on one batch.  The
metric is achieved HBM GB/s counted in ALGORITHMIC bytes: 552 bytes per option
(24 B per array-array op, 16 B per unary / array-scalar op or copy).  Inputs are
synthetic (seeded uniform draws with the example's ranges).

`value`  : inputs resident in HBM, CUDA-event time of K steps, max over ranks.
`e2e`    : same chain, every step copies its three input vectors from pinned
           host memory and reads call/put back to pinned host memory.
`roofline`: the contiguous elementwise kernel (ew_contig_vec), algorithmic bytes
           of the 26 ufunc launches / their summed CUDA-event durations.
`cpu_baseline`: the C restatement of the chain (oracle/, OpenMP over all host
           cores) on a bounded sample; same 552 B/option accounting.
`ops`    : the other benchmark configurations (add f32 2^24; the Black-Scholes
           chain hand-fused and through the `fuse` front-end; sum axis=1 / axis=0 /
           mean and running sums of f32 16384x65536; transposed broadcast multiply;
           max/argmax of int32 (8, 2^29)) and one representative shape per kernel
           family, each timed on its own.  Kernels of a few hundred microseconds
           are timed over several back-to-back calls per sample.

With N > 1 (torchrun, one rank per GPU) every rank prices its own 2^26 options
(weak scaling, no data-path collective); the reduction configurations are
sharded on the leading axis and their partials combined in rank order -- by one
kernel per rank over peer mailboxes where every rank owns a GPU of one box, else
through NCCL (`combine_us`: that step alone).  Every op is timed the same way at
every N: 4 back-to-back calls per sample, maximum over the ranks.
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_OPTIONS = 1 << 26
BYTES_PER_OPTION_CHAIN = 552      # 26 ufunc calls + 2 copies, algorithmic
BYTES_PER_OPTION_UFUNCS = 520     # the 26 ufunc launches alone
BYTES_PER_OPTION_FUSED = 40       # 3 loads + 2 stores
RATE, VOL = 0.1, 0.2
SEED = 7777777


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.device)], capture_output=True, text=True, timeout=5).stdout
                parts = [p.strip() for p in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.1)

    def start(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=6)
        mhz = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        reasons = set()
        for s in self.samples:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(self.samples)}


# ------------------------------------------------------------- CUDA helpers
class Events:
    def __init__(self, lib, check, stream):
        self.lib, self.check, self.stream = lib, check, C.c_void_p(stream)

    def new(self):
        e = C.c_void_p()
        self.check(self.lib.dpb_event_create(C.byref(e)))
        return e

    def record(self, e):
        self.check(self.lib.dpb_event_record(e, self.stream))

    def elapsed_ms(self, e0, e1):
        self.check(self.lib.dpb_event_synchronize(e1))
        ms = C.c_float()
        self.check(self.lib.dpb_event_elapsed_ms(e0, e1, C.byref(ms)))
        return float(ms.value)


def black_scholes(np_, price, strike, t, rate, vol, call, put, hook=None):
    """The body of examples/example_bs.py::black_scholes; `hook` wraps every array operation
    (used to time the individual launches)."""
    h = hook or (lambda nbytes, f: f())
    n8 = 8
    mr = -rate
    sig_sig_two = vol * vol * 2
    P, S, T = price, strike, t
    q = h(3 * n8, lambda: P / S)
    a = h(2 * n8, lambda: np_.log(q))
    b = h(2 * n8, lambda: T * mr)
    z = h(2 * n8, lambda: T * sig_sig_two)
    c = h(2 * n8, lambda: 0.25 * z)
    sq = h(2 * n8, lambda: np_.sqrt(z))
    y = h(2 * n8, lambda: 1.0 / sq)
    ab1 = h(3 * n8, lambda: a - b)
    abc1 = h(3 * n8, lambda: ab1 + c)
    w1 = h(3 * n8, lambda: abc1 * y)
    ab2 = h(3 * n8, lambda: a - b)
    abc2 = h(3 * n8, lambda: ab2 - c)
    w2 = h(3 * n8, lambda: abc2 * y)
    e1 = h(2 * n8, lambda: np_.erf(w1))
    he1 = h(2 * n8, lambda: 0.5 * e1)
    d1 = h(2 * n8, lambda: 0.5 + he1)
    e2 = h(2 * n8, lambda: np_.erf(w2))
    he2 = h(2 * n8, lambda: 0.5 * e2)
    d2 = h(2 * n8, lambda: 0.5 + he2)
    eb = h(2 * n8, lambda: np_.exp(b))
    Se = h(3 * n8, lambda: eb * S)
    pd1 = h(3 * n8, lambda: P * d1)
    sd2 = h(3 * n8, lambda: Se * d2)
    r = h(3 * n8, lambda: pd1 - sd2)
    call[:] = r
    rp = h(3 * n8, lambda: r - P)
    pt = h(3 * n8, lambda: rp + Se)
    put[:] = pt


# ------------------------------------------------------------------ CPU arm
def cpu_chain_throughput(n_sample, min_seconds=8.0, max_reps=6):
    """Options/s of the C restatement of the chain on all host cores (bounded sample)."""
    from oracle import dpnp_oracle as orc

    cpu_threads()
    rng = np.random.default_rng(SEED)
    p, k, t = rng.uniform(10, 50, n_sample), rng.uniform(10, 50, n_sample), rng.uniform(1, 2, n_sample)
    orc.black_scholes_c(p[:1024], k[:1024], t[:1024], RATE, VOL, threads=True)  # warm up the thread pool
    reps, total = 0, 0.0
    best = float("inf")
    while reps < max_reps and (total < min_seconds or reps < 2):
        t0 = time.perf_counter()
        orc.black_scholes_c(p, k, t, RATE, VOL, threads=True)
        dt = time.perf_counter() - t0
        best = min(best, dt)
        total += dt
        reps += 1
    return n_sample / best, reps, total


def cpu_threads():
    """Use every core this process may run on, whatever OMP_NUM_THREADS the launcher exported;
    returns the thread count the C port will actually use."""
    try:
        n = len(os.sched_getaffinity(0))
    except Exception:
        n = os.cpu_count() or 1
    try:
        from oracle import dpnp_oracle as orc

        orc.core().orc_set_num_threads(int(n))
        return int(orc.core().orc_max_threads())
    except Exception:
        return 1


def run_reference_arm(args):
    """The CPU arm: the reference cannot be installed here (needs DPC++/SYCL, dpctl, oneMKL), so the
    oracle's C restatement of the same chain is timed on all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_sample = 1 << 26
    threads = cpu_threads()
    # warm-up steps
    from oracle import dpnp_oracle as orc

    rng = np.random.default_rng(SEED)
    p, k, t = rng.uniform(10, 50, n_sample), rng.uniform(10, 50, n_sample), rng.uniform(1, 2, n_sample)
    for _ in range(max(args.warmup, 1)):
        orc.black_scholes_c(p, k, t, RATE, VOL, threads=True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.black_scholes_c(p, k, t, RATE, VOL, threads=True)
    dt = time.perf_counter() - t0
    opt_per_s = n_sample * args.steps / dt
    value = opt_per_s * BYTES_PER_OPTION_CHAIN / 1e9
    sample = f"all 2^26 options per step, {args.steps} steps, C chain with libm on {threads} threads"
    line = {
        "impl": "reference", "metric": "achieved algorithmic GB/s, Black-Scholes chain (552 B/option)",
        "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3 * (N_OPTIONS / n_sample), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "black_scholes_f64_2^26_chain_26ufuncs_2copies", "options": N_OPTIONS,
                   "rate": RATE, "vol": VOL, "seed": SEED},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference not installable offline (DPC++/SYCL, dpctl, oneMKL absent): CPU port timed instead",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------ GPU arm
def timed_steps(ev, fn, steps, flush=None):
    """CUDA-event time (ms) of `steps` back-to-back calls of fn."""
    e0, e1 = ev.new(), ev.new()
    ev.record(e0)
    for _ in range(steps):
        fn()
    ev.record(e1)
    return ev.elapsed_ms(e0, e1)


def median_time_ms(ev, fn, reps, warm=3, batch=1, prime=False):
    """Median over `reps` samples of the CUDA-event time of one call of fn.  A sample brackets
    `batch` back-to-back calls and is divided by it: with one call per sample the device sits
    idle between the first event and the launch while the host is still inside the call, and
    that idle time would be charged to a kernel of a few hundred microseconds."""
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(reps):
        e0, e1 = ev.new(), ev.new()
        if prime:
            # one call queued ahead of the start event: the device is still busy with it when the
            # timed calls arrive, so the host time of the first timed call is not charged either
            fn()
        ev.record(e0)
        for _ in range(batch):
            fn()
        ev.record(e1)
        ts.append(ev.elapsed_ms(e0, e1) / batch)
    ts.sort()
    return ts[len(ts) // 2]


def measure_fp64_peak(lib, check, ev, q):
    """FP64 fused multiply-adds per second the device sustains (dpb_probe_fp64_fma, best of 5)."""
    import dpnp_b200 as dp

    scr = dp.empty(1 << 20)
    cnt = C.c_int64()
    best = 0.0
    for _ in range(5):
        e0, e1 = ev.new(), ev.new()
        ev.record(e0)
        check(lib.dpb_probe_fp64_fma(20000, 8, C.c_void_p(scr.get_array()._ptr), scr.size, C.byref(cnt),
                                     C.c_void_p(q.stream)))
        ev.record(e1)
        best = max(best, cnt.value / (ev.elapsed_ms(e0, e1) * 1e-3))
    return best


# FP64 instructions executed per option by the two fused Black-Scholes kernels (thread-level
# dfma + dmul + dadd counts of one ncu capture on 2^24 options divided by the options; the capture
# is summarised under profiles/ and named in the JSON line)
FP64_INSTR_PER_OPTION = {"black_scholes_f64": 127.2, "ew_fused": 130.2, "ew_fused_specialized": 130.2}
FP64_INSTR_SOURCE = ("ncu smsp__sass_thread_inst_executed_op_{dfma,dmul,dadd}_pred_on.sum of `bench.py --profile-case "
                     "bs_fused` / `bs_fuse` / `bs_fuse_interpreted` (2^24 options)")


def run_gpu_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    saved_stdout = None
    if world > 1:
        # NCCL may print its version banner on stdout; keep stdout clean for the one JSON line
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)

    import dpnp_b200 as dp
    from dpnp_b200 import _lib, memory, sharded
    from dpnp_b200.memory import select_default_device

    if _lib.device_count() == 0:
        raise RuntimeError("bench.py needs a CUDA device for the GPU arm (no CPU fallback)")
    bind_to_gpu_cores(local_rank, world)
    select_default_device(local_rank)
    q = dp.get_default_queue()
    # the ranks of the job: the library's own host group and NCCL communicator (no PyTorch anywhere)
    comm = sharded.init(sharded.Communicator(queue=q)) if world > 1 else None
    lib, check = _lib.lib, _lib.check
    ev = Events(lib, check, q.stream)
    peak, peak_kind = load_peaks()
    n = N_OPTIONS

    def barrier():
        check(lib.dpb_device_synchronize())
        if comm is not None:
            comm.host.barrier()
            check(lib.dpb_device_synchronize())

    def max_over_ranks(ms):
        return ms if comm is None else comm.host.max_float(ms)

    # ---- inputs resident in HBM (each rank prices its own options: weak scaling)
    dp.random.seed(SEED + rank)
    price = dp.random.uniform(10.0, 50.0, n)
    strike = dp.random.uniform(10.0, 50.0, n)
    tt = dp.random.uniform(1.0, 2.0, n)
    call = dp.zeros(n, dtype=dp.float64)
    put = -dp.ones(n, dtype=dp.float64)

    def step():
        black_scholes(dp, price, strike, tt, RATE, VOL, call, put)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    _lib.reset_launch_count()
    barrier()
    ms = timed_steps(ev, step, args.steps)
    barrier()
    launches = _lib.launch_count()
    ms = max_over_ranks(ms)
    ms_per_step = ms / args.steps
    value = world * n * BYTES_PER_OPTION_CHAIN / (ms_per_step * 1e-3) / 1e9

    # ---- per-launch durations of the 26 ufunc kernels (roofline of ew_contig_vec)
    durations = []

    def hook(nbytes_per_elem, f):
        e0, e1 = ev.new(), ev.new()
        ev.record(e0)
        out = f()
        ev.record(e1)
        durations.append((nbytes_per_elem, e0, e1))
        return out

    passes = 3
    for _ in range(passes):
        black_scholes(dp, price, strike, tt, RATE, VOL, call, put, hook=hook)
    q.wait()
    tot_ms = sum(ev.elapsed_ms(e0, e1) for _, e0, e1 in durations)
    tot_bytes = sum(b for b, _, _ in durations) * n
    achieved = tot_bytes / (tot_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "ew_contig_vec (26 launches per step: f64 unary, binary, array-scalar)",
                "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "avg_launch_us": tot_ms * 1e3 / len(durations),
                "algorithmic_bytes_per_launch": tot_bytes / len(durations), "traffic": TRAFFIC_EW_CONTIG_F64,
                "traffic_source": TRAFFIC_SOURCE}
    # ---- end to end: pinned host -> device, chain, device -> pinned host, every step
    hp = [memory.PinnedHostBuffer(n, "f8") for _ in range(3)]
    ho = [memory.PinnedHostBuffer(n, "f8") for _ in range(2)]
    rng = np.random.default_rng(SEED + rank)
    hp[0].array[:] = rng.uniform(10, 50, n)
    hp[1].array[:] = rng.uniform(10, 50, n)
    hp[2].array[:] = rng.uniform(1, 2, n)

    # The batch is cut into chunks that rotate over a few in-order queues (3 by default; 4 or 6 measure the same): the copies of one chunk
    # overlap the chain of another and PCIe runs in both directions at once.  All work of one chunk
    # stays on one queue, as the API requires.
    from dpnp_b200.memory import StreamQueue

    nchunks = args.e2e_chunks
    csz = n // nchunks
    nq = args.e2e_queues
    queues = [StreamQueue(local_rank) for _ in range(nq)]
    chunk_bufs = []
    for k in range(nq):
        qk = queues[k]
        chunk_bufs.append([dp.empty(csz, dtype=dp.float64, sycl_queue=qk) for _ in range(5)])

    def e2e_step(h2d=True, compute=True, d2h=True):
        for ci in range(nchunks):
            qk = queues[ci % nq]
            cp, cs, ct, cc, cu = chunk_bufs[ci % nq]
            lo, hi = ci * csz, (ci + 1) * csz
            if h2d:
                for dst, src in zip((cp, cs, ct), hp):
                    memory.copy_host_to_device(dst, src.array[lo:hi], qk)
            if compute:
                black_scholes(dp, cp, cs, ct, RATE, VOL, cc, cu)
            if d2h:
                memory.copy_device_to_host(ho[0].array[lo:hi], cc, qk)
                memory.copy_device_to_host(ho[1].array[lo:hi], cu, qk)
        for qk in queues:
            qk.wait()

    def wall_ms(fn, reps=2):
        barrier()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        return max_over_ranks((time.perf_counter() - t0) * 1e3 / reps)

    e2e_steps = max(2, min(args.steps, 5))
    e2e_step()
    barrier()
    # several streams are involved, so the step is timed on the host clock between full
    # synchronisations (every step ends with a wait on all three queues)
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    e2e_ms = max_over_ranks(e2e_wall_ms)
    # what came back to the host must satisfy put-call parity on the inputs that went out:
    # call - put = P - S * exp(-r T)  (a property of the chain, checked on a strided sample)
    sl = slice(0, n, 4099)
    lhs = ho[0].array[sl] - ho[1].array[sl]
    rhs = hp[0].array[sl] - hp[1].array[sl] * np.exp(-RATE * hp[2].array[sl])
    e2e_check = bool(np.allclose(lhs, rhs, rtol=1e-11, atol=1e-11))
    if not e2e_check:
        raise RuntimeError("end-to-end outputs violate put-call parity")
    # what the links alone allow, all ranks copying at once and no kernel running: both directions
    # together (the step's copies) and each direction on its own
    copy_ms = wall_ms(lambda: e2e_step(compute=False))
    h2d_ms = wall_ms(lambda: e2e_step(compute=False, d2h=False))
    d2h_ms = wall_ms(lambda: e2e_step(h2d=False, compute=False))
    e2e = {"value": world * n * BYTES_PER_OPTION_CHAIN / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": 3 * 8 * n * world, "d2h_bytes_per_step": 2 * 8 * n * world, "ms_per_step": e2e_ms,
           "wall_ms_per_step": e2e_wall_ms, "steps": e2e_steps, "chunks": nchunks, "queues": nq,
           "copy_only_ms_per_step": copy_ms, "frac_of_copy_only": copy_ms / e2e_ms,
           "per_rank_h2d_gbs_alone": 3 * 8 * n / (h2d_ms * 1e-3) / 1e9,
           "per_rank_d2h_gbs_alone": 2 * 8 * n / (d2h_ms * 1e-3) / 1e9,
           "host_cores_of_rank0": len(os.sched_getaffinity(0)),
           }
    del chunk_bufs
    for b in hp + ho:
        b.free()

    # ---- the other configurations
    ops = []
    checks = {"e2e_put_call_parity_every_4099th_option": e2e_check}
    if not args.no_ops:
        ops = other_configs(dp, _lib, ev, q, peak, rank, world, comm, sharded, price, strike, tt, call, put, checks)
    host_us = host_latency(dp, q) if rank == 0 else None

    clocks = sampler.stop() if rank == 0 else None

    # ---- CPU baseline (rank 0, N=1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            n_sample = 1 << 26
            opt_s, reps, total = cpu_chain_throughput(n_sample, min_seconds=10.0, max_reps=40)
            cpu = {"value": opt_s * BYTES_PER_OPTION_CHAIN / 1e9, "unit": "GB/s", "cores": cpu_threads(),
                   "kind": "port",
                   "sample": f"all 2^26 options, best of {reps} runs ({total:.1f} s), C chain with libm, OpenMP"}
        except Exception as exc:  # the checker is optional for the measurement itself
            cpu = {"value": None, "unit": "GB/s", "cores": cpu_threads(), "kind": "port", "sample": f"failed: {exc}"}

    if saved_stdout is not None:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)
    if rank == 0:
        line = {
            "metric": "achieved algorithmic GB/s, Black-Scholes chain (552 B/option)",
            "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64", "data": "synthetic",
            "config": {"workload": "black_scholes_f64_2^26_chain_26ufuncs_2copies", "options_per_gpu": n,
                       "rate": RATE, "vol": VOL, "seed": SEED,
                       "l2": "inputs and temporaries (512 MiB each) exceed the 126 MB L2",
                       "parallelism": f"shard{world}_no_collective"},
            "frac_of_peak": value / world / peak, "peak_gbs": peak, "peak_kind": peak_kind,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks,
            "host_us_per_call": host_us, "checks": checks, "ops": ops,
        }
        print(json.dumps(line), flush=True)
    if comm is not None:
        os.dup2(2, 1)  # anything the teardown prints goes to stderr
        comm.barrier()
        comm.close()


# dram bytes read+written per launch of ew_contig_vec on 2^26 f64 operands, from one ncu capture of the
# kernel (named in the JSON line): 0.94 x the algorithmic bytes on 2^25 elements, scaled by the element
# count and averaged over the step's 13 array-array and 13 unary/array-scalar launches.
TRAFFIC_EW_CONTIG_F64 = 1.265e9
TRAFFIC_SOURCE = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of ew_contig_vec, `bench.py --profile-case "
                  "ew_mul_f64` (2^25 elements), scaled x2 by element count")


def other_configs(dp, _lib, ev, q, peak, rank, world, comm, sharded, price, strike, tt, call, put, checks):
    """Times the remaining benchmark configurations; returns a list of records.  `nbytes` of a
    record is the whole job's (all ranks'); `frac_of_peak` is per GPU."""
    lib = _lib.lib
    out = []
    S = C.c_void_p(q.stream)

    def rec(name, nbytes, ms, kernel=None, note=None, **extra):
        if os.environ.get("DPNP_B200_BENCH_VERBOSE"):
            print(f"[rank {rank}] {name}: {ms:.3f} ms", file=sys.stderr, flush=True)
        gbs = nbytes / (ms * 1e-3) / 1e9
        r = {"op": name, "ms": ms, "algorithmic_bytes": nbytes, "gbs": gbs, "frac_of_peak": gbs / peak / world,
             "kernel": kernel or _lib.last_kernel()}
        if note:
            r["note"] = note
        r.update(extra)
        out.append(r)

    n = N_OPTIONS
    # fused Black-Scholes (one pass)
    pp, ps, pt = (a.get_array()._ptr for a in (price, strike, tt))
    pc, pq = call.get_array()._ptr, put.get_array()._ptr
    fp64_peak = measure_fp64_peak(lib, _lib.check, ev, q)

    def fp64_roofline(kernel, ms_):
        per = FP64_INSTR_PER_OPTION.get(kernel)
        if not per:
            return {"fp64_fma_peak_per_s": fp64_peak}
        rate = per * n / (ms_ * 1e-3)
        return {"roofline_fp64": {"bound": "fp64 pipe", "achieved": rate, "peak": fp64_peak, "unit": "FP64 instr/s",
                                  "frac": rate / fp64_peak, "instr_per_option": per, "source": FP64_INSTR_SOURCE}}

    ms = median_time_ms(ev, lambda: lib.dpb_black_scholes_f64(n, pp, ps, pt, RATE, VOL, pc, pq, S), 10, batch=4)
    rec("c2_black_scholes_fused_f64_2^26", n * BYTES_PER_OPTION_FUSED * world, ms, "black_scholes_f64",
        "fp64-pipe bound: 2 erf + log + exp + sqrt + 2 div per option", **fp64_roofline("black_scholes_f64", ms))

    # the same chain through the general front-end, traced once: as the kernel compiled for it at
    # the first call (the default where NVRTC is found), and interpreted
    for mode, label, kern in (("auto", "c2_black_scholes_fuse_decorator_f64_2^26", "ew_fused_specialized"),
                              ("interpret", "c2_black_scholes_fuse_interpreted_f64_2^26", "ew_fused")):
        chain = dp.fuse(lambda p_, s_, t_, c_, q_: black_scholes(dp, p_, s_, t_, RATE, VOL, c_, q_), mode=mode)
        ms = median_time_ms(ev, lambda: chain(price, strike, tt, call, put), 10, batch=4)
        if chain.fused_calls == 0:
            raise RuntimeError(f"the Black-Scholes chain was not fused: {chain.last_reason}")
        if chain.last_executor == "interpreted":
            kern = "ew_fused"
        rec(label, n * BYTES_PER_OPTION_FUSED * world, ms,
            note=f"dpnp_b200.fuse(mode={mode!r}): the 26-call chain traced into one program, one launch, "
                 f"executor: {chain.last_executor}",
            **fp64_roofline(kern, ms))

    # C1: add f32 2^24, rotating over 4 buffer sets (768 MiB > L2)
    m = 1 << 24
    sets = [(dp.random.uniform(-1, 1, m, dtype="f4"), dp.random.uniform(-1, 1, m, dtype="f4"),
             dp.empty(m, dtype="f4")) for _ in range(4)]
    i = [0]

    def c1_api():
        a, b, o = sets[i[0] & 3]
        i[0] += 1
        dp.add(a, b, out=o)

    def c1_abi():
        a, b, o = sets[i[0] & 3]
        i[0] += 1
        lib.dpb_binary_contig(0, 10, 10, 10, m, a.get_array()._ptr, 0, b.get_array()._ptr, 0, o.get_array()._ptr, 0, S)

    ms = median_time_ms(ev, c1_api, 10, batch=16, prime=True)
    rec("c1_add_f32_2^24_api", 12 * m * world, ms,
        note="16 back-to-back dpnp.add calls per sample behind one queued call, rotating buffers")
    ms = median_time_ms(ev, c1_abi, 10, batch=16, prime=True)
    rec("c1_add_f32_2^24_c_abi", 12 * m * world, ms)
    del sets

    # further kernels of the path, one representative shape each (every rank runs its own copy);
    # 8 back-to-back calls per sample, operands of 512 MiB each (larger than L2)
    ne = 1 << 26
    xa, xb = dp.random.uniform(-1, 1, ne), dp.random.uniform(-1, 1, ne)
    xo = dp.empty(ne)
    cond = xa > 0.0
    ms = median_time_ms(ev, lambda: dp.where(cond, xa, xb, out=xo), 10, batch=8)
    rec("where_f64_2^26", 25 * ne * world, ms, note="bool condition + two f64 operands + result")
    ms = median_time_ms(ev, lambda: dp.where(cond, xa, 0.0, out=xo), 10, batch=8)
    rec("where_scalar_f64_2^26", 17 * ne * world, ms, note="second operand is a Python scalar (broadcast)")
    xf = dp.empty(ne, dtype="f4")
    ms = median_time_ms(ev, lambda: dp.copyto(xf, xa, casting="same_kind"), 10, batch=8)
    rec("copy_cast_f64_to_f32_2^26", 12 * ne * world, ms)
    ms = median_time_ms(ev, lambda: dp.add(xa, xb, out=xa), 10, batch=8)
    rec("inplace_add_f64_2^26", 24 * ne * world, ms)
    ms = median_time_ms(ev, lambda: dp.multiply(xa, 0.25, out=xo), 10, batch=8)
    rec("multiply_scalar_f64_2^26", 16 * ne * world, ms)
    del cond, xf
    mrows, mcols = 16384, 4096
    xm, xr = xa.reshape(mrows, mcols), xb[:mcols]
    xom = xo.reshape(mrows, mcols)
    ms = median_time_ms(ev, lambda: dp.subtract(xm, xr, out=xom), 10, batch=8)
    rec("row_broadcast_subtract_f64_16384x4096", 16 * ne * world, ms, note="matrix minus row vector")
    xv = xa.reshape(mrows, mcols)[:, 1:-1]
    xw = xo.reshape(mrows, mcols)[:, 1:-1]
    ms = median_time_ms(ev, lambda: dp.multiply(xv, 2.0, out=xw), 10, batch=8)
    rec("sliced_rows_multiply_f64_16384x4094", 16 * mrows * (mcols - 2) * world, ms,
        note="rows start off the 16-byte grid")
    xcol = xb[:mrows].reshape(mrows, 1)
    ms = median_time_ms(ev, lambda: dp.subtract(xm, xcol, out=xom), 10, batch=8)
    rec("col_broadcast_subtract_f64_16384x4096", 16 * ne * world, ms, note="matrix minus column vector")
    xt_src = xa.reshape(4096, 16384)
    ms = median_time_ms(ev, lambda: dp.copyto(xom, xt_src.T), 10, batch=8)
    rec("copy_transposed_f64_16384x4096", 16 * ne * world, ms, note="layout-changing copy (a.T into a C-ordered array)")
    xs2 = xa.reshape(mrows, mcols)[:, ::2]
    xo2 = xo.reshape(mrows, mcols)[:, : mcols // 2]
    ms = median_time_ms(ev, lambda: dp.multiply(xs2, 2.0, out=xo2), 10, batch=8)
    rec("inner_stride2_multiply_f64_16384x2048", 16 * mrows * (mcols // 2) * world, ms,
        note="input with inner stride 2: every 32-byte sector is half used (algorithmic bytes counted)")
    x3 = xa.reshape(64, 1024, 1024)
    ms = median_time_ms(ev, lambda: dp.sum(x3, axis=1), 10, batch=8)
    rec("sum_middle_axis_f64_64x1024x1024", 8 * ne * world, ms)
    ms = median_time_ms(ev, lambda: dp.sum(x3, axis=(0, 2)), 10, batch=8)
    rec("sum_axes02_f64_64x1024x1024", 8 * ne * world, ms)
    ms = median_time_ms(ev, lambda: dp.argmax(x3, axis=0), 10, batch=8)
    rec("argmax_axis0_f64_64x1024x1024", 8 * ne * world, ms)
    del xa, xb, xo, xm, xr, xom, xv, xw, x3

    # C3: sums of f32 16384 x 65536.  With several ranks the matrix is a ShardedArray (rows split
    # over the GPUs) and the benchmark makes the same calls as on one GPU.
    rows, cols = 16384 // world, 65536
    x_loc = dp.random.normal(0, 1, (rows, cols), dtype="f4")
    x = sharded.from_local(x_loc, comm) if comm is not None else x_loc
    nb = 4 * rows * cols * world

    def time_sharded(fn, reps):
        for _ in range(2):
            fn()
        ts = []
        for _ in range(reps):
            q.wait()
            if comm is not None:
                comm.host.barrier()
            # 4 back-to-back calls per sample keep the device busy while the host is inside the
            # next call -- at every N, so that the lines of different N compare like with like
            # (with several ranks every call that ends in an exchange waits for the slowest rank)
            batch = 4
            e0, e1 = ev.new(), ev.new()
            ev.record(e0)
            for _ in range(batch):
                fn()
            ev.record(e1)
            t = ev.elapsed_ms(e0, e1) / batch
            if comm is not None:
                t = comm.host.max_float(t)
            ts.append(t)
        ts.sort()
        return ts[len(ts) // 2]

    def combine_us(fn_partial, fn_combine):
        """Device time of the exchange + combine alone (median of 10), in microseconds."""
        if comm is None:
            return None
        part = fn_partial()
        return 1e3 * time_sharded(lambda: fn_combine(part), 10)

    ms = time_sharded(lambda: dp.sum(x, axis=1), 10)
    rec("c3a_sum_axis1_f32_16384x65536", nb, ms, note="rows stay whole on one GPU: no exchange")
    ms = time_sharded(lambda: dp.sum(x, axis=0), 10)
    rec("c3b_sum_axis0_f32_16384x65536", nb, ms,
        note="partials all-gathered over NCCL and added in rank order by one kernel on every rank" if world > 1 else None,
        combine_us=combine_us(lambda: dp.sum(x_loc, axis=0), comm.sum_ordered) if comm is not None else None)
    if comm is not None:
        # |combined - sum of the ranks' partials in float64| <= 1e-5 * sum|x| per column, and the
        # ranks agree bit for bit
        got = dp.sum(x, axis=0).asnumpy()
        parts = comm.host.allgather_object(dp.sum(x_loc, axis=0).asnumpy().astype("f8"))
        mags = comm.host.allgather_object(dp.sum(dp.abs(x_loc), axis=0).asnumpy().astype("f8"))
        err = np.abs(got.astype("f8") - np.sum(parts, axis=0))
        ok = bool(np.all(err <= 1e-5 * np.sum(mags, axis=0)))
        same = comm.host.allgather_object(got.tobytes())
        ok = ok and all(b == same[0] for b in same)
        checks["c3b_sharded_sum_within_1e-5_of_sum_abs_and_identical_on_all_ranks"] = ok
        if not ok:
            raise RuntimeError("sharded sum over axis 0 is outside 1e-5 * sum|x| or differs between ranks")
    ms = time_sharded(lambda: dp.mean(x), 10)
    rec("c3c_mean_f32_16384x65536", nb, ms,
        combine_us=combine_us(lambda: dp.sum(x_loc), comm.sum_ordered) if comm is not None else None)
    # running sums of the same matrix (every rank scans its own rows: no exchange is timed)
    xs = dp.empty((rows, cols), dtype="f4")
    ms = time_sharded(lambda: dp.cumsum(x_loc, axis=1, out=xs), 5)
    rec("cumsum_axis1_f32_16384x65536", 2 * nb, ms, note="read + write; one block per row, single pass")
    ms = time_sharded(lambda: dp.cumsum(x_loc, axis=0, out=xs), 5)
    rec("cumsum_axis0_f32_16384x65536", 2 * nb, ms, note="read + write; one thread per column")
    xflat, sflat = x_loc.reshape(-1)[: 1 << 28], xs.reshape(-1)[: 1 << 28]
    ms = time_sharded(lambda: dp.cumsum(xflat, out=sflat), 5)
    rec("cumsum_flat_f32_2^28", 8 * xflat.size * world, ms, note="one long row")
    del x, x_loc, xs, xflat, sflat

    # C4: multiply(a.transpose(2,0,1), b), `a` sharded along its leading axis
    ja = 1024 // world
    a = dp.random.uniform(-2, 2, (ja, 4096, 64), dtype="f4")
    b = dp.random.uniform(-2, 2, (64, 1, 4096), dtype="f4")
    o = dp.empty((64, ja, 4096), dtype="f4")
    at = a.transpose(2, 0, 1)
    ms = time_sharded(lambda: dp.multiply(at, b, out=o), 10)
    rec("c4_multiply_transposed_broadcast_f32", (2 * ja * 4096 * 64 * 4 + 64 * 4096 * 4) * world, ms)
    del a, b, o, at

    # C5: max / argmax of int32 (8, 2^29), leading axis sharded
    r5 = max(1, 8 // world)
    x_loc = dp.random.randint(0, 1000, (r5, 1 << 29), dtype="i4")
    x = sharded.from_local(x_loc, comm) if comm is not None else x_loc
    nb = 4 * r5 * (1 << 29) * world
    ms = time_sharded(lambda: dp.max(x), 5)
    rec("c5_max_flat_int32_8x2^29", nb, ms,
        combine_us=combine_us(lambda: dp.max(x_loc), lambda p: comm.extreme(p, "max")) if comm is not None else None)
    ms = time_sharded(lambda: dp.max(x, axis=-1), 5)
    rec("c5_max_lastaxis_int32_8x2^29", nb, ms)
    ms = time_sharded(lambda: dp.argmax(x), 5)
    li = dp.argmax(x_loc)
    rec("c5_argmax_flat_int32_8x2^29", nb, ms,
        combine_us=combine_us(lambda: li, lambda p: comm.arg_extreme(x_loc, p, rank * r5 * (1 << 29), "max"))
        if comm is not None else None)
    if comm is not None:
        # first occurrence across shards: the owner holds the maximum at that index and nothing equal
        # before it in its shard; every rank below the owner holds only smaller values
        gi = int(dp.argmax(x).asnumpy())
        vmax = int(dp.max(x).asnumpy())
        owner, local = divmod(gi, r5 * (1 << 29))
        flat = x_loc.reshape(-1)
        if rank == owner:
            ok = int(flat[local].asnumpy()) == vmax and (local == 0 or int(dp.max(flat[:local]).asnumpy()) < vmax)
        elif rank < owner:
            ok = int(dp.max(x_loc).asnumpy()) < vmax
        else:
            ok = int(dp.max(x_loc).asnumpy()) <= vmax
        oks = comm.host.allgather_object(bool(ok))
        checks["c5_sharded_argmax_is_the_first_occurrence_of_the_maximum"] = all(oks)
        if not all(oks):
            raise RuntimeError("sharded argmax is not the first occurrence of the maximum")
    ms = time_sharded(lambda: dp.argmax(x, axis=-1), 5)
    rec("c5_argmax_lastaxis_int32_8x2^29", nb, ms)
    return out


def host_latency(dp, q, calls=1000):
    """Host microseconds per call through the public API on tiny arrays (the device is never the
    bottleneck: the stream is drained before and after, the wall clock brackets `calls` calls)."""
    a, b = dp.ones(1024, dtype="f4"), dp.ones(1024, dtype="f4")
    m = dp.ones((64, 64), dtype="f4")
    mi = dp.ones((8, 512), dtype="i4")
    at, bb = dp.ones((16, 32, 8), dtype="f4").transpose(2, 0, 1), dp.ones((8, 1, 32), dtype="f4")
    cases = {"add": lambda: dp.add(a, b), "add_out": lambda: dp.add(a, b, out=a), "multiply_scalar": lambda: a * 2.0,
             "exp": lambda: dp.exp(a), "sum_axis1": lambda: dp.sum(m, axis=1), "max": lambda: dp.max(mi),
             "argmax_lastaxis": lambda: dp.argmax(mi, axis=-1), "multiply_transposed_broadcast": lambda: dp.multiply(at, bb)}
    out = {}
    for name, fn in cases.items():
        for _ in range(100):
            fn()
        q.wait()
        t0 = time.perf_counter()
        for _ in range(calls):
            fn()
        out[name] = round((time.perf_counter() - t0) * 1e6 / calls, 2)
        q.wait()
    return out


def bind_to_gpu_cores(local_rank, world):
    """With several ranks on one box, keep each rank (and the pinned buffers it is about to
    allocate, by first touch) on the cores nearest its GPU: the NUMA node of the GPU's PCI
    device when the box has several, else an even share of the cores this job may use.
    Read-only queries of sysfs / nvidia-smi; nothing on the GPU is changed."""
    if world <= 1:
        return None
    try:
        allowed = sorted(os.sched_getaffinity(0))
        cores = None
        bus = subprocess.run(["nvidia-smi", "--query-gpu=pci.bus_id", "--format=csv,noheader", "-i", str(local_rank)],
                             capture_output=True, text=True, timeout=10).stdout.strip().lower()
        if bus:
            dev = "0000:" + bus.split(":", 1)[1] if bus.count(":") == 2 else bus
            try:
                with open(f"/sys/bus/pci/devices/{dev}/local_cpulist") as fh:
                    near = set()
                    for part in fh.read().strip().split(","):
                        lo, _, hi = part.partition("-")
                        near.update(range(int(lo), int(hi or lo) + 1))
                near &= set(allowed)
                if near and len(near) < len(allowed):
                    cores = sorted(near)
            except (OSError, ValueError):
                pass
        if cores is None:
            share = max(1, len(allowed) // world)
            cores = allowed[local_rank * share:(local_rank + 1) * share] or allowed
        os.sched_setaffinity(0, cores)
        return cores
    except Exception:
        return None


PROFILE_CASES = ("ew_add_f32", "ew_mul_f64", "ew_mul_scalar_f64", "ew_erf_f64", "bs_fused", "bs_fuse", "bs_fuse_interpreted", "fuse_cheap", "cumsum_axis1", "cumsum_flat", "generic_stride2", "rows_bcast",
                 "argmax_axis0", "sum_axis1",
                 "sum_axis0", "mean_all", "transpose_c4", "max_i32", "argmax_i32")


def profile_case(name, launches=3):
    """Run one kernel a few times on a small input (larger than L2, about 1 GB on the device):
    the command line an ncu capture of that kernel is made with."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    q = dp.get_default_queue()
    if name == "ew_add_f32":
        n = 1 << 26
        a, b, o = dp.random.uniform(-1, 1, n, dtype="f4"), dp.random.uniform(-1, 1, n, dtype="f4"), dp.empty(n, dtype="f4")
        fn = lambda: dp.add(a, b, out=o)
    elif name in ("ew_mul_f64", "ew_mul_scalar_f64", "ew_erf_f64"):
        n = 1 << 25
        span = 4 if name == "ew_erf_f64" else 1         # erf: arguments over the whole table
        a, b, o = dp.random.uniform(-span, span, n), dp.random.uniform(-1, 1, n), dp.empty(n)
        fn = {"ew_mul_f64": lambda: dp.multiply(a, b, out=o), "ew_mul_scalar_f64": lambda: dp.multiply(a, 0.25, out=o),
              "ew_erf_f64": lambda: dp.erf(a, out=o)}[name]
    elif name == "bs_fused":
        n = 1 << 24
        p, s, t = dp.random.uniform(10, 50, n), dp.random.uniform(10, 50, n), dp.random.uniform(1, 2, n)
        c, u = dp.empty(n), dp.empty(n)
        S = C.c_void_p(q.stream)
        fn = lambda: _lib.lib.dpb_black_scholes_f64(n, p.get_array()._ptr, s.get_array()._ptr, t.get_array()._ptr,
                                                    RATE, VOL, c.get_array()._ptr, u.get_array()._ptr, S)
    elif name in ("bs_fuse", "bs_fuse_interpreted"):
        n = 1 << 24
        p, s, t = dp.random.uniform(10, 50, n), dp.random.uniform(10, 50, n), dp.random.uniform(1, 2, n)
        c, u = dp.empty(n), dp.empty(n)
        chain = dp.fuse(lambda p_, s_, t_, c_, q_: black_scholes(dp, p_, s_, t_, RATE, VOL, c_, q_),
                        mode="interpret" if name == "bs_fuse_interpreted" else "compile")
        fn = lambda: chain(p, s, t, c, u)
    elif name == "fuse_cheap":
        # 60 dependent multiply/add instructions with immediate operands: almost no arithmetic, so
        # the capture shows what interpreting one instruction costs
        n = 1 << 24
        x, o = dp.random.uniform(1, 2, n), dp.empty(n)

        def cheap(x_, o_):
            v = x_
            for _ in range(30):
                v = v * 1.0001 + 0.5
            o_[:] = v
        chain = dp.fuse(cheap)
        fn = lambda: chain(x, o)
    elif name in ("cumsum_axis1", "cumsum_flat"):
        x = dp.random.normal(0, 1, (4096, 65536), dtype="f4")
        o = dp.empty((4096, 65536), dtype="f4")
        if name == "cumsum_axis1":
            fn = lambda: dp.cumsum(x, axis=1, out=o)
        else:
            xf, of = x.reshape(-1), o.reshape(-1)
            fn = lambda: dp.cumsum(xf, out=of)
    elif name == "generic_stride2":
        x, o = dp.random.uniform(-1, 1, (8192, 4096)), dp.empty((8192, 2048))
        xs = x[:, ::2]
        fn = lambda: dp.multiply(xs, 2.0, out=o)
    elif name == "rows_bcast":
        x, r, o = dp.random.uniform(-1, 1, (8192, 4096)), dp.random.uniform(-1, 1, 4096), dp.empty((8192, 4096))
        fn = lambda: dp.subtract(x, r, out=o)
    elif name == "argmax_axis0":
        x = dp.random.uniform(-1, 1, (64, 1024, 512))
        fn = lambda: dp.argmax(x, axis=0)
    elif name in ("sum_axis1", "sum_axis0", "mean_all"):
        x = dp.random.normal(0, 1, (4096, 65536), dtype="f4")
        fn = {"sum_axis1": lambda: dp.sum(x, axis=1), "sum_axis0": lambda: dp.sum(x, axis=0),
              "mean_all": lambda: dp.mean(x)}[name]
    elif name == "transpose_c4":
        a = dp.random.uniform(-2, 2, (512, 4096, 64), dtype="f4")
        b = dp.random.uniform(-2, 2, (64, 1, 4096), dtype="f4")
        o = dp.empty((64, 512, 4096), dtype="f4")
        at = a.transpose(2, 0, 1)
        fn = lambda: dp.multiply(at, b, out=o)
    elif name in ("max_i32", "argmax_i32"):
        x = dp.random.randint(0, 1000, (8, 1 << 25), dtype="i4")
        fn = (lambda: dp.max(x, axis=-1)) if name == "max_i32" else (lambda: dp.argmax(x, axis=-1))
    else:
        raise SystemExit(f"unknown profile case {name}; choose from {PROFILE_CASES}")
    q.wait()
    for _ in range(launches):
        fn()
    q.wait()
    print(json.dumps({"profile_case": name, "launches": launches, "kernel": _lib.last_kernel()}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-ops", action="store_true", help="skip the per-configuration extras")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--e2e-queues", type=int, default=3,
                    help="in-order queues the chunks of the end-to-end measurement rotate over")
    ap.add_argument("--e2e-chunks", type=int, default=16,
                    help="pieces the batch is cut into for the pipelined end-to-end measurement")
    ap.add_argument("--profile-case", default=None, help="run one small case for an ncu capture: "
                    + ", ".join(PROFILE_CASES))
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
    elif args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
