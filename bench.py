"""Benchmark of the tile-program hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One JSON line.  Its contract fields (metric, value, e2e, roofline, cpu_baseline, clocks, gpu_launches) are
those of the fused element-wise + broadcast tile program Y = relu(exp(s*A) * b + C) on 8192x8192 bf16 with
fp32 intermediates, metric = HBM GB/s (algorithmic bytes / device time); one "step" is one pass of the
program over the whole tensor.  With N > 1 every rank runs its own replica of that program (it has no
cross-GPU exchange), so its scaling is weak and the value is the sum over ranks over the slowest rank's time.

The same line carries `workloads`: the other configurations measured in the same process at the same N -
`eltwise_add_1024` (one GPU only), `matmul_bf16_8192`, `matmul_bfp8w`, `attention` - each with its time per
step, compute-only time, TFLOP/s, roofline fraction, end-to-end figure from pinned host memory, sampled clocks
and (one GPU) a CPU baseline.  At N > 1 those three are the SHARDED runs (strong scaling: output row tiles /
weight column tiles / heads split over the ranks, full result gathered on every rank) and
`sharded_efficiency` = T1 / (N * T_N) per workload, T1 being the single-GPU kernel on the whole problem timed
in the same process.

`--workload NAME` prints the line of one workload alone (also: reduce_<sum|max>_<rows|cols|all>_8192,
softmax_8192, matmul_bfp4w).  `--impl reference` times the CPU implementation of the contract program on the
host cores: the reference simulator itself when oracle/_ref holds it (oracle/make_ref.py), else the torch
restatement of its numerics (oracle/tile_oracle.py).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "tt-lang_b200", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

N = 8192
ALGO_BYTES = (3 * N * N + N + 1) * 2  # A, C, Y full; b row vector; s scalar (bf16)
FUSED_EXPR = ("relu", ("add", ("mul", ("exp", ("mul", 0, 1)), 2), 3))


def measured_peak_hbm():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only) while the
    timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                break
            time.sleep(self.period)

    def stop(self):
        self._halt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except Exception:
            return local
    return local


def make_inputs():
    import cases

    a = cases.gen((N, N), "normal", 0)
    s = cases.gen((1, 1), "const:0.1", 0)
    b = cases.gen((1, N), "uniform", 1)
    c = cases.gen((N, N), "normal", 2)
    return a, s, b, c


def cpu_baseline(sample_rows: int, repeats: int):
    """Oracle port on a slab of `sample_rows` rows, GB/s of algorithmic bytes on the host cores."""
    import torch

    import cases
    from oracle import tile_oracle

    a = cases.gen((sample_rows, N), "normal", 0)
    s = cases.gen((1, 1), "const:0.1", 0)
    b = cases.gen((1, N), "uniform", 1)
    c = cases.gen((sample_rows, N), "normal", 2)
    tile_oracle.eval_expression(FUSED_EXPR, [a, s, b, c], (sample_rows, N), "f32")
    t0 = time.perf_counter()
    for _ in range(repeats):
        tile_oracle.eval_expression(FUSED_EXPR, [a, s, b, c], (sample_rows, N), "f32")
    dt = (time.perf_counter() - t0) / repeats
    nbytes = (3 * sample_rows * N + N + 1) * 2
    return nbytes / dt / 1e9, dt, torch.get_num_threads()


class SimulatorArm:
    """The reference simulator (installed unmodified under oracle/_ref by oracle/make_ref.py) running the very
    tile program the GPU arm runs, on a slab of rows.  The simulator steps its three threads per core in
    Python (python/sim/program.py:363-647), one tile block at a time, single-threaded."""

    def __init__(self):
        import importlib.util

        from oracle import make_ref

        self.sim = make_ref.load()
        if self.sim is None:
            raise FileNotFoundError("oracle/_ref/sim is not installed")
        import ttnn  # the simulator's, after its shadowing

        self.ttnn = ttnn
        spec = importlib.util.spec_from_file_location("bench_programs_sim_eltwise", ROOT / "tests" / "programs" / "eltwise.py")
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        self.program = mod.fused_exp_bcast

    def step(self, rows: int):
        """(GB/s of algorithmic bytes, seconds) for one pass over a [rows, 8192] slab."""
        import contextlib
        import io

        import torch

        import cases

        host = [cases.gen((rows, N), "normal", 0), cases.gen((1, 1), "const:0.1", 0), cases.gen((1, N), "uniform", 1),
                cases.gen((rows, N), "normal", 2)]
        tensors = [self.ttnn.from_torch(t) for t in host]
        out = self.ttnn.from_torch(torch.zeros((rows, N), dtype=torch.bfloat16))
        t0 = time.perf_counter()
        with contextlib.redirect_stdout(io.StringIO()):
            self.program(*tensors, out)
        dt = time.perf_counter() - t0
        return (3 * rows * N + N + 1) * 2 / dt / 1e9, dt


def simulator_sample(budget_s: float) -> dict:
    """cpu_baseline record of the reference simulator on a slab sized for about `budget_s` seconds."""
    arm = SimulatorArm()
    arm.step(32)             # first call: imports and one-time set-up
    _, t128 = arm.step(128)
    rows = int(max(128, min(1024, budget_s // max(t128, 1e-3) * 128)))
    v, dt = arm.step(rows)
    return {"value": v, "unit": "GB/s", "cores": 1, "kind": "reference",
            "sample": f"the reference simulator (oracle/_ref/sim, unmodified python/sim) running the same tile program on a "
                      f"{rows}x{N} row slab, one run ({dt:.2f} s); extrapolated to the full tensor: {dt * N / rows:.0f} s per step"}


def simulator_baseline(budget_s: float):
    """The same record, measured in a child interpreter (this process has the B200 backend installed under the
    module names `ttl` / `ttnn` / `sim`, which the simulator needs for itself); None when oracle/_ref is not
    installed or the child fails."""
    import subprocess

    if not (ROOT / "oracle" / "_ref" / "sim" / "__init__.py").exists():
        return None
    try:
        out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--sim-sample", str(budget_s)], capture_output=True,
                             text=True, timeout=120 + 20 * budget_s, cwd=str(ROOT))
        return json.loads(out.stdout.strip().splitlines()[-1])
    except Exception:
        return None


def run_reference(args):
    """Reference arm: the CPU implementation of the same program on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch

    # rank 0 runs alone: use every host core (torchrun starts its ranks with OMP_NUM_THREADS=1)
    torch.set_num_threads(max(torch.get_num_threads(), os.cpu_count() or 1))
    workload = "fused_eltwise_bcast_8192: Y=relu(exp(s*A)*b+C), bf16 in/out"
    try:
        arm = SimulatorArm()
    except Exception:
        arm = None
    port_v, port_dt, port_cores = cpu_baseline(1024, 3)
    port = {"value": port_v, "unit": "GB/s", "cores": port_cores, "kind": "port",
            "sample": f"oracle/tile_oracle.eval_expression on a 1024x{N} row slab, mean of 3 runs ({port_dt * 1e3:.1f} ms each)"}
    if arm is not None:
        # slab sized so that warm-up + steps stay within about two minutes of simulator time
        arm.step(32)         # first call: imports and one-time set-up
        _, t128 = arm.step(128)
        per_step = 120.0 / (args.steps + args.warmup)
        rows = int(max(128, min(1024, per_step // max(t128, 1e-3) * 128)))
        for _ in range(args.warmup):
            arm.step(rows)
        t0 = time.perf_counter()
        vals = [arm.step(rows)[0] for _ in range(args.steps)]
        total = time.perf_counter() - t0
        value = sum(vals) / len(vals)
        base = {"value": value, "unit": "GB/s", "cores": 1, "kind": "reference",
                "sample": f"the reference simulator (oracle/_ref/sim, unmodified python/sim) on a {rows}x{N} row slab per step; "
                          f"extrapolated to the full tensor: {total / args.steps * N / rows:.0f} s per step",
                "port": port}
        dtype, sample = "bf16", f"{rows} of {N} rows per step (simulator-native numerics: every op rounds to bf16)"
    else:
        rows = 1024
        for _ in range(max(args.warmup, 1)):
            cpu_baseline(rows, 1)
        t0 = time.perf_counter()
        vals = [cpu_baseline(rows, 1)[0] for _ in range(args.steps)]
        total = time.perf_counter() - t0
        value = sum(vals) / len(vals)
        base = dict(port, value=value,
                    sample=f"oracle/tile_oracle.eval_expression on a {rows}x{N} row slab per step (the reference simulator's "
                           "numerics: torch CPU ops, fp32 intermediates); oracle/_ref is not installed")
        dtype, sample = "f32", f"{rows} of {N} rows per step"
    line = {
        "impl": "reference", "metric": "eltwise HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# Sharded workloads (configs 3-5): matmul_bf16_8192 | matmul_bfp8w | attention
# --------------------------------------------------------------------------- #
NVLINK_MEASURED_GBS = 770.0    # peer copy, one direction, measured on this pool's B200 boxes
NVLINK_NOMINAL_GBS = 900.0
SHARDED_WORKLOADS = ("matmul_bf16_8192", "matmul_bfp8w", "attention")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from the ncu capture named in
# profiles/ (None: not captured for this workload)
TRAFFIC_BYTES = {
    "fused_eltwise_bcast_8192": 366.0e6,     # profiles/eltwise_jit_fused_bcast_8192.md (268.5 MB read + 97.6 MB written)
    "matmul_bf16_8192": 1331.0e6 + 134.2e6,  # profiles/gemm_bf16_8192.md (operands re-read from L2 misses + C written)
    "matmul_bfp8w": 778.0e6 + 224.0e6,        # profiles/matmul_bfp8w_4096x8192x28672.md (unpack kernel + GEMM of one step)
    "matmul_bfp8w_in_mainloop": 769.8e6 + 225.2e6,   # same file, ttlb_gemm_bfp8w_tmem_kernel
    "attention": 805.0e6 + 249.0e6,          # profiles/attention_b8_h32_s4096_d128.md
    "eltwise_add_1024": None,
}


def measured_peak_tensor():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            j = json.loads(f.read_text())
            return float(j["bf16_tflops"]), float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), "measured (MEASURED_PEAKS.json bf16_tflops, burst)"
        except Exception:
            pass
    return 1590.0, 1400.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


class Env:
    """Rank, device and (for more than one rank) the NCCL process group of this bench process."""

    def __init__(self):
        import torch

        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        if self.world > 1:
            import datetime

            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev, timeout=datetime.timedelta(seconds=120))
            self.dist = dist
        bind_to_gpu_numa_node(physical_gpu_index(self.local))

    def barrier(self):
        import torch

        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        import torch

        if self.dist is None:
            return ms
        t = torch.tensor([ms], device="cuda")
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


def bind_to_gpu_numa_node(gpu_index: int) -> None:
    """Run this process (and place the pinned buffers it allocates afterwards) on the CPU cores next to its
    GPU: the affinity NVML reports for the device (read-only query).  Without it every rank of a box
    allocates its pinned buffers from whichever node it happens to start on."""
    try:
        import pynvml

        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * w + b for w, m in enumerate(mask) for b in range(64) if (m >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


def timed(env: "Env", fn, steps: int, warmup: int) -> float:
    """ms per call of fn: warm-up, barrier + synchronize on both sides, CUDA events on the current stream,
    maximum over the ranks."""
    import torch

    for _ in range(warmup):
        fn()
    env.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    env.barrier()
    return env.max_over_ranks(e0.elapsed_time(e1) / steps)


def through_the_dsl(a_dev, b_operand, direct_out):
    """The same product through `@ttl.kernel`: the reference's multicore matmul tile program in 1x1-tile blocks
    (examples/multicore_matmul.py:28-139, restated in tests/programs/matmul.py) is traced, recognised as one launch
    and run; the record carries the time of trace + recognition and whether the bits equal the direct call's."""
    import importlib.util

    import torch

    import ttl_b200
    ttl_b200.install()
    import ttnn
    spec = importlib.util.spec_from_file_location("bench_programs_matmul", ROOT / "tests" / "programs" / "matmul.py")
    programs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(programs)
    A = ttnn.Tensor(a_dev)
    B = b_operand if isinstance(b_operand, ttnn.Tensor) else ttnn.Tensor(b_operand)
    out = ttnn.Tensor(torch.zeros_like(direct_out))
    t0 = time.perf_counter()
    plan = programs.multicore_matmul.plan(A, B, out)
    trace_s = time.perf_counter() - t0
    programs.multicore_matmul(A, B, out)
    torch.cuda.synchronize()
    return {"program": "multicore matmul tile program, 1x1-tile blocks, through @ttl.kernel (tests/programs/matmul.py)",
            "trace_and_recognise_s": round(trace_s, 3), "launches": [d["kind"] for d in plan.describe()],
            "same_bits_as_the_direct_call": bool(torch.equal(out._tensor, direct_out))}


def measure_sharded(args, wl: str, env: "Env", gather_mode: str = "auto") -> dict:
    """One record for a sharded workload.  One GPU: the single-GPU kernel on the whole problem.  N GPUs: strong
    scaling - the problem is split over the ranks (output row tiles / weight column tiles / heads,
    ttl_b200.shard), every rank runs the single-GPU kernel on its shard and the output shards are gathered so
    that every rank ends up with the full result; reported with and without the gather."""
    import torch

    import cases
    from ttl_b200 import capi, ops, shard, ttnn

    rank, world, dev = env.rank, env.world, env.dev
    ctx = capi.context(env.local)
    ctx.set_gemm_variant(args.gemm_variant)
    if args.bfp8_mode is not None:
        ctx.set_bfp8_mode(args.bfp8_mode)
    if args.bfp8_chunks is not None:
        ctx.set_bfp8_chunks(args.bfp8_chunks)
    T = ttnn.Tensor
    full_compute = None      # at N > 1: the single-GPU kernel on the whole problem (T1 of the efficiency figure)
    if wl == "matmul_bf16_8192":
        n = 8192
        a = cases.gen((n, n), f"normal*{n ** -0.5}", 0)
        b = cases.gen((n, n), f"normal*{n ** -0.5}", 1)
        chunks = shard.pick_chunks(n // 32, world)
        mine = shard.cyclic_units(n // 32, world, rank, chunks)
        host_in = [torch.cat([a[u0 * 32:(u0 + c) * 32] for u0, c in mine]).contiguous().pin_memory(), b.pin_memory()]
        flops = 2.0 * n * n * n
        out_bytes = n * n * 2
        kernel = "ttlb_gemm_bf16_kernel" if args.gemm_variant == 0 else "ttlb_gemm_bf16_2cta_kernel"

        def compute(x):
            return ops.matmul(T(x[0]), T(x[1]))._tensor

        def step(x):
            return shard.sharded_matmul(x[0], x[1], n, lambda p, q: ops.matmul(T(p), T(q))._tensor, chunks=chunks)
        if world > 1:
            a_full = a.to(dev)
            full_compute = lambda x: ops.matmul(T(a_full), T(x[1]))  # noqa: E731
        desc = ("A,B bf16 [8192,8192] N(0,1/sqrt(8192)) seeds 0/1, fp32 accumulate, bf16 out; output row tiles sharded")

        def cpu_base():
            rows = 256
            af, bf = a[:rows].float(), b.float()
            af @ bf
            t0 = time.perf_counter()
            for _ in range(3):
                af @ bf
            dt = (time.perf_counter() - t0) / 3
            return 2.0 * rows * n * n / dt / 1e12, f"torch fp32 matmul of a {rows}-row slab of A with all of B ({dt * 1e3:.0f} ms each, 3 runs)"
    elif wl in ("matmul_bfp8w", "matmul_bfp4w"):
        bits = 8 if wl == "matmul_bfp8w" else 4
        if bits == 4 and world > 1:
            raise SystemExit("matmul_bfp4w is a one-GPU workload")
        m, k, n = 4096, 8192, 28672
        x = cases.gen((m, k), "normal", 0)
        s0, c0 = shard.split_units(n // 32, world)[rank]
        # the weight shard is generated and packed per rank (N(0, 0.02), seed 1 + first column tile)
        w = cases.gen((k, c0 * 32), "normal*0.02", 1 + s0, torch.float32)
        W = ttnn.from_torch(w, dtype=ttnn.bfloat8_b if bits == 8 else ttnn.bfloat4_b)
        host_in = [x.pin_memory()]
        flops = 2.0 * m * k * n
        out_bytes = m * n * 2
        kernel = f"ttlb_unpack_bfp{bits}_kernel + " + ("ttlb_gemm_bf16_kernel" if args.gemm_variant == 0 else "ttlb_gemm_bf16_2cta_kernel")
        if bits == 8 and (capi.BFP8_MODE_DEFAULT if args.bfp8_mode is None else args.bfp8_mode) in (1, 2) and world == 1:
            kernel = "ttlb_gemm_bfp8w_tmem_kernel"   # expansion inside the mainloop (ttlb_set_bfp8_mode)
        chunks = 2 if world > 1 else 1

        def compute(xs):
            return ops.matmul(T(xs[0]), W)._tensor

        def step(xs):
            return shard.sharded_matmul_cols(xs[0], W, n, lambda p, q: ops.matmul(T(p), q)._tensor, chunks=chunks)
        if world > 1:
            # T1 needs all 28672 weight columns: the rank's shard repeated along the columns (tile rows of the
            # packed layout are contiguous; the timing does not depend on the values)
            tile_bytes = W._packed.numel() // ((k // 32) * c0)
            packed_full = W._packed.view(k // 32, c0 * tile_bytes).repeat(1, world).reshape(-1)
            W_full = T(torch.empty(0), _packed=packed_full, _logical_shape=(k, n), _packed_bits=bits)
            full_compute = lambda xs: ops.matmul(T(xs[0]), W_full)  # noqa: E731
        desc = (f"activations bf16 [4096,8192] N(0,1); weights [8192,28672] N(0,0.02) packed to bfloat{bits}_b tiles "
                f"(resident in HBM); fp32 accumulate, bf16 out; weight column tiles sharded")

        def cpu_base():
            from oracle import bfp8_oracle

            rows, cols = 128, 2048
            wf = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w[:, :cols].numpy()), k, cols)) if bits == 8 else w[:, :cols]
            xf = x[:rows].float()
            t0 = time.perf_counter()
            for _ in range(3):
                wf = torch.from_numpy(bfp8_oracle.unpack(bfp8_oracle.pack(w[:, :cols].numpy()), k, cols)) if bits == 8 else wf
                xf @ wf
            dt = (time.perf_counter() - t0) / 3
            return 2.0 * rows * k * cols / dt / 1e12, (f"oracle/bfp8_oracle pack + unpack of a {cols}-column weight stripe, torch fp32 "
                                                        f"matmul with {rows} activation rows ({dt * 1e3:.0f} ms each, 3 runs)")
    elif wl == "attention":
        B, H, S, D = 8, 32, 4096, 128
        chunks = shard.pick_chunks(B * H, world)
        mine = shard.cyclic_units(B * H, world, rank, chunks)
        n_local = sum(c for _, c in mine)
        host_in = [cases.gen((n_local * S, D), "normal", sd + 10 * mine[0][0]).reshape(n_local, S, D).pin_memory()
                   for sd in (0, 1, 2)]
        flops = 4.0 * B * H * S * S * D / 2
        out_bytes = B * H * S * D * 2
        kernel = "ttlb_attention_kernel"

        def compute(x):
            return ops.attention(T(x[0]), T(x[1]), T(x[2]), causal=True, scale=D ** -0.5)._tensor

        def step(x):
            return shard.sharded_attention(x[0], x[1], x[2], B * H, lambda q, k_, v: ops.attention(
                T(q), T(k_), T(v), causal=True, scale=D ** -0.5)._tensor, chunks=chunks)
        if world > 1:
            def full_compute(x, _cache={}):
                if "q" not in _cache:   # all 256 heads: the rank's heads repeated (the timing does not depend on the values)
                    for name, t in zip("qkv", x):
                        _cache[name] = t.repeat(world, 1, 1)
                    _cache["o"] = torch.empty_like(_cache["q"])
                return ops.attention(T(_cache["q"]), T(_cache["k"]), T(_cache["v"]), causal=True, scale=D ** -0.5,
                                     out=T(_cache["o"]))
        desc = ("Q,K,V bf16 [8,32,4096,128] N(0,1), causal, scale 1/sqrt(128); the 256 (batch, head) pairs sharded; "
                "FLOPs counted causal-halved")

        def cpu_base():
            from oracle import attention_oracle

            q, k_, v = (t[:1].clone() for t in host_in)
            t0 = time.perf_counter()
            attention_oracle.attention_tiles(q, k_, v, True, D ** -0.5)
            dt = time.perf_counter() - t0
            return 4.0 * S * S * D / 2 / dt / 1e12, f"oracle/attention_oracle.attention_tiles on one head ({dt * 1e3:.0f} ms, 1 run)"
    else:
        raise SystemExit(f"unknown workload {wl}")

    dev_in = [t.to(dev) for t in host_in]
    gather = "nccl all-gather"
    mode = gather_mode
    if mode == "auto":
        # measured on 2 and 4 GPUs: publication from the kernel's epilogue beats every separate gather; through the
        # switch (multimem.st) for the matmuls, and for attention on 2 GPUs; attention on 4 GPUs is faster with plain
        # peer stores (0.365 against 0.399 ms)
        mode = "peers" if (wl == "attention" and world >= 4) else "fused"
    rounds_used = None
    if world > 1 and mode != "nccl":
        so, why = None, ""
        try:
            if wl == "matmul_bf16_8192":
                so = shard.SymmetricOutput((n, n), torch.bfloat16, dev)
            elif wl == "matmul_bfp8w":
                so = shard.SymmetricOutput((m, n), torch.bfloat16, dev) if mode in ("multicast", "fused", "peers") else \
                    shard.SymmetricOutput((world, m, c0 * 32), torch.bfloat16, dev)
            else:
                so = shard.SymmetricOutput((B * H, S, D), torch.bfloat16, dev)
        except Exception as e:   # symmetric memory unavailable on this rank
            why = f"{type(e).__name__}: {e}"
        # every rank takes the same path: one rank without symmetric memory sends all of them to NCCL
        flag = torch.tensor([1 if so is not None else 0], device=dev)
        env.dist.all_reduce(flag, op=env.dist.ReduceOp.MIN)
        if int(flag.item()) == 0:
            mode = "nccl"
            gather = f"nccl all-gather (symmetric memory unavailable on some rank{': ' + why if why else ''})"[:160]
            so = None
        if so is not None:
            if mode == "fused" and not so.has_multicast:
                mode = "peers"
            if mode == "multicast" and not so.has_multicast:
                mode = "p2p"
            if mode == "multicast" and so.has_multicast:
                # compute into the local copy, then one kernel re-sends the shard through the switch
                # (multimem.st, coalesced): 1x outgoing traffic instead of (world-1)x
                esz = 2
                # run_chunk(x, u0, u1) computes units [u0, u1) of this rank's shard (rows / heads) in place
                if wl == "matmul_bf16_8192":
                    ml = n // world
                    a_contig = a[rank * ml:(rank + 1) * ml].contiguous().to(dev)
                    mine_view = so.buf[rank * ml:(rank + 1) * ml]
                    units = ml
                    run_chunk = lambda x, u0, u1: ops.matmul(T(a_contig[u0:u1]), T(x[1]), out=T(mine_view[u0:u1]))  # noqa: E731
                elif wl == "matmul_bfp8w":
                    nl = c0 * 32
                    mine_view = so.buf[:, rank * nl:(rank + 1) * nl]
                    units = m
                    run_chunk = lambda xs, u0, u1: ops.launch_gemm(ctx, T(xs[0]), W, T(mine_view), (u0, u1, 0, nl),  # noqa: E731
                                                                   capi.current_stream())
                else:
                    ul = (B * H) // world
                    mine_view = so.buf[rank * ul:(rank + 1) * ul]
                    host_in = [cases.gen((ul * S, D), "normal", sd + 10 * rank).reshape(ul, S, D).pin_memory() for sd in (0, 1, 2)]
                    dev_in = [t.to(dev) for t in host_in]
                    units = ul
                    run_chunk = lambda x, u0, u1: ops.attention(T(x[0][u0:u1]), T(x[1][u0:u1]), T(x[2][u0:u1]),  # noqa: E731
                                                                causal=True, scale=D ** -0.5, out=T(mine_view[u0:u1]))
                v2 = mine_view if mine_view.dim() == 2 else mine_view.reshape(mine_view.shape[0], -1)
                row_bytes_, ld_bytes_ = v2.shape[1] * esz, v2.stride(0) * esz
                want = args.mc_rounds if args.mc_rounds > 0 else (4 if world >= 4 else 1)
                rounds = max(1, min(want, units // 256 if wl != "attention" else units))
                while units % rounds:
                    rounds -= 1
                rounds_used = rounds
                side = torch.cuda.Stream()

                def step(x):
                    # the re-send of round r (a light kernel next to the persistent compute CTAs) runs on a side
                    # stream under the compute of round r + 1
                    main = torch.cuda.current_stream()
                    per = units // rounds
                    for r in range(rounds):
                        u0, u1 = r * per, (r + 1) * per
                        run_chunk(x, u0, u1)
                        ev = torch.cuda.Event()
                        ev.record(main)
                        side.wait_event(ev)
                        with torch.cuda.stream(side):
                            ctx.multimem_bcast(v2[u0:u1].data_ptr(), ld_bytes_, so.multicast_ptr_of(v2[u0:u1]), ld_bytes_,
                                               u1 - u0, row_bytes_, capi.current_stream())
                    main.wait_stream(side)
                    return so.barrier()
                gather = (f"local compute in {rounds} round(s); each round's part of the shard is re-sent once through the "
                          "NVSwitch (multimem.st kernel) under the next round's compute; barrier")
            elif mode in ("fused", "peers"):
                # publication fused into the GEMM epilogue: every tile is stored while the tensor cores work on the
                # next one - once with multimem.st (the NVSwitch delivers it to all ranks), or with plain stores into
                # every rank's copy of the buffer; one launch per rank, then a cross-rank barrier
                if wl == "matmul_bf16_8192":
                    ml = n // world
                    a_contig = a[rank * ml:(rank + 1) * ml].contiguous().to(dev)
                    mine_view = so.buf[rank * ml:(rank + 1) * ml]
                    where = ({"multicast_ptr": so.multicast_ptr_of(mine_view)} if mode == "fused" else
                             {"peer_ptrs": so.peer_ptrs_of(mine_view)})

                    def step(x):
                        ops.matmul(T(a_contig), T(x[1]), out=T(mine_view), **where)
                        return so.barrier()
                elif wl == "attention":
                    ul = (B * H) // world
                    mine_view = so.buf[rank * ul:(rank + 1) * ul]
                    host_in = [cases.gen((ul * S, D), "normal", sd + 10 * rank).reshape(ul, S, D).pin_memory() for sd in (0, 1, 2)]
                    dev_in = [t.to(dev) for t in host_in]
                    where = ({"multicast_ptr": so.multicast_ptr_of(mine_view)} if mode == "fused" else
                             {"peer_ptrs": so.peer_ptrs_of(mine_view)})

                    def step(x):
                        ops.attention(T(x[0]), T(x[1]), T(x[2]), causal=True, scale=D ** -0.5, out=T(mine_view), **where)
                        return so.barrier()
                else:
                    nl = c0 * 32
                    mine_view = so.buf[:, rank * nl:(rank + 1) * nl]
                    where = ({"multicast_ptr": so.multicast_ptr_of(mine_view)} if mode == "fused" else
                             {"peer_ptrs": so.peer_ptrs_of(mine_view)})

                    def step(xs):
                        ops.launch_gemm(ctx, T(xs[0]), W, T(mine_view), (0, m, 0, nl), capi.current_stream(), **where)
                        return so.barrier()
                gather = ("multimem.st in the kernel's epilogue (NVSwitch multicast, row-contiguous stores), then a cross-rank barrier"
                          if mode == "fused" else
                          "plain stores from the kernel's epilogue into every rank's copy of the output (peer memory, "
                          "row-contiguous), then a cross-rank barrier")
            else:
                mode = "p2p"
                if wl == "matmul_bf16_8192":
                    step = lambda x: shard.symmetric_matmul_rows(  # noqa: E731
                        so, x[0], x[1], lambda p_, q_, o_: ops.matmul(T(p_), T(q_), out=T(o_)), chunks)
                elif wl == "matmul_bfp8w":
                    final = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
                    step = lambda xs: shard.symmetric_matmul_cols(  # noqa: E731
                        so, xs[0], W, final, lambda p_, q_, o_: ops.matmul(T(p_), q_, out=T(o_)), 2)
                else:
                    step = lambda x: shard.symmetric_attention(  # noqa: E731
                        so, x[0], x[1], x[2], lambda q_, k_, v_, o_: ops.attention(T(q_), T(k_), T(v_), causal=True,
                                                                                 scale=D ** -0.5, out=T(o_)), chunks)
                gather = "peer-to-peer copies into a symmetric buffer (copy engines), overlapped with compute"

    steps = min(args.steps, 30)
    sampler = ClockSampler(physical_gpu_index(env.local))
    sampler.start()
    l0 = ctx.launch_count()
    ms_compute = timed(env, lambda: compute(dev_in), steps, args.warmup)
    launches = (ctx.launch_count() - l0) // (steps + args.warmup)
    clocks = sampler.stop()
    ms_step = timed(env, lambda: step(dev_in), steps, args.warmup) if world > 1 else ms_compute
    ms_single = timed(env, lambda: full_compute(dev_in), min(steps, 10), args.warmup) if full_compute is not None else ms_compute
    ctx.check_status(capi.current_stream())
    gathered_same = None
    if world > 1:
        # every rank must now hold the same full output, bit for bit: compare a checksum of it across the ranks
        full = step(dev_in)
        env.barrier()
        chk = full.reshape(-1).view(torch.int16).to(torch.int64)
        chk = torch.stack([chk.sum(), (chk * (torch.arange(chk.numel(), device=dev) % 8191 + 1)).sum()])
        allc = [torch.empty_like(chk) for _ in range(world)]
        env.dist.all_gather(allc, chk)
        gathered_same = all(torch.equal(allc[0], c) for c in allc)
        del full, chk, allc

    result_holder = {}

    def e2e():
        xs = [t.to(dev, non_blocking=True) for t in host_in]
        out = step(xs)
        if "host" not in result_holder:
            result_holder["host"] = torch.empty(out.shape, dtype=out.dtype).pin_memory()
        result_holder["host"].copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    e2e_ms = float("nan")
    if not args.no_e2e:
        e2e_ms = timed(env, e2e, args.e2e_steps, 1)
    burst, sustained, src = measured_peak_tensor()
    per_gpu_kernel_tf = flops / world / (ms_compute * 1e-3) / 1e12
    rec = {
        "workload": f"{wl}: {desc}", "n_gpus": world, "scaling": "strong", "unit": "TFLOP/s", "dtype": "bf16",
        "value": flops / (ms_step * 1e-3) / 1e12, "ms_per_step": ms_step, "steps": steps,
        "ms_compute_only": ms_compute, "tflops_compute_only": flops / (ms_compute * 1e-3) / 1e12,
        "gather": {"mode": mode if world > 1 else "none (1 GPU)", "how": gather if world > 1 else None},
        "l2": "operands exceed the 126 MB L2" if wl != "attention" else "Q,K,V,O 1 GB total exceed L2",
        "roofline": {"bound": "tensor", "achieved": per_gpu_kernel_tf, "peak": burst, "unit": "TFLOP/s",
                     "frac": per_gpu_kernel_tf / burst, "traffic": (TRAFFIC_BYTES.get(wl + "_in_mainloop" if kernel == "ttlb_gemm_bfp8w_tmem_kernel" else wl)
                                 if world == 1 else None),
                     "peak_source": src, "peak_sustained": sustained, "kernel": kernel},
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in),
                "d2h_bytes_per_step": int(result_holder["host"].numel() * 2) if "host" in result_holder else 0,
                "ms_per_step": e2e_ms, "steps": args.e2e_steps},
        "gpu_launches_per_step": launches,
        "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
    }
    if world == 1 and wl in ("matmul_bf16_8192", "matmul_bfp8w") and not args.no_dsl:
        rec["dsl"] = through_the_dsl(dev_in[0], dev_in[1] if wl == "matmul_bf16_8192" else W, compute(dev_in))
    if world > 1:
        recv = out_bytes * (world - 1) / world
        floor = recv / (NVLINK_MEASURED_GBS * 1e9) * 1e3
        rec["gather"].update({
            "rounds": rounds_used, "every_rank_holds_the_same_output": gathered_same, "bytes_received_per_gpu": recv, "gather_floor_ms": floor,
            "gather_floor_note": (f"every GPU must receive (N-1)/N of the output; {NVLINK_MEASURED_GBS:.0f} GB/s per direction "
                                  f"measured peer-copy rate ({NVLINK_NOMINAL_GBS:.0f} nominal)"),
            "step_floor_ms": max(floor, ms_compute), "frac_of_step_floor": max(floor, ms_compute) / ms_step})
        rec["ms_single_gpu"] = ms_single
        rec["sharded_efficiency"] = ms_single / (world * ms_step)
        rec["sharded_efficiency_compute_only"] = ms_single / (world * ms_compute)
    elif rank == 0 and not args.no_cpu_baseline:
        try:
            v, what = cpu_base()
            rec["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port", "sample": what}
        except Exception as e:   # the baseline is a reported figure, never a reason to lose the measurement
            rec["cpu_baseline"] = {"error": f"{type(e).__name__}: {e}"[:160]}
    return rec


def run_sharded(args, env: "Env") -> None:
    """`--workload matmul_bf16_8192 | matmul_bfp8w | matmul_bfp4w | attention`: one JSON line for that workload."""
    known = ["auto", "p2p", "multicast", "fused", "peers", "nccl"]
    modes = known[1:] if args.gather == "all" else args.gather.split(",")
    if any(m not in known for m in modes):
        raise SystemExit(f"--gather: one of {known + ['all']}, or several of them separated by commas")
    for mode in modes:
        rec = measure_sharded(args, args.workload, env, mode)
        if env.rank == 0:
            line = {"metric": "bf16/bfp8 matmul & attention TFLOP/s", "value": rec["value"], "unit": "TFLOP/s",
                    "n_gpus": env.world, "steps": rec["steps"], "warmup": args.warmup, "ms_per_step": rec["ms_per_step"],
                    "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                    "config": {"workload": rec["workload"], "gather": rec["gather"], "ms_compute_only": rec["ms_compute_only"],
                               "tflops_compute_only": rec["tflops_compute_only"], "l2": rec["l2"]},
                    "roofline": rec["roofline"], "e2e": rec["e2e"], "gpu_launches": rec["gpu_launches_per_step"] * rec["steps"],
                    "clocks": rec["clocks"]}
            for k in ("cpu_baseline", "ms_single_gpu", "sharded_efficiency", "sharded_efficiency_compute_only"):
                if k in rec:
                    line[k] = rec[k]
            print(json.dumps(line), flush=True)


def measure_add_1024(args) -> dict:
    """configs[0]: C = A + B on bf16 [1024, 1024] (the reference's own CPU-runnable case), one GPU.
    6.3 MB of traffic: the launch is latency-bound, so the line reports time and GB/s without a
    roofline claim.  The operands fit in L2, so a buffer larger than L2 is written between iterations
    and each iteration is timed on its own."""
    import importlib.util

    import torch

    import ttl_b200

    ttl_b200.install()
    import ttnn

    from ttl_b200 import capi

    torch.cuda.set_device(0)
    spec = importlib.util.spec_from_file_location("bench_programs_eltwise", ROOT / "tests" / "programs" / "eltwise.py")
    programs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(programs)
    n = 1024
    host = [torch.randn(n, n, generator=torch.Generator().manual_seed(s)).to(torch.bfloat16).pin_memory() for s in (0, 1)]
    dev = [ttnn.from_torch(t) for t in host]
    out = ttnn.empty((n, n), dtype=ttnn.bfloat16)
    plan = programs.eltwise_add.plan(*dev, out)
    assert len(plan.launches) == 1, plan.describe()
    desc = plan.launches[0].desc(dev + [out])
    ctx = capi.context(0)
    stream = capi.current_stream()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    algo = 3 * n * n * 2
    for _ in range(args.warmup):
        ctx.eltwise(desc, stream)
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    l0 = ctx.launch_count()
    times = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.eltwise(desc, stream)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    launches = ctx.launch_count() - l0
    clocks = sampler.stop()
    ms = sorted(times)[len(times) // 2]
    assert torch.equal(ttnn.to_torch(out), host[0] + host[1]), "C = A + B is not bit-exact"
    host_out = torch.empty((n, n), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        tensors = [ttnn.from_torch(t) for t in host]
        y = ttnn.empty((n, n), dtype=ttnn.bfloat16)
        programs.eltwise_add(*tensors, y)
        ttnn.to_torch(y, out=host_out)

    e2e_step()
    torch.cuda.synchronize()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    f1.record()
    torch.cuda.synchronize()
    e2e_ms = f0.elapsed_time(f1) / args.e2e_steps
    peak, peak_src = measured_peak_hbm()
    gbs = algo / (ms * 1e-3) / 1e9
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import tile_oracle

        tile_oracle.eval_expression(("add", 0, 1), host, (n, n), "native")
        t0 = time.perf_counter()
        for _ in range(5):
            tile_oracle.eval_expression(("add", 0, 1), host, (n, n), "native")
        dt = (time.perf_counter() - t0) / 5
        cpu = {"value": algo / dt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"oracle/tile_oracle.eval_expression on the whole 1024x1024 problem, mean of 5 runs ({dt * 1e3:.2f} ms each)"}
    rec = {
        "metric": "eltwise HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "eltwise_add_1024: C = A + B, bf16 [1024,1024], N(0,1) seeds 0/1, bf16 rounding, bit-exact "
                               "result checked in this run",
                   "l2": "256 MB written between iterations (operands fit in L2); median of per-iteration CUDA-event times",
                   "algorithmic_bytes_per_step": algo},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "peak_source": peak_src, "kernel": "ttlb_eltwise_jit",
                     "note": "6.3 MB per launch: launch-latency bound, no bandwidth claim"},
        "e2e": {"value": algo / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 2 * n * n * 2,
                "d2h_bytes_per_step": n * n * 2, "ms_per_step": e2e_ms, "steps": args.e2e_steps},
        "gpu_launches": launches, "clocks": clocks}
    if cpu is not None:
        rec["cpu_baseline"] = cpu
    try:
        rec["cuda_graph"] = add_1024_in_a_graph(ctx, plan, n, algo, peak)
    except Exception as e:   # reported, not fatal: the figure above stands on its own
        rec["cuda_graph"] = {"error": f"{type(e).__name__}: {e}"[:200]}
    return rec


def add_1024_in_a_graph(ctx, plan, n, algo, peak) -> dict:
    """The same launch without the host in the loop: 64 launches on 64 different operand sets (403 MB, so that no
    launch finds its operands in the 126 MB L2) captured in one CUDA graph and replayed.  A launch through the
    Python front end costs several microseconds of host time for one microsecond of traffic; a captured plan is
    what a caller with a launch-bound inner loop would replay."""
    import torch
    import ttnn

    from ttl_b200 import capi

    sets = 64
    g = torch.Generator(device="cuda").manual_seed(7)
    ops_ = [[ttnn.Tensor(torch.randn(n, n, generator=g, device="cuda").to(torch.bfloat16)) for _ in range(2)] +
            [ttnn.empty((n, n), dtype=ttnn.bfloat16)] for _ in range(sets)]
    descs = [plan.launches[0].desc(t) for t in ops_]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for d in descs[:2]:
            ctx.eltwise(d, capi.current_stream())
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for d in descs:
            ctx.eltwise(d, capi.current_stream())
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 20
    e0.record()
    for _ in range(reps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ctx.check_status(capi.current_stream())
    ms = e0.elapsed_time(e1) / (reps * sets)
    ok = all(torch.equal(t[2]._tensor, t[0]._tensor + t[1]._tensor) for t in (ops_[0], ops_[sets // 2], ops_[-1]))
    gbs = algo / (ms * 1e-3) / 1e9
    return {"launches_per_replay": sets, "replays_timed": reps, "ms_per_launch": ms, "value": gbs, "unit": "GB/s",
            "frac_of_hbm_peak": gbs / peak, "bit_exact": bool(ok),
            "l2": "64 operand sets of 6.3 MB used in turn (403 MB): no launch finds its operands in L2"}


def run_reduce_8192(args) -> None:
    """`ttl.math.reduce_sum / reduce_max` over a bf16 [8192, 8192] tensor (--workload reduce_<sum|max>_<rows|cols|all>_8192),
    one GPU.  HBM-bound: 134 MB read per launch; two input tensors are used in turn so that no launch finds
    its input in L2.  The result is checked against a float64 reduction in the same run."""
    import importlib.util

    import torch

    import ttl_b200

    ttl_b200.install()
    import ttnn

    from ttl_b200 import capi

    _, op, which, _n = args.workload.split("_")
    dims = {"rows": [0], "cols": [1], "all": [0, 1]}[which]
    torch.cuda.set_device(0)
    spec = importlib.util.spec_from_file_location("bench_programs_reduce", ROOT / "tests" / "programs" / "reduce.py")
    programs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(programs)
    n = 8192
    host = [torch.randn(n, n, generator=torch.Generator().manual_seed(s)).to(torch.bfloat16).pin_memory() for s in (0, 1)]
    dev = [ttnn.from_torch(t) for t in host]
    scaler = ttnn.from_torch(torch.ones(32, 32, dtype=torch.bfloat16))
    out_shape = (1 if 0 in dims else n, 1 if 1 in dims else n)
    out = ttnn.empty(out_shape, dtype=ttnn.bfloat16)
    prog = programs.make_reduce(op, dims)
    plan = prog.plan(dev[0], scaler, out)
    assert len(plan.launches) == 1, plan.describe()
    descs = [plan.launches[0].desc([d, scaler, out]) for d in dev]
    ctx = capi.context(0)
    stream = capi.current_stream()
    algo = n * n * 2 + out_shape[0] * out_shape[1] * 2
    for i in range(args.warmup):
        ctx.reduce(descs[i % 2], stream)
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    l0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        ctx.reduce(descs[i % 2], stream)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = ctx.launch_count() - l0
    clocks = sampler.stop()
    last = host[(args.steps - 1) % 2].double()
    ref = last.sum(dim=dims, keepdim=True) if op == "sum" else last.amax(dim=dims, keepdim=True)
    got = ttnn.to_torch(out).double()
    tol = 2.0 ** -8 * ref.abs().max().item() + (0.0 if op == "max" else 1e-3 * n)
    assert (got - ref).abs().max().item() <= tol, "reduction result is wrong"
    host_out = torch.empty(out_shape, dtype=torch.bfloat16).pin_memory()

    def e2e_step(i):
        x = ttnn.from_torch(host[i % 2])
        y = ttnn.empty(out_shape, dtype=ttnn.bfloat16)
        prog(x, scaler, y)
        ttnn.to_torch(y, out=host_out)

    e2e_step(0)
    torch.cuda.synchronize()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for i in range(args.e2e_steps):
        e2e_step(i)
    f1.record()
    torch.cuda.synchronize()
    e2e_ms = f0.elapsed_time(f1) / args.e2e_steps
    peak, peak_src = measured_peak_hbm()
    gbs = algo / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "eltwise HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"{args.workload}: reduce_{op}(A, s, dims={dims}), A bf16 [8192,8192] N(0,1), fp32 combine, "
                               "one bf16 rounding; result checked against a float64 reduction in this run",
                   "l2": "two 134 MB inputs used in turn (each larger than L2)", "algorithmic_bytes_per_step": algo},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "peak_source": peak_src, "kernel": "ttlb_reduce_jit",
                     "note": "peak is a copy (read + write); this kernel only reads"},
        "e2e": {"value": algo / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": n * n * 2,
                "d2h_bytes_per_step": out_shape[0] * out_shape[1] * 2, "ms_per_step": e2e_ms, "steps": args.e2e_steps},
        "gpu_launches": launches, "clocks": clocks}))


def run_softmax_8192(args) -> None:
    """Row softmax of a bf16 [8192, 8192] tensor written as a tile program (tests/programs/reduce.py,
    make_softmax): the plan is three launches - row maximum, row sum of exp(x - max) fused into the
    reduction, exp(x - max) / sum - so x is read three times and y written once.  Algorithmic bytes: one
    read and one write of the tensor (what a kernel holding a whole row on chip would move)."""
    import importlib.util

    import torch

    import ttl_b200

    ttl_b200.install()
    import ttnn

    from ttl_b200 import capi

    torch.cuda.set_device(0)
    spec = importlib.util.spec_from_file_location("bench_programs_reduce", ROOT / "tests" / "programs" / "reduce.py")
    programs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(programs)
    n = 8192
    host = torch.randn(n, n, generator=torch.Generator().manual_seed(0)).to(torch.bfloat16).pin_memory()
    x = ttnn.from_torch(host)
    scaler = ttnn.from_torch(torch.ones(32, 32, dtype=torch.bfloat16))
    y = ttnn.empty((n, n), dtype=ttnn.bfloat16)
    prog = programs.make_softmax(fp32_dest_acc_en=True)
    plan = prog.plan(x, scaler, y)
    kinds = [d["kind"] for d in plan.describe()]
    assert kinds in (["row_fused"], ["reduce_max", "reduce_sum", "eltwise"]), kinds
    ctx = capi.context(0)
    algo = 2 * n * n * 2
    for _ in range(args.warmup):
        plan.run([x, scaler, y])
    torch.cuda.synchronize()
    sampler = ClockSampler(physical_gpu_index(0))
    sampler.start()
    l0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        plan.run([x, scaler, y])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    launches = ctx.launch_count() - l0
    clocks = sampler.stop()
    got = ttnn.to_torch(y).double()
    want = torch.softmax(host.double(), dim=1)
    assert ((got - want).abs() <= 2.0 ** -6 * want + 1e-7).all(), "softmax result is wrong"
    host_out = torch.empty((n, n), dtype=torch.bfloat16).pin_memory()

    def e2e_step():
        xx = ttnn.from_torch(host)
        yy = ttnn.empty((n, n), dtype=ttnn.bfloat16)
        prog(xx, scaler, yy)
        ttnn.to_torch(yy, out=host_out)

    e2e_step()
    torch.cuda.synchronize()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record()
    for _ in range(args.e2e_steps):
        e2e_step()
    f1.record()
    torch.cuda.synchronize()
    e2e_ms = f0.elapsed_time(f1) / args.e2e_steps
    peak, peak_src = measured_peak_hbm()
    gbs = algo / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "eltwise HBM GB/s", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": "softmax_8192: row softmax as a tile program (reduce_max, reduce_sum, exp, broadcast), "
                               "bf16 [8192,8192] N(0,1), fp32 intermediates; checked against a float64 softmax in this run",
                   "l2": "input and output are 134 MB each (larger than L2)", "algorithmic_bytes_per_step": algo,
                   "plan": kinds, "launches_per_step": len(kinds)},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "traffic": None,
                     "peak_source": peak_src,
                     "kernel": "ttlb_rowfused_jit" if kinds == ["row_fused"] else "ttlb_reduce_jit x2 + ttlb_eltwise_jit",
                     "note": "row-resident kernel: x read once, y written once" if kinds == ["row_fused"] else
                             "three passes over x: at most half of the peak is reachable with this plan"},
        "e2e": {"value": algo / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": n * n * 2,
                "d2h_bytes_per_step": n * n * 2, "ms_per_step": e2e_ms, "steps": args.e2e_steps},
        "gpu_launches": launches, "clocks": clocks}))


def measure_contract(args, env: "Env") -> dict:
    """The contract line: the fused element-wise + broadcast program (replicas at N > 1)."""
    import importlib.util

    import torch

    import ttl_b200

    ttl_b200.install()
    import ttnn

    from ttl_b200 import capi

    rank, local, world = env.rank, env.local, env.world
    spec = importlib.util.spec_from_file_location("bench_programs_eltwise", ROOT / "tests" / "programs" / "eltwise.py")
    programs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(programs)
    program = programs.fused_exp_bcast_f32acc

    host = [t.pin_memory() for t in make_inputs()]
    dev = [ttnn.from_torch(t) for t in host]
    out = ttnn.empty((N, N), dtype=ttnn.bfloat16)
    t_trace0 = time.perf_counter()
    plan = program.plan(*dev, out)
    trace_s = time.perf_counter() - t_trace0
    assert len(plan.launches) == 1, plan.describe()
    desc = plan.launches[0].desc(dev + [out])
    ctx = capi.context(local)
    ctx.set_eltwise_mode({"auto": capi.ELTWISE_AUTO, "generic": capi.ELTWISE_GENERIC,
                          "specialised": capi.ELTWISE_SPECIALISED}[args.eltwise_mode])
    stream = capi.current_stream()

    for _ in range(args.warmup):
        ctx.eltwise(desc, stream)
    env.barrier()
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    l0 = ctx.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    env.barrier()
    e0.record()
    for _ in range(args.steps):
        ctx.eltwise(desc, stream)
    e1.record()
    env.barrier()
    launches = ctx.launch_count() - l0
    clocks = sampler.stop()
    ms_per_step = env.max_over_ranks(e0.elapsed_time(e1)) / args.steps
    per_gpu_gbs = ALGO_BYTES / (ms_per_step * 1e-3) / 1e9
    value = per_gpu_gbs * world

    # ---- end to end through the public API: pinned host -> HBM -> kernel -> pinned host
    host_out = torch.empty((N, N), dtype=torch.bfloat16).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = host_out.numel() * host_out.element_size()

    def e2e_step():
        if args.e2e_chunks > 1:   # row chunks: copy-in, kernel and copy-out overlapped on three streams
            ttl_b200.run_streamed(program, host, host_out, chunks=args.e2e_chunks)
            return
        tensors = [ttnn.from_torch(t) for t in host]
        y = ttnn.empty((N, N), dtype=ttnn.bfloat16)
        program(*tensors, y)
        ttnn.to_torch(y, out=host_out)

    e2e_ms = float("nan")
    if not args.no_e2e:
        e2e_step()
        env.barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(args.e2e_steps):
            e2e_step()
        f1.record()
        env.barrier()
        e2e_ms = env.max_over_ranks(f0.elapsed_time(f1) / args.e2e_steps)
    e2e_value = ALGO_BYTES / (e2e_ms * 1e-3) / 1e9 * world

    peak, peak_src = measured_peak_hbm()
    line = {
        "metric": "eltwise HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "fused_eltwise_bcast_8192: Y=relu(exp(s*A)*b+C), A,C,Y bf16 [8192,8192], "
                               "b bf16 [1,8192], s bf16 [1,1], fp32 intermediates",
                   "replicas": world, "l2": "inputs+output 403 MB > 126 MB L2, no flush needed",
                   "algorithmic_bytes_per_step": ALGO_BYTES, "trace_and_recognise_s": round(trace_s, 3)},
        "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": peak, "unit": "GB/s",
                     "frac": per_gpu_gbs / peak, "traffic": TRAFFIC_BYTES["fused_eltwise_bcast_8192"], "peak_source": peak_src,
                     "kernel": "ttlb_eltwise_jit" if ctx.eltwise_last_path() == capi.ELTWISE_SPECIALISED
                     else "ttlb_eltwise_kernel<bf16>"},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": args.e2e_steps,
                "api": (f"ttl_b200.run_streamed(kernel, pinned inputs, pinned output, chunks={args.e2e_chunks}): "
                        "host->HBM, kernel, HBM->host overlapped per row chunk" if args.e2e_chunks > 1 else
                        "ttnn.from_torch, kernel call, ttnn.to_torch(out=pinned), one after the other")},
        "gpu_launches": launches,
        "clocks": {k: clocks[k] for k in ("sm_mhz", "sm_max_mhz", "reasons")},
    }
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        v, dt, cores = cpu_baseline(1024, 5)
        port = {"value": v, "unit": "GB/s", "cores": cores, "kind": "port",
                "sample": f"oracle/tile_oracle.eval_expression on a 1024x{N} row slab, mean of 5 runs ({dt * 1e3:.1f} ms each)"}
        ref = simulator_baseline(4.0)
        line["cpu_baseline"] = dict(ref, port=port) if ref is not None else port
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all",
                    help="all (default): the contract line with every configuration under `workloads`; or one workload's own line")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--e2e-chunks", type=int, default=8,
                    help="row chunks of the end-to-end leg (1: plain from_torch / call / to_torch, no overlap)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (for profiler runs)")
    ap.add_argument("--eltwise-mode", default="auto", choices=["auto", "generic", "specialised"])
    ap.add_argument("--gemm-variant", type=int, default=1, choices=[0, 1, 2],
                    help="tensor-core GEMM kernel: 0 one CTA per 128x256 tile, 1 two-CTA clusters per 256x256 tile for large outputs, 2 two-CTA always")
    ap.add_argument("--bfp8-chunks", type=int, default=None, choices=[1, 2, 3, 4],
                    help="bfp8 weights, two-step path: column chunks whose expansion overlaps the previous chunk's GEMM")
    ap.add_argument("--mc-rounds", type=int, default=0,
                    help="multicast gather: rounds the local shard is computed and re-sent in (0: 4 rounds on 4 or more GPUs, else 1)")
    ap.add_argument("--no-dsl", action="store_true",
                    help="matmul workloads on one GPU: skip the run of the same product through @ttl.kernel")
    ap.add_argument("--bfp8-mode", type=int, default=None, choices=[0, 1, 2],
                    help="bfp8 weights: 0 unpack kernel + GEMM, 1 expansion inside the GEMM mainloop (operand through tensor memory) "
                         "for large outputs (default), 2 always inside")
    ap.add_argument("--gather", default="auto",
                    help="sharded workloads: how output shards reach the other ranks (p2p: peer-to-peer copies overlapped with "
                         "compute; multicast: multimem.st re-send kernel per round under the next round's compute; fused: "
                         "multimem.st from the kernel's epilogue; peers: plain stores from the epilogue into every rank's copy; "
                         "nccl: all-gather; all, or a comma-separated list: one line per mode)")
    ap.add_argument("--sim-sample", type=float, default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.sim_sample is not None:   # child of simulator_baseline()
        print(json.dumps(simulator_sample(args.sim_sample)))
        return

    if args.impl == "reference":
        run_reference(args)
        return

    import torch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200: the backend has no CPU fallback")
    if args.workload == "softmax_8192":
        run_softmax_8192(args)
        return
    if args.workload.startswith("reduce_"):
        run_reduce_8192(args)
        return
    if args.workload == "eltwise_add_1024":
        print(json.dumps(measure_add_1024(args)))
        return
    env = Env()
    try:
        if args.workload in SHARDED_WORKLOADS + ("matmul_bfp4w",):
            run_sharded(args, env)
            return
        if args.workload not in ("all", "fused_eltwise_bcast_8192"):
            raise SystemExit(f"unknown workload {args.workload}")
        line = measure_contract(args, env)
        if args.workload == "all":
            import gc

            workloads = {}
            if env.world == 1:
                workloads["eltwise_add_1024"] = measure_add_1024(args)
            for wl in SHARDED_WORKLOADS:
                gc.collect()
                torch.cuda.empty_cache()
                try:
                    workloads[wl] = measure_sharded(args, wl, env)
                except Exception as e:   # a workload that fails the same way on every rank must not cost the whole line
                    workloads[wl] = {"error": f"{type(e).__name__}: {e}"[:300]}
            line["workloads"] = workloads
            if env.world > 1:
                line["sharded_efficiency"] = {wl: workloads[wl].get("sharded_efficiency") for wl in SHARDED_WORKLOADS}
            line["gpu_launches_all_workloads"] = line["gpu_launches"] + sum(
                w.get("gpu_launches", 0) + w.get("gpu_launches_per_step", 0) * w.get("steps", 0) for w in workloads.values())
        if env.rank == 0:
            print(json.dumps(line), flush=True)
    finally:
        env.close()


if __name__ == "__main__":
    main()
