#!/usr/bin/env python3
"""Benchmark of the quantized matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one execution of the int8 matmul primitive with its full epilogue
(M = N = K = 4096 per GPU: s8 x s8 -> s8, per-N weight scales, bf16 bias,
GELU-tanh, sum 0.5 over the prior s8 destination, destination scale and
zero-point) through the public C API of libonednn_b200.so.  Inputs are seeded
synthetic tensors with the benchmark's value distributions.

Timing: W warm-up steps, then K steps bracketed by a barrier and a device
synchronisation on both sides and timed with CUDA events on the stream the
kernels run on; the maximum over ranks is reported.  Successive steps rotate
over several independent input sets whose total size exceeds the L2 cache, so
no step finds its operands cached by the previous one.

With N > 1 every rank runs the same per-GPU problem on its own rows of a
(4096*N) x 4096 x 4096 problem with replicated weights (M-split, no data-path
collective): weak scaling.

One JSON line is printed by rank 0.  `value` has the operands resident in HBM;
`e2e` repeats the measurement through the same API with host buffers, the
host-to-device copies of the step's activations and prior destination and the
device-to-host copy of the result inside the timed region.
`--impl reference` times the reference library's own CPU implementation
(oracle/_ref, all host threads) on the same configuration.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "int8_matmul_4096x4096x4096_postops_throughput"
UNIT = "TOPS"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the benchmark kernel, from the ncu
# capture summarised in profiles/tc8_int8_c1_full.md: `bench.py --case c1 --steps 6`, which rotates
# over the same input sets as the timed region, third launch captured
NCU_DRAM_BYTES_PER_LAUNCH = 50.74e6  # dram__bytes_read.sum + dram__bytes_write.sum of one launch, profiles/tc8_int8_c1_full.md
WORKLOAD = "int8 s8:s8:s8 4096x4096:4096x4096, per-N wei scales, bf16 bias, gelu_tanh + sum:0.5, dst scale 0.1 zp 3"


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=float(d["hbm_gbs"]), bf16=float(d["bf16_tflops"]), bf16_sustained=float(d["bf16_tflops_sustained"]),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """SM clock, power and clock-event reasons read through NVML (read-only queries) by a
    thread every few milliseconds while a timed region runs; ``nvidia-smi`` is the fallback."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.rows = []          # (sm_mhz, power_w, reasons bitmask)
        self.max_mhz = None
        self.nv = None
        self.h = None
        self.thread = None
        self.run = False
        self.proc = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            # CUDA_VISIBLE_DEVICES may renumber devices: match by PCI bus id
            import torch
            bus = getattr(torch.cuda.get_device_properties(index), "pci_bus_id", None)
            self.h = None
            if bus is not None:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    if pynvml.nvmlDeviceGetPciInfo(h).bus == bus:
                        self.h = h
                        break
            if self.h is None:
                self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        nv, h = self.nv, self.h
        while self.run:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                try:
                    reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    reasons = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                except Exception:
                    watts = 0.0
                self.rows.append((float(mhz), watts, int(reasons)))
            except Exception:
                pass
            time.sleep(0.002)

    def start(self):
        if self.nv is not None:
            import threading
            self.run = True
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
            return
        try:
            self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=self.f,
                                         stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def pause(self):
        """Stop sampling until the next start() (keeps what was collected)."""
        if self.thread is not None:
            self.run = False
            self.thread.join()
            self.thread = None

    def stop(self):
        if self.nv is not None:
            self.pause()
            if not self.rows:
                return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"]}
            nv = self.nv
            names = (("hw_slowdown", nv.nvmlClocksEventReasonHwSlowdown),
                     ("hw_thermal_slowdown", nv.nvmlClocksEventReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", nv.nvmlClocksEventReasonSwThermalSlowdown),
                     ("sw_power_cap", nv.nvmlClocksEventReasonSwPowerCap),
                     ("hw_power_brake_slowdown", nv.nvmlClocksEventReasonHwPowerBrakeSlowdown))
            mask = 0
            for r in self.rows:
                mask |= r[2]
            sm = sorted(r[0] for r in self.rows)
            return {"sm_mhz": sm[len(sm) // 2], "sm_min_mhz": sm[0], "sm_max_mhz": self.max_mhz, "samples": len(self.rows),
                    "power_w_max": max(r[1] for r in self.rows), "source": "nvml, sampled inside the timed regions",
                    "reasons": [n for n, bit in names if mask & bit]}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.proc.wait()
        self.f.flush()
        rows = [r.split(", ") for r in Path(self.f.name).read_text().strip().splitlines() if r.count(",") >= 8]
        os.unlink(self.f.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in rows)
        reasons = set()
        for r in rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(rows[0][2]), "samples": len(rows),
                "power_w_max": max(float(r[3]) for r in rows), "source": "nvidia-smi -lms 100",
                "reasons": sorted(reasons)}


def reference_arm(args):
    """The reference library's own CPU matmul (its JIT implementation, packed weights) on
    the benchmark configuration, all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from onednn_b200 import workloads as W
    from oracle import binding as B
    if not B.have_reference():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref was not built (reference tree absent at build time)"}))
        return 0
    case = W.config1()
    cores = B.set_threads(0)
    steps = max(1, args.steps)
    _, impl, _, _ = B.run_reference(case, weights_any=True, iters=max(1, args.warmup))
    _, impl, ms_min, ms_avg = B.run_reference(case, weights_any=True, iters=steps)
    value = case.ops / (ms_avg * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": ms_avg, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "s8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "reference_impl": impl, "weights": "packed by the reference's own reorder (not timed)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "reference",
                         "sample": "the full 4096^3 problem, %d executions, mean (min %.2f ms)" % (steps, ms_min)},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--sets", type=int, default=4, help="independent input sets rotated over (L2 defeat)")
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true", help="skip the two-second sustained run (launch lists under a profiler)")
    ap.add_argument("--case", default=None,
                    help="profiling aid: execute one named configuration --steps times and exit "
                         "(c0, c1, c2_m1, c2_m16, c2_m128, c3, c3_4096, c4); prints no benchmark line")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.case:
        return run_one_case(args)
    args.warmup = max(args.warmup, 3)

    import numpy as np
    import torch
    import torch.distributed as dist
    from onednn_b200 import api, dtypes as dt, workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peaks = read_peaks()
    eng = api.Engine(index=local)
    tstream = torch.cuda.current_stream()
    strm = api.Stream(eng, cuda_stream=tstream.cuda_stream)

    # ---- per-GPU problem: rows [rank*4096, (rank+1)*4096) of the M-split problem ----
    case = W.config1(seed=20240612 + rank)
    plan = api.CasePlan(case, eng, strm, weights="any")       # packs the weights once (not timed)
    impl = plan.impl
    M, N, K = case.M, case.N, case.K

    def dev(a):
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    def wrap(t, md):
        return api.Memory(md, eng, handle=t.data_ptr())

    # rotating input sets: src, prior dst / dst (weights and per-N vectors are shared)
    sets = []
    for i in range(args.sets):
        src_t = dev(np.roll(case.src, i, axis=0))
        dst0_t = dev(np.roll(case.dst_init, i, axis=0))
        dst_t = dst0_t.clone()
        a = dict(plan.args)
        a[api.ARG_SRC] = wrap(src_t, plan.mds["src"])
        a[api.ARG_DST] = wrap(dst_t, plan.mds["dst"])
        sets.append(dict(src=src_t, dst0=dst0_t, dst=dst_t, args=a))
    set_bytes = (M * K + 2 * M * N) * args.sets + K * N

    def step(i):
        plan.prim.execute(strm, sets[i % args.sets]["args"])

    sampler = ClockSampler(local)
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler.start()   # clocks are sampled inside the two timed regions only
    launches0 = api.lib().b200_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record(tstream)
    for i in range(args.steps):
        step(i)
    e1.record(tstream)
    barrier()
    ms_total = e0.elapsed_time(e1)
    sampler.pause()
    launches = api.lib().b200_launch_count() - launches0
    strm.wait()

    # ---- the dominant kernel alone: one launch per event pair ----
    kern_ms = []
    for i in range(min(args.steps, 20)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(tstream)
        step(i)
        b.record(tstream)
        b.synchronize()
        kern_ms.append(a.elapsed_time(b))
    kern_avg = sum(kern_ms) / len(kern_ms)

    # ---- the tensor pipe's own peak, measured: a bare tcgen05.mma issue loop on resident operands ----
    mma_peak = {}
    try:
        import ctypes as C
        from onednn_b200 import kernels_abi
        KL = kernels_abi.lib()
        for name, fp8 in (("int8", 0), ("fp8", 1)):
            ops = C.c_uint64()
            best = None
            for rep in range(4):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(tstream)
                rc = KL.b200_tc8_mma_peak_launch(fp8, 4096, None, C.byref(ops), tstream.cuda_stream)
                b.record(tstream)
                b.synchronize()
                if rc != 0:
                    raise RuntimeError("b200_tc8_mma_peak_launch: %d" % rc)
                if rep:  # the first launch pays for the kernel's load
                    ms = a.elapsed_time(b)
                    best = ms if best is None else min(best, ms)
            mma_peak[name] = {"TOPS": ops.value / (best * 1e-3) / 1e12, "ms": best,
                              "how": "tcgen05.mma cta_group::1 128x256x32, 4 per group, 4096 groups per CTA, one CTA per SM, "
                                     "operands resident in shared memory, no copies, no epilogue; best of 3 launches"}
    except Exception as ex:
        mma_peak = {"error": repr(ex)}

    # ---- the same kernel sustained: two seconds of back-to-back launches, clocks sampled throughout ----
    sustained = None
    if not args.no_extras and not args.no_sustained:
        try:
            sus = ClockSampler(local)
            n_sus = max(args.steps, int(2.0 / (ms_total / args.steps * 1e-3)))
            for i in range(args.warmup):
                step(i)
            barrier()
            sus.start()
            e0.record(tstream)
            for i in range(n_sus):
                step(i)
            e1.record(tstream)
            barrier()
            sus_ms = e0.elapsed_time(e1) / n_sus
            sc = sus.stop()
            sustained = {"launches": n_sus, "us_per_launch": sus_ms * 1e3, "TOPS": case.ops / (sus_ms * 1e-3) / 1e12,
                         "clocks": sc, "us_x_median_mhz": sus_ms * 1e3 * (sc.get("sm_mhz") or 0),
                         "note": "burst figure above: %.1f us at the clocks in `clocks`" % (ms_total / args.steps * 1e3)}
        except Exception as ex:
            sustained = {"error": repr(ex)}

    # ---- end to end: host buffers in, host buffer out, same API ----
    # Every step copies that step's src and prior dst (the sum operand) from pinned host memory,
    # executes the primitive and copies dst back to pinned host memory.  The three stages run on
    # three streams chained by events, so that the copies of neighbouring steps overlap the way
    # a caller streaming batches through the library would arrange them; the rotating input sets
    # are the pipeline's buffers.
    h_src = [torch.from_numpy(np.roll(case.src, i, axis=0).copy()).pin_memory() for i in range(2)]
    h_dst0 = [torch.from_numpy(np.roll(case.dst_init, i, axis=0).copy()).pin_memory() for i in range(2)]
    h_out = [torch.empty((M, N), dtype=torch.int8).pin_memory() for _ in range(2)]
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(args.sets)]
    ev_done = [torch.cuda.Event() for _ in range(args.sets)]
    ev_out = [torch.cuda.Event() for _ in range(args.sets)]
    used = [False] * args.sets

    def e2e_step(i):
        k = i % args.sets
        s = sets[k]
        with torch.cuda.stream(s_in):
            if used[k]:
                s_in.wait_event(ev_out[k])      # the set's previous result has left the device
            s["src"].copy_(h_src[i % 2], non_blocking=True)
            s["dst"].copy_(h_dst0[i % 2], non_blocking=True)
            ev_in[k].record(s_in)
        tstream.wait_event(ev_in[k])
        plan.prim.execute(strm, s["args"])
        ev_done[k].record(tstream)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_done[k])
            h_out[i % 2].copy_(s["dst"], non_blocking=True)
            ev_out[k].record(s_out)
        used[k] = True

    e2e_steps = max(3, min(args.steps, 50))
    for i in range(3):
        e2e_step(i)
    barrier()
    sampler.start()
    e0.record(tstream)
    for i in range(e2e_steps):
        e2e_step(i)
    tstream.wait_stream(s_out)
    tstream.wait_stream(s_in)
    e1.record(tstream)
    barrier()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    clocks = sampler.stop()

    # ---- max over ranks ----
    t = torch.tensor([ms_total, e2e_ms, kern_avg], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, kern_avg = (float(x) for x in t.tolist())
    ms_per_step = ms_total / args.steps
    ops = case.ops * world
    value = ops / (ms_per_step * 1e-3) / 1e12
    e2e_value = ops / (e2e_ms * 1e-3) / 1e12

    # ---- correctness of what was timed: sampled rows / columns against the CPU oracle ----
    check = None
    gpu_out = None
    extras = {}
    nsplit = None
    if world > 1 and not args.no_extras:
        # the sharded configuration: every rank takes part
        nsplit = run_c4_sharded(W, torch, dist, rank, world, local)
    cpu_baseline = None
    if rank == 0:
        try:
            from oracle import binding as B
            s = sets[0]
            s["dst"].copy_(s["dst0"])
            plan.prim.execute(strm, s["args"])
            strm.wait()
            got = s["dst"].cpu().numpy()
            gpu_out = got
            c0 = W.config1(seed=20240612 + rank)
            # the same sample under both accumulation orders: exact s32 sums scaled once (what the
            # tensor-core kernel and the reference's optimised implementation compute), and the
            # reference's scalar implementation, which scales every product and sums in f32
            want = B.run_oracle(c0, tanh_mode=1, exact_acc=1, m_step=61, n_step=53)
            want_scalar = B.run_oracle(c0, tanh_mode=0, exact_acc=0, m_step=61, n_step=53)
            samp = got[::61, ::53]
            check = {"sampled_elements": int(samp.size),
                     "mismatches_vs_cpu_oracle": int((samp != want[::61, ::53]).sum()),
                     "mismatches_vs_oracle_in_reference_scalar_order": int((samp != want_scalar[::61, ::53]).sum()),
                     "note": "first count: oracle with exact s32 accumulation (must be 0); second: oracle restating "
                             "ref_int8:any, which accumulates scaled products in f32 (its own +-1 LSB deviations)"}
        except Exception as ex:  # the check must not hide the measurement
            check = {"error": repr(ex)}

        if not args.no_extras:
            extras = run_extras(api, W, dt, eng, strm, tstream, torch, np, peaks)
        if nsplit is not None:
            extras["c4_int8_16384x8192x28672_sharded"] = nsplit
        if sustained is not None:
            extras["c1_sustained"] = sustained

        if not args.no_cpu_baseline:
            try:
                from oracle import binding as B
                cores = B.set_threads(0)
                if B.have_reference():
                    # the same seeded inputs as rank 0's GPU run, so that the outputs can be compared
                    _, rimpl, rmin, ravg = B.run_reference(W.config1(seed=20240612), weights_any=True, iters=10)
                    # once more, a single execution, for the output (the timed runs above each add the sum
                    # post-op onto the previous result)
                    rdst, _, _, _ = B.run_reference(W.config1(seed=20240612), weights_any=True, iters=0)
                    cpu_baseline = {"value": case.ops / (ravg * 1e-3) / 1e12, "unit": UNIT, "cores": cores,
                                    "kind": "reference",
                                    "sample": "the full 4096^3 problem, 10 executions of %s (weights packed by its own reorder), mean" % rimpl}
                    if isinstance(check, dict) and "error" not in check and gpu_out is not None:
                        d = np.abs(gpu_out.astype(np.int16) - rdst.astype(np.int16))
                        check["all_elements"] = int(d.size)
                        check["mismatches_vs_reference_jit_full_output"] = int((d != 0).sum())
                        check["max_abs_diff_vs_reference_jit"] = int(d.max())
                        check["reference_jit_impl"] = rimpl
                    if not args.no_extras:
                        extras["cpu_reference_other_configs"] = cpu_other_configs(B, W, cores)
                else:
                    small = W.config1(512, 512, 1024)
                    t0 = time.time()
                    B.run_oracle(small)
                    sec = time.time() - t0
                    cpu_baseline = {"value": small.ops / sec / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": "512x1024x512 slice of the workload, one execution of the C oracle"}
            except Exception as ex:
                cpu_baseline = {"error": repr(ex)}

    if rank == 0:
        int8_peak = 2.0 * peaks["bf16"]
        # one launch per step and nothing else in the timed region: its events give the launch duration
        achieved = case.ops / (ms_per_step * 1e-3) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "s8", "data": "synthetic",
            "config": {"workload": WORKLOAD, "per_gpu": "4096x4096x4096", "parallelism": "m-split x%d, replicated weights" % world,
                       "impl": impl, "l2": "rotating %d input sets, %.0f MB in total (> 126 MB L2)" % (args.sets, set_bytes / 1e6)},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s",
                         "frac": achieved / int8_peak, "traffic": NCU_DRAM_BYTES_PER_LAUNCH,
                         "traffic_note": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture of "
                                         "`bench.py --case c1` over rotating input sets summarised in "
                                         "profiles/tc8_int8_c1_full.md (below the algorithmic 67.1e6 bytes: the rotating sets partly survive in "
                                         "L2 and the s8 dst is written back after the kernel)",
                         "kernel": "matmul_tc8_kernel<int8, EPI_GELU_Q, SUM_8BIT>", "kernel_ms": ms_per_step, "kernel_ms_single_launch_between_events": kern_avg,
                         "peak_note": "2 x %s bf16 dense burst (%.1f TF/s): MEASURED_PEAKS.json holds no int8 figure; nominal 4500; "
                                      "`measured_mma_peak` is this run's own bare tcgen05.mma issue loop"
                                      % (peaks["source"], peaks["bf16"]),
                         "measured_mma_peak": mma_peak,
                         "frac_of_measured_mma_peak": (achieved / mma_peak["int8"]["TOPS"]) if "int8" in mma_peak else None,
                         "frac_of_nominal_4500": achieved / 4500.0},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": M * K + M * N,
                    "d2h_bytes_per_step": M * N, "steps": e2e_steps,
                    "how": "pinned host src + prior dst -> device, execute, dst -> pinned host, every step; "
                           "copy-in, execute and copy-out on three streams chained by events"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "check": check,
            "also": extras,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


def run_one_case(args):
    """Executes one configuration a few times through the public API; meant to be run under ncu.
    c1 rotates over --sets independent copies of its activations and prior destination, like the
    timed region, so that a captured launch finds its operands in HBM, not in L2."""
    import numpy as np
    from onednn_b200 import api, workloads as W
    cases = {"c0": W.config0, "c1": W.config1, "c2_m1": lambda: W.config2(1), "c2_m16": lambda: W.config2(16),
             "c2_m128": lambda: W.config2(128), "c3": W.config3, "c3_4096": lambda: W.config3(4096, 4096, 4096),
             "c4": W.config4}
    eng = api.Engine()
    strm = api.Stream(eng)
    case = cases[args.case]()
    plan = api.CasePlan(case, eng, strm, weights="any")
    argsets = [plan.args]
    if args.case == "c1":
        for i in range(1, args.sets):
            a = dict(plan.args)
            src = api.Memory(plan.mds["src"], eng)
            src.write(np.roll(case.src, i, axis=0))
            dst = api.Memory(plan.mds["dst"], eng)
            dst.write(np.roll(case.dst_init, i, axis=0))
            a[api.ARG_SRC], a[api.ARG_DST] = src, dst
            argsets.append(a)
    for i in range(max(1, args.steps)):
        plan.prim.execute(strm, argsets[i % len(argsets)])
    strm.wait()
    print("executed %s x%d with %s over %d input set(s)" % (args.case, max(1, args.steps), plan.impl, len(argsets)))
    return 0


def cpu_other_configs(B, W, cores):
    """The reference's CPU implementations on the other configurations, bounded samples: where its
    JIT cannot take a configuration on this host (grouped zero-points, fp8 without AMX-FP16) the
    scalar implementation it dispatches instead is timed, on a reduced shape where the full one
    would take minutes, and the nearest JIT-eligible variant beside it."""
    import copy
    import numpy as np
    from onednn_b200 import dtypes as dt
    from onednn_b200.workloads import Quant
    out = {"cores": cores}
    try:
        c = W.config2(1)
        _, impl, tmin, tavg = B.run_reference(c, iters=1)
        out["c2_wc_u4_m1"] = {"impl": impl, "ms": tavg, "GB/s": c.algorithmic_bytes() / (tavg * 1e-3) / 1e9,
                              "sample": "the full 1x4096x14336 problem, one execution"}
        v = copy.copy(c)  # one common zero-point instead of the grouped ones: the variant the JIT accepts
        v.wei_zp = Quant(np.array([8], dtype=np.int32), dt.S32, 0)
        _, impl, tmin, tavg = B.run_reference(v, weights_any=True, iters=3)
        out["c2_variant_common_zero_point_m1"] = {"impl": impl, "ms": tavg,
                                                  "GB/s": c.algorithmic_bytes() / (tavg * 1e-3) / 1e9,
                                                  "sample": "1x4096x14336, grouped scales, one s32 zero-point, 3 executions, mean"}
    except Exception as ex:
        out["c2_error"] = repr(ex)
    try:
        c = W.config3(512, 512, 512)
        _, impl, tmin, tavg = B.run_reference(c, weights_any=True, iters=1)
        out["c3_fp8"] = {"impl": impl, "ms": tavg, "TFLOPS": c.ops / (tavg * 1e-3) / 1e12,
                         "sample": "512^3 of the 8192^3 problem, one execution"}
    except Exception as ex:
        out["c3_error"] = repr(ex)
    try:
        c = W.config0()
        _, impl, tmin, tavg = B.run_reference(c, weights_any=True, iters=50)
        out["c0_int8_128x1024x1024"] = {"impl": impl, "us": tavg * 1e3, "sample": "the full problem, 50 executions, mean"}
    except Exception as ex:
        out["c0_error"] = repr(ex)
    return out


def run_c4_sharded(W, torch, dist, rank, world, local, reps=5):
    """The large configuration (16384 x 8192 x 28672, s8 -> bf16) over the ranks, three ways:

      m_split                   rows of src / dst over the ranks, weights replicated, no exchange;
      n_split_nccl_all_gather   columns of the weights over the ranks, NCCL all-gather of the dst
                                slices plus a layout kernel;
      n_split_epilogue_stores   the same split with the matmul's epilogue storing its tiles into
                                every GPU's copy of dst.

    Each leg is device-timed (max over ranks) and then executed once more on a destination filled
    with a sentinel byte and compared, element for element, with what the unsharded primitive
    computes on the same GPU (a sharded run must reproduce it exactly); about a thousand elements
    per rank are checked against the CPU oracle as well.  The counts are summed over ranks."""
    from onednn_b200 import multi_gpu
    from oracle import binding as B
    out = {}
    try:
        case = W.config4()
        full = multi_gpu.unsharded_on_this_gpu(case, local)     # (M, N * 2) bytes: the yardstick
        elem = 2
        # oracle sample: a 32 x 32 lattice, shifted per rank
        ms_, ns_ = case.M // 32, case.N // 32
        m0, n0 = (7 * rank) % ms_, (11 * rank) % ns_
        want = B.run_oracle(case, tanh_mode=1, exact_acc=1, m_step=ms_, n_step=ns_, m0=m0, n0=n0)
        want_s = torch.from_numpy(want[m0::ms_, n0::ns_].copy().view("uint8")).cuda()

        def oracle_bad(dst_full):
            got = dst_full.view(case.M, case.N, elem)[m0::ms_, n0::ns_].reshape(want_s.shape)
            return int((got != want_s).view(got.shape[0], -1, elem).any(dim=2).sum().item())

        def timed(op, extra=None):
            for _ in range(2):
                op.execute()
            torch.cuda.synchronize()
            dist.barrier()
            a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
            for _ in range(reps):
                op.execute()
            b.record()
            if extra is not None:
                for _ in range(reps):
                    extra()
            c.record()
            c.synchronize()
            t = torch.tensor([a.elapsed_time(b) / reps, b.elapsed_time(c) / reps], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return (float(x) for x in t.tolist())

        def summed(*vals):
            t = torch.tensor(list(vals), device="cuda", dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
            return [int(x) for x in t.tolist()]

        # ---- M-split ----
        try:
            op = multi_gpu.MSplitMatmul(case, rank, world, local)
            ms, _ = timed(op)
            op.dst.fill_(multi_gpu.SENTINEL)
            op.execute()
            torch.cuda.synchronize()
            bad = multi_gpu.count_mismatched_elements(op.dst, full[op.rows], elem)
            rows_here = [m for m in range(m0, case.M, ms_) if op.rows.start <= m < op.rows.stop]
            got = op.dst.view(op.local.M, case.N, elem)[[m - op.rows.start for m in rows_here]][:, n0::ns_]
            ref = want_s.view(-1, want_s.shape[1] // elem, elem)[[(m - m0) // ms_ for m in rows_here]]
            obad = int((got != ref).any(dim=2).sum().item()) if rows_here else 0
            bad, obad, nel, osamp = summed(bad, obad, op.local.M * case.N, len(rows_here) * ref.shape[1] if rows_here else 0)
            out["m_split"] = {"impl": op.impl, "ranks": world, "ms": ms, "TOPS": case.ops / (ms * 1e-3) / 1e12,
                              "rows_per_rank": op.local.M, "bytes_exchanged": 0,
                              "mismatches_vs_unsharded_primitive": bad, "elements_compared": nel,
                              "mismatches_vs_cpu_oracle": obad, "oracle_samples": osamp,
                              "how": "each rank its rows through the ordinary primitive, replicated packed weights; max over ranks"}
            del op
        except Exception as ex:
            out["m_split"] = {"error": repr(ex)}
        torch.cuda.empty_cache()
        # ---- N-split, two ways ----
        for key, mode in (("n_split_nccl_all_gather", "nccl"), ("n_split_epilogue_stores", "p2p")):
            try:
                op = multi_gpu.NSplitMatmul(case, rank, world, local, mode=mode)
                ms, ms_mm = timed(op, lambda: op.plan.prim.execute(op.strm, op.args))
                torch.cuda.synchronize()
                dist.barrier()
                op.dst.fill_(multi_gpu.SENTINEL)
                torch.cuda.synchronize()
                dist.barrier()      # nobody stores into a copy its owner is still filling
                op.execute()
                torch.cuda.synchronize()
                dist.barrier()
                bad = multi_gpu.count_mismatched_elements(op.dst, full, elem)
                obad = oracle_bad(op.dst)
                bad, obad, nel, osamp = summed(bad, obad, case.M * case.N, want_s.shape[0] * want_s.shape[1] // elem)
                nsl = case.N // world
                out[key] = {"impl": op.impl, "ranks": world, "ms": ms, "TOPS": case.ops / (ms * 1e-3) / 1e12,
                            "ms_matmul_slice_only": ms_mm, "bytes_received_per_rank": (world - 1) * case.M * nsl * 2,
                            "mismatches_vs_unsharded_primitive": bad, "elements_compared": nel,
                            "mismatches_vs_cpu_oracle": obad, "oracle_samples": osamp,
                            "how": ("slice matmul -> ncclAllGather of [M][N/g] bf16 slices -> layout kernel" if mode == "nccl" else
                                    "slice matmul whose epilogue stores each tile into every GPU's copy of dst -> barrier")
                            + "; max over ranks"}
                del op
            except Exception as ex:
                out[key] = {"error": repr(ex)}
            torch.cuda.empty_cache()
    except Exception as ex:
        out["error"] = repr(ex)
    return out


def run_extras(api, W, dt, eng, strm, tstream, torch, np, peaks):
    """Secondary configurations of the same path.

    These kernels run for microseconds, less than a host-side launch takes, so each is
    captured into a CUDA graph and the replay is timed: the launches then run back to back
    on the device.  To keep the operands out of L2 the graph cycles over several independent
    copies of the weights whose total size exceeds the cache (the decode GEMV is judged on
    HBM bandwidth, and its 28 MiB of weights would otherwise stay cache-resident)."""
    out = {}
    gs = torch.cuda.Stream()
    gstrm = api.Stream(eng, cuda_stream=gs.cuda_stream)

    def graph_time(plans, reps=5):
        for pl in plans:
            pl.execute()
        gstrm.wait()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=gs):
            for pl in plans:
                pl.execute()
        g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            b.synchronize()
            ts.append(a.elapsed_time(b) / len(plans))
        ts.sort()
        return ts[len(ts) // 2], ts[0]

    try:
        for m in (1, 16, 128):
            c = W.config2(m)
            copies = 9  # 9 x 29.4 MB of packed weights = 264 MB > L2
            plans = [api.CasePlan(c, eng, gstrm, weights="any") for _ in range(copies)]
            med, best = graph_time(plans)
            nbytes = c.algorithmic_bytes()
            gbs = nbytes / (med * 1e-3) / 1e9
            out["c2_wc_u4_m%d" % m] = {
                "impl": plans[0].impl, "us": med * 1e3, "us_min": best * 1e3, "algorithmic_bytes": nbytes, "GB/s": gbs,
                "frac_of_hbm_%s" % peaks["source"]: gbs / peaks["hbm"], "frac_of_8TBs_nominal": gbs / 8000.0,
                "GOPS": c.ops / (med * 1e-3) / 1e9,
                "timing": "CUDA graph of %d executions over %d weight copies (L2-cold), median of 5 replays" % (copies, copies)}
            del plans
    except Exception as ex:
        out["c2_error"] = repr(ex)
    try:
        c = W.config0()
        plans = [api.CasePlan(c, eng, gstrm, weights="any") for _ in range(4)]
        med, best = graph_time(plans)
        out["c0_int8_128x1024x1024"] = {"impl": plans[0].impl, "us": med * 1e3, "us_min": best * 1e3,
                                        "timing": "CUDA graph of 4 executions, median of 5 replays"}
        del plans
    except Exception as ex:
        out["c0_error"] = repr(ex)
    try:
        c = W.config3()
        plans = [api.CasePlan(c, eng, gstrm, weights="any")]
        med, best = graph_time(plans, reps=3)
        out["c3_fp8_8192"] = {"impl": plans[0].impl, "ms": med, "TFLOPS": c.ops / (med * 1e-3) / 1e12,
                              "frac_of_2x_bf16_%s" % peaks["source"]: c.ops / (med * 1e-3) / 1e12 / (2 * peaks["bf16"])}
        del plans
    except Exception as ex:
        out["c3_error"] = repr(ex)
    try:
        c = W.config4()
        plans = [api.CasePlan(c, eng, gstrm, weights="any")]
        med, best = graph_time(plans, reps=3)
        out["c4_int8_16384x8192x28672_1gpu"] = {"impl": plans[0].impl, "ms": med, "TOPS": c.ops / (med * 1e-3) / 1e12,
                                                "frac_of_2x_bf16_%s" % peaks["source"]: c.ops / (med * 1e-3) / 1e12 / (2 * peaks["bf16"])}
        del plans
    except Exception as ex:
        out["c4_error"] = repr(ex)
    try:
        # the caller in front of the int8 matmul: activations quantised on the device (dnnl_reorder with scales)
        for name, src_dt, per_row in (("reorder_quant_f32_s8_8192", dt.F32, False), ("reorder_quant_bf16_s8_per_row_8192", dt.BF16, True)):
            c = W.quantize_case(8192, 8192, src_dt, dt.S8, per_row=per_row)
            plans = [api.ReorderPlan(c, eng, gstrm) for _ in range(3)]  # 3 x (268 or 134) + 67 MB > L2
            med, best = graph_time(plans)
            nbytes = c.rows * c.cols * (np.dtype(dt.RAW[src_dt]).itemsize + 1)
            gbs = nbytes / (med * 1e-3) / 1e9
            out[name] = {"impl": plans[0].impl, "us": med * 1e3, "us_min": best * 1e3, "algorithmic_bytes": nbytes, "GB/s": gbs,
                         "frac_of_hbm_%s" % peaks["source"]: gbs / peaks["hbm"],
                         "timing": "CUDA graph of 3 executions over 3 buffer sets, median of 5 replays"}
            del plans
    except Exception as ex:
        out["reorder_quant_error"] = repr(ex)
    return out


if __name__ == "__main__":
    sys.exit(main())
