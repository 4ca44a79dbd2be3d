#!/usr/bin/env python
"""Benchmark of the 2D-CrossScan selective scan: forward + backward scanned
elements per second (B*K*D*H*W*N per pass) and the fraction of the HBM roofline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--config NAME]

One process per GPU (torchrun for N > 1).  A step is one forward plus one
backward of the operator over one synthetic batch; with N > 1 every rank owns
its own batch of the configured size (weak scaling, the headline `value`) and
the step ends with the single all-reduce of the per-channel parameter
gradients.  The same line carries, as sub-records, the split the benchmark
configuration itself names - the configured batch sharded over the N ranks
("strong") with a check that the all-reduced parameter gradients of the shards
equal the single-GPU result - and the four-corner operator on the
segmentation-scale configuration ("cross").  Rank 0 prints one JSON line.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (os.path.join(ROOT, "official-cross-scan_b200"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)

METRIC = "fwd+bwd scanned elems/s (B*K*D*H*W*N)"
UNIT = "elements/s"
DEFAULT_CONFIG = "c2_vmamba_t_stage1"


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def load_traffic(workload):
    """DRAM bytes per backward launch from the committed ncu capture, if any."""
    try:
        with open(os.path.join(ROOT, "profiles", "traffic.json")) as f:
            return json.load(f).get(workload)
    except Exception:
        return None


class ClockSampler:
    """Samples SM clocks and throttle reasons while a region runs: NVML read calls from a thread every
    20 ms (a timed region of a fraction of a second still gets samples, on every rank), and
    nvidia-smi in a loop when the NVML binding is missing.  Reads only; nothing is set."""
    Q = ("index,clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index, uuid=None):
        self.index, self.uuid, self.rows, self.proc, self.stop = index, uuid, [], None, threading.Event()
        self.source = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        if self.uuid:
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{self.uuid}")
            except Exception:
                pass
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def __enter__(self):
        try:
            self.nv, self.h = self._nvml_handle()
            self.mx = self.nv.nvmlDeviceGetMaxClockInfo(self.h, self.nv.NVML_CLOCK_SM)
            self.source = "nvml"
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.source = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            self.source = "nvidia-smi"
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _poll(self):
        while not self.stop.is_set():
            try:
                mhz = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
                bits = self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                self.rows.append([self.index, mhz, self.mx] + ["Active" if bits & b else "Not Active" for _, b in self.BITS])
            except Exception:
                pass
            self.stop.wait(0.02)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def __exit__(self, *a):
        if self.source == "nvml":
            self.stop.set()
            self.thread.join(timeout=2)
        elif self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        for r in self.rows:
            try:
                mhz.append(int(r[1])); mx = max(mx, int(r[2]))
            except Exception:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if str(v).lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz), "source": self.source}


def cpu_port(shape, sample_batch, steps=1):
    """Times the CPU restatement (float32, all host threads) on `sample_batch` samples."""
    import torch
    from cs2d.synthetic import make_inputs, elements
    from oracle import cs2d_oracle as O
    import numpy as np
    B, K, D, N, H, W = shape
    inp = make_inputs(sample_batch, K, D, N, H, W, dtype=torch.float32, seed=0)
    a = [inp[k].numpy() if inp[k] is not None else None for k in ("u", "delta", "A", "B", "C", "D", "delta_bias")]
    dout = inp["dout"].numpy()
    O.fwd(*[x[:1] if i in (0, 1, 3, 4) else x for i, x in enumerate(a)], True, dtype=np.float32)  # build + warm
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.fwd(*a, True, dtype=np.float32)
        O.bwd(*a, dout, True, dtype=np.float32)
        times.append(time.perf_counter() - t0)
    el = elements(sample_batch, K, D, N, H, W)
    return el / (sum(times) / len(times)), O.max_threads(), sum(times) / len(times)


def cpu_sample_size(shape, budget_s):
    """Samples of the workload the CPU port gets through in about `budget_s` seconds."""
    from cs2d.synthetic import elements
    rate, _, _ = cpu_port(shape, 1, 1)
    per_sample = elements(1, *shape[1:])
    return int(max(1, min(shape[0], budget_s * rate / per_sample)))


def config_dict(name, shape, dtype, world):
    return {"workload": name, "shape_BKDNHW": list(shape), "io_dtype": str(dtype)[6:], "per_gpu_batch": shape[0],
            "l2": "inputs larger than L2 (no flush needed)",
            "sharding": "batch per rank, one all-reduce of the parameter gradients" if world > 1 else "none"}


def reference_cuda_side_record(name):
    """A labelled side record, outside every timed region: the reference's own CUDA extension (the
    kernels this library replaces) timed on the same configuration with the state dimension capped
    at 12, in a subprocess of its own.  Absent build or GPU -> a one-line reason instead."""
    script = os.path.join(ROOT, "oracle", "ref_cuda_timing.py")
    if not os.path.exists(os.path.join(ROOT, "oracle", "_ref", "selective_nd_scan_cuda_oflex.so")):
        return {"unavailable": "the reference extension is not built (make -C oracle ref)"}
    try:
        out = subprocess.run([sys.executable, script, name], capture_output=True, text=True, timeout=300)
        if out.returncode != 0:
            return {"unavailable": (out.stderr.strip().splitlines() or ["failed"])[-1][:200]}
        return json.loads(out.stdout.strip().splitlines()[-1])
    except Exception as e:  # no GPU, time-out, ...
        return {"unavailable": str(e)[:200]}


def run_reference(args, shape, name, dtype):
    """The reference ships no CPU implementation of this operator (its only
    implementation is the CUDA extension), so the reference arm times the CPU
    restatement of its algorithm on the host cores: one rank's whole batch per
    step when that takes a few seconds, else a bounded sample of it."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from cs2d.synthetic import elements
    B, K, D, N, H, W = shape
    rate = cpu_port(shape, 1, 1)[0]
    for _ in range(args.warmup):
        cpu_port(shape, 1, 1)
    full_s = elements(*shape) / rate
    sample = B if full_s <= 8.0 else int(max(1, min(B, 8.0 * rate / elements(1, *shape[1:]))))
    val, cores, sec = cpu_port(shape, sample, max(1, args.steps))
    what = f"{sample} of {B} samples of {name} per step, float32, OpenMP"
    print(json.dumps({
        "reference_cuda_extension": reference_cuda_side_record(name),
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(name, shape, dtype, args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": what},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def measure_cross(name, steps, warmup, dev, world, rank, timed, batch=0):
    """The four-corner operator (directions, shared u / dy and the weighted merge inside the kernels),
    forward + backward on resident inputs, with the all-reduce of the parameter gradients in the
    timed region.  Algorithmic bytes of this operator: u, y, dy, du once per channel, delta and ddelta
    per direction and channel, B, C, dB, dC per direction and state."""
    import torch
    import cs2d
    from cs2d import cross, parallel
    from cs2d.synthetic import CONFIGS, make_inputs
    B, K, D, N, H, W, dtype = CONFIGS[name]
    B = batch or B
    s = 4 if dtype == torch.float32 else 2
    host = make_inputs(B, K, D, N, H, W, dtype=dtype, seed=rank)
    gen = torch.Generator().manual_seed(100 + rank)
    u0 = host["u"][:, :D].to(dev)                      # direction 0 of the synthetic input is the image itself
    dy = torch.randn(B, D, H, W, generator=gen).to(dtype).to(dev)
    w = torch.full((K, D), 1.0 / K, device=dev)
    t = {k: (v.to(dev) if v is not None else None) for k, v in host.items() if k not in ("u", "dout")}
    del host

    def step():
        y, saved = cross._dir_forward(u0, t["delta"], t["A"], t["B"], t["C"], w, t["D"], t["delta_bias"], True)
        g = cross._dir_backward(u0, t["delta"], t["A"], t["B"], t["C"], w, t["D"], t["delta_bias"], dy, saved, True)
        if world > 1:
            flat = torch.cat([g[2].reshape(-1), g[5].reshape(-1), g[6], g[7]])
            parallel.allreduce_param_grads(flat)
        return y, g

    for _ in range(warmup):
        step()
    n0 = cs2d.launch_count()
    ms = timed(step, steps) / steps
    launches = cs2d.launch_count() - n0
    assert cs2d.device_status() == 0, "a kernel gave up on a bounded wait"
    el = B * K * D * N * H * W * world
    nbytes = B * H * W * s * (5 * D + 3 * K * D + 6 * K * N)
    peak, peak_kind = load_peaks()
    achieved = nbytes / (ms * 1e-3) / 1e9

    e2e = None
    if world == 1:   # one GPU only: with N ranks the host link is shared and the figure says nothing about the operator
        # end to end: u, delta, B, C, dy from pinned host memory, every output back to it, inside the timed
        # region (cs2d.CrossHostPipeline); u and dy cross the bus once for all K directions
        hx = {"u": u0.cpu().pin_memory(), "delta": t["delta"].cpu().pin_memory(), "B": t["B"].cpu().pin_memory(),
              "C": t["C"].cpu().pin_memory(), "dy": dy.cpu().pin_memory()}
        params = {"A": t["A"], "D": t["D"], "delta_bias": t["delta_bias"], "w": w}
        del u0, dy
        for k in ("delta", "B", "C"):
            t.pop(k)
        torch.cuda.empty_cache()
        hout = cs2d.alloc_cross_host_outputs(hx["u"], hx["delta"], hx["B"], params["A"], params["D"] is not None,
                                             params["delta_bias"] is not None)
        pipe = cs2d.CrossHostPipeline(hx, params, True)
        for _ in range(2):
            pipe.run(hx, hout, allreduce=world > 1)
        torch.cuda.synchronize()
        e2e_steps = max(2, min(steps, 3))
        e2e_ms = timed(lambda: pipe.run(hx, hout, allreduce=world > 1), e2e_steps) / e2e_steps
        assert cs2d.device_status() == 0, "a kernel gave up on a bounded wait"
        h2d = sum(v.numel() * v.element_size() for v in hx.values())
        d2h = sum(v.numel() * v.element_size() for v in hout.values())
        e2e = {"value": el / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "chunk": pipe.chunk}
        del pipe, hx, hout
        torch.cuda.empty_cache()
    return {"value": el / (ms * 1e-3), "unit": UNIT, "ms_per_step": ms, "steps": steps, "scaling": "weak", "e2e": e2e,
            "config": {"workload": name, "op": "four-corner operator with fusion weights, all-reduce of the parameter "
                                               "gradients in the timed region" if world > 1 else
                                               "four-corner operator with fusion weights",
                       "shape_BKDNHW": [B, K, D, N, H, W], "io_dtype": str(dtype)[6:], "per_gpu_batch": B},
            "roofline": {"bound": "hbm", "kernel": "fwd_kernel + bwd_kernel", "achieved": achieved, "peak": peak,
                         "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                         "algorithmic_bytes": nbytes},
            "gpu_launches": launches}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default=DEFAULT_CONFIG)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cross", action="store_true", help="skip the four-corner operator sub-record")
    ap.add_argument("--e2e-chunks", type=int, default=0,
                    help="batch chunks of the host-buffer pipeline (0: chosen by the library, about 32 MB each)")
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (profiling captures only)")
    ap.add_argument("--op", choices=("scan", "cross"), default="scan",
                    help="scan: the drop-in fwd/bwd operator (the headline); cross: the four-corner operator with "
                         "fusion weights alone, timed on resident inputs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference" or int(os.environ.get("WORLD_SIZE", "1")) == 1:
        # the CPU arm uses every host core; torchrun exports OMP_NUM_THREADS=1, which must be undone
        # before any OpenMP runtime is loaded
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)

    from cs2d.synthetic import CONFIGS, algorithmic_bytes, elements, make_inputs
    B, K, D, N, H, W, dtype = CONFIGS[args.config]
    if args.batch > 0:
        B = args.batch
    shape = (B, K, D, N, H, W)
    if args.impl == "reference":
        return run_reference(args, shape, args.config, dtype)

    import torch
    import torch.distributed as dist
    import cs2d
    from cs2d import parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    # Libraries (NCCL prints its version banner at communicator creation) must not write into
    # the one-JSON-line stdout: route fd 1 to stderr until the result is printed.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    s = 4 if dtype == torch.float32 else 2

    def timed(fn, n):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.barrier()
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    def emit(line):
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
        if rank == 0:
            print(json.dumps(line))
        if world > 1:
            dist.destroy_process_group()

    gpu_index = torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ else local
    gpu_uuid = str(torch.cuda.get_device_properties(local).uuid)
    if args.op == "cross":
        with ClockSampler(gpu_index, gpu_uuid) as clk:
            rec = measure_cross(args.config, args.steps, args.warmup, dev, world, rank, timed, args.batch)
        rec.update({"metric": METRIC, "n_gpus": world, "warmup": args.warmup, "higher_is_better": True, "vs_baseline": None,
                    "dtype": "f32", "data": "synthetic", "cpu_baseline": None, "e2e": None, "clocks": clk.summary()})
        return emit(rec)

    # ---- inputs: generated on the host, pinned, then made resident -----------------
    host = make_inputs(B, K, D, N, H, W, dtype=dtype, seed=rank)
    host = {k: (v.pin_memory() if v is not None else None) for k, v in host.items()}
    d = {k: (v.to(dev, non_blocking=True) if v is not None else None) for k, v in host.items()}
    torch.cuda.synchronize()

    # ---- value: inputs resident in HBM, every rank its own batch of B (weak scaling) ------------
    # forward, backward, the zero fills, the all-reduce and the dB/dC cast, on preallocated buffers
    rs = parallel.ResidentStep(d, True)
    for _ in range(args.warmup):
        rs.run(d)
    n0 = cs2d.launch_count()
    with ClockSampler(gpu_index, gpu_uuid) as clk:
        ms = timed(lambda: rs.run(d), args.steps)
    launches = cs2d.launch_count() - n0
    assert cs2d.device_status() == 0, "a kernel gave up on a bounded wait"
    el_step = elements(B, K, D, N, H, W) * world
    value = el_step / (ms / args.steps * 1e-3)

    # ---- roofline of the dominant kernel (backward), timed alone on its stream ---------
    L = cs2d._lib.lib()
    vp = lambda t: ctypes.c_void_p(t.data_ptr()) if t is not None else None
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = rs.p

    def bwd_kernel():
        p.out_dtype = cs2d.ops._DT[d["dout"].dtype]
        rc = L.cs2d_bwd(ctypes.byref(p), vp(d["dout"]), d["dout"].stride(0), d["dout"].stride(1), d["dout"].stride(2),
                        vp(rs.saved), vp(rs.scratch), vp(rs.du), vp(rs.ddelta), vp(rs._part("dA")), vp(rs.dB32), vp(rs.dC32),
                        vp(rs._part("dD")), vp(rs._part("ddelta_bias")), None, stream)
        assert rc == 0, cs2d._lib.last_error()

    def fwd_kernel():
        p.out_dtype = cs2d.ops._DT[rs.out.dtype]
        rc = L.cs2d_fwd(ctypes.byref(p), vp(rs.out), rs.out.stride(0), rs.out.stride(1), rs.out.stride(2), vp(rs.saved),
                        stream)
        assert rc == 0, cs2d._lib.last_error()

    for _ in range(3):
        fwd_kernel(); bwd_kernel()
    fwd_ms = timed(fwd_kernel, args.steps) / args.steps
    bwd_ms = timed(bwd_kernel, args.steps) / args.steps
    peak, peak_kind = load_peaks()
    bwd_bytes = algorithmic_bytes(B, K, D, N, H, W, s, fwd=False, bwd=True)
    fwd_bytes = algorithmic_bytes(B, K, D, N, H, W, s, fwd=True, bwd=False)
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "backward kernel", "achieved": achieved, "peak": peak, "peak_kind": peak_kind,
                "unit": "GB/s", "frac": achieved / peak, "traffic": load_traffic(args.config),
                "algorithmic_bytes": bwd_bytes, "launch_ms": bwd_ms,
                "fwd_kernel": {"launch_ms": fwd_ms, "achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                               "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak},
                "fwd_plus_bwd_frac": (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak}

    # ---- the split the configuration names: its batch sharded over the ranks (strong scaling) ------
    # every rank generates the same global batch (seed 0) and keeps its shard; before timing, the
    # all-reduced parameter gradients of the shards are compared with one rank's full-batch result
    strong = {"value": value, "unit": UNIT, "ms_per_step": ms / args.steps, "per_gpu_batch": B, "global_batch": B,
              "note": "one GPU: the same run as the headline"}
    if world > 1 and B >= world:
        del rs
        glob = make_inputs(B, K, D, N, H, W, dtype=dtype, seed=0)
        lo, hi = parallel.shard_bounds(B, rank, world)
        big = ("u", "delta", "B", "C", "dout")
        sh = {k: (v[lo:hi].contiguous().to(dev) if k in big else (v.to(dev) if v is not None else None))
              for k, v in glob.items()}
        rss = parallel.ResidentStep(sh, True)
        rss.run(sh)
        torch.cuda.synchronize()
        check = None
        if rank == 0:   # the whole batch on one GPU, no collective
            full = {k: (v.to(dev) if v is not None else None) for k, v in glob.items()}
            ref = parallel.ResidentStep(full, True).run(full, allreduce=False).flat.double()
            got = rss.flat.double()
            rtol, atol = 1e-4, 1e-5
            ratio = float(((got - ref).abs() / (atol + rtol * ref.abs())).max())
            # two fp32 summation orders of ~1e5 terms each: the reduced-sum tolerance is ten times the element one
            check = {"tensors": "dA | dD | ddelta_bias, all-reduced over the shards vs the full batch on one GPU",
                     "worst_ratio": ratio, "rtol": rtol, "atol": atol, "allowed_ratio": 10.0, "passed": ratio <= 10.0}
            assert check["passed"], f"all-reduced parameter gradients differ from the single-GPU result: {check}"
            del full, ref
        del glob
        for _ in range(args.warmup):
            rss.run(sh)
        sms = timed(lambda: rss.run(sh), args.steps) / args.steps
        assert cs2d.device_status() == 0, "a kernel gave up on a bounded wait"
        strong = {"value": elements(B, K, D, N, H, W) / (sms * 1e-3), "unit": UNIT, "ms_per_step": sms,
                  "per_gpu_batch": hi - lo, "global_batch": B, "scaling": "strong", "cross_rank_check": check}
        del rss, sh
        rs = None

    # ---- end to end: host buffers in, host buffers out, copies inside the timed region ----
    # cs2d.fwd_bwd_from_host is the call a user with host-resident tensors makes: it pipelines
    # batch chunks over copy-in / kernel / copy-out streams.
    del rs
    torch.cuda.empty_cache()
    big = ("u", "delta", "B", "C", "dout")
    h2d = sum(host[k].numel() * host[k].element_size() for k in big)
    hout = cs2d.alloc_host_outputs(host["u"], host["B"], d["A"], True, True)
    d2h = sum(t.numel() * t.element_size() for t in hout.values())
    params = {"A": d["A"], "D": d["D"], "delta_bias": d["delta_bias"]}

    def e2e_step():
        cs2d.fwd_bwd_from_host(host, params, hout, True, False, chunks=args.e2e_chunks or None, allreduce=world > 1)

    for _ in range(3):   # the chunk shapes are new to the allocator and the kernels' attribute caches
        e2e_step()
    torch.cuda.synchronize()
    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms = timed(e2e_step, e2e_steps) / e2e_steps
    assert cs2d.device_status() == 0, "a kernel gave up on a bounded wait"
    e2e = {"value": el_step / (e2e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
           "ms_per_step": e2e_ms, "chunks": args.e2e_chunks or "auto (about 32 MB of input each)"}
    del hout, host, d, params
    cs2d.host._cache.clear()
    torch.cuda.empty_cache()

    # ---- the four-corner operator on the segmentation-scale configuration (sub-record) -----------
    cross_rec = None
    if not args.no_cross and args.config == DEFAULT_CONFIG and args.batch == 0:
        cross_rec = measure_cross("c5_segmentation", max(2, min(args.steps, 5)), 3, dev, world, rank, timed)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample = cpu_sample_size(shape, budget_s=15.0)
        val, cores, sec = cpu_port(shape, sample, 1)
        cpu = {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"{sample} of {B} samples of {args.config}, float32, OpenMP, {sec:.1f} s"}

    emit({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_dict(args.config, shape, dtype, world),
        "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clk.summary(),
        "strong": strong, "cross": cross_rec,
    })


if __name__ == "__main__":
    main()
