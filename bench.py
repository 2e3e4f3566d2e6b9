#!/usr/bin/env python
"""Benchmark of the DIA sparse hot path on B200.

Default workload (``--case rbm_cfg4``): the sparse-RBM CD-1 step of BASELINE config 4 - visible and
hidden layers of 65536 units, a banded DIA weight matrix with 1024 diagonals (row_fact 1), global
batch 8192 whose columns are sharded over the ranks (strong scaling); per step: prod up, prod down
(transposed), prod up again for the negative phase, two densedense_to_dia, four bias reductions,
the element-wise glue, and with more than one rank an NCCL all-reduce of the gradient diagonals
and bias gradients.  Inputs are synthetic with the configuration's shapes and distributions.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line (rank 0).  Launched under
``torch.distributed.run`` for N > 1.  ``--impl reference`` times the CPU oracle (the restatement of
CUV's host code) on all host cores on a bounded batch slice of the same workload.

Other cases (single routines, used for profiling and for the per-configuration table):
``--case prod_n|prod_t|dd2dia|reduce|glue|glue_sum|update`` on the band shape given by --units/--num-dia/--batch, and
``--case cfg0|cfg1|cfg2|rbm_cfg3`` for the other BASELINE configurations, ``--case spmv_speed_n|spmv_speed_t|dd2dia_speed``
for the reference's own speed fixtures (convolution-pattern matrices), ``--case wide_n|wide_dd`` for scattered
diagonals that no shared-memory window covers (the plain kernels).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "DIA prod / densedense_to_dia effective HBM GB/s and % of roofline at 1/2/4/8 B200"
CASES = {
    "rbm_cfg4": dict(units=65536, num_dia=1024, batch=8192),
    "rbm_cfg3": dict(units=16384, num_dia=512, batch=1024),
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU through NVML on a thread while the timed
    region runs (every ~10 ms); falls back to one nvidia-smi query if NVML is not importable."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, index):
        self.index, self.samples, self.thread, self.stop_flag = index, [], None, False
        self.handle = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index(index))
        except Exception:
            self.nv = None

    @staticmethod
    def _physical_index(index):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v for v in vis.split(",") if v.strip() != ""]
            if index < len(ids) and ids[index].strip().isdigit():
                return int(ids[index])
        return index

    def _sample(self):
        nv, h = self.nv, self.handle
        sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
        try:
            mask = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
        except Exception:
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
        try:
            power = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
        except Exception:
            power = 0.0
        self.samples.append((sm, mask, power))

    def _loop(self):
        while not self.stop_flag:
            try:
                self._sample()
            except Exception:
                break
            time.sleep(0.01)

    def start(self):
        if self.handle is None:
            return
        import threading
        self.stop_flag = False
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self):
        if self.handle is None:
            return self._smi_once()
        self.stop_flag = True
        self.thread.join(timeout=2)
        if not self.samples:
            try:
                self._sample()
            except Exception:
                return self._smi_once()
        smax = self.nv.nvmlDeviceGetMaxClockInfo(self.handle, self.nv.NVML_CLOCK_SM)
        reasons = set()
        for _, mask, _ in self.samples:
            for bit, name in self.REASONS.items():
                if mask & bit:
                    reasons.add(name)
        powers = [p for _, _, p in self.samples]
        cut = statistics.median(powers)
        loaded = [s for s, _, p in self.samples if p >= cut] or [s for s, _, _ in self.samples]
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(self.samples), "power_w_max": max(powers)}

    def _smi_once(self):
        try:
            out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=clocks.sm,clocks.max.sm",
                                  "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=10).stdout
            a, b = [float(x) for x in out.strip().split(",")[:2]]
            return {"sm_mhz": a, "sm_max_mhz": b, "reasons": ["sampled once after the run (NVML unavailable)"]}
        except Exception:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["clock sampling unavailable"]}


def fp32_peak_tflops(fused=True):
    """FP32 issue ceiling of the current device in TFLOP/s (a multiply-add = 2 flops), measured by the bench-side
    library ``libbench_fp32_peak.so`` (bench_fp32_peak.cu; not part of the product library): a register-resident
    loop of fused multiply-adds, or of separate multiplies and adds (the EXACT arithmetic of prod)."""
    import ctypes
    lib = os.path.join(ROOT, "libbench_fp32_peak.so")
    if not os.path.exists(lib):
        subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "--fmad=false", "-shared",
                               "-Xcompiler", "-fPIC", os.path.join(ROOT, "bench_fp32_peak.cu"), "-o", lib])
    L = ctypes.CDLL(lib)
    out = ctypes.c_float()
    rc = L.bench_fp32_peak_tflops(1 if fused else 0, ctypes.byref(out))
    if rc != 0:
        raise RuntimeError("bench_fp32_peak_tflops failed with CUDA error %d" % rc)
    return float(out.value)


def band_offsets(nd):
    import numpy as np
    return np.arange(-(nd // 2), nd - nd // 2, dtype=np.int32)


def event_ms(pairs):
    return [a.elapsed_time(b) for a, b in pairs]


# ---------------------------------------------------------------------------------------------------
# CPU arm: the oracle on the host cores, on a bounded batch slice
# ---------------------------------------------------------------------------------------------------

def cpu_rbm(units, nd, batch, sample_cols, steps, warmup):
    """Times the CPU oracle's CD-1 step on ``sample_cols`` batch columns of the workload, with all host
    threads; returns (seconds per step on the slice, threads)."""
    from oracle import rbm_oracle
    threads = os.cpu_count() or 1
    W, V0, U_h, U_v = rbm_oracle.make_inputs(1004, units, units, band_offsets(nd), sample_cols, nthreads=threads)
    ts = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        rbm_oracle.cd1_step(W, V0, U_h, U_v, batch_global=batch, nthreads=threads)
        if i >= warmup:
            ts.append(time.perf_counter() - t0)
    return sum(ts) / len(ts), threads, W.nnz()


def run_reference(args, cfg):
    from cuv_b200 import rbm
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    units, nd, batch = cfg["units"], cfg["num_dia"], cfg["batch"]
    # a first, small slice tells how long a column takes; the timed slice is then sized so that all steps together
    # stay near two minutes of host time (at most --cpu-sample-cols columns)
    probe = min(batch, 64)
    t_probe, _, _ = cpu_rbm(units, nd, batch, probe, 1, 0)
    steps, warm = max(1, args.steps), max(0, min(args.warmup, 1))
    budget_cols = int(120.0 / max(t_probe / probe, 1e-9) / (steps + warm))
    sample = max(probe, min(batch, args.cpu_sample_cols, budget_cols // 64 * 64))
    t, threads, nnz = cpu_rbm(units, nd, batch, sample, steps, warm)
    work = rbm.algorithmic_work(units, units, nd, nnz, batch)
    t_full = t * (batch / float(sample))
    value = work["bytes"] / t_full / 1e9
    sample_txt = ("CD-1 step of the CPU oracle on the first %d of %d batch columns (same matrix), %d threads; "
                  "time scaled linearly to the full batch" % (sample, batch, threads))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_full * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.case, cfg), "units": units, "num_dia": nd, "row_fact": 1,
                   "global_batch": batch, "l2": "inputs larger than L2"},
        "gflops": work["flops"] / t_full / 1e9,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample_txt},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def pin_to_gpu_numa_node(torch, local):
    """Restricts this process to the CPUs next to its GPU (the PCI device's local_cpulist in sysfs), so that the
    pinned host buffers it allocates and fills afterwards land in that NUMA node's memory: with several ranks on
    one host, input copies that cross the socket interconnect share its bandwidth.  Returns the CPU list used, or
    None if the topology cannot be read (then nothing is changed)."""
    try:
        prop = torch.cuda.get_device_properties(local)
        bdf = "%04x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
        with open("/sys/bus/pci/devices/%s/local_cpulist" % bdf) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return text
    except Exception:
        pass
    return None


def workload_name(case, cfg):
    if case == "rbm_cfg4":
        return ("BASELINE config 4: sparse RBM CD-1 step, visible=hidden=%d, DIA weights num_dia=%d row_fact=1 "
                "band centred on 0, global batch %d sharded by columns" % (cfg["units"], cfg["num_dia"], cfg["batch"]))
    if case == "rbm_cfg3":
        return ("BASELINE config 3: sparse RBM CD-1 step, visible=hidden=%d, num_dia=%d, batch %d"
                % (cfg["units"], cfg["num_dia"], cfg["batch"]))
    return "%s on a %dx%d band with %d diagonals, batch %d" % (case, cfg["units"], cfg["units"], cfg["num_dia"],
                                                              cfg["batch"])


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------

def binding_bound(byts, flops, ms, hbm_peak, fp32_peak):
    """Roofline position of one routine: t_min = max(bytes / HBM peak, flops / FP32 peak); the larger
    term names the bound and frac = t_min / t_measured."""
    t_mem, t_fp = byts / (hbm_peak * 1e9), flops / (fp32_peak * 1e12)
    t = ms * 1e-3
    return {"bound": "fp32" if t_fp > t_mem else "hbm", "frac": max(t_mem, t_fp) / t,
            "t_min_us": max(t_mem, t_fp) * 1e6, "t_mem_us": t_mem * 1e6, "t_fp32_us": t_fp * 1e6,
            "hbm_frac": t_mem / t, "fp32_frac": t_fp / t}


DRAW_SEED = 20260711


def shard_inputs(cb, torch, units, nb, dev, shard, uniforms=True):
    """The batch columns of shard ``shard`` of the global batch: V0 ~ Bernoulli(0.3) from the shard's own seed, so any
    rank can rebuild any other rank's columns (the unsharded check does); U_h, U_v = the uniform numbers in [0, 1) that
    the device-drawn step draws for those columns in step 0 (cuvdia_uniform_f32), so the step that reads them from
    memory and the step that draws them compute the same thing."""
    gen = torch.Generator(device=dev)
    gen.manual_seed(2000 + shard)
    V0 = cb.colmajor_empty(units, nb, dev)
    tmp = torch.rand((nb, units), device=dev, generator=gen)
    V0.t().copy_((tmp < 0.3).float())
    del tmp
    if not uniforms:
        return V0, None, None
    U_h, U_v = cb.colmajor_empty(units, nb, dev), cb.colmajor_empty(units, nb, dev)
    cb.fill_rnd_uniform(U_h, DRAW_SEED, 0, shard * nb, 0)
    cb.fill_rnd_uniform(U_v, DRAW_SEED, 0, shard * nb, 1)
    return V0, U_h, U_v


def check_allreduce(cb, rbm, torch, dist, step, V0, U_h, U_v, W, units, nd, batch, world, rank, dev, mode, drawn):
    """Outside every timed region: (1) three diagonals (first, middle, last) of the all-reduced gradient against the
    rank-order sum of the per-rank partial values gathered to rank 0; (2) on rank 0, the whole all-reduced gradient and
    the bias gradients against the unsharded step on the full batch (all shards rebuilt from their seeds)."""
    stride = W.stride
    some = [0, nd // 2, nd - 1]
    nb = batch // world
    if drawn:
        step.step_drawn(V0, DRAW_SEED, 0, rank * nb)
    else:
        step.step(V0, U_h, U_v)
    part = torch.cat([step.G.vec[k * stride:(k + 1) * stride] for k in some]).clone()
    parts = [torch.empty_like(part) for _ in range(world)] if rank == 0 else None
    dist.gather(part, parts, dst=0)
    step.allreduce()
    torch.cuda.synchronize()
    if rank != 0:
        return None
    got = torch.cat([step.G.vec[k * stride:(k + 1) * stride] for k in some])
    want = parts[0].clone()
    for q in parts[1:]:
        want += q
    d1 = float((got - want).abs().max().item())
    full_in = [shard_inputs(cb, torch, units, nb, dev, s, uniforms=not drawn) for s in range(world)]
    cat = lambda k: torch.cat([f[k].t() for f in full_in], dim=0).t()        # column blocks side by side
    FV0 = cat(0)
    FUh, FUv = (None, None) if drawn else (cat(1), cat(2))
    del full_in
    full = rbm.SparseRBMStep(W, batch, batch, mode, dev)
    if drawn:
        full.step_drawn(FV0, DRAW_SEED, 0, 0)      # the unsharded run draws what the shards drew (col0 = rank * nb)
    else:
        full.step(FV0, FUh, FUv)
    torch.cuda.synchronize()
    d2 = float((step.G.vec - full.G.vec).abs().max().item())
    d3 = float((step.bias_grad - full.bias_grad).abs().max().item())
    # (1) is the same sum in another order over at most `world` terms; (2) compares tree sums of `batch` terms, each
    # at most 1/batch in size, taken in different orders (two such sums per gradient cell on either side): the
    # worst-case rounding is 4 * 2^-24 * (log2(batch) + 2), far inside the 1e-4*sqrt(batch/128) relative tolerance
    # of batch-summed gradients
    import math
    tol = 4.0 * 2.0 ** -24 * (math.log2(batch) + 2)
    ok = d1 <= tol and d2 <= tol and d3 <= tol
    del full, FV0, FUh, FUv
    torch.cuda.empty_cache()
    return {"result": "ok" if ok else "MISMATCH", "tolerance_abs": tol,
            "max_abs_diff_vs_sum_of_gathered_partials_3_diagonals": d1,
            "max_abs_diff_G_vs_unsharded_step_on_rank0": d2, "max_abs_diff_bias_grad_vs_unsharded_step_on_rank0": d3}


def run_ours(args, cfg):
    import numpy as np
    import torch
    import torch.distributed as dist
    import cuv_b200 as cb
    from cuv_b200 import rbm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the DIA path has no CPU fallback "
                         "(use --impl reference for the CPU oracle)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = pin_to_gpu_numa_node(torch, local) if world > 1 else None
    # Libraries (NCCL prints its version banner) write to file descriptor 1; point it at stderr for the
    # run and keep the real stdout for the one JSON line.
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    units, nd, batch = cfg["units"], cfg["num_dia"], cfg["batch"]
    assert batch % world == 0
    nb = batch // world
    mode = cb.MODE_FAST if args.mode == "fast" else cb.MODE_EXACT
    gen = torch.Generator(device=dev)
    gen.manual_seed(1004)                      # identical weights on every rank
    W = cb.dev_dia_matrix_f(units, units, band_offsets(nd), units, 1, device=dev)
    W.vec.normal_(0.0, 0.01, generator=gen)
    drawn = args.uniforms == "drawn"
    col0 = rank * nb
    V0, U_h, U_v = shard_inputs(cb, torch, units, nb, dev, rank)        # this rank's batch columns
    step = rbm.SparseRBMStep(W, nb, batch, mode, dev, keep_v1p=False)
    # The metric counts the GLOBAL problem's algorithmic bytes at every N (strong scaling: value_N / value_1 is the
    # ratio of the step times); `local` is this rank's share, used for the per-kernel figures.
    work = rbm.algorithmic_work(units, units, nd, W.nnz, batch)
    local_work = rbm.algorithmic_work(units, units, nd, W.nnz, nb)

    def one_step(i=0, drawn=drawn):
        # one call of the C ABI: cuvdia_rbm_cd1_step[_drawn][_allreduce]_f32
        if drawn:
            if world > 1:
                step.step_drawn_allreduce(V0, DRAW_SEED, i, col0)
            else:
                step.step_drawn(V0, DRAW_SEED, i, col0)
        elif world > 1:
            step.step_allreduce(V0, U_h, U_v)
        else:
            step.step(V0, U_h, U_v)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing ----
    for _ in range(args.warmup):
        one_step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = cb.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        one_step(i)
    e1.record()
    barrier()
    launches = cb.launch_count() - launches0
    clocks = sampler.stop()
    ms_total = max_over_ranks(e0.elapsed_time(e1))
    ms_step = ms_total / args.steps
    host_uniforms = None
    if drawn:
        # for the record: the same step with the uniform numbers read from tensors resident in HBM
        for _ in range(2):
            one_step(0, False)
        barrier()
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        h0.record()
        for _ in range(args.steps):
            one_step(0, False)
        h1.record()
        barrier()
        host_uniforms = {"ms_per_step": max_over_ranks(h0.elapsed_time(h1)) / args.steps}

    # ---- the same kernels call by call with an event pair around each (outside the timed region) ----
    step.timers = {}
    for i in range(3):
        if drawn:
            step.forward(V0, None, None, draw=(DRAW_SEED, i, col0))
            step.gradients(V0)
        else:
            step.step(V0, U_h, U_v)
    torch.cuda.synchronize()
    op_ms = {k: statistics.mean(event_ms(v)) for k, v in step.timers.items()}
    step.timers = None
    ar_ms = None
    if world > 1:
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a0.record(); step.allreduce(); a1.record()
        torch.cuda.synchronize()
        ar_ms = max_over_ranks(a0.elapsed_time(a1))

    # ---- end to end: host buffers in, results out, every step ----
    e2e = None
    if not args.no_e2e:
        hV0 = torch.empty((nb, units), dtype=torch.float32, pin_memory=True)
        hUh, hUv = torch.empty_like(hV0, pin_memory=True), torch.empty_like(hV0, pin_memory=True)
        hV0.copy_(V0.t()); hUh.copy_(U_h.t()); hUv.copy_(U_v.t())
        # the gradients go back to the host every step: after the all-reduce every rank holds them all, so each rank
        # sends its own 1/N of the diagonals' array over its own link (rank 0 also the bias gradients)
        n_g = step.G.vec.numel()
        g_lo, g_hi = (n_g * rank) // world, (n_g * (rank + 1)) // world
        hG = torch.empty(g_hi - g_lo, dtype=torch.float32, pin_memory=True)
        hb = torch.empty(step.bias_grad.numel(), dtype=torch.float32, pin_memory=True) if rank == 0 else None

        def measure_e2e(drawn_inputs):
            fed = rbm.HostFedRBM(step, allreduce=world > 1, draw=(DRAW_SEED, col0) if drawn_inputs else None)
            host_in = (hV0,) if drawn_inputs else (hV0, hUh, hUv)

            def e2e_steps(k):
                # copies of step i+1 overlap the compute of step i; every step's inputs cross PCIe inside the region
                fed.submit(*host_in)
                for i in range(k):
                    if i + 1 < k:
                        fed.submit(*host_in)
                    fed.run(hG, hb, (g_lo, g_hi))
                fed.wait()

            e2e_steps(2)
            barrier()
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            e2e_steps(args.steps)
            a1.record()
            barrier()
            e2e_ms = max_over_ranks(a0.elapsed_time(a1)) / args.steps
            # For the record, the same loop with the pipeline already primed: the region starts when the first step's
            # inputs are on the device and contains one input copy (for the following step) and one read-back per step.
            fed.submit(*host_in)
            fed.wait()
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for i in range(args.steps):
                fed.submit(*host_in)
                fed.run(hG, hb, (g_lo, g_hi))
            fed.wait()
            s1.record()
            barrier()
            steady_ms = max_over_ranks(s0.elapsed_time(s1)) / args.steps
            fed.run()                                        # consume the copy that is still queued
            torch.cuda.synchronize()
            # the host link alone: one step's input matrices copied with no kernel running - first on this rank
            # alone (rank 0), then on all ranks at once (what a step's input copies share when several GPUs hang off
            # one host)
            def copy_inputs_ms():
                l0, l1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                l0.record()
                for dst, src in zip(fed.inputs[0], host_in):
                    dst.t().copy_(src, non_blocking=True)
                l1.record()
                torch.cuda.synchronize()
                return l0.elapsed_time(l1)
            in_bytes = len(host_in) * units * nb * 4
            alone_ms = copy_inputs_ms() if rank == 0 else 0.0
            barrier()
            all_ms = max_over_ranks(copy_inputs_ms())
            barrier()
            del fed
            torch.cuda.empty_cache()
            return {"value": work["bytes"] / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": int(world * in_bytes),
                    "d2h_bytes_per_step": int((step.G.vec.numel() + step.bias_grad.numel()) * 4),
                    "ms_per_step": e2e_ms,
                    "ms_per_step_pipeline_primed": steady_ms,
                    "host_link_GB/s_one_rank_alone": max_over_ranks(in_bytes / (alone_ms * 1e-3) / 1e9 if rank == 0 else 0.0),
                    "host_link_GB/s_all_ranks_at_once": world * in_bytes / (all_ms * 1e-3) / 1e9,
                    "ms_input_copies_all_ranks_at_once": all_ms,
                    "how": ("pinned host input V0 copied to the device every step on a copy stream, overlapped with the "
                            "previous step's compute; the uniform numbers of the two samples are drawn on the device "
                            "inside the element-wise passes (cuvdia_bias_sigmoid_draw_sum_f32), as the reference draws "
                            "them on the device (rnd_binarize, random/random.cu:139-156); gradients read back to pinned "
                            "host memory every step, every rank its 1/N of the diagonals over its own link") if drawn_inputs else
                           ("pinned host inputs (V0, U_h, U_v) copied to the device every step on a copy stream, "
                            "overlapped with the previous step's compute; gradients read back to pinned host memory "
                            "every step, every rank its 1/N of the diagonals over its own link")}

        e2e = measure_e2e(drawn)
        if drawn:
            host_uniforms["e2e"] = measure_e2e(False)

    # the products once more in the other arithmetic, for the record (outside every timed region)
    other = cb.MODE_EXACT if mode == cb.MODE_FAST else cb.MODE_FAST
    step.mode, step.timers = other, {}
    for _ in range(2):
        step.step(V0, U_h, U_v)
    torch.cuda.synchronize()
    other_ms = {k: min(event_ms(v)) for k, v in step.timers.items() if k.startswith("prod")}
    step.mode, step.timers = mode, None

    ar_check = None
    if world > 1:
        ar_check = check_allreduce(cb, rbm, torch, dist, step, V0, U_h, U_v, W, units, nd, batch, world, rank, dev, mode, drawn)

    status = cb.plan_status(W) if rank == 0 else 0

    if rank != 0:
        if world > 1:
            step._reducer.close()
            dist.destroy_process_group()
        return

    peak, peak_src = load_peaks()
    fp32_fused = fp32_peak_tflops(True)
    fp32_split = fp32_peak_tflops(False)
    # dominant kernel: the banded prod (3 of the 5 large launches per step)
    prod_ms = (2 * op_ms["prod_n"] + op_ms["prod_t"]) / 3.0
    prod_bytes = (2 * local_work["per_call_bytes"]["prod_n"] + local_work["per_call_bytes"]["prod_t"]) / 3.0
    prod_flops = local_work["per_call_flops"]["prod_n"]
    fp32_peak = fp32_fused if args.mode == "fast" else fp32_split
    pos = binding_bound(prod_bytes, prod_flops, prod_ms, peak, fp32_peak)
    per_op = {}
    for k, ms in op_ms.items():
        per_op[k] = {"ms": ms, "calls_per_step": {"prod_n": 2, "prod_t": 1, "dd2dia": 2, "glue": 3, "reduce": 1}.get(k),
                     "gbs": local_work["per_call_bytes"]["reduce_v0" if k == "reduce" else k] / (ms * 1e-3) / 1e9}
        if k in local_work["per_call_flops"]:
            per_op[k]["tflops"] = local_work["per_call_flops"][k] / (ms * 1e-3) / 1e12
            per_op[k]["roofline"] = binding_bound(local_work["per_call_bytes"][k], local_work["per_call_flops"][k], ms, peak,
                                                  fp32_fused if (k == "dd2dia" or args.mode == "fast") else fp32_split)
        else:
            per_op[k]["hbm_frac"] = per_op[k]["gbs"] / peak
    if ar_ms is not None:
        n_ar = step.G.vec.numel() + step.bias_grad.numel()
        per_op["allreduce"] = {"ms": ar_ms, "bytes": 4 * n_ar,
                               "bus_GB/s": 4 * n_ar * 2.0 * (world - 1) / world / (ar_ms * 1e-3) / 1e9,
                               "how": "timed alone here: one ncclAllReduce over the diagonals' values and both bias gradients "
                                      "(one buffer) through cuvdia_allreduce_grad.  In the timed step "
                                      "(cuvdia_rbm_cd1_step_allreduce_f32) the last densedense_to_dia is cut in two launches by "
                                      "column tiles and the diagonals the first one completes are all-reduced on a side stream "
                                      "under the second"}
    tflops = prod_flops / (prod_ms * 1e-3) / 1e12
    if pos["bound"] == "fp32":
        roof = {"bound": "fp32", "achieved": tflops, "peak": fp32_peak, "unit": "TFLOP/s", "frac": tflops / fp32_peak,
                "peak_source": "measured on this device by bench_fp32_peak.cu (register-resident %s loop); "
                               "MEASURED_PEAKS.json has no FP32 CUDA-core entry"
                               % ("fused multiply-add" if args.mode == "fast" else "multiply + add")}
    else:
        roof = {"bound": "hbm", "achieved": prod_bytes / (prod_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                "frac": prod_bytes / (prod_ms * 1e-3) / 1e9 / peak, "peak_source": peak_src}
    roof.update({
        "kernel": "prod_band_kernel", "ms_per_launch": prod_ms,
        "why_this_bound": "t_min = max(bytes / HBM peak, flops / FP32 peak) = max(%.0f, %.0f) us: no tensor cores on "
                          "this path, so FP32 issue binds" % (pos["t_mem_us"], pos["t_fp32_us"]),
        "hbm_achieved": prod_bytes / (prod_ms * 1e-3) / 1e9, "hbm_peak": peak, "hbm_unit": "GB/s",
        "hbm_frac": prod_bytes / (prod_ms * 1e-3) / 1e9 / peak, "hbm_peak_source": peak_src,
        # DRAM bytes per launch: the ncu capture of a smaller case of the same kernel (16384 rows, 512
        # diagonals, 2048 columns: 267.1 MB of dram read+write for 301.7 MB algorithmic, see
        # profiles/prod_n_units16384_nd512_batch2048.md) scaled by the algorithmic bytes of this launch
        "traffic": prod_bytes * (267.1 / 301.7),
        "traffic_source": "ncu dram__bytes_read+write of a smaller case (16384 rows, 512 diagonals, 2048 columns) "
                          "scaled by the algorithmic bytes of this launch"})
    line = {
        "metric": METRIC, "value": work["bytes"] / (ms_step * 1e-3) / 1e9, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.case, cfg), "units": units, "num_dia": nd, "row_fact": 1,
                   "global_batch": batch, "batch_per_gpu": nb, "parallelism": "batch columns x%d" % world, "host_cpus": numa,
                   "prod_arithmetic": args.mode + (" (fused multiply-add; bit-identical to the reference on this workload: "
                                                     "the dense operand of every product is 0/1)" if args.mode == "fast" else
                                                     " (separate multiply and add, reference order)"), "l2": "inputs larger than L2 (each activation matrix %.0f MB)"
                   % (units * nb * 4 / 1e6),
                   "uniforms": ("drawn on the device inside the sampling passes, a pure function of (seed, step, row, "
                                "global column) that the CPU oracle restates bit for bit; the step that reads them from "
                                "precomputed tensors is timed beside it under host_uniforms") if drawn else
                               "precomputed tensors U_h, U_v (inputs of the step)",
                   "algorithmic_bytes_per_step": work["bytes"],
                   "bytes_counted": "the global problem's routines as the reference issues them (3 prod, 2 "
                                    "densedense_to_dia, 4 reduce_to_col), the same number at every N"},
        "gflops": work["flops"] / (ms_step * 1e-3) / 1e9,
        "roofline": roof,
        "fp32": {"achieved_tflops": tflops, "peak_fused_tflops": fp32_fused,
                 "peak_mul_add_tflops": fp32_split, "frac": tflops / fp32_peak},
        "per_op": per_op,
        "prod_other_arithmetic": {"mode": "exact" if args.mode == "fast" else "fast",
                                  "ms": other_ms,
                                  "tflops": {k: local_work["per_call_flops"][k] / (v * 1e-3) / 1e12 for k, v in other_ms.items()}},
        "clocks": clocks, "gpu_launches": int(launches), "plan_status": status,
    }
    if ar_check is not None:
        line["allreduce_check"] = ar_check["result"]
        line["allreduce_check_detail"] = ar_check
    if e2e:
        line["e2e"] = e2e
    if host_uniforms:
        line["host_uniforms"] = host_uniforms
    if world == 1 and not args.no_extra:
        # The step's big kernels are bound by FP32 issue.  Beside them, the same routines on a shape that HBM
        # bounds (2^20 rows, 16 diagonals, 32 columns; operands larger than L2), as a fraction of the HBM peak.
        del step, V0, U_h, U_v
        torch.cuda.empty_cache()
        shapes = {}
        for case, key in (("membound_n", "prod"), ("membound_t", "prod_transposed"), ("membound_dd", "densedense_to_dia")):
            sub = argparse.Namespace(**vars(args))
            sub.case, sub.steps, sub.warmup, sub.flush_l2, sub.cpu = case, 10, 3, False, False
            r = measure_single(sub, cfg)
            shapes[key] = {"GB/s": r["gbs"], "frac_of_hbm_peak": r["hbm_frac"], "us": r["ms"] * 1e3,
                           "arithmetic": args.mode if key != "densedense_to_dia" else "fused"}
        line["hbm_bound_shape"] = {"shape": "2^20 x 2^20, 16 diagonals, 32 batch columns (335 MB algorithmic, ~3 flop/B)",
                                   "peak_GB/s": peak, "routines": shapes}
        # The other BASELINE configurations (single routines and the config-3 step), each against the roofline that
        # binds it; parity for them is in the tests, these are their speeds in the same driver-run record.
        line["configs"] = other_configs(args, cfg, peak, fp32_fused, fp32_split)
    if world == 1 and not args.no_cpu:
        sample = min(batch, args.cpu_sample_cols)
        t, threads, _ = cpu_rbm(units, nd, batch, sample, 1, 0)
        t_full = t * (batch / float(sample))
        line["cpu_baseline"] = {
            "value": work["bytes"] / t_full / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "CD-1 step of the CPU oracle on the first %d of %d batch columns, %d threads, %.1f s; "
                      "time scaled linearly to the full batch" % (sample, batch, threads, t)}
    sys.stdout.flush()
    os.write(real_stdout, (json.dumps(line) + "\n").encode())
    if world > 1:
        step._reducer.close()
        dist.destroy_process_group()


def other_configs(args, cfg, peak, fp32_fused, fp32_split):
    """BASELINE configs 0-2 (single routines, timed as CUDA graphs of back-to-back launches, exact arithmetic) and
    the config-3 RBM step, each with its binding roofline."""
    import torch
    import cuv_b200 as cb
    from cuv_b200 import rbm
    out = {}
    for case in ("cfg0", "cfg1", "cfg2"):
        sub = argparse.Namespace(**vars(args))
        sub.case, sub.steps, sub.warmup, sub.flush_l2, sub.cpu, sub.mode = case, 10, 3, False, False, "exact"
        r = measure_single(sub, cfg)
        pk = fp32_fused if r["op"] == "dd2dia" else fp32_split
        out[case] = {"routine": r["op"], "shape": "%dx%d, %d diagonals, row_fact %d, batch %d" % (
                         r["h"], r["w"], r["num_dia"], r["row_fact"], r["batch"]),
                     "us": r["ms"] * 1e3, "GB/s": r["gbs"], "TFLOP/s": r["tflops"], "timing": r["timing"],
                     "arithmetic": "fused" if r["op"] == "dd2dia" else "exact",
                     "roofline": binding_bound(r["bytes"], r["flops"], r["ms"], peak, pk)}
        torch.cuda.empty_cache()
    c3 = CASES["rbm_cfg3"]
    units, nd, nb = c3["units"], c3["num_dia"], c3["batch"]
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev); gen.manual_seed(1003)
    W = cb.dev_dia_matrix_f(units, units, band_offsets(nd), units, 1, device=dev)
    W.vec.normal_(0.0, 0.01, generator=gen)
    V0, U_h, U_v = shard_inputs(cb, torch, units, nb, dev, 0)
    step = rbm.SparseRBMStep(W, nb, nb, cb.MODE_FAST, dev, keep_v1p=False)
    for _ in range(3):
        step.step(V0, U_h, U_v)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(20):
        step.step(V0, U_h, U_v)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 20
    work = rbm.algorithmic_work(units, units, nd, W.nnz, nb)
    out["rbm_cfg3"] = {"routine": "CD-1 step", "shape": "%d units, %d diagonals, batch %d" % (units, nd, nb),
                       "us": ms * 1e3, "GB/s": work["bytes"] / (ms * 1e-3) / 1e9, "TFLOP/s": work["flops"] / (ms * 1e-3) / 1e12,
                       "arithmetic": "fast (0/1 operands: bit-identical to exact)", "timing": "20 steps back to back",
                       "roofline": binding_bound(work["bytes"], work["flops"], ms, peak, fp32_fused)}
    return out


def run_single(args, cfg):
    """One routine on one GPU (profiling and per-configuration figures)."""
    print(json.dumps(measure_single(args, cfg)), flush=True)


def measure_single(args, cfg):
    import numpy as np
    import torch
    import cuv_b200 as cb
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the DIA path has no CPU fallback")
    torch.cuda.set_device(0)
    mode = cb.MODE_FAST if args.mode == "fast" else cb.MODE_EXACT
    rng = np.random.Generator(np.random.PCG64(1000))
    case = args.case
    if case in ("cfg0", "cfg0_t"):
        # cfg0_t: the transposed product on config 0's matrix (not a BASELINE configuration)
        h = w = 4096; nb = 128; rf = 1
        offs = np.sort(rng.choice(np.arange(-2047, 2048), 64, replace=False)).astype(np.int32)
        op = "prod_n" if case == "cfg0" else "prod_t"
    elif case == "cfg1":
        h, w, nb, rf = 16384, 4096, 512, 4
        offs = np.arange(-128, 128, dtype=np.int32); op = "prod_t"
    elif case == "cfg2":
        h = w = 4096; nb = 1024; rf = 1
        offs = np.sort(rng.choice(np.arange(-2047, 2048), 128, replace=False)).astype(np.int32); op = "dd2dia"
    elif case in ("wide_n", "wide_dd"):
        # scattered diagonals spread over tens of thousands of rows: no shared-memory window fits, the plain
        # one-thread-per-row kernels run (prod_generic_kernel, dd2dia_generic_kernel)
        h = w = 65536; nb = 128 if case == "wide_n" else 256; rf = 1
        offs = np.sort(rng.choice(np.arange(-30000, 30001), 64, replace=False)).astype(np.int32)
        op = "prod_n" if case == "wide_n" else "dd2dia"
    elif case == "membound_dd":
        # densedense_to_dia where HBM bounds it: 2^20 rows, 16 diagonals, 32 batch columns
        h = w = 1 << 20; nb = 32; rf = 1
        offs = band_offsets(16); op = "dd2dia"
    elif case in ("membound_n", "membound_t"):
        # a shape where HBM, not FP32, bounds prod: 2^20 rows, 16 diagonals, 32 batch columns (3 flop/B)
        h = w = 1 << 20; nb = 32; rf = 1
        offs = band_offsets(16); op = "prod_n" if case == "membound_n" else "prod_t"
    elif case in ("spmv_speed_n", "spmv_speed_t"):
        # the reference's own speed fixture (src/tests/spmv_speed.cpp:50-104,155-176): a 256x256 image, 16 output
        # maps, 8x8 filters stored as offsets i*px + j once per map, 14 images, factAv 2, factC 1.3
        px, fs, nm = 256, 8, 16
        h, w, nb, rf = px * px, 16 * px * px, 14, 1
        offs = np.array([i * px + j for _ in range(nm) for i in range(fs) for j in range(fs)], dtype=np.int32)
        op = "prod_n" if case == "spmv_speed_n" else "prod_t"
    elif case == "conv_dd":
        # densedense_to_dia on the convolution-pattern matrix of the spmv speed fixture (65536 x 1048576, 1024 diagonals in
        # 128 runs of 8, 14 images): the weight gradient of that layer
        px, fs, nm = 256, 8, 16
        h, w, nb, rf = px * px, 16 * px * px, 14, 1
        offs = np.array([i * px + j for _ in range(nm) for i in range(fs) for j in range(fs)], dtype=np.int32)
        op = "dd2dia"
    elif case == "dd2dia_speed":
        # the reference's densedense_to_dia speed fixture (src/tests/densedense_to_dia_speed.cpp:65-106): a 28x28
        # image, two output maps, 8x8 filters stored as offsets i*28 + j once per map, 96 images
        h, w, nb, rf = 784, 2 * 784, 96, 1
        offs = np.array([i * 28 + j for _ in range(2) for i in range(8) for j in range(8)], dtype=np.int32)
        op = "dd2dia"
    else:
        h = w = cfg["units"]; nb = cfg["batch"]; rf = 1
        offs = band_offsets(cfg["num_dia"]); op = case
    A = cb.dev_dia_matrix_f(h, w, offs, h, rf)
    A.vec.uniform_(-1, 1)
    X, Y = cb.colmajor_empty(h, nb), cb.colmajor_empty(w, nb)
    X.uniform_(-1, 1); Y.uniform_(-1, 1)
    vec = torch.empty(h, device="cuda")
    vec2 = torch.empty(h, device="cuda")
    nnz, nd = A.nnz, offs.size
    if op == "prod_n":
        fa, fc = (2.0, 1.3) if case.startswith("spmv_speed") else (1.0, 0.0)
        fn = lambda: cb.prod(X, A, Y, "n", "n", fa, fc, mode)
        # B rows the stored cells can address (all of them unless the matrix is much wider than tall)
        b_rows = min(w, h // rf + int(offs.max()) + 1) - max(0, int(offs.min()))
        byts, flops = 4 * (nnz + nd + b_rows * nb + h * nb * (2 if fc else 1)), 2.0 * nnz * nb
    elif op == "prod_t":
        fa, fc = (2.0, 1.3) if case.startswith("spmv_speed") else (1.0, 0.5 if case == "cfg1" else 0.0)
        fn = lambda: cb.prod(Y, A, X, "t", "n", fa, fc, mode)
        byts, flops = 4 * (nnz + nd + h * nb + w * nb * (2 if fc else 1)), 2.0 * nnz * nb
    elif op == "dd2dia":
        fa, fc = (0.01, 0.9) if case == "cfg2" else (1.0, 0.0) if case in ("dd2dia_speed", "conv_dd") else (1.0 / nb, 0.0)
        fn = lambda: cb.densedense_to_dia(A, None, X, Y, fa, fc)
        byts, flops = 4 * (h * nb + w * nb + nd + nnz * (2 if fc else 1)), 2.0 * nnz * nb
    elif op == "reduce":
        fn = lambda: cb.reduce_to_col(vec, X, cb.RF_ADD, 1.0, 0.0)
        byts, flops = 4 * (h * nb + h), float(h * nb)
    elif op == "glue":
        S = cb.colmajor_empty(h, nb)
        fn = lambda: cb.bias_sigmoid_sample(X, vec, Y[:h] if w >= h else X, S)
        byts, flops = 16 * h * nb, 4.0 * h * nb
    elif op == "glue_sum":
        # the element-wise pass that also takes the per-unit batch sum (16 bytes per element + the sums)
        S = cb.colmajor_empty(h, nb)
        fn = lambda: cb.bias_sigmoid_sample_sum(X, vec, Y[:h] if w >= h else X, S, vec2, False, 1.0 / nb, 0.0)
        byts, flops = 16 * h * nb + 4 * h, 5.0 * h * nb
    elif op == "glue_draw":
        # the same pass with the uniform numbers drawn in registers (12 bytes per element + the sums)
        S = cb.colmajor_empty(h, nb)
        fn = lambda: cb.bias_sigmoid_draw_sum(X, vec, S, vec2, 1234, 0, 0, 0, False, 1.0 / nb, 0.0)
        byts, flops = 12 * h * nb + 4 * h, 5.0 * h * nb
    elif op == "update":
        # the weight update of the step over the diagonals' whole value array (12 bytes per value)
        Gd = torch.empty_like(A.vec).uniform_(-1, 1)
        fn = lambda: cb.learn_step_weight_decay(A, Gd, 0.01, 0.05)
        byts, flops = 12 * A.vec.numel(), 3.0 * A.vec.numel()
    else:
        raise SystemExit("unknown case " + case)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if args.flush_l2 else None
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    # a first estimate with plain launches; short kernels are then timed as a CUDA graph of many
    # back-to-back launches so that host launch overhead does not hide the device time
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(); fn(); b.record(); torch.cuda.synchronize()
    est = a.elapsed_time(b)
    reps = 1 if (est > 1.0 or flush is not None) else int(min(200, max(2, 2.0 / max(est, 1e-3))))
    graph = None
    if reps > 1:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()                      # the library's per-stream workspace is allocated on first use: not while recording
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(reps):
                    fn()
        torch.cuda.current_stream().wait_stream(side)
        graph.replay()
        torch.cuda.synchronize()
    l0 = cb.launch_count()
    ts = []
    for _ in range(args.steps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        if graph is not None:
            graph.replay()
        else:
            fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) / reps)
    ms = statistics.median(ts)
    peak, peak_src = load_peaks()
    cpu = None
    if args.cpu and op in ("prod_n", "prod_t", "dd2dia", "reduce"):
        # the CPU oracle on the same shapes (seeded host inputs), one thread and all threads
        from oracle import host_oracle as ho
        Ah = ho.DiaHost(h, w, offs, h, rf, rng.uniform(-1, 1, offs.size * h).astype(np.float32))
        Xh = np.asfortranarray(rng.uniform(-1, 1, (h, nb)).astype(np.float32))
        Yh = np.asfortranarray(rng.uniform(-1, 1, (w, nb)).astype(np.float32))
        vh = np.zeros(h, dtype=np.float32)
        cpu = {}
        for label, nt in (("1", 1), (str(os.cpu_count()), os.cpu_count())):
            t0 = time.perf_counter()
            if op == "prod_n":
                ho.prod(Xh, Ah, Yh, "n", fa, fc, nt)
            elif op == "prod_t":
                ho.prod(Yh, Ah, Xh, "t", fa, fc, nt)
            elif op == "dd2dia":
                ho.densedense_to_dia(Ah, Xh, Yh, fa, fc, nthreads=nt)
            else:
                ho.reduce_to_col(vh, Xh, ho.RF_ADD, 1.0, 0.0, nt)
            cpu["ms_%s_threads" % label] = (time.perf_counter() - t0) * 1e3
    return {"case": case, "op": op, "cpu_oracle": cpu, "h": h, "w": w, "num_dia": int(nd), "row_fact": rf, "batch": nb,
            "mode": args.mode, "ms": ms, "ms_min": min(ts), "bytes": float(byts), "flops": float(flops),
            "gbs": byts / (ms * 1e-3) / 1e9,
            "hbm_frac": byts / (ms * 1e-3) / 1e9 / peak, "tflops": flops / (ms * 1e-3) / 1e12,
            "l2_flushed": bool(args.flush_l2), "launches_per_timing": reps,
            "timing": "CUDA graph of %d back-to-back launches" % reps if reps > 1 else "single launch",
            "gpu_launches": int(cb.launch_count() - l0) if reps == 1 else reps * args.steps}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default=None, choices=["exact", "fast"],
                    help="prod arithmetic; default: fast for the RBM step (bit-identical there, its dense operands are 0/1), "
                         "exact for single routines")
    ap.add_argument("--case", default="rbm_cfg4")
    ap.add_argument("--units", type=int)
    ap.add_argument("--num-dia", type=int)
    ap.add_argument("--batch", type=int)
    ap.add_argument("--cpu-sample-cols", type=int, default=512,
                    help="batch columns of the workload the CPU oracle is timed on (its time is scaled to the full batch)")
    ap.add_argument("--uniforms", default="drawn", choices=["drawn", "host"],
                    help="RBM step: uniform numbers of the samples drawn on the device (default) or read from "
                         "precomputed tensors that the end-to-end run copies from the host every step")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="skip the HBM-bound side measurement of the default run")
    ap.add_argument("--flush-l2", action="store_true")
    ap.add_argument("--cpu", action="store_true", help="single-routine cases: also time the CPU oracle")
    args = ap.parse_args()
    cfg = dict(CASES.get(args.case, CASES["rbm_cfg3"]))
    for k, v in (("units", args.units), ("num_dia", args.num_dia), ("batch", args.batch)):
        if v:
            cfg[k] = v
    if args.mode is None:
        args.mode = "fast" if args.case.startswith("rbm") else "exact"
    if args.impl == "reference":
        return run_reference(args, cfg)
    if args.case.startswith("rbm"):
        return run_ours(args, cfg)
    return run_single(args, cfg)


if __name__ == "__main__":
    main()
