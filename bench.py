#!/usr/bin/env python
"""Benchmark of the thnets forward pass on B200: images/second of a whole network.

One "step" = one forward of one batch.  The default workload is the headline configuration:
ResNet-50, fp16, batch 256 per GPU, 3x224x224 synthetic inputs ~N(0,1), seeded He-normal weights
(no dataset, no trained weights).  With N GPUs every rank runs the whole network on its own batch of
256 (weak scaling: nothing is exchanged between ranks on the data path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload resnet50|resnet18|vgg16|alexnet_owt|segnet]
                    [--dtype fp16|fp32|bf16|int8] [--batch B] [--impl reference]

JSON line (rank 0):
  value    device-resident throughput: the fp32 NCHW batch already in HBM, K forwards (boundary kernels at both ends
           included) timed with CUDA events on the launching stream, max over ranks;
  e2e      the same through THProcessFloat with a pinned HOST batch: H2D of the fp32 input and D2H of the
           logits inside the timed region (wall clock, max over ranks); e2e.pageable_host_buffer: an ordinary buffer;
  roofline the dominant kernels (the implicit-GEMM convolutions): algorithmic FLOPs of all their launches in one
           forward / their time per step (the step's event time x their share of the per-launch profile), against
           the measured burst bf16 GEMM peak (twice that for uint8; the sustained figure beside it);
           roofline.two_roof_bound: the time those launches would take if each ran at the slower of its two roofs
           (FLOPs / tensor peak, algorithmic bytes / measured HBM bandwidth) and its ratio to the measured time --
           more than half the launches of a residual network are HBM-bound; roofline.traffic: DRAM bytes per step
           from the ncu capture summarised under profiles/;
  parity   the logits of this run against the reference's for the same batch (max-abs error / max-abs value, argmax
           agreement), when the reference ran;
  cpu_baseline the unmodified reference CPU build timed on this box's host cores on a bounded sample;
  other_configs   (N = 1) the baseline's other configurations -- AlexNet-OWT fp32 batch 1, ResNet-18 fp16 batch 64, VGG-16 uint8 /
           fp16 batch 32, the segmentation net fp16 batch 16 -- each measured like the headline at its own size;
  e2e_images, int8, strong   sub-records: THProcessImages from byte images, the uint8 engine on the same network,
           and (N > 1) one batch of 256 sharded over the N GPUs by rank 0 alone.
`--impl reference` times only that CPU reference and prints the same line with "impl": "reference".
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("THB200_NO_EXIT", "1")

from thnets_b200 import fixtures as fx  # noqa: E402

WORKLOADS = {
    # name: (builder, default batch, default dtype, loader format)
    "resnet50": (fx.resnet50, 256, "fp16", "py"),
    "resnet18": (fx.resnet18, 64, "fp16", "py"),
    "vgg16": (fx.vgg16, 32, "int8", "t7"),
    "alexnet_owt": (fx.alexnet_owt, 1, "fp32", "t7"),
    "segnet": (fx.segnet, 16, "fp16", "py"),
}
LOWP_RANGE = 20.0


# dram__bytes_read.sum + dram__bytes_write.sum of the convolution launches of ONE forward, from the ncu capture whose
# summary is profiles/conv_resnet50_fp16_b128_dram_tensor.md (captured at batch 128: 4.423 GB, of which 0.051 GB are
# weights; activations scaled to batch 256, weights counted once); None for workloads without a capture
NCU_DRAM_BYTES_PER_STEP = {("resnet50", "fp16", 256): 8.80e9}


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"tflops": d.get("bf16_tflops_sustained", d.get("bf16_tflops")), "tflops_burst": d.get("bf16_tflops"),
                "hbm": d.get("hbm_gbs"), "src": "measured"}
    return {"tflops": 1400.0, "tflops_burst": 1590.0, "hbm": 6650.0, "src": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 50 ms from before the warm-up on; the samples that fall
    inside the timed region are reported (or, if the region was too short to hold three, those since the warm-up began:
    the GPU runs the same forward throughout)."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows, self.proc, self.gpu = [], None, gpu_index
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                                          "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), [c.strip() for c in line.split(",")]))

    def mark_begin(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        good = [(ts, r) for ts, r in self.rows if len(r) > 8 and r[1].replace(".", "").isdigit()]
        inside = [r for ts, r in good if self.t0 is not None and self.t0 <= ts <= (self.t1 or ts)]
        window = "timed region"
        if len(inside) < 3:
            inside, window = [r for ts, r in good], "warm-up + timed region"
        sm = sorted(float(r[1]) for r in inside)
        mx = [float(r[2]) for r in inside if r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[5 + i].lower().startswith("active") for r in inside)]
        # the busiest half of the samples = the clock under load
        load = sm[len(sm) // 2:] if sm else []
        return {"sm_mhz": load[len(load) // 2] if load else None, "sm_max_mhz": mx[0] if mx else None,
                "reasons": reasons, "samples": len(sm), "window": window}


def prefer_gpu_numa_node(local_rank):
    """Ask the kernel to place this process's new pages on the NUMA node of its GPU (set_mempolicy, MPOL_PREFERRED), so that
    the pinned host batch is local to the PCIe root the GPU hangs off.  Returns what was found and done, for the JSON line;
    never fatal (containers may hide the topology or refuse the call).  THB200_BENCH_NUMA=0 skips it."""
    info = {"gpu_node": None, "policy": "default"}
    if os.environ.get("THB200_BENCH_NUMA", "1") == "0":
        return info
    try:
        import torch
        bus = torch.cuda.get_device_properties(local_rank).pci_bus_id
        dom = getattr(torch.cuda.get_device_properties(local_rank), "pci_domain_id", 0)
        path = "/sys/bus/pci/devices/%04x:%02x:00.0/numa_node" % (dom, bus)
        node = int(open(path).read().strip())
        info["gpu_node"] = node
        nodes = [d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()]
        info["nodes"] = len(nodes)
        if node < 0 or len(nodes) < 2:
            return info
        libc = C.CDLL(None, use_errno=True)
        mask = C.c_ulong(1 << node)
        rc = libc.syscall(238, 1, C.byref(mask), 64)   # x86-64 set_mempolicy(MPOL_PREFERRED, &mask, maxnode)
        info["policy"] = "preferred node %d" % node if rc == 0 else "set_mempolicy failed (errno %d)" % C.get_errno()
    except Exception as e:  # noqa: BLE001
        info["policy"] = "unavailable: %s" % str(e)[:80]
    return info


def build_fixture(workload, tmpdir, dtype=None):
    builder, _, _, kind = WORKLOADS[workload]
    # the uint8 engine cannot quantise an all-zero bias: the residual networks get a small random one on their classifier
    g = builder(fc_bias=0.01) if dtype == "int8" and workload in ("resnet50", "resnet18") else builder()
    if kind == "t7":
        path = os.path.join(tmpdir, workload)
        fx.write_torch7(g, path)
    else:
        path = os.path.join(tmpdir, workload + ".net")
        fx.write_pymodel(g, path)
    return g, path


def usable_cores():
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


def omp_threads_for(batch):
    """The reference's batch-parallel GEMM deadlocks unless the OpenMP team divides the batch, and its scratch
    tables hold 32 threads (OpenBLAS-stripped/sgemm.c:967-980, blas.h:1)."""
    cores = min(usable_cores(), 32)
    if batch < 4:
        return cores
    return max(d for d in range(1, cores + 1) if batch % d == 0)


def available_host_gb():
    """Memory this process may still take: the smaller of what the machine reports free and the cgroup's limit."""
    avail = None
    try:
        for line in open("/proc/meminfo"):
            if line.startswith("MemAvailable:"):
                avail = int(line.split()[1]) / 1e6
    except OSError:
        pass
    try:
        lim = open("/sys/fs/cgroup/memory.max").read().strip()
        cur = int(open("/sys/fs/cgroup/memory.current").read().strip())
        if lim != "max":
            room = (int(lim) - cur) / 1e9
            avail = room if avail is None else min(avail, room)
    except (OSError, ValueError):
        pass
    return avail if avail is not None else 16.0


# host memory the reference takes per image of a forward (it keeps every module's output and an im2col buffer per
# thread): measured on ResNet-50, 0.16 GB; the other networks' figures are scaled by their activation sizes
REF_GB_PER_IMAGE = {"resnet50": 0.16, "resnet18": 0.05, "vgg16": 0.25, "alexnet_owt": 0.02, "segnet": 0.5}


def reference_batch(workload, full_batch):
    """The configuration's own batch when the host has room for it (with a margin of two), else the largest
    halving of it that fits."""
    room = available_host_gb() / 2
    b = full_batch
    while b > 1 and b * REF_GB_PER_IMAGE[workload] + 1.0 > room:
        b //= 2
    return max(b, 1)


def reference_child(args):
    """Runs in a fresh process (OMP_NUM_THREADS must be set before the reference library loads): the unmodified reference
    through its own THLoadNetwork / THProcessFloat on the first `ref_batch` images of the benchmark batch.  Saves the
    first forward's output for the parity record of the GPU arm."""
    from oracle.oracle import ref_lib
    from thnets_b200.capi import THNets
    lib = ref_lib()
    if lib is None:
        raise SystemExit("reference library not built (oracle/_ref)")
    with tempfile.TemporaryDirectory() as tmp:
        g, path = build_fixture(args.workload, tmp)
        th = THNets(lib)
        h = th.load_network(path)
        th.set_stats(h, g.mean, g.std)
        x = g.make_input(args.batch, seed=1234)[:args.ref_batch]
        times = []
        for i in range(args.warmup_ref + args.steps_ref):
            t0 = time.perf_counter()
            out, _, _ = th.process_float(h, x)
            times.append(time.perf_counter() - t0)
            if i == 0 and args.ref_out:
                np.save(args.ref_out, out.reshape(args.ref_batch, -1))
        t = sum(times[args.warmup_ref:]) / args.steps_ref
    print(json.dumps({"images_per_s": args.ref_batch / t, "ms_per_step": t * 1e3, "kind": "reference",
                      "lib": os.path.basename(lib), "first_forward_s": times[0]}))


def run_reference(args, steps, warmup, ref_out=None):
    """The reference's own CPU implementation on this box's host cores: the workload's network in fp32 (the reference's
    only CPU precision) at the configuration's batch when host memory allows, `warmup` + `steps` forwards."""
    _, dbatch, _, _ = WORKLOADS[args.workload]
    batch = args.batch or dbatch
    sample = reference_batch(args.workload, batch)
    threads = omp_threads_for(sample)
    env = dict(os.environ, OMP_NUM_THREADS=str(threads))
    cmd = [sys.executable, os.path.abspath(__file__), "--_ref_child", "--workload", args.workload, "--batch", str(batch),
           "--ref-batch", str(sample), "--steps-ref", str(steps), "--warmup-ref", str(warmup)]
    if ref_out:
        cmd += ["--ref-out", ref_out]
    try:
        out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500)
    except subprocess.TimeoutExpired:
        return None, "reference run exceeded 1500 s"
    if out.returncode != 0:
        return None, f"reference run failed: {out.stderr.strip()[-200:]}"
    r = json.loads(out.stdout.strip().splitlines()[-1])
    return {"value": r["images_per_s"], "unit": "images/s", "cores": threads, "kind": r["kind"], "batch": sample,
            "steps": steps, "warmup": warmup,
            "sample": f"{args.workload} fp32, batch {sample} of {batch}, THProcessFloat of {r['lib']}, {threads} OpenMP threads "
                      f"on {usable_cores()} usable cores, {warmup} warm-up + {steps} timed forwards",
            "ms_per_step": r["ms_per_step"]}, None


class Arm:
    """One converted network on this rank's GPU and the host batch it is measured on."""

    def __init__(self, th, workload, dtype, batch, rank, tmpdir):
        self.th, self.lib = th, th.lib
        self.workload, self.dtype, self.batch = workload, dtype, batch
        lib = self.lib
        self.g, path = build_fixture(workload, tmpdir, dtype)
        h = th.load_network(path)
        th.set_stats(h, self.g.mean, self.g.std)
        if dtype == "int8":
            if workload == "vgg16":
                th.make_spatial(h, self.g.input_shape[1])
            self.net = th.create_lowp_network(h, LOWP_RANGE)
        else:
            lib.THB200_SetPrecision({"fp32": 0, "fp16": 1, "bf16": 2}[dtype])
            self.net = lib.THCreateCudaNetwork(h)
            lib.THB200_SetPrecision(0)
            if not self.net:
                raise SystemExit("THCreateCudaNetwork failed: %s" % lib.THB200_LastErrorString())
        th.free_network(h)
        c, hh, ww = self.g.input_shape
        self.shape = (batch, c, hh, ww)
        self.nbytes = batch * c * hh * ww * 4
        self.hptr = lib.THB200_HostAlloc(self.nbytes)          # pinned host batch
        self.host = np.ctypeslib.as_array(C.cast(self.hptr, C.POINTER(C.c_float)), shape=self.shape)
        self.host[...] = self.g.make_input(batch, seed=1234 + rank)
        self.res = C.POINTER(C.c_float)()
        self.ow, self.oh = C.c_int(), C.c_int()
        self.out_count = 0

    def forward(self, ptr=None):
        """THProcessFloat on the host batch (H2D of the batch and D2H of the result inside the call)."""
        b, c, hh, ww = self.shape
        n = self.lib.THProcessFloat(self.net, ptr or self.hptr, b, ww, hh, c, C.byref(self.res), C.byref(self.ow), C.byref(self.oh))
        if n <= 0:
            raise SystemExit("THProcessFloat failed: %s" % self.lib.THB200_LastErrorString())
        self.out_count = n
        return n

    def output(self):
        return np.ctypeslib.as_array(self.res, shape=(self.out_count,)).reshape(self.batch, -1).copy()

    def close(self):
        self.lib.THB200_HostFree(self.hptr)
        self.th.free_network(self.net)


def time_loop(fn, steps, barrier, max_over_ranks):
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    dt = (time.perf_counter() - t0) / steps
    barrier()
    return max_over_ranks(dt)


def measure(arm, steps, warmup, world, barrier, max_over_ranks, peaks):
    """Device-resident value, end-to-end figures and the roofline of the convolution kernel for one converted network."""
    lib, batch = arm.lib, arm.batch
    # The device-resident loop runs the whole-batch plan, so stage the batch into it with the copy/compute pipelining of
    # THProcessFloat switched off once; the end-to-end loops run with the library's default (pipelined sub-batches).
    lib.THB200_SetPipelineChunks(1)
    arm.forward()                      # plans the network, uploads the weights, stages the batch
    first_out = arm.output()           # (later calls re-normalise the host batch in place when mean/std are not the identity)
    lib.THB200_SetPipelineChunks(0)
    for _ in range(warmup):
        arm.forward()
    if lib.THB200_TimeForward(arm.net, warmup) < 0:
        raise SystemExit("THB200_TimeForward failed: %s" % lib.THB200_LastErrorString())
    # --- device-resident: K forwards from the fp32 batch in HBM to the fp32 result in HBM, events on the launching stream
    barrier()
    l0 = lib.THB200_KernelLaunches()
    ms_step = lib.THB200_TimeForward(arm.net, steps)
    launches = lib.THB200_KernelLaunches() - l0
    barrier()
    if ms_step < 0:
        raise SystemExit("THB200_TimeForward failed: %s" % lib.THB200_LastErrorString())
    ms_step = max_over_ranks(ms_step)
    # --- end to end through the public API: pinned host batch, then an ordinary pageable one
    e2e_s = time_loop(arm.forward, steps, barrier, max_over_ranks)
    pageable = np.array(arm.host, copy=True)
    pp = pageable.ctypes.data_as(C.c_void_p)
    arm.forward(pp)
    e2e_pageable_s = time_loop(lambda: arm.forward(pp), max(2, steps // 4), barrier, max_over_ranks)
    del pageable
    out = {"value": world * batch / (ms_step * 1e-3), "ms_per_step": ms_step, "gpu_launches": launches,
           "e2e": {"value": world * batch / e2e_s, "unit": "images/s", "h2d_bytes_per_step": arm.nbytes,
                   "d2h_bytes_per_step": arm.out_count * 4, "ms_per_step": e2e_s * 1e3, "entry": "THProcessFloat",
                   "host_buffer": "pinned (THB200_HostAlloc)", "h2d_gbs_per_gpu": arm.nbytes / e2e_s / 1e9,
                   "pageable_host_buffer": {"value": world * batch / e2e_pageable_s, "ms_per_step": e2e_pageable_s * 1e3}}}
    # --- per-launch profile -> roofline of the dominant kernel
    maxs = 4096
    kinds, ms, fl, by = (C.c_int * maxs)(), (C.c_float * maxs)(), (C.c_double * maxs)(), (C.c_double * maxs)()
    nst = lib.THB200_ProfileForward(arm.net, 5, maxs, kinds, ms, fl)
    if nst > 0:
        u8 = arm.dtype == "int8"
        conv_prof = sum(ms[i] for i in range(nst) if kinds[i] == 0)
        conv_fl = sum(fl[i] for i in range(nst) if kinds[i] == 0)
        tot_prof = sum(ms[i] for i in range(nst))
        nconv = sum(1 for i in range(nst) if kinds[i] == 0)
        # Events between launches switch off the overlap of one kernel's tail with the next one's set-up, so the
        # per-launch times add up to more than a step.  The convolution kernel's time per step is its SHARE of the
        # profile applied to the step as timed above: it cannot exceed the step.
        share = conv_prof / tot_prof if tot_prof else 0.0
        conv_ms = ms_step * share
        # The timed region is far shorter than the seconds it takes a B200 to settle under its power cap: the burst
        # GEMM peak is the denominator (the sustained figure is given beside it).
        peak = peaks["tflops_burst"] * (2 if u8 else 1)
        ach = conv_fl / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0
        roof = {"bound": "tensor",
                "kernel": "conv_simt_kernel" if arm.dtype == "fp32" else "conv_tc_kernel" if u8 else "conv_tc_kernel + conv_patch_tc_kernel",
                "achieved": ach, "peak": peak, "unit": "TFLOP/s" if not u8 else "TOP/s", "frac": ach / peak,
                "peak_source": "of " + peaks["src"] + (": bf16_tflops (burst)" if not u8 else ": 2 x bf16_tflops (burst)"),
                "frac_of_sustained_peak": ach / (peaks["tflops"] * (2 if u8 else 1)),
                "traffic": NCU_DRAM_BYTES_PER_STEP.get((arm.workload, arm.dtype, batch)),
                "launches_per_step": nconv, "kernel_ms_per_step": conv_ms, "share_of_step": share,
                "profile_ms": {"convolutions": conv_prof, "all_launches": tot_prof,
                               "boundary_kernels": sum(ms[i] for i in range(nst) if kinds[i] == 3)},
                "flops_per_step": conv_fl}
        # the bound a forward of this network cannot beat when every launch ran at the slower of its two roofs
        # (algorithmic FLOPs / measured tensor peak, algorithmic bytes / measured HBM copy bandwidth)
        if lib.THB200_ProfileForwardBytes(arm.net, maxs, by) == nst and peaks["hbm"]:
            tpk = peak * 1e12
            bound_ms = sum(max(fl[i] / tpk, by[i] / (peaks["hbm"] * 1e9)) for i in range(nst) if kinds[i] == 0) * 1e3
            hbm_launches = sum(1 for i in range(nst) if kinds[i] == 0 and by[i] / (peaks["hbm"] * 1e9) > fl[i] / tpk)
            roof["two_roof_bound"] = {"kernel_ms_per_step": bound_ms, "frac": bound_ms / conv_ms if conv_ms else None,
                                      "hbm_bound_launches": hbm_launches,
                                      "bytes_per_step": sum(by[i] for i in range(nst) if kinds[i] == 0)}
        out["roofline"] = roof
    return out, first_out


def measure_images(arm, steps, world, barrier, max_over_ranks):
    """End to end through THProcessImages: HWC byte images in host memory (a quarter of the fp32 batch's bytes), converted
    and normalised on the GPU."""
    lib = arm.lib
    b, c, hh, ww = arm.shape
    nbytes = b * hh * ww * 3
    hptr = lib.THB200_HostAlloc(nbytes)
    img = np.ctypeslib.as_array(C.cast(hptr, C.POINTER(C.c_ubyte)), shape=(b, hh, ww, 3))
    img[...] = np.random.default_rng(99).integers(0, 256, img.shape, dtype=np.uint8)
    ptrs = (C.c_void_p * b)(*[hptr + i * hh * ww * 3 for i in range(b)])
    res, ow, oh = C.POINTER(C.c_float)(), C.c_int(), C.c_int()

    def fwd():
        n = lib.THProcessImages(arm.net, ptrs, b, ww, hh, ww * 3, C.byref(res), C.byref(ow), C.byref(oh), 0)
        if n <= 0:
            raise SystemExit("THProcessImages failed: %s" % lib.THB200_LastErrorString())
        return n

    for _ in range(3):
        n = fwd()
    dt = time_loop(fwd, steps, barrier, max_over_ranks)
    # the same images in an ordinary (pageable) array, as a caller of the reference would pass them
    pageable = np.array(img, copy=True)
    base = pageable.ctypes.data
    ptrs = (C.c_void_p * b)(*[base + i * hh * ww * 3 for i in range(b)])
    fwd()
    dt_pageable = time_loop(fwd, max(2, steps // 4), barrier, max_over_ranks)
    del pageable
    lib.THB200_HostFree(hptr)
    return {"value": world * b / dt, "unit": "images/s", "ms_per_step": dt * 1e3, "entry": "THProcessImages",
            "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": n * 4, "host_buffer": "pinned (THB200_HostAlloc)",
            "pageable_host_buffer": {"value": world * b / dt_pageable, "ms_per_step": dt_pageable * 1e3}}


def measure_strong(th, workload, dtype, batch, ngpus, steps, warmup, tmpdir, one_gpu_out):
    """One batch of `batch` images sharded over `ngpus` GPUs by the library itself (contiguous slices, whole network and
    resident weights on every GPU, results gathered into GPU 0 by peer copies): device-resident and end-to-end rates,
    and whether the result equals the single-GPU result of the same batch bit for bit."""
    lib = th.lib
    lib.THB200_SetDevices(ngpus)
    try:
        arm = Arm(th, workload, dtype, batch, 0, tmpdir)
    finally:
        lib.THB200_SetDevices(1)
    arm.forward()
    same = bool(np.array_equal(arm.output(), one_gpu_out))
    for _ in range(warmup):
        arm.forward()
    noop = lambda: None
    ident = lambda v: v
    e2e_s = time_loop(arm.forward, steps, noop, ident)
    lib.THB200_SetPipelineChunks(1)
    arm.forward()
    lib.THB200_SetPipelineChunks(0)
    lib.THB200_TimeForward(arm.net, warmup)
    ms = lib.THB200_TimeForward(arm.net, steps)
    rec = {"scaling": "strong", "n_gpus": ngpus, "global_batch": batch, "images_per_gpu": batch / ngpus,
           "value": batch / (ms * 1e-3) if ms > 0 else None, "unit": "images/s", "ms_per_step": ms,
           "e2e": {"value": batch / e2e_s, "ms_per_step": e2e_s * 1e3, "entry": "THProcessFloat",
                   "gather": "cudaMemcpyPeerAsync into GPU 0, one copy to the host"},
           "bit_identical_to_1gpu": same}
    arm.close()
    return rec


def parity_record(gpu_out, ref_path, tol):
    """The GPU arm's first forward against the reference's output on the same images (max-abs error / max-abs reference)."""
    try:
        ref = np.load(ref_path)
    except OSError:
        return None
    n = min(len(ref), len(gpu_out))
    a, r = gpu_out[:n].astype(np.float64), ref[:n].astype(np.float64)
    rel = float(np.abs(a - r).max() / max(np.abs(r).max(), 1e-30))
    rec = {"images": n, "rel_err": rel, "tol": tol, "ok": bool(rel < tol), "against": "the reference CPU forward of the same images"}
    if r.shape[1] > 1:
        rec["argmax_agree"] = float((a.argmax(1) == r.argmax(1)).mean())
    return rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="resnet50", choices=list(WORKLOADS))
    ap.add_argument("--dtype", default=None, choices=["fp32", "fp16", "bf16", "int8"])
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sub-records", action="store_true", help="headline measurement only (no int8 / THProcessImages records)")
    ap.add_argument("--_ref_child", action="store_true")
    ap.add_argument("--ref-batch", type=int, default=8)
    ap.add_argument("--steps-ref", type=int, default=2)
    ap.add_argument("--warmup-ref", type=int, default=1)
    ap.add_argument("--ref-out", default=None)
    args = ap.parse_args()
    if args._ref_child:
        return reference_child(args)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl != "reference" and world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus N > 1 must be launched with one process per GPU: python -m torch.distributed.run "
                         "--nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 bench.py --gpus N ...")
    _, dbatch, ddtype, _ = WORKLOADS[args.workload]
    batch = args.batch or dbatch
    dtype = args.dtype or ddtype
    warmup = max(args.warmup, 3)
    config = {"workload": f"{args.workload}_{dtype}_b{batch}", "batch_per_gpu": batch, "input": "3x224x224" if args.workload != "segnet" else "3x512x512",
              "parallelism": f"replicated x{world}, batch sharded, no collective",
              "l2": "activations of every large layer exceed the 126 MB L2 (input tensor alone: %.0f MB)" % (batch * 224 * 224 * 8 * 2 / 1e6)}

    # ---------------------------------------------------------------- reference arm
    if args.impl == "reference":
        if rank != 0:
            return
        rsteps = max(1, min(args.steps, 2))
        ref, why = run_reference(args, rsteps, 1)
        if ref is None:
            print(json.dumps({"impl": "reference", "unavailable": why}))
            return
        config["workload"] = f"{args.workload}_fp32_b{ref['batch']}"
        config["batch_per_gpu"] = ref["batch"]
        config["parallelism"] = "host cores only"
        print(json.dumps({"impl": "reference", "metric": "images_per_second", "value": ref["value"], "unit": "images/s",
                          "n_gpus": args.gpus, "steps": ref["steps"], "warmup": ref["warmup"], "requested_steps": args.steps,
                          "requested_warmup": args.warmup, "ms_per_step": ref["ms_per_step"],
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": config, "cpu_baseline": {k: ref[k] for k in ("value", "unit", "cores", "kind", "sample")},
                          "e2e": {"value": ref["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ---------------------------------------------------------------- B200 arm
    os.environ["THB200_DEVICE"] = str(local_rank)
    numa = prefer_gpu_numa_node(local_rank)
    from thnets_b200.distributed import Ranks
    ranks = Ranks("nccl" if world > 1 else None)
    from thnets_b200.capi import THNets
    th = THNets()
    lib = th.lib
    lib.THB200_ProfileForward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.THB200_ProfileForwardBytes.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    lib.THB200_KernelLaunches.restype = C.c_int
    lib.THB200_HostAlloc.restype = C.c_void_p
    barrier, max_over_ranks = ranks.barrier, ranks.max
    peaks = read_peaks()
    tmp = tempfile.TemporaryDirectory()

    # the reference CPU forward runs after the GPU measurements (rank 0 of a single-GPU run only)
    ref_out = os.path.join(tmp.name, "ref_logits.npy")
    want_ref = rank == 0 and world == 1 and not args.no_cpu_baseline

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    arm = Arm(th, args.workload, dtype, batch, rank, tmp.name)
    sampler.mark_begin()
    head, first_out = measure(arm, args.steps, warmup, world, barrier, max_over_ranks, peaks)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None

    out = None
    if rank == 0:
        out = {"metric": "images_per_second", "value": head["value"], "unit": "images/s", "n_gpus": world,
               "steps": args.steps, "warmup": warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": {"fp16": "f16", "fp32": "f32", "bf16": "bf16", "int8": "u8"}[dtype], "data": "synthetic",
               "config": config, "e2e": head["e2e"], "gpu_launches": head["gpu_launches"], "clocks": clocks, "host_numa": numa,
               "roofline": head.get("roofline"),
               "timed_region": "value: boundary kernels (fp32 NCHW <-> the engine's layout) and every planned launch, batch and "
                               "result resident in HBM; e2e: the THProcessFloat call with host buffers"}
    # ---- sub-records measured in the same run: the byte-image entry point and the uint8 engine
    if not args.no_sub_records:
        images = measure_images(arm, args.steps, world, barrier, max_over_ranks)
        if rank == 0:
            out["e2e_images"] = images
    arm.close()
    if not args.no_sub_records and dtype != "int8" and args.workload in ("resnet50", "resnet18", "vgg16"):
        arm8 = Arm(th, args.workload, "int8", batch, rank, tmp.name)
        sub, _ = measure(arm8, args.steps, warmup, world, barrier, max_over_ranks, peaks)
        arm8.close()
        if rank == 0:
            out["int8"] = {"config": f"{args.workload}_int8_b{batch} (uint8 lowp engine, range {LOWP_RANGE:g})", "value": sub["value"],
                           "unit": "images/s", "ms_per_step": sub["ms_per_step"], "e2e": sub["e2e"], "gpu_launches": sub["gpu_launches"],
                           "roofline": sub.get("roofline")}
    # ---- the other configurations of the baseline (its CPU-runnable case, the small-batch and the segmentation cases), each
    # measured the same way at its own batch size on this rank's GPU: N = 1 only, they are parity cases, not the headline
    if world == 1 and not args.no_sub_records and args.workload == "resnet50" and args.batch is None and args.dtype is None:
        others = []
        for wl, dt, b in (("alexnet_owt", "fp32", 1), ("resnet18", "fp16", 64), ("vgg16", "int8", 32), ("vgg16", "fp16", 32),
                          ("segnet", "fp16", 16)):
            try:
                a2 = Arm(th, wl, dt, b, rank, tmp.name)
                sub, _ = measure(a2, args.steps, warmup, world, barrier, max_over_ranks, peaks)
                a2.close()
                rf = sub.get("roofline") or {}
                others.append({"workload": f"{wl}_{dt}_b{b}", "value": sub["value"], "unit": "images/s",
                               "ms_per_step": sub["ms_per_step"], "e2e": sub["e2e"]["value"], "gpu_launches": sub["gpu_launches"],
                               "roofline_frac": rf.get("frac"), "two_roof_frac": (rf.get("two_roof_bound") or {}).get("frac")})
            except SystemExit as e:
                others.append({"workload": f"{wl}_{dt}_b{b}", "unavailable": str(e)[:200]})
        out["other_configs"] = others
    # ---- strong scaling inside the library: ONE batch over the N GPUs of this box (rank 0 alone drives them; the other
    # ranks hold no work and wait on the host, through the rendezvous store, so that no kernel of theirs sits on a GPU)
    if world > 1 and not args.no_sub_records:
        import torch
        torch.cuda.synchronize()
        barrier()
        if rank == 0:
            try:
                out["strong"] = measure_strong(th, args.workload, dtype, batch, world, args.steps, warmup, tmp.name, first_out)
            except (SystemExit, RuntimeError) as e:
                out["strong"] = {"unavailable": str(e)[:200]}
            ranks.host_signal("strong_done")
        else:
            ranks.host_wait("strong_done")
    if rank == 0:
        if want_ref:
            ref, why = run_reference(args, 2, 1, ref_out)
            out["cpu_baseline"] = ({k: ref[k] for k in ("value", "unit", "cores", "kind", "sample")} if ref
                                   else {"value": None, "unit": "images/s", "cores": 0, "kind": "reference", "sample": why})
            if ref and dtype != "int8":
                out["parity"] = parity_record(first_out, ref_out, {"fp32": 1e-4, "fp16": 1e-2, "bf16": 6e-2}[dtype])
        print(json.dumps(out))
    ranks.close()


if __name__ == "__main__":
    main()
