#!/usr/bin/env python
"""Benchmark of the thnets forward pass on B200: images/second of a whole network.

One "step" = one forward of one batch.  The default workload is the headline configuration:
ResNet-50, fp16, batch 256 per GPU, 3x224x224 synthetic inputs ~N(0,1), seeded He-normal weights
(no dataset, no trained weights).  With N GPUs every rank runs the whole network on its own batch of
256 (weak scaling: nothing is exchanged between ranks on the data path).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload resnet50|resnet18|vgg16|alexnet_owt|segnet]
                    [--dtype fp16|fp32|bf16|int8] [--batch B] [--impl reference]

JSON line (rank 0):
  value    device-resident throughput: inputs already in HBM, K forwards timed with CUDA events on the
           launching stream, max over ranks;
  e2e      the same through THProcessFloat with a pinned HOST batch: H2D of the fp32 input and D2H of the
           logits inside the timed region (wall clock, max over ranks);
  roofline the dominant kernel (implicit-GEMM convolution): algorithmic FLOPs of all its launches in one
           forward / their summed event-timed durations, against the measured bf16 GEMM peak (twice that for
           uint8); roofline.two_roof_bound: the time those launches would take if each ran at the slower of its
           two roofs (FLOPs / tensor peak, algorithmic bytes / measured HBM bandwidth) and its ratio to the
           measured time -- many layers of a residual network are HBM-bound;
  cpu_baseline the unmodified reference CPU build timed on this box's host cores on a bounded sample.
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
# summary is kept under profiles/ (captured at batch 128, activations scaled to batch 256, weights once)
NCU_DRAM_BYTES_PER_STEP = {("resnet50", "fp16", 256): 9.08e9}


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"tflops": d.get("bf16_tflops_sustained", d.get("bf16_tflops")), "hbm": d.get("hbm_gbs"), "src": "measured"}
    return {"tflops": 1590.0, "hbm": 6650.0, "src": "fallback"}


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


def omp_threads_for(batch):
    """The reference's batch-parallel GEMM deadlocks unless the OpenMP team divides the batch, and its scratch
    tables hold 32 threads (OpenBLAS-stripped/sgemm.c:967-980, blas.h:1)."""
    cores = min(os.cpu_count() or 1, 32)
    if batch < 4:
        return cores
    return max(d for d in range(1, cores + 1) if batch % d == 0)


def reference_child(args):
    """Runs in a fresh process (OMP_NUM_THREADS must be set before the reference library loads)."""
    from oracle.oracle import ref_lib
    from thnets_b200.capi import THNets
    lib = ref_lib()
    kind = "reference"
    if lib is None:
        raise SystemExit("reference library not built (oracle/_ref)")
    with tempfile.TemporaryDirectory() as tmp:
        g, path = build_fixture(args.workload, tmp)
        th = THNets(lib)
        h = th.load_network(path)
        th.set_stats(h, g.mean, g.std)
        x = g.make_input(args.ref_batch)
        times = []
        for i in range(args.warmup_ref + args.steps_ref):
            t0 = time.perf_counter()
            th.process_float(h, x)
            times.append(time.perf_counter() - t0)
        t = sum(times[args.warmup_ref:]) / args.steps_ref
    print(json.dumps({"images_per_s": args.ref_batch / t, "ms_per_step": t * 1e3, "kind": kind,
                      "lib": os.path.basename(lib)}))


def run_reference(args, steps, warmup):
    """The reference's own CPU implementation on this box's host cores, on a bounded sample of the workload."""
    _, batch, dtype, _ = WORKLOADS[args.workload]
    sample = {"resnet50": 16, "resnet18": 32, "vgg16": 4, "alexnet_owt": 1, "segnet": 2}[args.workload]
    threads = omp_threads_for(sample)
    env = dict(os.environ, OMP_NUM_THREADS=str(threads))
    cmd = [sys.executable, os.path.abspath(__file__), "--_ref_child", "--workload", args.workload, "--ref-batch", str(sample),
           "--steps-ref", str(steps), "--warmup-ref", str(warmup)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    if out.returncode != 0:
        return None, f"reference run failed: {out.stderr.strip()[-200:]}"
    r = json.loads(out.stdout.strip().splitlines()[-1])
    return {"value": r["images_per_s"], "unit": "images/s", "cores": threads, "kind": r["kind"],
            "sample": f"{args.workload} fp32, batch {sample}, THProcessFloat of {r['lib']}, {warmup} warm-up + {steps} timed forwards",
            "ms_per_step": r["ms_per_step"]}, None


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
    ap.add_argument("--_ref_child", action="store_true")
    ap.add_argument("--ref-batch", type=int, default=8)
    ap.add_argument("--steps-ref", type=int, default=3)
    ap.add_argument("--warmup-ref", type=int, default=1)
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
        ref, why = run_reference(args, max(2, min(args.steps, 5)), 1)
        if ref is None:
            print(json.dumps({"impl": "reference", "unavailable": why}))
            return
        print(json.dumps({"impl": "reference", "metric": "images_per_second", "value": ref["value"], "unit": "images/s",
                          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ref["ms_per_step"],
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": config, "cpu_baseline": {k: ref[k] for k in ("value", "unit", "cores", "kind", "sample")},
                          "e2e": {"value": ref["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    # ---------------------------------------------------------------- B200 arm
    os.environ["THB200_DEVICE"] = str(local_rank)
    from thnets_b200.distributed import Ranks
    ranks = Ranks("nccl" if world > 1 else None)
    from thnets_b200.capi import THNets
    th = THNets()
    lib = th.lib
    lib.THB200_ProfileForward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.THB200_ProfileForwardBytes.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    lib.THB200_KernelLaunches.restype = C.c_int

    tmp = tempfile.TemporaryDirectory()
    g, path = build_fixture(args.workload, tmp.name, dtype)
    h = th.load_network(path)
    th.set_stats(h, g.mean, g.std)
    if dtype == "int8":
        if args.workload == "vgg16":
            th.make_spatial(h, g.input_shape[1])
        net = th.create_lowp_network(h, LOWP_RANGE)
    else:
        lib.THB200_SetPrecision({"fp32": 0, "fp16": 1, "bf16": 2}[dtype])
        net = lib.THCreateCudaNetwork(h)
        if not net:
            raise SystemExit("THCreateCudaNetwork failed: %s" % lib.THB200_LastErrorString())
    th.free_network(h)

    # pinned host batch (the e2e path copies it to the device every step)
    c, hh, ww = g.input_shape
    nbytes = batch * c * hh * ww * 4
    hptr = lib.THB200_HostAlloc(nbytes)
    host = np.ctypeslib.as_array(C.cast(hptr, C.POINTER(C.c_float)), shape=(batch, c, hh, ww))
    host[...] = g.make_input(batch, seed=1234 + rank)
    res = C.POINTER(C.c_float)()
    ow, oh = C.c_int(), C.c_int()

    def forward_e2e():
        n = lib.THProcessFloat(net, hptr, batch, ww, hh, c, C.byref(res), C.byref(ow), C.byref(oh))
        if n <= 0:
            raise SystemExit("THProcessFloat failed: %s" % lib.THB200_LastErrorString())
        return n

    barrier, max_over_ranks = ranks.barrier, ranks.max

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # The device-resident loop runs the whole-batch plan, so stage the batch into it with the copy/compute pipelining of
    # THProcessFloat switched off once; the end-to-end loop below runs with the library's default (pipelined sub-batches).
    lib.THB200_SetPipelineChunks(1)
    out_count = forward_e2e()          # plans the network, uploads the weights, stages the batch
    lib.THB200_SetPipelineChunks(0)
    for _ in range(warmup):
        forward_e2e()
    if lib.THB200_TimeForward(net, warmup) < 0:
        raise SystemExit("THB200_TimeForward failed: %s" % lib.THB200_LastErrorString())

    # --- device-resident: K forwards, events on the launching stream
    barrier()
    sampler.mark_begin()
    l0 = lib.THB200_KernelLaunches()
    ms_step = lib.THB200_TimeForward(net, args.steps)
    launches = lib.THB200_KernelLaunches() - l0
    barrier()
    if ms_step < 0:
        raise SystemExit("THB200_TimeForward failed: %s" % lib.THB200_LastErrorString())
    ms_step = max_over_ranks(ms_step)
    # --- end to end through the public API with host buffers
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        forward_e2e()
    e2e_s = (time.perf_counter() - t0) / args.steps
    barrier()
    e2e_s = max_over_ranks(e2e_s)
    sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None

    # --- per-launch profile for the roofline of the dominant kernel
    maxs = 4096
    kinds = (C.c_int * maxs)()
    ms = (C.c_float * maxs)()
    fl = (C.c_double * maxs)()
    nst = lib.THB200_ProfileForward(net, 5, maxs, kinds, ms, fl)
    roof = None
    peaks = read_peaks()
    if nst > 0:
        conv_ms = sum(ms[i] for i in range(nst) if kinds[i] == 0)
        conv_fl = sum(fl[i] for i in range(nst) if kinds[i] == 0)
        tot_ms = sum(ms[i] for i in range(nst))
        nconv = sum(1 for i in range(nst) if kinds[i] == 0)
        ach = conv_fl / (conv_ms * 1e-3) / 1e12 if conv_ms > 0 else 0.0
        roof = {"bound": "tensor", "kernel": "conv_tc_kernel" if dtype != "fp32" else "conv_simt_kernel",
                "achieved": ach, "peak": peaks["tflops"] if dtype != "int8" else peaks["tflops"] * 2, "unit": "TFLOP/s",
                "frac": ach / (peaks["tflops"] * (2 if dtype == "int8" else 1)), "peak_source": "of " + peaks["src"],
                "traffic": NCU_DRAM_BYTES_PER_STEP.get((args.workload, dtype, batch)), "launches_per_step": nconv, "kernel_ms_per_step": conv_ms, "share_of_step": conv_ms / tot_ms if tot_ms else None,
                "flops_per_step": conv_fl}
        # the bound a forward of this network cannot beat when every launch ran at the slower of its two roofs
        # (algorithmic FLOPs / measured tensor peak, algorithmic bytes / measured HBM copy bandwidth)
        by = (C.c_double * maxs)()
        if lib.THB200_ProfileForwardBytes(net, maxs, by) == nst and peaks["hbm"]:
            tpk = peaks["tflops"] * 1e12 * (2 if dtype == "int8" else 1)
            bound_ms = sum(max(fl[i] / tpk, by[i] / (peaks["hbm"] * 1e9)) for i in range(nst) if kinds[i] == 0) * 1e3
            hbm_launches = sum(1 for i in range(nst) if kinds[i] == 0 and by[i] / (peaks["hbm"] * 1e9) > fl[i] / tpk)
            roof["two_roof_bound"] = {"kernel_ms_per_step": bound_ms, "frac": bound_ms / conv_ms if conv_ms else None,
                                      "hbm_bound_launches": hbm_launches, "bytes_per_step": sum(by[i] for i in range(nst) if kinds[i] == 0)}

    if rank == 0:
        out = {"metric": "images_per_second", "value": world * batch / (ms_step * 1e-3), "unit": "images/s", "n_gpus": world,
               "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": {"fp16": "f16", "fp32": "f32", "bf16": "bf16", "int8": "u8"}[dtype], "data": "synthetic",
               "config": config,
               "e2e": {"value": world * batch / e2e_s, "unit": "images/s", "h2d_bytes_per_step": nbytes,
                       "d2h_bytes_per_step": out_count * 4, "ms_per_step": e2e_s * 1e3},
               "gpu_launches": launches, "clocks": clocks, "roofline": roof}
        if world == 1 and not args.no_cpu_baseline:
            ref, why = run_reference(args, 3, 1)
            out["cpu_baseline"] = ({k: ref[k] for k in ("value", "unit", "cores", "kind", "sample")} if ref
                                   else {"value": None, "unit": "images/s", "cores": 0, "kind": "reference", "sample": why})
        print(json.dumps(out))
    lib.THB200_HostFree(hptr)
    th.free_network(net)
    ranks.close()


if __name__ == "__main__":
    main()
