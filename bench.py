#!/usr/bin/env python3
"""Benchmark of the fused gather -> forward -> scatter step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--precision bf16|fp32|fp8w] [--workload column|stencil|...]
    python bench.py --impl reference ...     # the CPU implementation of the same path on the host cores

Workload (default "column", BASELINE config 2): 49,152 columns x 60 levels; 244 features gathered from four
Fortran (ncol,60) fp32 fields + 4 per-column scalars; 244 -> 768 x4 -> 128 MLP with LeakyReLU(0.15); 128 outputs
scattered into two (ncol,60) arrays and eight (ncol) vectors.  Synthetic seeded inputs with the configuration's
shapes and distributions stand in for the climate data the reference measured on.

One "step" = one call of the fused entry point over all columns of this rank.  `value` is measured with the
Fortran arrays resident in HBM; `e2e` is the same call given HOST arrays (pinned), so the H2D of every input
array and the D2H of every output array are inside the timed region.  Multi-GPU: one process per GPU, each rank
owns its own contiguous column block (weak scaling, no data-path collective); the per-rank fp64 checksums are
summed with one NCCL all-reduce after the timed loop.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FLOP_PER_COL = {"column": 2 * (244 * 768 + 3 * 768 * 768 + 768 * 128), "stencil": 2 * (27 * 20 + 20 * 20 + 20 * 3),
                "toy": 2 * (64 * 256 + 256 * 256 + 256 * 64), "conv": 2 * 27 * (3 * 64 + 12 * 64 * 64 + 64 * 3)}
BYTES_PER_COL = {"column": 4 * (244 + 128), "stencil": 24, "toy": 4 * 128}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="fortis_b200", choices=["fortis_b200", "reference"])
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp32", "fp8w"])
    ap.add_argument("--workload", default="column", choices=["column", "column_c5", "stencil", "toy", "conv"])
    ap.add_argument("--ncol", type=int, default=0, help="override the per-rank column count (column workloads)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-incumbent", action="store_true")
    return ap.parse_args()


# -----------------------------------------------------------------------------------------------------------------
# workloads
# -----------------------------------------------------------------------------------------------------------------
def make_workload(name, rank, ncol_override=0):
    from oracle import fortis_oracle as fo     # descriptor builders only (plain dict construction)
    import fortis_b200
    if name in ("column", "column_c5"):
        ncol = ncol_override or (49152 if name == "column" else 1 << 20)
        nlev = 60
        G, S, Lp, K = fo.column_descriptors(ncol, nlev)
        rng = np.random.default_rng((2 if name == "column" else 7000) + rank)
        f32 = np.float32
        gin = [np.asfortranarray((250 + 20 * rng.standard_normal((ncol, nlev), dtype=f32))),
               np.asfortranarray(np.exp(-6 + rng.standard_normal((ncol, nlev), dtype=f32))),
               np.asfortranarray(10 * rng.standard_normal((ncol, nlev), dtype=f32)),
               np.asfortranarray(10 * rng.standard_normal((ncol, nlev), dtype=f32))]
        gin += [rng.standard_normal(ncol, dtype=f32) for _ in range(4)]
        sout = [np.zeros((ncol, nlev), f32, order="F") for _ in range(2)] + [np.zeros(ncol, f32) for _ in range(8)]
        layers = fortis_b200.mlp_layers([244, 768, 768, 768, 768, 128], seed=0)
        return dict(G=G, S=S, Lp=Lp, K=K, gin=gin, sout=sout, layers=layers, units=ncol, kind="column",
                    label="climate column MLP, %d columns x 60 levels, 244->768x4->128" % ncol)
    if name == "stencil":
        nx, ny, nz = 1440, 1080, 4
        G, S, Lp, K = fo.stencil_descriptors(nx, ny, nz)
        rng = np.random.default_rng(3 + rank)
        gin = [np.asfortranarray(rng.standard_normal((nx + 2, ny + 2, nz), dtype=np.float32)) for _ in range(3)]
        sout = [np.zeros((nx + 2, ny + 2, nz), np.float32, order="F") for _ in range(3)]
        layers = fortis_b200.mlp_layers([27, 20, 20, 3], seed=4, init="uniform", act="relu", bias="uniform")
        return dict(G=G, S=S, Lp=Lp, K=K, gin=gin, sout=sout, layers=layers, units=nx * ny * nz, kind="stencil",
                    label="ocean stencil MLP, 1440x1080x4 points, 27->20->20->3")
    if name == "conv":
        shape = (8, 33, 33, 33)
        rng = np.random.default_rng(5 + rank)
        x = rng.standard_normal(shape + (3,), dtype=np.float32)
        y = np.zeros(shape + (3,), np.float32)
        layers = fortis_b200.conv_layers(3, 64, 3, nblocks=6, seed=6)
        return dict(G=None, S=None, Lp=None, K=None, gin=[x], sout=[y], layers=layers, units=int(np.prod(shape)), kind="conv",
                    shape=shape, label="conv3d super-resolution net, 8 x 33^3 x 3 NDHWC, 3->64, 6 residual blocks, 64->3")
    ncol = 4096
    G, S, Lp, K = fo.identity_descriptors(64, 64, ncol)
    rng = np.random.default_rng(rank)
    gin = [np.asfortranarray((2 * rng.random((64, ncol)) - 1).astype(np.float32))]
    sout = [np.zeros((64, ncol), np.float32, order="F")]
    layers = fortis_b200.mlp_layers([64, 256, 256, 64], seed=1, init="kaiming_uniform", act="relu")
    return dict(G=G, S=S, Lp=Lp, K=K, gin=gin, sout=sout, layers=layers, units=ncol, kind="toy", label="toy MLP, 4096 columns")


# -----------------------------------------------------------------------------------------------------------------
# clocks
# -----------------------------------------------------------------------------------------------------------------
class ClockSampler:
    """One `nvidia-smi -lms` process sampling SM clock and throttle reasons while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE, text=True)
            time.sleep(0.3)            # let it produce its first sample before the region starts
        except Exception:
            self.proc = None

    def stop(self):
        samples = []
        if self.proc:
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
            except Exception:
                self.proc.kill()
                out = ""
            samples = [[x.strip() for x in l.split(",")] for l in out.splitlines() if l.strip()]
        sm = sorted(int(s[0]) for s in samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(s) > 2 + i and s[2 + i].lower().startswith("active") for s in samples)]
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(samples)}


# -----------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's C port of the native forward, all host threads, bounded sample
# -----------------------------------------------------------------------------------------------------------------
def cpu_step_fn(wl, sample_units):
    import ctypes
    from oracle import build as ob
    from oracle import cport
    lib = ctypes.CDLL(ob.build_port(verbose=False))
    # all host cores this process may use (torchrun exports OMP_NUM_THREADS=1, which is not what a CPU baseline wants)
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    from oracle import fortis_oracle as fo
    G, S, Lp, K = wl["G"], wl["S"], wl["Lp"], wl["K"]
    P = fo.loop_params(Lp, K)
    Ag = fo.plan_arrays(G, [(s["array"], s["idx"]) for s in G["slots"]])
    As = fo.plan_arrays(S, [(s["array"], s["idx"]) for s in S["stores"]])

    def slot_tables(J, A, key):
        arr = (ctypes.c_int * len(J[key]))(*[s["array"] for s in J[key]])
        off = (ctypes.c_long * len(J[key]))(*[int(fo._elem(A, s["array"], s["idx"], P["ilo"], P["jlo"])) for s in J[key]])
        na = len(J["arrays"])
        si, sj, sk = [0] * na, [0] * na, [0] * na
        for s in J[key]:
            a = s["array"]
            for d, c in enumerate(s["idx"]):
                if c[0] == "i":
                    si[a] = A[a]["strides"][d]
                elif c[0] == "j":
                    sj[a] = A[a]["strides"][d]
            sk[a] = A[a]["plane"] if A[a]["vdims"] else 0
        L = ctypes.c_long * na
        return arr, off, L(*si), L(*sj), L(*sk)
    ia, io, isi, isj, isk = slot_tables(G, Ag, "slots")
    oa, oo, osi, osj, osk = slot_tables(S, As, "stores")
    fpp = ctypes.POINTER(ctypes.c_float)
    inp = (fpp * len(wl["gin"]))(*[a.ctypes.data_as(fpp) for a in wl["gin"]])
    outp = (fpp * len(wl["sout"]))(*[a.ctypes.data_as(fpp) for a in wl["sout"]])
    PL = cport.pack_layers(wl["layers"])
    # a sample of `sample_units` columns of the first plane (columns are independent, cost is per column)
    count = min(sample_units, P["count"])
    cs = ctypes.c_double()

    step_count = count

    def step():
        lib.oracle_step(ctypes.c_long(count), 1, P["ni"], len(G["slots"]), inp, ia, io, isi, isj, isk,
                        len(S["stores"]), outp, oa, oo, osi, osj, osk, PL["n"], PL["dims"], PL["Wp"], PL["bp"], PL["act"],
                        PL["slope"], threads, ctypes.byref(cs))
        return count
    return step, threads


def time_cpu(wl, target_s=12.0):
    probe_units = 256 if wl["kind"] != "stencil" else 65536
    step, threads = cpu_step_fn(wl, probe_units)
    t0 = time.perf_counter(); n = step(); dt = time.perf_counter() - t0
    t0 = time.perf_counter(); n = step(); dt = min(dt, time.perf_counter() - t0)
    rate = n / dt
    sample = int(min(wl["units"], max(probe_units, rate * target_s)))
    step, threads = cpu_step_fn(wl, sample)
    done, passes, t0 = 0, 0, time.perf_counter()
    while True:                                   # whole passes over the sample until about target_s of CPU work
        done += step(); passes += 1
        dt = time.perf_counter() - t0
        if dt >= target_s or passes >= 64:
            break
    return dict(value=done / dt, unit="columns/s", cores=threads, kind="port",
                sample="%d of %d columns of the same workload x %d passes, %.1f s; C port of the reference's native "
                       "Fortran forward (no Fortran compiler in the image), OpenMP over columns" % (done // passes, wl["units"], passes, dt))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = make_workload(args.workload, 0, args.ncol)
    probe = 256 if wl["kind"] != "stencil" else 65536
    step, threads = cpu_step_fn(wl, probe)
    t0 = time.perf_counter(); n = step(); dt = time.perf_counter() - t0
    budget = 120.0 / max(1, args.steps + args.warmup)
    sample = int(min(wl["units"], max(probe, (n / dt) * min(budget, 10.0))))
    step, threads = cpu_step_fn(wl, sample)
    sample = step()
    for _ in range(max(0, args.warmup - 1)):
        step()
    t0 = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        done += step()
    dt = time.perf_counter() - t0
    v = done / dt
    line = {"impl": "reference", "metric": "fused-step columns/sec", "value": v, "unit": "columns/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": wl["label"], "columns_per_step_sample": sample},
            "cpu_baseline": {"value": v, "unit": "columns/s", "cores": threads, "kind": "port",
                             "sample": "%d of %d columns per step" % (sample, wl["units"])},
            "e2e": {"value": v, "unit": "columns/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


# -----------------------------------------------------------------------------------------------------------------
# GPU arm
# -----------------------------------------------------------------------------------------------------------------
# the library path the reference's runtime takes on a GPU, for comparison (column workloads): materialise X with a
# gather, one cuBLAS SGEMM per layer with a separate bias / activation pass, scatter Y (runtime/fortis_rt.c:87-100,
# compiler/FortisFuse.cpp:587-655).  torch's fp32 matmul with TF32 off is that SGEMM.  Reported beside the result;
# never part of `value`.
# -----------------------------------------------------------------------------------------------------------------
def time_incumbent(torch, wl, d_in, d_out, flush, steps=10):
    torch.backends.cuda.matmul.allow_tf32 = False
    ncol = wl["units"]
    W = [torch.from_numpy(L["W"]).cuda() for L in wl["layers"]]
    B = [torch.from_numpy(L["b"]).cuda() for L in wl["layers"]]
    views_in = [a.view(-1, ncol).t() for a in d_in]                # Fortran (ncol, nlev) -> (ncol, nlev) strided views
    outs = [a.view(-1, ncol).t() for a in d_out]

    def step():
        x = torch.cat(views_in, dim=1).contiguous()                # the gather kernel's X
        for l, L in enumerate(wl["layers"]):
            x = torch.addmm(B[l], x, W[l].t())
            if L["act"] == "leaky":
                x = torch.nn.functional.leaky_relu(x, L["slope"])
            elif L["act"] == "relu":
                x = torch.relu(x)
        o = 0
        for v in outs:                                             # the scatter kernel
            v.copy_(x[:, o:o + v.shape[1]])
            o += v.shape[1]

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    ms = []
    for _ in range(steps):
        flush.fill_(1)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        step()
        e.record()
        torch.cuda.synchronize()
        ms.append(s.elapsed_time(e))
    med = float(np.median(ms))
    return {"value": ncol / (med * 1e-3), "unit": "columns/s", "ms_per_step": med,
            "what": "torch fp32: gather (cat) -> cuBLAS SGEMM + bias + activation per layer -> scatter (copy); library kernels, comparison only"}


# -----------------------------------------------------------------------------------------------------------------
def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import fortis_b200
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    wl = make_workload(args.workload, rank, args.ncol)
    prec = args.precision
    h = fortis_b200.Host()
    h.reset()
    is_conv = wl["kind"] == "conv"
    if not is_conv:
        h.configure(gather=wl["G"], scatter=wl["S"], loop=wl["Lp"], kdist=wl["K"])
    h.load_model(fortis_b200.write_blob(wl["layers"]))
    h.option("precision", prec)
    if is_conv:
        h.option("conv_shape", "%d,%d,%d,%d" % wl["shape"])
        h.option("graph", 1)                               # FORTIS_GRAPH: the 14 launches of a step replay as one graph
    h.option("checksum", 1)
    h.option("async", 1)
    stream = torch.cuda.ExternalStream(h.stream())
    to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a.reshape(-1, order="F"))).cuda()
    d_in = [to_dev(a) for a in wl["gin"]]
    d_out = [to_dev(a) for a in wl["sout"]]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")     # > 126 MB L2

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for s, e in ev:
            flush.fill_(1)                       # L2 flush between timed iterations (outside the event pair)
            torch.cuda.synchronize()
            s.record(stream)
            fn()
            e.record(stream)
        barrier()
        ms = [s.elapsed_time(e) for s, e in ev]
        total = float(sum(ms))
        if dist is not None:
            t = torch.tensor([total], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            total = float(t.item())
        return total, ms

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    if is_conv:
        h.L.mlp_upload(wl["gin"][0].ctypes.data)           # input resident in HBM; every step runs the whole network
        step_fn = lambda: h.L.mlp_forward_dev()
    else:
        step_fn = lambda: h.step(d_in, d_out)
    total_ms, per = timed(step_fn, args.steps, max(3, args.warmup))
    clocks = sampler.stop() if sampler else None
    status = h.L.fortis_device_status()
    if status != 0:
        raise SystemExit("device status %d: a bounded wait in the tensor-core kernel gave up" % status)
    cs_local = h.step_checksum() if not is_conv else 0.0
    if is_conv:
        h.L.mlp_download(wl["sout"][0].ctypes.data)
        cs_local = float(wl["sout"][0].astype(np.float64).sum())
    units = wl["units"] * world
    value = units * args.steps / (total_ms * 1e-3)
    kernel_ms = float(np.median(per))

    e2e = None
    if not args.no_e2e:
        # host arrays: the library pins them once, then every step copies all inputs H2D and all outputs D2H
        h.option("async", 0)
        e_steps = max(3, min(args.steps, 20))
        e_fn = (lambda: h.forward(wl["gin"][0], wl["sout"][0])) if is_conv else (lambda: h.step(wl["gin"], wl["sout"]))
        e_total, _ = timed(e_fn, e_steps, 3)
        e2e = {"value": units * e_steps / (e_total * 1e-3), "unit": "columns/s",
               "h2d_bytes_per_step": int(sum(a.nbytes for a in wl["gin"])), "d2h_bytes_per_step": int(sum(a.nbytes for a in wl["sout"]))}
    incumbent = None
    if wl["kind"] == "column" and world == 1 and not args.no_incumbent and wl["units"] <= 1 << 18:
        incumbent = time_incumbent(torch, wl, d_in, d_out, flush)
    cs_global = cs_local
    if dist is not None:
        t = torch.tensor([cs_local], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)               # the one collective: per-rank checksums
        cs_global = float(t.item())

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        kind = wl["kind"]
        if kind == "stencil":
            peak, src = (peaks.get("hbm_gbs"), "measured") if peaks.get("hbm_gbs") else (6650.0, "fallback")
            ach = wl["units"] * BYTES_PER_COL[kind] / (kernel_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_source": src}
        else:
            peak, src = (peaks.get("bf16_tflops"), "measured burst") if peaks.get("bf16_tflops") else (1590.0, "fallback")
            ach = wl["units"] * FLOP_PER_COL[kind] / (kernel_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s", "frac": ach / peak, "peak_source": src}
        traffic = None
        try:
            traffic = json.load(open(os.path.join(ROOT, "profiles", "ncu_traffic.json"))).get("%s_%s" % (args.workload, prec))
        except Exception:
            pass
        roof["traffic"] = traffic
        roof["kernel_ms"] = kernel_ms
        cpu = None if (args.no_cpu or is_conv or world > 1) else time_cpu(wl)      # the CPU baseline is an N = 1 figure
        launches_per_step = (len(wl["layers"]) + (1 if prec != "fp32" else 0)) if is_conv else 2 if (prec != "fp32" or kind == "stencil") else (2 + len(wl["layers"]))
        line = {"metric": "fused-step columns/sec", "value": value, "unit": "columns/s", "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": {"bf16": "bf16", "fp32": "f32", "fp8w": "bf16 (fp8-e4m3 weights)"}[prec],
                "data": "synthetic",
                "config": {"workload": wl["label"], "columns_per_gpu": wl["units"], "precision": prec, "l2": "flushed between timed steps (256 MB write)",
                           "parallelism": "contiguous column block per rank, no data-path collective"},
                "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "roofline": roof, "cpu_baseline": cpu,
                "incumbent_gpu_library_path": incumbent, "clocks": clocks, "checksum": cs_global}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
