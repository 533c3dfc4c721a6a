"""Benchmark of the diffusion sampler: denoiser evaluations per second on the headline configuration
(512 tokens, 4096 atoms, 5 samples x 200 steps, bf16, seeded synthetic inputs).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one fold per GPU: every step of every sample of one seed, i.e. one launch of the
persistent sampler kernel (S x nsteps denoiser evaluations). With N GPUs (torchrun, one rank per
GPU) each rank folds its own seed with no data-path collective (weak scaling); coordinates are
gathered at the end. With --units K the job is K (seed, S) units dealt over the ranks instead
(strong scaling: 40 samples = 8 units of 5 on 1, 2, 4 or 8 GPUs). Rank 0 prints one JSON line.

`--impl reference` times the CPU restatement of the reference's math (oracle/) on the host cores:
the reference has no CPU implementation of this path and its JAX model is not part of its tree.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "colabfold-cuda-kernels_b200"))
from mkharness import driver, shard, synth  # noqa: E402

METRIC = "denoiser evals/sec at 512 tokens, 5 samples x 200 steps"
UNIT = "evals/s"


def fold_flops(N, A, S, nsteps, nb=24, cs=384, plc=128):
    per_eval = synth.flops_per_eval(N, A, S)  # includes the per-step conditioning shared by S samples
    np_ = (N + 63) // 64 * 64
    return S * nsteps * per_eval + 2 * np_ * np_ * plc * 16 * nb


# DRAM bytes of one launch at the headline shapes, from an ncu capture of a 2-step launch
# (dram__bytes_read.sum + dram__bytes_write.sum): once for the pair logits plus a part per sampling
# step, scaled to the launch's step count
TRAFFIC_ONCE_B, TRAFFIC_PER_STEP_B = 0.27e9, 2.05e9


def launch_traffic(N, S, nsteps):
    return TRAFFIC_ONCE_B + nsteps * TRAFFIC_PER_STEP_B if (N, S) == (512, 5) else None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        p = json.load(open(path))
        return float(p["bf16_tflops_sustained"]), float(p["hbm_gbs"]), "measured (MEASURED_PEAKS.json, sustained cuBLAS bf16)"
    return 1400.0, 6650.0, "fallback (earlier measurement on this pool, sustained)"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                                       "-lms", "200"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        self.p.wait()
        self.f.flush()
        rows = [r.split(", ") for r in open(self.f.name).read().strip().splitlines() if r.count(",") >= 8]
        os.unlink(self.f.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(float(r[1]) for r in rows)
        load = [float(r[1]) for r in rows if float(r[3]) > 300.0] or sm
        reasons = set()
        for r in rows:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(load)), "sm_max_mhz": float(rows[0][2]), "samples": len(rows),
                "power_w_max": max(float(r[3]) for r in rows), "reasons": sorted(reasons)}


def pin(arrays):
    """Page-lock the host arrays so that the library's host-to-device copies run at pinned speed."""
    import torch

    rt = torch.cuda.cudart()
    for a in arrays:
        if a.nbytes:
            rt.cudaHostRegister(a.ctypes.data, a.nbytes, 0)


def workload(meta, nsteps):
    """The workload's name: the same string in both arms."""
    tag = " (headline)" if (meta["N"], meta["S"], nsteps) == (512, 5, 200) else ""
    return "N_token=%d N_atom=%d samples=%d nsteps=%d%s" % (meta["N"], meta["A"], meta["S"], nsteps, tag)


def cpu_sample(x, meta, steps_timed=1):
    """The oracle on a bounded sample of the same workload: `steps_timed` sampling steps of all S
    samples after one untimed step (pair logits built, weights widened). Returns evals/s."""
    orc = driver.Oracle()
    orc.set_threads(0)  # every host core, whatever OMP_NUM_THREADS the launcher exported
    orc.setup(x, meta)
    orc.run(mode=0, nsteps=1, seed=0)
    t0 = time.time()
    orc.run(mode=0, nsteps=1 + steps_timed, seed=0)
    dt = time.time() - t0
    # the timed call reruns the warm step: count both
    evals = meta["S"] * (1 + steps_timed)
    threads = orc.lib.orc_threads()
    orc.teardown()
    return evals / dt, threads, "%d sampling steps x %d samples of the workload (%.1f s)" % (1 + steps_timed, meta["S"], dt)


def reference_arm(args, rank):
    """The CPU restatement as the reference arm: each step is one sampling step of all S samples."""
    if rank != 0:
        return
    x, meta = synth.make_inputs(args.tokens, samples=args.samples, steps=args.nsteps, seed=0)
    orc = driver.Oracle()
    threads = orc.set_threads(0)  # torchrun exports OMP_NUM_THREADS=1: take every host core all the same
    orc.setup(x, meta)
    for _ in range(max(args.warmup, 1)):
        orc.run(mode=0, nsteps=1, seed=0)
    t0 = time.time()
    for _ in range(args.steps):
        orc.run(mode=0, nsteps=1, seed=0)
    dt = time.time() - t0
    value = args.steps * meta["S"] / dt
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": workload(meta, args.nsteps),
                   "step": "bounded sample: one sampling step of all %d samples on the CPU" % meta["S"]},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "%d x (1 sampling step x %d samples)" % (args.steps, meta["S"])},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path; this is the CPU restatement of its math (oracle/), bf16-faithful mode",
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--tokens", type=int, default=512)
    ap.add_argument("--samples", type=int, default=5)
    ap.add_argument("--nsteps", type=int, default=200)
    ap.add_argument("--units", type=int, default=0, help="deal this many (seed, samples) units over the ranks (strong scaling); 0: one unit per rank")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-ref-kernel", action="store_true", help="skip the leg that times the reference's own CUDA kernel")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl != "reference" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        reference_arm(args, rank)
        return

    import torch
    import torch.distributed as dist

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    # every rank holds the replicated inputs; a unit is one (seed, S samples) fold, independent of the
    # others: rank r folds unit r (weak scaling), or with --units its share of K units, no exchange
    x, meta = synth.make_inputs(args.tokens, samples=args.samples, steps=args.nsteps, seed=0)
    lib = driver.MkLib()  # raises if the CUDA library is missing: there is no fallback
    pin(x)
    lib.setup(x, meta)
    S, N, A, nsteps = meta["S"], meta["N"], meta["A"], args.nsteps
    n_units = args.units if args.units > 0 else world
    mine = shard.deal_units(n_units, rank, world)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def fold(seed):
        ms = lib.run(mode=0, nsteps=nsteps, seed=seed)  # CUDA events on the launching stream
        return lib.read("POS").copy(), ms

    for _ in range(args.warmup):
        lib.run(mode=0, nsteps=nsteps, seed=1000 + rank)
    barrier()
    clocks = ClockSampler(local) if rank == 0 else None
    dev_ms = 0.0
    t0 = time.time()
    for _ in range(args.steps):
        done, ms = shard.fold_units(fold, mine, 1000)
        dev_ms += ms
    barrier()
    wall = time.time() - t0
    clk = clocks.stop() if clocks else None

    # end to end through the C ABI with host buffers: upload of all inputs, the folds, positions back
    h2d = sum(a.nbytes for a in x)
    d2h = sum(p.nbytes for p in done.values())
    barrier()
    e0 = time.time()
    e2e_steps = max(2, min(args.steps, 3))
    for _ in range(e2e_steps):
        lib.setup(x, meta)
        shard.fold_units(fold, mine, 1000)
    barrier()
    e2e_s = time.time() - e0

    # the reference's own CUDA kernel (its diffusion.cu compiled for sm_100 under oracle/_ref) on the
    # same inputs, seed and steps: the kernel to beat. Rank 0 of a single-GPU run only.
    ref_kernel = None
    if rank == 0 and world == 1 and not args.no_ref_kernel:
        if os.path.isfile(driver.REFERENCE_LIB):
            lib.teardown()
            try:
                ref = driver.MkLib(driver.REFERENCE_LIB)
                ref.setup(x, meta)
                ref.run(mode=0, nsteps=nsteps, seed=1000)
                rms = [ref.run(mode=0, nsteps=nsteps, seed=1000) for _ in range(2)]
                rpos = ref.read("POS")
                d = (done[mine[0]].ravel() - rpos.ravel()[: done[mine[0]].size]).reshape(-1, 3)
                ref_kernel = {"ms_per_fold": float(np.mean(rms)), "value": S * nsteps / (float(np.mean(rms)) * 1e-3), "unit": UNIT,
                              "folds_timed": 2, "rmsd_vs_this_library_A": float(np.sqrt((d ** 2).sum(-1).mean())),
                              "what": "the reference's diffusion.cu compiled unmodified for sm_100 (mma.sync), same inputs, seed and steps"}
                ref.teardown()
            except Exception as e:  # the record says why, the bench line stands
                ref_kernel = {"unavailable": "%s: %s" % (type(e).__name__, e)}
        else:
            ref_kernel = {"unavailable": "oracle/_ref/libref_sm100.so is not built on this machine"}

    # MAX over ranks of the device time; the coordinates of every unit gathered at the end
    allpos, dev_ms = shard.gather(done, dev_ms, n_units, rank, world, dist if world > 1 else None, device="cuda")
    t = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t[0])
    assert len(allpos) == n_units and all(a is not None and np.isfinite(a).all() for a in allpos)
    if rank == 0:
        evals = n_units * args.steps * S * nsteps
        value = evals / (dev_ms * 1e-3)
        flops = fold_flops(N, A, S, nsteps)
        peak, hbm, which = measured_peaks()
        per_rank = (n_units + world - 1) // world  # folds of the slowest rank in one step
        achieved = flops * per_rank / (dev_ms * 1e-3 / args.steps) / 1e12
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "strong" if args.units > 0 else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload(meta, nsteps),
                       "units": "%d (seed, %d samples) folds, %s" % (n_units, S, "dealt over the ranks" if args.units > 0 else "one per GPU"),
                       "step": "one fold = one persistent launch = %d denoiser evaluations; a step is every rank's share of the units" % (S * nsteps),
                       "l2": "inputs larger than L2: %d MB of weights and pair bias stream every sampling step" % (h2d >> 20),
                       "ms_per_fold": dev_ms / args.steps / per_rank, "wall_s": wall},
            "clocks": clk,
            "e2e": {"value": n_units * e2e_steps * S * nsteps / e2e_s, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": n_units * args.steps,
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "traffic": launch_traffic(N, S, nsteps), "traffic_unit": "bytes per launch (ncu 2-step capture, scaled by steps)",
                         "peak_source": which, "flops_per_launch": flops},
        }
        if ref_kernel is not None:
            line["ref_kernel"] = ref_kernel
        if not args.no_cpu and world == 1:
            v, cores, sample = cpu_sample(x, meta)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    lib.teardown()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
