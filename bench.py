#!/usr/bin/env python
"""Throughput bench of the batched articulated step.

    python bench.py --gpus N --steps K --warmup W          (torchrun launches it for N > 1)
    python bench.py --impl reference ...                   (the CPU arm: the oracle port on all host cores)

A "step" is one physics step of every env of the workload: 4096 quadrupeds per GPU (BASELINE.json configs[1]).
N > 1 gives every rank its own 4096-env shard (weak scaling, no collective in the step); every `--exchange-every` steps (4,
the decimation at which the reference's gym env composes observations) each rank packs observation + reward records
straight into its slice of one of two gather buffers, and the in-place all-gather of that buffer runs on a side stream
under the next step (configs[4]'s exchange, double-buffered; the last gather of a timed run is added as a tail).

State preparation.  The cost of a step depends on what the robots are doing: while they drop onto their feet the solver
runs all its sweeps, once they stand it stops early.  So both arms first run `config.settle_steps` untimed steps from
the seeded start, and every figure below is measured on that prepared state:
    value    drives hold the standing pose (the reference gate's protocol, tests/perf/test_go2_4096env_step_time.cpp)
    active   every step gets fresh drive targets (standing pose + noise), as an RL caller's policy would write them
    e2e      value's workload through the C ABI with host buffers: pinned-host targets uploaded, step, observations
             (q and base pose) downloaded, wall clock per step with the same L2 flush between steps
Prints one JSON line on rank 0.
"""
import argparse
import ctypes
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "nuka-physics_b200"))

ENVS_PER_GPU = 4096
SETTLE_STEPS = 1000
METRIC = "env-steps/sec (whole box) 4096-env 12-DoF quadruped"
WORKLOAD = "quadruped (13 links, 18 DoF, 4 foot spheres + trunk box on a plane), configs[1]"
NJ, NF, NL = 12, 1, 13
ACTIVE_NOISE = 0.15          # rad, standard deviation of the per-step target noise of the `active` figure
ACTIVE_POOL = 16             # distinct target sets cycled through


def algorithmic_bytes(slots, points, free_bodies=0):
    """Compulsory bytes per env-step: q, qdot, target, base pose + twist in; q, qdot, base out; link pose + velocity out;
    free bodies in + out; warm-start multipliers in + out; contact ids and points out."""
    return 12 * NJ + 52 * NF + 8 * NJ + 52 * NF + 52 * NL + 104 * free_bodies + 8 * (NJ + 3 * points) + 8 * slots + 32 * points


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs (read-only queries)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._halt = index, [], set(), None, threading.Event()

    def run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def _run_nvml(self):
        # the device is addressed by its UUID so CUDA_VISIBLE_DEVICES remapping cannot mislead it
        import pynvml as nv
        import torch
        nv.nvmlInit()
        uuid = "GPU-" + str(torch.cuda.get_device_properties(self.index).uuid).replace("GPU-", "")
        h = nv.nvmlDeviceGetHandleByUUID(uuid)
        self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
        masks = {"hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40, "sw_power_cap": 0x4}
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self._halt.is_set():
            self.samples.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
            bits = int(get_reasons(h))
            for name, mask in masks.items():
                if bits & mask:
                    self.reasons.add(name)
            self._halt.wait(0.02)

    def _run_smi(self):
        q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
            "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._halt.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip().split(",")
                self.samples.append(float(out[0]))
                self.max_mhz = float(out[1])
                for name, v in zip(names, out[2:]):
                    if "Active" in v and "Not" not in v:
                        self.reasons.add(name)
            except Exception:
                pass
            self._halt.wait(0.1)

    def stop(self):
        self._halt.set()
        self.join(timeout=5)
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


# ---- CPU legs: the oracle port (the reference has no CPU implementation of this path) ------------------------------------

def _oracle(native=True):
    """The oracle module bound to a build made for this machine (-O3 -march=native) when that compiles here."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orc
    path = orc.build_native() if native else None
    orc.lib(path)
    return orc, ("-O3 -march=native" if path else "-O2 -march=x86-64-v3")


def _time_oracle(world, threads, repeats, steps):
    """Median over `repeats` of the time of `steps` steps."""
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        world.step(steps, threads)
        times.append(time.perf_counter() - t0)
    return statistics.median(times), times


def run_reference(args):
    """`--impl reference`: the whole workload (all 4096 envs, same settle) on the host cores, rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from nuka import templates as T
    orc, flags = _oracle()
    E = ENVS_PER_GPU
    w = orc.World(T.quadruped(0).blob(), E)
    st = T.quadruped_state(E, 0)
    w.set("q", st["q"]); w.set("base_pose", st["base_pose"]); w.refresh()
    threads = orc.lib().orc_hw_threads()
    t0 = time.perf_counter()
    w.step(args.settle, threads)
    settle_s = time.perf_counter() - t0
    w.step(args.warmup, threads)
    repeats = 5
    per_repeat = max(1, args.steps // repeats)
    median, times = _time_oracle(w, threads, repeats, per_repeat)
    value = E * per_repeat / median
    sample = f"all {E} envs x {per_repeat} steps, median of {repeats} repeats, after {args.settle} settle + {args.warmup} warm-up steps, OpenMP over envs, {flags}"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "env-steps/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": median / per_repeat * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "envs_per_gpu": E, "dt": 1.0 / 200.0, "velocity_iterations": 4, "settle_steps": args.settle,
                   "drives": "hold the standing pose", "settle_seconds": settle_s,
                   "note": "CPU oracle port on the host cores; the reference has no CPU implementation of this path"},
        "cpu_baseline": {"value": value, "unit": "env-steps/s", "cores": threads, "kind": "port", "sample": sample,
                         "spread": [E * per_repeat / t for t in times]},
        "e2e": {"value": value, "unit": "env-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline(state):
    """The oracle on all host cores, seeded with the GPU run's prepared state (a bounded sample of the same workload)."""
    from nuka import templates as T
    orc, flags = _oracle()
    E = ENVS_PER_GPU
    w = orc.World(T.quadruped(0).blob(), E)
    for name, value in state.items():
        w.set(name, value)
    w.refresh()
    w.set("link_velocity", state["link_velocity"])
    threads = orc.lib().orc_hw_threads()
    w.step(60, threads)                      # rebuilds the contact cache and carried solver state the transfer does not hold
    median, times = _time_oracle(w, threads, 5, 6)
    return {"value": E * 6 / median, "unit": "env-steps/s", "cores": threads, "kind": "port",
            "sample": f"all {E} envs x 6 steps, median of 5 repeats, started from this run's prepared state (+60 untimed steps), "
                      f"OpenMP over envs, {flags}",
            "spread": [E * 6 / t for t in times]}


def fp32_peak(device_index):
    """Register-resident FMA rate of this GPU in TFLOP/s (csrc/probe/fp32_peak.cu), or None."""
    try:
        from nuka import _build
        lib = ctypes.CDLL(_build.build_probe())
        tflops, ms = ctypes.c_float(), ctypes.c_float()
        if lib.nkb_probe_fp32_peak(int(device_index), 5, ctypes.byref(tflops), ctypes.byref(ms)) != 0:
            return None
        return float(tflops.value)
    except Exception:
        return None


def captured_counters():
    """Per-launch counters of one ncu capture of the step kernel on the prepared state (profiles/), or {}."""
    try:
        with open(os.path.join(ROOT, "profiles", "step_kernel_quadruped_counters.txt")) as f:
            return json.load(f)
    except Exception:
        return {}


OTHER_WORKLOADS = {
    # name: (description, default envs per GPU, settle steps, template, state, upload fields, (nj, F, L, free bodies))
    "c1": ("configs[0]: 7-link fixed-base arm, no contacts, dt 1/500", 4096, 200, lambda T: T.arm7(0), lambda T, E, s: T.arm7_state(E, s), (7, 0, 8, 0)),
    "c3": ("configs[2]: 35-coordinate humanoid, capsules, ground + limb self-contact, dt 1/200, 8 iterations", 8192, 300,
           lambda T: T.humanoid(0), lambda T, E, s: T.humanoid_state(E, s), (29, 1, 30, 0)),
    "c4": ("configs[3]: 48 free boxes on a plane, dt 1/240, 8 iterations", 16384, 240,
           lambda T: T.box_pile(0), lambda T, E, s: T.box_pile_state(E, s), (0, 0, 0, 48)),
    "c5": ("configs[4]'s shard: quadruped + 4 free 0.1 m boxes, dt 1/200, 4 iterations", 8192, 300,
           lambda T: T.quadruped(0, boxes=4), lambda T, E, s: T.quadruped_state(E, s), (12, 1, 13, 4)),
}


def run_other_workload(args):
    """`--workload c1|c3|c4|c5`: the other configurations of BASELINE.json on one GPU, device-timed on a prepared state.
    They are parity-test configurations, not the headline; the line has the same keys minus the CPU and end-to-end legs."""
    import torch
    import nuka
    from nuka import Field as F, templates as T
    text, default_envs, settle, make, state, (nj, nf, nl, nb) = OTHER_WORKLOADS[args.workload]
    E = args.envs if args.envs != ENVS_PER_GPU else default_envs
    settle = args.settle if args.settle != SETTLE_STEPS else settle
    dev = nuka.Device.create(0)
    tb = make(T)
    w = nuka.World.create_from_template(dev, tb.blob(), E)
    names = {"q": F.JOINT_POSITION, "qdot": F.JOINT_VELOCITY, "base_pose": F.BASE_POSE, "body_pose": F.RIGID_BODY_TRANSFORM}
    for k, v in state(T, E, 0).items():
        w.upload(names[k], v)
    w.forward_kinematics()
    w.set_contact_readout(False)
    ptr = ctypes.c_void_p()
    nuka._check(nuka._abi.lib().nuka_world_get_stream(w._h, ctypes.byref(ptr)))
    stream = torch.cuda.ExternalStream(ptr.value)
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device="cuda")
    t0 = time.perf_counter()
    with torch.cuda.stream(stream):
        w.step_n(settle)
        stream.synchronize()
        settle_s = time.perf_counter() - t0
        for _ in range(args.warmup):
            w.step()
        stream.synchronize()
        sampler = ClockSampler(0)
        sampler.start()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        for k in range(args.steps):
            flush.add_(1.0)
            starts[k].record(stream)
            w.step()
            ends[k].record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        w.set_contact_readout(True)
        w.step()
    w.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in zip(starts, ends)) / args.steps
    counts = w.download(F.CONTACT_COUNT) if tb.cfg["max_contacts"] else np.zeros((E, 1), np.uint32)
    slots, points = float((counts > 0).sum(axis=1).mean()), float(counts.sum(axis=1).mean())
    flags = w.download(F.ENV_STATUS).reshape(-1)
    status, flagged = int(np.bitwise_or.reduce(flags)), int((flags != 0).sum())
    info = w.info
    bytes_per = 12 * nj + 52 * nf + 8 * nj + 52 * nf + 52 * nl + 104 * nb + 8 * (nj + 3 * points) + 8 * slots + 32 * points
    peak, peak_kind = hbm_peak()
    value = E / (ms * 1e-3)
    print(json.dumps({
        "metric": f"env-steps/sec, {args.workload}", "value": value, "unit": "env-steps/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": text, "envs_per_gpu": E, "dt": float(info.fixed_dt), "velocity_iterations": int(tb.cfg["vel_iters"]),
                   "settle_steps": settle, "settle_seconds": settle_s, "l2_flush_between_steps": True, "mean_contact_slots": slots,
                   "mean_contact_points": points, "shared_bytes_per_env": int(info.shared_bytes_per_env), "status_or": status, "envs_with_status": flagged},
        "roofline": {"bound": "hbm", "achieved": bytes_per * value / 1e9, "peak": peak, "unit": "GB/s", "frac": bytes_per * value / 1e9 / peak,
                     "traffic": None, "peak_source": peak_kind, "algorithmic_bytes_per_env_step": bytes_per, "kernel": "step_kernel", "kernel_ms": ms},
        "gpu_launches": args.steps, "clocks": clocks}))
    w.destroy()
    dev.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="native")
    ap.add_argument("--envs", type=int, default=ENVS_PER_GPU)
    ap.add_argument("--settle", type=int, default=SETTLE_STEPS, help="untimed steps from the seeded start that prepare the measured state")
    ap.add_argument("--no-flush", action="store_true", help="skip the L2 flush between timed steps")
    ap.add_argument("--no-gather", action="store_true", help="N > 1: skip the observation all-gather")
    ap.add_argument("--exchange-every", type=int, default=4,
                    help="N > 1: physics steps per observation exchange; 4 is the decimation of the reference's gym env, which composes "
                         "observations once per step_n(decimation) (python/nuka/gym/env.py:98, 255-256)")
    ap.add_argument("--no-extra", action="store_true", help="skip the configs[4] figure (65536 quadruped + 4-box envs split over the ranks)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--workload", default="c2", choices=["c2"] + sorted(OTHER_WORKLOADS),
                    help="c2 is the headline (configs[1]); the others are single-GPU lines of the parity configurations")
    ap.add_argument("--boxes", type=int, default=0,
                    help="free 0.1 m boxes beside each quadruped: 4 with --envs 8192 per GPU is configs[4]'s shard (not the headline workload)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload != "c2":
        run_other_workload(args)
        return
    import torch
    import nuka
    from nuka import Field as F, shard, templates as T

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    cuda = torch.device("cuda", local_rank)
    distributed = world_size > 1
    gather = distributed and not args.no_gather
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=cuda)
    dev = nuka.Device.create(local_rank)
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=cuda) if not args.no_flush else None

    def make_world(E, boxes, seed):
        w = nuka.World.create_from_template(dev, T.quadruped(0, boxes=boxes).blob(), E)
        st = T.quadruped_state(E, seed=seed)
        w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
        w.set_contact_readout(False)            # the bench reads robot state only; contact statistics are taken once at the end
        w.synchronize()
        return w

    def stream_of(w):
        ptr = ctypes.c_void_p()
        nuka._check(nuka._abi.lib().nuka_world_get_stream(w._h, ctypes.byref(ptr)))
        return torch.cuda.ExternalStream(ptr.value, device=cuda)

    class Exchange:
        """Per-step observation + reward exchange of one world: the pack kernel writes this rank's records into its slice of
        one of two gather buffers (on the world's stream, inside the step's timed span); the in-place all-gather of that
        buffer runs on a side stream, released when the NEXT step starts, so it overlaps that step and not the L2 flush
        between the spans.  The last gather of a run is timed as a tail."""

        def __init__(self, w, E):
            self.w = w
            self.link = shard.ObservationExchange(E, world_size, rank, shard.RECORD_FLOATS, device=cuda)
            self.base = w.view(F.BASE_POSE).torch()
            self.reward = torch.zeros(E, dtype=torch.float32, device=cuda)
            self.command = torch.tensor([0.5, 0.0, 0.0], dtype=torch.float32, device=cuda)
            self.last_action = torch.zeros((E, NJ), dtype=torch.float32, device=cuda)
            self.desc = w.observation_desc(self.command, last_action=self.last_action, reward=self.reward, row_stride=shard.RECORD_FLOATS)

        def pack(self, stream):
            self.reward.copy_(self.base[:, 2])           # the caller's reward: base height
            self.w.pack_observations(self.desc, self.link.pack_target(stream))
            self.link.packed_on(stream)

        def release(self, after=None):
            self.link.gather(after)

        def drain(self, stream):
            """Issues what is pending and orders `stream` behind it."""
            self.link.gather()
            self.link.wait(stream)

    def timed(w, stream, steps, warmup, before_step=None, exchange=None):
        """`warmup` untimed then `steps` timed steps; per-step CUDA events on the world's stream, L2 flushed between steps
        outside the timed spans.  Returns the per-step times in ms (the exchange's tail added to the last) and the kernel
        launches inside the timed steps."""
        def one(k, start=None):
            if before_step is not None:
                before_step(k)
            w.step()
            if exchange is not None:
                # a packed buffer's gather runs under the step after its pack: enqueued after that step's launch, so that
                # the host's time in the NCCL call passes while the step kernel runs, and held back on the device until
                # the step's start event (nothing happens here when no buffer is pending)
                exchange.release(after=start)
                if (k + 1) % args.exchange_every == 0:
                    exchange.pack(stream)
        with torch.cuda.stream(stream):
            for k in range(warmup):
                one(k)
            if exchange is not None:
                exchange.drain(stream)
            # everything that takes host time happens before the ranks line up: events, the collector, the first use of
            # the flush kernel (its module load would otherwise delay a rank's first timed launch)
            if flush is not None:
                flush.add_(1.0)
            starts = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
            ends = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
            gc.collect()
            gc.disable()                                  # no collector pause between a start event and its step's launch
            stream.synchronize()
            torch.cuda.synchronize()
            launches0 = w.launch_count()
            if distributed:
                dist.barrier()
                torch.cuda.synchronize()
            for k in range(steps):
                if flush is not None:
                    flush.add_(1.0)                       # evicts the 126 MB L2 (outside the timed spans)
                starts[k].record(stream)
                one(warmup + k, starts[k])
                ends[k].record(stream)
            starts[steps].record(stream)                  # tail: the last step's gather, with nothing to hide under
            if exchange is not None:
                exchange.drain(stream)
            ends[steps].record(stream)
            gc.enable()
            stream.synchronize()
            torch.cuda.synchronize()
            if distributed:
                dist.barrier()
        times = [s.elapsed_time(e) for s, e in zip(starts[:steps], ends[:steps])]
        if exchange is not None:
            times[-1] += starts[steps].elapsed_time(ends[steps])
        return times, w.launch_count() - launches0

    def max_over_ranks(values):
        t = torch.tensor(values, dtype=torch.float64, device=cuda)
        if distributed:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t]

    # ---- the headline workload ----------------------------------------------------------------------------------------
    E = args.envs
    w = make_world(E, args.boxes, seed=rank)
    stream = stream_of(w)
    exchange = Exchange(w, E) if gather else None
    if gather:
        with torch.cuda.stream(stream):          # NCCL's first-use cost (channel set-up, registration) lands here, not in the timed steps
            for _ in range(20):
                exchange.pack(stream)
                exchange.release()
            exchange.drain(stream)
        stream.synchronize()
        torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        w.step_n(args.settle)
    stream.synchronize()
    sampler = ClockSampler(local_rank)
    sampler.start()
    hold_ms, launches = timed(w, stream, args.steps, args.warmup, exchange=exchange)
    clocks = sampler.stop()
    # contact statistics of the measured (hold) state
    with torch.cuda.stream(stream):
        w.set_contact_readout(True)
        w.step()
    w.synchronize()
    counts = w.download(F.CONTACT_COUNT)
    slots = float((counts > 0).sum(axis=1).mean())
    points = float(counts.sum(axis=1).mean())
    sweeps = float(w.download(F.SOLVER_SWEEPS).mean())
    w.set_contact_readout(False)

    # ---- end to end through the C ABI with host buffers, on the same hold state -----------------------------------------
    lib = nuka._abi.lib()
    targets = torch.from_numpy(w.download(F.DRIVE_TARGET)).pin_memory()
    out_q = torch.empty((E, NL), dtype=torch.float32).pin_memory()
    out_b = torch.empty((E, 7), dtype=torch.float32).pin_memory()

    e2e_count = [0]

    def e2e_step():
        nuka._check(lib.nuka_world_upload_field(w._h, int(F.DRIVE_TARGET), targets.data_ptr(), targets.numel() * 4, 0))
        w.step()
        if exchange is not None:
            exchange.release()                   # a packed buffer's gather runs under the step after its pack
            e2e_count[0] += 1
            if e2e_count[0] % args.exchange_every == 0:
                with torch.cuda.stream(stream):
                    exchange.pack(stream)
        nuka._check(lib.nuka_world_download_field(w._h, int(F.JOINT_POSITION), out_q.data_ptr(), out_q.numel() * 4, 0))
        nuka._check(lib.nuka_world_download_field(w._h, int(F.BASE_POSE), out_b.data_ptr(), out_b.numel() * 4, 0))

    for _ in range(3):
        e2e_step()
    e2e_steps = max(10, args.steps // 4)
    e2e_s = 0.0
    for _ in range(e2e_steps):
        if flush is not None:
            flush.add_(1.0)
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        t0 = time.perf_counter()
        e2e_step()                               # the downloads synchronise: the step's results are on the host when it returns
        e2e_s += time.perf_counter() - t0
    if exchange is not None:                     # the last step's gather, timed with nothing to hide under
        t0 = time.perf_counter()
        with torch.cuda.stream(stream):
            exchange.drain(stream)
        stream.synchronize()
        e2e_s += time.perf_counter() - t0
    # active drives: each step copies one of a pool of target sets (standing pose + noise) into DRIVE_TARGET on the stream
    targets_view = w.view(F.DRIVE_TARGET).torch()
    hold_targets = targets_view.clone()
    gen = torch.Generator(device=cuda).manual_seed(1234 + rank)
    pool = [hold_targets + ACTIVE_NOISE * torch.randn(hold_targets.shape, generator=gen, device=cuda) for _ in range(ACTIVE_POOL)]
    for p in pool:
        p[:, 0] = hold_targets[:, 0]
    active_steps = max(10, args.steps // 2)
    active_ms, _ = timed(w, stream, active_steps, max(args.warmup, 10), before_step=lambda k: targets_view.copy_(pool[k % ACTIVE_POOL]), exchange=exchange)
    with torch.cuda.stream(stream):
        targets_view.copy_(hold_targets)

    hold_total, active_total, e2e_total = max_over_ranks([sum(hold_ms), sum(active_ms), e2e_s * 1e3])
    per_rank = None
    if distributed:
        mine = torch.tensor([min(hold_ms), statistics.median(hold_ms), max(hold_ms), float(hold_ms.index(max(hold_ms)))], dtype=torch.float64, device=cuda)
        every = [torch.zeros_like(mine) for _ in range(world_size)]
        dist.all_gather(every, mine)
        per_rank = [[round(float(v), 4) for v in t] for t in every]

    # the prepared state, for the CPU baseline leg (rank 0, N = 1 only)
    prepared = None
    if rank == 0 and world_size == 1 and not args.no_cpu and not args.boxes and E == ENVS_PER_GPU:
        prepared = {"q": w.download(F.JOINT_POSITION), "qdot": w.download(F.JOINT_VELOCITY), "base_pose": w.download(F.BASE_POSE),
                    "link_velocity": w.download(F.LINK_VELOCITY), "drive_target": w.download(F.DRIVE_TARGET)}
    if exchange is not None:
        with torch.cuda.stream(stream):
            exchange.drain(stream)
        torch.cuda.synchronize()
    w.destroy()

    # ---- configs[4]: 65536 envs of quadruped + 4 free boxes split evenly over the ranks, same exchange ---------------------
    extra = None
    if not args.no_extra and not args.boxes:
        total = 65536
        Ex = total // world_size
        wx = make_world(Ex, 4, seed=100 + rank)
        sx = stream_of(wx)
        ex = Exchange(wx, Ex) if gather else None
        with torch.cuda.stream(sx):
            wx.step_n(200)                        # boxes and robots land
        sx.synchronize()
        x_steps = 10
        x_ms, _ = timed(wx, sx, x_steps, 3, exchange=ex)
        (x_total,) = max_over_ranks([sum(x_ms)])
        torch.cuda.synchronize()
        wx.destroy()
        extra = {"workload": "configs[4]: 65536 envs of quadruped + 4 free 0.1 m boxes split evenly over the ranks, observation all-gather as in the headline run (double-buffered, under the next step)",
                 "scaling": "strong", "total_envs": total, "envs_per_gpu": Ex, "steps": x_steps, "settle_steps": 200,
                 "ms_per_step": x_total / x_steps, "value": total * x_steps / (x_total * 1e-3), "unit": "env-steps/s"}

    if rank == 0:
        total_envs = E * world_size
        value = total_envs * args.steps / (hold_total * 1e-3)
        active_value = total_envs * active_steps / (active_total * 1e-3)
        e2e_value = total_envs * e2e_steps / (e2e_total * 1e-3)
        peak, peak_kind = hbm_peak()
        bytes_per = algorithmic_bytes(slots, points, args.boxes)
        kernel_ms = hold_total / args.steps
        achieved = bytes_per * E * args.steps / (hold_total * 1e-3) / 1e9
        counters = captured_counters() if not args.boxes else {}
        issue = fp32 = None
        if counters.get("warp_instructions_per_env_step") and clocks.get("sm_mhz"):
            issued = counters["warp_instructions_per_env_step"] * value / world_size
            issue_peak = 148 * 4 * clocks["sm_mhz"] * 1e6
            issue = {"achieved": issued / 1e9, "peak": issue_peak / 1e9, "unit": "G warp-instructions/s", "frac": issued / issue_peak,
                     "note": "148 SMs x 4 schedulers x sampled SM clock; instruction count from the ncu capture named in `counters`"}
        peak_tflops = fp32_peak(local_rank)
        if counters.get("fp32_flop_per_env_step") and peak_tflops:
            flops = counters["fp32_flop_per_env_step"] * value / world_size
            fp32 = {"achieved": flops / 1e12, "peak": peak_tflops, "unit": "TFLOP/s", "frac": flops / 1e12 / peak_tflops,
                    "flop_per_env_step": counters["fp32_flop_per_env_step"],
                    "note": "executed FADD + FMUL + 2 FFMA of the captured launch (ncu thread-instruction counters) against the FMA rate "
                            "measured by csrc/probe/fp32_peak.cu in this run"}
        line = {
            "metric": METRIC, "value": value, "unit": "env-steps/s", "n_gpus": world_size, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": kernel_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD if not args.boxes else WORKLOAD.replace("configs[1]", f"configs[4]'s env: + {args.boxes} free 0.1 m boxes"),
                       "envs_per_gpu": E, "dt": 1.0 / 200.0, "velocity_iterations": 4, "settle_steps": args.settle,
                       "drives": "hold the standing pose", "l2_flush_between_steps": flush is not None,
                       "obs_allgather": f"every {args.exchange_every} steps (the gym env's decimation), double-buffered; issued on a side stream when the next step starts" if gather else False, "mean_contact_slots": slots, "mean_contact_points": points, "mean_solver_sweeps": sweeps},
            "active": {"value": active_value, "unit": "env-steps/s", "ms_per_step": active_total / active_steps, "steps": active_steps,
                       "drives": f"targets redrawn every step: standing pose + N(0, {ACTIVE_NOISE}) rad"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": counters.get("dram_bytes_per_launch"), "peak_source": peak_kind, "algorithmic_bytes_per_env_step": bytes_per,
                         "kernel": "step_kernel", "kernel_ms": kernel_ms, "issue": issue, "fp32": fp32,
                         "counters": counters.get("source")},
            "e2e": {"value": e2e_value, "unit": "env-steps/s", "ms_per_step": e2e_total / e2e_steps, "steps": e2e_steps,
                    "h2d_bytes_per_step": int(targets.numel() * 4), "d2h_bytes_per_step": int(out_q.numel() * 4 + out_b.numel() * 4)},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if per_rank is not None:
            line["per_rank_step_ms_min_median_max_slowest_step"] = per_rank
        if extra is not None:
            line["extra"] = extra
        if prepared is not None:
            line["cpu_baseline"] = cpu_baseline(prepared)
        print(json.dumps(line))
    dev.destroy()
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
