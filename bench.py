#!/usr/bin/env python
"""Throughput bench of the batched articulated step.

    python bench.py --gpus N --steps K --warmup W          (torchrun launches it for N > 1)
    python bench.py --impl reference ...                   (the CPU arm: the oracle on the host cores)

A "step" is one physics step of every env of the workload.  N = 1 runs the 4096-env quadruped
(BASELINE.json configs[1]); N > 1 gives every rank its own 4096-env shard (weak scaling, no data-path
collective) and all-gathers the packed observations after every step (configs[4]'s exchange).
Prints one JSON line on rank 0.
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
sys.path.insert(0, os.path.join(ROOT, "nuka-physics_b200"))

ENVS_PER_GPU = 4096
METRIC = "env-steps/sec (whole box) 4096-env 12-DoF quadruped"
WORKLOAD = "quadruped (13 links, 18 DoF, 4 foot spheres + trunk box on a plane), configs[1], hold drives at the standing pose"
# algorithmic bytes per env-step: B = 12 nj + 52 F + 8 nj + 52 F + 52 L + 8 (nj + 3 P) + 8 S + 32 P
NJ, NF, NL = 12, 1, 13


def algorithmic_bytes(slots, points, free_bodies=0):
    return 12 * NJ + 52 * NF + 8 * NJ + 52 * NF + 52 * NL + 104 * free_bodies + 8 * (NJ + 3 * points) + 8 * slots + 32 * points


def hbm_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._halt = index, [], set(), None, threading.Event()

    def run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def _run_nvml(self):
        # read-only NVML queries; the device is addressed by its UUID so CUDA_VISIBLE_DEVICES remapping cannot mislead it
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


def run_reference(args):
    """CPU arm: the reference has no CPU implementation of this path, so the oracle port is timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orc
    from nuka import templates as T
    sample_envs = 512
    tb = T.quadruped(0)
    w = orc.World(tb.blob(), sample_envs)
    st = T.quadruped_state(sample_envs, 0)
    w.set("q", st["q"]); w.set("base_pose", st["base_pose"]); w.refresh()
    threads = orc.lib().orc_hw_threads()
    for _ in range(args.warmup):
        w.step(1, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        w.step(1, threads)
    dt = time.perf_counter() - t0
    value = sample_envs * args.steps / dt
    sample = f"{sample_envs} of {ENVS_PER_GPU} envs per step, {args.steps} steps, OpenMP over envs"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "env-steps/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3 * ENVS_PER_GPU / sample_envs, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "envs_per_gpu": ENVS_PER_GPU, "dt": 1.0 / 200.0, "velocity_iterations": 4,
                   "note": "CPU oracle port on the host cores, bounded sample per step"},
        "cpu_baseline": {"value": value, "unit": "env-steps/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "env-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def cpu_baseline():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import orc
    from nuka import templates as T
    envs, steps = 512, 40
    w = orc.World(T.quadruped(0).blob(), envs)
    st = T.quadruped_state(envs, 0)
    w.set("q", st["q"]); w.set("base_pose", st["base_pose"]); w.refresh()
    threads = orc.lib().orc_hw_threads()
    w.step(5, threads)
    t0 = time.perf_counter()
    w.step(steps, threads)
    dt = time.perf_counter() - t0
    return {"value": envs * steps / dt, "unit": "env-steps/s", "cores": threads, "kind": "port",
            "sample": f"{envs} of {ENVS_PER_GPU} envs x {steps} steps of the same workload, OpenMP over envs"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    # defaults follow the reference's own harness for this metric: 100 warm-up + 1000 timed steps with hold drives
    # (tests/perf/test_go2_4096env_step_time.cpp)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=100)
    ap.add_argument("--impl", default="native")
    ap.add_argument("--envs", type=int, default=ENVS_PER_GPU)
    ap.add_argument("--no-flush", action="store_true", help="skip the L2 flush between timed steps")
    ap.add_argument("--no-gather", action="store_true", help="N > 1: skip the per-step observation all-gather")
    ap.add_argument("--boxes", type=int, default=0,
                    help="free 0.1 m boxes beside each quadruped: 4 with --envs 8192 per GPU is configs[4]'s shard (not the headline workload)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import nuka
    from nuka import Field as F, templates as T

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    distributed = world_size > 1
    if distributed:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    E = args.envs
    dev = nuka.Device.create(local_rank)
    w = nuka.World.create_from_template(dev, T.quadruped(0, boxes=args.boxes).blob(), E)
    st = T.quadruped_state(E, seed=rank)
    w.upload(F.JOINT_POSITION, st["q"]); w.upload(F.BASE_POSE, st["base_pose"]); w.forward_kinematics()
    w.synchronize()
    stream_ptr = __import__("ctypes").c_void_p()
    nuka._check(nuka._abi.lib().nuka_world_get_stream(w._h, __import__("ctypes").byref(stream_ptr)))
    stream = torch.cuda.ExternalStream(stream_ptr.value, device=torch.device("cuda", local_rank))
    views = {f: w.view(f).torch() for f in (F.JOINT_POSITION, F.JOINT_VELOCITY, F.BASE_POSE, F.LINK_VELOCITY, F.DRIVE_TARGET)}
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device="cuda") if not args.no_flush else None
    obs_local = torch.empty((E, 49), dtype=torch.float32, device="cuda")
    obs_all = torch.empty((E * world_size, 49), dtype=torch.float32, device="cuda") if distributed else None

    from nuka import shard

    def one_step():
        w.step()
        if distributed and not args.no_gather:
            # 48 observation floats + 1 reward per env, gathered as the RL caller would
            w.pack_observations(obs_local)
            shard.gather_observations(obs_local, obs_all)

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            one_step()
        stream.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()
        launches0 = w.launch_count()
        sampler = ClockSampler(local_rank)
        sampler.start()
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
        for k in range(args.steps):
            if flush is not None:
                flush.add_(1.0)                       # evicts the 126 MB L2 between timed steps (outside the timed spans)
            starts[k].record(stream)
            one_step()
            ends[k].record(stream)
        stream.synchronize()
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        clocks = sampler.stop()
        gpu_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))
        launches = w.launch_count() - launches0
        # contact statistics of the timed window's last step
        w.synchronize()
        counts = w.download(F.CONTACT_COUNT)
        slots = float((counts > 0).sum(axis=1).mean())
        points = float(counts.sum(axis=1).mean())
        # ---- end to end: host targets in, host observations out, through the public API ----
        targets = torch.from_numpy(w.download(F.DRIVE_TARGET)).pin_memory()
        out_q = torch.empty((E, 13), dtype=torch.float32).pin_memory()
        out_b = torch.empty((E, 7), dtype=torch.float32).pin_memory()
        lib = nuka._abi.lib()

        def e2e_step():
            nuka._check(lib.nuka_world_upload_field(w._h, int(F.DRIVE_TARGET), targets.data_ptr(), targets.numel() * 4, 0))
            one_step()
            nuka._check(lib.nuka_world_download_field(w._h, int(F.JOINT_POSITION), out_q.data_ptr(), out_q.numel() * 4, 0))
            nuka._check(lib.nuka_world_download_field(w._h, int(F.BASE_POSE), out_b.data_ptr(), out_b.numel() * 4, 0))

        for _ in range(3):
            e2e_step()
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        e2e_steps = max(10, args.steps // 4)
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        e2e_s = time.perf_counter() - t0
    times = torch.tensor([gpu_ms, e2e_s * 1e3 / e2e_steps * args.steps], dtype=torch.float64, device="cuda")
    if distributed:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    gpu_ms, e2e_ms = float(times[0]), float(times[1])
    if rank == 0:
        total_envs = E * world_size
        value = total_envs * args.steps / (gpu_ms * 1e-3)
        e2e_value = total_envs * args.steps / (e2e_ms * 1e-3)
        peak, peak_kind = hbm_peak()
        bytes_per = algorithmic_bytes(slots, points, args.boxes)
        achieved = bytes_per * E * args.steps / (gpu_ms * 1e-3) / 1e9
        traffic, issue = None, None
        try:
            with open(os.path.join(ROOT, "profiles", "step_kernel_quadruped_traffic.txt")) as f:
                captured = json.load(f)
            if args.boxes:
                raise ValueError("the capture is of the headline workload")
            traffic = captured.get("dram_bytes_per_launch_4096_envs")
            # the bound that explains this kernel: warp instructions issued per second (instruction count of one
            # captured 4096-env launch, scaled by envs) against one instruction per scheduler per cycle
            instructions = captured.get("warp_instructions_per_launch_4096_envs")
            if instructions and clocks.get("sm_mhz"):
                issued = instructions / 4096.0 * E * args.steps / (gpu_ms * 1e-3)
                issue_peak = 148 * 4 * clocks["sm_mhz"] * 1e6
                issue = {"achieved": issued / 1e9, "peak": issue_peak / 1e9, "unit": "G warp-instructions/s",
                         "frac": issued / issue_peak, "note": "148 SMs x 4 schedulers x SM clock; instruction count from the ncu capture"}
        except Exception:
            pass
        line = {
            "metric": METRIC, "value": value, "unit": "env-steps/s", "n_gpus": world_size, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": gpu_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD if not args.boxes else WORKLOAD.replace("configs[1]", f"configs[4]'s env: + {args.boxes} free 0.1 m boxes"),
                       "envs_per_gpu": E, "dt": 1.0 / 200.0, "velocity_iterations": 4, "l2_flush_between_steps": flush is not None,
                       "obs_allgather": distributed and not args.no_gather, "mean_contact_slots": slots, "mean_contact_points": points},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_kind, "algorithmic_bytes_per_env_step": bytes_per,
                         "kernel": "step_kernel", "kernel_ms": gpu_ms / args.steps, "issue": issue},
            "e2e": {"value": e2e_value, "unit": "env-steps/s", "h2d_bytes_per_step": int(targets.numel() * 4),
                    "d2h_bytes_per_step": int(out_q.numel() * 4 + out_b.numel() * 4)},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if world_size == 1:
            line["cpu_baseline"] = cpu_baseline()
        print(json.dumps(line))
    w.destroy()
    dev.destroy()
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
