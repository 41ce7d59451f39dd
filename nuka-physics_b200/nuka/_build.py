"""Builds the native library (CUDA kernels + C ABI) in-tree for sm_100a."""
import os
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
LIB_PATH = os.path.join(os.path.dirname(_HERE), "libnuka_b200.so")
SOURCES = ["nkb_step_n1.cu", "nkb_step_n1s.cu", "nkb_step_n1r.cu", "nkb_step_n2.cu", "nkb_step_n2r.cu",
           "nkb_step_n1c.cu", "nkb_step_n1rc.cu", "nkb_step_n2c.cu", "nkb_step_n2rc.cu", "nkb_kernels.cu", "nkb_static_reset.cu", "nkb_world.cpp", "nkb_scene.cpp", "nkb_abi.cpp"]
# nvcc defaults for floating point, as the reference builds its physics ops: IEEE division and square root, denormals
# kept, fused multiply-add on.  (Approximate division / square root and flush-to-zero for the whole library measured 4 %
# faster on the 4096-env quadruped step and changed no parity figure; the few places that use rsqrtf / __fdividef on
# purpose say so where they do.)
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]


def _stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if os.path.isfile(os.path.join(CSRC, f))] + [os.path.join(os.path.dirname(os.path.dirname(_HERE)), "include", "nuka_b200.h")]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build_native(force=False, verbose=False):
    """Compiles every source with nvcc and links libnuka_b200.so next to the package."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    flags = list(NVCC_FLAGS)
    if os.environ.get("NUKA_B200_STAGE_TAPS") == "1":       # profiling build: per-stage cycle counters in the step kernel
        flags.append("-DNKB_STAGE_TAPS")
    objects = []
    procs = []
    for src in SOURCES:
        obj = os.path.join(CSRC, src.rsplit(".", 1)[0] + ".o")
        cmd = [nvcc, *flags, "-c", os.path.join(CSRC, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(obj)
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
        if verbose and out:
            print(out)
    subprocess.run([nvcc, "-shared", "-o", LIB_PATH, *objects, "-Xcompiler", "-fPIC"], check=True)
    return LIB_PATH


PROBE_PATH = os.path.join(os.path.dirname(_HERE), "libnkb_probe.so")


def build_probe(force=False):
    """Compiles the measurement aid used by the bench report (csrc/probe/fp32_peak.cu) into libnkb_probe.so."""
    src = os.path.join(CSRC, "probe", "fp32_peak.cu")
    if not force and os.path.exists(PROBE_PATH) and os.path.getmtime(PROBE_PATH) >= os.path.getmtime(src):
        return PROBE_PATH
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
                    src, "-o", PROBE_PATH], check=True, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    return PROBE_PATH


if __name__ == "__main__":
    print(build_native(force=True, verbose=True))
