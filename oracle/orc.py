"""ctypes binding of the CPU oracle (test infrastructure; never imported by the shipped package)."""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


REFERENCE_CHECKOUT = os.environ.get("NUKA_REFERENCE_CHECKOUT", "/root/reference")


def build():
    """Builds the restatement (portable and contraction-free variants) and, where the reference checkout is present,
    the binding of the reference's own headers (oracle/_ref)."""
    subprocess.run(["make", "-C", _HERE, "liborc.so", "liborc_strict.so"], check=True, stdout=subprocess.DEVNULL)
    if os.path.isdir(os.path.join(REFERENCE_CHECKOUT, "src")):
        subprocess.run(["make", "-C", _HERE, "_ref/libref_headers.so", f"REF={REFERENCE_CHECKOUT}"], check=True, stdout=subprocess.DEVNULL)


def build_native():
    """-O3 -march=native build for the machine that times the CPU baseline; returns its path or None."""
    done = subprocess.run(["make", "-C", _HERE, "liborc_native.so"], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    path = os.path.join(_HERE, "liborc_native.so")
    return path if done.returncode == 0 and os.path.exists(path) else None


def _declare_kat(L, prefix):
    f = getattr(L, prefix + "_manifold_frames")
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p,
                  ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p]
    g = getattr(L, prefix + "_law_batch")
    g.restype = None
    g.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32, ctypes.c_void_p, ctypes.c_uint32]
    return L


def strict_lib():
    """The restatement compiled without floating-point contraction (differential tests)."""
    path = os.path.join(_HERE, "liborc_strict.so")
    if not os.path.exists(path):
        build()
    return _declare_kat(ctypes.CDLL(path), "orc")


def ref_lib():
    """The reference's own headers behind a C binding, or None where neither the built file nor the checkout exists."""
    path = os.path.join(_HERE, "_ref", "libref_headers.so")
    if not os.path.exists(path):
        if not os.path.isdir(os.path.join(REFERENCE_CHECKOUT, "src")):
            return None
        build()
    return _declare_kat(ctypes.CDLL(path), "ref")


def lib(path=None):
    """The restatement; `path` selects another build of it (liborc_native.so) for the caller's own use."""
    global _LIB
    if _LIB is None or path is not None:
        if path is None:
            path = os.path.join(_HERE, "liborc.so")
            if not os.path.exists(path):
                build()
        L = ctypes.CDLL(path)
        L.orc_world_create.restype = ctypes.c_void_p
        L.orc_world_create.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_uint32]
        L.orc_world_destroy.argtypes = [ctypes.c_void_p]
        L.orc_world_reset.argtypes = [ctypes.c_void_p]
        L.orc_world_set_control_mode.argtypes = [ctypes.c_void_p, ctypes.c_uint32]
        L.orc_world_set_broadphase.argtypes = [ctypes.c_void_p, ctypes.c_uint32]
        L.orc_world_set_task_link.argtypes = [ctypes.c_void_p, ctypes.c_uint32]
        L.orc_lbvh_pair_set.restype = ctypes.c_uint32
        L.orc_lbvh_pair_set.argtypes = [ctypes.c_uint32, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint32]
        L.orc_world_refresh.argtypes = [ctypes.c_void_p]
        L.orc_world_step.argtypes = [ctypes.c_void_p, ctypes.c_uint32, ctypes.c_int]
        L.orc_stage_dynamics.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.orc_stage_collide.argtypes = [ctypes.c_void_p]
        L.orc_get.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t]
        L.orc_set.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_size_t]
        L.orc_hw_threads.restype = ctypes.c_int
        _LIB = L
    return _LIB


_U32 = {"pair_count", "candidate_pairs", "contact_count", "env_status", "solver_sweeps", "contact_points"}


class World:
    def __init__(self, blob, env_count):
        self._blob = bytes(blob)
        self.env_count = env_count
        self._h = lib().orc_world_create(self._blob, len(self._blob), env_count)
        if not self._h:
            raise RuntimeError("oracle rejected the template")

    def close(self):
        if self._h:
            lib().orc_world_destroy(self._h)
            self._h = None

    __del__ = close

    def step(self, n=1, threads=0):
        lib().orc_world_step(self._h, n, threads)

    def set_control_mode(self, mode):
        lib().orc_world_set_control_mode(self._h, int(mode))

    def set_task_link(self, link):
        """Mode 4: the link that carries the task frame."""
        lib().orc_world_set_task_link(self._h, int(link))

    def set_broadphase(self, mode):
        """0: the reference's route rule, 1: all-pairs, 2: LBVH tree walk."""
        lib().orc_world_set_broadphase(self._h, int(mode))

    def reset(self):
        lib().orc_world_reset(self._h)

    def refresh(self):
        lib().orc_world_refresh(self._h)

    def dynamics(self, integrate_velocity=False):
        lib().orc_stage_dynamics(self._h, int(integrate_velocity))

    def collide(self):
        lib().orc_stage_collide(self._h)

    def get(self, field, per_env):
        dt = np.uint32 if field in _U32 else np.float32
        out = np.zeros((self.env_count, per_env), dtype=dt)
        rc = lib().orc_get(self._h, field.encode(), out.ctypes.data, out.nbytes)
        if rc:
            raise KeyError(f"oracle field {field} (rc={rc}, per_env={per_env})")
        return out

    def set(self, field, value):
        dt = np.uint32 if field in _U32 else np.float32
        a = np.ascontiguousarray(value, dtype=dt)
        rc = lib().orc_set(self._h, field.encode(), a.ctypes.data, a.nbytes)
        if rc:
            raise KeyError(f"oracle field {field} (rc={rc})")
