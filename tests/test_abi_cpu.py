"""Boundary checks that need no GPU: the library loads, exports every declared symbol, maps failures to
result codes and never falls back to a CPU path."""
import ctypes
import os
import re

import numpy as np
import pytest

import nuka
from nuka import _abi, nkt, templates as T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "nuka_b200.h")).read()
    declared = set(re.findall(r"\b(nuka_[a-z0-9_]+)\s*\(", header))
    declared -= {"nuka_device_t", "nuka_world_t"}
    lib = _abi.lib()
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, missing
    assert set(_abi.EXPORTS) <= declared


def test_result_messages_and_error_text():
    lib = _abi.lib()
    assert lib.nuka_result_message(0) == b"ok"
    assert lib.nuka_result_message(7) == b"not supported"
    out = ctypes.c_void_p()
    assert lib.nuka_device_create(None, ctypes.byref(out)) == _abi.INVALID_ARG
    assert b"null" in lib.nuka_last_error_message()
    assert lib.nuka_last_error_message() == b""          # reading clears it


def test_null_handles_are_reported():
    lib = _abi.lib()
    assert lib.nuka_world_step(None) == _abi.NULL_HANDLE
    assert lib.nuka_world_step_n(ctypes.c_void_p(12345), 3) == _abi.NULL_HANDLE
    assert lib.nuka_world_reset(None) == _abi.NULL_HANDLE
    view = _abi.BufferView()
    assert lib.nuka_world_get_buffer_view(None, 2, ctypes.byref(view)) == _abi.NULL_HANDLE
    desc = _abi.WorldDesc()
    desc.env_count = 4
    out = ctypes.c_void_p()
    blob = T.arm7().blob()
    assert lib.nuka_world_create_from_template(None, ctypes.byref(desc), blob, len(blob), ctypes.byref(out)) == _abi.NULL_HANDLE


@pytest.mark.skipif(os.path.exists("/dev/nvidiactl"), reason="a GPU is present")
def test_no_cpu_fallback_without_a_gpu():
    with pytest.raises(nuka.NukaError) as err:
        nuka.Device.create(0)
    assert err.value.code == _abi.CUDA_ERROR


def test_world_desc_layout_matches_the_reference_abi():
    # nuka.h:57-173 on LP64: 8-byte pointers, natural alignment
    assert ctypes.sizeof(_abi.WorldDesc) == 160
    assert _abi.WorldDesc.env_count.offset == 8 and _abi.WorldDesc.gravity_x.offset == 96
    assert _abi.WorldDesc.solver_vel_iters.offset == 120 and _abi.WorldDesc.contact_detection_substeps.offset == 156
    assert ctypes.sizeof(_abi.BufferView) == 24 and ctypes.sizeof(_abi.DeviceDesc) == 24


def test_template_container_round_trip():
    arrays = T.quadruped().arrays()
    back = nkt.unpack(nkt.pack(arrays))
    assert list(back) == list(arrays)
    for k in arrays:
        assert back[k].dtype == arrays[k].dtype and np.array_equal(back[k].ravel(), np.asarray(arrays[k]).ravel())


def test_templates_have_the_configured_shapes():
    a = T.arm7().arrays()
    assert a["cfg_u"][4] == 8 and T.dof_count(a) == 7
    q = T.quadruped().arrays()
    assert q["cfg_u"][4] == 13 and q["cfg_u"][5] == 14 and T.dof_count(q) == 18
    assert len(q["excluded"]) == 12 and (np.diff(q["excluded"].astype(np.int64)) > 0).all()
    h = T.humanoid().arrays()
    assert h["cfg_u"][4] == 30 and T.dof_count(h) == 35
    b = T.box_pile().arrays()
    assert b["cfg_u"][5] == 49 and (b["inv_mass"][:48] > 0).all() and b["inv_mass"][48] == 0
    s = T.quadruped(boxes=4).arrays()
    assert s["cfg_u"][5] == 18
