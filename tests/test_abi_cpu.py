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


def test_transfer_checks_run_in_the_reference_order():
    """src/c_abi/buffer.cpp:98-110: a null buffer with a size is INVALID_ARG before the handle is looked at; an empty
    transfer on an unknown handle is still NULL_HANDLE."""
    lib = _abi.lib()
    assert lib.nuka_world_upload_field(None, 2, None, 16, 0) == _abi.INVALID_ARG
    assert lib.nuka_world_download_field(ctypes.c_void_p(99), 2, None, 16, 0) == _abi.INVALID_ARG
    assert lib.nuka_world_upload_field(None, 2, None, 0, 0) == _abi.NULL_HANDLE
    buf = (ctypes.c_float * 4)()
    assert lib.nuka_world_upload_field(ctypes.c_void_p(99), 2, buf, 16, 0) == _abi.NULL_HANDLE


def _parse(blob):
    """Runs the library's template parser without a GPU: create_from_template parses after validating the device, so
    the parser is reached through its own entry."""
    lib = _abi.lib()
    lib.nuka_b200_template_check.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    return lib.nuka_b200_template_check(blob, len(blob))


def _retag(blob, field, dtype=None, count=None):
    """Returns the blob with one record's dtype and/or element count overwritten (payload untouched)."""
    raw = bytearray(blob)
    at = 8
    for _ in range(int.from_bytes(raw[4:8], "little")):
        name = bytes(raw[at:at + 32]).split(b"\0", 1)[0].decode()
        d, n = int.from_bytes(raw[at + 32:at + 36], "little"), int.from_bytes(raw[at + 40:at + 48], "little")
        if name == field:
            if dtype is not None:
                raw[at + 32:at + 36] = dtype.to_bytes(4, "little")
            if count is not None:
                raw[at + 40:at + 48] = count.to_bytes(8, "little")
            return bytes(raw)
        at += 48 + ((n * (8 if d == 3 else 4) + 7) & ~7)
    raise KeyError(field)


def test_template_parser_rejects_malformed_blobs():
    good = T.quadruped(0).blob()
    assert _parse(good) == _abi.OK
    assert _parse(b"junk" * 8) == _abi.PARSE_ERROR
    assert _parse(good[:len(good) // 2]) == _abi.PARSE_ERROR                   # truncated in the middle of a record
    assert _parse(good[:-8]) == _abi.PARSE_ERROR                               # last record cut short
    # a record whose dtype is not the one the field is read as: 'excluded' is u64; tagging it f32 would halve the bytes
    # the bounds check covered
    assert _parse(_retag(good, "excluded", dtype=0)) == _abi.PARSE_ERROR
    assert _parse(_retag(good, "parent", dtype=0)) == _abi.PARSE_ERROR
    assert _parse(_retag(good, "axis", dtype=1)) == _abi.PARSE_ERROR
    assert _parse(_retag(good, "q0", dtype=7)) == _abi.PARSE_ERROR             # unknown dtype code
    assert _parse(_retag(good, "inv_mass", count=1 << 50)) == _abi.PARSE_ERROR  # count far beyond the blob
    arrays = T.quadruped(0).arrays()
    for field, bad in (("limit_flags", 9), ("geom_kind", 5), ("shape_kind", 11)):
        broken = {k: np.array(v, copy=True) for k, v in arrays.items()}
        broken[field][1] = bad
        assert _parse(nkt.pack(broken)) in (_abi.PARSE_ERROR, _abi.NOT_SUPPORTED), field
    slow = {k: np.array(v, copy=True) for k, v in arrays.items()}
    slow["cfg_u"][0] = 1 << 20                                                  # sweep count far above 65535
    assert _parse(nkt.pack(slow)) == _abi.INVALID_ARG
    slow["cfg_u"][0] = 4; slow["cfg_u"][1] = 70000
    assert _parse(nkt.pack(slow)) == _abi.INVALID_ARG


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
