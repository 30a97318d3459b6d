"""Host-side checks that need no GPU: the C ABI loads, exports what include/tcec.h
declares, and rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

from wmma_extension_b200 import tcec

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "tcec.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tcec_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = tcec.load()
    names = declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), name
    assert set(tcec.EXPORTED_SYMBOLS) <= set(names)


def test_version_and_status_strings():
    lib = tcec.load()
    assert b"sm_100a" in lib.tcec_version()
    assert tcec.status_string(tcec.OK) == "ok"
    assert "argument" in tcec.status_string(tcec.ERR_INVALID_ARGUMENT)
    assert "wait" in tcec.status_string(tcec.ERR_TIMEOUT)


def test_invalid_arguments_are_rejected_without_a_device():
    lib = tcec.load()
    z = None
    # unknown layout, negative size, bad policy, leading dimension too small, missing pointer
    assert lib.tcec_sgemm(7, 0, 0, 4, 4, 4, 1.0, z, 4, z, 4, 0.0, z, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm(0, 0, 0, -1, 4, 4, 1.0, z, 4, z, 4, 0.0, z, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm(0, 0, 0, 4, 4, 4, 1.0, z, 4, z, 4, 0.0, z, 4, 9, z) == tcec.ERR_INVALID_ARGUMENT
    buf = ctypes.create_string_buffer(64)
    p = ctypes.cast(buf, ctypes.c_void_p)
    assert lib.tcec_sgemm(0, 0, 0, 4, 4, 4, 1.0, p, 3, p, 4, 0.0, p, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm(0, 0, 0, 4, 4, 4, 1.0, p, 4, p, 4, 0.0, p, 2, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm(0, 0, 0, 4, 4, 4, 1.0, z, 4, p, 4, 0.0, p, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    # empty problems are fine and launch nothing
    assert lib.tcec_sgemm(0, 0, 0, 0, 4, 4, 1.0, z, 4, z, 4, 0.0, z, 4, 0, z) == tcec.OK
    assert lib.tcec_sgemm_batched(0, 0, 0, 4, 4, 4, 1.0, z, 4, z, 4, 0.0, z, 4, 0, 0, z) == tcec.OK
    assert lib.tcec_split(z, z, z, 0, 0, z) == tcec.OK
    assert lib.tcec_split(z, z, z, 5, 0, z) == tcec.ERR_INVALID_ARGUMENT
    one = (ctypes.c_float * 2)(1.0, 0.0)
    assert lib.tcec_cgemm(0, 0, 0, 4, 4, 4, None, p, 4, p, 4, one, p, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_cgemm(0, 0, 0, 4, 4, 4, one, p, 3, p, 4, one, p, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_cgemm(0, 3, 0, 4, 4, 4, one, p, 4, p, 4, one, p, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_cgemm(0, 0, 0, 0, 4, 4, one, z, 4, z, 4, one, z, 4, 0, z) == tcec.OK
    assert lib.tcec_pack_a(0, 4, 4, z, 4, z, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_packed(0, 4, 4, 4, 1.0, z, z, 0.0, z, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT


def test_new_entry_points_reject_bad_arguments_without_a_device():
    lib = tcec.load()
    z = None
    buf = ctypes.create_string_buffer(256)
    p = ctypes.cast(buf, ctypes.c_void_p)
    # host-operand GEMM: layouts, sizes, policy, pointers and leading dimensions are checked first
    assert lib.tcec_sgemm_host(9, 0, 0, 4, 4, 4, 1.0, p, 4, p, 4, 0.0, p, 4, 0, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_host(0, 0, 0, 4, 4, 4, 1.0, z, 4, p, 4, 0.0, p, 4, 0, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_host(0, 0, 0, 4, 4, 4, 1.0, p, 3, p, 4, 0.0, p, 4, 0, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_host(0, 0, 0, 4, 4, 4, 1.0, p, 4, p, 4, 0.0, p, 2, 0, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_host(0, 0, 0, 0, 4, 4, 1.0, z, 4, z, 4, 0.0, z, 4, 0, 0, z) == tcec.OK
    # device lists
    i2 = (ctypes.c_int * 2)(0, 0)
    n2 = (ctypes.c_int * 2)(4, 4)
    ld2 = (ctypes.c_longlong * 2)(4, 4)
    pp = (ctypes.c_void_p * 2)(p.value, p.value)
    assert lib.tcec_sgemm_multi(0, i2, 0, 0, 0, 4, n2, 4, 1.0, p, 4, pp, ld2, 0.0, pp, ld2, 0, None) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_multi(2, i2, 0, 0, 0, 4, n2, 4, 1.0, p, 4, pp, ld2, 0.0, pp, ld2, 0, None) == tcec.ERR_INVALID_ARGUMENT  # a device named twice
    assert lib.tcec_sgemm_multi(2, None, 0, 0, 0, 4, n2, 4, 1.0, p, 4, pp, ld2, 0.0, pp, ld2, 0, None) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_batched_multi(0, i2, 0, 0, 0, 4, 4, 4, 1.0, pp, 4, 16, pp, 4, 16, 0.0, pp, 4, 16, n2, 0, None) == tcec.ERR_INVALID_ARGUMENT
    # communicator
    assert lib.tcec_comm_init_rank(2, 5, p) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_comm_init_rank(2, 0, None) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_comm_unique_id(None) == tcec.ERR_INVALID_ARGUMENT
    assert lib.tcec_sgemm_column_shard(0, 0, 0, 7, 4, 4, 4, 1.0, p, 4, p, 4, 0.0, p, 4, 0, z) == tcec.ERR_INVALID_ARGUMENT
    assert "NCCL" in tcec.status_string(tcec.ERR_COMM)


def test_a_failing_communication_library_is_reported_as_a_status(tmp_path):
    """An error code from a fake of the failing call: with a stand-in libnccl whose calls fail,
    obtaining a communicator id returns TCEC_ERR_COMM (and a missing library likewise)."""
    import subprocess
    import sys

    fake = tmp_path / "libfake_nccl.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(fake), os.path.join(ROOT, "tests", "fake_nccl.c")], check=True)
    code = (
        "import ctypes, sys\n"
        "sys.path.insert(0, %r)\n"
        "from wmma_extension_b200 import tcec\n"
        "lib = tcec.load()\n"
        "assert lib.tcec_comm_set_library(sys.argv[1].encode()) == tcec.OK\n"
        "buf = ctypes.create_string_buffer(128)\n"
        "print(lib.tcec_comm_unique_id(buf))\n" % ROOT)
    for path, want in ((str(fake), tcec.ERR_COMM), (str(tmp_path / "no_such_library.so"), tcec.ERR_COMM)):
        out = subprocess.run([sys.executable, "-c", code, path], capture_output=True, text=True, timeout=120)
        assert out.returncode == 0, out.stderr[-1000:]
        assert int(out.stdout.strip()) == want


def test_options_round_trip():
    old = tcec.get_option("promote_k")
    try:
        assert old == -1  # automatic by default
        tcec.set_option("promote_k", 64)
        assert tcec.get_option("promote_k") == 64
        with pytest.raises(tcec.TcecError):
            tcec.set_option("promote_k", -2)
        with pytest.raises(tcec.TcecError):
            tcec.set_option("tile_n", 96)
        with pytest.raises(tcec.TcecError):
            tcec.set_option("no_such_option", 1)
        for name, default, other in (("cta_pair", -1, 1), ("path", 0, 2), ("store_turn", 1, 0), ("reserve_sms", 0, 8),
                                     ("static_tiles", 0, 1), ("tile_n", 0, 128), ("comm_sms", 8, 16),
                                     ("comm_panel_rows", 2048, 512), ("comm_helper", 1, 0), ("half_tiles", 1, 0)):
            assert tcec.get_option(name) == default
            tcec.set_option(name, other)
            assert tcec.get_option(name) == other
            tcec.set_option(name, default)
        with pytest.raises(tcec.TcecError):
            tcec.set_option("store_turn", 2)
        with pytest.raises(tcec.TcecError):
            tcec.set_option("comm_panel_rows", 300)  # not a multiple of 256
        with pytest.raises(tcec.TcecError):
            tcec.set_option("debug_flags", 1)  # development switches do not exist in the product library
    finally:
        tcec.set_option("promote_k", old)


def test_workspace_and_packed_sizes():
    # fp16+ec: hi and lo, 2 bytes each -> 4 bytes per padded element
    assert tcec.packed_bytes(4096, 4096, "fp16_ec") == 4096 * 4096 * 4
    assert tcec.packed_bytes(4096, 4096, "fp16_no_ec") == 4096 * 4096 * 2
    assert tcec.packed_bytes(4096, 4096, "tf32_ec") == 4096 * 4096 * 8
    assert tcec.packed_bytes(1, 1, "fp16_ec") == 256 * 32 * 4  # padded to 256 rows x one k block
    assert tcec.workspace_bytes(4096, 4096, 4096) == 2 * 4096 * 4096 * 4
    assert tcec.packed_row_offset(256, 64, "fp16_ec") == tcec.packed_bytes(256, 64, "fp16_ec")
    assert tcec.packed_row_offset(512, 64, "tf32_ec") == 2 * tcec.packed_bytes(256, 64, "tf32_ec")
    assert tcec.packed_row_offset(128, 64, "fp16_ec") == 0  # row blocks are read in pairs: multiples of 256 only
    assert tcec.packed_row_offset(100, 64, "fp16_ec") == 0


def test_layout_detection():
    import torch

    a = torch.zeros(6, 4)
    assert tcec._layout_ld(a) == (tcec.ROW_MAJOR, 4)
    assert tcec._layout_ld(a.t()) == (tcec.COL_MAJOR, 4)
    assert tcec._layout_ld(torch.zeros(6, 8)[:, :4]) == (tcec.ROW_MAJOR, 8)
    with pytest.raises(ValueError):
        tcec._layout_ld(torch.zeros(6, 8)[:, ::2])
    with pytest.raises(ValueError):
        tcec.sgemm(torch.zeros(2, 2), torch.zeros(2, 2))  # CPU tensors: there is no CPU path
