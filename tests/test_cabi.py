"""CPU: the shared library loads, exports every symbol the header declares, and rejects bad
arguments before touching the GPU.  No compute call is made here."""
import ctypes
import os
import re

import pytest

from conftest import PKG, ROOT

LIB = os.path.join(PKG, "lib", "libfal_b200.so")
HEADER = os.path.join(ROOT, "include", "fal_b200.h")


@pytest.fixture(scope="module")
def lib():
    return ctypes.CDLL(LIB)


def declared_functions():
    text = open(HEADER).read()
    return sorted(set(re.findall(r"FAL_API\s+[\w\s\*]+?\b(fal_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("fal_fwd", "fal_fwd_kvcache", "fal_fwd_varlen", "fal_bwd", "fal_bwd_varlen", "fal_decode", "fal_decode_ranged",
                 "fal_bwd_workspace_bytes", "fal_decode_workspace_bytes", "fal_strerror", "fal_set_fwd_variant"):
        assert must in names


def test_every_declared_symbol_is_exported(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/fal_b200.h but not exported"


def test_only_fal_symbols_are_exported():
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", LIB], capture_output=True, text=True).stdout
    ours = [l.split()[-1] for l in out.splitlines() if " T " in l]
    assert ours and all(s.startswith("fal_") for s in ours), ours


def test_strerror_and_version(lib):
    lib.fal_strerror.restype = ctypes.c_char_p
    lib.fal_version.restype = ctypes.c_char_p
    assert lib.fal_strerror(0) == b"ok"
    assert b"head_dim" in lib.fal_strerror(-2)
    assert lib.fal_strerror(-12345) == b"unknown error"
    assert re.fullmatch(rb"\d+\.\d+\.\d+", lib.fal_version())


def test_workspace_sizes(lib):
    lib.fal_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.fal_decode_workspace_bytes.restype = ctypes.c_size_t
    # rows padded to a multiple of 128 plus one spare 128-row tile; fp32 accumulator + fp32 delta
    rows = 4096 + 128
    expect = 4 * 32 * rows * 128 * 4 + 4 * 32 * rows * 4
    assert lib.fal_bwd_workspace_bytes(4, 32, 4096, 128) == expect
    assert lib.fal_bwd_workspace_bytes(0, 32, 4096, 128) == 0
    # head dims 32 and 96 run on the 64 / 128 kernels: their scratch is that of the kernel they run on
    assert lib.fal_bwd_workspace_bytes(4, 32, 4096, 96) == expect
    assert lib.fal_bwd_workspace_bytes(1, 2, 100, 32) == lib.fal_bwd_workspace_bytes(1, 2, 100, 64)
    assert lib.fal_decode_workspace_bytes(2, 8, 5000, 96) == lib.fal_decode_workspace_bytes(2, 8, 5000, 128)
    # 32 splits of 1024 positions, (d + 2) floats per (batch, head, split)
    assert lib.fal_decode_workspace_bytes(64, 32, 32768, 128) == 64 * 32 * 32 * 130 * 4
    assert lib.fal_decode_workspace_bytes(1, 8, 1000, 64) == 1 * 8 * 1 * 66 * 4


class Strides(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int64), ("head", ctypes.c_int64), ("row", ctypes.c_int64)]


def test_bad_arguments_are_rejected_without_a_gpu(lib):
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    sp = ctypes.POINTER(Strides)
    lib.fal_fwd.restype = i
    lib.fal_fwd.argtypes = [vp] * 5 + [i] * 6 + [sp] * 4 + [f, i, vp, vp]
    st = Strides(64 * 128, 128 * 64, 64)
    fake = 0x1000  # never dereferenced: validation fails first
    # null pointer
    assert lib.fal_fwd(None, fake, fake, fake, fake, 1, 2, 2, 128, 128, 64, st, st, st, st, 0.125, 0, None, None) == -1
    # heads_q not divisible by heads_kv
    assert lib.fal_fwd(fake, fake, fake, fake, fake, 1, 3, 2, 128, 128, 64, st, st, st, st, 0.125, 0, None, None) == -1
    # unsupported head_dim
    assert lib.fal_fwd(fake, fake, fake, fake, fake, 1, 2, 2, 128, 128, 80, st, st, st, st, 0.125, 0, None, None) == -2
    # non-positive scale
    assert lib.fal_fwd(fake, fake, fake, fake, fake, 1, 2, 2, 128, 128, 64, st, st, st, st, 0.0, 0, None, None) == -1
    # causal mode outside {0, 1, 2}; bottom-right alignment with fewer keys than queries
    assert lib.fal_fwd(fake, fake, fake, fake, fake, 1, 2, 2, 128, 128, 64, st, st, st, st, 0.125, 3, None, None) == -1
    assert lib.fal_fwd(fake, fake, fake, fake, fake, 1, 2, 2, 128, 64, 64, st, st, st, st, 0.125, 2, None, None) == -1
    # misaligned output pointer
    assert lib.fal_fwd(fake, fake, fake, fake + 2, fake, 1, 2, 2, 128, 128, 64, st, st, st, st, 0.125, 0, None, None) == -1

    # causal modes outside {0, 1, 2} are refused everywhere; the batched backward refuses the
    # bottom-right-aligned mask when there are fewer keys than queries, like the forward
    cu = fake
    lib.fal_fwd_varlen.restype = i
    lib.fal_fwd_varlen.argtypes = [vp] * 7 + [i] * 8 + [sp] * 4 + [f, i, vp, vp]
    assert lib.fal_fwd_varlen(fake, fake, fake, fake, fake, cu, cu, 1, 128, 128, 128, 128, 2, 2, 64,
                              st, st, st, st, 0.125, 3, None, None) == -1
    lib.fal_bwd.restype = i
    lib.fal_bwd.argtypes = [vp] * 9 + [i] * 6 + [sp] * 8 + [f, i, vp, ctypes.c_size_t, vp, vp]
    assert lib.fal_bwd(fake, fake, fake, fake, fake, fake, fake, fake, fake, 1, 2, 2, 128, 64, 64,
                       st, st, st, st, st, st, st, st, 0.125, 2, fake, 1 << 30, None, None) == -1
    assert lib.fal_bwd(fake, fake, fake, fake, fake, fake, fake, fake, fake, 1, 2, 2, 128, 128, 64,
                       st, st, st, st, st, st, st, st, 0.125, 3, fake, 1 << 30, None, None) == -1
    lib.fal_bwd_varlen.restype = i
    lib.fal_bwd_varlen.argtypes = [vp] * 9 + [vp, vp] + [i] * 8 + [sp] * 8 + [f, i, vp, ctypes.c_size_t, vp, vp]
    assert lib.fal_bwd_varlen(fake, fake, fake, fake, fake, fake, fake, fake, fake, cu, cu, 1, 128, 128, 128, 128,
                              2, 2, 64, st, st, st, st, st, st, st, st, 0.125, -1, fake, 1 << 30, None, None) == -1

    lib.fal_decode.restype = i
    lib.fal_decode.argtypes = [vp, vp, vp, sp, sp, vp, vp, vp, vp, vp, i, i, i, i, i, f, vp, ctypes.c_size_t, vp, vp]
    # k_new without v_new
    assert lib.fal_decode(fake, fake, fake, st, st, fake, fake, None, fake, None, 1, 8, 2, 128, 64, 0.125,
                          fake, 1 << 20, None, None) == -1
    # workspace too small
    assert lib.fal_decode(fake, fake, fake, st, st, fake, None, None, fake, None, 1, 8, 2, 128, 64, 0.125,
                          fake, 16, None, None) == -3

    # the ranged form without its first-position array
    lib.fal_decode_ranged.restype = i
    lib.fal_decode_ranged.argtypes = [vp, vp, vp, sp, sp, vp, vp, vp, vp, vp, vp, i, i, i, i, i, f, vp,
                                      ctypes.c_size_t, vp, vp]
    assert lib.fal_decode_ranged(fake, fake, fake, st, st, None, fake, None, None, fake, None, 1, 8, 2, 128, 64,
                                 0.125, fake, 1 << 20, None, None) == -1
    assert lib.fal_decode_ranged(fake, fake, fake, st, st, fake, fake, None, None, fake, None, 1, 8, 2, 128, 64,
                                 0.125, fake, 16, None, None) == -3
    # the allocation-free form validates the same arguments, then its size limit (8 MiB), before any CUDA call
    lib.fal_decode_static.restype = i
    lib.fal_decode_static.argtypes = [vp, vp, vp, sp, sp, vp, vp, vp, vp, vp, i, i, i, i, i, f, vp, vp]
    assert lib.fal_decode_static(fake, fake, fake, st, st, fake, fake, None, fake, None, 1, 8, 2, 128, 64, 0.125,
                                 None, None) == -1
    assert lib.fal_decode_static(fake, fake, fake, st, st, fake, None, None, fake, None, 64, 32, 8, 32768, 128,
                                 0.125, None, None) == -7


def test_profile_api_is_inert_without_launches(lib):
    total, n = ctypes.c_double(-1), ctypes.c_int(-1)
    lib.fal_profile_read.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int)]
    assert lib.fal_profile_read(1, ctypes.byref(total), ctypes.byref(n)) == 0
    assert total.value == 0.0 and n.value == 0
    assert lib.fal_profile_read(7, ctypes.byref(total), ctypes.byref(n)) == -1
