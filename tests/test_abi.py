"""The C-ABI library without a GPU: it loads, exports every function include/sepal_b200.h declares (and nothing else), and fails
with a message instead of crashing or falling back when there is no device. No compute calls."""
import ctypes as C
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__ as ge
    import sepal_runner_b200 as sb

    if not os.path.exists(sb.library_path()):
        ge.build()
    return sb.library()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "sepal_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"SEPAL_B200_API\s+[\w\s\*]+?\b(sepal_b200_\w+)\s*\(", text)))


def test_header_and_binding_agree(lib):
    from sepal_runner_b200.lib import SIGNATURES

    names = declared_functions()
    assert len(names) >= 20
    assert sorted(SIGNATURES) == names


def test_every_declared_symbol_is_exported_and_nothing_else(lib):
    import sepal_runner_b200 as sb

    out = subprocess.run(["nm", "-D", "--defined-only", sb.library_path()], capture_output=True, text=True, check=True).stdout
    exported = sorted(line.split()[-1] for line in out.splitlines() if " T " in line)
    assert exported == declared_functions()
    for name in declared_functions():
        assert getattr(lib, name) is not None


def test_api_version_and_error_string(lib):
    assert lib.sepal_b200_api_version() == 1
    assert lib.sepal_b200_last_error() in (b"",) or isinstance(lib.sepal_b200_last_error(), bytes)


def test_open_without_a_device_fails_with_a_message_and_no_fallback(lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("this check is for the CPU-only box")
    handle = C.c_void_p(1234)
    rc = lib.sepal_b200_open(0, 0, C.byref(handle))
    assert rc != 0 and handle.value is None  # *out = NULL on failure, as sepal_open (runner/include/sepal/c_api.h:39)
    assert len(lib.sepal_b200_last_error()) > 0
    prov = C.c_void_p(1234)
    assert lib.sepal_b200_provider_open(0, 0, C.byref(prov)) != 0 and prov.value is None
    lib.sepal_b200_close(None)  # closing NULL is allowed (runner/tests/test_capi.cpp:102)
    lib.sepal_b200_provider_close(None)
    lib.sepal_b200_host_free(None)


def test_null_arguments_are_errors_not_crashes(lib):
    assert lib.sepal_b200_open(0, 0, None) != 0
    assert b"null" in lib.sepal_b200_last_error()
    assert lib.sepal_b200_gemm_f16(None, None, 8, None, 8, None, 8, 1, 1, 8, 8, 0, -1, None) != 0
    assert b"ctx is null" in lib.sepal_b200_last_error()
    st = C.c_int32(0)
    assert lib.sepal_b200_status(None, None, C.byref(st)) != 0
    assert lib.sepal_b200_info(None, None, 0, None) != 0


def test_quantiser_argument_checks_run_before_any_device_call(lib):
    # K not a multiple of 128 is refused by the launcher itself (runner/cuda/src/gemm_simt_kernels.cu:335)
    assert lib.sepal_b200_quantize_group_s8(None, 100, None, 100, None, 1, 4, 100, None) != 0
    assert b"multiple of 128" in lib.sepal_b200_last_error()
    # an empty matrix is a no-op, as in the reference
    assert lib.sepal_b200_quantize_group_s8(None, 128, None, 128, None, 1, 0, 128, None) == 0
    assert lib.sepal_b200_last_error() == b""
    assert lib.sepal_b200_pack_gate_up(None, 16, None, 16, 63, 16, None) != 0


def test_python_binding_fails_loudly_when_the_library_is_missing(monkeypatch, tmp_path):
    import sepal_runner_b200.lib as L

    monkeypatch.setattr(L, "_LIB", None)
    monkeypatch.setattr(L, "HERE", str(tmp_path))
    with pytest.raises(L.SepalB200Error, match="no fallback"):
        L.library()


def test_pack_gate_up_source_is_the_reference_formula():
    import sepal_runner_b200 as sb

    inter = 192
    src = [sb.pack_gate_up_source(p, inter) for p in range(2 * inter)]
    assert sorted(src) == list(range(2 * inter))
    assert src[:64] == list(range(64)) and src[64:128] == list(range(inter, inter + 64)) and src[128] == 64


def test_int8_schedule_query_is_host_arithmetic(lib):
    """sepal_b200_w8g_schedule needs no GPU: the automatic choice between the swapped int8 kernel (tokens to a tile; 256 and 320 are
    two blocks of half as many) and the unswapped ones (0) for the trunk's shapes on a 148-SM GPU, as measured sweeps fixed it."""
    import sepal_runner_b200 as sb

    assert sb.w8g_schedule(148, 900, 2560, 9728, sb.ADD) == 320      # the headline: 30 tiles of two blocks of 160 tokens, each shared by two pairs
    assert sb.w8g_schedule(148, 900, 2560, 9728, sb.STORE) == 160    # stored, not added: 60 whole-k tiles of 160 tokens
    assert sb.w8g_schedule(148, 900, 2560, 4096, sb.ADD) == 160      # o + residual
    assert sb.w8g_schedule(148, 300, 2560, 9728, sb.STORE) == 96     # few tokens: the narrowest tile
    assert sb.w8g_schedule(148, 300, 2560, 9728, sb.ADD) == 128      # a float32 residual update: 30 tiles, the other pairs take half of each
    assert sb.w8g_schedule(148, 600, 2560, 9728, sb.ADD) == 160      # 40 tiles, 23 of the 76 groups of each go to the 34 spare pairs
    assert sb.w8g_schedule(148, 900, 9728, 2560, sb.STORE) == 320    # up: three tiles of two blocks of 160 by 38 tiles of weight rows
    assert sb.w8g_schedule(148, 4096, 2560, 9728, sb.ADD) == 320     # down at 4096 tokens
    assert sb.w8g_schedule(148, 4096, 19456, 2560, sb.SWIGLU) == 320
    assert sb.w8g_schedule(148, 2048, 19456, 2560, sb.SWIGLU) == 0   # 16.4 waves of unswapped tiles against 22 of swapped ones
    assert sb.w8g_schedule(148, 128, 2560, 9728, sb.ADD) == 0        # up to 128 tokens: the lone-CTA kernel
    assert sb.w8g_schedule(148, 900, 2560, 9700, sb.ADD) == 0        # k not a multiple of 128: not an int8-group shape
    assert sb.w8g_schedule(0, 900, 2560, 9728, sb.ADD) == 0
    # the unhidden epilogue counts: a result stored lane by lane costs several us a wave more
    assert sb.w8g_schedule(148, 900, 4096, 2560, sb.STORE, staged=True) == 256 and sb.w8g_schedule(148, 900, 4096, 2560, sb.STORE, staged=False) == 0
