"""ctypes binding of include/sepal_b200.h.

`Context` mirrors the reference's kernel launchers (device pointers; arguments in the order of launch_gemm_nt /
launch_gemm_simt, runner/cuda/src/gemm_kernels.hpp:30-31 and gemm_simt_kernels.hpp:55-56) and `Provider` mirrors its
host-pointer GEMM provider (sepal::cuda::CudaGemm, runner/cuda/include/sepal/cuda/cuda_gemm.hpp:112-160).
"""
from __future__ import annotations

import ctypes as C
import json
import os
from dataclasses import dataclass
from typing import Optional

HERE = os.path.dirname(os.path.abspath(__file__))
STORE, ADD, SWIGLU = 0, 1, 2
F32, F16 = 0, 1
GROUP = 128

_vp, _u64, _i32, _u32 = C.c_void_p, C.c_uint64, C.c_int32, C.c_uint32


class SepalB200Error(RuntimeError):
    pass


def library_path() -> str:
    return os.path.join(HERE, "libsepal_b200.so")


_LIB: Optional[C.CDLL] = None

# name -> (restype, argtypes); every function include/sepal_b200.h declares
SIGNATURES = {
    "sepal_b200_api_version": (_i32, []),
    "sepal_b200_last_error": (C.c_char_p, []),
    "sepal_b200_open": (_i32, [_i32, _u64, C.POINTER(_vp)]),
    "sepal_b200_close": (None, [_vp]),
    "sepal_b200_info": (_i32, [_vp, C.c_char_p, _u64, C.POINTER(_u64)]),
    "sepal_b200_status": (_i32, [_vp, _vp, C.POINTER(_i32)]),
    "sepal_b200_take_launch_count": (_u64, []),
    "sepal_b200_debug_leave_status": (_i32, [_vp, _vp, _i32, _u32]),
    "sepal_b200_w8g_schedule": (_i32, [_u32, _u64, _u64, _u64, _i32, _i32]),
    "sepal_b200_gemm_f16": (_i32, [_vp, _vp, _u64, _vp, _u64, _vp, _u64, _i32, _u64, _u64, _u64, _i32, _i32, _vp]),
    "sepal_b200_gemm_f16_noalloc": (_i32, [_vp, _u64, _vp, _u64, _vp, _u64, _i32, _u64, _u64, _u64, _i32, _vp, C.POINTER(_i32)]),
    "sepal_b200_gemm_w8g": (_i32, [_vp, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _vp, _u64, _i32, _u64, _u64, _u64, _i32, _i32, _vp]),
    "sepal_b200_gemm_w8r": (_i32, [_vp, _vp, _u64, _vp, _u64, _vp, _vp, _u64, _i32, _u64, _u64, _u64, _i32, _i32, _vp]),
    "sepal_b200_quantize_rows_s8": (_i32, [_vp, _u64, _vp, _u64, _vp, _u64, _u64, _vp, _vp]),
    "sepal_b200_quantize_group_s8": (_i32, [_vp, _u64, _vp, _u64, _vp, _u64, _u64, _u64, _vp]),
    "sepal_b200_prepare_w8g_scales": (_i32, [_vp, _u64, _u64, _u64, _vp, _u64, _vp, _vp, _vp]),
    "sepal_b200_pack_gate_up": (_i32, [_vp, _u64, _vp, _u64, _u64, _u64, _vp]),
    "sepal_b200_float_to_half": (_i32, [_vp, _vp, _u64, _vp]),
    "sepal_b200_half_to_float": (_i32, [_vp, _vp, _u64, _vp]),
    "sepal_b200_embed": (_i32, [_vp, _vp, _vp, _u64, _u64, _u64, _vp]),
    "sepal_b200_embed_rms_norm_half": (_i32, [_vp, _vp, _vp, _vp, _vp, _u64, _u64, _u64, _u64, C.c_float, _vp]),
    "sepal_b200_rms_norm_half": (_i32, [_vp, _u64, _vp, _vp, _u64, _u64, _u64, C.c_float, _vp]),
    "sepal_b200_trunk_open": (_i32, [_i32, _vp, C.POINTER(_vp)]),
    "sepal_b200_trunk_close": (None, [_vp]),
    "sepal_b200_set_launch_overlap": (None, [_i32]),
    "sepal_b200_set_static_weights": (_i32, [_vp, _i32]),
    "sepal_b200_attention_prepare": (_i32, [_vp, _vp, _vp, _u64, _vp, _u64, _i32, _vp, _u64, _i32, _vp, _u64, _i32, _vp, _vp, _vp, _u64, _vp, _vp, _u64, _vp]),
    "sepal_b200_attention": (_i32, [_vp, _vp, _vp, _u64, _u64, _vp, _u64, _vp, _vp, _u64, _vp, _u64, _i32, _vp, _u64, _vp]),
    "sepal_b200_deltanet": (_i32, [_vp, _vp, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _vp, _u64, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u64, _vp, _u64, _vp]),
    "sepal_b200_trunk_open_checkpoint": (_i32, [_i32, _vp, _vp, _vp]),
    "sepal_b200_trunk_save": (_i32, [_vp, C.c_char_p]),
    "sepal_b200_checkpoint_open": (_i32, [C.c_char_p, _vp]),
    "sepal_b200_checkpoint_close": (None, [_vp]),
    "sepal_b200_checkpoint_count": (_i32, [_vp, _vp]),
    "sepal_b200_checkpoint_tensor": (_i32, [_vp, _u64, C.c_char_p, _vp]),
    "sepal_b200_checkpoint_metadata": (_i32, [_vp, C.c_char_p, _vp, _u64, _vp]),
    "sepal_b200_tensor_file_write": (_i32, [C.c_char_p, _u64, _vp, _u64, _vp, _vp]),
    "sepal_b200_model_preset": (_i32, [C.c_char_p, _vp]),
    "sepal_b200_plan_weight_bytes": (_i32, [_vp, C.c_char_p, _vp]),
    "sepal_b200_trunk_run": (_i32, [_vp, _vp, _u64, _vp, _vp, _vp]),
    "sepal_b200_trunk_score": (_i32, [_vp, _u64, _vp, _vp, _vp, _vp]),
    "sepal_b200_trunk_weight": (_i32, [_vp, _u32, _i32, _vp, _u64, C.POINTER(_u64)]),
    "sepal_b200_trunk_info": (_i32, [_vp, C.POINTER(_u64), C.POINTER(_u64)]),
    "sepal_b200_provider_open": (_i32, [_i32, _u64, C.POINTER(_vp)]),
    "sepal_b200_provider_close": (None, [_vp]),
    "sepal_b200_provider_upload_weights": (_i32, [_vp, _vp, _i32, _u64, _u64, C.POINTER(_u32)]),
    "sepal_b200_provider_upload_weights_w8g": (_i32, [_vp, _vp, _u64, _u64, C.POINTER(_u32)]),
    "sepal_b200_provider_gemm_f": (_i32, [_vp, _vp, _i32, _u64, _u32, _vp, C.c_float]),
    "sepal_b200_host_alloc": (_i32, [_u64, C.POINTER(_vp)]),
    "sepal_b200_host_free": (None, [_vp]),
}


def library() -> C.CDLL:
    """The loaded shared library. Raises when it has not been built: there is nothing to fall back to."""
    global _LIB
    if _LIB is None:
        path = library_path()
        if not os.path.exists(path):
            raise SepalB200Error(f"{path} is missing: build it with `python -m sepal_runner_b200.build` (nvcc, sm_100a); there is no fallback path")
        lib = C.CDLL(path)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _LIB = lib
    return _LIB


def _check(rc: int) -> None:
    if rc != 0:
        raise SepalB200Error(library().sepal_b200_last_error().decode())


def w8g_schedule(sm_count: int, t: int, n: int, k: int, epilogue: int = 0, staged: bool = True) -> int:
    """Tokens to a tile of the swapped int8 kernel that the automatic schedule of gemm_w8g gives this multiply on a GPU of `sm_count`
    SMs (256 and 320: two blocks of half as many), or 0 for the unswapped kernels (sepal_b200_w8g_schedule: host arithmetic, needs no GPU)."""
    return int(library().sepal_b200_w8g_schedule(sm_count, t, n, k, epilogue, 1 if staged else 0))


def pack_gate_up_source(p: int, inter: int) -> int:
    """Row of the stacked [gate; up] matrix that packed row p holds (runner/cuda/src/gemm_simt_kernels.hpp:72-77)."""
    b, r = divmod(p, 128)
    return 64 * b + r if r < 64 else inter + 64 * b + (r - 64)


def _stream_ptr(stream) -> int:
    import torch

    s = stream if stream is not None else torch.cuda.current_stream()
    return int(s.cuda_stream)


@dataclass
class W8gWeight:
    """An int8-group weight matrix on the device, in the form the tensor-core multiply reads (W8gMatrix in csrc/gemm.hpp)."""

    q: "object"          # torch.int8 [N, K]
    scales: "object"     # torch.float32 [N, K / 128]: the quantiser's (and the reference's) layout, kept for checks
    scales_t: "object"   # torch.float16 [K / 128, N rounded up to 256]: prepared
    descale: "object"    # torch.float32 [1]


class Context:
    """Per-device state + the launchers. All tensors are CUDA tensors of the context's device; launches go to the current stream."""

    def __init__(self, device: int = 0, workspace_bytes: int = 0) -> None:
        self._lib = library()
        handle = _vp()
        _check(self._lib.sepal_b200_open(device, workspace_bytes, C.byref(handle)))
        self._h = handle
        self.device = device

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.sepal_b200_close(self._h)
            self._h = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def info(self) -> dict:
        needed = _u64()
        self._lib.sepal_b200_info(self._h, None, 0, C.byref(needed))
        buf = C.create_string_buffer(needed.value)
        _check(self._lib.sepal_b200_info(self._h, buf, needed.value, C.byref(needed)))
        return json.loads(buf.value.decode())

    def status(self, stream=None) -> int:
        """Waits for the stream, returns and clears the device status word (0 = every kernel ran to completion)."""
        out = _i32()
        _check(self._lib.sepal_b200_status(self._h, _stream_ptr(stream), C.byref(out)))
        return out.value

    def set_static_weights(self, on: bool = True) -> None:
        """Promises (or withdraws the promise) that no kernel directly before a multiply of this context writes that multiply's weights
        (sepal_b200_set_static_weights): the kernels then request their first weight tiles before they wait for the kernel before them."""
        _check(self._lib.sepal_b200_set_static_weights(self._h, 1 if on else 0))

    def debug_leave_status(self, code: int, stale_counters: int = 0, stream=None) -> None:
        """Leaves the context as a kernel that gave up waiting would (sepal_b200_debug_leave_status): for tests of the recovery path."""
        _check(self._lib.sepal_b200_debug_leave_status(self._h, _stream_ptr(stream), code, stale_counters))

    def check_status(self, stream=None) -> None:
        st = self.status(stream)
        if st != 0:
            raise SepalB200Error(f"a kernel gave up waiting: status {st} (wait {st & 0xFF}, CTA {st >> 8})")

    # ---- launchers -------------------------------------------------------------------------------------------------------
    @staticmethod
    def _out(x, n_out: int, y, y_half: bool):
        """The output tensor: a new one, or the caller's after checking that the C ABI (which only sees a pointer and a row stride) would
        write inside it: [T, n_out], float16 or float32, on x's device, last dimension contiguous."""
        import torch

        if y is None:
            return torch.empty((x.shape[0], n_out), dtype=torch.float16 if y_half else torch.float32, device=x.device)
        if tuple(y.shape) != (x.shape[0], n_out):
            raise ValueError(f"the output must be [{x.shape[0]}, {n_out}], not {tuple(y.shape)}")
        if y.dtype not in (torch.float16, torch.float32) or y.device != x.device or (y.numel() > 0 and y.stride(-1) != 1):
            raise ValueError("the output must be float16 or float32, on the input's device, with a contiguous last dimension")
        return y

    def gemm_f16(self, x, w, y=None, *, epilogue: int = STORE, y_half: bool = True, config: int = -1, stream=None):
        """y = epilogue(x @ w.T): x [T, K] and w [N, K] float16 (last dimension contiguous), y float16 or float32."""
        import torch

        assert x.dtype == torch.float16 and w.dtype == torch.float16 and x.stride(-1) == 1 and w.stride(-1) == 1
        t, k = x.shape
        n = w.shape[0]
        if w.shape[1] != k or w.device != x.device:
            raise ValueError(f"x is [{t}, {k}] but w is {tuple(w.shape)} on {w.device}: the inner dimensions and the devices must agree")
        if y is not None:
            y_half = y.dtype == torch.float16
        y = self._out(x, n // 2 if epilogue == SWIGLU else n, y, y_half)
        _check(self._lib.sepal_b200_gemm_f16(self._h, x.data_ptr(), x.stride(0) if t > 1 else max(x.stride(0), k), w.data_ptr(),
                                             w.stride(0) if n > 1 else max(w.stride(0), k), y.data_ptr(), y.stride(0) if t > 1 else y.shape[1],
                                             1 if y_half else 0, t, n, k, epilogue, config, _stream_ptr(stream)))
        return y

    def quantize_group_s8(self, w32, stream=None):
        """float32 [N, K] -> (int8 [N, K], float32 [N, K / 128]) with the reference's group quantiser."""
        import torch

        assert w32.dtype == torch.float32 and w32.is_contiguous()
        n, k = w32.shape
        q = torch.empty((n, k), dtype=torch.int8, device=w32.device)
        s = torch.empty((n, k // GROUP), dtype=torch.float32, device=w32.device)
        _check(self._lib.sepal_b200_quantize_group_s8(w32.data_ptr(), k, q.data_ptr(), k, s.data_ptr(), k // GROUP, n, k, _stream_ptr(stream)))
        return q, s

    def prepare_w8g(self, q, s, stream=None) -> W8gWeight:
        """Weight placement of an int8-group matrix: q int8 [N, K] and s float32 [N, K / 128] -> W8gWeight."""
        import torch

        assert q.dtype == torch.int8 and s.dtype == torch.float32 and q.is_contiguous() and s.is_contiguous()
        n, k = q.shape
        groups = k // GROUP
        assert s.shape == (n, groups)
        ld_st = (n + 255) // 256 * 256  # rows padded to whole tiles (zeros): the kernels copy a tile's scales in 16-byte pieces
        st = torch.zeros((groups, ld_st), dtype=torch.float16, device=q.device)
        descale = torch.empty((2,), dtype=torch.float32, device=q.device)  # [0] the factor, [1] scratch for the maximum
        _check(self._lib.sepal_b200_prepare_w8g_scales(s.data_ptr(), groups, n, groups, st.data_ptr(), ld_st, descale.data_ptr(),
                                                       descale.data_ptr() + 4, _stream_ptr(stream)))
        return W8gWeight(q=q, scales=s, scales_t=st, descale=descale)

    def gemm_w8g(self, x, w: W8gWeight, y=None, *, epilogue: int = STORE, y_half: bool = True, config: int = -1, stream=None):
        """y = epilogue(x @ dequant(w).T): x [T, K] float16, w int8 groups."""
        import torch

        assert x.dtype == torch.float16 and x.stride(-1) == 1
        t, k = x.shape
        n = w.q.shape[0]
        if w.q.shape[1] != k or w.q.device != x.device:
            raise ValueError(f"x is [{t}, {k}] but the weights are {tuple(w.q.shape)} on {w.q.device}: the inner dimensions and the devices must agree")
        if y is not None:
            y_half = y.dtype == torch.float16
        y = self._out(x, n // 2 if epilogue == SWIGLU else n, y, y_half)
        _check(self._lib.sepal_b200_gemm_w8g(self._h, x.data_ptr(), x.stride(0) if t > 1 else max(x.stride(0), k), w.q.data_ptr(), w.q.stride(0),
                                             w.scales_t.data_ptr(), w.scales_t.stride(0), w.descale.data_ptr(), y.data_ptr(),
                                             y.stride(0) if t > 1 else y.shape[1], 1 if y_half else 0, t, n, k, epilogue, config, _stream_ptr(stream)))
        return y

    def quantize_rows_s8(self, w16, col_scale=None, stream=None):
        """float16 [N, K] -> (int8 [N, K], float32 [N]) with the reference's per-output-row quantiser (plain byte order)."""
        import torch

        assert w16.dtype == torch.float16 and w16.is_contiguous()
        n, k = w16.shape
        q = torch.empty((n, k), dtype=torch.int8, device=w16.device)
        sw = torch.empty((n,), dtype=torch.float32, device=w16.device)
        if col_scale is not None:
            assert col_scale.dtype == torch.float32 and col_scale.is_contiguous() and col_scale.numel() == k
        _check(self._lib.sepal_b200_quantize_rows_s8(w16.data_ptr(), k, q.data_ptr(), k, sw.data_ptr(), n, k,
                                                     col_scale.data_ptr() if col_scale is not None else None, _stream_ptr(stream)))
        return q, sw

    def gemm_w8r(self, x, q, sw, y=None, *, epilogue: int = STORE, y_half: bool = True, config: int = -1, stream=None):
        """y = epilogue(sw * (x @ q.T)): x [T, K] float16, q int8 [N, K], sw float32 [N] (one scale per output row)."""
        import torch

        assert x.dtype == torch.float16 and x.stride(-1) == 1 and q.dtype == torch.int8 and q.stride(-1) == 1 and sw.dtype == torch.float32
        t, k = x.shape
        n = q.shape[0]
        if q.shape[1] != k or sw.numel() != n or q.device != x.device or sw.device != x.device:
            raise ValueError(f"x is [{t}, {k}], q is {tuple(q.shape)}, sw has {sw.numel()} scales: the shapes and the devices must agree")
        if y is not None:
            y_half = y.dtype == torch.float16
        y = self._out(x, n // 2 if epilogue == SWIGLU else n, y, y_half)
        _check(self._lib.sepal_b200_gemm_w8r(self._h, x.data_ptr(), x.stride(0) if t > 1 else max(x.stride(0), k), q.data_ptr(), q.stride(0),
                                             sw.data_ptr(), y.data_ptr(), y.stride(0) if t > 1 else y.shape[1], 1 if y_half else 0, t, n, k,
                                             epilogue, config, _stream_ptr(stream)))
        return y

    def pack_gate_up(self, stacked, stream=None):
        """[gate; up] (2 I rows) -> the packed row order of the fused SwiGLU multiply."""
        import torch

        assert stacked.is_contiguous()
        rows, cols = stacked.shape
        out = torch.empty_like(stacked)
        nbytes = cols * stacked.element_size()
        _check(self._lib.sepal_b200_pack_gate_up(stacked.data_ptr(), nbytes, out.data_ptr(), nbytes, rows // 2, nbytes, _stream_ptr(stream)))
        return out

    def float_to_half(self, src, stream=None):
        import torch

        dst = torch.empty(src.shape, dtype=torch.float16, device=src.device)
        _check(self._lib.sepal_b200_float_to_half(src.data_ptr(), dst.data_ptr(), src.numel(), _stream_ptr(stream)))
        return dst

    @staticmethod
    def take_launch_count() -> int:
        return int(library().sepal_b200_take_launch_count())


class AttentionShape(C.Structure):
    """sepal_b200_attention_shape."""

    _fields_ = [("heads", _u32), ("kv_heads", _u32), ("head_dim", _u32), ("rotary_dims", _u32), ("rope_theta", C.c_double), ("eps", C.c_float),
                ("reserved", _u32)]


class AttentionRow(C.Structure):
    """sepal_b200_attention_row."""

    _fields_ = [("q_begin", _u32), ("length", _u32), ("kv_begin", _u32), ("context", _u32)]


def attention_prepare(ctx, shape, rows, q_gate, k, v, q_norm, k_norm, q_out, k_arena, v_arena, stream=None):
    """Norm, RoPE and cache append (sepal_b200_attention_prepare). rows: list of (q_begin, length, kv_begin, context); torch tensors."""
    import torch

    table = (AttentionRow * len(rows))(*[AttentionRow(*r) for r in rows])
    half = lambda t: 1 if t.dtype == torch.float16 else 0  # noqa: E731
    _check(ctx._lib.sepal_b200_attention_prepare(ctx._h, C.byref(shape), table, len(rows), q_gate.data_ptr(), q_gate.stride(0), half(q_gate), k.data_ptr(),
                                                 k.stride(0), half(k), v.data_ptr(), v.stride(0), half(v), q_norm.data_ptr(), k_norm.data_ptr(),
                                                 q_out.data_ptr(), q_out.stride(0), k_arena.data_ptr(), v_arena.data_ptr(), k_arena.shape[0], _stream_ptr(stream)))


def attention(ctx, shape, rows, q, k_arena, v_arena, gate, out, stream=None):
    """Causal grouped-query flash attention times sigmoid(gate) (sepal_b200_attention)."""
    import torch

    table = (AttentionRow * len(rows))(*[AttentionRow(*r) for r in rows])
    _check(ctx._lib.sepal_b200_attention(ctx._h, C.byref(shape), table, len(rows), q.shape[0], q.data_ptr(), q.stride(0), k_arena.data_ptr(), v_arena.data_ptr(),
                                         k_arena.shape[0], gate.data_ptr(), gate.stride(0), 1 if gate.dtype == torch.float16 else 0, out.data_ptr(),
                                         out.stride(0), _stream_ptr(stream)))


class DeltaNetShape(C.Structure):
    """sepal_b200_deltanet_shape."""

    _fields_ = [("key_heads", _u32), ("value_heads", _u32), ("head_dim", _u32), ("conv_kernel", _u32), ("eps", C.c_float), ("reserved", _u32)]


class DeltaNetRow(C.Structure):
    """sepal_b200_deltanet_row."""

    _fields_ = [("q_begin", _u32), ("length", _u32), ("slot", _u32), ("fresh", _u32)]


def deltanet(ctx, shape, rows, mixed, z, b, a, conv, a_log, dt_bias, norm, states, tails, out, stream=None):
    """The Gated DeltaNet core (sepal_b200_deltanet). rows: list of (q_begin, length, slot, fresh); mixed, z, b, a: torch bands of one
    dtype (float16 or float32); states [slots, value_heads, 128, 128] and tails [slots, K - 1, conv_dim] float32, updated in place."""
    import torch

    table = (DeltaNetRow * len(rows))(*[DeltaNetRow(*r) for r in rows])
    n = max((r[0] + r[1] for r in rows), default=0)
    kd, vd = shape.key_heads * shape.head_dim, shape.value_heads * shape.head_dim
    scratch = torch.empty(max(1, n * (264 * shape.key_heads + 2 * vd + 58 * shape.value_heads)), dtype=torch.float32, device=out.device)
    assert mixed.dtype == z.dtype == b.dtype == a.dtype
    _check(ctx._lib.sepal_b200_deltanet(ctx._h, C.byref(shape), table, len(rows), mixed.data_ptr(), mixed.stride(0), z.data_ptr(), z.stride(0), b.data_ptr(),
                                        b.stride(0), a.data_ptr(), a.stride(0), 1 if mixed.dtype == torch.float16 else 0, conv.data_ptr(), a_log.data_ptr(),
                                        dt_bias.data_ptr(), norm.data_ptr(), scratch.data_ptr(), states.data_ptr(), tails.data_ptr(), states.shape[0],
                                        out.data_ptr(), out.stride(0), _stream_ptr(stream)))
    return scratch  # kept alive by the caller until the stream has run


class TrunkConfig(C.Structure):
    """sepal_b200_trunk_config. The defaults are BASELINE's long-log geometry: 36 layers, hidden 2560, MLP 9728, 3 DeltaNet : 1 attention."""

    _fields_ = [("layers", _u32), ("hidden", _u32), ("intermediate", _u32), ("vocab", _u32), ("attn_q", _u32), ("attn_kv", _u32),
                ("dn_in", _u32), ("dn_v_offset", _u32), ("dn_v", _u32), ("max_call_tokens", _u32), ("mlp_int8", _u32), ("eps", C.c_float),
                ("seed", _u64), ("attn_o", _u32), ("attn_heads", _u32), ("attn_kv_heads", _u32), ("attn_head_dim", _u32), ("attn_rotary_dims", _u32),
                ("dn_key_heads", _u32), ("dn_value_heads", _u32), ("dn_conv_kernel", _u32), ("rope_theta", C.c_double)]

    def __init__(self, **kw):
        base = dict(layers=36, hidden=2560, intermediate=9728, vocab=151936, attn_q=4096, attn_kv=1024, dn_in=8192, dn_v_offset=4096, dn_v=2048,
                    max_call_tokens=4096, mlp_int8=0, eps=1e-6, seed=1, attn_o=0, attn_heads=0, attn_kv_heads=0, attn_head_dim=0, attn_rotary_dims=0,
                    dn_key_heads=0, dn_value_heads=0, dn_conv_kernel=4, rope_theta=1.0e7)
        base.update(kw)
        super().__init__(**base)


class Trunk:
    """The synthetic GEMM-chain trunk (sepal_b200_trunk_*): whole requests of host token ids in, final hidden states out."""

    WEIGHTS = {"embedding": 0, "norm_in": 1, "mix_in": 2, "mix_out": 3, "norm_post": 4, "gate_up": 5, "down": 6, "q_norm": 7, "k_norm": 8, "dn_conv": 9, "dn_a_log": 10,
               "dn_dt_bias": 11, "dn_norm": 12, "gate_up_scales": 13, "down_scales": 14}

    def __init__(self, device: int = 0, config: Optional[TrunkConfig] = None, checkpoint: "Optional[Checkpoint]" = None) -> None:
        self._lib = library()
        self.config = config if config is not None else TrunkConfig()
        handle = _vp()
        if checkpoint is None:
            _check(self._lib.sepal_b200_trunk_open(device, C.addressof(self.config), C.byref(handle)))
        else:
            _check(self._lib.sepal_b200_trunk_open_checkpoint(device, C.addressof(self.config), checkpoint._h, C.byref(handle)))
        self._h = handle
        flops, nbytes = _u64(), _u64()
        _check(self._lib.sepal_b200_trunk_info(self._h, C.byref(flops), C.byref(nbytes)))
        self.gemm_flops_per_token = flops.value
        self.weight_bytes = nbytes.value

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.sepal_b200_trunk_close(self._h)
            self._h = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def save(self, path: str) -> None:
        """The placed weights (stacked, interleaved, quantised) as one file that Trunk(checkpoint=Checkpoint(path)) copies back as it is."""
        _check(self._lib.sepal_b200_trunk_save(self._h, os.fsencode(path)))

    def run(self, tokens, want_all: bool = False):
        """tokens: uint32 numpy array. Returns (last hidden [hidden], all hidden [n, hidden] or None, device ms)."""
        import numpy as np

        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        n = tokens.shape[0]
        last = np.empty(self.config.hidden, np.float32)
        allh = np.empty((n, self.config.hidden), np.float32) if want_all else None
        times = (C.c_double * 2)()
        _check(self._lib.sepal_b200_trunk_run(self._h, tokens.ctypes.data, n, last.ctypes.data, allh.ctypes.data if want_all else None, times))
        return last, allh, float(times[0])

    def score(self, requests):
        """requests: a list of uint32 token arrays. They are packed into calls of up to max_call_tokens rows (short requests share a call).
        Returns (last hidden [n_requests, hidden], seconds until each request's result was complete on the device)."""
        import numpy as np

        offsets = np.zeros(len(requests) + 1, np.uint64)
        offsets[1:] = np.cumsum([len(r) for r in requests])
        flat = np.ascontiguousarray(np.concatenate([np.asarray(r, np.uint32) for r in requests])) if requests else np.zeros(0, np.uint32)
        last = np.empty((len(requests), self.config.hidden), np.float32)
        times = np.zeros(len(requests), np.float64)
        _check(self._lib.sepal_b200_trunk_score(self._h, len(requests), flat.ctypes.data, offsets.ctypes.data, last.ctypes.data, times.ctypes.data))
        return last, times

    def weight(self, which: str, layer: int = 0):
        """A stored weight as a numpy array (float16 matrices as flat arrays: reshape with the known geometry)."""
        import numpy as np

        code = self.WEIGHTS[which]
        needed = _u64()
        _check(self._lib.sepal_b200_trunk_weight(self._h, layer, code, None, 0, C.byref(needed)))
        is_norm = code in (1, 4, 7, 8, 9, 10, 11, 12, 13, 14)  # float32 arrays
        int8 = self.config.mlp_int8 and code in (5, 6)
        out = np.empty(needed.value // (4 if is_norm else 1 if int8 else 2), np.float32 if is_norm else np.int8 if int8 else np.float16)
        _check(self._lib.sepal_b200_trunk_weight(self._h, layer, code, out.ctypes.data, needed.value, C.byref(needed)))
        return out


class TensorInfo(C.Structure):
    """sepal_b200_tensor_info."""

    _fields_ = [("name", C.c_char * 256), ("dtype", _i32), ("rank", _u32), ("shape", _u64 * 8), ("data", _vp), ("bytes", _u64)]


# element type codes of sepal_b200_tensor_info.dtype -> numpy dtype (bfloat16 travels as its 16-bit patterns)
ELEMENT_TYPES = {0: "float32", 1: "float16", 2: "uint16", 3: "int8", 4: "uint8", 5: "int32", 6: "int64", 7: "float64", 8: "bool", 9: "int16",
                 10: "uint16", 11: "uint32", 12: "uint64"}
BF16 = 2


class Checkpoint:
    """A safetensors file or checkpoint directory, mapped and checked (sepal_b200_checkpoint_*). Host-only: needs no GPU."""

    def __init__(self, path: str) -> None:
        self._lib = library()
        handle = _vp()
        _check(self._lib.sepal_b200_checkpoint_open(os.fsencode(path), C.byref(handle)))
        self._h = handle

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.sepal_b200_checkpoint_close(self._h)
            self._h = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    def __len__(self) -> int:
        n = _u64()
        _check(self._lib.sepal_b200_checkpoint_count(self._h, C.byref(n)))
        return int(n.value)

    def _info(self, index: int = 0, name: Optional[str] = None) -> TensorInfo:
        info = TensorInfo()
        _check(self._lib.sepal_b200_checkpoint_tensor(self._h, index, name.encode() if name is not None else None, C.byref(info)))
        return info

    def names(self):
        return [self._info(i).name.decode() for i in range(len(self))]

    def tensor(self, name: str):
        """(numpy array copied out of the mapping, element type code)."""
        import numpy as np

        info = self._info(name=name)
        shape = tuple(int(info.shape[d]) for d in range(info.rank))
        dtype = np.dtype(ELEMENT_TYPES[info.dtype])
        raw = C.string_at(info.data, info.bytes) if info.bytes else b""
        return np.frombuffer(raw, dtype=dtype).reshape(shape).copy(), int(info.dtype)

    def metadata(self, key: str) -> str:
        needed = _u64()
        _check(self._lib.sepal_b200_checkpoint_metadata(self._h, key.encode(), None, 0, C.byref(needed)))
        buf = C.create_string_buffer(needed.value)
        _check(self._lib.sepal_b200_checkpoint_metadata(self._h, key.encode(), buf, needed.value, None))
        return buf.value.decode()

    @property
    def prefix(self) -> str:
        return self.metadata("__prefix__")


def write_tensor_file(path: str, tensors, metadata=None, bf16=()) -> None:
    """tensors: dict name -> numpy array (names in `bf16` hold bfloat16 bit patterns as uint16). Written in the order of the dict."""
    import numpy as np

    codes = {"float32": 0, "float16": 1, "int8": 3, "uint8": 4, "int32": 5, "int64": 6, "float64": 7, "bool": 8, "int16": 9, "uint16": 10, "uint32": 11,
             "uint64": 12}
    infos = (TensorInfo * len(tensors))()
    keep = []
    for i, (name, value) in enumerate(tensors.items()):
        a = np.ascontiguousarray(value)
        keep.append(a)
        infos[i].name = name.encode()
        infos[i].dtype = BF16 if name in bf16 else codes[a.dtype.name]
        infos[i].rank = a.ndim
        for d, extent in enumerate(a.shape):
            infos[i].shape[d] = extent
        infos[i].data = a.ctypes.data
        infos[i].bytes = a.nbytes
    metadata = metadata or {}
    keys = (C.c_char_p * len(metadata))(*[k.encode() for k in metadata])
    values = (C.c_char_p * len(metadata))(*[v.encode() for v in metadata.values()])
    _check(library().sepal_b200_tensor_file_write(os.fsencode(path), len(tensors), infos, len(metadata), keys, values))


class Model(C.Structure):
    """sepal_b200_model: the geometry of a served model (presets 0.8b, 2b, 4b, 9b)."""

    _fields_ = [(f, _u64) for f in ("layers", "hidden", "intermediate", "vocab", "attn_heads", "attn_kv_heads", "attn_head_dim", "dn_key_heads",
                                    "dn_value_heads", "dn_key_head_dim", "dn_value_head_dim", "conv_kernel", "attention_interval")]

    @classmethod
    def preset(cls, name: str) -> "Model":
        m = cls()
        _check(library().sepal_b200_model_preset(name.encode(), C.byref(m)))
        return m

    def weight_bytes(self, profile: str) -> int:
        out = _u64()
        _check(library().sepal_b200_plan_weight_bytes(C.byref(self), profile.encode(), C.byref(out)))
        return int(out.value)


class Provider:
    """Host-pointer GEMM: weights uploaded once, X uploaded and Y downloaded inside every call (numpy arrays or raw pointers)."""

    def __init__(self, device: int = 0, arena_bytes: int = 0) -> None:
        self._lib = library()
        handle = _vp()
        _check(self._lib.sepal_b200_provider_open(device, arena_bytes, C.byref(handle)))
        self._h = handle
        self._shapes = {}

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.sepal_b200_provider_close(self._h)
            self._h = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    @staticmethod
    def _dtype_code(a) -> int:
        import numpy as np

        if a.dtype == np.float32:
            return F32
        if a.dtype == np.float16:
            return F16
        raise TypeError("float32 or float16 arrays only")

    def upload_weights(self, w) -> int:
        import numpy as np

        w = np.ascontiguousarray(w)
        wid = _u32()
        _check(self._lib.sepal_b200_provider_upload_weights(self._h, w.ctypes.data, self._dtype_code(w), w.shape[0], w.shape[1], C.byref(wid)))
        self._shapes[wid.value] = w.shape
        return wid.value

    def upload_weights_w8g(self, w) -> int:
        import numpy as np

        w = np.ascontiguousarray(w, dtype=np.float32)
        wid = _u32()
        _check(self._lib.sepal_b200_provider_upload_weights_w8g(self._h, w.ctypes.data, w.shape[0], w.shape[1], C.byref(wid)))
        self._shapes[wid.value] = w.shape
        return wid.value

    def gemm_f(self, x, weight_id: int, y=None, beta: float = 0.0):
        import numpy as np

        x = np.ascontiguousarray(x)
        n, k = self._shapes[weight_id]
        assert x.shape[1] == k
        if y is None:
            y = np.empty((x.shape[0], n), np.float32)
        assert y.dtype == np.float32 and y.flags.c_contiguous and y.shape == (x.shape[0], n)
        _check(self._lib.sepal_b200_provider_gemm_f(self._h, x.ctypes.data, self._dtype_code(x), x.shape[0], weight_id, y.ctypes.data, beta))
        return y

    def gemm_f_raw(self, x_ptr: int, x_dtype: int, t: int, weight_id: int, y_ptr: int, beta: float = 0.0) -> None:
        _check(self._lib.sepal_b200_provider_gemm_f(self._h, x_ptr, x_dtype, t, weight_id, y_ptr, beta))


def gemm_f16_noalloc(x, w, y, *, epilogue: int = STORE, stream=None, wait: bool = True) -> int:
    """sepal_b200_gemm_f16_noalloc on CUDA tensors of the current device: y = epilogue(x @ w.T) without a Context and without any
    device allocation inside the library. Returns the kernel status word when `wait` (0 = fine), else 0 right after enqueueing."""
    import torch

    assert x.dtype == torch.float16 and w.dtype == torch.float16 and x.stride(-1) == 1 and w.stride(-1) == 1
    t, k = x.shape
    n = w.shape[0]
    if w.shape[1] != k or w.device != x.device:
        raise ValueError(f"x is [{t}, {k}] but w is {tuple(w.shape)} on {w.device}: the inner dimensions and the devices must agree")
    Context._out(x, n // 2 if epilogue == SWIGLU else n, y, y.dtype == torch.float16)
    status = _i32(0)
    _check(library().sepal_b200_gemm_f16_noalloc(x.data_ptr(), x.stride(0) if t > 1 else max(x.stride(0), k), w.data_ptr(),
                                                 w.stride(0) if n > 1 else max(w.stride(0), k), y.data_ptr(), y.stride(0) if t > 1 else y.shape[1],
                                                 1 if y.dtype == torch.float16 else 0, t, n, k, epilogue, _stream_ptr(stream),
                                                 C.byref(status) if wait else None))
    return status.value


def host_alloc(nbytes: int) -> int:
    out = _vp()
    _check(library().sepal_b200_host_alloc(nbytes, C.byref(out)))
    return out.value


def host_free(ptr: int) -> None:
    library().sepal_b200_host_free(ptr)
