"""ctypes loaders for the checkers. TEST INFRASTRUCTURE, not product code.

`Oracle`  -> oracle/libsepal_oracle.so, the C restatement (sepal_oracle.c).
`Ref`     -> oracle/_ref/libsepal_ref.so, the reference's own CPU GEMM compiled from its sources (ref_shim.cpp, Makefile).
`RefGpu`  -> oracle/_ref/libsepal_ref_gpu.so, the reference's own GPU multiplies compiled from its sources for sm_100, and
             the cuBLAS call its engine makes (ref_gpu_shim.cu, Makefile).

Only tests/, the smoke check and the benchmark's baseline legs import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libsepal_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libsepal_ref.so")
REF_GPU_SO = os.path.join(HERE, "_ref", "libsepal_ref_gpu.so")


def reference_root() -> str:
    """Where the reference tree is: the environment variable SEPAL_REFERENCE, else a directory `reference` beside this repository."""
    return os.environ.get("SEPAL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(dtype=np.float64, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(dtype=np.int8, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_sz = C.c_size_t


def build(want_ref: bool = True) -> None:
    """Compile the checkers (make in oracle/). The reference library is built only where the reference tree exists."""
    targets = ["oracle"]
    root = reference_root()
    if want_ref and os.path.exists(os.path.join(root, "runner", "src", "cpu", "gemm.cpp")):
        targets += ["ref", "ref_gpu"]
    subprocess.run(["make", "-s", "-C", HERE, f"REF={root}", *targets], check=True)


def f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    """The C restatement. Every method takes and returns float32 / int8 numpy arrays (16-bit operands widened exactly)."""

    def __init__(self) -> None:
        if not os.path.exists(ORACLE_SO):
            build(want_ref=False)
        L = self.lib = C.CDLL(ORACLE_SO)
        L.oracle_f32_to_bf16.restype = C.c_uint16
        L.oracle_f32_to_bf16.argtypes = [C.c_float]
        L.oracle_f32_to_f16.restype = C.c_uint16
        L.oracle_f32_to_f16.argtypes = [C.c_float]
        L.oracle_f16_to_f32.restype = C.c_float
        L.oracle_f16_to_f32.argtypes = [C.c_uint16]
        L.oracle_bf16_to_f32.restype = C.c_float
        L.oracle_bf16_to_f32.argtypes = [C.c_uint16]
        L.oracle_gemm_f64acc.argtypes = [_f32p, _sz, _f32p, _sz, _f32p, _sz, _sz, _sz, _sz, C.c_float]
        L.oracle_gemm_fma_chain.argtypes = [_f32p, _sz, _f32p, _sz, _f32p, _sz, _sz, _sz, _sz]
        L.oracle_gemm_f64acc_sample.argtypes = [_f32p, _sz, _f32p, _sz, _sz, _u32p, _u32p, _sz, _f64p]
        L.oracle_rmsnorm_f32_ordered.restype = C.c_int
        L.oracle_rmsnorm_f32_ordered.argtypes = [_f32p, _sz, _f32p, _sz, _sz, _sz, _f32p, C.c_float]
        L.oracle_quantize_rows_s8.restype = C.c_int
        L.oracle_quantize_rows_s8.argtypes = [_f32p, _sz, _i8p, _sz, _f32p, _sz, _sz, C.c_void_p]
        L.oracle_quantize_group_s8.restype = C.c_int
        L.oracle_quantize_group_s8.argtypes = [_f32p, _sz, _i8p, _sz, _f32p, _sz, _sz, _sz]
        L.oracle_dequant_group_s8.argtypes = [_i8p, _sz, _f32p, _sz, _f32p, _sz, _sz, _sz]
        L.oracle_swiglu.restype = C.c_float
        L.oracle_swiglu.argtypes = [C.c_float, C.c_float]
        L.oracle_pack_gate_up_source.restype = _sz
        L.oracle_pack_gate_up_source.argtypes = [_sz, _sz]
        L.oracle_swiglu_packed.argtypes = [_f32p, _sz, _f32p, _sz, _sz, _sz]
        L.oracle_add.argtypes = [_f32p, _sz, _f32p, _sz, _sz, _sz]
        L.oracle_rmsnorm.argtypes = [_f32p, _sz, _f32p, _sz, _sz, _sz, _f32p, C.c_double]

    def gemm(self, x, w, y0=None, beta: float = 0.0) -> np.ndarray:
        """float64-accumulated product x [T,K] . w[N,K]^T (+ beta y0), rounded to float32 once."""
        x, w = f32(x), f32(w)
        t, k = x.shape
        n = w.shape[0]
        assert w.shape[1] == k
        y = np.zeros((t, n), np.float32) if y0 is None else f32(y0).copy()
        self.lib.oracle_gemm_f64acc(x, k, w, k, y, n, t, n, k, beta)
        return y

    def gemm_fma_chain(self, x, w) -> np.ndarray:
        x, w = f32(x), f32(w)
        t, k = x.shape
        n = w.shape[0]
        y = np.zeros((t, n), np.float32)
        self.lib.oracle_gemm_fma_chain(x, k, w, k, y, n, t, n, k)
        return y

    def gemm_sample(self, x, w, rows, cols) -> np.ndarray:
        x, w = f32(x), f32(w)
        rows = np.ascontiguousarray(rows, np.uint32)
        cols = np.ascontiguousarray(cols, np.uint32)
        out = np.zeros(rows.shape[0], np.float64)
        self.lib.oracle_gemm_f64acc_sample(x, x.shape[1], w, w.shape[1], x.shape[1], rows, cols, rows.shape[0], out)
        return out

    def rmsnorm_ordered(self, x, w, eps):
        """The norm with the float32 arithmetic and summation order of the reference's CUDA kernel (bit for bit); float32 result."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        w = np.ascontiguousarray(w, dtype=np.float32)
        rows, cols = x.shape
        y = np.empty_like(x)
        if self.lib.oracle_rmsnorm_f32_ordered(x, cols, y, cols, rows, cols, w, np.float32(eps)) != 0:
            raise ValueError("oracle_rmsnorm_f32_ordered: the row length must be a multiple of 4")
        return y

    def quantize_rows_s8(self, w, col_scale=None):
        """float32 values on the binary16 grid [N, K] -> (int8 [N, K], float32 [N]): the reference's per-output-row quantiser."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        n, k = w.shape
        q = np.empty((n, k), dtype=np.int8)
        s = np.empty((n,), dtype=np.float32)
        cs = None
        if col_scale is not None:
            cs = np.ascontiguousarray(col_scale, dtype=np.float32)
            assert cs.shape == (k,)
        if self.lib.oracle_quantize_rows_s8(w, k, q, k, s, n, k, cs.ctypes.data if cs is not None else None) != 0:
            raise ValueError("oracle_quantize_rows_s8 rejected its arguments")
        return q, s

    def quantize_group_s8(self, w):
        w = f32(w)
        n, k = w.shape
        q = np.zeros((n, k), np.int8)
        s = np.zeros((n, k // 128), np.float32)
        if self.lib.oracle_quantize_group_s8(w, k, q, k, s, k // 128, n, k) != 0:
            raise ValueError("K must be a multiple of 128")
        return q, s

    def dequant_group_s8(self, q, s) -> np.ndarray:
        q = np.ascontiguousarray(q, np.int8)
        s = f32(s)
        n, k = q.shape
        wd = np.zeros((n, k), np.float32)
        self.lib.oracle_dequant_group_s8(q, k, s, s.shape[1], wd, k, n, k)
        return wd

    def swiglu_packed(self, acc, inter: int) -> np.ndarray:
        acc = f32(acc)
        t = acc.shape[0]
        out = np.zeros((t, inter), np.float32)
        self.lib.oracle_swiglu_packed(acc, acc.shape[1], out, inter, t, inter)
        return out

    def pack_gate_up(self, gate, up) -> np.ndarray:
        """[gate; up] -> the packed row order of the fused SwiGLU multiply (blocks of 64 gate rows, 64 up rows)."""
        gate, up = np.asarray(gate), np.asarray(up)
        inter = gate.shape[0]
        stacked = np.concatenate([gate, up], axis=0)
        src = np.array([self.lib.oracle_pack_gate_up_source(p, inter) for p in range(2 * inter)], np.int64)
        return np.ascontiguousarray(stacked[src])

    def add(self, y, acc) -> np.ndarray:
        y = f32(y).copy()
        acc = f32(acc)
        self.lib.oracle_add(y, y.shape[1], acc, acc.shape[1], y.shape[0], y.shape[1])
        return y

    def rmsnorm(self, x, w, eps: float = 1e-6) -> np.ndarray:
        x, w = f32(x), f32(w)
        y = np.zeros_like(x)
        self.lib.oracle_rmsnorm(x, x.shape[1], y, x.shape[1], x.shape[0], x.shape[1], w, eps)
        return y

    def to_f16_grid(self, a) -> np.ndarray:
        """Round float32 values to binary16 and back (numpy's conversion is round-to-nearest-even, as the oracle's scalar one)."""
        return f32(a).astype(np.float16).astype(np.float32)

    def to_bf16_grid(self, a) -> np.ndarray:
        bits = f32(a).view(np.uint32).astype(np.uint64)
        nan = (bits & 0x7FFFFFFF) > 0x7F800000
        rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
        rounded = np.where(nan, ((bits >> 16) | 0x40) << 16, rounded)
        return rounded.astype(np.uint32).view(np.float32).reshape(np.shape(a))


class Ref:
    """The reference's own CPU GEMM (compiled from its sources). `available()` is False where it was never built."""

    KINDS = {"f32": 0, "bf16": 1, "i8": 2}

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def __init__(self) -> None:
        if not self.available():
            raise RuntimeError("oracle/_ref/libsepal_ref.so is not built (needs the reference tree: make -C oracle ref)")
        L = self.lib = C.CDLL(REF_SO)
        L.ref_last_error.restype = C.c_char_p
        L.ref_pool_threads.restype = C.c_uint
        L.ref_pool_threads.argtypes = [C.c_uint]
        L.ref_variant_name.restype = C.c_char_p
        L.ref_variant_name.argtypes = [C.c_int, C.c_char_p]
        L.ref_cpu_brand.restype = C.c_char_p
        L.ref_float_to_bf16.restype = C.c_uint16
        L.ref_float_to_bf16.argtypes = [C.c_float]
        L.ref_cpu_gemm.restype = C.c_int
        L.ref_cpu_gemm.argtypes = [C.c_int, C.c_char_p, C.c_uint, _f32p, _sz, _sz, _sz, _f32p, _sz, _sz, _f32p, _sz, C.c_int]
        L.ref_cpu_gemm_swiglu.restype = C.c_int
        L.ref_cpu_gemm_swiglu.argtypes = [C.c_int, C.c_char_p, C.c_uint, _f32p, _sz, _sz, _sz, _f32p, _f32p, _sz, _sz, _f32p, _sz]
        L.ref_pack.restype = C.c_void_p
        L.ref_pack.argtypes = [C.c_int, C.c_char_p, C.c_uint, _f32p, _sz, _sz, _sz]
        L.ref_packed_free.argtypes = [C.c_void_p]
        L.ref_packed_run.restype = C.c_int
        L.ref_packed_run.argtypes = [C.c_void_p, C.c_uint, _f32p, _sz, _sz, _f32p, _sz, C.c_int, _f64p]
        L.ref_gemm_f64acc.restype = C.c_int
        L.ref_gemm_f64acc.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, _sz, _sz, _sz, _f32p, C.c_float]
        L.ref_rmsnorm_rows.restype = C.c_int
        L.ref_rmsnorm_rows.argtypes = [C.c_uint, _f32p, _sz, _f32p, _sz, _sz, _sz, _f32p, C.c_double]
        d, u = C.c_double, C.c_uint
        L.ref_attention_core.restype = C.c_int
        L.ref_attention_core.argtypes = [_f64p, _f64p, _f64p, _f64p, _f64p, _f64p, _sz, _f64p, _f64p, _sz, u, u, u, u, d, d, _f64p, _f64p, _f64p]
        L.ref_deltanet_core.restype = C.c_int
        L.ref_deltanet_core.argtypes = [_f64p] * 10 + [_sz, u, u, u, u, u, d, _f64p, _f64p, _f64p]

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def threads(self, threads: int = 0) -> int:
        return int(self.lib.ref_pool_threads(threads))

    def variant(self, kind: str = "bf16", isa: str = "") -> str:
        return self.lib.ref_variant_name(self.KINDS[kind], isa.encode()).decode()

    def brand(self) -> str:
        return self.lib.ref_cpu_brand().decode()

    def cpu_gemm(self, x, w, kind: str = "bf16", isa: str = "", threads: int = 0, y0=None) -> np.ndarray:
        x, w = f32(x), f32(w)
        t, k = x.shape
        n = w.shape[0]
        y = np.zeros((t, n), np.float32) if y0 is None else f32(y0).copy()
        self._check(self.lib.ref_cpu_gemm(self.KINDS[kind], isa.encode(), threads, x, k, t, k, w, k, n, y, n, 0 if y0 is None else 1))
        return y

    def cpu_gemm_swiglu(self, x, gate, up, kind: str = "bf16", isa: str = "", threads: int = 0) -> np.ndarray:
        x, gate, up = f32(x), f32(gate), f32(up)
        t, k = x.shape
        n = gate.shape[0]
        y = np.zeros((t, n), np.float32)
        self._check(self.lib.ref_cpu_gemm_swiglu(self.KINDS[kind], isa.encode(), threads, x, k, t, k, gate, up, k, n, y, n))
        return y

    def gemm_f64acc(self, x, w, beta: float = 0.0, y0=None) -> np.ndarray:
        """The reference provider; x and w may be float32 or float16 arrays."""
        codes = {np.dtype(np.float32): 0, np.dtype(np.float16): 1}
        x = np.ascontiguousarray(x)
        w = np.ascontiguousarray(w)
        t, k = x.shape
        n = w.shape[0]
        y = np.zeros((t, n), np.float32) if y0 is None else f32(y0).copy()
        self._check(self.lib.ref_gemm_f64acc(x.ctypes.data, codes[x.dtype], w.ctypes.data, codes[w.dtype], t, n, k, y, beta))
        return y

    def rmsnorm_rows(self, x, w1, eps: float = 1e-6, threads: int = 0) -> np.ndarray:
        x, w1 = f32(x), f32(w1)
        y = np.zeros_like(x)
        self._check(self.lib.ref_rmsnorm_rows(threads, x, x.shape[1], y, x.shape[1], x.shape[0], x.shape[1], w1, eps))
        return y

    def attention_core(self, q_gate, k, v, q_norm, k_norm, positions, heads, kv_heads, head_dim, rotary_dims, theta, eps, ctx_keys=None, ctx_values=None):
        """The reference's attention mixer between its projections (float64 template code). -> (gated output [T, heads * hd], this run's
        keys [T, kvh, hd] (normed, rotated), values [T, kvh, hd]). ctx_keys / ctx_values [C, kvh, hd]: the tokens before this run."""
        f = lambda a: np.ascontiguousarray(a, np.float64)
        q_gate, k, v = f(q_gate), f(k), f(v)
        t = q_gate.shape[0]
        context = 0 if ctx_keys is None else int(np.shape(ctx_keys)[0])
        ck = f(ctx_keys).reshape(-1) if context else np.zeros(1)
        cv = f(ctx_values).reshape(-1) if context else np.zeros(1)
        out = np.zeros((t, heads * head_dim))
        keys = np.zeros((t, kv_heads, head_dim))
        values = np.zeros((t, kv_heads, head_dim))
        self._check(self.lib.ref_attention_core(q_gate, k, v, f(q_norm), f(k_norm), f(positions), t, ck, cv, context, heads, kv_heads, head_dim, rotary_dims,
                                                float(theta), float(eps), out, keys.reshape(-1), values.reshape(-1)))
        return out, keys, values

    def deltanet_core(self, mixed, z, b, a, conv, a_log, dt_bias, norm, key_heads, value_heads, dim, eps, state=None, tail=None):
        """The reference's Gated DeltaNet mixer between its projections (float64 template code), heads of `dim` for keys and values.
        -> (out [T, value_heads * dim], state [value_heads, dim, dim], tail [taps - 1, conv_dim])."""
        f = lambda x: np.ascontiguousarray(x, np.float64)
        mixed, conv = f(mixed), f(conv)
        t, conv_dim = mixed.shape
        taps = conv.shape[1]
        state = np.zeros((value_heads, dim, dim)) if state is None else f(state)
        tail = np.zeros((taps - 1, conv_dim)) if tail is None else f(tail)
        out = np.zeros((t, value_heads * dim))
        state_out, tail_out = np.zeros_like(state), np.zeros_like(tail)
        self._check(self.lib.ref_deltanet_core(mixed.reshape(-1), f(z).reshape(-1), f(b).reshape(-1), f(a).reshape(-1), conv.reshape(-1), f(a_log), f(dt_bias), f(norm),
                                               state.reshape(-1), tail.reshape(-1) if tail.size else np.zeros(1), t, key_heads, value_heads, dim, dim, taps, float(eps),
                                               out.reshape(-1), state_out.reshape(-1), tail_out.reshape(-1) if tail_out.size else np.zeros(1)))
        return out, state_out, tail_out

    def time_gemm(self, x, w, kind: str = "bf16", isa: str = "", threads: int = 0, reps: int = 5):
        """(pack seconds, product seconds) per repeat, weights packed once, as the reference's own bench times it."""
        x, w = f32(x), f32(w)
        t, k = x.shape
        n = w.shape[0]
        handle = self.lib.ref_pack(self.KINDS[kind], isa.encode(), threads, w, k, n, k)
        if not handle:
            raise RuntimeError(self.lib.ref_last_error().decode())
        y = np.zeros((t, n), np.float32)
        out = []
        sec = np.zeros(2, np.float64)
        try:
            for _ in range(reps):
                self._check(self.lib.ref_packed_run(handle, threads, x, k, t, y, n, 0, sec))
                out.append((float(sec[0]), float(sec[1])))
        finally:
            self.lib.ref_packed_free(handle)
        return out, y


class RefGpu:
    """The reference's own GPU multiplies and its cuBLAS call, on torch CUDA tensors. `available()` is False where it was never built."""

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_GPU_SO)

    def __init__(self) -> None:
        if not self.available():
            raise RuntimeError("oracle/_ref/libsepal_ref_gpu.so is not built (needs the reference tree: make -C oracle ref_gpu)")
        L = self.lib = C.CDLL(REF_GPU_SO)
        p, z, i, u = C.c_void_p, C.c_size_t, C.c_int, C.c_uint
        L.ref_gpu_last_error.restype = C.c_char_p
        L.ref_gpu_gemm_nt.argtypes = [p, z, p, z, p, z, i, z, z, z, i, u, i, p]
        L.ref_gpu_quantize_weights_s8.argtypes = [p, z, p, p, z, z, i, p]
        L.ref_gpu_gemm_w8a16.argtypes = [p, z, p, z, p, p, z, i, z, z, z, i, p]
        L.ref_gpu_gemm_simt.argtypes = [p, z, p, z, p, z, i, p, z, z, z, z, i, i, p]
        L.ref_gpu_quantize_group_s8.argtypes = [p, z, p, z, p, z, z, z, p]
        L.ref_gpu_cublas_gemm.argtypes = [p, z, p, p, z, i, z, z, z, i, p]

    def _check(self, rc: int) -> None:
        if rc != 0:
            raise RuntimeError(self.lib.ref_gpu_last_error().decode())

    @staticmethod
    def _stream() -> int:
        import torch

        return int(torch.cuda.current_stream().cuda_stream)

    def gemm_nt(self, x, w, y_half: bool = False, accumulate: int = 0, flush_k: int = 0, config: int = -1, y=None):
        """launch_gemm_nt: x [T, K], w [N, K] float16 CUDA tensors -> y [T, N] float32 (or float16)."""
        import torch

        t, k = x.shape
        n = w.shape[0]
        if y is None:
            y = torch.empty((t, n), dtype=torch.float16 if y_half else torch.float32, device=x.device)
        self._check(self.lib.ref_gpu_gemm_nt(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), y.data_ptr(), y.stride(0), int(y_half), t, n, k,
                                             accumulate, flush_k, config, self._stream()))
        return y

    def cublas(self, x, w, y_half: bool = False, compute16: bool = False, y=None):
        """cublasGemmEx as the reference's engine calls it (COMPUTE_32F, or COMPUTE_16F with a float16 result)."""
        import torch

        t, k = x.shape
        n = w.shape[0]
        assert w.is_contiguous()
        if y is None:
            y = torch.empty((t, n), dtype=torch.float16 if (y_half or compute16) else torch.float32, device=x.device)
        self._check(self.lib.ref_gpu_cublas_gemm(x.data_ptr(), x.stride(0), w.data_ptr(), y.data_ptr(), y.stride(0), int(y.dtype == torch.float16), t, n, k,
                                                 int(compute16), self._stream()))
        return y

    def quantize_group_s8(self, w32):
        """launch_quantize_group_s8: float32 [N, K] -> (int8 [N, K], float32 [N, K / 128])."""
        import torch

        n, k = w32.shape
        q = torch.empty((n, k), dtype=torch.int8, device=w32.device)
        s = torch.empty((n, k // 128), dtype=torch.float32, device=w32.device)
        self._check(self.lib.ref_gpu_quantize_group_s8(w32.data_ptr(), w32.stride(0), q.data_ptr(), k, s.data_ptr(), k // 128, n, k, self._stream()))
        return q, s

    def gemm_simt(self, x32, w, scales=None, kind: int = 2, epilogue: int = 0, config: int = -1, y=None):
        """launch_gemm_simt: x float32 [T, K]; w int8 [N, K] with scales [N, K / 128] (kind 2), or float32 (kind 0). y float32, in place for Add."""
        import torch

        t, k = x32.shape
        n = w.shape[0]
        if y is None:
            y = torch.zeros((t, n // 2 if epilogue == 2 else n), dtype=torch.float32, device=x32.device)
        self._check(self.lib.ref_gpu_gemm_simt(x32.data_ptr(), x32.stride(0), w.data_ptr(), w.stride(0), scales.data_ptr() if scales is not None else None,
                                               scales.stride(0) if scales is not None else 0, kind, y.data_ptr(), y.stride(0), t, n, k, epilogue, config,
                                               self._stream()))
        return y

    def quantize_weights_s8(self, w16, pairs: bool):
        """launch_quantize_weights_s8: float16 [N, K] -> (int8 [N, K] in the Plain or Fp16Pairs layout, float32 [N])."""
        import torch

        n, k = w16.shape
        q = torch.empty((n, k), dtype=torch.int8, device=w16.device)
        s = torch.empty((n,), dtype=torch.float32, device=w16.device)
        self._check(self.lib.ref_gpu_quantize_weights_s8(w16.data_ptr(), w16.stride(0), q.data_ptr(), s.data_ptr(), n, k, 1 if pairs else 0, self._stream()))
        return q, s

    def gemm_w8a16(self, x, wq_pairs, sw, y_half: bool = False, config: int = -1):
        """launch_gemm_w8a16: x float16 [T, K], wq int8 [N, K] in the Fp16Pairs layout, sw float32 [N]."""
        import torch

        t, k = x.shape
        n = wq_pairs.shape[0]
        y = torch.empty((t, n), dtype=torch.float16 if y_half else torch.float32, device=x.device)
        self._check(self.lib.ref_gpu_gemm_w8a16(x.data_ptr(), x.stride(0), wq_pairs.data_ptr(), wq_pairs.stride(0), sw.data_ptr(), y.data_ptr(), y.stride(0),
                                                int(y_half), t, n, k, config, self._stream()))
        return y
