"""The CPU oracle (oracle/sepal_oracle.c) against the reference: its committed golden outputs (tests/golden/golden.npz, produced by
the reference's own CPU code) and, where oracle/_ref is built, the reference's code itself. No GPU."""
import numpy as np
import pytest

CASES = ["g0", "g1", "g2", "g3"]


def rel_fro(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


@pytest.mark.parametrize("name", CASES)
def test_f64acc_product_is_bit_equal_to_the_reference_provider(oracle, golden, name):
    # runner/src/provider/gemm_ref.cpp:58-78: float64 accumulation in k order, one rounding
    x, w = golden[f"{name}_x"].astype(np.float32), golden[f"{name}_w"].astype(np.float32)
    assert np.array_equal(oracle.gemm(x, w), golden[f"{name}_y_f64acc"])


@pytest.mark.parametrize("name", CASES)
def test_fma_chain_is_bit_equal_to_cpu_bf16_avx2(oracle, golden, name):
    # the AVX2 bf16 kernels are one fp32 fma chain in increasing k on exactly widened weights (runner/tests/test_cpu_gemm.cpp:385-397);
    # the fixture's operands are bf16-exact, so rounding W changes nothing
    x, w = golden[f"{name}_x"].astype(np.float32), golden[f"{name}_w"].astype(np.float32)
    assert np.array_equal(oracle.gemm_fma_chain(x, oracle.to_bf16_grid(w)), golden[f"{name}_y_cpu_bf16_avx2"])


@pytest.mark.parametrize("name", CASES)
def test_cpu_bf16_result_is_within_its_own_bound_of_the_oracle(oracle, golden, name):
    # runner/tests/test_cpu_gemm.cpp:140-157: |y - exact| <= 2e-6 * sum |x w| per element
    x, w = golden[f"{name}_x"].astype(np.float32), golden[f"{name}_w"].astype(np.float32)
    exact = oracle.gemm(x, w).astype(np.float64)
    bound = 2e-6 * (np.abs(x).astype(np.float64) @ np.abs(w).astype(np.float64).T) + 1e-30
    assert np.all(np.abs(golden[f"{name}_y_cpu_bf16"] - exact) <= bound)
    assert rel_fro(golden[f"{name}_y_cpu_bf16"], exact) < 1e-5


def test_beta_and_accumulate(oracle, golden):
    x, w = golden["g0_x"].astype(np.float32), golden["g0_w"].astype(np.float32)
    y0 = golden["acc_y0"]
    assert np.array_equal(oracle.gemm(x, w, y0=y0, beta=1.0), golden["acc_y_f64acc_beta1"])
    assert np.array_equal(oracle.gemm(x, w, y0=y0, beta=-0.5), golden["acc_y_f64acc_betam05"])
    # the residual epilogue is one float32 addition to the finished sum (runner/cuda/src/gemm_simt_kernels.cu:223-226)
    added = oracle.add(y0, oracle.gemm(x, w))
    assert rel_fro(added, golden["acc_y_cpu"]) < 1e-6


def test_swiglu_pair(oracle, golden):
    x = golden["sw_x"].astype(np.float32)
    gate, up = golden["sw_gate"].astype(np.float32), golden["sw_up"].astype(np.float32)
    inter = gate.shape[0]
    packed = oracle.pack_gate_up(gate, up)
    # the packed order: block b holds gate rows 64 b .. 64 b + 63 then up rows 64 b .. 64 b + 63 (gemm_simt_kernels.hpp:72-77)
    assert np.array_equal(packed[0:64], gate[0:64]) and np.array_equal(packed[64:128], up[0:64]) and np.array_equal(packed[128:192], gate[64:128])
    acc = oracle.gemm(x, packed)
    got = oracle.swiglu_packed(acc, inter)
    # the CPU engine's exp polynomial differs from libm by about 1e-7 relative (runner/src/cpu/vmath.hpp:16-38)
    assert rel_fro(got, golden["sw_y_cpu_f32_avx2"]) < 2e-6
    assert rel_fro(got, golden["sw_y_cpu_bf16"]) < 2e-6
    # against the textbook definition
    g, u = acc[:, :64].astype(np.float64), acc[:, 64:128].astype(np.float64)
    assert np.allclose(got[:, :64], g / (1 + np.exp(-g)) * u, rtol=1e-5, atol=1e-7)


def test_rmsnorm(oracle, golden):
    got = oracle.rmsnorm(golden["rn_x"], golden["rn_w"], 1e-6)
    assert np.allclose(got, golden["rn_y"], rtol=2e-6, atol=1e-7)


def test_ordered_rmsnorm_agrees_with_the_float64_form(oracle):
    """The float32 chain in the reference kernel's order against the float64 mean: a few units in the last place, never more."""
    rng = np.random.default_rng(41)
    for cols in (4, 256, 1024, 2560, 4100):
        x = (rng.standard_normal((5, cols)) * 3).astype(np.float32)
        w = (rng.standard_normal(cols) * 0.1).astype(np.float32)
        got = oracle.rmsnorm_ordered(x, w, 1e-6)
        want = oracle.rmsnorm(x, w, 1e-6)
        assert np.abs(got - want).max() <= 4e-6 * np.abs(want).max()
    one = np.zeros((1, 8), np.float32)
    one[0, :4] = [3.0, 4.0, 0.0, 0.0]                    # sum of squares 25, mean 25 / 8, exactly representable steps
    y = oracle.rmsnorm_ordered(one, np.zeros(8, np.float32), 0.0)
    rms = np.sqrt(np.float32(25.0) / np.float32(8.0))
    assert y[0, 0] == np.float32(3.0) / rms and y[0, 1] == np.float32(4.0) / rms and y[0, 2] == 0.0


def test_bf16_rounding(oracle, golden):
    got = np.array([oracle.lib.oracle_f32_to_bf16(float(v)) for v in golden["bf_vals"]], np.uint16)
    assert np.array_equal(got, golden["bf_bits"])
    assert np.array_equal(oracle.to_bf16_grid(golden["bf_vals"]).view(np.uint32) >> 16, golden["bf_bits"])


def test_f16_rounding_matches_ieee(oracle):
    rng = np.random.default_rng(7)
    vals = (rng.standard_normal(20000) * 10.0 ** rng.integers(-9, 5, 20000)).astype(np.float32)
    vals = np.concatenate([vals, np.array([65504.0, 65519.99, 65520.0, 2.9802322e-08, 2.9802326e-08, 8.940697e-08, 6.1035156e-05, 0.0, -0.0], np.float32)])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.lib.oracle_f32_to_f16(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, want)
    back = np.array([oracle.lib.oracle_f16_to_f32(int(b)) for b in range(0, 0x7C00, 7)], np.float32)
    assert np.array_equal(back, np.arange(0, 0x7C00, 7, dtype=np.uint16).view(np.float16).astype(np.float32))


def test_group_quantiser_known_answers(oracle):
    # runner/cuda/src/gemm_simt_kernels.cu:276-281 and its host twin runner/cuda/tests/test_gemm_simt_kernels.cpp:73-90
    w = np.zeros((3, 256), np.float32)
    w[0, :128] = np.linspace(-1.27, 1.27, 128, dtype=np.float32)  # scale 0.01
    w[0, 128:] = 0.0                                               # an all-zero group: scale 0, q 0
    w[1, 0] = 127.0                                                # scale exactly 1: q = rint(w)
    w[1, 1:8] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5]          # ties go to even
    w[2, 128] = -3.0e38                                            # a huge group still quantises to +-127
    w[2, 129] = 1.5e38
    q, s = oracle.quantize_group_s8(w)
    assert s[0, 1] == 0.0 and not q[0, 128:].any()
    assert s[0, 0] == np.float32(1.27) / np.float32(127.0)
    assert q[0, 0] == -127 and q[0, 127] == 127
    assert s[1, 0] == 1.0 and list(q[1, 0:8]) == [127, 0, 2, 2, 0, -2, -2, 126]
    assert q[2, 128] == -127 and q[2, 129] == 64 or q[2, 129] == 63
    # q * s reproduces w to half a step, and the dequantised matrix is float32(q) * s
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((8, 512)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_group_s8(w)
    wd = oracle.dequant_group_s8(q, s)
    assert np.array_equal(wd, q.astype(np.float32) * np.repeat(s, 128, axis=1))
    assert np.all(np.abs(wd - w) <= 0.5 * np.repeat(s, 128, axis=1) * (1 + 1e-6))
    assert np.abs(q).max() == 127


def test_quantiser_matches_a_numpy_restatement(oracle):
    rng = np.random.default_rng(11)
    w = (rng.standard_normal((16, 384)) / np.sqrt(384)).astype(np.float32)
    q, s = oracle.quantize_group_s8(w)
    g = w.reshape(16, 3, 128)
    scale = (np.abs(g).max(axis=2) / np.float32(127.0)).astype(np.float32)
    want = np.clip(np.rint(g / scale[:, :, None]), -127, 127).astype(np.int8).reshape(16, 384)
    assert np.array_equal(s, scale) and np.array_equal(q, want)


def test_row_quantiser_known_answers_and_numpy_restatement(oracle):
    # runner/cuda/src/gemm_s8_kernels.cu:28-31 (quantize_one) and :83-118 (one scale per output row, Plain layout)
    w = np.zeros((4, 32), np.float32)
    w[0, :8] = [127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5]  # amax 127: inv = 1, scale = 1, ties go to even
    w[1, :4] = [0.25, -0.125, 0.0625, 0.0]                        # amax 0.25: inv = 508
    w[3, :3] = [1.0, 2.0, 4.0]
    q, s = oracle.quantize_rows_s8(w)
    assert s[0] == 1.0 and list(q[0, :8]) == [127, 0, 2, 2, 0, -2, -2, 126]
    assert s[1] == np.float32(0.25) / np.float32(127.0) and list(q[1, :4]) == [127, -64, 32, 0]  # -63.5 -> -64, 31.75 -> 32
    assert s[2] == 0.0 and not q[2].any()                         # a zero row: scale 0 and zeros
    col = np.ones(32, np.float32)
    col[:3] = [4.0, 2.0, 1.0]                                    # smoothing factors multiply the columns first: all three become 4
    q, s = oracle.quantize_rows_s8(w, col)
    assert list(q[3, :3]) == [127, 127, 127] and s[3] == np.float32(4.0) / np.float32(127.0)
    rng = np.random.default_rng(12)
    w = oracle.to_f16_grid((rng.standard_normal((24, 256)) * 0.02).astype(np.float32))
    q, s = oracle.quantize_rows_s8(w)
    amax = np.abs(w).max(axis=1)
    inv = (np.float32(127.0) / amax).astype(np.float32)
    want = np.clip(np.rint((w * inv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    assert np.array_equal(q, want) and np.array_equal(s, (amax / np.float32(127.0)).astype(np.float32))
    assert np.all(np.abs(q.astype(np.float32) * s[:, None] - w) <= 0.5 * s[:, None] * (1 + 1e-5))


# ---- against the reference's code itself, where it was built -------------------------------------------------------------------


def test_oracle_matches_reference_code_on_fresh_inputs(oracle, ref):
    rng = np.random.default_rng(99)
    x = oracle.to_f16_grid(oracle.to_bf16_grid(rng.standard_normal((53, 320), dtype=np.float32)))
    w = oracle.to_f16_grid(oracle.to_bf16_grid(rng.standard_normal((72, 320), dtype=np.float32) * np.float32(0.02)))
    assert np.array_equal(oracle.gemm(x, w), ref.gemm_f64acc(x, w))
    assert np.array_equal(oracle.gemm(x, w), ref.gemm_f64acc(x.astype(np.float16), w.astype(np.float16)))
    assert np.array_equal(oracle.gemm_fma_chain(x, w), ref.cpu_gemm(x, w, kind="bf16", isa="avx2"))
    assert rel_fro(ref.cpu_gemm(x, w, kind="bf16"), oracle.gemm(x, w)) < 1e-5
    xr = rng.standard_normal((7, 128), dtype=np.float32)
    wr = (rng.standard_normal(128) * 0.1).astype(np.float32)
    assert np.allclose(oracle.rmsnorm(xr, wr), ref.rmsnorm_rows(xr, (1 + wr).astype(np.float32)), rtol=2e-6, atol=1e-7)


def test_reference_cpu_gemm_config1_shape_sample(oracle, ref):
    """BASELINE config 1's shape through the reference's cpu-bf16 kernel, checked at sampled places against the oracle."""
    rng = np.random.default_rng(1001)
    t, n, k = 900, 9728, 2560
    x = oracle.to_f16_grid(oracle.to_bf16_grid(rng.standard_normal((t, k), dtype=np.float32)))
    w = oracle.to_f16_grid(oracle.to_bf16_grid(rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)))
    y = ref.cpu_gemm(x, w, kind="bf16")
    rows = rng.integers(0, t, 4000).astype(np.uint32)
    cols = rng.integers(0, n, 4000).astype(np.uint32)
    exact = oracle.gemm_sample(x, w, rows, cols)
    assert rel_fro(y[rows, cols], exact) < 2e-3  # the tolerance BASELINE states for the fp16 path; the CPU result is ~1e-6
    assert rel_fro(y[rows, cols], exact) < 1e-5
