"""The Gated DeltaNet core on the device against the float64 restatement of the reference's mixer (oracle/deltanet_oracle.py). The
device keeps the recurrent state in float32 and forms a chunk's matrix products on the tensor cores with TF32 operands (10 bits of
mantissa, the precision the reference's chunked kernels give theirs by rounding to binary16), so the bounds are those of a 2^-11
rounding per operand: relative Frobenius error 2e-3 on the binary16 output and 1e-3 on the float32 states (measured: 4e-4)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def rel_fro(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))


@pytest.fixture(scope="module")
def ctx():
    import sepal_runner_b200 as sb

    c = sb.Context(0)
    yield c
    c.close()


def run_case(ctx, key_heads, value_heads, taps, requests, seed, half, a_log=None):
    """requests: list of (first call's tokens, second call's tokens): every request runs as two calls; the second continues the first."""
    import torch

    import sepal_runner_b200 as sb
    from oracle import deltanet_oracle as do

    rng = np.random.default_rng(seed)
    dim = 128
    shape = sb.DeltaNetShape(key_heads=key_heads, value_heads=value_heads, head_dim=dim, conv_kernel=taps, eps=1e-6)
    kd, vd = key_heads * dim, value_heads * dim
    conv_dim = 2 * kd + vd
    conv = (rng.standard_normal((conv_dim, taps)) * 0.5).astype(np.float32)
    a_log = (rng.standard_normal(value_heads) * 0.5).astype(np.float32) if a_log is None else np.asarray(a_log, np.float32)
    dt_bias = (rng.standard_normal(value_heads) * 0.5).astype(np.float32)
    norm = (1.0 + rng.standard_normal(dim) * 0.1).astype(np.float32)
    slots = len(requests) + 1
    states = torch.full((slots, value_heads, dim, dim), float("nan"), dtype=torch.float32, device="cuda")  # fresh rows must not read them
    tails = torch.full((slots, max(taps - 1, 1), conv_dim), float("nan"), dtype=torch.float32, device="cuda")
    dt = torch.float16 if half else torch.float32
    np_dt = np.float16 if half else np.float32
    data = []
    for first, second in requests:
        t = first + second
        data.append(tuple((rng.standard_normal((t, w)) * s).astype(np_dt).astype(np.float32)
                          for w, s in ((conv_dim, 1.0), (vd, 1.0), (value_heads, 1.0), (value_heads, 1.0))))
    dev = lambda x: torch.from_numpy(x).cuda()  # noqa: E731
    outs = [[] for _ in requests]
    for call in (0, 1):
        rows, parts = [], []
        at = 0
        for i, (first, second) in enumerate(requests):
            lo, n = (0, first) if call == 0 else (first, second)
            if n == 0:
                continue
            rows.append((at, n, i + 1, 1 if lo == 0 else 0))  # slot 0 stays unused
            parts.append((i, lo, n))
            at += n
        if not rows:
            continue
        bands = [dev(np.concatenate([data[i][w][lo:lo + n] for i, lo, n in parts])).to(dt) for w in range(4)]
        out = torch.full((at, vd), float("nan"), dtype=torch.float16, device="cuda")
        keep = sb.deltanet(ctx, shape, rows, bands[0], bands[1], bands[2], bands[3], dev(conv), dev(a_log), dev(dt_bias), dev(norm), states, tails, out)
        ctx.check_status()
        del keep
        got = out.float().cpu().numpy()
        for (q_begin, n, slot, fresh), (i, lo, _) in zip(rows, parts):
            outs[i].append(got[q_begin:q_begin + n])
    for i, (first, second) in enumerate(requests):
        mixed, z, b, a = data[i]
        want, state, tail = do.core(mixed, z, b, a, conv, a_log, dt_bias, norm, key_heads, value_heads, dim, 1e-6)
        got = np.concatenate(outs[i])
        assert np.isfinite(got).all()
        assert rel_fro(got, want) < 2e-3, (i, rel_fro(got, want))
        assert rel_fro(states[i + 1].cpu().numpy(), state) < 1e-3, (i, rel_fro(states[i + 1].cpu().numpy(), state))
        if taps > 1:
            assert np.array_equal(tails[i + 1, :taps - 1].cpu().numpy(), tail.astype(np.float32))


def test_one_request_in_one_and_in_two_calls(ctx):
    run_case(ctx, key_heads=1, value_heads=1, taps=4, requests=[(37, 0)], seed=1, half=False)
    run_case(ctx, key_heads=2, value_heads=4, taps=4, requests=[(100, 63)], seed=2, half=True)
    run_case(ctx, key_heads=1, value_heads=2, taps=4, requests=[(2, 1)], seed=3, half=True)  # runs shorter than the conv tail


def test_several_requests_and_other_tap_counts(ctx):
    run_case(ctx, key_heads=2, value_heads=2, taps=4, requests=[(5, 70), (1, 1), (64, 0), (33, 200)], seed=4, half=True)
    run_case(ctx, key_heads=1, value_heads=2, taps=1, requests=[(20, 20)], seed=5, half=False)
    run_case(ctx, key_heads=1, value_heads=1, taps=3, requests=[(20, 20), (7, 3)], seed=6, half=False)


def test_chunk_boundaries(ctx):
    """Run lengths around the scan's chunk of sixteen tokens, as one call and cut at every kind of place
    (runner/cuda/tests/test_kernels_deltanet.cpp:1061 walks the same lengths)."""
    run_case(ctx, key_heads=1, value_heads=2, taps=4, requests=[(1, 0), (5, 0), (16, 0), (17, 0), (33, 0), (70, 0)], seed=7, half=True)
    run_case(ctx, key_heads=1, value_heads=1, taps=4, requests=[(16, 16), (15, 1), (1, 15), (17, 47), (31, 33)], seed=8, half=True)


def test_strong_decay(ctx):
    """Decays from 0.97 a token down to exactly zero in float32 (runner/cuda/tests/test_kernels_deltanet.cpp:1015-1030): the products
    of decays inside a chunk underflow to zero, which must stay zero and not turn into a NaN."""
    heads = 4
    a_log = [np.log(0.03 + h / (heads - 1) * 200.0) for h in range(heads)]
    run_case(ctx, key_heads=2, value_heads=heads, taps=4, requests=[(1, 0), (5, 12), (16, 1), (33, 37)], seed=9, half=True, a_log=a_log)


def test_arguments_are_checked(ctx):
    import torch

    import sepal_runner_b200 as sb

    shape = sb.DeltaNetShape(key_heads=1, value_heads=1, head_dim=128, conv_kernel=4, eps=1e-6)
    z = torch.zeros((8, 384), dtype=torch.float16, device="cuda")
    w = torch.zeros((384, 4), device="cuda")
    v1 = torch.zeros(128, device="cuda")
    states = torch.zeros((2, 1, 128, 128), device="cuda")
    tails = torch.zeros((2, 3, 384), device="cuda")
    out = torch.zeros((8, 128), dtype=torch.float16, device="cuda")
    args = (z, z[:, :128], z[:, :1], z[:, :1], w, v1[:1], v1[:1], v1, states, tails, out)
    with pytest.raises(sb.SepalB200Error, match="slot that does not exist"):
        sb.deltanet(ctx, shape, [(0, 8, 2, 1)], *args)
    with pytest.raises(sb.SepalB200Error, match="share a state slot"):
        sb.deltanet(ctx, shape, [(0, 4, 1, 1), (4, 4, 1, 1)], *args)
    with pytest.raises(sb.SepalB200Error, match="head_dim must be 128"):
        sb.deltanet(ctx, sb.DeltaNetShape(key_heads=1, value_heads=1, head_dim=64, conv_kernel=4, eps=1e-6), [(0, 8, 1, 1)], *args)
