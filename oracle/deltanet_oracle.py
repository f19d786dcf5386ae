"""CPU restatement (numpy, float64) of the Gated DeltaNet mixer between its projections, following the reference function by function
(runner/include/sepal/ref/deltanet.hpp): causal_conv (:44-78: the LAST tap multiplies the current token; the window is the tail, then the
run's inputs), silu, split_heads (:128-143: q, k of the key heads, then v), l2_normalise (:84-92: x / sqrt(sum x^2 + 1e-6)),
share_key_heads (:98-113: value head h reads key head h // (value heads // key heads)), decay_gate (:146-154), delta_rule_update
(:163-184: decay first, then S += k (x) beta (v - k . S)), delta_rule_scan (:204-232: a token reads the state after its own update, the
read scaled by 1 / sqrt(dk)), gated_rms_norm (:236-263: the norm weight itself, gate silu(z)). Test infrastructure only.

Pinned to the reference: oracle/_ref/libsepal_ref.so binds the reference's own template code for this mixer (ref_deltanet_core in
oracle/ref_shim.cpp); tests/test_deltanet_oracle.py holds this restatement to it within 1e-12, on the committed vectors
tests/golden/golden_mixers.npz (generated from that library by tests/golden/make_golden.py) and, where the library is built, on fresh
seeded inputs, state and convolution tail carried across a cut included."""
import numpy as np


def softplus(x):
    return np.maximum(x, 0.0) + np.log1p(np.exp(-np.abs(x)))


def sigmoid(x):
    return np.exp(-softplus(-x))


def silu(x):
    return x * sigmoid(x)


def causal_conv(inputs, kernel, tail):
    """inputs [T, C], kernel [C, K], tail [K - 1, C] (oldest first) -> (outputs [T, C], new tail [K - 1, C])."""
    inputs = np.asarray(inputs, np.float64)
    taps = kernel.shape[1]
    window = np.concatenate([np.asarray(tail, np.float64), inputs], axis=0)
    out = np.zeros_like(inputs)
    for j in range(taps):
        out += np.asarray(kernel, np.float64)[:, j][None, :] * window[j:j + inputs.shape[0]]
    return out, window[window.shape[0] - (taps - 1):].copy() if taps > 1 else np.zeros((0, inputs.shape[1]))


def core(mixed, z, b, a, conv, a_log, dt_bias, norm, key_heads, value_heads, dim, eps, state=None, tail=None):
    """One run of tokens continuing (state [Hv, dk, dv], tail [K - 1, conv_dim]) or starting from zero.
    -> (out [T, value_heads * dim], state, tail)."""
    t = mixed.shape[0]
    key_dim, value_dim = key_heads * dim, value_heads * dim
    taps = conv.shape[1]
    if tail is None:
        tail = np.zeros((taps - 1, mixed.shape[1]))
    if state is None:
        state = np.zeros((value_heads, dim, dim))
    state = np.array(state, np.float64)
    activated, tail = causal_conv(mixed, conv, tail)
    activated = silu(activated)
    q = activated[:, :key_dim].reshape(t, key_heads, dim)
    k = activated[:, key_dim:2 * key_dim].reshape(t, key_heads, dim)
    v = activated[:, 2 * key_dim:].reshape(t, value_heads, dim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6)
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    repeat = value_heads // key_heads
    q = np.repeat(q, repeat, axis=1)
    k = np.repeat(k, repeat, axis=1)
    decay = np.exp(-np.exp(np.asarray(a_log, np.float64))[None, :] * softplus(np.asarray(a, np.float64) + np.asarray(dt_bias, np.float64)[None, :]))
    beta = sigmoid(np.asarray(b, np.float64))
    scale = 1.0 / np.sqrt(float(dim))
    reads = np.zeros((t, value_heads, dim))
    for i in range(t):
        state *= decay[i][:, None, None]
        recalled = np.einsum("hk,hkv->hv", k[i], state)
        correction = beta[i][:, None] * (v[i] - recalled)
        state += k[i][:, :, None] * correction[:, None, :]
        reads[i] = scale * np.einsum("hk,hkv->hv", q[i], state)
    rms = np.sqrt((reads * reads).mean(-1, keepdims=True) + eps)
    out = reads / rms * np.asarray(norm, np.float64)[None, None, :] * silu(np.asarray(z, np.float64).reshape(t, value_heads, dim))
    return out.reshape(t, value_dim), state, tail
