"""CPU restatement (numpy, float64) of the full-attention mixer between its projections, following the reference function by function
(runner/include/sepal/ref/attention.hpp): unpack_query_and_gate (:33-49), rope_angles (:57-68), apply_rope (:76-97), attention_scale
(:100-102), grouped_query_attention (:113-166: query head h reads kv head h // (heads // kv_heads); token t sees the context and its own
tokens 0..t; hidden keys get probability exactly 0), the per-head rms_norm of ref/primitives.hpp:57-69 with the "1 + weight" form, and
the output gate sigmoid of attention_mixer (:176-231). Test infrastructure: only tests/ and the smoke check import it.

Pinned to the reference: oracle/_ref/libsepal_ref.so binds the reference's own template code for this mixer (ref_attention_core in
oracle/ref_shim.cpp); tests/test_attention_oracle.py holds this restatement to it within 1e-12, on the committed vectors
tests/golden/golden_mixers.npz (generated from that library by tests/golden/make_golden.py) and, where the library is built, on fresh
seeded inputs."""
import numpy as np


def rms_norm_heads(x, weight, eps):
    """x [..., head_dim] -> x / sqrt(mean(x^2) + eps) * (1 + weight)."""
    x = np.asarray(x, np.float64)
    rms = np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return x / rms * (1.0 + np.asarray(weight, np.float64))


def rope_angles(positions, rotary_dims, theta):
    half = rotary_dims // 2
    inv = np.power(float(theta), -np.arange(half, dtype=np.float64) * 2.0 / float(2 * half))
    return np.asarray(positions, np.float64)[:, None] * inv[None, :]


def apply_rope(x, angles):
    """x [T, heads, head_dim]: the first 2 * half dims rotate, dim i with dim i + half."""
    x = np.array(x, np.float64)
    half = angles.shape[1]
    cos, sin = np.cos(angles)[:, None, :], np.sin(angles)[:, None, :]
    first, second = x[..., :half].copy(), x[..., half:2 * half].copy()
    x[..., :half] = first * cos - second * sin
    x[..., half:2 * half] = second * cos + first * sin
    return x


def prepare(q_gate, k, v, q_norm, k_norm, positions, heads, kv_heads, head_dim, rotary_dims, theta, eps):
    """-> (q [T, heads, hd], gate [T, heads, hd], k [T, kvh, hd], v [T, kvh, hd]) in float64."""
    t = q_gate.shape[0]
    packed = np.asarray(q_gate, np.float64).reshape(t, heads, 2 * head_dim)
    query, gate = packed[..., :head_dim], packed[..., head_dim:]
    angles = rope_angles(positions, rotary_dims, theta)
    q = apply_rope(rms_norm_heads(query, q_norm, eps), angles)
    kk = apply_rope(rms_norm_heads(np.asarray(k, np.float64).reshape(t, kv_heads, head_dim), k_norm, eps), angles)
    return q, gate, kk, np.asarray(v, np.float64).reshape(t, kv_heads, head_dim)


def attend(q, keys, values, context):
    """q [T, heads, hd]; keys, values [context + T, kvh, hd]. Token t sees keys 0 .. context + t. -> [T, heads, hd]."""
    t, heads, hd = q.shape
    kvh = keys.shape[1]
    group = heads // kvh
    scale = 1.0 / np.sqrt(float(hd))
    out = np.zeros((t, heads, hd), np.float64)
    visible = np.arange(keys.shape[0])[None, :] <= (context + np.arange(t))[:, None]
    for h in range(heads):
        s = q[:, h, :] @ keys[:, h // group, :].T * scale
        s = np.where(visible, s, -np.inf)
        s = s - s.max(axis=1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=1, keepdims=True)
        out[:, h, :] = p @ values[:, h // group, :]
    return out


def gated(attended, gate):
    return attended / (1.0 + np.exp(-np.asarray(gate, np.float64)))
