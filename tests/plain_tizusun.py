"""A plain, slow Tizusun: whole sequences, no cache, one function for each mechanism.

Tizusun is a decoder-only model of post-norm layers.  With ``a`` the constant
``postln_alpha`` and ``N`` an RMS norm with a weight,

    x <- N1(a x + mixer(x)) ;  x <- N2(a x + ff(x))

(the sublayers read x itself; there is no norm in front of them).  The mixer is
grouped-query attention whose values are the key projections as they leave the
matrix (before the key norm and the rotation; there is no value matrix), with a
per-head RMS norm of q and k, a partial rotation in the "rotate half" layout
with frequencies rescaled by wavelength, a causal mask restricted to the
query's own block of ``mask.size`` positions, and a sigmoid gate on the
concatenated heads in front of the output matrix.  The feed-forward is a gated
unit ``Wd (act(Wg h) * (Wu h))`` with act = relu, or a mixture of such units
with act = silu, of which every token uses the ``top`` with the largest router
logits, weighted by the softmax over those logits alone.

This file shares no code with the package: it reads config.json and the
safetensors file itself, with numpy only, and runs in float64 by default.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


def read_safetensors(path):
    """name -> numpy array (bfloat16 widened exactly; integer tables as they are)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        b, en = e["data_offsets"]
        raw = data[b:en]
        if e["dtype"] == "BF16":
            a = (np.frombuffer(raw, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif e["dtype"] == "F32":
            a = np.frombuffer(raw, dtype=np.float32)
        elif e["dtype"] == "I32":
            a = np.frombuffer(raw, dtype=np.int32)
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = a.reshape(e["shape"]).copy()
    return out


# ------------------------------------------------------------------- mechanisms

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2, then rescaled by wavelength l = 2 pi / f: kept where
    l < original/high, divided by ``factor`` where l > original/low, and blended in between with
    s = (original/l - low) / (high - low): (1 - s) f / factor + s f."""
    i = np.arange(dims // 2, dtype=np.float64)
    f = np.power(float(base), -2.0 * i / dims)
    if scaling:
        factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
        out = np.empty_like(f)
        for j, fj in enumerate(f):
            lam = 2.0 * math.pi / fj
            if lam < orig / high:
                out[j] = fj
            elif lam > orig / low:
                out[j] = fj / factor
            else:
                s = (orig / lam - low) / (high - low)
                out[j] = (1.0 - s) * fj / factor + s * fj
        f = out
    return f


def rotate_half(x, positions, freqs, dims):
    """x [T, heads, dim]: dimension i < dims/2 pairs with i + dims/2; (u, v) at position p becomes
    (u cos a - v sin a, v cos a + u sin a) with a = p f_i.  Dimensions from ``dims`` on pass unchanged."""
    half = dims // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freqs[None, :]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def block_causal_mask(positions, size):
    """visible[i, j]: j <= i and both in the same block of ``size`` positions counted from 0
    (``size`` None: plain causal)."""
    p = np.asarray(positions)
    vis = p[None, :] <= p[:, None]
    if size:
        vis &= (p[None, :] // size) == (p[:, None] // size)
    return vis


def masked_softmax(scores, visible):
    s = np.where(visible, scores, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    e = np.exp(s)
    return e / e.sum(axis=-1, keepdims=True)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


ACTIVATIONS = {
    "relu": lambda z: np.maximum(z, 0.0),
    "silu": lambda z: z * sigmoid(z),
    "gelu_tanh": lambda z: 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3))),
}


def attention_mixer(h, w, m, eps, positions):
    """h [T, d]; ``w`` maps 'q', 'k', 'q.norm', 'k.norm', 'g', 'o' to arrays; ``m`` is the mixer's config."""
    T = h.shape[0]
    H, G, dim = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w["q"].T).reshape(T, H, dim)
    k_raw = (h @ w["k"].T).reshape(T, G, dim)
    v = k_raw                                         # the values: keys as projected
    q = rms_norm(q, w["q.norm"], eps)
    k = rms_norm(k_raw, w["k.norm"], eps)
    rot = m.get("rot")
    if rot:
        f = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = rotate_half(q, positions, f, rot["dims"])
        k = rotate_half(k, positions, f, rot["dims"])
    vis = block_causal_mask(positions, (m.get("mask") or {}).get("size"))
    out = np.empty((T, H, dim), dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        p = masked_softmax((q[:, hh] @ k[:, g].T) * m["scale"], vis)
        out[:, hh] = p @ v[:, g]
    out = out.reshape(T, H * dim) * sigmoid(h @ w["g"].T)
    return out @ w["o"].T


def gated_unit(h, gate, up, down, act):
    return (ACTIVATIONS[act](h @ gate.T) * (h @ up.T)) @ down.T


def router(h, w, b, top):
    """Indices [T, top] of the largest logits (largest first) and their softmax over the chosen ones."""
    z = h @ w.T + b
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, idx, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return idx, e / e.sum(axis=-1, keepdims=True)


def mixture(h, w, n_experts, top, act="silu"):
    idx, wt = router(h, w["router"], w["router.b"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            out[t] += wt[t, j] * gated_unit(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], act)[0]
    return out


# ------------------------------------------------------------------------ model

class PlainTizusun:
    def __init__(self, model_dir, dtype=np.float64):
        with open(os.path.join(model_dir, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = {k: v.astype(dtype) for k, v in read_safetensors(os.path.join(model_dir, "model.safetensors")).items()}
        self.dtype = dtype

    def sub(self, prefix):
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def feed_forward(self, h, i, margins=None):
        mlp = self.cfg["layers"][i]["mlp"]
        w = self.sub(f"l{i}.mlp.")
        if mlp["kind"] == "dense":
            return gated_unit(h, w["gate"], w["up"], w["down"], "relu")
        E, top = mlp["router"]["experts"], mlp["router"]["top"]
        if margins is not None and top < E:
            z = np.sort(h @ w["router"].T + w["router.b"], axis=-1)[:, ::-1]
            margins.append(z[:, top - 1] - z[:, top])
        return mixture(h, w, E, top, "silu")

    def forward(self, tokens, residuals=None, margins=None):
        """Logits [T, vocab] of one whole sequence; ``residuals`` (a list) gets x after every layer,
        ``margins`` (a list) for every mixture layer the gap, token by token, between the last chosen
        router logit and the first one left out."""
        c = self.cfg
        eps, alpha = c["norm"]["eps"], c["postln_alpha"]
        pos = np.arange(len(tokens))
        x = self.w["embed"][np.asarray(tokens)]
        for i, layer in enumerate(c["layers"]):
            assert layer["type"] == "attention"
            x = rms_norm(alpha * x + attention_mixer(x, self.sub(f"l{i}.mix."), layer["mixer"], eps, pos),
                         self.w[f"l{i}.norm1"], eps)
            if layer.get("mlp") is not None:
                x = rms_norm(alpha * x + self.feed_forward(x, i, margins), self.w[f"l{i}.norm2"], eps)
            if residuals is not None:
                residuals.append(x.copy())
        return rms_norm(x, self.w["final.norm"], eps) @ self.w["head"].T
