"""A plain, slow Vekuzen: whole sequences, no cache, one function for each mechanism.

Vekuzen is a decoder-only model of pre-norm layers,

    x <- x + mixer(N1(x)) ;  x <- x + ff(N2(x)) ;  x <- x + side(x, token)

with N an RMS norm with a weight.  The embedding is ``embed[token] * scale + pos[p]``.  A stretch of the
layers (``loop.start .. loop.stop - 1``) runs ``loop.times`` times in a row with the same weights; in front of
every pass the residual is mixed with the embedding output x0, ``x <- W_in [x; x0]``.  Two mixers: *lightning*
(linear attention with a per-head decay: ``S_t = a_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` with silu on q, k
and v, a norm over all heads together, a sigmoid gate) and *latent attention* (queries, keys and values are
expanded from normed low-rank latents; plain causal softmax without positions; a sigmoid gate).  Two
feed-forwards: a gated unit with tanh-gelu, and a mixture of silu units chosen by ``softmax(z) + correction``
and weighted by ``softmax(z) * scale``, whose last router outputs stand for identity experts, with a shared
unit gated by one sigmoid a token.  The side input of layer i reads columns ``[i dim, (i + 1) dim)`` of a
second token table.

This file shares no code with the package: it reads config.json and the safetensors file itself, with numpy
only, and runs in float64.
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


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def embed(tokens, table, scale, pos_table, first_pos=0):
    """embed[token] * scale + pos[p], p counted from ``first_pos``."""
    tokens = np.asarray(tokens)
    p = first_pos + np.arange(len(tokens))
    return table[tokens] * scale + pos_table[p]


def loop_entry(x, x0, w_in):
    """x <- W_in [x; x0] row by row (W_in is [width, 2 width], the columns of x first)."""
    return np.concatenate([x, x0], axis=-1) @ w_in.T


def lightning(h, wq, wk, wv, wg, wo, norm_w, decay, heads, dim, vdim, eps, state=None):
    """Linear attention with decay, token by token.  ``state`` [heads, dim, vdim] is the state before the first
    row (zero if None); returns (output rows, state after the last row)."""
    T = h.shape[0]
    q = silu(h @ wq.T).reshape(T, heads, dim)
    k = silu(h @ wk.T).reshape(T, heads, dim)
    v = silu(h @ wv.T).reshape(T, heads, vdim)
    S = np.zeros((heads, dim, vdim)) if state is None else np.array(state, dtype=np.float64)
    a = np.asarray(decay, dtype=np.float64)[:, None, None]
    o = np.empty((T, heads, vdim))
    for t in range(T):                                             # (all heads at once: S [heads, dim, vdim])
        S = a * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o.reshape(T, heads * vdim), norm_w, eps) * sigmoid(h @ wg.T)
    return o @ wo.T, S


def causal_softmax_attention(q, k, v, scale, first_key=None):
    """q, k [T, H, dim], v [T, H, vdim]; row i reads keys j <= i (and j >= first_key[i] if given)."""
    T, H, _ = q.shape
    out = np.empty((T, H, v.shape[2]))
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = j <= i
    if first_key is not None:
        seen &= j >= np.asarray(first_key)[:, None]
    for h in range(H):                                             # (a head at a time: scores [T, T])
        s = np.where(seen, (q[:, h] @ k[:, h].T) * scale, -np.inf)
        w = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h] = (w / w.sum(axis=1, keepdims=True)) @ v[:, h]
    return out


def latent_attention(h, w, heads, dim, vdim, scale, eps):
    """``w``: the mixer's tensors by their short names (dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o)."""
    T = h.shape[0]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, heads, dim)
    c = rms_norm(h @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).reshape(T, heads, dim)
    v = (c @ w["uv"].T).reshape(T, heads, vdim)
    o = causal_softmax_attention(q, k, v, scale).reshape(T, heads * vdim)
    return (o * sigmoid(h @ w["g"].T)) @ w["o"].T


def gated_unit(h, wg, wu, wd, act):
    return (act(h @ wg.T) * (h @ wu.T)) @ wd.T


def route(h, w_router, correction, top, scale):
    """(chosen experts [T, top], their weights [T, top], all scores [T, E]).  Scores are the softmax over all
    router outputs; the choice adds ``correction`` to them, the weights do not; no renormalisation."""
    z = h @ w_router.T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    s /= s.sum(axis=-1, keepdims=True)
    choice = s + correction
    idx = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    return idx, np.take_along_axis(s, idx, axis=-1) * scale, s


def choice_margin(h, w_router, correction, top):
    """For every row the gap between the last chosen and the first unchosen choice score (inf if all are chosen)."""
    z = h @ w_router.T
    s = np.exp(z - z.max(axis=-1, keepdims=True))
    c = np.sort(s / s.sum(axis=-1, keepdims=True) + correction, axis=-1)[:, ::-1]
    return c[:, top - 1] - c[:, top] if top < c.shape[1] else np.full(h.shape[0], np.inf)


def mixture(h, w_router, correction, experts, n_identity, top, scale, shared=None):
    """``experts``: list of (Wg, Wu, Wd); the router has len(experts) + n_identity outputs, the last of which
    stand for experts that return their input.  ``shared`` = (Wg, Wu, Wd, w_sg): a unit every token uses,
    times sigmoid(w_sg . h)."""
    idx, wts, _ = route(h, w_router, correction, top, scale)
    out = np.zeros_like(h)
    for r in range(h.shape[0]):
        for j in range(top):
            e = int(idx[r, j])
            y = gated_unit(h[r], *experts[e], silu) if e < len(experts) else h[r]
            out[r] += wts[r, j] * y
    if shared is not None:
        wg, wu, wd, wsg = shared
        out += gated_unit(h, wg, wu, wd, silu) * sigmoid(h @ wsg.T)
    return out


def token_side(x, tokens, table, part, dim, w_gate, w_proj, norm_w, eps):
    """x + norm(W_proj (gelu(W_gate x) * e)) with e = table[token, part dim : (part + 1) dim]."""
    e = table[np.asarray(tokens)][:, part * dim:(part + 1) * dim]
    y = (gelu_tanh(x @ w_gate.T) * e) @ w_proj.T
    return x + rms_norm(y, norm_w, eps)


# ------------------------------------------------------------------------ model

def layer_runs(cfg):
    """The order in which layers run: [(layer, first of a pass?)], the looped stretch repeated."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, False) for i in range(a)]
    for _ in range(times):
        runs += [(i, i == a) for i in range(a, b)]
    return runs + [(i, False) for i in range(b, n)]


class PlainVekuzen:
    def __init__(self, model_dir=None, config=None, tensors=None):
        if model_dir is not None:
            with open(os.path.join(model_dir, "config.json")) as f:
                config = json.load(f)
            tensors = read_safetensors(os.path.join(model_dir, "model.safetensors"))
        self.cfg = config
        self.w = {k: np.asarray(v, dtype=np.float64) for k, v in tensors.items()}
        self.eps = float(config["norm"]["eps"])

    def _mixer(self, i, h):
        L, w = self.cfg["layers"][i], self.w
        m, p = L["mixer"], f"l{i}.mix."
        if L["type"] == "lightning":
            return lightning(h, w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"], w[p + "o"], w[p + "norm"], m["decay"],
                             int(m["heads"]), int(m["dim"]), int(m["vdim"]), self.eps)[0]
        if L["type"] == "latent_attention":
            names = ("dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "g", "o")
            return latent_attention(h, {n: w[p + n] for n in names}, int(m["heads"]), int(m["dim"]), int(m["vdim"]),
                                    float(m["scale"]), self.eps)
        raise ValueError(L["type"])

    def _ff(self, i, h, margins=None):
        mlp, w, p = self.cfg["layers"][i]["mlp"], self.w, f"l{i}.mlp."
        if mlp["kind"] == "dense":
            return gated_unit(h, w[p + "gate"], w[p + "up"], w[p + "down"], gelu_tanh)
        r = mlp["router"]
        E, ident = int(r["experts"]), int(r.get("identity", 0))
        experts = [(w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"]) for e in range(E)]
        shared = None
        if mlp.get("shared"):
            shared = (w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], w[p + "shared.sg"])
        if margins is not None:
            margins.append(choice_margin(h, w[p + "router"], w[p + "correction"], int(r["top"])))
        return mixture(h, w[p + "router"], w[p + "correction"], experts, ident, int(r["top"]), float(r["scale"]), shared)

    def forward(self, tokens, layers_out=None, margins=None):
        """Logits [T, vocab] of a whole sequence; ``layers_out`` (a list) gets the residual after every layer run,
        ``margins`` (a list) every mixture's choice margins [T]."""
        cfg, w = self.cfg, self.w
        x = embed(tokens, w["embed"], float(cfg["embedding"]["scale"]), w["pos"])
        x0 = x.copy()
        side = cfg.get("token_side")
        for i, enters in layer_runs(cfg):
            if enters:
                x = loop_entry(x, x0, w["loop.in"])
            p = f"l{i}."
            x = x + self._mixer(i, rms_norm(x, w[p + "norm1"], self.eps))
            if cfg["layers"][i].get("mlp") is not None:
                x = x + self._ff(i, rms_norm(x, w[p + "norm2"], self.eps), margins)
            if side:
                x = token_side(x, tokens, w["side.embed"], i, int(side["dim"]), w[p + "side.gate"], w[p + "side.proj"],
                               w[p + "side.norm"], self.eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        return rms_norm(x, w["final.norm"], self.eps) @ w["head"].T * float(cfg["logit_scale"])
