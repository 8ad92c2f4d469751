"""Small Tizusun configurations that differ in every size, constant and option, and a writer of model folders
whose weights are large enough that every sublayer moves the residual (with weights of 0.02 a wrong key or a lost
expert would hide below the tolerances)."""
import json
import math
import os
import tempfile

import numpy as np


def _attn(heads, kv_heads, dim, rot=None, mask=None, scale=None):
    return {"dim": dim, "vdim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot,
            "mask": {"size": mask} if mask else None, "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}


def _layer(mixer, mlp):
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


_DENSE = lambda ff: {"kind": "dense", "ff": ff}
_MOE = lambda experts, top, ff: {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
_SCALED = {"factor": 8.0, "low": 2.0, "high": 8.0, "original": 64}

# P: head size 32 (the split-key kernel takes every 32-bit row and the decoded rows), two kv heads, rotation of
# half a head with rescaled frequencies, blocks of 24 positions, six experts of which two
TIZ_P = {"architecture": "Tizusun", "vocab": 211, "width": 64, "postln_alpha": 1.5, "norm": {"eps": 1e-5}, "layers": [
    _layer(_attn(4, 2, 32, {"base": 10000.0, "dims": 16, "scaling": _SCALED}, 24), _MOE(6, 2, 32)),
    _layer(_attn(4, 2, 32, {"base": 10000.0, "dims": 16, "scaling": _SCALED}, 24), _DENSE(96)),
    _layer(_attn(4, 2, 32, {"base": 10000.0, "dims": 16, "scaling": _SCALED}, 24), _MOE(6, 2, 32)),
]}
# Q: layers that differ among themselves (two page groups), a layer without a feed-forward, whole-head rotation
# without rescaling, one expert a token, alpha 1, blocks of 40 and of 7 positions, a scale that is not 1/sqrt(dim)
TIZ_Q = {"architecture": "Tizusun", "vocab": 97, "width": 48, "postln_alpha": 1.0, "norm": {"eps": 1e-6}, "layers": [
    _layer(_attn(3, 1, 48, {"base": 500.0, "dims": 48}, 40, 0.2), _DENSE(80)),
    _layer(_attn(6, 3, 16, {"base": 500.0, "dims": 8}, 7), None),
    _layer(_attn(3, 1, 48, {"base": 500.0, "dims": 48}, 40, 0.2), _MOE(3, 1, 24)),
    _layer(_attn(6, 3, 16, {"base": 500.0, "dims": 8}, 7), _MOE(4, 4, 16)),
]}
# R: sizes the fast kernels refuse (width 36, head size 24, ten query heads on one kv head), no mask, no rotation
# in one layer, every expert used
TIZ_R = {"architecture": "Tizusun", "vocab": 150, "width": 36, "postln_alpha": 3.0, "norm": {"eps": 1e-5}, "layers": [
    _layer(_attn(10, 1, 24, {"base": 1000.0, "dims": 12}, None), _MOE(5, 3, 20)),
    _layer(_attn(10, 1, 24, None, 33), _DENSE(44)),
]}
# S: head size 64 with a block of 100 positions that page borders (64) and key chunks (256) cut
TIZ_S = {"architecture": "Tizusun", "vocab": 300, "width": 128, "postln_alpha": 2.0, "norm": {"eps": 1e-5}, "layers": [
    _layer(_attn(4, 1, 64, {"base": 10000.0, "dims": 32, "scaling": {"factor": 3.0, "low": 1.5, "high": 6.0, "original": 128}}, 100),
           _MOE(8, 2, 64)),
    _layer(_attn(4, 1, 64, {"base": 10000.0, "dims": 32, "scaling": {"factor": 3.0, "low": 1.5, "high": 6.0, "original": 128}}, 100),
           _MOE(8, 2, 64)),
]}

# T: widths at which the decode products stream their weights (K a multiple of 512) and the prompt products run on
# tcgen05; head size 128 (mma.sync prompt kernel, split-key tensor-core decode), as many kv heads as heads, a block
# as long as a page, rotation of half a head
TIZ_T = {"architecture": "Tizusun", "vocab": 500, "width": 512, "postln_alpha": 2.25, "norm": {"eps": 1e-5}, "layers": [
    _layer(_attn(4, 4, 128, {"base": 20000.0, "dims": 64, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 64}}, 64),
           _DENSE(1024)),
    _layer(_attn(4, 4, 128, {"base": 20000.0, "dims": 64, "scaling": {"factor": 2.0, "low": 1.0, "high": 2.0, "original": 64}}, 64),
           _MOE(4, 2, 128)),
]}
# U: blocks of one position (a token reads itself alone) and of three, two experts of which one, a vocabulary smaller than a warp
TIZ_U = {"architecture": "Tizusun", "vocab": 19, "width": 32, "postln_alpha": 1.25, "norm": {"eps": 1e-3}, "layers": [
    _layer(_attn(2, 1, 16, {"base": 100.0, "dims": 16}, 1), _MOE(2, 1, 8)),
    _layer(_attn(2, 2, 16, {"base": 100.0, "dims": 4}, 3), _DENSE(8)),
    _layer(_attn(1, 1, 32, None, None), _MOE(2, 2, 40)),
]}

# V: prompts long enough that a step has more than 512 (row, expert) pairs: the experts' products then run as grouped
# tcgen05 tiles, some experts with several tiles, some with a part of one
TIZ_V = {"architecture": "Tizusun", "vocab": 400, "width": 256, "postln_alpha": 1.75, "norm": {"eps": 1e-5}, "layers": [
    _layer(_attn(4, 2, 64, {"base": 10000.0, "dims": 32}, 150), _MOE(8, 2, 72)),
    _layer(_attn(4, 2, 64, {"base": 10000.0, "dims": 32}, 150), _MOE(5, 3, 136)),
]}

CONFIGS = {"P": (TIZ_P, 3), "Q": (TIZ_Q, 4), "R": (TIZ_R, 5), "S": (TIZ_S, 6), "T": (TIZ_T, 7), "U": (TIZ_U, 8), "V": (TIZ_V, 9)}


def tensor_shapes(cfg):
    d, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "head": (cfg["vocab"], cfg["width"]),
                            "final.norm": (cfg["width"],)}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out[p + "norm1"] = (d,)
        out[p + "mix.q"] = (m["heads"] * m["dim"], d)
        out[p + "mix.k"] = (m["kv_heads"] * m["dim"], d)
        out[p + "mix.q.norm"] = (m["dim"],)
        out[p + "mix.k.norm"] = (m["dim"],)
        out[p + "mix.g"] = (m["heads"] * m["vdim"], d)
        out[p + "mix.o"] = (d, m["heads"] * m["vdim"])
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (d,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], d), p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        else:
            E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
            out[p + "mlp.router"] = (E, d)
            out[p + "mlp.router.b"] = (E,)
            for e in range(E):
                out.update({f"{p}mlp.e{e}.gate": (ff, d), f"{p}mlp.e{e}.up": (ff, d), f"{p}mlp.e{e}.down": (d, ff)})
    return out


def make_weights(cfg, seed):
    """name -> float32 array holding bfloat16 values.  Matrices have unit gain (std 1/sqrt(inputs)), output
    matrices a gain of 2, router rows a gain of 3, norm weights 1 +- 0.2, the embedding std 1."""
    import torch
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            a = rng.normal(0.0, 0.5, shape) if name.endswith("router.b") else 1.0 + rng.normal(0.0, 0.2, shape)
        elif name in ("embed",):
            a = rng.normal(0.0, 1.0, shape)
        else:
            gain = 3.0 if name.endswith("router") else (2.0 if name.endswith((".o", ".down")) else 1.0)
            a = rng.normal(0.0, gain / math.sqrt(shape[1]), shape)
        out[name] = torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)
    return out


def make_model_dir(name, root=None):
    from kappai_b200.weights.safetensors_io import save_safetensors

    cfg, seed = CONFIGS[name]
    d = tempfile.mkdtemp(prefix=f"tiz_{name}_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(d, "model.safetensors"), make_weights(cfg, seed))
    return d
