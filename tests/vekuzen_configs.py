"""Small Vekuzen configurations that differ in every size, constant and option, and a writer of model folders whose
weights are large enough that every sublayer moves the residual (with weights of 0.02 a wrong key, a lost state or a
lost expert would hide below the tolerances)."""
import json
import math
import os
import tempfile

import numpy as np


def _lightning(heads, dim, vdim, decay):
    assert len(decay) == heads
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def _latent(heads, dim, vdim, q_rank, kv_rank, scale=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                                                  "scale": scale if scale is not None else 1.0 / math.sqrt(dim)}}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


_DENSE = lambda ff: {"kind": "dense", "ff": ff}


def _MOE(experts, identity, top, scale, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def _model(vocab, width, layers, eps=1e-5, emb_scale=1.0, logit_scale=1.0, max_positions=512, loop=None, side=None):
    c = {"architecture": "Vekuzen", "vocab": vocab, "width": width, "embedding": {"scale": emb_scale}, "norm": {"eps": eps},
         "logit_scale": logit_scale, "max_positions": max_positions, "layers": layers}
    if loop:
        c["loop"] = dict(zip(("start", "stop", "times"), loop))
    if side:
        c["token_side"] = {"dim": side}
    return c


# A: the loop comes first and runs three times over two layers; values twice as wide as keys in the lightning layer;
# five experts and one identity expert of which two, with a shared unit; side inputs of 8 columns
VEK_A = _model(211, 64, [
    _layer(_lightning(2, 16, 32, [0.9, 0.995]), _MOE(5, 1, 2, 1.5, 24, 40)),
    _layer(_latent(4, 16, 16, 24, 40, 0.3), _DENSE(96)),
    _layer(_lightning(2, 16, 32, [0.5, 1.0]), _DENSE(80)),
], emb_scale=2.0, logit_scale=0.5, loop=(0, 2, 3), side=8)
# B: no loop and no side inputs; keys wider than values (a cache head is padded), three heads; one expert a token,
# no identity expert, no shared unit; a layer without a feed-forward; lightning heads of 40 x 24
VEK_B = _model(97, 48, [
    _layer(_latent(3, 24, 8, 16, 16), _MOE(4, 0, 1, 1.0, 32)),
    _layer(_lightning(3, 40, 24, [0.8, 0.97, 0.999]), None),
    _layer(_latent(3, 24, 8, 16, 16), _DENSE(72)),
    _layer(_lightning(3, 40, 24, [0.3, 0.9, 0.99]), _MOE(4, 0, 1, 1.0, 32)),
], eps=1e-6, emb_scale=0.5, logit_scale=2.0, max_positions=300)
# C: sizes the fast kernels refuse (width 36, ranks 12 and 20, side inputs of 5 columns, a vocabulary smaller than a
# warp); the loop runs once and reaches the last layer; every router output is used (top = experts + identity);
# values wider than keys
VEK_C = _model(19, 36, [
    _layer(_latent(2, 12, 20, 12, 20, 0.4), _DENSE(44)),
    _layer(_lightning(1, 36, 12, [0.95]), _MOE(3, 2, 5, 0.7, 20, 28)),
    _layer(_latent(5, 8, 8, 20, 12), _MOE(2, 1, 2, 2.0, 12)),
], eps=1e-3, emb_scale=1.5, loop=(1, 3, 1), side=5)
# D: widths at which the decode products stream their weights and the prompt products run on tcgen05; head size 64
# (tensor-core attention kernels); prompts long enough that a step's experts run as grouped tcgen05 tiles; the loop
# in the middle, a layer behind it
VEK_D = _model(400, 512, [
    _layer(_latent(4, 64, 64, 192, 128), _DENSE(1024)),
    _layer(_lightning(4, 64, 64, [0.6, 0.9, 0.99, 0.999]), _MOE(8, 2, 3, 2.0, 128, 256)),
    _layer(_latent(4, 64, 64, 192, 128), _MOE(8, 2, 3, 2.0, 128, 256)),
    _layer(_lightning(4, 64, 64, [0.7, 0.95, 0.98, 1.0]), _DENSE(512)),
], emb_scale=4.0, logit_scale=0.25, max_positions=1024, loop=(1, 3, 2), side=32)
# E: head size 128 in both mixers (the lightning state 128 x 64), two heads
VEK_E = _model(300, 256, [
    _layer(_lightning(2, 128, 64, [0.97, 0.999]), _DENSE(256)),
    _layer(_latent(2, 128, 128, 64, 96), _MOE(4, 1, 2, 1.0, 64, 64)),
], emb_scale=1.0, logit_scale=1.0, max_positions=640, loop=(0, 2, 2), side=16)

CONFIGS = {"A": (VEK_A, 3), "B": (VEK_B, 4), "C": (VEK_C, 5), "D": (VEK_D, 6), "E": (VEK_E, 7)}


def tensor_shapes(cfg):
    d, V, n = cfg["width"], cfg["vocab"], len(cfg["layers"])
    out = {"embed": (V, d), "pos": (cfg["max_positions"], d), "head": (V, d), "final.norm": (d,)}
    if cfg.get("loop"):
        out["loop.in"] = (d, 2 * d)
    side = cfg.get("token_side")
    if side:
        out["side.embed"] = (V, n * side["dim"])
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        H, dim, vdim = m["heads"], m["dim"], m["vdim"]
        out[p + "norm1"] = (d,)
        if layer["type"] == "lightning":
            out.update({p + "mix.q": (H * dim, d), p + "mix.k": (H * dim, d), p + "mix.v": (H * vdim, d),
                        p + "mix.g": (H * vdim, d), p + "mix.o": (d, H * vdim), p + "mix.norm": (H * vdim,)})
        else:
            out.update({p + "mix.dq": (m["q_rank"], d), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (H * dim, m["q_rank"]),
                        p + "mix.dkv": (m["kv_rank"], d), p + "mix.dkv.norm": (m["kv_rank"],),
                        p + "mix.uk": (H * dim, m["kv_rank"]), p + "mix.uv": (H * vdim, m["kv_rank"]),
                        p + "mix.g": (H * vdim, d), p + "mix.o": (d, H * vdim)})
        if side:
            out.update({p + "side.gate": (side["dim"], d), p + "side.proj": (d, side["dim"]), p + "side.norm": (d,)})
        mlp = layer["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = (d,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.gate": (mlp["ff"], d), p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        else:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            E = r["experts"] + r["identity"]
            out[p + "mlp.router"] = (E, d)
            out[p + "mlp.correction"] = (E,)
            for e in range(r["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (ff, d), f"{p}mlp.e{e}.up": (ff, d), f"{p}mlp.e{e}.down": (d, ff)})
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (sf, d), p + "mlp.shared.up": (sf, d), p + "mlp.shared.down": (d, sf),
                            p + "mlp.shared.sg": (1, d)})
    return out


def make_weights(cfg, seed):
    """name -> bfloat16 tensor.  Matrices have unit gain (std 1/sqrt(inputs)), output matrices a gain of 2, router rows a
    gain of 3, norm weights 1 +- 0.2, the embedding tables std 1, the corrections of the choice std 0.05 (the scores
    they are added to are about 1 / experts)."""
    import torch
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("correction"):
            a = rng.normal(0.0, 0.05, shape)
        elif len(shape) == 1:
            a = 1.0 + rng.normal(0.0, 0.2, shape)
        elif name in ("embed", "side.embed"):
            a = rng.normal(0.0, 1.0, shape)
        elif name == "pos":
            a = rng.normal(0.0, 0.5, shape)
        else:
            gain = 3.0 if name.endswith("router") else (2.0 if name.endswith((".o", ".down", ".proj")) else 1.0)
            a = rng.normal(0.0, gain / math.sqrt(shape[1]), shape)
        out[name] = torch.from_numpy(a.astype(np.float32)).to(torch.bfloat16)
    return out


def make_model_dir(name, root=None):
    from kappai_b200.weights.safetensors_io import save_safetensors

    cfg, seed = CONFIGS[name]
    d = tempfile.mkdtemp(prefix=f"vek_{name}_", dir=root)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_safetensors(os.path.join(d, "model.safetensors"), make_weights(cfg, seed))
    return d
