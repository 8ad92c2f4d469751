"""Tizusun: a decoder of post-norm layers, each an attention mixer and a gated feed-forward
(dense, or a mixture of experts).

    x <- norm1(alpha x + mixer(x)) ;  x <- norm2(alpha x + ff(x))        (a layer; ``alpha`` = ``postln_alpha``)

The mixer is grouped-query attention whose values are the key projections themselves (there is no value
matrix), with per-head RMS norm of q and k, a partial "rotate half" rotation whose frequencies are rescaled
by wavelength, a causal mask that stays inside the query's own block of ``mask.size`` positions, and a
sigmoid gate on the concatenated heads in front of the output matrix.  The dense feed-forward is
``Wd (relu(Wg h) * (Wu h))``; the experts of a mixture use silu, and a token's ``top`` experts are weighted by
the softmax over their router logits alone.  After the last layer: the final norm, then the (untied) head.

This file is the only place that knows the design's ``config.json`` keys and tensor names.  The layers are
listed in ``layers``, each with its ``type`` (the mixer), the mixer's sizes (``mixer``) and its feed-forward
(``mlp``, or null for none); layer i's tensors start with ``l<i>.``.  Every size and constant is read from
there; what the design fixes (the activations, the pairing of the rotation, the place of the norms) is
written below.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from ..config.schema import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TypedConfig, cfg
from ..config.registry import register_architecture

ARCHITECTURE = "Tizusun"
DENSE_ACTIVATION = "relu"
EXPERT_ACTIVATION = "silu"
SOFTMAX_WEIGHTS = "float32"        # the design computes scores and weights in 32-bit, also where they meet the values
DEFAULT_MAX_POSITIONS = 131072     # the design itself sets no limit; an optional key ``max_positions`` overrides


def _get(d: Dict[str, Any], key: str, where: str, typ=(int, float)):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing required key '{where}.{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, typ):
        raise ConfigError(f"config key '{where}.{key}': unexpected value {v!r}")
    return v


def _int(d, key, where) -> int:
    v = _get(d, key, where)
    if int(v) != v:
        raise ConfigError(f"config key '{where}.{key}': expected an integer, got {v!r}")
    return int(v)


@dataclass
class TizusunConfig(TypedConfig):
    vocab: int = cfg()
    width: int = cfg()
    layers: List[dict] = cfg()
    norm: dict = cfg()
    postln_alpha: float = cfg()
    max_positions: int = cfg(DEFAULT_MAX_POSITIONS)
    eos_token_id: Optional[int] = cfg(None)

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("vocab and width must be positive")
        if not self.layers:
            raise ConfigError("layers must list at least one layer")
        self.eps = float(_get(self.norm, "eps", "norm"))
        if self.eps <= 0:
            raise ConfigError("norm.eps must be positive")
        if self.max_positions < 1:
            raise ConfigError("max_positions must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config key '{where}': expected an object")
            kind = _get(layer, "type", where, str)
            if kind != "attention":
                raise ConfigError(f"config key '{where}.type'='{kind}': this design has the mixer 'attention' only")
            m = layer.get("mixer")
            H, G = _int(m, "heads", where + ".mixer"), _int(m, "kv_heads", where + ".mixer")
            dim, vdim = _int(m, "dim", where + ".mixer"), _int(m, "vdim", where + ".mixer")
            _get(m, "scale", where + ".mixer")
            if H < 1 or G < 1 or H % G:
                raise ConfigError(f"{where}.mixer: heads={H} must be a positive multiple of kv_heads={G}")
            if vdim != dim:
                raise ConfigError(f"{where}.mixer: vdim={vdim} differs from dim={dim}, but the values are the key projections")
            if m.get("mask"):
                if _int(m["mask"], "size", where + ".mixer.mask") < 1:
                    raise ConfigError(f"{where}.mixer.mask.size must be positive")
            rot = m.get("rot")
            if rot:
                dims = _int(rot, "dims", where + ".mixer.rot")
                _get(rot, "base", where + ".mixer.rot")
                if dims < 2 or dims % 2 or dims > dim:
                    raise ConfigError(f"{where}.mixer.rot.dims={dims} must be even and at most dim={dim}")
                if rot.get("scaling"):
                    for k in ("factor", "low", "high", "original"):
                        _get(rot["scaling"], k, where + ".mixer.rot.scaling")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", where + ".mlp", str)
                if mk == "dense":
                    if _int(mlp, "ff", where + ".mlp") < 1:
                        raise ConfigError(f"{where}.mlp.ff must be positive")
                elif mk == "moe":
                    if _int(mlp.get("expert"), "ff", where + ".mlp.expert") < 1:
                        raise ConfigError(f"{where}.mlp.expert.ff must be positive")
                    E = _int(mlp.get("router"), "experts", where + ".mlp.router")
                    top = _int(mlp.get("router"), "top", where + ".mlp.router")
                    if E < 1 or not (1 <= top <= E):
                        raise ConfigError(f"{where}.mlp.router: top={top} must lie between 1 and experts={E}")
                else:
                    raise ConfigError(f"config key '{where}.mlp.kind'='{mk}': expected 'dense' or 'moe'")


def _mixer_spec(c: TizusunConfig, m: Dict[str, Any], prefix: str) -> PartSpec:
    rot, mask = m.get("rot"), m.get("mask")
    position = None
    if rot:
        position = PartSpec("rope", {"rotary_dim": int(rot["dims"]), "theta": float(rot["base"]), "pairing": "neox",
                                     "scaling": dict(rot["scaling"]) if rot.get("scaling") else None})
    return PartSpec(
        "attention",
        {"hidden_size": c.width, "num_heads": int(m["heads"]), "num_kv_heads": int(m["kv_heads"]),
         "head_dim": int(m["dim"]), "qk_norm_eps": c.eps, "scale": float(m["scale"]), "window": None,
         "block": int(mask["size"]) if mask else None, "values": "keys", "gate": "sigmoid",
         "softmax_weights": SOFTMAX_WEIGHTS,
         "position": position, "bias": False},
        prefix,
        rename={"q_proj.weight": "q", "k_proj.weight": "k", "q_norm.weight": "q.norm", "k_norm.weight": "k.norm",
                "gate_proj.weight": "g", "out_proj.weight": "o"})


def _ffn_spec(c: TizusunConfig, mlp: Optional[Dict[str, Any]], prefix: str) -> Optional[PartSpec]:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("glu", {"hidden_size": c.width, "intermediate_size": int(mlp["ff"]), "bias": False,
                                "activation": DENSE_ACTIVATION},
                        prefix, rename={"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"})
    E = int(mlp["router"]["experts"])
    rename = {"router.weight": "router", "router.bias": "router.b"}
    for e in range(E):
        for local, name in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
            rename[f"experts.{e}.{local}.weight"] = f"e{e}.{name}"
    return PartSpec("moe", {"hidden_size": c.width, "expert_size": int(mlp["expert"]["ff"]), "num_experts": E,
                            "top": int(mlp["router"]["top"]), "activation": EXPERT_ACTIVATION, "router_bias": True},
                    prefix, rename=rename)


def build_spec(c: TizusunConfig) -> ModelSpec:
    norm = lambda prefix, name: PartSpec("rmsnorm", {"size": c.width, "eps": c.eps}, prefix, rename={"weight": name})
    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        ffn = _ffn_spec(c, layer.get("mlp"), p + "mlp.")
        layers.append(LayerSpec(mixer=_mixer_spec(c, layer["mixer"], p + "mix."), ffn=ffn,
                                mixer_norm=norm(p, "norm1"), ffn_norm=norm(p, "norm2") if ffn is not None else None,
                                block="postnorm_residual", block_params={"alpha": float(c.postln_alpha)}))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": None}, "",
                           rename={"weight": "embed"}),
        layers=layers,
        schedule=[ScheduleEntry(i) for i in range(len(layers))],
        final_norm=norm("", "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": False}, "",
                      rename={"weight": "head"}),
        eos_token_id=c.eos_token_id,
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, TizusunConfig, build_spec)
