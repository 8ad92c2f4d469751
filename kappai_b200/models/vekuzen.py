"""Vekuzen: a decoder of pre-norm layers with two kinds of mixer, a looped stretch of layers and a per-layer
token input.

    x = embed[token] * embedding.scale + pos[p]                                   (x0: this x, kept)
    a layer:   x <- x + mixer(norm1(x)) ;  x <- x + ff(norm2(x)) ;  x <- x + side_i(x, token)
    a loop:    layers loop.start .. loop.stop - 1 run loop.times times in a row with the same weights, every pass
               with caches and states of its own; in front of every pass x <- W_in [x; x0]
    output:    logits = head(norm(x)) * logit_scale

The mixers: ``lightning`` (linear attention with one decay a head and a float32 state, silu on q, k and v, a norm
over all heads together, a sigmoid gate; parts/lightning.py) and ``latent_attention`` (queries, keys and values
expanded from normed low-rank latents, causal softmax without positions, a sigmoid gate; parts/attention.py).  The
feed-forwards: a gated unit with tanh-gelu, or a mixture of silu units chosen by ``softmax(z) + correction`` and
weighted by ``softmax(z) * router.scale`` (not renormalised), whose last ``router.identity`` router outputs stand
for experts that return their input, beside a shared unit times one sigmoid gate a token.  The side input of layer
i reads columns ``[i dim, (i + 1) dim)`` of the table ``side.embed`` (``token_side.dim``), in every pass of a loop
the same.

This file is the only place that knows the design's ``config.json`` keys and tensor names.  The layers are listed
in ``layers``, each with its ``type`` (the mixer), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or
null for none); layer i's tensors start with ``l<i>.``.  Every size and constant is read from there; what the
design fixes (activations, the kinds of gates, the place of the norms) is written below.  ``loop``,
``token_side``, ``embedding`` and ``logit_scale`` may be left out: the model then has no loop, no side inputs, an
embedding that is not scaled, logits that are not scaled.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

from ..config.schema import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TypedConfig, cfg
from ..config.registry import register_architecture

ARCHITECTURE = "Vekuzen"
DENSE_ACTIVATION = "gelu_tanh"
EXPERT_ACTIVATION = "silu"
SIDE_ACTIVATION = "gelu_tanh"
LIGHTNING_ACTIVATION = "silu"
SOFTMAX_WEIGHTS = "float32"        # scores and weights are 32-bit, also where they meet the values


def _get(d: Any, key: str, where: str, typ=(int, float)):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: missing required key '{where}.{key}'")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, typ):
        raise ConfigError(f"config key '{where}.{key}': unexpected value {v!r}")
    return v


def _int(d, key, where, least: int = 1) -> int:
    v = _get(d, key, where)
    if int(v) != v or int(v) < least:
        raise ConfigError(f"config key '{where}.{key}': expected an integer of at least {least}, got {v!r}")
    return int(v)


@dataclass
class VekuzenConfig(TypedConfig):
    vocab: int = cfg()
    width: int = cfg()
    layers: List[dict] = cfg()
    norm: dict = cfg()
    embedding: Optional[dict] = cfg(None)
    max_positions: int = cfg()
    logit_scale: float = cfg(1.0)
    loop: Optional[dict] = cfg(None)
    token_side: Optional[dict] = cfg(None)
    eos_token_id: Optional[int] = cfg(None)

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1:
            raise ConfigError("vocab and width must be positive")
        if not self.layers:
            raise ConfigError("layers must list at least one layer")
        if self.max_positions < 1:
            raise ConfigError("max_positions must be positive")
        self.eps = float(_get(self.norm, "eps", "norm"))
        if self.eps <= 0:
            raise ConfigError("norm.eps must be positive")
        # (an embedding without a scale is not scaled)
        self.embedding_scale = float(_get(self.embedding, "scale", "embedding")) if self.embedding is not None else 1.0
        self.side_dim = _int(self.token_side, "dim", "token_side") if self.token_side is not None else None
        n = len(self.layers)
        if self.loop is not None:
            a, b = _int(self.loop, "start", "loop", 0), _int(self.loop, "stop", "loop", 0)
            _int(self.loop, "times", "loop")
            if not (0 <= a < b <= n):
                raise ConfigError(f"loop: start={a}, stop={b} must name a stretch of the {n} layers")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict):
                raise ConfigError(f"config key '{where}': expected an object")
            kind = _get(layer, "type", where, str)
            m, mw = layer.get("mixer"), where + ".mixer"
            H = _int(m, "heads", mw)
            _int(m, "dim", mw), _int(m, "vdim", mw)
            if kind == "lightning":
                decay = _get(m, "decay", mw, list)
                if len(decay) != H or any(isinstance(a, bool) or not isinstance(a, (int, float)) for a in decay):
                    raise ConfigError(f"{mw}.decay must list one number for each of the {H} heads")
            elif kind == "latent_attention":
                _int(m, "q_rank", mw), _int(m, "kv_rank", mw)
                _get(m, "scale", mw)
            else:
                raise ConfigError(f"config key '{where}.type'='{kind}': expected 'lightning' or 'latent_attention'")
            mlp = layer.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", where + ".mlp", str)
                if mk == "dense":
                    _int(mlp, "ff", where + ".mlp")
                elif mk == "moe":
                    _int(mlp.get("expert"), "ff", where + ".mlp.expert")
                    r, rw = mlp.get("router"), where + ".mlp.router"
                    E, top = _int(r, "experts", rw), _int(r, "top", rw)
                    ident = _int(r, "identity", rw, 0) if r.get("identity") is not None else 0
                    _get(r, "scale", rw)
                    if top > E + ident:
                        raise ConfigError(f"{rw}: top={top} exceeds the {E + ident} router outputs")
                    if mlp.get("shared"):
                        _int(mlp["shared"], "ff", where + ".mlp.shared")
                else:
                    raise ConfigError(f"config key '{where}.mlp.kind'='{mk}': expected 'dense' or 'moe'")


def _mixer_spec(c: VekuzenConfig, layer: Dict[str, Any], prefix: str) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "lightning":
        return PartSpec(
            "lightning",
            {"hidden_size": c.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
             "decay": [float(a) for a in m["decay"]], "norm_eps": c.eps, "activation": LIGHTNING_ACTIVATION,
             "gate": "sigmoid"},
            prefix,
            rename={"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "gate_proj.weight": "g",
                    "out_proj.weight": "o", "norm.weight": "norm"})
    return PartSpec(
        "latent_attention",
        {"hidden_size": c.width, "num_heads": int(m["heads"]), "head_dim": int(m["dim"]), "value_dim": int(m["vdim"]),
         "q_rank": int(m["q_rank"]), "kv_rank": int(m["kv_rank"]), "scale": float(m["scale"]), "norm_eps": c.eps,
         "gate": "sigmoid", "softmax_weights": SOFTMAX_WEIGHTS},
        prefix,
        rename={"q_down.weight": "dq", "q_norm.weight": "dq.norm", "q_up.weight": "uq", "kv_down.weight": "dkv",
                "kv_norm.weight": "dkv.norm", "k_up.weight": "uk", "v_up.weight": "uv", "gate_proj.weight": "g",
                "out_proj.weight": "o"})


def _ffn_spec(c: VekuzenConfig, mlp: Optional[Dict[str, Any]], prefix: str) -> Optional[PartSpec]:
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("glu", {"hidden_size": c.width, "intermediate_size": int(mlp["ff"]), "bias": False,
                                "activation": DENSE_ACTIVATION},
                        prefix, rename={"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"})
    r = mlp["router"]
    E = int(r["experts"])
    rename = {"router.weight": "router", "router.correction": "correction"}
    for e in range(E):
        for local, name in (("gate_proj", "gate"), ("up_proj", "up"), ("down_proj", "down")):
            rename[f"experts.{e}.{local}.weight"] = f"e{e}.{name}"
    params = {"hidden_size": c.width, "expert_size": int(mlp["expert"]["ff"]), "num_experts": E, "top": int(r["top"]),
              "activation": EXPERT_ACTIVATION, "routing": "softmax_all", "router_scale": float(r["scale"]),
              "identity_experts": int(r.get("identity") or 0)}
    if mlp.get("shared"):
        params.update(shared_size=int(mlp["shared"]["ff"]), shared_gate="sigmoid")
        rename.update({"shared.gate_proj.weight": "shared.gate", "shared.up_proj.weight": "shared.up",
                       "shared.down_proj.weight": "shared.down", "shared.gate.weight": "shared.sg"})
    return PartSpec("moe", params, prefix, rename=rename)


def layer_schedule(c: VekuzenConfig) -> List[ScheduleEntry]:
    """The order in which the layers run: the looped stretch ``times`` times, the head of every pass marked."""
    n = len(c.layers)
    if c.loop is None:
        return [ScheduleEntry(i) for i in range(n)]
    a, b, times = int(c.loop["start"]), int(c.loop["stop"]), int(c.loop["times"])
    sched = [ScheduleEntry(i) for i in range(a)]
    for _ in range(times):
        sched += [ScheduleEntry(i, enter=(i == a)) for i in range(a, b)]
    return sched + [ScheduleEntry(i) for i in range(b, n)]


def build_spec(c: VekuzenConfig) -> ModelSpec:
    norm = lambda prefix, name: PartSpec("rmsnorm", {"size": c.width, "eps": c.eps}, prefix, rename={"weight": name})
    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        ffn = _ffn_spec(c, layer.get("mlp"), p + "mlp.")
        side = None
        if c.side_dim is not None:
            side = PartSpec("token_gated", {"hidden_size": c.width, "dim": c.side_dim, "part": i, "eps": c.eps,
                                            "activation": SIDE_ACTIVATION},
                            p + "side.", rename={"gate.weight": "gate", "proj.weight": "proj", "norm.weight": "norm"})
        layers.append(LayerSpec(mixer=_mixer_spec(c, layer, p + "mix."), ffn=ffn, mixer_norm=norm(p, "norm1"),
                                ffn_norm=norm(p, "norm2") if ffn is not None else None, block="prenorm_residual",
                                side=side))
    spec = ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("embedding", {"vocab_size": c.vocab, "hidden_size": c.width, "scale": c.embedding_scale,
                                         "positions": c.max_positions}, "",
                           rename={"weight": "embed", "positions.weight": "pos"}),
        layers=layers,
        schedule=layer_schedule(c),
        final_norm=norm("", "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": c.width, "tied": False,
                                  "scale": float(c.logit_scale)}, "", rename={"weight": "head"}),
        eos_token_id=c.eos_token_id,
        entry=PartSpec("concat_linear", {"hidden_size": c.width}, "", rename={"weight": "loop.in"}) if c.loop is not None else None,
        token_table=(PartSpec("token_table", {"vocab_size": c.vocab, "width": c.side_dim * len(c.layers)}, "",
                              rename={"weight": "side.embed"}) if c.side_dim is not None else None),
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, VekuzenConfig, build_spec)
