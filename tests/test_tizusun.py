"""Tizusun without a GPU: configuration, tensor names, the registry, the rotary frequencies and the plain
implementation's own mechanisms on cases small enough to work out by hand."""
import copy
import json
import math
import os

import numpy as np
import pytest

import plain_tizusun as P
from tizusun_configs import CONFIGS, TIZ_P, TIZ_Q, make_model_dir, tensor_shapes


def _spec(cfg):
    from kappai_b200.config.registry import config_from_dict
    arch, c = config_from_dict(cfg)
    return arch, arch.build_spec(c)


def test_the_architecture_is_chosen_by_config_json():
    arch, spec = _spec(TIZ_P)
    assert arch.name == "Tizusun" and spec.vocab_size == 211 and len(spec.layers) == 3
    assert spec.layers[0].block == "postnorm_residual" and spec.layers[0].block_params == {"alpha": 1.5}
    assert spec.layers[0].ffn.kind == "moe" and spec.layers[1].ffn.kind == "glu"
    assert spec.layers[1].ffn.params["activation"] == "relu" and spec.layers[0].ffn.params["activation"] == "silu"
    m = spec.layers[0].mixer.params
    assert m["values"] == "keys" and m["gate"] == "sigmoid" and m["block"] == 24 and m["position"].params["rotary_dim"] == 16


@pytest.mark.parametrize("name", list(CONFIGS))
def test_tensor_names_and_shapes(name):
    import torch
    from kappai_b200.engine.model import Model
    from kappai_b200.parts.base import BuildEnv
    cfg = CONFIGS[name][0]
    _, spec = _spec(cfg)
    table = Model(spec, BuildEnv(torch.device("cpu"), torch.float32, 16)).weight_table()
    want = tensor_shapes(cfg)
    assert set(table) == set(want)
    assert all(tuple(table[n].shape) == tuple(want[n]) for n in want)


def test_a_layer_without_feed_forward_has_one_norm():
    _, spec = _spec(TIZ_Q)
    assert spec.layers[1].ffn is None and spec.layers[1].ffn_norm is None and spec.layers[1].mixer_norm is not None


@pytest.mark.parametrize("path,value,match", [
    (("layers", 0, "type"), "recurrent", "type"),
    (("layers", 0, "mixer", "vdim"), 16, "vdim"),
    (("layers", 0, "mixer", "heads"), 3, "multiple"),
    (("layers", 0, "mixer", "rot", "dims"), 15, "dims"),
    (("layers", 0, "mlp", "router", "top"), 7, "top"),
    (("layers", 1, "mlp", "kind"), "sparse", "kind"),
    (("norm",), {}, "norm.eps"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask"),
])
def test_bad_configurations_name_the_key(path, value, match):
    from kappai_b200.config.schema import ConfigError
    cfg = copy.deepcopy(TIZ_P)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        _spec(cfg)


def test_missing_weights_are_listed(tmp_path):
    import torch
    from kappai_b200.engine.model import Model
    from kappai_b200.parts.base import BuildEnv
    from kappai_b200.weights.loader import WeightError, load_weights
    from kappai_b200.weights.safetensors_io import SafetensorsFile, save_safetensors
    d = make_model_dir("Q", str(tmp_path))
    f = SafetensorsFile(os.path.join(d, "model.safetensors"))
    tensors = {k: f.tensor(k).clone() for k in f.keys() if k not in ("l2.mlp.router.b", "l1.mix.g")}
    f.close()
    tensors["l1.mix.v"] = torch.zeros(3)
    save_safetensors(os.path.join(d, "model.safetensors"), tensors)
    _, spec = _spec(CONFIGS["Q"][0])
    with pytest.raises(WeightError) as e:
        load_weights(Model(spec, BuildEnv(torch.device("cpu"), torch.float32, 16)), d)
    assert set(e.value.missing) == {"l2.mlp.router.b", "l1.mix.g"} and e.value.unexpected == ["l1.mix.v"]


@pytest.mark.parametrize("dims,base,scaling", [
    (16, 10000.0, {"factor": 8.0, "low": 2.0, "high": 8.0, "original": 64}),
    (48, 500.0, None),
    (64, 500000.0, {"factor": 32.0, "low": 1.0, "high": 4.0, "original": 8192}),
])
def test_rotary_frequencies_of_the_part_are_the_plain_ones(dims, base, scaling):
    from kappai_b200.parts.position import scaled_frequencies
    f = np.power(base, -2.0 * np.arange(dims // 2, dtype=np.float64) / dims)
    sc = None if scaling is None else tuple(float(scaling[k]) for k in ("factor", "low", "high", "original"))
    got = scaled_frequencies(f, sc)
    want = P.rotary_frequencies(dims, base, scaling)
    assert np.allclose(got, want, rtol=1e-14, atol=0)
    if scaling is not None:
        lam = 2 * math.pi / f
        kept, cut = lam < scaling["original"] / scaling["high"], lam > scaling["original"] / scaling["low"]
        assert kept.any() and np.array_equal(got[kept], f[kept]) and np.allclose(got[cut], f[cut] / scaling["factor"])
        mid = ~kept & ~cut
        assert np.all(got[mid] < f[mid]) and np.all(got[mid] > f[mid] / scaling["factor"])


# ---- the plain mechanisms on cases that can be checked by hand

def test_plain_block_mask():
    vis = P.block_causal_mask(np.arange(7), 3)
    assert vis.astype(int).tolist() == [[1, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0],
                                        [0, 0, 0, 1, 0, 0, 0], [0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 0],
                                        [0, 0, 0, 0, 0, 0, 1]]
    assert P.block_causal_mask(np.arange(4), None).astype(int).tolist() == np.tril(np.ones((4, 4), int)).tolist()


def test_plain_rotation_and_norm():
    x = np.zeros((1, 1, 6)); x[0, 0] = [1, 2, 3, 4, 5, 6]
    y = P.rotate_half(x, [1], np.array([math.pi / 2, math.pi]), 4)          # pairs (0,2) and (1,3); 4, 5 pass
    assert np.allclose(y[0, 0], [-3, -2, 1, -4, 5, 6])
    assert np.allclose(P.rms_norm(np.array([3.0, 4.0]), np.array([2.0, 1.0]), 0.0), [2 * 3 / math.sqrt(12.5), 4 / math.sqrt(12.5)])


def test_plain_router_and_mixture():
    h = np.array([[1.0, 0.0], [0.0, 1.0]])
    w = np.array([[1.0, 0.0], [2.0, 0.0], [0.0, 3.0]]); b = np.array([0.0, 0.0, -1.0])
    idx, wt = P.router(h, w, b, 2)
    assert idx.tolist() == [[1, 0], [2, 0]]
    assert np.allclose(wt[0], np.exp([2.0, 1.0]) / np.exp([2.0, 1.0]).sum()) and np.allclose(wt[1], np.exp([2.0, 0.0]) / (np.exp(2.0) + 1))
    ws = {"router": w, "router.b": b}
    for e in range(3):
        ws.update({f"e{e}.gate": np.full((1, 2), 1.0), f"e{e}.up": np.full((1, 2), float(e + 1)), f"e{e}.down": np.array([[1.0], [0.0]])})
    out = P.mixture(h, ws, 3, 2, "silu")
    silu1 = 1.0 / (1.0 + math.exp(-1.0))
    assert np.allclose(out[0], [silu1 * (2 * wt[0, 0] + 1 * wt[0, 1]), 0.0])


def test_plain_values_are_the_unrotated_keys():
    """One head, identity matrices, a score that singles out key 1 for the last row: the output is W_k h of that
    key as it is (no norm, no rotation), times the gate."""
    d = 4
    h = np.array([[0.0, 1.0, 0.0, 0.0], [5.0, 0.0, 0.0, 0.0], [1.0, 0.0, 0.0, 0.0]])
    w = {"q": np.eye(d) * 1.0, "k": np.eye(d), "q.norm": np.ones(d), "k.norm": np.ones(d), "g": np.zeros((d, d)), "o": np.eye(d)}
    m = {"heads": 1, "kv_heads": 1, "dim": d, "vdim": d, "scale": 10.0, "rot": None, "mask": None}
    out = P.attention_mixer(h, w, m, 1e-6, np.arange(3))
    # row 2's query is parallel to keys 1 and 2 (equal after the norm): it reads the mean of their values, halved by the gate
    assert np.allclose(out[2], 0.5 * (h[1] + h[2]) / 2, atol=1e-3)
