"""Vekuzen without a GPU: the configuration reader and its errors, the tensor names and shapes of every test
configuration, the order of the layer runs, and the plain mechanisms on cases worked out by hand."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_vekuzen as P
from vekuzen_configs import CONFIGS, make_model_dir, tensor_shapes


def _spec(cfg):
    from kappai_b200.config.registry import config_from_dict
    arch, c = config_from_dict(cfg)
    assert arch.name == "Vekuzen"
    return arch.build_spec(c)


def _model(cfg):
    from kappai_b200.engine.model import Model
    from kappai_b200.parts.base import BuildEnv
    return Model(_spec(cfg), BuildEnv(torch.device("cpu"), torch.float32, 32))


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    cfg = CONFIGS[name][0]
    table = {n: tuple(ws.shape) for n, ws in _model(cfg).weight_table().items()}
    assert table == tensor_shapes(cfg)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_order_of_the_layer_runs_and_their_caches(name):
    from kappai_b200.cache.spec import PagedKVSpec, StateSpec
    cfg = CONFIGS[name][0]
    m = _model(cfg)
    runs = P.layer_runs(cfg)
    assert [(e.layer, e.enter) for e in m.schedule] == runs
    specs = m.cache_specs()
    assert len(specs) == len(runs)                   # every run has a cache or a state of its own
    for (i, _), s in zip(runs, specs):
        mix = cfg["layers"][i]["mixer"]
        if cfg["layers"][i]["type"] == "lightning":
            assert s == StateSpec((mix["heads"], mix["dim"], mix["vdim"]), "float32")
        else:
            assert isinstance(s, PagedKVSpec) and s.num_kv_heads == mix["heads"]
            assert s.head_dim >= max(mix["dim"], mix["vdim"]) and s.head_dim % 16 == 0 and s.window is None


def test_no_loop_and_no_side_inputs_mean_no_such_tensors():
    cfg = CONFIGS["B"][0]
    names = set(_model(cfg).weight_table())
    assert "loop.in" not in names and "side.embed" not in names and not any(".side." in n for n in names)
    m = _model(cfg)
    assert m.entry is None and m.token_table is None and all(b.side is None for b in m.blocks)


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][0].update(type="attention"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"].pop("scale"), "scale"),
    (lambda c: c["layers"][1]["mlp"].update(kind="conv"), "kind"),
    (lambda c: c.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda c: c.update(loop={"start": 0, "stop": 9, "times": 2}), "loop"),
    (lambda c: c["loop"].pop("times"), "times"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["token_side"].pop("dim"), "dim"),
    (lambda c: c["embedding"].pop("scale"), "scale"),
])
def test_configuration_errors_name_the_key(change, word):
    from kappai_b200.config.schema import ConfigError
    cfg = copy.deepcopy(CONFIGS["A"][0])
    change(cfg)
    with pytest.raises(ConfigError) as e:
        _spec(cfg)
    assert word in str(e.value)


def test_keys_that_may_be_left_out():
    cfg = copy.deepcopy(CONFIGS["A"][0])
    for k in ("embedding", "logit_scale", "loop", "token_side"):
        cfg.pop(k)
    spec = _spec(cfg)
    assert spec.embedding.params["scale"] == 1.0 and spec.head.params["scale"] == 1.0
    assert spec.entry is None and spec.token_table is None and [e.layer for e in spec.schedule] == [0, 1, 2]


def test_missing_and_unexpected_tensors_are_listed(tmp_path):
    from kappai_b200.weights.loader import WeightError, load_weights
    from kappai_b200.weights.safetensors_io import save_safetensors
    from vekuzen_configs import make_weights
    import json, os
    cfg, seed = CONFIGS["C"]
    w = make_weights(cfg, seed)
    w.pop("l1.mlp.correction"); w.pop("loop.in")
    w["l0.mix.k"] = w["l0.mix.uk"]
    d = tmp_path / "m"
    os.makedirs(d)
    (d / "config.json").write_text(json.dumps(cfg))
    save_safetensors(str(d / "model.safetensors"), w)
    with pytest.raises(WeightError) as e:
        load_weights(_model(cfg), str(d))
    assert set(e.value.missing) == {"l1.mlp.correction", "loop.in"} and e.value.unexpected == ["l0.mix.k"]


# ------------------------------------------------------------------------- the plain mechanisms, by hand

def test_plain_lightning_by_hand():
    # one head, dim 1, vdim 1, identity projections: S_t = a S_(t-1) + k_t v_t, o_t = S_t q_t
    one = np.ones((1, 1))
    h = np.array([[1.0], [2.0], [0.5]])
    s = P.silu(h[:, 0])
    a = 0.5
    S, want = 0.0, []
    for t in range(3):
        S = a * S + s[t] * s[t]
        want.append(S * s[t])
    # the norm over a single value leaves its sign (times the weight); so look at the state instead
    _, state = P.lightning(h, one, one, one, one, one, np.ones(1), [a], 1, 1, 1, 1e-12)
    assert abs(state[0, 0, 0] - S) < 1e-12
    # and a state handed in continues the recurrence: two halves equal the whole
    rng = np.random.default_rng(0)
    hh = rng.normal(size=(9, 6))
    W = [rng.normal(size=(8, 6)) for _ in range(2)] + [rng.normal(size=(4, 6)) for _ in range(2)]
    args = (rng.normal(size=(6, 4)), np.ones(4), [0.9, 0.5], 2, 4, 2, 1e-6)
    whole, S_all = P.lightning(hh, *W, *args)
    first, S1 = P.lightning(hh[:4], *W, *args)
    second, S2 = P.lightning(hh[4:], *W, *args, state=S1)
    assert np.allclose(np.concatenate([first, second]), whole) and np.allclose(S2, S_all)


def test_plain_route_by_hand():
    # logits ln 1, ln 2, ln 5 -> scores 1/8, 2/8, 5/8; the correction lifts the first over the second for the choice only
    h = np.ones((1, 1))
    w_router = np.log(np.array([[1.0], [2.0], [5.0]]))
    idx, wts, s = P.route(h, w_router, np.array([0.2, 0.0, 0.0]), 2, 3.0)
    assert np.allclose(s, [[0.125, 0.25, 0.625]])
    assert idx.tolist() == [[2, 0]] and np.allclose(wts, [[0.625 * 3, 0.125 * 3]])
    assert np.allclose(P.choice_margin(h, w_router, np.array([0.2, 0.0, 0.0]), 2), [0.325 - 0.25])


def test_plain_identity_expert_returns_its_input():
    h = np.array([[1.0, -2.0]])
    w_router = np.array([[0.0, 0.0], [10.0, 0.0]])              # the second output (an identity expert) wins
    zero = (np.zeros((3, 2)), np.zeros((3, 2)), np.zeros((2, 3)))
    out = P.mixture(h, w_router, np.zeros(2), [zero], 1, 1, 2.0)
    s = 1.0 / (1.0 + math.exp(-10.0))
    assert np.allclose(out, 2.0 * s * h)


def test_plain_side_input_and_loop_entry_by_hand():
    x = np.array([[3.0, 4.0]])
    table = np.array([[9.0, 9.0, 1.0, 0.5]])                    # part 1 of two columns: (1, 0.5)
    w_gate = np.array([[1.0, 0.0], [0.0, 1.0]])
    w_proj = np.array([[1.0, 0.0], [0.0, 2.0]])
    g = P.gelu_tanh(x[0]) * np.array([1.0, 0.5])
    y = np.array([g[0], 2 * g[1]])
    want = x[0] + y / math.sqrt((y ** 2).mean() + 1e-5) * np.array([1.0, 3.0])
    got = P.token_side(x, [0], table, 1, 2, w_gate, w_proj, np.array([1.0, 3.0]), 1e-5)
    assert np.allclose(got[0], want)
    w_in = np.array([[1.0, 0.0, 0.0, 2.0], [0.0, 1.0, 3.0, 0.0]])
    assert np.allclose(P.loop_entry(x, np.array([[5.0, 6.0]]), w_in), [[3 + 12, 4 + 15]])


def test_plain_model_prefix_property():
    """The logits at a position depend on the tokens up to it only (every mixer is causal)."""
    import tempfile
    d = make_model_dir("C", tempfile.mkdtemp())
    m = P.PlainVekuzen(d)
    toks = list(np.random.default_rng(1).integers(0, 19, 23))
    full = m.forward(toks)
    assert np.allclose(m.forward(toks[:11]), full[:11], atol=1e-9)


def test_chunk_list_of_the_lightning_kernels():
    """Segments in chunks of 64 rows from their first row in the step; the short segments that lead are left out
    (the scan takes them) and the others are numbered from 0; a short segment further on keeps its chunk."""
    from kappai_b200.engine.batch import StepSegments
    from kappai_b200.parts.lightning import CHUNKED_FROM, lightning_chunks
    lens = [1, 3, 100, 1, 70]
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    t = lightning_chunks(StepSegments(sum(lens), 5, cu, np.zeros(5, np.int32), lens, max(lens), False), 64)
    assert t.scalars == {"n_chunks": 5, "n_lead": 2}
    assert t.arrays["chunk_seg"].tolist() == [0, 0, 1, 2, 2]
    assert t.arrays["chunk_row0"].tolist() == [4, 68, 104, 105, 169]
    assert t.arrays["seg_chunk0"].tolist() == [0, 2, 3, 5]
    short = [CHUNKED_FROM - 1, 1]
    cu = np.array([0, short[0], sum(short)], np.int32)
    assert lightning_chunks(StepSegments(sum(short), 2, cu, np.zeros(2, np.int32), short, max(short), False), 64) is None
