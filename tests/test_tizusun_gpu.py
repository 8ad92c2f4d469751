"""Tizusun on the GPU: every new mechanism's kernel against the plain functions, then whole models through the
step function, the trace runner and the engine in every way of cutting the work."""
import math

import numpy as np
import pytest
import torch

import plain_tizusun as P
import replay_util as R
from tizusun_configs import CONFIGS, make_model_dir
from tolerances import tol_for

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=torch.float32).to(DEV).to(dtype).contiguous()


def bf16_round(a):
    return torch.as_tensor(np.asarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy().astype(np.float64)


@pytest.fixture(scope="module")
def tiz_dirs(tmp_path_factory):
    root = tmp_path_factory.mktemp("tizusun")
    return {n: make_model_dir(n, str(root)) for n in CONFIGS}


@pytest.fixture(scope="module")
def tiz_plain(tiz_dirs):
    return {n: P.PlainTizusun(d) for n, d in tiz_dirs.items()}


# ------------------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("n,d", [(1, 48), (5, 328), (300, 36), (3, 2500), (2, 9000), (4, 37)])
def test_postnorm_rows(n, d):
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(d)
    a, w = rng.normal(0, 3, (n, d)), 1 + rng.normal(0, 0.2, d)
    want = P.rms_norm(a, w, 1e-5)
    acc = dev(a)
    x, h, sc = torch.empty_like(acc), torch.empty((n, d), dtype=torch.bfloat16, device=DEV), torch.empty_like(acc)
    K.postnorm_rows(acc, dev(w), 1e-5, x_out=x, h_out=h, scaled_out=sc, alpha=1.75)
    assert np.abs(x.cpu().numpy() - want).max() < 1e-5
    assert np.abs(sc.cpu().numpy() - 1.75 * want).max() < 3e-5
    assert torch.equal(h, x.to(torch.bfloat16))
    K.postnorm_rows(acc, dev(w), 1e-5, scaled_out=acc, alpha=1.75)               # in place, the other outputs left out
    assert torch.equal(acc, sc)
    h32, sc2 = torch.empty_like(x), torch.empty_like(x)
    K.scale_cast(x, h32, sc2, 0.5)
    assert torch.equal(h32, x) and torch.equal(sc2, x * 0.5)


def test_sigmoid_gate_reads_columns_of_a_wider_row():
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(1)
    for dt, tol in ((torch.float32, 1e-6), (torch.bfloat16, 1e-2)):
        for c0 in (50, 56):                                     # columns that are not, and that are, 16-byte aligned
            o, wide = rng.normal(0, 1, (7, 40)), rng.normal(0, 2, (7, 104))
            od, wd = dev(o, dt), dev(wide, dt)
            K.sigmoid_gate(od, wd[:, c0:c0 + 40])
            want = dev(o, dt).float().cpu().numpy() * P.sigmoid(wd[:, c0:c0 + 40].float().cpu().numpy())
            assert np.abs(od.float().cpu().numpy() - want).max() <= tol


@pytest.mark.parametrize("act", ["relu", "silu", "gelu_tanh"])
def test_gated_activation_kernel(act):
    from kappai_b200.ops import kernels as K
    gu = np.random.default_rng(2).normal(0, 2, (9, 2 * 33))
    out = torch.empty((9, 33), dtype=torch.float32, device=DEV)
    K.swiglu(dev(gu), out, act)
    want = P.ACTIVATIONS[act](gu[:, :33]) * gu[:, 33:]
    assert np.abs(out.cpu().numpy() - want).max() < 1e-5


@pytest.mark.parametrize("M,K_,ff", [(4, 512, 256), (4, 96, 40), (100, 128, 64), (40, 1024, 512)])
def test_relu_in_the_products_gated_epilogue(M, K_, ff):
    """The fused epilogues of the weight-streaming, register-streaming and tcgen05 products with relu."""
    from kappai_b200.ops.linear import linear_swiglu
    rng = np.random.default_rng(M)
    a, w = bf16_round(rng.normal(0, 1, (M, K_))), bf16_round(rng.normal(0, 1 / math.sqrt(K_), (2 * ff, K_)))
    got = linear_swiglu(dev(a, torch.bfloat16), dev(w, torch.bfloat16), None, "relu").float().cpu().numpy()
    g, u = bf16_round(a @ w[:ff].T), bf16_round(a @ w[ff:].T)
    want = np.maximum(g, 0) * u
    assert np.abs(got - want).max() <= 0.02 * np.abs(want).max()
    assert np.array_equal(got == 0, want == 0) or np.mean((got == 0) != (want == 0)) < 0.01     # relu's zeros are zeros


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,hd,rot", [(4, 2, 32, 16), (3, 1, 48, 48), (10, 1, 24, 12), (4, 1, 64, 64), (2, 2, 128, 128),
                                        (4, 2, 64, 32), (3, 1, 64, 16), (2, 1, 128, 64), (2, 1, 128, 48), (5, 1, 64, 8)])
def test_qk_kernel_takes_the_values_from_the_key_columns(H, G, hd, rot, dt):
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(hd)
    n, page, extra = 11, 8, 24
    row = bf16_round(rng.normal(0, 1, (n, (H + G) * hd + extra)))
    qw, kw = 1 + rng.normal(0, 0.2, hd), 1 + rng.normal(0, 0.2, hd)
    pos = rng.permutation(40)[:n]
    f = P.rotary_frequencies(rot, 1000.0, {"factor": 3.0, "low": 2.0, "high": 8.0, "original": 32})
    ang = np.arange(64)[:, None] * f[None, :]
    q = P.rotate_half(P.rms_norm(row[:, :H * hd].reshape(n, H, hd), qw, 1e-5), pos, f, rot)
    k_raw = row[:, H * hd:(H + G) * hd].reshape(n, G, hd)
    k = P.rotate_half(P.rms_norm(k_raw, kw, 1e-5), pos, f, rot)
    cache = torch.zeros((8, 2, G, page, hd), dtype=dt, device=DEV)
    slots = rng.permutation(8 * page)[:n]
    q_out = torch.empty((n, H * hd), dtype=dt, device=DEV)
    K.qk_norm_rope_kv(dev(row, dt), dev(qw), dev(kw), 1e-5, dev(np.cos(ang)), dev(np.sin(ang)), rot, False,
                      torch.as_tensor(pos, dtype=torch.int32).to(DEV), torch.as_tensor(slots, dtype=torch.int32).to(DEV),
                      q_out, cache, page, H, G, hd, v_col=H * hd)
    tol = 1e-5 if dt == torch.float32 else 3e-2
    assert np.abs(q_out.float().cpu().numpy().reshape(n, H, hd) - q).max() < tol
    c = cache.float().cpu().numpy()
    for r in range(n):
        pg, off = divmod(int(slots[r]), page)
        assert np.abs(c[pg, 0, :, off] - k[r]).max() < tol
        assert np.array_equal(c[pg, 1, :, off], k_raw[r])                         # the values: the projection as it came


def _attention_case(rng, n_keys, H, G, hd, page, standout):
    """Keys and values of one sequence in a shuffled paged cache; ``standout`` maps a query row to the key whose
    score dwarfs the others if the row may see it."""
    k = rng.normal(0, 0.3, (n_keys, G, hd))
    v = rng.normal(0, 1, (n_keys, G, hd))
    n_pages = -(-n_keys // page)
    pages = rng.permutation(n_pages + 3)[:n_pages]
    cache = np.zeros((n_pages + 3, 2, G, page, hd))
    for t in range(n_keys):
        cache[pages[t // page], 0, :, t % page] = k[t]
        cache[pages[t // page], 1, :, t % page] = v[t]
    return k, v, pages, cache


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kernel", ["rows", "split", "split, whole weights"])
@pytest.mark.parametrize("H,G,hd,block,page", [(4, 2, 32, 24, 16), (3, 1, 48, 100, 64), (8, 1, 64, 512, 64), (2, 1, 16, 7, 8),
                                               (4, 2, 128, 300, 32)])
def test_a_key_just_inside_and_just_outside_the_block(H, G, hd, block, page, kernel, dt):
    """Rows at the first and last position of a block, in its middle and far into the sequence, with one key made to
    stand out: the block's first key (just inside), the key before it (just outside: it must not be seen), and a
    key far back inside a long block.  The kernels are compared with the plain masked softmax."""
    from kappai_b200.ops import kernels as K
    rng = np.random.default_rng(block)
    n_keys = max(3 * block + 5, 300) if block < 512 else 1300
    k, v, pages, cache = _attention_case(rng, n_keys, H, G, hd, page, None)
    k, v = bf16_round(k), bf16_round(v)
    cachet = dev(bf16_round(cache), dt)
    rows = sorted({0, 1, block - 1, block, block + 1, 2 * block - 1, 2 * block, 2 * block + block // 2, n_keys - 1,
                   (n_keys - 1) // block * block, (n_keys - 1) // block * block - 1} & set(range(n_keys)))
    q = bf16_round(rng.normal(0, 0.3, (len(rows), H, hd)))
    for i, p in enumerate(rows):
        b0 = p // block * block
        target = [b0, b0 - 1, b0 + (p - b0) // 2][i % 3]              # just inside, just outside, in the middle
        if target >= 0:
            g = rng.integers(0, G)
            q[i, g * (H // G):(g + 1) * (H // G)] = bf16_round(6.0 * k[target, g] / np.linalg.norm(k[target, g]))
            k[target, g] = bf16_round(6.0 * k[target, g] / np.linalg.norm(k[target, g]))
            pg = pages[target // page]
            cachet[pg, 0, g, target % page] = dev(k[target, g], dt)
    k = cachet.float().cpu().numpy()[pages].transpose(0, 3, 1, 2, 4)[:, :, 0].reshape(-1, G, hd)[:n_keys]     # what the kernels read
    want = np.zeros((len(rows), H, hd))
    for i, p in enumerate(rows):
        vis = P.block_causal_mask(np.arange(n_keys), block)[p]
        for h in range(H):
            g = h // (H // G)
            w = P.masked_softmax(((k[:, g] @ q[i, h]) * 0.7)[None], vis[None])[0]
            want[i, h] = w @ v[:, g]
    bt = torch.as_tensor(pages[None], dtype=torch.int32).to(DEV).contiguous()
    pos = torch.as_tensor(rows, dtype=torch.int32).to(DEV)
    row_seg = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
    qd = dev(q.reshape(len(rows), H * hd), dt)
    out = torch.empty_like(qd)
    if kernel == "rows":
        K.attention_rows(qd, cachet, bt, row_seg, pos, out, 0.7, None, page, H, G, hd, block)
    else:
        n_chunks = -(-n_keys // K.SPLIT_CHUNK)
        ws = torch.zeros(K.attention_split_scratch(len(rows), H, hd, n_chunks), dtype=torch.float32, device=DEV)
        K.attention_split(qd, cachet, bt, row_seg, pos, out, ws, n_chunks, 0.7, None, page, H, G, hd, block,
                          exact_weights="whole" in kernel)
    got = out.float().cpu().numpy().reshape(len(rows), H, hd)
    assert np.abs(got - want).max() < (2e-5 if dt == torch.float32 else 2e-2), (kernel, np.abs(got - want).max())
    if dt == torch.bfloat16 and "whole" in kernel:
        # nothing but the rounding of the output itself is left: half a unit in the last of bfloat16's 8 bits
        assert np.all(np.abs(got - want) <= np.abs(want) * 2.0 ** -8 + 1e-4), np.abs(got - want).max()


@pytest.mark.parametrize("variant", ["tcgen05 two heads a CTA", "tcgen05 one head a CTA", "mma.sync", "mma.sync, whole weights"])
@pytest.mark.parametrize("H,G,hd,page,block", [(4, 2, 64, 64, 100), (6, 1, 64, 16, 24), (2, 2, 128, 32, 130), (8, 2, 64, 64, 512),
                                               (2, 1, 64, 64, 128)])
def test_tiled_prompt_kernels_keep_to_the_block(H, G, hd, page, block, variant):
    """Prompt portions (from position 0, from the middle of a block, from a block's first position, single rows)
    through the tensor-core kernels with a block mask, against the plain masked softmax.  In every sequence the
    block's first key and the key before it are made to stand out for some rows."""
    from kappai_b200.ops import kernels as Kn
    from kappai_b200.ops.build import load_library
    from test_kernels_gpu import dev as dv, i32, paged_setup, rt
    DT = torch.bfloat16
    rng = np.random.default_rng(block)
    seq_lens = [3 * block + 17, 2 * block, block + 1, 700, 64]
    q_from = [0, block + block // 2, block, 650, 63]
    cache, bt, ks, vs = paged_setup(rng, seq_lens, page, G, hd, DT)
    qs = [rt(rng.standard_normal((L, H, hd)), DT) for L in seq_lens]
    for i, L in enumerate(seq_lens):
        for p in range(q_from[i], L, 5):
            b0 = p // block * block
            target = b0 if (p // 5) % 2 == 0 else b0 - 1                    # just inside / just outside
            if target >= 0:
                g = (p // 5) % G
                qs[i][p, g * (H // G):(g + 1) * (H // G)] = rt(ks[i][target, g] * 3.0, DT)
    old = Kn.USE_TC_ATTENTION
    Kn.USE_TC_ATTENTION = not variant.startswith("mma.sync")
    load_library("attention_tc").kp_attention_tc_set_pair(1 if "two heads" in variant else 0)
    try:
        rows, cu, seg_pos, tile_seg, tile_row0, big = [], [0], [], [], [], []
        for i, (L, a) in enumerate(zip(seq_lens, q_from)):
            rows.append(qs[i][a:])
            for r0 in range(cu[-1], cu[-1] + L - a, Kn.PREFILL_TILE):
                tile_seg.append(i); tile_row0.append(r0)
            for r0 in range(cu[-1], cu[-1] + L - a, 128):
                big.append((-(a + min(r0 + 128, cu[-1] + L - a) - cu[-1] - 1), i, r0))
            cu.append(cu[-1] + L - a)
            seg_pos.append(a)
        big.sort()
        q_rows = np.concatenate(rows, 0).reshape(cu[-1], H * hd)
        out = torch.empty((cu[-1], H * hd), dtype=DT, device=DEV)
        scale = 1.0 / math.sqrt(hd)
        Kn.attention_prefill(dv(q_rows, DT), dv(cache, DT), i32(bt), i32(cu), i32(seg_pos), i32(tile_seg), i32(tile_row0), out,
                             scale, None, page, H, G, hd, i32([x[1] for x in big]), i32([x[2] for x in big]), block=block,
                             exact_weights="whole" in variant)
        got = out.cpu().double().numpy().reshape(cu[-1], H, hd)
        assert Kn.attention_tc_status() == 0 and Kn.attention_mma_status() == 0
    finally:
        Kn.USE_TC_ATTENTION = old
        load_library("attention_tc").kp_attention_tc_set_pair(1)
    for i, (L, a) in enumerate(zip(seq_lens, q_from)):
        vis = P.block_causal_mask(np.arange(L), block)[a:]
        for h in range(H):
            g = h // (H // G)
            w = P.masked_softmax((qs[i][a:, h] @ ks[i][:, g].T) * scale, vis)
            ref = w @ vs[i][:, g]
            err = np.abs(got[cu[i]:cu[i + 1], h] - ref).max()
            assert err <= 2e-2, (variant, i, h, err)
            if "whole" in variant:                                 # only the output's own rounding is left
                assert np.all(np.abs(got[cu[i]:cu[i + 1], h] - ref) <= np.abs(ref) * 2.0 ** -8 + 1e-4), (i, h)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,E,top,d,ff,force_tc", [
    (1, 4, 2, 32, 16, False), (5, 6, 1, 64, 24, False), (70, 3, 2, 48, 40, False), (33, 8, 8, 40, 12, False),
    (200, 16, 3, 128, 64, False), (9, 5, 2, 36, 10, False),
    (300, 4, 2, 128, 64, True), (700, 3, 1, 200, 72, True), (40, 6, 2, 64, 136, True), (1000, 16, 4, 256, 192, True)])
def test_mixture_kernels_against_plain(n, E, top, d, ff, force_tc, dt):
    """The last cases run the grouped tcgen05 tiles in 16 bits (experts with more rows than a tile, with fewer, with
    none; widths and expert sizes that are no multiple of the tile), the others the mma.sync and CUDA-core tiles."""
    from kappai_b200.ops import kernels as K
    K.moe_set_tc_min_pairs(1 if force_tc else 1 << 40)
    rng = np.random.default_rng(n * E)
    h = bf16_round(rng.normal(0, 1, (n, d)))
    w = {"router": bf16_round(rng.normal(0, 3 / math.sqrt(d), (E, d))), "router.b": bf16_round(rng.normal(0, 0.5, E))}
    for e in range(E):
        w[f"e{e}.gate"] = bf16_round(rng.normal(0, 1 / math.sqrt(d), (ff, d)))
        w[f"e{e}.up"] = bf16_round(rng.normal(0, 1 / math.sqrt(d), (ff, d)))
        w[f"e{e}.down"] = bf16_round(rng.normal(0, 2 / math.sqrt(ff), (d, ff)))
    z = h @ w["router"].T + w["router.b"]
    want_idx, want_w = P.router(h, w["router"], w["router.b"], top)
    idx = torch.empty((n, top), dtype=torch.int32, device=DEV)
    wts = torch.empty((n, top), dtype=torch.float32, device=DEV)
    layout = torch.empty(K.moe_layout_ints(n, E, top), dtype=torch.int32, device=DEV)
    K.moe_route(dev(z), top, idx, wts, layout)
    assert np.array_equal(idx.cpu().numpy(), want_idx)
    assert np.abs(wts.cpu().numpy() - want_w).max() < 1e-5
    lay = layout.cpu().numpy()
    offsets, perm, inv = lay[:E + 1], lay[3 * (E + 1):3 * (E + 1) + n * top], lay[3 * (E + 1) + n * top:]
    assert offsets[E] == n * top and sorted(perm.tolist()) == list(range(n * top)) and np.array_equal(perm[inv], np.arange(n * top))
    assert all(want_idx.reshape(-1)[perm[p]] == e for e in range(E) for p in range(offsets[e], offsets[e + 1]))
    if K.moe_router_ok(d, E):                                                     # the same from the fused router
        idx2, wts2, layout2 = torch.empty_like(idx), torch.empty_like(wts), torch.empty_like(layout)
        K.moe_router(dev(h, dt), dev(w["router"]), dev(w["router.b"]), top, idx2, wts2, layout2)
        assert torch.equal(idx2, idx) and (wts2 - wts).abs().max().item() < 1e-5
        assert torch.equal(layout2[:3 * (E + 1)], layout[:3 * (E + 1)])
    base = rng.normal(0, 1, (n, d)).astype(np.float32)
    out = dev(base)
    w_gu = torch.stack([torch.cat([dev(w[f"e{e}.gate"], dt), dev(w[f"e{e}.up"], dt)], 0) for e in range(E)]).contiguous()
    w_dn = torch.stack([dev(w[f"e{e}.down"], dt) for e in range(E)]).contiguous()
    K.moe_experts(dev(h, dt), w_gu, w_dn, layout, wts, top, out, "silu")
    K.moe_set_tc_min_pairs(512)
    assert K.moe_tc_status() == 0
    want = base + P.mixture(h, w, E, top, "silu")
    err = np.abs(out.cpu().numpy() - want).max()
    assert err < (3e-5 if dt == torch.float32 else 4e-2), err


# ------------------------------------------------------------------------------------------ whole models

def _requests(plain, lengths, seed, min_margin=0.0):
    """Random requests.  With ``min_margin`` every router choice in them has at least that gap to the first
    logit left out, so that a 16-bit run (whose router inputs differ from the plain ones by a per cent or so) does
    not choose otherwise than the plain one: a request grows four tokens at a time, and four tokens that bring a
    closer call are drawn again (what a token's routers see depends on the tokens before it only)."""
    rng = np.random.default_rng(seed)
    reqs = {}
    for i, n in enumerate(lengths):
        toks = []
        while len(toks) < n:
            new = rng.integers(0, plain.cfg["vocab"], min(4, n - len(toks))).tolist()
            if min_margin:
                m = []
                plain.forward(toks + new, margins=m)
                if m and min(float(x[len(toks):].min()) for x in m) < min_margin:
                    continue
            toks += new
        reqs[f"r{i}"] = toks
    return reqs


LENGTHS = {"P": [70, 3, 121, 49], "Q": [90, 41, 2, 130], "R": [77, 20, 101], "S": [330, 64, 201, 129], "T": [200, 65, 140],
           "U": [40, 7, 25], "V": [420, 300, 60]}
PROMPTS = {"P": [30, 1, 60, 48], "Q": [50, 40, 1, 100], "R": [40, 19, 60], "S": [220, 3, 101, 128], "T": [150, 64, 30],
           "U": [20, 1, 24], "V": [400, 280, 30]}
BF16_REL_RMS = 0.03    # bound on a row's 16-bit error (rms over the vocabulary / the row's spread) for 95 % of the rows, twice
                       # that for all (measured: median 0.3 to 1.2 %, 95 % of rows below 2.2 %, worst row 3.9 %)
MARGIN = 0.12          # router logits here have a spread of about 3; 16-bit inputs move them by about 0.01


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", [("P", 16), ("Q", None), ("R", 32), ("S", None), ("T", None), ("U", 8), ("V", None)])
def test_every_cut_agrees_with_plain(name, page_size, dtype, tiz_dirs, tiz_plain, tmp_path):
    """Whole prompts, the last tokens decoded one by one (more of them than a block is long), portions down to
    two tokens, and up to four requests mixed in a pool so small that pages and slots go round."""
    plain = tiz_plain[name]
    reqs = _requests(plain, LENGTHS[name], 31, MARGIN if dtype == "bfloat16" else 1e-4)
    prompt_len = dict(zip(reqs, PROMPTS[name]))
    expected = {rid: plain.forward(t) for rid, t in reqs.items()}
    # (16-bit: these models' weights have unit gain, so that every sublayer moves the residual and its roundings
    # weigh twice what they do in models with small weights; the sharp comparison is the 32-bit one)
    tol = 1e-4 if dtype == "float32" else 2 * min(tol_for(dtype, e) for e in expected.values())
    page = page_size or 64
    max_tokens = max(-(-len(t) // page) * page for t in reqs.values()) + 2 * page
    tr = R.Trace()
    R.whole(tr, reqs)
    R.last_decoded(tr, reqs, n_last=110)
    R.portions(tr, reqs)
    b = len(tr.steps)
    R.mixed(tr, reqs, prompt_len, seed=5, max_live=4, page=page, max_tokens=max_tokens)
    assert max(len(s["entries"]) for s in tr.steps[b:]) >= 2
    out = R.run_trace(tiz_dirs[name], dtype, tr, str(tmp_path / "out"), max_tokens, page_size)
    if dtype == "bfloat16":
        # 16-bit: the error of a row as a root mean square over the vocabulary, in units of the row's spread; rounding
        # alone gives a few per cent (these weights have unit gain: every sublayer moves the residual), a wrong key,
        # page or expert gives tens
        rel = []
        for st, rows in zip(tr.steps, tr.rows):
            for j, (rid, pos) in enumerate(rows):
                e = expected[rid][pos]
                rel.append((float(np.sqrt(np.mean((out[st["step"]][j] - e) ** 2)) / e.std()), st["step"], rid, pos))
        r = np.array([x[0] for x in rel])
        print(f"{name} bfloat16: relative rms error median {np.median(r):.4f}, 95 % {np.quantile(r, 0.95):.4f}, worst {r.max():.4f}")
        assert np.quantile(r, 0.95) <= BF16_REL_RMS and r.max() <= 2 * BF16_REL_RMS, max(rel)
        worst = float(r.max())
    else:
        worst = R.compare(tr, out, expected, tol, f"{name}/{dtype}")
    stats = R.cache_stats(str(tmp_path / "out"))
    assert stats and all(g["reused"] > 0 and g["handed_out"] > g["pages"] for g in stats.values()), stats
    if dtype == "float32":
        for place, rows in R.rows_by_place(tr, out).items():
            assert len(rows) >= 2, place
            for r in rows[1:]:
                assert np.array_equal(rows[0], r), f"{name}: float32 logits of {place} differ between cuts"
    print(f"{name} {dtype}: worst |error| {worst:.3e} (tolerance {tol:.3e}), {len(tr.steps)} steps")


@pytest.mark.parametrize("name", ["P", "S"])
def test_residual_after_every_layer(name, tiz_dirs, tiz_plain):
    from kappai_b200 import ModelRunner, StepEntry
    plain = tiz_plain[name]
    toks = _requests(plain, [57], 8)["r0"]
    want = []
    plain.forward(toks, want)
    r = ModelRunner(tiz_dirs[name], dtype="float32", max_tokens=256, max_requests=2, cuda_graphs=False)
    got = []
    r.observer = lambda i, x: got.append(x.detach().cpu().numpy().copy())
    r.step([StepEntry("a", toks, [0])])
    assert len(got) == len(want) + 1
    for i, w in enumerate(want):
        assert np.abs(got[i + 1] - w).max() < 3e-5, (i, np.abs(got[i + 1] - w).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_batched_requests_equal_each_alone_and_captured_steps_equal_eager(dtype, tiz_dirs, tiz_plain):
    """Unequal requests decode together for many steps (the steps are captured into CUDA graphs on the way); every
    row equals the row of the request run alone without graphs."""
    from kappai_b200 import ModelRunner, StepEntry
    plain = tiz_plain["P"]
    n_dec = 40
    reqs = _requests(plain, [61 + n_dec, 9 + n_dec, 30 + n_dec], 12, MARGIN)

    def run(runner, group):
        out = {rid: [] for rid in group}
        lg = runner.step([StepEntry(rid, reqs[rid][:len(reqs[rid]) - n_dec], [len(reqs[rid]) - n_dec - 1]) for rid in group])
        for j, rid in enumerate(group):
            out[rid].append(lg[j].cpu().numpy().copy())
        for s in range(n_dec):
            lg = runner.step([StepEntry(rid, [reqs[rid][len(reqs[rid]) - n_dec + s]], [0]) for rid in group])
            for j, rid in enumerate(group):
                out[rid].append(lg[j].cpu().numpy().copy())
        for rid in group:
            runner.end(rid)
        return out

    together = run(ModelRunner(tiz_dirs["P"], dtype=dtype, max_tokens=512, max_requests=4, page_size=16), list(reqs))
    alone_runner = ModelRunner(tiz_dirs["P"], dtype=dtype, max_tokens=512, max_requests=4, page_size=16, cuda_graphs=False)
    for rid in reqs:
        alone = run(alone_runner, [rid])[rid]
        for a, b in zip(alone, together[rid]):
            if dtype == "float32":
                assert np.array_equal(a, b)
            else:
                assert np.abs(a - b).max() <= 2 * tol_for(dtype, a)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_engine(name, dtype, tiz_dirs, tiz_plain):
    from kappai_b200 import Engine, EngineArgs, SamplingParams
    plain = tiz_plain[name]
    prompts = list(_requests(plain, [5, 26, 60], 21).values())
    n_new = 50
    eng = Engine(EngineArgs(model=tiz_dirs[name], dtype=dtype, max_batch=4, max_step_tokens=16, page_size=16, kv_tokens=1024))
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, n_predict=n_new))
    assert [len(o) for o in outs] == [n_new] * len(prompts)
    for p, o in zip(prompts, outs):
        m = []
        lg = plain.forward(p + o, margins=m)[len(p) - 1:-1]
        if dtype == "bfloat16" and m and min(float(x.min()) for x in m) < MARGIN:
            continue                                                  # a router choice too close for 16 bits to call
        for j, t in enumerate(o):
            best = int(np.argmax(lg[j]))
            assert t == best or lg[j][best] - lg[j][t] <= 4 * tol_for(dtype, lg[j]), (j, t, best)
    assert eng.runner.cache.slots.n_free == 4 and all(p.n_free == p.n_pages for p in eng.runner.cache.pools.values())


def test_command_line_and_random_weights(tiz_dirs, tiz_plain, tmp_path):
    """The command line runs the design like any other: greedy tokens equal the plain model's, --time names the
    design's kernels, and --random-weights writes a loadable model folder from a Tizusun config.json."""
    import json
    import os
    import subprocess
    import sys
    plain = tiz_plain["P"]
    prompt = _requests(plain, [30], 77)["r0"]
    cmd = [sys.executable, "-m", "kappai_b200.cli", "-m", tiz_dirs["P"], "-p", ",".join(map(str, prompt)), "-n", "12", "-t", "0",
           "--fp32", "--time"]
    p = subprocess.run(cmd, cwd=R.ROOT, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    out = [int(t) for t in p.stdout.split()]
    assert len(out) == 12
    lg = plain.forward(prompt + out)[len(prompt) - 1:-1]
    for j, t in enumerate(out):
        best = int(np.argmax(lg[j]))
        assert t == best or lg[j][best] - lg[j][t] <= 1e-4, (j, t, best)
    for name in ("postnorm_rows", "moe_router", "moe_experts", "sigmoid_gate", "attention_split"):
        assert name in p.stderr, (name, p.stderr[-3000:])
    cfgp = tmp_path / "c.json"
    cfgp.write_text(json.dumps(CONFIGS["Q"][0]))
    made = tmp_path / "rw"
    cmd = [os.path.join(R.ROOT, "bin", "kappai-cli"), "--random-weights", str(cfgp), "-s", "5", "-m", str(made), "-t", "0", "-n", "5",
           "1 2 3"]
    p = subprocess.run(cmd, cwd=str(tmp_path), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert len(p.stdout.split()) == 5 and os.path.isfile(made / "model.safetensors")
