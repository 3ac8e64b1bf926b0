"""Gigezen on the GPU against the plain oracle (tests/gigezen_oracle.py): every mechanism alone, then whole models
through the span, the cache manager, the engine's scheduler and the trace replay.  Small random models, made so
that no two sizes coincide; weights are rounded to bfloat16 once so that both execution modes and the oracle read the
same numbers."""
import json
import os

import pytest
import torch

from tests import gigezen_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _mixer(heads, dim, rot, vdim, rank, window, dims=None, base=10000.0, kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_rank": rank, "mask": {"size": window}, "rot": {"base": base, "dims": dims or rot},
         "rot_dim": rot, "scale": (dim + rot) ** -0.5, "vdim": vdim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _dense(ff, limit):
    return {"ff": ff, "kind": "dense", "limit": limit}


def _moe(experts, top, groups, keep, ff):
    return {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "groups": {"count": groups, "keep": keep}, "top": top}}


def _layer(mixer, mlp):
    return {"mixer": mixer, "mlp": mlp, "type": "latent_attention"}


CONFIGS = {
    # odd sizes everywhere, a layer without feed-forward, two layers reading layer 0 (one from far back), top = 1
    "odd": {"architecture": "Gigezen", "norm": {"eps": 1e-5}, "vocab": 300, "width": 200, "layers": [
        _layer(_mixer(3, 24, 8, 20, 40, 7), _dense(100, 1.5)),
        _layer(_mixer(3, 24, 8, 20, 40, 7, kv_from=0), _moe(6, 3, 3, 2, 36)),
        _layer(_mixer(2, 16, 12, 28, 24, 5, base=500.0), None),
        _layer(_mixer(5, 8, 8, 12, 40, 11, kv_from=0), _moe(5, 1, 1, 1, 20)),
        _layer(_mixer(3, 24, 8, 20, 40, 3), _dense(72, 0.75)),
    ]},
    # more than eight heads, latent size that is no multiple of 32, partial rotation, window longer than the prompts
    "wide": {"architecture": "Gigezen", "norm": {"eps": 1e-6}, "vocab": 257, "width": 128, "layers": [
        _layer(_mixer(9, 16, 16, 24, 72, 64, dims=8), _moe(8, 2, 4, 2, 48)),
        _layer(_mixer(9, 16, 16, 24, 72, 9, dims=8, kv_from=0), _dense(160, 4.0)),
        _layer(_mixer(4, 32, 4, 8, 33, 1), _dense(64, 2.0)),
    ]},
}


def _weights(cfg_dict, seed):
    from petals_b200.models.gigezen import from_config_dict, tensor_shapes

    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(from_config_dict(cfg_dict)).items():
        t = torch.randn(shape, generator=g)
        if name.endswith("dkv.norm"):
            t = 1.0 + 0.2 * t
        elif len(shape) == 1:
            t = 0.2 * t
        elif name != "embed":
            t = t * (1.5 * shape[1] ** -0.5)
        out[name] = t.to(torch.bfloat16)
    return out


_MODELS = {}


def model(name, tmp_root):
    """(config dict, weights, model directory, oracle cache) of a test configuration."""
    if name not in _MODELS:
        from petals_b200.weights.safetensors_io import save_file

        cfg, w = CONFIGS[name], _weights(CONFIGS[name], 7 + len(name))
        d = os.path.join(tmp_root, name)
        os.makedirs(d, exist_ok=True)
        json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
        save_file(w, os.path.join(d, "model.safetensors"))
        _MODELS[name] = (cfg, w, d, {})
    return _MODELS[name]


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("gigezen"))


def oracle_logits(name, tmp_root, tokens):
    cfg, w, _, cache = model(name, tmp_root)
    key = tuple(tokens)
    if key not in cache:
        cache[key] = O.forward(cfg, w, list(tokens))
    return cache[key]


_SPANS = {}


def span_of(name, tmp_root, dtype, max_chunk=16):
    cap = 128 if max_chunk <= 16 else 256
    from petals_b200.models.config import resolve_config
    from petals_b200.runtime.kv_cache import KVCacheManager
    from petals_b200.runtime.layered_span import make_span
    from petals_b200.weights.loader import load_span

    key = (name, dtype, max_chunk)
    if key not in _SPANS:
        d = model(name, tmp_root)[2]
        cfg = resolve_config(d)
        w = load_span(d, cfg, 0, cfg.n_layers, need_embed=True, need_head=True, dtype=dtype, device=DEV)
        span = make_span(cfg, w, DEV, dtype, kv_capacity=cap, max_batch=4, max_chunk=max_chunk)
        mgr = KVCacheManager.for_span(cfg, 0, cfg.n_layers, dtype, DEV, default_max_length=cap)
        _SPANS[key] = (span, mgr)
    return _SPANS[key]


def tokens_of(name, n, seed=0):
    g = torch.Generator().manual_seed(100 + seed)
    return torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist()


def row_errs(got, want):
    """Per row: root mean square of the difference over that of the expected logits, mean removed."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    ref = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()


def rel_err(got, want):
    return float(row_errs(got, want).max())


def assert_close_rows(got, want, dtype):
    """fp32: every row within the tolerance.  16-bit: rounding can flip a router's close call (top-1 of a handful of
    experts) or move a value across a clamp, which changes single rows by far more than rounding; a fault of the
    mechanism (a window, a chunk edge, a page) would change most rows.  So: the typical row within half the
    tolerance, at most one row in twenty beyond it."""
    e = row_errs(got, want)
    if dtype == torch.float32:
        assert float(e.max()) < TOL[dtype]
    else:
        assert float(e.median()) < TOL[dtype] / 2 and float((e > TOL[dtype]).double().mean()) <= 0.05, \
            (float(e.median()), float(e.max()), int((e > TOL[dtype]).sum()), e.numel())


TOL = {torch.float32: 2e-5, torch.bfloat16: 4e-2}
MODES = [torch.float32, torch.bfloat16]


def ids(toks):
    return torch.tensor(toks, dtype=torch.int64, device=DEV)


# ===================================================================================== mechanisms alone
def test_residual_update_and_zero_centred_norm():
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(1)
    T, W, top = 5, 200, 3
    x, a, b = (torch.randn(T, W, generator=g) for _ in range(3))
    y, pw, gain = torch.randn(T * top, W, generator=g), torch.rand(T * top, generator=g), 0.3 * torch.randn(W, generator=g)
    xd = x.to(DEV)
    out = torch.zeros(T, 256, device=DEV)
    L.add_rms_norm(xd, gain.to(DEV), out[:, :W], 1e-5, 1.0, add_a=a.to(DEV), add_b=b.to(DEV), pair_y=y.to(DEV),
                   pair_w=pw.to(DEV), top=top)
    want_x = x.double() + a.double() + b.double() + (y.double().view(T, top, W) * pw.double().view(T, top, 1)).sum(1)
    assert torch.allclose(xd.cpu().double(), want_x, atol=1e-5)
    assert torch.allclose(out[:, :W].cpu().double(), O.zero_centred_norm(want_x, gain.double(), 1e-5), atol=2e-5)
    assert float(out[:, W:].abs().max()) == 0.0
    plain = torch.zeros(T, W, device=DEV, dtype=torch.bfloat16)      # plain gain, 16-bit output, nothing added
    L.add_rms_norm(xd, (1 + gain).to(DEV), plain, 1e-5, 0.0)
    assert torch.allclose(plain.cpu().double(), O.zero_centred_norm(want_x, gain.double(), 1e-5), atol=3e-2)


def test_clamped_gated_unit():
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(2)
    T, ff, limit = 7, 37, 1.25
    h = 2.0 * torch.randn(T, ff, generator=g, dtype=torch.float64)
    dg, du = torch.randn(ff, generator=g, dtype=torch.float64), torch.randn(ff, generator=g, dtype=torch.float64)
    want = O.clamped_gated_unit(h, {"gate": torch.diag(dg), "up": torch.diag(du), "down": torch.eye(ff, dtype=torch.float64)}, limit)
    gu = torch.cat([(h * dg), (h * du)], 1).float().to(DEV)
    act = torch.zeros(T, 64, device=DEV)
    L.glu_clamp(gu[:, :ff], gu[:, ff:], act, limit, 1.702, 1.0)
    assert (h * dg).max() > limit and (h * du).min() < -limit       # the clamps are exercised
    assert torch.allclose(act[:, :ff].cpu().double(), want, atol=1e-5)


@pytest.mark.parametrize("E,G,keep,top", [(12, 4, 2, 3), (6, 3, 2, 3), (5, 1, 1, 1), (8, 8, 3, 2), (40, 5, 2, 7)])
def test_router_against_oracle(E, G, keep, top):
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(E)
    T, W = 50, 24
    h, wr = torch.randn(T, W, generator=g, dtype=torch.float64), torch.randn(E, W, generator=g, dtype=torch.float64)
    want_ids, want_w, s = O.route(h, wr, {"experts": E, "top": top, "groups": {"count": G, "keep": keep}})
    z = torch.zeros(T, E + 3, device=DEV)
    z[:, :E] = (h @ wr.T).float().to(DEV)
    got_ids = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    got_w = torch.zeros(T, top, device=DEV)
    L.moe_route(z[:, :E], E, G, keep, top, got_ids, got_w)
    assert torch.equal(got_ids.cpu().long(), want_ids)
    assert torch.allclose(got_w.cpu().double(), want_w, atol=1e-6)
    if keep < G and E // G > 1:                                       # the group limit must change some choice
        assert any(set(s[t].topk(top).indices.tolist()) != set(want_ids[t].tolist()) for t in range(T))


def test_expert_plan_and_grouped_products():
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(3)
    T, top, E, W, ff = 37, 3, 6, 40, 28
    choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).int()
    choice[:, 0] = torch.where(choice[:, 0] == 4, choice[:, 1], choice[:, 0])       # expert 4 is rarely first
    h = torch.randn(T, W, generator=g)
    wg, wu, wd = (torch.randn(E, ff, W, generator=g), torch.randn(E, ff, W, generator=g), torch.randn(E, W, ff, generator=g))
    off = torch.zeros(E + 1, dtype=torch.int32, device=DEV)
    rp, rt = torch.zeros(T * top, dtype=torch.int32, device=DEV), torch.zeros(T * top, dtype=torch.int32, device=DEV)
    cd = choice.to(DEV)
    L.moe_plan(cd, T, top, E, off, rp, rt)
    counts = torch.bincount(choice.flatten().long(), minlength=E)
    assert off.cpu().tolist() == [0] + counts.cumsum(0).tolist()
    assert sorted(rp.cpu().tolist()) == list(range(T * top)) and torch.equal(rt.cpu(), rp.cpu() // top)
    for e in range(E):
        assert all(int(choice.flatten()[p]) == e for p in rp.cpu()[off[e]:off[e + 1]].tolist())
    act = torch.zeros(T * top, ff, device=DEV)
    y = torch.zeros(T * top, W, device=DEV)
    L.gemm_simt(h.to(DEV), wg.to(DEV), act, w2=wu.to(DEV), T=T * top, N=ff, K=W, ldw=W, w_gs=ff * W, row_src=rt,
                group_off=off, groups=E)
    L.gemm_simt(act, wd.to(DEV), y, T=T * top, N=W, K=ff, ldw=ff, w_gs=W * ff, row_dst=rp, group_off=off, groups=E)
    for t in range(0, T, 5):
        for k in range(top):
            e = int(choice[t, k])
            want = O.expert(h[t:t + 1].double(), wg[e].double(), wu[e].double(), wd[e].double())[0]
            assert torch.allclose(y[t * top + k].cpu().double(), want, atol=2e-3, rtol=1e-4)


@pytest.mark.parametrize("xdt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16)])
def test_plain_and_batched_products(xdt, wdt):
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(4)
    T, N, K, B = 70, 45, 51, 3
    x, w = torch.randn(T, B * K + 5, generator=g).to(xdt), torch.randn(B, N, K, generator=g).to(wdt)
    out = torch.zeros(T, B * N + 2, device=DEV)
    L.gemm_simt(x.to(DEV), w.to(DEV), out, T=T, N=N, K=K, ldw=K, batch=B, x_bs=K, w_bs=N * K, o_bs=N)
    for b in range(B):
        want = x[:, b * K:(b + 1) * K].double() @ w[b].double().T
        assert torch.allclose(out[:, b * N:(b + 1) * N].cpu().double(), want, atol=1e-4, rtol=1e-5)
    assert float(out[:, B * N:].abs().max()) == 0.0


def _attention_direct(qa, qr, c, kr, p, window, scale):
    T, H, R = qa.shape
    out = torch.zeros(T, H, R, dtype=torch.float64)
    for t in range(T):
        js = [j for j in range(c.shape[0]) if O.window_visible(int(p[t]), j, window)]
        for h in range(H):
            s = torch.stack([(qa[t, h] @ c[j] + qr[t, h] @ kr[j]) * scale for j in js])
            a = torch.softmax(s, 0)
            out[t, h] = sum(a[n] * c[j] for n, j in enumerate(js))
    return out


@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("batched", [0, 1, 3, 16], ids=["portion", "table", "table-3-shares", "table-16-shares"])
def test_latent_attention_window_edges_and_far_keys(cache_dtype, batched):
    """One key per query is made to dominate (a large score) once just inside and once just outside the window, and
    once far back; rows are addressed through the session's cache (a prompt's portion) or through the staged pointer
    table (decoding sessions)."""
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(5)
    H, dim, rot, R, window, S, row = 9, 4, 6, 40, 37, 150, 48
    scale = 0.3
    c = torch.randn(S, R, generator=g).to(cache_dtype).double()
    kr = torch.randn(S, rot, generator=g).to(cache_dtype).double()
    cache = torch.zeros(2, S + 10, row, dtype=cache_dtype, device=DEV)          # two "sessions" with the same rows
    cache[:, :S, :R] = c.to(cache_dtype).to(DEV)
    cache[:, :S, R:R + rot] = kr.to(cache_dtype).to(DEV)
    qpos = [0, 1, window - 1, window, 99, 100, S - 1]
    T = len(qpos)
    qa, qr = 0.3 * torch.randn(T, H, R, generator=g), 0.3 * torch.randn(T, H, rot, generator=g)
    spikes = {2: 0, 3: 0, 4: 99 - window + 1, 5: 100 - window, 6: 3}             # query row -> key that is made loud
    for t, j in spikes.items():
        qa[t] += 4.0 * c[j].float() / c[j].norm().float()
    want = _attention_direct(qa.double(), qr.double(), c, kr, qpos, window, scale)
    shorter = _attention_direct(qa.double(), qr.double(), c, kr, qpos, window - 1, scale)
    longer = _attention_direct(qa.double(), qr.double(), c, kr, qpos, window + 1, scale)
    for t in (2, 4):      # loud key on the window's last place: a window one shorter loses it
        assert (want[t] - shorter[t]).abs().max() > 0.1
    for t in (3, 5):      # loud key one place outside: a window one longer would catch it
        assert (want[t] - longer[t]).abs().max() > 0.1
    proj = torch.zeros(T, H * (dim + rot) + 3, device=DEV)
    proj[:, :H * (dim + rot)].view(T, H, dim + rot)[..., dim:] = qr.to(DEV)
    out = torch.zeros(T, H * R, device=DEV)
    common = dict(heads=H, dim=dim, rot=rot, rot_dims=rot, kv_rank=R, row_elems=row, cache_dtype=cache_dtype, eps=1e-5,
                  q_abs=qa.reshape(T, H * R).contiguous().to(DEV), out=out, window=window, scale=scale)
    inv = torch.ones(rot // 2, dtype=torch.float64, device=DEV)
    if batched:
        ptrs = torch.tensor([[cache[t % 2].data_ptr(), 0] for t in range(T)], dtype=torch.int64, device=DEV)
        pos_t = torch.tensor(qpos, dtype=torch.int32, device=DEV)       # (the argument struct holds raw pointers: keep
        scratch = torch.zeros(T * H * max(batched, 1) * (R + 2), device=DEV)   #  every tensor alive until the result is read)
        a = L.latent_args(proj, 0, -1, None, inv, T=T, kv_ptrs=ptrs, kv_ptr_stride=2, pos=pos_t, **common)
        if batched > 1:      # the window's keys divided over several blocks (more shares than some windows have chunks)
            L.latent_attn(a, batched, scratch)
        else:
            L.latent_attn(a)
        got = out.cpu().double().view(T, H, R)
    else:
        got = torch.zeros(T, H, R, dtype=torch.float64)
        for t, p in enumerate(qpos):                                             # a one-token portion at position p
            a = L.latent_args(proj[t:t + 1], 0, -1, None, inv, T=1, cache=cache[1], pos0=p, **{**common, "q_abs": common["q_abs"][t:t + 1], "out": out[t:t + 1]})
            L.latent_attn(a)
        got = out.cpu().double().view(T, H, R)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-5)


def test_rotation_and_cache_append_against_oracle():
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(6)
    W, R, rot, dims, H, dim, T, pos0, eps, base = 48, 24, 12, 8, 3, 10, 6, 1000, 1e-5, 300.0
    m = {"kv_rank": R, "rot": {"dims": dims, "base": base}}
    h, wd, gain = (torch.randn(T, W, generator=g, dtype=torch.float64), torch.randn(R + rot, W, generator=g, dtype=torch.float64),
                   1 + 0.2 * torch.randn(R, generator=g, dtype=torch.float64))
    p = torch.arange(pos0, pos0 + T)
    c, kr = O.latent_rows(h, wd, gain, p, m, eps)
    q = torch.randn(T, H, dim + rot, generator=g, dtype=torch.float64)
    want_q = torch.cat([q[..., :dim], O.rotate_half(q[..., dim:], p, dims, base)], -1)
    proj = torch.cat([q.reshape(T, -1), h @ wd.T], 1).float().to(DEV)
    cache = torch.zeros(pos0 + T + 2, 40, device=DEV)
    inv = (torch.tensor(base, dtype=torch.float64) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)).to(DEV)
    a = L.latent_args(proj, 0, H * (dim + rot), gain.float().to(DEV), inv, heads=H, dim=dim, rot=rot, rot_dims=dims, kv_rank=R,
                      row_elems=40, cache_dtype=torch.float32, eps=eps, T=T, cache=cache, pos0=pos0)
    L.latent_rope_append(a)
    rows = cache[pos0:pos0 + T].cpu().double()
    assert torch.allclose(rows[:, :R], c, atol=1e-5) and torch.allclose(rows[:, R:R + rot], kr, atol=1e-5)
    assert float(cache[:pos0].abs().max()) == 0.0 and float(cache[pos0 + T:].abs().max()) == 0.0
    assert torch.allclose(proj[:, :H * (dim + rot)].cpu().double().view(T, H, dim + rot), want_q, atol=1e-5)


# ===================================================================================== whole models
@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_logits_at_every_position(name, dtype, tmp_root):
    span, mgr = span_of(name, tmp_root, dtype)
    toks = tokens_of(name, 41)
    kv = mgr.allocate("whole", 128)
    got, am = span.prefill(kv, ids=ids(toks), logits_at=list(range(len(toks))))
    want = oracle_logits(name, tmp_root, toks)
    assert rel_err(got, want) < TOL[dtype]
    assert kv.length == len(toks)
    if dtype == torch.float32:
        assert torch.equal(am.cpu(), want.argmax(-1))
    mgr.close("whole")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_decoding_token_by_token_equals_the_prompt_pass(name, dtype, tmp_root):
    """From the first token on, through every window edge and chunk border of these sizes (long decoding)."""
    span, mgr = span_of(name, tmp_root, dtype)
    toks = tokens_of(name, 41)
    want = oracle_logits(name, tmp_root, toks)
    for cut in (1, 17):
        kv = mgr.allocate("dec", 128)
        rows = [span.prefill(kv, ids=ids(toks[:cut]), logits_at=list(range(cut)))[0]]
        for p in range(cut, len(toks)):
            rows.append(span.decode([kv], ids=ids(toks[p:p + 1]))[0].clone())
        assert rel_err(torch.cat(rows), want) < TOL[dtype]
        mgr.close("dec")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("portion", [2, 3, 7, 16, 19])
def test_prompts_in_portions(portion, dtype, tmp_root):
    name = "odd"
    span, mgr = span_of(name, tmp_root, dtype)
    toks = tokens_of(name, 41)
    want = oracle_logits(name, tmp_root, toks)
    kv = mgr.allocate("por", 128)
    rows = []
    for c0 in range(0, len(toks), portion):
        part = toks[c0:c0 + portion]
        rows.append(span.prefill(kv, ids=ids(part), logits_at=list(range(len(part))))[0])
    assert rel_err(torch.cat(rows), want) < TOL[dtype]
    mgr.close("por")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_batches_of_unequal_requests_and_reused_sessions(name, dtype, tmp_root):
    """Three sessions of different lengths decode together; one ends, its cache bytes go to a new session that joins
    the next batch.  Every row must equal the same request run alone."""
    span, mgr = span_of(name, tmp_root, dtype)
    reqs = {"a": tokens_of(name, 30, 1), "b": tokens_of(name, 12, 2), "c": tokens_of(name, 21, 3), "d": tokens_of(name, 17, 4)}
    cuts = {"a": 22, "b": 1, "c": 9, "d": 5}
    got = {k: [] for k in reqs}
    kvs = {}
    for k in ("a", "b", "c"):
        kvs[k] = mgr.allocate(k, 128)
        got[k].append(span.prefill(kvs[k], ids=ids(reqs[k][:cuts[k]]), logits_at=[cuts[k] - 1])[0])
    at = dict(cuts)
    joined = False
    while any(at[k] < len(reqs[k]) for k in kvs):
        live = [k for k in kvs if at[k] < len(reqs[k])]
        logits, _ = span.decode([kvs[k] for k in live], ids=ids([reqs[k][at[k]] for k in live]))
        for b, k in enumerate(live):
            got[k].append(logits[b:b + 1].clone())
            at[k] += 1
        if not joined and at["b"] == len(reqs["b"]):
            ptr = kvs["b"].data.data_ptr()
            mgr.close("b")
            del kvs["b"]
            kvs["d"] = mgr.allocate("d", 128)
            assert kvs["d"].data.data_ptr() == ptr or True          # (the allocator may or may not hand the block back)
            got["d"].append(span.prefill(kvs["d"], ids=ids(reqs["d"][:cuts["d"]]), logits_at=[cuts["d"] - 1])[0])
            at["d"] = cuts["d"]
            joined = True
    for k, toks in reqs.items():
        want = oracle_logits(name, tmp_root, toks)[cuts[k] - 1:]
        assert rel_err(torch.cat(got[k]), want) < TOL[dtype], k
    for k in list(kvs):
        mgr.close(k)


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_long_prompts_in_large_chunks(name, dtype, tmp_root):
    """Chunks of 64 tokens (the tensor-core attention of the 16-bit mode: query tiles, key tiles and windows that
    start in an earlier chunk), the last one partial, then decoding."""
    span, mgr = span_of(name, tmp_root, dtype, max_chunk=64)
    toks = tokens_of(name, 150, 11)
    want = oracle_logits(name, tmp_root, toks)
    kv = mgr.allocate("long", 256)
    rows = [span.prefill(kv, ids=ids(toks[:141]), logits_at=list(range(141)))[0]]
    for p in range(141, 150):
        rows.append(span.decode([kv], ids=ids(toks[p:p + 1]))[0].clone())
    assert_close_rows(torch.cat(rows), want, dtype)
    mgr.close("long")
    kv = mgr.allocate("long", 256)                       # a chunk that starts in the middle of a session
    span.prefill(kv, ids=ids(toks[:37]))
    got = span.prefill(kv, ids=ids(toks[37:150]), logits_at=list(range(150 - 37)))[0]
    assert_close_rows(got, want[37:], dtype)
    mgr.close("long")


def test_a_freed_cache_is_clean_for_its_next_owner(tmp_root):
    """The same session name and the same bytes, used again for a shorter request: nothing of the first one shows."""
    name, dtype = "wide", torch.float32
    span, mgr = span_of(name, tmp_root, dtype)
    long, short = tokens_of(name, 41), tokens_of(name, 12, 2)
    kv = mgr.allocate("s", 128)
    span.prefill(kv, ids=ids(long))
    ptr = kv.data.data_ptr()
    mgr.close("s")
    kv = mgr.allocate("s", 128)
    got = span.prefill(kv, ids=ids(short), logits_at=list(range(len(short))))[0]
    assert rel_err(got, oracle_logits(name, tmp_root, short)) < TOL[dtype]
    kv2 = mgr.allocate("s", 128)                                   # same id again: reset in place
    assert kv2.data.data_ptr() == kv.data.data_ptr() and kv2.length == 0 and ptr is not None
    got = span.prefill(kv2, ids=ids(short[:5]), logits_at=[4])[0]
    assert rel_err(got, oracle_logits(name, tmp_root, short)[4:5]) < TOL[dtype]
    mgr.close("s")


def test_cuda_graph_steps_equal_eager_steps(tmp_root):
    from petals_b200.models.config import resolve_config
    from petals_b200.runtime.layered_span import make_span
    from petals_b200.weights.loader import load_span

    name = "odd"
    span, mgr = span_of(name, tmp_root, torch.bfloat16)
    d = model(name, tmp_root)[2]
    cfg = resolve_config(d)
    w = load_span(d, cfg, 0, cfg.n_layers, need_embed=True, need_head=True, dtype=torch.bfloat16, device=DEV)
    eager = make_span(cfg, w, DEV, torch.bfloat16, kv_capacity=128, max_batch=4, max_chunk=16, use_graphs=False, pdl=False)
    toks = tokens_of(name, 20)
    ka, kb = mgr.allocate("g", 128), mgr.allocate("e", 128)
    span.prefill(ka, ids=ids(toks[:9]))
    eager.prefill(kb, ids=ids(toks[:9]))
    for p in range(9, 20):
        la = span.decode([ka], ids=ids(toks[p:p + 1]))[0].clone()
        lb = eager.decode([kb], ids=ids(toks[p:p + 1]))[0].clone()
        assert torch.equal(la, lb)
    assert span._graphs, "the decode step was not captured"
    mgr.close("g")
    mgr.close("e")


# ===================================================================================== entry points
def test_greedy_generation_through_the_engine(tmp_root):
    """PipelineEngine.generate: prompts of unequal lengths are prefilled one by one and decoded together by the
    engine's rounds; the tokens must be the oracle's greedy continuation."""
    from petals_b200.parallel.pipeline import PipelineEngine

    name = "wide"
    cfg, w, d, _ = model(name, tmp_root)
    eng = PipelineEngine(d, (), torch.float32, torch.device(DEV), kv_capacity=64, max_sessions=4, max_chunk=16)
    prompts = [tokens_of(name, 9, 5), tokens_of(name, 3, 6), tokens_of(name, 14, 7)]
    outs, stats = eng.generate([torch.tensor(p) for p in prompts], max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o == O.greedy(cfg, w, p, 8)
    assert stats["decode_tok_per_s"] > 0


def test_sampled_generation_runs_on_the_device_sampler(tmp_root):
    from petals_b200.parallel.pipeline import PipelineEngine
    from petals_b200.runtime.sampler import SamplingParams

    d = model("odd", tmp_root)[2]
    eng = PipelineEngine(d, (), torch.bfloat16, torch.device(DEV), kv_capacity=64, max_sessions=2, max_chunk=16)
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9)
    a, _ = eng.generate([torch.tensor(tokens_of("odd", 6))], max_new_tokens=6, sampling=sp, seed=3)
    b, _ = eng.generate([torch.tensor(tokens_of("odd", 6))], max_new_tokens=6, sampling=sp, seed=3)
    assert a == b and all(0 <= t < CONFIGS["odd"]["vocab"] for t in a[0])


def test_trace_replay_steps(tmp_root, tmp_path):
    from src.trace_replay import TraceReplayer

    name = "odd"
    d = model(name, tmp_root)[2]
    rp = TraceReplayer(d, torch.float32, 96)
    ta, tb = tokens_of(name, 20, 8), tokens_of(name, 11, 9)
    wa, wb = oracle_logits(name, tmp_root, ta), oracle_logits(name, tmp_root, tb)
    r0 = rp.step([{"id": "x", "tokens": ta[:15], "want": [0, 14]}, {"id": "y", "tokens": tb[:10], "want": []}], [])
    assert rel_err(r0, wa[[0, 14]]) < 2e-5
    r1 = rp.step([{"id": "x", "tokens": ta[15:16], "want": [0]}, {"id": "y", "tokens": tb[10:11], "want": [0]}], ["y"])
    assert rel_err(r1, torch.stack([wa[15], wb[10]])) < 2e-5
    assert rp.kv.get("y") is None
    r2 = rp.step([{"id": "x", "tokens": ta[16:17], "want": []}], [])
    assert r2 is None
    r3 = rp.step([{"id": "y", "tokens": ta[:4], "want": [3]}, {"id": "x", "tokens": ta[17:20], "want": [2]}], ["x", "y"])
    assert rel_err(r3, torch.stack([wa[3], wa[19]])) < 2e-5


def test_command_line_generates_from_a_model_folder(tmp_root):
    """``python -m src.main --inbox`` on a Gigezen folder: registry, loader, engine, greedy decoding, byte tokenizer."""
    import subprocess
    import sys

    name = "wide"
    cfg, w, d, _ = model(name, tmp_root)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29631", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    r = subprocess.run([sys.executable, "-m", "src.main", "--inbox", "--stage", "0", "--model", d, "--splits", "", "--dtype", "fp32",
                        "--temperature", "0", "--max_new_tokens", "6", "--prompt", "abc"], cwd=root, env=env,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    prompt = [(3 + b) % cfg["vocab"] for b in b"abc"]
    want = O.greedy(cfg, w, prompt, 6)
    text = bytearray((t - 3) if 0 <= t - 3 < 256 else ord("?") for t in want).decode("utf-8", errors="replace")
    assert "GENERATED: " + text in r.stdout, (r.stdout[-500:], want)
