"""Seledra on the GPU against the plain oracle (tests/seledra_oracle.py): every mechanism alone, then whole models
through the span, the cache manager, the engine's scheduler and the trace replay.  Small random models whose sizes do
not coincide (group sizes 1, 2, 3 and 5, one to five taps, value sizes below and above the key size, layers with and
without value mixing or feed-forward, a recurrent layer in front); weights are rounded to bfloat16 once so that both
execution modes and the oracle read the same numbers."""
import json
import os

import pytest
import torch

from tests import seledra_oracle as O

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F64 = torch.float64


def _attn(heads, kv, dim, vdim, scale, v_mix, ff=None):
    return {"type": "attention", "mixer": {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale, "v_mix": v_mix, "vdim": vdim},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


def _delta(heads, kv, dim, vdim, conv, ff=None):
    return {"type": "delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim},
            "mlp": None if ff is None else {"ff": ff, "kind": "dense"}}


CONFIGS = {
    # a recurrent layer in front, three value-mixing layers around one that does not mix, one tap, groups of 1, 2, 3 and 5
    "mixed": {"architecture": "Seledra", "max_positions": 300, "norm": {"eps": 1e-5}, "residual_mult": 0.45, "vocab": 210,
              "width": 136, "layers": [
                  _delta(4, 2, 24, 40, 3, ff=100),
                  _attn(6, 2, 24, 20, 0.2, True),
                  _attn(2, 2, 40, 20, 0.15, True, ff=72),
                  _attn(5, 1, 16, 36, 0.25, False),
                  _delta(3, 3, 20, 12, 1, ff=64),
                  _attn(4, 2, 8, 20, 0.35, True)]},
    # no value mixing at all but one lone mixing layer, a state wider than one block's columns, five taps, plain residual sum
    "plain": {"architecture": "Seledra", "max_positions": 260, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "vocab": 257,
              "width": 128, "layers": [
                  _attn(9, 3, 32, 64, 0.18, False, ff=192),
                  _delta(2, 1, 72, 136, 5),
                  _attn(1, 1, 128, 16, 0.09, True, ff=50)]},
}


# one kind of mixer only, sizes that are multiples of nothing (the kernels' scalar paths), width that is no multiple of 8
EXTRA_CONFIGS = {
    "recurrent-only": {"architecture": "Seledra", "max_positions": 80, "norm": {"eps": 1e-5}, "residual_mult": 0.7, "vocab": 150,
                       "width": 100, "layers": [_delta(3, 1, 18, 22, 2, ff=36), _delta(2, 2, 10, 6, 7)]},
    "attention-only": {"architecture": "Seledra", "max_positions": 80, "norm": {"eps": 1e-5}, "residual_mult": 0.7, "vocab": 150,
                       "width": 100, "layers": [_attn(3, 1, 20, 12, 0.2, True), _attn(2, 1, 6, 12, 0.4, True, ff=44),
                                                _attn(4, 4, 10, 18, 0.3, False)]},
    # equal key and value sizes of 64 and 128: prompt portions of the 16-bit mode run on the tcgen05 attention kernel
    "square": {"architecture": "Seledra", "max_positions": 200, "norm": {"eps": 1e-5}, "residual_mult": 0.6, "vocab": 190,
               "width": 128, "layers": [_attn(4, 2, 64, 64, 0.12, True, ff=96), _delta(2, 1, 32, 48, 4),
                                        _attn(2, 1, 128, 128, 0.08, False), _attn(2, 2, 64, 64, 0.12, True, ff=64)]},
}


def _weights(cfg_dict, seed):
    from petals_b200.models.seledra import from_config_dict, tensor_shapes

    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(from_config_dict(cfg_dict)).items():
        t = torch.randn(shape, generator=g)
        leaf = name.split(".", 1)[1] if "." in name and name[0] == "l" else name
        if leaf.endswith(("norm", "norm1", "norm2")):
            t = 1.0 + 0.2 * t
        elif leaf == "mix.temp":
            t = 1.0 + 0.3 * t
        elif leaf == "mix.vmix":
            t = 0.4 + 0.1 * t
        elif leaf == "mix.A_log":
            t = -0.5 + 0.5 * t
        elif leaf in ("mix.dt_bias", "mlp.act"):
            t = 0.7 * t
        elif leaf.endswith(".conv"):
            t = 0.6 * t
        elif len(shape) == 1:
            t = 0.3 * t                                   # biases
        elif name == "pos":
            t = 0.5 * t
        elif name != "embed":
            t = t * (1.5 * shape[-1] ** -0.5)
        out[name] = t.to(torch.bfloat16)
    return out


_MODELS = {}


def model(name, tmp_root):
    """(config dict, weights, model directory, oracle cache) of a test configuration."""
    if name not in _MODELS:
        from petals_b200.weights.safetensors_io import save_file

        cfg = CONFIGS.get(name) or EXTRA_CONFIGS[name]
        w = _weights(cfg, 11 + len(name))
        d = os.path.join(tmp_root, name)
        os.makedirs(d, exist_ok=True)
        json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
        save_file(w, os.path.join(d, "model.safetensors"))
        _MODELS[name] = (cfg, w, d, {})
    return _MODELS[name]


@pytest.fixture(scope="module")
def tmp_root(tmp_path_factory):
    return str(tmp_path_factory.mktemp("seledra"))


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
    g = torch.Generator().manual_seed(300 + seed)
    return torch.randint(0, (CONFIGS.get(name) or EXTRA_CONFIGS[name])["vocab"], (n,), generator=g).tolist()


def row_errs(got, want):
    """Per row: root mean square of the difference over that of the expected logits, mean removed."""
    d = got.double().cpu() - want.double()
    d = d - d.mean(-1, keepdim=True)
    ref = want.double() - want.double().mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt()


def rel_err(got, want):
    return float(row_errs(got, want).max())


TOL = {torch.float32: 2e-5, torch.bfloat16: 4e-2}
MODES = [torch.float32, torch.bfloat16]


def ids(toks):
    return torch.tensor(toks, dtype=torch.int64, device=DEV)


# ===================================================================================== mechanisms alone
def test_embedding_with_learned_positions():
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(1)
    table, pos = torch.randn(50, 24, generator=g).bfloat16().to(DEV), torch.randn(40, 24, generator=g).bfloat16().to(DEV)
    tok = torch.tensor([3, 49, 0, 7, 7], device=DEV)
    out = torch.zeros(5, 24, device=DEV)
    L.embed_pos_f32(tok, table, pos, out, pos0=17)
    assert torch.equal(out, table[tok].float() + pos[17:22].float())
    where = torch.tensor([0, 39, 5, 5, 12], dtype=torch.int32, device=DEV)
    L.embed_pos_f32(tok, table, pos, out, pos=where)
    assert torch.equal(out, table[tok].float() + pos[where.long()].float())


def test_scaled_residual_update_and_plain_norm():
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(2)
    x, y, gain = torch.randn(7, 136, generator=g), torch.randn(7, 136, generator=g), 1 + 0.2 * torch.randn(136, generator=g)
    xd, out = x.to(DEV), torch.zeros(7, 136, device=DEV)
    L.add_rms_norm(xd, gain.to(DEV), out, 1e-5, 0.0, add_a=y.to(DEV), add_scale=0.3)
    want_x = x.double() + 0.3 * y.double()
    assert torch.allclose(xd.cpu().double(), want_x, atol=1e-6)
    assert torch.allclose(out.cpu().double(), O.rms_normalise(want_x, 1e-5) * gain.double(), atol=1e-5)


def test_piecewise_activation_both_branches():
    from petals_b200.ops import layered as L

    z = torch.linspace(-9, 9, 601).reshape(1, -1).contiguous()
    z[0, 300] = 0.0
    for params in ([0.3, -0.8], [-2.0, 1.5], [0.0, 0.0]):
        p = torch.tensor(params)
        act = torch.zeros(1, 601, device=DEV)
        L.xielu(z.to(DEV), p.to(DEV), act)
        assert torch.allclose(act.cpu().double(), O.xielu(z.double(), p.double()), atol=1e-5, rtol=1e-6)


def test_gated_norm_per_head():
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(3)
    T, H, V = 5, 3, 44
    o, gate, gain = torch.randn(T, H * V, generator=g), torch.randn(T, H * V + 3, generator=g), torch.randn(V, generator=g)
    out = torch.zeros(T, H * V, device=DEV)
    L.gated_head_norm(o.to(DEV), gate.to(DEV)[:, 3:], gain.to(DEV), out, H, V, 1e-5)
    want = O.rms_normalise(o.double().view(T, H, V), 1e-5) * gain.double() * O.swish(gate[:, 3:].double()).view(T, H, V)
    assert torch.allclose(out.cpu().double().view(T, H, V), want, atol=1e-5)


@pytest.mark.parametrize("dt,V", [(torch.bfloat16, 64), (torch.bfloat16, 12), (torch.float32, 20)])
def test_gate_per_head_in_place(dt, V):
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(4)
    T, H = 7, 3
    x = torch.randn(T, H * V + 8, generator=g).to(dt)
    gate = torch.randn(T, H + 2, generator=g)
    xd = x.clone().to(DEV)
    L.head_gate(xd, gate.to(DEV)[:, 1:], H, V)
    want = x.float()[:, :H * V].view(T, H, V) * torch.sigmoid(gate[:, 1:1 + H])[..., None]
    assert torch.allclose(xd[:, :H * V].float().cpu().view(T, H, V), want, atol=2e-2 if dt == torch.bfloat16 else 1e-6, rtol=1e-2)
    assert torch.equal(xd[:, H * V:].cpu(), x[:, H * V:])


def _sink_reference(q, k, v, qpos, H, G, sink):
    """q [T, H, dk] (scale folded in), k [S, G, dk], v [S, G, dv] float64 -> [T, H, dv]."""
    out = torch.zeros(q.shape[0], H, v.shape[-1], dtype=F64)
    for t, p in enumerate(qpos):
        for h in range(H):
            g = h // (H // G)
            w = O.sink_softmax((k[: p + 1, g] @ q[t, h])[None, :], sink)[0]
            out[t, h] = (w[:, None] * v[: p + 1, g]).sum(0)
    return out


@pytest.mark.parametrize("cache_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["portion", "table", "table-3-shares", "table-16-shares", "tensor-core"])
def test_sink_attention_far_keys_chunk_edges_and_the_sink(cache_dtype, mode):
    """Queries at the first positions, around the kernels' 32-key chunks and 64-key tiles, and far along; one key per
    query is made loud - the first one, the last one, one in the middle - so that a lost key shows; one query has only
    small scores, so that the unit in the denominator carries most of the weight."""
    from petals_b200.ops import layered as L

    if mode == "tensor-core" and cache_dtype == torch.float32:
        pytest.skip("the tensor-core kernel reads 16-bit caches")
    g = torch.Generator().manual_seed(5)
    H, G, dk, dv, S, row = 6, 2, 24, 20, 200, 56
    k = torch.randn(S, G, dk, generator=g).to(cache_dtype).double()
    v = torch.randn(S, G, dv, generator=g).to(cache_dtype).double()
    planes = torch.zeros(2, 2, S + 8, row, dtype=cache_dtype, device=DEV)          # two "sessions" with the same rows
    planes[:, 0, :S, :G * dk] = k.reshape(S, -1).to(cache_dtype).to(DEV)
    planes[:, 1, :S, :G * dv] = v.reshape(S, -1).to(cache_dtype).to(DEV)
    if mode == "tensor-core":
        qpos = list(range(130))                    # a portion of three query tiles, the last one partial
        loud = {3: 0, 40: 32, 63: 0, 64: 63, 65: 64, 100: 0, 128: 1, 129: 64}      # query row -> key that is made loud
    else:
        qpos = [0, 1, 2, 31, 32, 33, 63, 64, 127, 128, 150, S - 1]
        loud = {3: 0, 4: 32, 5: 0, 6: 63, 7: 64, 8: 1, 9: 128, 10: 75, 11: 0}
    T = len(qpos)
    q = 0.25 * torch.randn(T, H, dk, generator=g)
    for t, j in loud.items():
        for h in range(H):
            q[t, h] += 5.0 * k[j, h // (H // G)].float() / k[j, h // (H // G)].norm().float()
    q[2] *= 0.01                                                                    # all scores near 0: the sink holds 1/4
    if mode == "tensor-core":
        q = q.bfloat16().float()
    gate = torch.randn(T, H, generator=g)
    want = _sink_reference(q.double(), k, v, qpos, H, G, 1.0) * torch.sigmoid(gate.double())[..., None]
    plain = _sink_reference(q.double(), k, v, qpos, H, G, 0.0) * torch.sigmoid(gate.double())[..., None]
    assert (want[2] - plain[2]).abs().max() > 0.05                                  # the sink is visible in the expectation
    proj = torch.zeros(T, H * dk + H + 5, device=DEV)
    proj[:, :H * dk] = q.reshape(T, -1).to(DEV)
    proj[:, H * dk:H * dk + H] = gate.to(DEV)
    out_dtype = cache_dtype if mode == "tensor-core" else torch.float32
    out = torch.zeros(T, H * dv, dtype=out_dtype, device=DEV)
    common = dict(q_off=0, k_off=0, v_off=0, g_off=H * dk, heads=H, kv_heads=G, dim=dk, vdim=dv, row_elems=row,
                  cache_dtype=cache_dtype, eps=1e-5, scale=1.0, sink=1.0)
    if mode == "tensor-core":
        a = L.sink_attn_args(proj, T=T, k_cache=planes[1, 0], v_cache=planes[1, 1], pos0=qpos[0], out=out, **common)
        L.sink_attn_prefill(a)
        got = out.float().cpu().double().view(T, H, dv)
        assert torch.allclose(got, want, atol=2e-2, rtol=2e-2)
        assert (got - want).abs().mean() < 2e-3
        return
    if mode == "portion":
        for t, p in enumerate(qpos):                                                # a one-token portion at position p
            a = L.sink_attn_args(proj[t:t + 1], T=1, k_cache=planes[1, 0], v_cache=planes[1, 1], pos0=p, out=out[t:t + 1], **common)
            L.sink_attn(a)
    else:
        shares = {"table": 1, "table-3-shares": 3, "table-16-shares": 16}[mode]
        ptrs = torch.tensor([[planes[t % 2, 0].data_ptr(), planes[t % 2, 1].data_ptr()] for t in range(T)], dtype=torch.int64, device=DEV)
        pos_t = torch.tensor(qpos, dtype=torch.int32, device=DEV)
        scratch = torch.zeros(T * H * shares * (dv + 2), device=DEV)
        a = L.sink_attn_args(proj, T=T, kv_ptrs=ptrs, kv_ptr_stride=2, pos=pos_t, out=out, **common)
        L.sink_attn(a, shares, scratch)
    got = out.cpu().double().view(T, H, dv)
    assert torch.allclose(got, want, atol=2e-5, rtol=1e-5)


@pytest.mark.parametrize("vmix_mode", [0, 1, 2])
def test_projection_norms_value_blending_and_cache_append(vmix_mode):
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(6)
    T, H, G, dk, dv, row, eps, scale = 5, 6, 3, 10, 14, 48, 1e-5, 0.3
    nq, nk, nv = H * dk, G * dk, G * dv
    raw = torch.randn(T, nq + nk + nv + H, generator=g)
    bias, qg, kg = torch.randn(nq + nk + nv, generator=g), torch.randn(nq, generator=g), torch.randn(nk, generator=g)
    temp, lam = 1 + 0.3 * torch.randn(H, generator=g), torch.tensor([0.37])
    first = torch.randn(T, nv, generator=g)
    proj, vf = raw.clone().to(DEV), first.clone().to(DEV)
    planes = torch.zeros(2, 40, row, device=DEV)
    a = L.sink_attn_args(proj, q_off=0, k_off=nq, v_off=nq + nk, g_off=nq + nk + nv, heads=H, kv_heads=G, dim=dk, vdim=dv,
                         row_elems=row, cache_dtype=torch.float32, eps=eps, scale=scale, sink=1.0, T=T, bias=bias.to(DEV),
                         q_gain=qg.to(DEV), k_gain=kg.to(DEV), temp=temp.to(DEV), vmix=lam.to(DEV), v_first=vf, vmix_mode=vmix_mode,
                         k_cache=planes[0], v_cache=planes[1], pos0=9)
    L.sink_attn_append(a)
    x = raw.double()
    q = O.rms_normalise(x[:, :nq] + bias[:nq].double(), eps) * qg.double()
    q = q.view(T, H, dk) * (scale * temp.double())[None, :, None]
    k = O.rms_normalise(x[:, nq:nq + nk] + bias[nq:nq + nk].double(), eps) * kg.double()
    v = O.rms_normalise((x[:, nq + nk:nq + nk + nv] + bias[nq + nk:].double()).view(T, G, dv), eps).reshape(T, nv)
    if vmix_mode == 1:
        assert torch.allclose(vf.cpu().double(), v, atol=1e-5)
    if vmix_mode == 2:
        v = (1 - 0.37) * v + 0.37 * first.double()
    assert torch.allclose(proj[:, :nq].cpu().double(), q.reshape(T, nq), atol=1e-5)
    assert torch.allclose(planes[0, 9:9 + T, :nk].cpu().double(), k, atol=1e-5)
    assert torch.allclose(planes[1, 9:9 + T, :nv].cpu().double(), v, atol=1e-5)
    assert float(planes[:, :9].abs().max()) == 0 and float(planes[:, 9 + T:].abs().max()) == 0


def _delta_reference(x, conv_w, blog, alog, A_log, dt_bias, H, G, dk, dv, unit_eps=1e-6):
    """x [T, C] convolution inputs, blog / alog [T, H] -> (work rows, raw read-out [T, H, dv]) in float64."""
    T = x.shape[0]
    y = O.causal_conv(x, conv_w)
    q, k, v = y[:, :G * dk].reshape(T, G, dk), y[:, G * dk:2 * G * dk].reshape(T, G, dk), y[:, 2 * G * dk:].reshape(T, H, dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * dk ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
    beta = torch.sigmoid(blog)
    decay = torch.exp(-torch.exp(A_log) * O.soft_plus(alog + dt_bias))
    read = torch.zeros(T, H, dv, dtype=F64)
    for h in range(H):
        S = torch.zeros(dk, dv, dtype=F64)
        for i in range(T):
            S = decay[i, h] * S
            u = beta[i, h] * (v[i, h] - S.T @ k[i, h // (H // G)])
            S = S + k[i, h // (H // G)][:, None] * u[None, :]
            read[i, h] = S.T @ q[i, h // (H // G)]
    work = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), beta, decay], 1)
    return work, read


@pytest.mark.parametrize("H,G,dk,dv,taps", [(4, 2, 24, 40, 3), (3, 3, 20, 12, 1), (2, 1, 72, 136, 5), (2, 2, 130, 8, 2), (2, 1, 260, 20, 4), (1, 1, 520, 8, 2)])
@pytest.mark.parametrize("cuts", [(57,), (1, 1, 1, 2, 17, 16, 15, 4), (33, 24)], ids=["whole", "pieces", "two"])
def test_delta_rule_in_pieces_carries_state_and_convolution_inputs(H, G, dk, dv, taps, cuts):
    """The recurrence over one sequence cut into launches of many sizes (one token, two, the kernel's 16-token batches
    and their neighbours): matrices and convolution inputs pass from launch to launch through the session's state."""
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(7)
    T = sum(cuts)
    C = 2 * G * dk + H * dv
    x = torch.randn(T, C, generator=g)
    blog, alog = torch.randn(T, H, generator=g), torch.randn(T, H, generator=g)
    conv_w, A_log, dt_bias = 0.6 * torch.randn(C, taps, generator=g), -0.5 + 0.5 * torch.randn(H, generator=g), torch.randn(H, generator=g)
    want_work, want_read = _delta_reference(x.double(), conv_w.double(), blog.double(), alog.double(), A_log.double(), dt_bias.double(), H, G, dk, dv)
    proj = torch.cat([torch.zeros(T, 2), x, blog, alog], 1).to(DEV).contiguous()
    pad = 5
    state = torch.full((pad + 2 * H * dk * dv + taps * C,), 7.0, device=DEV)     # stale numbers: position 0 must not read them
    work, o = torch.zeros(T, C + 2 * H + G, device=DEV), torch.zeros(T, H * dv, device=DEV)
    at = 0
    for n in cuts:
        a = L.delta_args(proj[at:at + n], c_off=2, b_off=2 + C, a_off=2 + C + H, conv_w=conv_w.to(DEV), A_log=A_log.to(DEV),
                         dt_bias=dt_bias.to(DEV), work=work[at:at + n], o=o[at:at + n], heads=H, kv_heads=G, dim=dk, vdim=dv,
                         taps=taps, unit_eps=1e-6, n_seq=1, seq_len=n, state=state, state_off=pad, pos0=at)
        L.delta_prep(a)
        L.delta_rule(a)
        at += n
    assert torch.allclose(work[:, :C + 2 * H].cpu().double(), want_work, atol=2e-5, rtol=1e-5)
    kq = (want_work[:, :G * dk].view(T, G, dk) * want_work[:, G * dk:2 * G * dk].view(T, G, dk)).sum(-1)
    assert torch.allclose(work[:, C + 2 * H:].cpu().double(), kq, atol=2e-6)
    assert torch.allclose(o.cpu().double().view(T, H, dv), want_read, atol=2e-5, rtol=1e-4)
    assert float((state[:pad] - 7.0).abs().max()) == 0


def test_delta_rule_step_for_a_batch_of_sequences_is_repeatable():
    """One token for each of three sequences at different positions through the pointer table; running the same step
    twice (as the warm-up before a graph capture does) leaves the same state and the same result."""
    from petals_b200.ops import layered as L

    g = torch.Generator().manual_seed(8)
    H, G, dk, dv, taps = 4, 2, 16, 24, 4
    C = 2 * G * dk + H * dv
    lens = [9, 1, 30]
    conv_w, A_log, dt_bias = 0.6 * torch.randn(C, taps, generator=g), -0.5 + 0.5 * torch.randn(H, generator=g), torch.randn(H, generator=g)
    par = dict(conv_w=conv_w.to(DEV), A_log=A_log.to(DEV), dt_bias=dt_bias.to(DEV), heads=H, kv_heads=G, dim=dk, vdim=dv, taps=taps,
               unit_eps=1e-6, c_off=0, b_off=C, a_off=C + H)
    seqs = [torch.randn(n, C + 2 * H, generator=g) for n in lens]
    states = [torch.zeros(2 * H * dk * dv + taps * C, device=DEV) for _ in lens]
    want = []
    for s, n in zip(seqs, lens):
        want.append(_delta_reference(s[:, :C].double(), conv_w.double(), s[:, C:C + H].double(), s[:, C + H:].double(), A_log.double(),
                                     dt_bias.double(), H, G, dk, dv)[1][-1])
    for s, n, st in zip(seqs, lens, states):                                      # everything but the last token
        if n > 1:
            p = s[:n - 1].to(DEV).contiguous()
            a = L.delta_args(p, work=torch.zeros(n - 1, C + 2 * H + G, device=DEV), o=torch.zeros(n - 1, H * dv, device=DEV), n_seq=1,
                             seq_len=n - 1, state=st, pos0=0, **par)
            L.delta_prep(a)
            L.delta_rule(a)
    last = torch.stack([s[-1] for s in seqs]).to(DEV).contiguous()
    ptrs = torch.tensor([[st.data_ptr(), 0] for st in states], dtype=torch.int64, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    work, o = torch.zeros(3, C + 2 * H + G, device=DEV), torch.zeros(3, H * dv, device=DEV)
    a = L.delta_args(last, work=work, o=o, n_seq=3, seq_len=1, state_ptrs=ptrs, state_ptr_stride=2, pos=pos, **par)
    L.delta_prep(a)
    L.delta_rule(a)
    first, snap = o.clone(), [st.clone() for st in states]
    L.delta_prep(a)
    L.delta_rule(a)
    assert torch.equal(first, o) and all(torch.equal(x, y) for x, y in zip(snap, states))
    assert torch.allclose(o.cpu().double().view(3, H, dv), torch.stack(want), atol=2e-5, rtol=1e-4)


# ===================================================================================== whole models
@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_logits_at_every_position(name, dtype, tmp_root):
    span, mgr = span_of(name, tmp_root, dtype)
    toks = tokens_of(name, 45)
    kv = mgr.allocate("p", 128)
    got = span.prefill(kv, ids=ids(toks), logits_at=list(range(len(toks))))[0]      # three chunks of 16, the last partial
    assert rel_err(got, oracle_logits(name, tmp_root, toks)) < TOL[dtype]
    mgr.close("p")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(EXTRA_CONFIGS))
def test_models_with_one_kind_of_mixer_and_odd_sizes(name, dtype, tmp_root):
    """No cache rows at all (only state), or no state at all (only rows); a 70-token prompt in 64-token chunks (the
    tensor-core attention with sizes that rule out its 16-byte loads), then decoding.  And a model whose attention
    layers have equal key and value sizes of 64 / 128 (their portions run on the tcgen05 kernel over the planes with
    the sink's zero row in front, the gate applied behind it)."""
    span, mgr = span_of(name, tmp_root, dtype, max_chunk=64)
    n = 158 if name == "square" else 78          # (square: a second full chunk that starts mid-session)
    toks = tokens_of(name, n, 9)
    want = oracle_logits(name, tmp_root, toks)
    kv = mgr.allocate("x", 256)
    assert (kv.state is None) == (name == "attention-only")
    assert (span.q16 is not None) == (name == "square" and dtype != torch.float32)
    rows = [span.prefill(kv, ids=ids(toks[:n - 8]), logits_at=list(range(n - 8)))[0]]
    for p in range(n - 8, n):
        rows.append(span.decode([kv], ids=ids(toks[p:p + 1]))[0].clone())
    assert rel_err(torch.cat(rows), want) < TOL[dtype]
    mgr.close("x")


def test_the_stream_after_every_layer(tmp_root):
    """fp32 mode: the residual stream after each layer (its pending update applied) against the oracle's."""
    name = "mixed"
    cfg, w, _, _ = model(name, tmp_root)
    span, mgr = span_of(name, tmp_root, torch.float32)
    toks = tokens_of(name, 13, 4)
    want = []
    O.forward(cfg, w, toks, layers_out=want)
    seen = []
    inner = span._layer

    def spy(T, x, P, where):
        inner(T, x, P, where)
        seen.append((x[:T] + span.residual_mult * span._pending["add_a"][:T]).clone())

    span._layer = spy
    try:
        kv = mgr.allocate("layers", 128)
        span.prefill(kv, ids=ids(toks))
    finally:
        span._layer = inner
        mgr.close("layers")
    assert len(seen) == len(want)
    for got, ref in zip(seen, want):
        assert float((got.cpu().double() - ref).abs().max()) < 2e-4 * float(ref.abs().max())


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_decoding_token_by_token_equals_the_prompt_pass(name, dtype, tmp_root):
    """From the very first token: a one-token prompt, then 40 decode steps (the first tokens of a sequence, the
    convolutions' start, state copies alternating for a long run)."""
    span, mgr = span_of(name, tmp_root, dtype)
    toks = tokens_of(name, 41, 1)
    kv = mgr.allocate("d", 128)
    rows = [span.prefill(kv, ids=ids(toks[:1]), logits_at=[0])[0]]
    for p in range(1, len(toks)):
        rows.append(span.decode([kv], ids=ids(toks[p:p + 1]))[0].clone())
    assert rel_err(torch.cat(rows), oracle_logits(name, tmp_root, toks)) < TOL[dtype]
    mgr.close("d")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("portion", [2, 3, 7, 16, 19])
def test_prompts_in_portions(portion, dtype, tmp_root):
    name = "mixed"
    span, mgr = span_of(name, tmp_root, dtype)
    toks = tokens_of(name, 50, 2)
    kv = mgr.allocate("q", 128)
    rows = []
    for c0 in range(0, len(toks), portion):
        part = toks[c0:c0 + portion]
        rows.append(span.prefill(kv, ids=ids(part), logits_at=list(range(len(part))))[0])
    assert rel_err(torch.cat(rows), oracle_logits(name, tmp_root, toks)) < TOL[dtype]
    mgr.close("q")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_batches_of_unequal_requests_and_reused_sessions(name, dtype, tmp_root):
    """Three requests of different lengths decode together; the shortest ends, its session is freed and a fourth
    request takes a new one (possibly the same bytes) and joins the others' later steps."""
    span, mgr = span_of(name, tmp_root, dtype)
    reqs = {"a": tokens_of(name, 33, 3), "b": tokens_of(name, 12, 4), "c": tokens_of(name, 21, 5), "d": tokens_of(name, 17, 6)}
    cuts = {"a": 20, "b": 5, "c": 1, "d": 9}
    kvs = {k: mgr.allocate(k, 128) for k in "abc"}
    got = {k: [] for k in reqs}
    at = {}
    for k in "abc":
        got[k].append(span.prefill(kvs[k], ids=ids(reqs[k][:cuts[k]]), logits_at=[cuts[k] - 1])[0])
        at[k] = cuts[k]
    joined = False
    while any(at[k] < len(reqs[k]) for k in kvs):
        live = [k for k in kvs if at[k] < len(reqs[k])]
        logits, _ = span.decode([kvs[k] for k in live], ids=ids([reqs[k][at[k]] for k in live]))
        for b, k in enumerate(live):
            got[k].append(logits[b:b + 1].clone())
            at[k] += 1
        if not joined and at["b"] == len(reqs["b"]):
            mgr.close("b")
            del kvs["b"]
            kvs["d"] = mgr.allocate("d", 128)
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
    """Chunks of 64 tokens (the tensor-core attention of the 16-bit mode: query tiles and key tiles from earlier
    chunks), the last one partial, then decoding; then a chunk that starts in the middle of a session."""
    span, mgr = span_of(name, tmp_root, dtype, max_chunk=64)
    toks = tokens_of(name, 150, 11)
    want = oracle_logits(name, tmp_root, toks)
    kv = mgr.allocate("long", 256)
    rows = [span.prefill(kv, ids=ids(toks[:141]), logits_at=list(range(141)))[0]]
    for p in range(141, 150):
        rows.append(span.decode([kv], ids=ids(toks[p:p + 1]))[0].clone())
    assert rel_err(torch.cat(rows), want) < TOL[dtype]
    mgr.close("long")
    kv = mgr.allocate("long", 256)
    span.prefill(kv, ids=ids(toks[:37]))
    got = span.prefill(kv, ids=ids(toks[37:150]), logits_at=list(range(150 - 37)))[0]
    assert rel_err(got, want[37:]) < TOL[dtype]
    mgr.close("long")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
def test_long_decoding_with_a_large_cache(dtype, tmp_root):
    """A cache of 1024 positions (decode attention divides every token's keys over 8 blocks; the shares' borders move with
    the length) and 150 decode steps behind a 100-token prompt: state copies alternate 150 times, the key count passes
    the 128-key borders of the shares."""
    from petals_b200.models.config import resolve_config
    from petals_b200.runtime.kv_cache import KVCacheManager
    from petals_b200.runtime.layered_span import make_span
    from petals_b200.weights.loader import load_span

    name = "plain"
    d = model(name, tmp_root)[2]
    cfg = resolve_config(d)
    w = load_span(d, cfg, 0, cfg.n_layers, need_embed=True, need_head=True, dtype=dtype, device=DEV)
    span = make_span(cfg, w, DEV, dtype, kv_capacity=1024, max_batch=2, max_chunk=64)
    assert span._sink_splits(1, cfg.layers[0].mixer)[0] == 8
    mgr = KVCacheManager.for_span(cfg, 0, cfg.n_layers, dtype, DEV, default_max_length=1024)
    toks = tokens_of(name, 250, 21)
    want = oracle_logits(name, tmp_root, toks)
    kv = mgr.allocate("far", 1024)
    rows = [span.prefill(kv, ids=ids(toks[:100]), logits_at=[99])[0]]
    for p in range(100, 250):
        rows.append(span.decode([kv], ids=ids(toks[p:p + 1]))[0].clone())
    assert rel_err(torch.cat(rows), want[99:]) < TOL[dtype]
    mgr.close("far")


@pytest.mark.parametrize("dtype", MODES, ids=["fp32", "bf16"])
def test_two_spans_in_a_row_equal_the_whole_model(dtype, tmp_root):
    """The model cut after its first layer, as two pipeline stages would hold it: the first span embeds and hands the fp32
    stream on, the second one owns the recurrent layer's state and the last attention layer's cache and the head."""
    from petals_b200.models.config import resolve_config
    from petals_b200.runtime.kv_cache import KVCacheManager
    from petals_b200.runtime.layered_span import make_span
    from petals_b200.weights.loader import load_span

    name = "plain"
    d = model(name, tmp_root)[2]
    cfg = resolve_config(d)
    wa = load_span(d, cfg, 0, 1, need_embed=True, need_head=False, dtype=dtype, device=DEV)
    wb = load_span(d, cfg, 1, 3, need_embed=False, need_head=True, dtype=dtype, device=DEV)
    sa = make_span(cfg, wa, DEV, dtype, kv_capacity=128, max_batch=2, max_chunk=16)
    sb = make_span(cfg, wb, DEV, dtype, kv_capacity=128, max_batch=2, max_chunk=16)
    ma = KVCacheManager.for_span(cfg, 0, 1, dtype, DEV, default_max_length=128)
    mb = KVCacheManager.for_span(cfg, 1, 3, dtype, DEV, default_max_length=128)
    ka, kb = ma.allocate("s", 128), mb.allocate("s", 128)
    assert ka.state is None and kb.state is not None and kb.state.numel() == cfg.state_elems(1, 3)
    toks = tokens_of(name, 30, 22)
    want = oracle_logits(name, tmp_root, toks)
    h = sa.prefill(ka, ids=ids(toks[:21]))
    assert h.dtype == torch.float32 and tuple(h.shape) == (21, cfg.hidden)
    rows = [sb.prefill(kb, h_in=h, logits_at=list(range(21)))[0]]
    for p in range(21, 30):
        h1 = sa.decode([ka], ids=ids(toks[p:p + 1]))
        rows.append(sb.decode([kb], h_in=h1)[0].clone())
    assert rel_err(torch.cat(rows), want) < TOL[dtype]
    with pytest.raises(ValueError):
        resolve_config(model("mixed", tmp_root)[2]).check_span(2, 4)      # layer 2 blends with layer 1's values


def test_a_session_holds_one_token_less_than_its_rows(tmp_root):
    """Attention with a sink keeps row 0 of its planes for the sink: 127 tokens fit into 128 rows, the 128th is refused;
    the last rows are read correctly."""
    name, dtype = "mixed", torch.float32
    span, mgr = span_of(name, tmp_root, dtype)
    toks = tokens_of(name, 128, 13)
    kv = mgr.allocate("full", 128)
    span.prefill(kv, ids=ids(toks[:125]))
    rows = [span.decode([kv], ids=ids(toks[p:p + 1]))[0].clone() for p in (125, 126)]
    assert rel_err(torch.cat(rows), oracle_logits(name, tmp_root, toks[:127])[125:]) < TOL[dtype]
    assert float(kv.data[:, :, :, 0].abs().max()) == 0.0
    with pytest.raises(ValueError):
        span.decode([kv], ids=ids(toks[127:128]))
    mgr.close("full")


def test_a_freed_or_reset_session_is_clean_for_its_next_owner(tmp_root):
    """The same session name and the same bytes, used again for another request: neither cache rows nor matrices nor
    convolution inputs of the first one show (a recurrent layer reads no state at a sequence's first token)."""
    name, dtype = "plain", torch.float32
    span, mgr = span_of(name, tmp_root, dtype)
    long, short = tokens_of(name, 41), tokens_of(name, 12, 2)
    kv = mgr.allocate("s", 128)
    span.prefill(kv, ids=ids(long))
    mgr.close("s")
    kv = mgr.allocate("s", 128)
    got = span.prefill(kv, ids=ids(short), logits_at=list(range(len(short))))[0]
    assert rel_err(got, oracle_logits(name, tmp_root, short)) < TOL[dtype]
    kv2 = mgr.allocate("s", 128)                                   # same id again: reset in place, state left as it was
    assert kv2.data.data_ptr() == kv.data.data_ptr() and kv2.length == 0 and float(kv2.state.abs().max()) > 0
    rows = [span.prefill(kv2, ids=ids(long[:1]), logits_at=[0])[0]]
    for p in range(1, 6):
        rows.append(span.decode([kv2], ids=ids(long[p:p + 1]))[0].clone())
    assert rel_err(torch.cat(rows), oracle_logits(name, tmp_root, long)[:6]) < TOL[dtype]
    with pytest.raises(ValueError):
        kv2.rollback(3)                                            # matrices cannot be wound back
    kv2.rollback(0)
    mgr.close("s")


def test_cuda_graph_steps_equal_eager_steps(tmp_root):
    from petals_b200.models.config import resolve_config
    from petals_b200.runtime.layered_span import make_span
    from petals_b200.weights.loader import load_span

    name = "mixed"
    span, mgr = span_of(name, tmp_root, torch.bfloat16)
    d = model(name, tmp_root)[2]
    cfg = resolve_config(d)
    w = load_span(d, cfg, 0, cfg.n_layers, need_embed=True, need_head=True, dtype=torch.bfloat16, device=DEV)
    eager = make_span(cfg, w, DEV, torch.bfloat16, kv_capacity=128, max_batch=4, max_chunk=16, use_graphs=False, pdl=False)
    toks = tokens_of(name, 24)
    ka, kb = mgr.allocate("g", 128), mgr.allocate("e", 128)
    span.prefill(ka, ids=ids(toks[:9]))
    eager.prefill(kb, ids=ids(toks[:9]))
    for p in range(9, 24):
        la = span.decode([ka], ids=ids(toks[p:p + 1]))[0].clone()
        lb = eager.decode([kb], ids=ids(toks[p:p + 1]))[0].clone()
        assert torch.equal(la, lb)
    assert span._graphs, "the decode step was not captured"
    assert torch.equal(ka.state, kb.state)
    mgr.close("g")
    mgr.close("e")


def test_beam_reorder_copies_rows_and_state(tmp_root):
    name, dtype = "mixed", torch.float32
    span, mgr = span_of(name, tmp_root, dtype)
    ta, tb = tokens_of(name, 14, 7), tokens_of(name, 9, 8)
    ka, kb = mgr.allocate("ra", 128), mgr.allocate("rb", 128)
    span.prefill(ka, ids=ids(ta[:13]))
    span.prefill(kb, ids=ids(tb))
    mgr.reorder(["ra", "rb"], [0, 0])                              # both continue the first hypothesis
    got = span.decode([ka, kb], ids=ids([ta[13], ta[13]]))[0].clone()
    want = oracle_logits(name, tmp_root, ta)[13:14]
    assert rel_err(got[0:1], want) < TOL[dtype] and rel_err(got[1:2], want) < TOL[dtype]
    mgr.close("ra")
    mgr.close("rb")


# ===================================================================================== entry points
def test_greedy_generation_through_the_engine(tmp_root):
    """PipelineEngine.generate: prompts of unequal lengths are prefilled one by one and decoded together by the
    engine's rounds; the tokens must be the oracle's greedy continuation."""
    from petals_b200.parallel.pipeline import PipelineEngine

    name = "plain"
    cfg, w, d, _ = model(name, tmp_root)
    eng = PipelineEngine(d, (), torch.float32, torch.device(DEV), kv_capacity=64, max_sessions=4, max_chunk=16)
    prompts = [tokens_of(name, 9, 5), tokens_of(name, 3, 6), tokens_of(name, 14, 7)]
    outs, stats = eng.generate([torch.tensor(p) for p in prompts], max_new_tokens=8)
    for p, o in zip(prompts, outs):
        assert o == O.greedy(cfg, w, p, 8)
    assert stats["decode_tok_per_s"] > 0


def test_preset_with_random_weights_generates():
    """``tiny-seledra``: no folder, weights drawn from the tensor names; two runs give the same tokens."""
    from petals_b200.parallel.pipeline import PipelineEngine

    eng = PipelineEngine("tiny-seledra", (), torch.bfloat16, torch.device(DEV), kv_capacity=64, max_sessions=2, max_chunk=16)
    prompt = [torch.tensor([5, 9, 200, 17, 3])]
    a, _ = eng.generate(prompt, max_new_tokens=6)
    b, _ = eng.generate(prompt, max_new_tokens=6)
    assert a == b and len(a[0]) == 6 and all(0 <= t < 512 for t in a[0])


def test_sampled_generation_runs_on_the_device_sampler(tmp_root):
    from petals_b200.parallel.pipeline import PipelineEngine
    from petals_b200.runtime.sampler import SamplingParams

    d = model("mixed", tmp_root)[2]
    eng = PipelineEngine(d, (), torch.bfloat16, torch.device(DEV), kv_capacity=64, max_sessions=2, max_chunk=16)
    sp = SamplingParams(temperature=0.8, top_k=20, top_p=0.9)
    a, _ = eng.generate([torch.tensor(tokens_of("mixed", 6))], max_new_tokens=6, sampling=sp, seed=3)
    b, _ = eng.generate([torch.tensor(tokens_of("mixed", 6))], max_new_tokens=6, sampling=sp, seed=3)
    assert a == b and all(0 <= t < CONFIGS["mixed"]["vocab"] for t in a[0])


def test_trace_replay_steps(tmp_root):
    from src.trace_replay import TraceReplayer

    name = "mixed"
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
    """``python -m src.main --inbox`` on a Seledra folder: registry, loader, engine, greedy decoding, byte tokenizer."""
    import subprocess
    import sys

    name = "plain"
    cfg, w, d, _ = model(name, tmp_root)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29633", RANK="0", WORLD_SIZE="1", LOCAL_RANK="0")
    r = subprocess.run([sys.executable, "-m", "src.main", "--inbox", "--stage", "0", "--model", d, "--splits", "", "--dtype", "fp32",
                        "--temperature", "0", "--max_new_tokens", "6", "--prompt", "abc"], cwd=root, env=env,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    prompt = [(3 + b) % cfg["vocab"] for b in b"abc"]
    want = O.greedy(cfg, w, prompt, 6)
    text = bytearray((t - 3) if 0 <= t - 3 < 256 else ord("?") for t in want).decode("utf-8", errors="replace")
    assert "GENERATED: " + text in r.stdout, (r.stdout[-500:], want)
