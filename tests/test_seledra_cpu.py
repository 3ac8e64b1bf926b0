"""Host-side parts of the Seledra integration (no GPU): configuration registry, tensor names, cache and state layout,
span checks, random models, and the oracle's own consistency."""
import json

import pytest
import torch

from petals_b200.models import seledra as S
from petals_b200.models.config import from_hf_dict, resolve_config
from petals_b200.runtime.kv_cache import KVCacheManager
from petals_b200.weights.loader import RandomSource, load_span
from tests import seledra_oracle as O


def _cfg():
    return S.make_config("dAaD", hidden=96, vocab=130, heads=6, kv_heads=3, dim=8, vdim=12, delta_heads=4, delta_kv_heads=2,
                         delta_dim=16, delta_vdim=20, conv=3, ff=40, residual_mult=0.6, max_positions=64)


def test_config_round_trip_and_registry(tmp_path):
    cfg = _cfg()
    d = S.to_config_dict(cfg)
    assert from_hf_dict(json.loads(json.dumps(d))).layers == cfg.layers
    (tmp_path / "config.json").write_text(json.dumps(d))
    got = resolve_config(str(tmp_path))
    assert got.family == "seledra" and got.n_layers == 4 and got.hidden == 96 and got.vocab == 130
    assert [L.mixer.kind for L in got.layers] == ["delta", "attention", "attention", "delta"]
    assert [L.mlp is not None for L in got.layers] == [False, True, False, True]
    assert got.residual_mult == 0.6 and got.max_positions == 64 and got.layer_list and not got.parallel_block
    assert resolve_config("tiny-seledra").family == "seledra" and resolve_config("tiny-gigezen").family == "gigezen"


def test_config_rejects_what_cannot_run():
    d = S.to_config_dict(_cfg())
    bad = json.loads(json.dumps(d))
    bad["layers"][1]["mixer"]["kv_heads"] = 4            # 6 heads do not divide into 4 groups
    with pytest.raises(ValueError):
        from_hf_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][2]["mixer"]["vdim"] = 16               # blends its values with layer 1's, which have another size
    with pytest.raises(ValueError):
        from_hf_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        from_hf_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][3]["mlp"]["kind"] = "moe"
    with pytest.raises(ValueError):
        from_hf_dict(bad)


def test_cache_and_state_layout_and_span_checks():
    cfg = _cfg()
    assert cfg.cache_layers() == [1, 2] and cfg.cache_row() == 40 and cfg.cache_planes == 2
    per_delta = 2 * 4 * 16 * 20 + 3 * (2 * 2 * 16 + 4 * 20)
    assert cfg.layers[0].mixer.state_elems == per_delta and cfg.state_elems() == 2 * per_delta
    assert cfg.state_offsets() == {0: 0, 3: per_delta} and cfg.state_offsets(2, 4) == {3: 0}
    mgr = KVCacheManager.for_span(cfg, 0, 4, torch.float32, "cpu", default_max_length=32)
    kv = mgr.allocate("s", 32)
    assert tuple(kv.data.shape) == (2, 2, 1, 32, 40) and tuple(kv.plane(1, 1).shape) == (32, 40)
    assert kv.state.dtype == torch.float32 and kv.state.numel() == 2 * per_delta
    assert mgr.bytes_per_token() == 2 * 2 * 40 * 4
    kv.plane(1, 1)[5, 3] = 1.0
    assert float(kv.data[1, 1, 0, 5, 3]) == 1.0
    kv.length = 7
    with pytest.raises(ValueError):
        kv.rollback(3)
    kv.rollback(0)
    cfg.check_span(0, 4)
    cfg.check_span(0, 2)
    with pytest.raises(ValueError):
        cfg.check_span(2, 4)                             # layer 2 needs layer 1's values


def test_state_counts_against_the_byte_budget():
    cfg = _cfg()
    mgr = KVCacheManager.for_span(cfg, 0, 4, torch.float32, "cpu", default_max_length=16, max_tokens=32, max_sessions=2)
    assert mgr.cache.max_size_bytes == 32 * mgr.bytes_per_token() + 2 * 4 * cfg.state_elems()
    a, b = mgr.allocate("a", 16), mgr.allocate("b", 16)
    assert mgr.cache.bytes_left == 0 and a.state.data_ptr() != b.state.data_ptr()
    mgr.close("a")
    assert mgr.cache.bytes_left == 16 * mgr.bytes_per_token() + 4 * cfg.state_elems()


def test_reorder_copies_state():
    cfg = _cfg()
    mgr = KVCacheManager.for_span(cfg, 0, 4, torch.float32, "cpu", default_max_length=8)
    a, b = mgr.allocate("a", 8), mgr.allocate("b", 8)
    a.state.fill_(2.0)
    a.data.fill_(3.0)
    a.length = 4
    mgr.reorder(["a", "b"], [0, 0])
    assert b.length == 4 and float(b.state.min()) == 2.0 and float(b.data[:, :, :, :4].min()) == 3.0
    assert float(b.data[:, :, :, 5:].abs().max()) == 0.0          # (one row beyond the length travels too)


def test_tensor_names_and_random_models():
    cfg = _cfg()
    shapes = S.tensor_shapes(cfg)
    assert shapes["pos"] == (64, 96) and shapes["l1.mix.vmix"] == () and shapes["l1.mix.q.norm"] == (48,)
    assert shapes["l0.mix.b"] == (4, 96) and shapes["l0.mix.q.conv"] == (32, 3) and shapes["l0.mix.norm"] == (20,)
    assert "l0.norm2" not in shapes and shapes["l1.mlp.act"] == (2,) and shapes["l3.mix.o"] == (96, 80)
    src = RandomSource(cfg, seed=1)
    assert set(src.shapes) == set(shapes)
    w = load_span("random:x", cfg, 0, 4, need_embed=True, need_head=True, dtype=torch.float32, device="cpu", src=src)
    assert w["pos_embed"].shape == (64, 96) and w["layers"][1]["qkv_b"].shape == (48 + 24 + 36,)
    assert w["layers"][0]["conv_w"].shape == (32 + 32 + 80, 3) and w["layers"][1]["vmix"].shape == (1,)
    assert w["layers"][0]["A_log"].dtype == torch.float32 and "norm2_w" not in w["layers"][0]


def test_oracle_is_causal_and_step_consistent():
    cfg = _cfg()
    d = S.to_config_dict(cfg)
    src = RandomSource(cfg, seed=2)
    w = {k: src.get(k) for k in src.shapes}
    toks = [5, 9, 77, 3, 128, 0, 41, 6, 6, 90]
    full = O.forward(d, w, toks)
    assert full.shape == (10, 130) and torch.isfinite(full).all()
    assert torch.allclose(O.forward(d, w, toks[:6]), full[:6], atol=1e-12)        # later tokens change nothing earlier
    assert len(O.greedy(d, w, toks[:3], 4)) == 4


def test_oracle_sink_and_delta_rule_identities():
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=torch.float64)
    p = O.sink_softmax(s)
    assert torch.allclose(p.sum(), torch.exp(s).sum() / (1 + torch.exp(s).sum()))
    assert torch.allclose(O.sink_softmax(s, 0.0), torch.softmax(s, -1))
    # with beta = 1, no decay and a unit key the state returns the stored value for that key
    k = torch.tensor([0.6, 0.8], dtype=torch.float64)
    v = torch.tensor([1.0, -2.0, 3.0], dtype=torch.float64)
    S0 = torch.randn(2, 3, dtype=torch.float64)
    S1 = S0 + k[:, None] * (v - S0.T @ k)[None, :]
    assert torch.allclose(S1.T @ k, v)
    z = torch.tensor([-3.0, 0.0, 2.0], dtype=torch.float64)
    y = O.xielu(z, torch.tensor([0.0, 0.0], dtype=torch.float64))
    ln2 = torch.log(torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(y[2], ln2 * 4 + 1.0) and y[1] == 0 and torch.allclose(y[0], (0.5 + ln2) * (torch.expm1(z[0]) - z[0]) + 0.5 * z[0])
