"""Host-side parts of the Gigezen integration (no GPU): configuration registry, tensor names, cache layout,
span checks, and the oracle's own consistency."""
import json

import pytest
import torch

from petals_b200.models import gigezen as Z
from petals_b200.models.config import from_hf_dict, resolve_config
from petals_b200.runtime.kv_cache import KVCacheManager
from petals_b200.weights.loader import RandomSource, load_span
from tests import gigezen_oracle as O


def _cfg():
    return Z.make_config(n_layers=5, hidden=96, vocab=130, heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, window=6,
                         ff=40, experts=6, top=2, groups=3, keep=2, expert_ff=16, share_every=2, moe_every=3)


def test_config_round_trip_and_registry(tmp_path):
    cfg = _cfg()
    d = Z.to_config_dict(cfg)
    assert from_hf_dict(json.loads(json.dumps(d))).layers == cfg.layers
    (tmp_path / "config.json").write_text(json.dumps(d))
    got = resolve_config(str(tmp_path))
    assert got.family == "gigezen" and got.n_layers == 5 and got.hidden == 96 and got.vocab == 130
    assert [L.mixer.kv_from for L in got.layers] == [None, 0, None, 2, None]
    assert isinstance(got.layers[2].mlp, Z.MoESpec) and isinstance(got.layers[0].mlp, Z.GatedMLPSpec)
    assert resolve_config("tiny-gigezen").family == "gigezen" and resolve_config("tiny-llama").family == "llama"


def test_config_rejects_what_cannot_run():
    d = Z.to_config_dict(_cfg())
    bad = json.loads(json.dumps(d))
    bad["layers"][1]["mixer"]["kv_from"] = 1
    with pytest.raises(ValueError):
        from_hf_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][1]["mixer"]["kv_rank"] = 24            # differs from the layer whose cache it reads
    with pytest.raises(ValueError):
        from_hf_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][2]["mlp"]["router"]["top"] = 5         # more than the kept groups hold
    with pytest.raises(ValueError):
        from_hf_dict(bad)
    bad = json.loads(json.dumps(d))
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ValueError):
        from_hf_dict(bad)


def test_cache_layout_and_span_checks():
    cfg = _cfg()
    assert cfg.cache_layers() == [0, 2, 4] and cfg.cache_row() == 64
    mgr = KVCacheManager.for_span(cfg, 0, 5, torch.float32, "cpu", default_max_length=32)
    kv = mgr.allocate("s", 32)
    assert tuple(kv.data.shape) == (3, 1, 1, 32, 64) and tuple(kv.rows(1).shape) == (32, 64)
    assert mgr.bytes_per_token() == 3 * 64 * 4
    kv.rows(2)[5, 3] = 1.0
    assert float(kv.data[2, 0, 0, 5, 3]) == 1.0
    cfg.check_span(0, 2)
    cfg.check_span(2, 5)
    with pytest.raises(ValueError):
        cfg.check_span(1, 3)                             # layer 1 reads layer 0's cache
    llama = KVCacheManager.for_span(resolve_config("tiny-llama"), 1, 3, torch.float16, "cpu")
    assert tuple(llama.allocate("t", 16).data.shape) == (2, 2, 2, 16, 128)


def test_tensor_names_and_random_weights():
    cfg = _cfg()
    shapes = Z.tensor_shapes(cfg)
    assert shapes["l1.mix.q"] == (3 * 12, 96) and "l1.mix.dkv" not in shapes and shapes["l0.mix.dkv"] == (24, 96)
    assert shapes["l2.mlp.e5.down"] == (96, 16) and shapes["l2.mlp.router"] == (6, 96) and shapes["head"] == (130, 96)
    w = load_span("x", cfg, 0, 5, need_embed=True, need_head=True, dtype=torch.float32, device="cpu", src=RandomSource(cfg, 1))
    assert tuple(w["layers"][2]["e_gate"].shape) == (6, 16, 96) and "dkv_w" not in w["layers"][3]
    assert w["layers"][0]["norm1_w"].dtype == torch.float32 and tuple(w["lm_head"].shape) == (130, 96)
    again = RandomSource(cfg, 1).get("l0.mix.q")
    assert torch.equal(again, RandomSource(cfg, 1).get("l0.mix.q")) and not torch.equal(again, RandomSource(cfg, 2).get("l0.mix.q"))


def test_oracle_prefix_property_and_window():
    """The oracle's logits at a position depend on the tokens up to it only, and a token outside every window of a
    layer stack stops mattering."""
    cfg = Z.make_config(n_layers=2, hidden=32, vocab=50, heads=2, dim=4, rot_dim=4, vdim=4, kv_rank=8, window=3, ff=16,
                        experts=4, top=2, groups=2, keep=1, expert_ff=8, share_every=0)
    d = Z.to_config_dict(cfg)
    src = RandomSource(cfg, 3)
    w = {k: src.get(k) for k in Z.tensor_shapes(cfg)}
    toks = [3, 9, 27, 31, 4, 18, 44, 2, 7]
    full = O.forward(d, w, toks)
    assert torch.allclose(O.forward(d, w, toks[:5]), full[:5], atol=1e-12)
    other = O.forward(d, w, [11] + toks[1:])
    # two layers of window 3: position i sees the first token through at most 2 * (3 - 1) steps
    assert not torch.allclose(other[4], full[4], atol=1e-9) and torch.allclose(other[5:], full[5:], atol=1e-12)
    assert O.window_visible(5, 3, 3) and not O.window_visible(5, 2, 3) and not O.window_visible(3, 5, 3)


def test_oracle_router_keeps_to_the_best_groups():
    h = torch.eye(6, dtype=torch.float64)
    wr = torch.tensor([[5.0, 0, 0, 0, 0, 0], [0, 0, 0, 0, 0, 0], [4.0, 0, 0, 0, 0, 0], [3.9, 0, 0, 0, 0, 0],
                       [4.5, 0, 0, 0, 0, 0], [0, 0, 0, 0, 0, 0]], dtype=torch.float64)
    ids, wts, s = O.route(h[:1], wr, {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}})
    assert ids.tolist() == [[0, 1]]                      # expert 4 scores higher than expert 1 but its group is not kept
    assert abs(float(wts.sum()) - float(s[0, 0] + s[0, 1])) < 1e-12 and float(wts.sum()) < 1.0
