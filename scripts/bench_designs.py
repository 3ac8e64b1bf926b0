"""Prefill and decode throughput of the layer-list designs (Gigezen, Seledra) beside the closest uniform family (Llama) at
equal layer sizes, random weights, one GPU.  Run as ``python bench.py --designs [--design-sizes small,7b] [--design-only X]``.

Per size: the models get the same width, head count, query/key width per head (Gigezen: unrotated + rotated), dense
feed-forward width, layer count and vocabulary.  Seledra: attention and delta-rule layers alternate (attention, delta,
delta, attention), every layer with a feed-forward, as many key/value heads as query heads like the Llama beside it.  Timed with CUDA events on the launching stream after warm-up; a prefill
pass streams every weight of the span and more activations than the L2 holds at 2048 tokens; decode steps are graph
replays whose weights alone exceed the L2 from the "7b" size on (the "small" size is L2-resident and says so).
One JSON line per (size, design).
"""
from __future__ import annotations

import json
import statistics

SIZES = {
    #            hidden heads ff     layers window
    "small": dict(hidden=2048, heads=16, ff=5632, layers=4, window=1024),
    "7b": dict(hidden=4096, heads=32, ff=11008, layers=4, window=2048),
}
VOCAB = 32000


def _configs(s):
    from petals_b200.models.config import ModelConfig
    from petals_b200.models.gigezen import make_config
    from petals_b200.models.seledra import make_config as make_seledra

    llama = ModelConfig("llama", s["layers"], s["hidden"], s["heads"], s["heads"], 128, s["ff"], VOCAB, name="llama-like")
    gz = make_config(n_layers=s["layers"], hidden=s["hidden"], vocab=VOCAB, heads=s["heads"], dim=64, rot_dim=64, vdim=128,
                     kv_rank=512, window=s["window"], ff=s["ff"], experts=8, top=2, groups=4, keep=2,
                     expert_ff=s["ff"] // 4 // 64 * 64, share_every=2, moe_every=2, limit=7.0, name="gigezen-like")
    sd = make_seledra("ADDA"[:s["layers"]] if s["layers"] <= 4 else "ADDA" * (s["layers"] // 4), hidden=s["hidden"], vocab=VOCAB,
                      heads=s["heads"], kv_heads=s["heads"], dim=128, vdim=128, delta_heads=s["heads"], delta_kv_heads=s["heads"],
                      delta_dim=128, delta_vdim=128, conv=4, ff=s["ff"], v_mix=True, residual_mult=0.5, max_positions=8192,
                      name="seledra-like")
    return {"llama": llama, "gigezen": gz, "seledra": sd}


def _time(fn, reps, warm=3):
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def run(args):
    import torch

    from petals_b200.runtime.kv_cache import KVCacheManager
    from petals_b200.runtime.layered_span import make_span
    from petals_b200.weights.loader import load_span

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    dt = torch.bfloat16
    only = set(args.design_only.split(",")) if args.design_only else None
    for size in args.design_sizes.split(","):
        s = SIZES[size]
        for design, cfg in _configs(s).items():
            if only and design not in only:
                continue
            cap = 4096
            w = load_span("random:" + design, cfg, 0, cfg.n_layers, need_embed=True, need_head=True, dtype=dt, device=dev, seed=1)
            span = make_span(cfg, w, dev, dt, kv_capacity=cap, max_batch=16, max_chunk=2048)
            mgr = KVCacheManager.for_span(cfg, 0, cfg.n_layers, dt, dev, default_max_length=cap)
            kvs = [mgr.allocate(f"s{i}", cap) for i in range(16)]
            g = torch.Generator().manual_seed(5)
            res = {"design": design, "size": size, "dtype": "bf16", "layers": cfg.n_layers, "hidden": cfg.hidden,
                   "weight_mb": round(span.weight_bytes() / 2 ** 20, 1), "data": "synthetic tokens, random-init weights"}
            for T in (512, 2048):
                ids = torch.randint(0, VOCAB, (T,), generator=g).to(dev)

                def pre():
                    kvs[0].length = 0
                    span.prefill(kvs[0], ids=ids)

                ms = _time(pre, 5)
                res[f"prefill_{T}_ms"] = round(ms, 3)
                res[f"prefill_{T}_tok_s"] = round(T / ms * 1e3, 1)
            ctx = torch.randint(0, VOCAB, (1024,), generator=g).to(dev)
            for B in (1, 16):
                for kv in kvs[:B]:
                    kv.length = 0
                    span.prefill(kv, ids=ctx)
                tok = torch.randint(0, VOCAB, (B,), generator=g).to(dev)
                steps = 32

                def dec():
                    for kv in kvs[:B]:
                        kv.length = 1024
                    for _ in range(steps):
                        span.decode(kvs[:B], ids=tok)

                ms = _time(dec, 3, warm=2) / steps
                res[f"decode_b{B}_ctx1024_ms_per_step"] = round(ms, 4)
                res[f"decode_b{B}_ctx1024_tok_s"] = round(B / ms * 1e3, 1)
            res["gpu_launches"] = span.kernel_launches
            print(json.dumps(res), flush=True)
            del span, w, mgr, kvs
            torch.cuda.empty_cache()
