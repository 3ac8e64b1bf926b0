"""Teacher-forced replay of a trace: given token ids go through the model step by step, nothing is sampled.

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

``entries``: per request its next tokens and the places among them whose logits are wanted; ``end``: requests whose
cache is released after the step.  For a step with wanted places ``<out>/<step>.f32`` receives the logits
``[wanted, vocab]`` as little-endian fp32 in entry / want order; every step is answered with a ``done <step>`` line.

The replay drives the same objects as generation: the in-box engine (``PipelineEngine`` on one GPU) with its cache
manager and its span - a request's first tokens run as a (chunked) prefill of its session, requests that go on by one
token run together as one batched decode step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, List

EXIT_UNSUPPORTED_DTYPE = 3


def _ensure_library(cfg) -> None:
    """Compile, on the first call in a fresh checkout, the kernels this model's family launches."""
    from petals_b200.ops import native

    if native.available():
        return
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, os.path.join(root, "csrc"))
    import build as csrc_build

    unit_set = "layered" if getattr(cfg, "layer_list", False) else None
    native.LIB_PATH = csrc_build.build(unit_set=unit_set)


class TraceReplayer:
    def __init__(self, model: str, dtype, max_tokens: int, device=None):
        import torch

        from petals_b200.models.config import resolve_config
        from petals_b200.runtime.layered_span import span_runs_natively
        from petals_b200.runtime.native_span import MAX_DECODE_BATCH

        self.torch = torch
        self.cfg = resolve_config(model)
        if not torch.cuda.is_available():
            raise RuntimeError("the replay runs the CUDA path: no GPU is visible")
        self.device = torch.device(device or "cuda:0")
        torch.cuda.set_device(self.device)
        if not span_runs_natively(self.cfg, self.device, dtype):
            raise NotImplementedError(f"{self.cfg.family} has no {dtype} span")
        _ensure_library(self.cfg)
        from petals_b200.parallel.pipeline import PipelineEngine

        cap = max(64, (int(max_tokens) + 1 + 63) // 64 * 64)       # (+ 1: a family may keep one row of its planes for itself)
        self.eng = PipelineEngine(model, (), dtype, self.device, kv_capacity=cap, max_sessions=MAX_DECODE_BATCH,
                                  max_chunk=512, cfg=self.cfg)
        self.span, self.kv = self.eng.span, self.eng.kv
        self.capacity = cap

    def _session(self, rid: str):
        s = self.kv.get(rid)
        return s if s is not None else self.kv.allocate(rid, self.capacity)

    def step(self, entries: List[dict], end: List[str]):
        """-> fp32 tensor [wanted, vocab] on the host (None when nothing is wanted)."""
        torch = self.torch
        outs: Dict[int, torch.Tensor] = {}
        single = []
        for n, e in enumerate(entries):
            kv = self._session(e["id"])
            toks = torch.tensor(e["tokens"], dtype=torch.int64, device=self.device)
            if len(e["tokens"]) == 1 and kv.length > 0:
                single.append((n, kv, toks))
                continue
            if not hasattr(self.span, "hidden_dtype") and [int(w) for w in e["want"]] not in ([], [len(e["tokens"]) - 1]):
                raise NotImplementedError("this family's prefill reports the last position's logits only")
            if e["want"]:
                lg = self.span.prefill(kv, ids=toks, logits_at=e["want"])[0] if hasattr(self.span, "hidden_dtype") \
                    else self.span.prefill(kv, ids=toks)[0].clone()
                outs[n] = lg
            else:
                self.span.prefill(kv, ids=toks)
        mb = self.span.max_batch
        for c0 in range(0, len(single), mb):          # requests that go on by one token: one batched decode step
            part = single[c0:c0 + mb]
            logits, _ = self.span.decode([kv for _, kv, _ in part], ids=torch.cat([t for _, _, t in part]))
            for b, (n, _, _) in enumerate(part):
                if entries[n]["want"]:
                    outs[n] = logits[b:b + 1].clone()
        for rid in end:
            self.kv.close(rid)
        rows = [outs[n] for n in range(len(entries)) if n in outs]
        return torch.cat(rows, 0).float().cpu() if rows else None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32", "float16"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, default=4096, help="most tokens live requests hold at any time")
    a = ap.parse_args(argv)
    import torch

    try:
        rp = TraceReplayer(a.model, getattr(torch, a.dtype), a.max_tokens)
    except NotImplementedError as e:
        print(f"trace_run: {e}", file=sys.stderr)
        return EXIT_UNSUPPORTED_DTYPE
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        res = rp.step(st.get("entries", []), st.get("end", []))
        if res is not None:
            tmp = os.path.join(a.out, f".{st['step']}.f32.part")
            res.contiguous().numpy().astype("<f4").tofile(tmp)
            os.replace(tmp, os.path.join(a.out, f"{st['step']}.f32"))
        sys.stdout.write(f"done {st['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
