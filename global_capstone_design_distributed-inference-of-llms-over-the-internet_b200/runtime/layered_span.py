"""B200 execution of a span of a layer-list design (Gigezen, Seledra) with an fp32 residual stream.

``LayeredSpan`` plugs into everything a :class:`NativeSpan` plugs into - sessions of the cache manager, the
captured decode step with its staged positions / cache pointers, the device sampler, the pipeline engine and the
served stages - and replaces what is specific to the uniform families: the weights it packs, the kernels of a layer
and the head.  Per layer (T tokens of any mix of sessions):

    hn    = rms_norm(x += previous layer's outputs) * (1 + g)        b200_add_rms_norm      fp32 -> 16-bit
    proj  = hn . [Wq | Wdkv | Wrouter | Wgate | Wup]^T               tcgen05 GEMM, fp32 out (one launch)
    rotary on q / shared key part, latent norm, cache append         b200_latent_rope_append
    q_abs = q_unrotated pulled through W_uk, per head                b200_gemm_simt (batched over heads)
    o_lat = softmax(window scores) . latents                         b200_latent_attn
    cat   = [ W_uv o_lat per head | clamped gated unit ]             b200_gemm_simt (batched) + b200_glu_clamp
    y     = cat . [Wo | Wdown]^T                                     tcgen05 GEMM, fp32 out: mixer + dense ff in one
    experts (mixture layers): route, plan, grouped gate/up and down  b200_moe_* + b200_gemm_simt (grouped)

A design whose layers update the stream in two steps (Seledra: ``x += m mixer(norm1 x)``, ``x += m ff(norm2 x)``) runs

    hn    = rms_norm(x += m * previous sublayer's output) * g         b200_add_rms_norm
    proj  = hn . [Wq | Wk | Wv | Wgate]^T  (attention)                tcgen05 GEMM, fp32 out (one launch)
            hn . [Wq | Wk | Wv | Wbeta | Wdecay | Wgate]^T  (delta)
    attention: norms, value blending, cache append                   b200_sink_attn_append
               softmax with a sink over the cached rows, head gate    b200_sink_attn / b200_sink_attn_prefill
    delta:     convolutions, unit q / k, beta, decay                  b200_delta_prep
               the recurrence over the session's state                b200_delta_rule
               gated RMS norm per head                                b200_gated_head_norm
    y     = heads . Wo^T                                              tcgen05 GEMM, fp32 out
    feed-forward: norm (as above), up GEMM, b200_xielu, down GEMM

``dtype=torch.float32`` runs the same step with every product in true fp32 (``b200_gemm_simt`` instead of the
tensor-core GEMM) and an fp32 cache.
"""
from __future__ import annotations

import os
from typing import Dict, List, Optional, Sequence

import torch

from ..models import gigezen as Z
from ..models import seledra as SD
from ..ops import elementwise as E
from ..ops import gemm as G
from ..ops import layered as L
from ..ops import packing
from .kv_cache import SessionKV
from .native_span import MAX_DECODE_BATCH, NativeSpan, _pdl_default


# Mixtures whose experts / top ratio is at most this run their experts densely on the tensor cores (16-bit modes).
DENSE_EXPERTS_MAX_RATIO = int(os.environ.get("B200_DENSE_EXPERTS_MAX_RATIO", "16"))


ATTN_MAX_SPLITS = 16
# Chunks of one session with at least this many tokens run their attention on the tensor cores (16-bit modes).
TC_ATTN_MIN_TOKENS = int(os.environ.get("B200_LATENT_TC_MIN_TOKENS", "33"))


def _pad64(n: int) -> int:
    return (n + 63) // 64 * 64


class _Linear:
    """One weight in the form the span's mode multiplies with: packed tiles (16-bit) or the dense fp32 matrix."""

    def __init__(self, w: torch.Tensor, exact: bool):
        self.n, self.k = w.shape
        self.k_padded = self.k if exact else _pad64(self.k)
        self.dense = w.contiguous() if exact else None
        self.packed = None if exact else packing.pack_weight(w)
        self.nbytes = w.numel() * w.element_size()


class LayeredSpan(NativeSpan):
    hidden_dtype = torch.float32        # what enters and leaves the span between pipeline stages

    def __init__(self, cfg, weights: Dict[str, object], device, dtype: torch.dtype, *,
                 kv_capacity: int = 2048, max_batch: int = 8, max_chunk: int = 512, use_graphs: bool = True,
                 pdl: Optional[bool] = None, free_source_weights: bool = True, weight_format: str = "native",
                 head_rows: Optional[tuple] = None, attn_splits: int = 0, streamed_layers: int = 0):
        if dtype not in (torch.bfloat16, torch.float16, torch.float32):
            raise ValueError("a layered span runs in bfloat16 / float16 (tensor-core products) or float32 (all fp32)")
        if weight_format != "native" or head_rows is not None or streamed_layers:
            raise NotImplementedError("layered spans: 16-bit or fp32 weights, whole head, resident layers")
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.exact = dtype == torch.float32
        self.kv_capacity, self.max_batch, self.max_chunk = kv_capacity, min(max_batch, MAX_DECODE_BATCH), max_chunk
        self.use_graphs = use_graphs
        self.weight_format = "native"
        self.pdl = _pdl_default() if pdl is None else pdl
        self.l2_prefetch_mb = None
        self.streamed_layers = 0
        self._prefill_plans = {}
        self.has_embed = bool(weights.get("has_embed", False))
        self.has_head = bool(weights.get("has_head", "lm_head" in weights))
        self.start = int(weights.get("start", 0))
        W = cfg.hidden
        ex = self.exact
        specs = cfg.layers[self.start:self.start + len(weights["layers"])]    # type: ignore[arg-type]
        cfg.check_span(self.start, self.start + len(specs))
        slots = {a: s for s, a in enumerate(cfg.cache_layers(self.start, self.start + len(specs)))}
        self.n_slots = max(1, len(slots))
        self.row_elems = cfg.cache_row(self.start, self.start + len(specs))
        self.cache_planes = cfg.cache_planes
        # recurrent layers: a session carries fp32 state; its address travels in one more row of the pointer table
        self.state_elems = cfg.state_elems(self.start, self.start + len(specs))
        self.state_slot = self.n_slots if self.state_elems else None
        state_off = cfg.state_offsets(self.start, self.start + len(specs)) if self.state_elems else {}
        # Attention with a sink keeps row 0 of its planes at zero and stores position p in row p + 1: a key of score 0
        # without a value IS the sink, so a plain causal softmax over rows 0 .. p + 1 (the tcgen05 kernel of the uniform
        # families) gives the same weights; this span's own kernels get the planes from row 1 on and start their
        # running sums at the sink instead.  A session therefore holds one token less than its rows.
        self.sink_row = 1 if any(isinstance(S.mixer, SD.SinkAttentionSpec) for S in specs) else 0
        self.gain_offset = float(cfg.norm_gain_offset)
        self.residual_mult = float(cfg.residual_mult)
        with torch.cuda.device(self.device):
            self.layers: List[dict] = []
            self._inv_freq: Dict[tuple, torch.Tensor] = {}
            for i, (S, Lw) in enumerate(zip(specs, weights["layers"])):   # type: ignore[arg-type]
                m = S.mixer
                if isinstance(m, (SD.SinkAttentionSpec, SD.DeltaRuleSpec)):
                    self.layers.append(self._pack_two_step_layer(S, Lw, slots.get(self.start + i),
                                                                 state_off.get(self.start + i, 0), self.start + i,
                                                                 free_source_weights))
                    continue
                parts, P = [Lw["q_w"]], {"spec": S, "norm_w": Lw["norm1_w"], "q_off": 0, "kv_off": -1}
                n = m.q_size
                if m.owns_cache:
                    P["kv_off"], P["c_gain"] = n, Lw["dkv_norm_w"]
                    parts.append(Lw["dkv_w"])
                    n += m.row
                P["slot"] = slots[self.start + i if m.owns_cache else m.kv_from]
                if isinstance(S.mlp, Z.MoESpec):
                    P["r_off"] = n
                    parts.append(Lw["router_w"])
                    n += S.mlp.experts
                    e = S.mlp
                    if not ex and e.experts <= DENSE_EXPERTS_MAX_RATIO * e.top:
                        # tensor-core form: ALL experts as one gate/up GEMM (fused gated unit) and one down GEMM over the
                        # concatenated experts, the routing weights (0 = not chosen) applied in between.  experts / top
                        # times the FLOPs of the chosen experts alone, on a GEMM that is ~30 times faster than the grouped
                        # CUDA-core one; a decode step streams every expert once, which a batch of a few tokens does anyway.
                        P["e_in"] = packing.pack_dual(Lw["e_gate"].reshape(e.experts * e.ff, W), Lw["e_up"].reshape(e.experts * e.ff, W))
                        P["e_out"] = _Linear(Lw["e_down"].permute(1, 0, 2).reshape(W, e.experts * e.ff), ex)
                    else:
                        P["e_gate"], P["e_up"], P["e_down"] = Lw["e_gate"], Lw["e_up"], Lw["e_down"]
                elif isinstance(S.mlp, Z.GatedMLPSpec):
                    P["g_off"], P["u_off"] = n, n + S.mlp.ff
                    parts += [Lw["gate_w"], Lw["up_w"]]
                    n += 2 * S.mlp.ff
                P["proj"] = _Linear(torch.cat(parts, 0), ex)
                hv = m.heads * m.vdim
                dense = isinstance(S.mlp, Z.GatedMLPSpec)
                P["out"] = _Linear(torch.cat([Lw["o_w"], Lw["down_w"]], 1) if dense else Lw["o_w"], ex)
                if not ex:      # prompt-size chunks expand the visible latents into per-head keys and values with one GEMM
                    P["kvx_w"] = _Linear(torch.cat([Lw["uk_w"], Lw["uv_w"]], 0), ex)
                P["ukT"] = Lw["uk_w"].view(m.heads, m.dim, m.kv_rank).transpose(1, 2).contiguous()     # [H, R, dim]
                P["uv"] = Lw["uv_w"].view(m.heads, m.vdim, m.kv_rank).contiguous()                     # [H, vdim, R]
                key = (m.rope_base, m.rope_dims)
                if key not in self._inv_freq:
                    j = torch.arange(m.rope_dims // 2, dtype=torch.float64)
                    self._inv_freq[key] = (torch.tensor(m.rope_base, dtype=torch.float64) ** (-2.0 * j / m.rope_dims)).to(self.device)
                P["inv_freq"] = self._inv_freq[key]
                P["hv"] = hv
                self.layers.append(P)
                if free_source_weights:
                    for k in ("q_w", "dkv_w", "router_w", "gate_w", "up_w", "o_w", "down_w", "uk_w") + \
                            (("e_gate", "e_up", "e_down") if "e_in" in P else ()):
                        Lw.pop(k, None)
            self.embed_w = weights.get("embed") if self.has_embed else None
            self.pos_embed_w = weights.get("pos_embed") if self.has_embed else None
            self.head_lo, self.head_hi = 0, cfg.vocab
            if self.has_head:
                self.final_norm_w = weights["final_norm_w"]
                self.lm_head = _Linear(weights["lm_head"], ex)       # type: ignore[arg-type]
            Tm = max(self.max_chunk, self.max_batch)
            adt = dtype                                             # element type of GEMM inputs
            f32 = lambda *s: torch.zeros(*s, dtype=torch.float32, device=self.device)  # noqa: E731
            act = lambda *s: torch.zeros(*s, dtype=adt, device=self.device)  # noqa: E731
            mx = lambda f: max([f(P) for P in self.layers] or [1])  # noqa: E731
            self.h_a = f32(Tm, W)
            self.h_b = self.h_a                                      # (one stream buffer: layers update it in place)
            self.hn = act(Tm, _pad64(W))
            self.proj = f32(Tm, mx(lambda P: max(P["proj"].n, P["up"].n if "up" in P else 0)))
            latent = lambda P: isinstance(P["spec"].mixer, Z.LatentAttentionSpec)  # noqa: E731
            self.qa = f32(Tm, mx(lambda P: P["spec"].mixer.heads * P["spec"].mixer.kv_rank if latent(P) else 1))
            self.ol = torch.zeros_like(self.qa)
            self.cat = act(Tm, mx(lambda P: _pad64(max(P["out"].k, P["down"].k if "down" in P else 0))))
            self.y = f32(Tm, W)
            self.attn_part = f32(MAX_DECODE_BATCH * ATTN_MAX_SPLITS *
                                 mx(lambda P: P["spec"].mixer.heads * ((P["spec"].mixer.kv_rank if latent(P) else
                                                                        getattr(P["spec"].mixer, "vdim", 0)) + 2)))
            deltas = [P["spec"].mixer for P in self.layers if isinstance(P["spec"].mixer, SD.DeltaRuleSpec)]
            if deltas:     # what the recurrence reads (q | k | v | beta | decay | k.q) and its raw read-out, fp32
                self.delta_work = f32(Tm, max((d.conv_channels + 2 * d.heads + d.kv_heads + 3) // 4 * 4 for d in deltas))
                self.delta_o = f32(Tm, max(d.v_size for d in deltas))
            vm = [P["spec"].mixer for P in self.layers if getattr(P["spec"].mixer, "v_mix", False)]
            self.v_first = f32(Tm, max(v.v_size for v in vm)) if vm else None
            tcq = [P["spec"].mixer for P in self.layers if isinstance(P["spec"].mixer, SD.SinkAttentionSpec) and not ex
                   and L.attn_prefill_rows_fits(P["spec"].mixer.dim, P["spec"].mixer.vdim, self.row_elems)]
            self.q16 = act(Tm, max(q.q_size for q in tcq)) if tcq else None      # queries for the TMA-fed attention kernel
            moe = [P["spec"].mlp for P in self.layers if isinstance(P["spec"].mlp, Z.MoESpec)]
            if moe:
                top, ne, ffe = max(e.top for e in moe), max(e.experts for e in moe), max(e.ff for e in moe)
                self.moe_ids = torch.zeros(Tm, top, dtype=torch.int32, device=self.device)
                self.moe_w = f32(Tm, top)
                self.moe_off = torch.zeros(ne + 1, dtype=torch.int32, device=self.device)
                self.moe_row_pair = torch.zeros(Tm * top, dtype=torch.int32, device=self.device)
                self.moe_row_token = torch.zeros(Tm * top, dtype=torch.int32, device=self.device)
                self.moe_act = f32(Tm * top, ffe) if any("e_gate" in P for P in self.layers) else None
                self.moe_y = f32(Tm * top, W) if self.moe_act is not None else f32(Tm, W)
                wide = [P["e_out"].k_padded for P in self.layers if "e_out" in P]
                self.moe_act_all = act(Tm, max(wide)) if wide else None
            self.ids_in = torch.zeros(Tm, dtype=torch.int64, device=self.device)
            # expanded keys / values of the rows a chunk can see (16-bit modes, allocated with the first such chunk)
            self.kvx = None
            self.kvx_rows = Tm + min(mx(lambda P: getattr(P["spec"].mixer, "window", 1) - 1), self.kv_capacity)
            self.ws = None if ex else G.GemmWorkspace.create(self.device, max(Tm, min(self.kvx_rows, 256)))
            self._make_stage_buffers(self._cache_slots())
            self.sampler = None
            self._seq_host = 0
            self.chain_tokens = 0
            self._ptr_tables = {}
            if self.has_head:
                self.head_rows_max = min(max(self.max_batch, 32), Tm)      # rows per head call (they pass through hn)
                self.logits = f32(self.head_rows_max, cfg.vocab)
                self.ids_out = torch.zeros(self.head_rows_max, dtype=torch.int64, device=self.device)
                self.argmax_ws = E.ArgmaxWorkspace(self.device, self.head_rows_max)
        self._graphs = {}
        self._ptr_key = None
        self.kernel_launches = 0
        self._launches_per_graph = {}
        self._pending = None

    # ------------------------------------------------------------------ framework hooks
    def _cache_slots(self) -> int:
        return self.n_slots + (1 if self.state_elems else 0)

    def _ptr_column(self, kv: SessionKV, nl: int) -> torch.Tensor:
        col = super()._ptr_column(kv, nl)
        if self.sink_row:             # this span's decode kernels see the planes from row 1 on (row 0 is the sink's)
            col[:self.n_slots] += self.sink_row * self.row_elems * kv.data.element_size()
        if self.state_elems:          # last row: where the session's recurrent state lives
            if kv.state is None or kv.state.numel() < self.state_elems:
                raise ValueError(f"session {kv.session_id} carries no state for this span's recurrent layers")
            col[self.state_slot, 0] = kv.state.data_ptr()
            col[self.state_slot, 1] = 0
        return col

    def _pack_two_step_layer(self, S, Lw: dict, slot: Optional[int], state_off: int, index: int, free: bool) -> dict:
        """Weights of a layer that updates the stream in two steps (mixer, then feed-forward), in the span's mode."""
        ex, m = self.exact, S.mixer
        P = {"spec": S, "norm_w": Lw["norm1_w"], "slot": slot, "state_off": state_off, "hv": m.heads * m.vdim}
        if isinstance(m, SD.SinkAttentionSpec):
            P["proj"] = _Linear(torch.cat([Lw["q_w"], Lw["k_w"], Lw["v_w"], Lw["g_w"]], 0), ex)
            P["q_off"], P["k_off"], P["v_off"], P["g_off"] = 0, m.q_size, m.q_size + m.k_size, m.q_size + m.k_size + m.v_size
            for k in ("qkv_b", "q_norm_w", "k_norm_w", "temp", "vmix"):
                P[k] = Lw[k]
            P["vmix_mode"] = 0 if not m.v_mix else (1 if index == self.cfg.first_vmix_layer() else 2)
        else:
            P["proj"] = _Linear(torch.cat([Lw["q_w"], Lw["k_w"], Lw["v_w"], Lw["b_w"], Lw["a_w"], Lw["g_w"]], 0), ex)
            P["c_off"], P["b_off"], P["a_off"] = 0, m.conv_channels, m.conv_channels + m.heads
            P["g_off"] = m.conv_channels + 2 * m.heads
            for k in ("conv_w", "A_log", "dt_bias", "o_norm_w"):
                P[k] = Lw[k]
        P["out"] = _Linear(Lw["o_w"], ex)
        if S.mlp is not None:
            P["norm2_w"], P["act"] = Lw["norm2_w"], Lw["act"]
            P["up"], P["down"] = _Linear(Lw["up_w"], ex), _Linear(Lw["down_w"], ex)
        if free:
            for k in ("q_w", "k_w", "v_w", "g_w", "b_w", "a_w", "o_w", "up_w", "down_w"):
                Lw.pop(k, None)
        return P

    def subspan(self, a: int, b: int):
        if (a, b) == (0, len(self.layers)):
            return self
        raise NotImplementedError("sub-spans of a layered span (cache slots are shared between its layers)")

    def weight_bytes(self) -> int:
        n = 0
        for P in self.layers:
            n += P["proj"].nbytes + P["out"].nbytes + sum(P[k].numel() * P[k].element_size() for k in ("ukT", "uv") if k in P)
            n += sum(P[k].nbytes for k in ("up", "down") if k in P)
            if "e_gate" in P:
                n += sum(P[k].numel() * P[k].element_size() for k in ("e_gate", "e_up", "e_down"))
            if "e_in" in P:
                n += P["e_in"].nbytes + P["e_out"].nbytes
        if self.has_head:
            n += self.lm_head.nbytes
        return n

    # ------------------------------------------------------------------ pieces
    def _linear(self, x: torch.Tensor, w: _Linear, out: torch.Tensor) -> torch.Tensor:
        """out (fp32 [T, >= n] view) = x[:, :k] . W^T"""
        T = x.shape[0]
        if self.exact:
            L.gemm_simt(x, w.dense, out, T=T, N=w.n, K=w.k, pdl=self.pdl)
        else:
            G.linear(x[:, :w.k_padded], w.packed, out=out[:, :w.n], out_fp32=True, workspace=self.ws, pdl=self.pdl)
        self._count()
        return out

    def _embed(self, T: int, pos0: int, use_pos_buffer: bool) -> torch.Tensor:
        h = self.h_a[:T]
        if self.pos_embed_w is not None:      # learned positions, added in fp32
            L.embed_pos_f32(self.ids_in[:T], self.embed_w, self.pos_embed_w, h, pos=self.pos[:T] if use_pos_buffer else None,
                            pos0=pos0, pdl=self.pdl)
        else:
            L.embed_f32(self.ids_in[:T], self.embed_w, h, pdl=self.pdl)
        self._count()
        return h

    def _flush(self, x: torch.Tensor, gain: Optional[torch.Tensor], out: Optional[torch.Tensor]) -> None:
        """Adds what the previous layer left pending to the stream and (optionally) norms the result."""
        pend, self._pending = self._pending or {}, None
        if not pend and out is None:
            return
        L.add_rms_norm(x, gain, out, self.cfg.norm_eps, self.gain_offset, add_scale=self.residual_mult, pdl=self.pdl, **pend)
        self._count()

    def _attn_splits(self, T: int, m) -> tuple:
        """Decode-size steps divide every token's window over several blocks (tokens x head groups alone leave most SMs
        idle); the split depends on the window and the step's size only, so a captured step keeps it."""
        if T > MAX_DECODE_BATCH:
            return 1, None
        keys = min(m.window, self.kv_capacity)
        blocks = T * ((m.heads + 7) // 8)
        splits = max(1, min(ATTN_MAX_SPLITS, keys // 64, (4 * 148) // blocks))
        return (splits, self.attn_part) if splits > 1 else (1, None)

    def _layer(self, T: int, x: torch.Tensor, P: dict, where: dict) -> None:
        S, pdl = P["spec"], self.pdl
        m = S.mixer
        if not isinstance(m, Z.LatentAttentionSpec):
            return self._layer_two_step(T, x, P, where)
        W = self.cfg.hidden
        hn, proj, cat = self.hn[:T], self.proj[:T], self.cat[:T]
        self._flush(x, P["norm_w"], hn[:, :W])
        self._linear(hn, P["proj"], proj)
        common = dict(heads=m.heads, dim=m.dim, rot=m.rot_dim, rot_dims=m.rope_dims, kv_rank=m.kv_rank,
                      row_elems=self.row_elems, cache_dtype=self.dtype, eps=self.cfg.norm_eps, T=T, pdl=pdl)
        if "kv" in where:      # one session: rows of its cache slot, consecutive positions
            common.update(cache=where["kv"].rows(P["slot"]), pos0=where["pos0"])
        else:                  # a batch of sessions: staged pointer table and positions
            common.update(kv_ptrs=self.kv_ptrs[P["slot"]], kv_ptr_stride=2, pos=self.pos)
        a = L.latent_args(proj, P["q_off"], P["kv_off"], P.get("c_gain"), P["inv_freq"], q_abs=self.qa, out=self.ol,
                          window=m.window, scale=m.scale, **common)
        a.ldqa = a.ldout = m.heads * m.kv_rank
        L.latent_rope_append(a)
        self._count()
        if "kv" in where and not self.exact and T >= TC_ATTN_MIN_TOKENS:
            self._attn_tensor_core(T, P, where, proj, cat)
        else:
            self._attn_latent(T, P, a, proj, cat)
        if isinstance(S.mlp, Z.GatedMLPSpec):
            ff = S.mlp.ff
            L.glu_clamp(proj[:, P["g_off"]:P["g_off"] + ff], proj[:, P["u_off"]:P["u_off"] + ff], cat[:, P["hv"]:],
                        S.mlp.limit, Z.DENSE_GATE_ALPHA, Z.DENSE_UP_SHIFT, pdl=pdl)
            self._count()
        self._linear(cat, P["out"], self.y[:T])
        self._pending = dict(add_a=self.y[:T])
        if isinstance(S.mlp, Z.MoESpec):
            self._experts(T, P, hn, proj)

    # ------------------------------------------------------------------ layers of two residual steps
    def _layer_two_step(self, T: int, x: torch.Tensor, P: dict, where: dict) -> None:
        S, pdl = P["spec"], self.pdl
        W = self.cfg.hidden
        hn, proj, cat = self.hn[:T], self.proj[:T], self.cat[:T]
        self._flush(x, P["norm_w"], hn[:, :W])
        self._linear(hn, P["proj"], proj)
        if isinstance(S.mixer, SD.SinkAttentionSpec):
            self._mixer_sink_attention(T, P, where, proj, cat)
        else:
            self._mixer_delta(T, P, where, proj, cat)
        self._linear(cat, P["out"], self.y[:T])
        self._pending = dict(add_a=self.y[:T])
        if S.mlp is not None:
            ff = S.mlp.ff
            self._flush(x, P["norm2_w"], hn[:, :W])
            self._linear(hn, P["up"], proj)
            L.xielu(proj[:, :ff], P["act"], cat, lin=SD.XIELU_LINEAR, neg_base=SD.XIELU_LINEAR, pdl=pdl)
            self._count()
            self._linear(cat, P["down"], self.y[:T])
            self._pending = dict(add_a=self.y[:T])

    def _sink_splits(self, T: int, m) -> tuple:
        """Decode-size steps divide every token's keys over several blocks; the split depends on the step's size and
        the sessions' capacity only, so a captured step keeps it."""
        if T > MAX_DECODE_BATCH:
            return 1, None
        splits = max(1, min(ATTN_MAX_SPLITS, self.kv_capacity // 128, (16 * 148) // (T * m.heads)))
        return (splits, self.attn_part) if splits > 1 else (1, None)

    def _mixer_sink_attention(self, T: int, P: dict, where: dict, proj: torch.Tensor, cat: torch.Tensor) -> None:
        m = P["spec"].mixer
        kw = dict(q_off=P["q_off"], k_off=P["k_off"], v_off=P["v_off"], g_off=P["g_off"], heads=m.heads, kv_heads=m.kv_heads,
                  dim=m.dim, vdim=m.vdim, row_elems=self.row_elems, cache_dtype=self.dtype, eps=self.cfg.norm_eps,
                  scale=m.scale, sink=m.sink, T=T, bias=P["qkv_b"], q_gain=P["q_norm_w"], k_gain=P["k_norm_w"], temp=P["temp"],
                  vmix=P["vmix"], v_first=self.v_first, vmix_mode=P["vmix_mode"], out=cat, pdl=self.pdl)
        portion = "kv" in where and not self.exact and T >= TC_ATTN_MIN_TOKENS
        tcgen05 = portion and self.q16 is not None and L.attn_prefill_rows_fits(m.dim, m.vdim, self.row_elems)
        if "kv" in where:      # one session: its planes (from the first token's row on), consecutive positions
            kv = where["kv"]
            kw.update(k_cache=kv.plane(P["slot"], 0)[self.sink_row:], v_cache=kv.plane(P["slot"], 1)[self.sink_row:],
                      pos0=where["pos0"])
        else:                  # a batch of sessions: staged pointer table and positions
            kw.update(kv_ptrs=self.kv_ptrs[P["slot"]], kv_ptr_stride=2, pos=self.pos)
        if tcgen05:
            kw.update(q16=self.q16[:T])
        a = L.sink_attn_args(proj, **kw)
        L.sink_attn_append(a)
        if tcgen05:            # equal key / value sizes of 64 or 128: the uniform families' kernel over rows 0 .. p + 1, then the gate
            L.attn_prefill_rows(self.q16[:T, :m.q_size], cat, kv.plane(P["slot"], 0), kv.plane(P["slot"], 1), heads=m.heads,
                                kv_heads=m.kv_heads, dim=m.dim, rows=kv.max_len, pos0=where["pos0"] + self.sink_row, scale=1.0,
                                pdl=self.pdl)
            L.head_gate(cat, proj[:, P["g_off"]:], m.heads, m.vdim, pdl=self.pdl)
            self._count()
        elif portion and L.sink_attn_prefill_fits(m.dim, m.vdim):
            L.sink_attn_prefill(a)
        else:
            L.sink_attn(a, *self._sink_splits(T, m))
        self._count(2)

    def _mixer_delta(self, T: int, P: dict, where: dict, proj: torch.Tensor, cat: torch.Tensor) -> None:
        m = P["spec"].mixer
        kw = dict(c_off=P["c_off"], b_off=P["b_off"], a_off=P["a_off"], conv_w=P["conv_w"], A_log=P["A_log"],
                  dt_bias=P["dt_bias"], work=self.delta_work[:T], o=self.delta_o[:T], heads=m.heads, kv_heads=m.kv_heads,
                  dim=m.dim, vdim=m.vdim, taps=m.conv, unit_eps=m.unit_eps, state_off=P["state_off"], pdl=self.pdl)
        if "kv" in where:      # a chunk of one session: its tokens in order
            kw.update(state=where["kv"].state, pos0=where["pos0"], n_seq=1, seq_len=T)
        else:                  # a batch of sessions, one token each
            kw.update(state_ptrs=self.kv_ptrs[self.state_slot], state_ptr_stride=2, pos=self.pos, n_seq=T, seq_len=1)
        a = L.delta_args(proj, **kw)
        L.delta_prep(a)
        L.delta_rule(a)
        L.gated_head_norm(self.delta_o[:T], proj[:, P["g_off"]:], P["o_norm_w"], cat, m.heads, m.vdim, self.cfg.norm_eps,
                          pdl=self.pdl)
        self._count(3)

    def _attn_tensor_core(self, T: int, P: dict, where: dict, proj: torch.Tensor, cat: torch.Tensor) -> None:
        """A chunk of one session: expand the visible latents with one tensor-core GEMM, then flash attention on them."""
        m = P["spec"].mixer
        kv, pos0 = where["kv"], where["pos0"]
        s0 = max(0, pos0 - m.window + 1)
        rows = pos0 + T - s0
        w = P["kvx_w"]
        if self.kvx is None:
            width = max(Q["kvx_w"].n for Q in self.layers)
            self.kvx = torch.zeros(self.kvx_rows, (width + 7) // 8 * 8, dtype=self.dtype, device=self.device)
        cache = kv.rows(P["slot"])
        G.linear(cache[s0:s0 + rows, :w.k_padded], w.packed, out=self.kvx[:rows, :w.n], workspace=self.ws, pdl=self.pdl)
        L.latent_attn_prefill(proj, P["q_off"], self.kvx, m.heads * m.dim, cache, m.kv_rank, cat, T=T, heads=m.heads,
                              dim=m.dim, rot=m.rot_dim, vdim=m.vdim, pos0=pos0, s0=s0, window=m.window, scale=m.scale,
                              pdl=self.pdl)
        self._count(2)

    def _attn_latent(self, T: int, P: dict, a, proj: torch.Tensor, cat: torch.Tensor) -> None:
        """Decode steps and the all-fp32 mode: queries pulled through W_uk, attention over the latents, W_uv after it."""
        m, pdl = P["spec"].mixer, self.pdl
        hd = m.dim + m.rot_dim
        L.gemm_simt(proj[:, P["q_off"]:], P["ukT"], self.qa, T=T, N=m.kv_rank, K=m.dim, ldx=proj.stride(0), ldw=m.dim,
                    ldo=m.heads * m.kv_rank, batch=m.heads, x_bs=hd, w_bs=m.kv_rank * m.dim, o_bs=m.kv_rank, pdl=pdl)
        L.latent_attn(a, *self._attn_splits(T, m))
        L.gemm_simt(self.ol, P["uv"], cat, T=T, N=m.vdim, K=m.kv_rank, ldx=m.heads * m.kv_rank, ldw=m.kv_rank,
                    ldo=cat.stride(0), batch=m.heads, x_bs=m.kv_rank, w_bs=m.vdim * m.kv_rank, o_bs=m.vdim, pdl=pdl)
        self._count(3)

    def _experts(self, T: int, P: dict, hn: torch.Tensor, proj: torch.Tensor) -> None:
        """Mixture of experts of a layer: route, then the experts densely on the tensor cores or grouped on the CUDA
        cores; leaves its output pending for the next residual update."""
        pdl, W = self.pdl, self.cfg.hidden
        e = P["spec"].mlp
        n = T * e.top
        ids, wts = self.moe_ids[:T, :e.top], self.moe_w[:T, :e.top]
        if e.top != self.moe_ids.shape[1]:
            ids, wts = self.moe_ids.view(-1)[:n].view(T, e.top), self.moe_w.view(-1)[:n].view(T, e.top)
        L.moe_route(proj[:, P["r_off"]:P["r_off"] + e.experts], e.experts, e.groups, e.keep, e.top, ids, wts, pdl=pdl)
        if "e_in" in P:
            act_all = self.moe_act_all[:T]
            G.linear(hn, P["e_in"], out=act_all[:, :e.experts * e.ff], epilogue=G.EPI_SWIGLU, workspace=self.ws, pdl=pdl)
            L.moe_scale(act_all, ids, wts, e.experts, e.ff, e.top, pdl=pdl)
            self._linear(act_all, P["e_out"], self.moe_y[:T])
            self._pending["add_b"] = self.moe_y[:T]
            self._count(3)
            return
        L.moe_plan(ids, T, e.top, e.experts, self.moe_off, self.moe_row_pair, self.moe_row_token, pdl=pdl)
        grouped = dict(group_off=self.moe_off, groups=e.experts, T=n, pdl=pdl)
        L.gemm_simt(hn, P["e_gate"], self.moe_act, w2=P["e_up"], N=e.ff, K=W, ldw=W, w_gs=e.ff * W,
                    row_src=self.moe_row_token, **grouped)
        L.gemm_simt(self.moe_act, P["e_down"], self.moe_y, N=W, K=e.ff, ldw=e.ff, w_gs=W * e.ff,
                    row_dst=self.moe_row_pair, **grouped)
        self._pending.update(pair_y=self.moe_y, pair_w=wts, top=e.top)
        self._count(4)

    def _run_layers(self, T: int, x: torch.Tensor, where: dict, norm_out: bool = False) -> torch.Tensor:
        self._pending = None
        for P in self.layers:
            self._layer(T, x, P, where)
        if norm_out and self.has_head:     # every row goes to the head: fold the final norm into the last update
            self._flush(x, self.final_norm_w, self.hn[:T, :self.cfg.hidden])
            self._normed = True
        else:
            self._flush(x, None, None)
            self._normed = False
        return x

    def _decode_layers(self, T: int, h: torch.Tensor, with_head: bool = False) -> torch.Tensor:
        self._head_done = False
        return self._run_layers(T, h, {}, norm_out=with_head)

    def _head(self, h_rows: torch.Tensor, greedy, out_ids: Optional[torch.Tensor] = None, init_pair=None, out_pair=None,
              gemm_done: bool = False, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h_rows: fp32 [B, W] rows of the stream -> logits [B, V] fp32 (and ids_out when greedy / sampling)."""
        B, W = h_rows.shape
        assert B <= self.head_rows_max and init_pair is None and out_pair is None
        hn = self.hn[:B]
        if not (getattr(self, "_normed", False) and h_rows.data_ptr() == self.h_a.data_ptr()):
            L.add_rms_norm(h_rows, self.final_norm_w, hn[:, :W], self.cfg.norm_eps, self.gain_offset, pdl=self.pdl)
            self._count()
        self._normed = False
        logits = self.logits[:B]
        self._linear(hn, self.lm_head, logits)
        if greedy == "sample":
            assert self.sampler is not None, "sampling needs enable_sampling()"
            idx = self.samp_idx[:B] if row_index is None else row_index
            self.sampler.sample(logits, idx, self.ids_out[:B] if out_ids is None else out_ids, pdl=self.pdl)
            self._count()
        elif greedy:
            E.argmax(logits, self.ids_out[:B] if out_ids is None else out_ids, self.argmax_ws, pdl=self.pdl)
            self._count()
        return logits

    # ------------------------------------------------------------------ prefill
    def prefill(self, kv: SessionKV, h_in: Optional[torch.Tensor] = None, ids: Optional[torch.Tensor] = None,
                pos0: Optional[int] = None, greedy=True, logits_at: Optional[Sequence[int]] = None):
        """Append T tokens of one session (chunked to ``max_chunk``).

        Returns the stream [T, W] (fp32, new tensor) on a span without a head, else ``(logits, ids_out)`` of the last
        position - or, with ``logits_at`` (indices into this call's tokens), a new [len(logits_at), V] fp32 tensor
        with the logits at those positions and the arg-max ids beside it."""
        self._prestaged = None
        pos0 = kv.length if pos0 is None else pos0
        T = ids.shape[0] if h_in is None else h_in.shape[0]
        if pos0 + T > kv.max_len - self.sink_row:
            raise ValueError(f"session {kv.session_id}: {pos0}+{T} tokens exceed max_length {kv.max_len - self.sink_row}")
        if kv.max_len != self.kv_capacity or kv.data.shape[0] != self.n_slots or kv.data.shape[-1] != self.row_elems or \
                kv.data.shape[1] != self.cache_planes or (self.state_elems and (kv.state is None or kv.state.numel() < self.state_elems)):
            raise ValueError(f"session cache {tuple(kv.data.shape)} does not fit this span "
                             f"({self.n_slots} slots x {self.cache_planes} planes x {self.kv_capacity} rows x {self.row_elems}, "
                             f"{self.state_elems} state elements)")
        W = self.cfg.hidden
        want = None if logits_at is None else sorted(set(int(i) for i in logits_at))
        out = None if self.has_head else torch.empty(T, W, dtype=torch.float32, device=self.device)
        rows = []
        last_h = None
        for c0 in range(0, T, self.max_chunk):
            n = min(self.max_chunk, T - c0)
            if h_in is None:
                self.ids_in[:n].copy_(ids[c0:c0 + n], non_blocking=True)
                x = self._embed(n, pos0 + c0, False)
            else:
                x = self.h_a[:n]
                x.copy_(h_in[c0:c0 + n], non_blocking=True)
            self._run_layers(n, x, {"kv": kv, "pos0": pos0 + c0})
            if out is not None:
                out[c0:c0 + n].copy_(x, non_blocking=True)
            elif want is not None:
                sel = [i - c0 for i in want if c0 <= i < c0 + n]
                if sel:
                    rows.append(x[torch.tensor(sel, device=self.device)])
            last_h = x[n - 1:n]
        kv.length = pos0 + T
        kv.touch()
        if not self.has_head:
            return out
        if want is None:
            self.last_hidden = last_h
            ri = None
            if greedy == "sample":
                ri = torch.tensor([getattr(kv, "sampler_row", 0) or 0], dtype=torch.int32, device=self.device)
            self._head(last_h.clone(), greedy, row_index=ri)
            return self.logits[:1], self.ids_out[:1]
        xs = torch.cat(rows, 0) if rows else torch.empty(0, W, dtype=torch.float32, device=self.device)
        res = torch.empty(len(want), self.cfg.vocab, dtype=torch.float32, device=self.device)
        res_ids = torch.empty(len(want), dtype=torch.int64, device=self.device)
        for r0 in range(0, len(want), self.head_rows_max):
            r1 = min(len(want), r0 + self.head_rows_max)
            self._head(xs[r0:r1], True)
            res[r0:r1].copy_(self.logits[:r1 - r0])
            res_ids[r0:r1].copy_(self.ids_out[:r1 - r0])
        order = {p: k for k, p in enumerate(want)}
        pick = torch.tensor([order[int(i)] for i in logits_at], device=self.device)
        return res[pick], res_ids[pick]

    def forward(self, h: torch.Tensor, kv: SessionKV, pos0: Optional[int] = None) -> torch.Tensor:
        assert not self.has_head
        if h.shape[0] == 1 and (pos0 is None or pos0 == kv.length):
            return self.decode([kv], h_in=h).clone()
        return self.prefill(kv, h_in=h, pos0=pos0)


def make_span(cfg, weights, device, dtype, **kw):
    """The span class of a configuration's family (the one place the runtime chooses between them)."""
    if getattr(cfg, "layer_list", False):
        return LayeredSpan(cfg, weights, device, dtype, **kw)
    return NativeSpan(cfg, weights, device, dtype, **kw)


def span_runs_natively(cfg, device, dtype) -> bool:
    """Does the family have a CUDA span for this element type?"""
    if torch.device(device).type != "cuda":
        return False
    if getattr(cfg, "layer_list", False):
        return dtype in (torch.float16, torch.bfloat16, torch.float32)
    return dtype in (torch.float16, torch.bfloat16)
