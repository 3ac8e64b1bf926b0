"""Gigezen: a layer-list decoder design (every size and constant comes from ``config.json``).

    embed -> N x [ h = norm1(x);  x += mixer(h) + ff(h) ] -> final norm -> head

* one RMS norm per layer with gains stored around zero (``1 + w``); mixer and feed-forward both read it (parallel block);
* mixer ``latent_attention``: low-rank key/value latent + one rotated key part shared by all heads, sliding window,
  optionally reading the cache of an earlier layer (``kv_from``);
* feed-forward: a dense clamped gated unit, or a mixture of experts with a softmax router and group-limited top-k.

The mechanisms are described by small spec objects (``LatentAttentionSpec``, ``GatedMLPSpec``, ``MoESpec``) that the
loader, the cache manager and the span read; another layer-list design can reuse them with its own constants.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

# constants the design fixes (not in config.json)
DENSE_GATE_ALPHA = 1.702       # y = g * sigmoid(alpha * g) * (u + DENSE_UP_SHIFT)
DENSE_UP_SHIFT = 1.0
NORM_GAIN_OFFSET = 1.0         # layer / final norm gains are stored around zero


@dataclass(frozen=True)
class LatentAttentionSpec:
    heads: int
    dim: int                    # unrotated query/key dimensions per head
    rot_dim: int                # rotated query/key dimensions per head (the key part is shared by all heads)
    vdim: int
    kv_rank: int
    window: int                 # causal band: query i attends to the keys j in (i - window, i]
    scale: float
    rope_base: float
    rope_dims: int              # rotated dimensions of the rot part (pairs i, i + rope_dims/2)
    kv_from: Optional[int] = None   # absolute index of the layer whose cache rows this layer reads

    @property
    def q_size(self) -> int:
        return self.heads * (self.dim + self.rot_dim)

    @property
    def row(self) -> int:
        """Elements of one cache row."""
        return self.kv_rank + self.rot_dim

    @property
    def owns_cache(self) -> bool:
        return self.kv_from is None


@dataclass(frozen=True)
class GatedMLPSpec:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoESpec:
    experts: int
    top: int
    groups: int
    keep: int
    ff: int


@dataclass(frozen=True)
class LayerSpec:
    mixer: LatentAttentionSpec
    mlp: Any                    # GatedMLPSpec | MoESpec | None


@dataclass(frozen=True)
class GigezenConfig:
    layers: Tuple[LayerSpec, ...]
    hidden: int
    vocab: int
    norm_eps: float
    name: str = ""
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    family: str = "gigezen"
    max_positions: int = 1 << 20
    tie_embeddings: bool = False

    is_llama = False
    layer_list = True           # the runtime serves it with the layer-list span
    parallel_block = True       # mixer and feed-forward read one norm and update the stream together
    norm_gain_offset = NORM_GAIN_OFFSET
    learned_positions = False
    residual_mult = 1.0
    cache_planes = 1

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    def state_elems(self, start: int = 0, end: Optional[int] = None) -> int:
        return 0                # no recurrent layers: a sequence carries cache rows only

    # ---- cache layout: one plane of rows per cache-owning layer, all rows padded to the widest one
    def cache_layers(self, start: int = 0, end: Optional[int] = None) -> List[int]:
        end = self.n_layers if end is None else end
        return [i for i in range(start, end) if self.layers[i].mixer.owns_cache]

    def cache_row(self, start: int = 0, end: Optional[int] = None) -> int:
        rows = [self.layers[i].mixer.row for i in self.cache_layers(start, end)]
        return (max(rows) + 63) // 64 * 64 if rows else 64      # (whole 64-element k-blocks: rows are a GEMM operand)

    def check_span(self, start: int, end: int) -> None:
        for i in range(start, end):
            src = self.layers[i].mixer.kv_from
            if src is not None and not (start <= src < i):
                raise ValueError(f"layer {i} reads the cache of layer {src}, which is outside the span [{start}, {end}): "
                                 "split the model between such groups of layers")

    def layer_param_count(self, i: Optional[int] = None) -> int:
        if i is None:
            return max(self.layer_param_count(j) for j in range(self.n_layers))
        L, W = self.layers[i], self.hidden
        m = L.mixer
        n = W + m.q_size * W + m.heads * (m.dim + m.vdim) * m.kv_rank + W * m.heads * m.vdim
        if m.owns_cache:
            n += (m.kv_rank + m.rot_dim) * W + m.kv_rank
        if isinstance(L.mlp, GatedMLPSpec):
            n += 3 * L.mlp.ff * W
        elif isinstance(L.mlp, MoESpec):
            n += L.mlp.experts * (3 * L.mlp.ff * W + W)
        return n

    def layer_bytes(self, elem_size: int = 2) -> int:
        return self.layer_param_count() * elem_size

    def kv_bytes_per_token(self, n_layers: int, elem_size: int = 2) -> int:
        return self.cache_row() * max(1, len(self.cache_layers(0, min(n_layers, self.n_layers)))) * elem_size

    def to_dict(self) -> Dict[str, Any]:
        return to_config_dict(self)


def _mixer_from(d: Dict[str, Any], kind: str) -> LatentAttentionSpec:
    if kind != "latent_attention":
        raise ValueError(f"unsupported mixer type {kind!r} (supported: latent_attention)")
    rot = d.get("rot") or {}
    rot_dim = int(d["rot_dim"])
    return LatentAttentionSpec(heads=int(d["heads"]), dim=int(d["dim"]), rot_dim=rot_dim, vdim=int(d["vdim"]),
                               kv_rank=int(d["kv_rank"]), window=int(d["mask"]["size"]), scale=float(d["scale"]),
                               rope_base=float(rot["base"]), rope_dims=int(rot.get("dims", rot_dim)),
                               kv_from=None if d.get("kv_from") is None else int(d["kv_from"]))


def _mlp_from(d: Optional[Dict[str, Any]]):
    if d is None:
        return None
    if d["kind"] == "dense":
        return GatedMLPSpec(ff=int(d["ff"]), limit=float(d["limit"]))
    if d["kind"] == "moe":
        r = d["router"]
        g = r.get("groups") or {}
        return MoESpec(experts=int(r["experts"]), top=int(r["top"]), groups=int(g.get("count", 1)),
                       keep=int(g.get("keep", g.get("count", 1))), ff=int(d["expert"]["ff"]))
    raise ValueError(f"unsupported mlp kind {d['kind']!r} (supported: dense, moe)")


def from_config_dict(d: Dict[str, Any], name: str = "") -> GigezenConfig:
    layers = tuple(LayerSpec(_mixer_from(L["mixer"], L["type"]), _mlp_from(L.get("mlp"))) for L in d["layers"])
    cfg = GigezenConfig(layers, int(d["width"]), int(d["vocab"]), float(d["norm"]["eps"]), name,
                        d.get("bos_token_id"), d.get("eos_token_id"))
    for i, L in enumerate(layers):
        m = L.mixer
        if m.kv_from is not None:
            if not 0 <= m.kv_from < i or not layers[m.kv_from].mixer.owns_cache:
                raise ValueError(f"layer {i}: kv_from {m.kv_from} must name an earlier layer with a cache of its own")
            s = layers[m.kv_from].mixer
            if (s.kv_rank, s.rot_dim, s.rope_base, s.rope_dims) != (m.kv_rank, m.rot_dim, m.rope_base, m.rope_dims):
                raise ValueError(f"layer {i}: latent size / rotation differ from layer {m.kv_from}, whose cache it reads")
        if m.rope_dims > m.rot_dim or m.rope_dims % 2:
            raise ValueError(f"layer {i}: rot.dims {m.rope_dims} must be even and <= rot_dim {m.rot_dim}")
        if isinstance(L.mlp, MoESpec):
            e = L.mlp
            if e.experts % e.groups or not 1 <= e.keep <= e.groups or not 1 <= e.top <= e.keep * (e.experts // e.groups):
                raise ValueError(f"layer {i}: router sizes do not fit together ({e})")
    return cfg


def to_config_dict(cfg: GigezenConfig) -> Dict[str, Any]:
    """The ``config.json`` of this configuration."""
    layers = []
    for L in cfg.layers:
        m = L.mixer
        md: Dict[str, Any] = {"dim": m.dim, "heads": m.heads, "kv_rank": m.kv_rank, "mask": {"size": m.window},
                              "rot": {"base": m.rope_base, "dims": m.rope_dims}, "rot_dim": m.rot_dim, "scale": m.scale,
                              "vdim": m.vdim}
        if m.kv_from is not None:
            md["kv_from"] = m.kv_from
        if isinstance(L.mlp, GatedMLPSpec):
            ml: Any = {"ff": L.mlp.ff, "kind": "dense", "limit": L.mlp.limit}
        elif isinstance(L.mlp, MoESpec):
            ml = {"expert": {"ff": L.mlp.ff}, "kind": "moe",
                  "router": {"experts": L.mlp.experts, "groups": {"count": L.mlp.groups, "keep": L.mlp.keep}, "top": L.mlp.top}}
        else:
            ml = None
        layers.append({"mixer": md, "mlp": ml, "type": "latent_attention"})
    return {"architecture": "Gigezen", "layers": layers, "norm": {"eps": cfg.norm_eps}, "vocab": cfg.vocab,
            "width": cfg.hidden}


# ---------------------------------------------------------------- tensor names and shapes
def layer_tensor_shapes(cfg: GigezenConfig, i: int) -> Dict[str, tuple]:
    L, W, p = cfg.layers[i], cfg.hidden, f"l{i}."
    m = L.mixer
    out = {p + "norm1": (W,), p + "mix.q": (m.q_size, W), p + "mix.uk": (m.heads * m.dim, m.kv_rank),
           p + "mix.uv": (m.heads * m.vdim, m.kv_rank), p + "mix.o": (W, m.heads * m.vdim)}
    if m.owns_cache:
        out[p + "mix.dkv"] = (m.kv_rank + m.rot_dim, W)
        out[p + "mix.dkv.norm"] = (m.kv_rank,)
    if isinstance(L.mlp, GatedMLPSpec):
        out.update({p + "mlp.gate": (L.mlp.ff, W), p + "mlp.up": (L.mlp.ff, W), p + "mlp.down": (W, L.mlp.ff)})
    elif isinstance(L.mlp, MoESpec):
        out[p + "mlp.router"] = (L.mlp.experts, W)
        for e in range(L.mlp.experts):
            q = f"{p}mlp.e{e}."
            out.update({q + "gate": (L.mlp.ff, W), q + "up": (L.mlp.ff, W), q + "down": (W, L.mlp.ff)})
    return out


def tensor_shapes(cfg: GigezenConfig) -> Dict[str, tuple]:
    out: Dict[str, tuple] = {"embed": (cfg.vocab, cfg.hidden), "final.norm": (cfg.hidden,), "head": (cfg.vocab, cfg.hidden)}
    for i in range(cfg.n_layers):
        out.update(layer_tensor_shapes(cfg, i))
    return out


def make_config(n_layers: int = 4, hidden: int = 256, vocab: int = 512, heads: int = 4, dim: int = 32, rot_dim: int = 16,
                vdim: int = 32, kv_rank: int = 64, window: int = 48, ff: int = 512, experts: int = 8, top: int = 2,
                groups: int = 4, keep: int = 2, expert_ff: int = 128, share_every: int = 2, moe_every: int = 2,
                limit: float = 3.0, rope_base: float = 10000.0, eps: float = 1e-5, name: str = "") -> GigezenConfig:
    """A regular configuration: every ``share_every``-th layer reads the cache of the layer before it, every
    ``moe_every``-th layer carries a mixture of experts (0 = never)."""
    layers = []
    for i in range(n_layers):
        shares = share_every > 0 and i % share_every == share_every - 1 and i > 0 and layers[i - 1].mixer.owns_cache
        m = LatentAttentionSpec(heads, dim, rot_dim, vdim, kv_rank, window, (dim + rot_dim) ** -0.5, rope_base, rot_dim,
                                i - 1 if shares else None)
        moe = moe_every > 0 and i % moe_every == moe_every - 1
        layers.append(LayerSpec(m, MoESpec(experts, top, groups, keep, expert_ff) if moe else GatedMLPSpec(ff, limit)))
    return GigezenConfig(tuple(layers), hidden, vocab, eps, name)


PRESETS: Dict[str, GigezenConfig] = {
    "tiny-gigezen": make_config(name="tiny-gigezen"),
}
