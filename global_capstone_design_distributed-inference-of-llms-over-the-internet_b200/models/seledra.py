"""Seledra: a layer-list decoder design that mixes softmax attention with a recurrent layer.

    x = embed[token] + pos[p]
    per layer:  x += m * mixer(norm1(x));   x += m * ff(norm2(x))   (a layer may have no feed-forward)
    logits = head . norm(x)

* mixer ``attention``: grouped-query attention without rotation; biased projections, one RMS norm over the WHOLE query
  (and key) projection, a weight-free RMS norm per value head, a per-head temperature, a softmax whose denominator
  carries one extra unit (a "sink" key of score 0 and value 0), values blended with the values of the first such
  layer of the same token (``v_mix``), one sigmoid output gate per head;
* mixer ``delta``: the gated delta rule - a matrix state per head that decays, is corrected towards the current value
  along the current key and is read with the query - behind short causal convolutions, with a gated RMS norm on the
  way out.  Its state (fp32) and the convolutions' last inputs are carried per sequence;
* feed-forward: ``W_down xielu(W_up h)`` with a piecewise activation of two learned numbers.

Every size and every constant that ``config.json`` carries lives in a spec object (``SinkAttentionSpec``,
``DeltaRuleSpec``, ``XieluMLPSpec``) that the loader, the cache manager and the span read; another layer-list design can
reuse the mechanisms with its own constants.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

# constants the design fixes (not in config.json)
DELTA_UNIT_EPS = 1e-6          # q, k of the delta rule: x / sqrt(sum(x^2) + DELTA_UNIT_EPS)
NORM_GAIN_OFFSET = 0.0         # norm gains are stored as they are applied
XIELU_LINEAR = 0.5             # slope of the activation's linear term on both sides of 0


@dataclass(frozen=True)
class SinkAttentionSpec:
    heads: int
    kv_heads: int
    dim: int                    # query / key size per head
    vdim: int                   # value size per head
    scale: float
    v_mix: bool = False         # values are blended with those of the first v_mix layer
    sink: float = 1.0           # what the softmax denominator carries besides the keys (exp(0): a key of score 0)
    kind = "attention"

    @property
    def q_size(self) -> int:
        return self.heads * self.dim

    @property
    def k_size(self) -> int:
        return self.kv_heads * self.dim

    @property
    def v_size(self) -> int:
        return self.kv_heads * self.vdim

    @property
    def proj_rows(self) -> int:
        """Rows of the fused projection [W_q ; W_k ; W_v ; W_gate]."""
        return self.q_size + self.k_size + self.v_size + self.heads

    @property
    def owns_cache(self) -> bool:
        return True

    state_elems = 0


@dataclass(frozen=True)
class DeltaRuleSpec:
    heads: int                  # value heads (one state matrix each)
    kv_heads: int               # query / key heads
    dim: int
    vdim: int
    conv: int                   # taps of the short convolutions
    unit_eps: float = DELTA_UNIT_EPS
    kind = "delta"

    @property
    def qk_size(self) -> int:
        return self.kv_heads * self.dim

    @property
    def v_size(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return 2 * self.qk_size + self.v_size

    @property
    def proj_rows(self) -> int:
        """Rows of the fused projection [W_q ; W_k ; W_v ; W_beta ; W_decay ; W_gate]."""
        return self.conv_channels + 2 * self.heads + self.v_size

    @property
    def owns_cache(self) -> bool:
        return False

    @property
    def state_elems(self) -> int:
        """fp32 numbers a sequence carries for this layer: two copies of the heads' matrices (a step at position p
        reads copy p & 1 and writes the other, so running a step twice leaves the same state) and a ring of the
        convolutions' last ``conv`` inputs (slot = position mod conv)."""
        return 2 * self.heads * self.dim * self.vdim + self.conv * self.conv_channels

    @property
    def ring_offset(self) -> int:
        return 2 * self.heads * self.dim * self.vdim


@dataclass(frozen=True)
class XieluMLPSpec:
    ff: int


@dataclass(frozen=True)
class LayerSpec:
    mixer: Any                  # SinkAttentionSpec | DeltaRuleSpec
    mlp: Optional[XieluMLPSpec]


@dataclass(frozen=True)
class SeledraConfig:
    layers: Tuple[LayerSpec, ...]
    hidden: int
    vocab: int
    norm_eps: float
    residual_mult: float
    max_positions: int
    name: str = ""
    bos_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    family: str = "seledra"
    tie_embeddings: bool = False

    is_llama = False
    layer_list = True           # the runtime serves it with the layer-list span
    parallel_block = False      # mixer and feed-forward are two residual updates, each behind its own norm
    norm_gain_offset = NORM_GAIN_OFFSET
    learned_positions = True

    @property
    def n_layers(self) -> int:
        return len(self.layers)

    # ---- cache layout: K and V planes of rows per attention layer (rows padded to the widest), plus fp32 state
    def cache_layers(self, start: int = 0, end: Optional[int] = None) -> List[int]:
        end = self.n_layers if end is None else end
        return [i for i in range(start, end) if self.layers[i].mixer.owns_cache]

    def cache_row(self, start: int = 0, end: Optional[int] = None) -> int:
        rows = [max(self.layers[i].mixer.k_size, self.layers[i].mixer.v_size) for i in self.cache_layers(start, end)]
        return (max(rows) + 7) // 8 * 8 if rows else 8          # (16-byte rows in 16-bit caches)

    cache_planes = 2

    def state_offsets(self, start: int = 0, end: Optional[int] = None) -> Dict[int, int]:
        """layer -> offset (fp32 elements) of its share of a sequence's recurrent state."""
        end = self.n_layers if end is None else end
        out, n = {}, 0
        for i in range(start, end):
            e = self.layers[i].mixer.state_elems
            if e:
                out[i] = n
                n += (e + 3) // 4 * 4
        return out

    def state_elems(self, start: int = 0, end: Optional[int] = None) -> int:
        end = self.n_layers if end is None else end
        return sum((self.layers[i].mixer.state_elems + 3) // 4 * 4 for i in range(start, end))

    def first_vmix_layer(self) -> Optional[int]:
        for i, L in enumerate(self.layers):
            if getattr(L.mixer, "v_mix", False):
                return i
        return None

    def check_span(self, start: int, end: int) -> None:
        first = self.first_vmix_layer()
        for i in range(start, end):
            if getattr(self.layers[i].mixer, "v_mix", False) and i != first and not (start <= first < i):
                raise ValueError(f"layer {i} blends its values with those of layer {first}, which is outside the span "
                                 f"[{start}, {end}): keep the value-mixing layers in one span")

    def layer_param_count(self, i: Optional[int] = None) -> int:
        if i is None:
            return max(self.layer_param_count(j) for j in range(self.n_layers))
        L, W = self.layers[i], self.hidden
        m = L.mixer
        if isinstance(m, SinkAttentionSpec):
            n = W + (m.proj_rows + m.heads * m.vdim) * W + 2 * m.q_size + 2 * m.k_size + m.v_size + m.heads + 1
        else:
            n = W + (m.proj_rows + m.v_size) * W + m.conv * m.conv_channels + 3 * m.heads + m.vdim
        if L.mlp is not None:
            n += W + 2 * L.mlp.ff * W + 2
        return n

    def layer_bytes(self, elem_size: int = 2) -> int:
        return self.layer_param_count() * elem_size

    def kv_bytes_per_token(self, n_layers: int, elem_size: int = 2) -> int:
        n = min(n_layers, self.n_layers)
        return self.cache_planes * self.cache_row(0, n) * max(1, len(self.cache_layers(0, n))) * elem_size

    def to_dict(self) -> Dict[str, Any]:
        return to_config_dict(self)


def _mixer_from(d: Dict[str, Any], kind: str):
    if kind == "attention":
        return SinkAttentionSpec(heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]),
                                 scale=float(d["scale"]), v_mix=bool(d.get("v_mix", False)))
    if kind == "delta":
        return DeltaRuleSpec(heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]),
                             conv=int(d["conv"]))
    raise ValueError(f"unsupported mixer type {kind!r} (supported: attention, delta)")


def _mlp_from(d: Optional[Dict[str, Any]]):
    if d is None:
        return None
    if d.get("kind", "dense") == "dense":
        return XieluMLPSpec(ff=int(d["ff"]))
    raise ValueError(f"unsupported mlp kind {d['kind']!r} (supported: dense)")


def from_config_dict(d: Dict[str, Any], name: str = "") -> SeledraConfig:
    layers = tuple(LayerSpec(_mixer_from(L["mixer"], L["type"]), _mlp_from(L.get("mlp"))) for L in d["layers"])
    cfg = SeledraConfig(layers, int(d["width"]), int(d["vocab"]), float(d["norm"]["eps"]), float(d.get("residual_mult", 1.0)),
                        int(d["max_positions"]), name, d.get("bos_token_id"), d.get("eos_token_id"))
    first = cfg.first_vmix_layer()
    for i, L in enumerate(layers):
        m = L.mixer
        if m.heads % m.kv_heads or min(m.heads, m.kv_heads, m.dim, m.vdim) < 1:
            raise ValueError(f"layer {i}: {m.heads} heads do not divide into {m.kv_heads} key heads")
        if isinstance(m, DeltaRuleSpec) and m.conv < 1:
            raise ValueError(f"layer {i}: a convolution needs at least one tap")
        if getattr(m, "v_mix", False) and (m.kv_heads, m.vdim) != (layers[first].mixer.kv_heads, layers[first].mixer.vdim):
            raise ValueError(f"layer {i}: value heads differ from layer {first}, whose values it blends with its own")
    return cfg


def to_config_dict(cfg: SeledraConfig) -> Dict[str, Any]:
    """The ``config.json`` of this configuration."""
    layers = []
    for L in cfg.layers:
        m = L.mixer
        if isinstance(m, SinkAttentionSpec):
            md: Dict[str, Any] = {"dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "scale": m.scale, "v_mix": m.v_mix,
                                  "vdim": m.vdim}
        else:
            md = {"conv": m.conv, "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "vdim": m.vdim}
        layers.append({"mixer": md, "mlp": None if L.mlp is None else {"ff": L.mlp.ff, "kind": "dense"}, "type": m.kind})
    return {"architecture": "Seledra", "layers": layers, "max_positions": cfg.max_positions, "norm": {"eps": cfg.norm_eps},
            "residual_mult": cfg.residual_mult, "vocab": cfg.vocab, "width": cfg.hidden}


# ---------------------------------------------------------------- tensor names and shapes
def layer_tensor_shapes(cfg: SeledraConfig, i: int) -> Dict[str, tuple]:
    L, W, p = cfg.layers[i], cfg.hidden, f"l{i}."
    m = L.mixer
    out: Dict[str, tuple] = {p + "norm1": (W,)}
    if isinstance(m, SinkAttentionSpec):
        out.update({p + "mix.q": (m.q_size, W), p + "mix.q.b": (m.q_size,), p + "mix.k": (m.k_size, W),
                    p + "mix.k.b": (m.k_size,), p + "mix.v": (m.v_size, W), p + "mix.v.b": (m.v_size,),
                    p + "mix.q.norm": (m.q_size,), p + "mix.k.norm": (m.k_size,), p + "mix.vmix": (),
                    p + "mix.temp": (m.heads,), p + "mix.g": (m.heads, W), p + "mix.o": (W, m.heads * m.vdim)})
    else:
        out.update({p + "mix.q": (m.qk_size, W), p + "mix.q.conv": (m.qk_size, m.conv), p + "mix.k": (m.qk_size, W),
                    p + "mix.k.conv": (m.qk_size, m.conv), p + "mix.v": (m.v_size, W), p + "mix.v.conv": (m.v_size, m.conv),
                    p + "mix.b": (m.heads, W), p + "mix.A_log": (m.heads,), p + "mix.norm": (m.vdim,),
                    p + "mix.a": (m.heads, W), p + "mix.dt_bias": (m.heads,), p + "mix.g": (m.v_size, W),
                    p + "mix.o": (W, m.v_size)})
    if L.mlp is not None:
        out.update({p + "norm2": (W,), p + "mlp.up": (L.mlp.ff, W), p + "mlp.down": (W, L.mlp.ff), p + "mlp.act": (2,)})
    return out


def tensor_shapes(cfg: SeledraConfig) -> Dict[str, tuple]:
    out: Dict[str, tuple] = {"embed": (cfg.vocab, cfg.hidden), "pos": (cfg.max_positions, cfg.hidden),
                             "final.norm": (cfg.hidden,), "head": (cfg.vocab, cfg.hidden)}
    for i in range(cfg.n_layers):
        out.update(layer_tensor_shapes(cfg, i))
    return out


def make_config(pattern: str = "addA", hidden: int = 256, vocab: int = 512, heads: int = 4, kv_heads: int = 2, dim: int = 32,
                vdim: int = 32, delta_heads: int = 4, delta_kv_heads: int = 2, delta_dim: int = 32, delta_vdim: int = 32,
                conv: int = 4, ff: int = 512, v_mix: bool = True, residual_mult: float = 0.5, max_positions: int = 1024,
                eps: float = 1e-5, name: str = "") -> SeledraConfig:
    """A regular configuration from a pattern of layers: ``a`` / ``A`` = attention without / with a feed-forward,
    ``d`` / ``D`` = delta rule without / with one."""
    layers = []
    for c in pattern:
        if c in "aA":
            m: Any = SinkAttentionSpec(heads, kv_heads, dim, vdim, dim ** -0.5, v_mix)
        elif c in "dD":
            m = DeltaRuleSpec(delta_heads, delta_kv_heads, delta_dim, delta_vdim, conv)
        else:
            raise ValueError(f"pattern letter {c!r} (a, A, d, D)")
        layers.append(LayerSpec(m, XieluMLPSpec(ff) if c.isupper() else None))
    return SeledraConfig(tuple(layers), hidden, vocab, eps, residual_mult, max_positions, name)


PRESETS: Dict[str, SeledraConfig] = {
    "tiny-seledra": make_config("AdDa", name="tiny-seledra"),
}
