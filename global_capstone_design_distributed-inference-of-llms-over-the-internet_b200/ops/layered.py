"""Python front-ends of the kernels for layer-list designs with an fp32 residual stream
(csrc/stream32.cu, csrc/gemm_simt.cu, csrc/latent_attention.cu, csrc/moe.cu, csrc/sink_attention.cu, csrc/delta_rule.cu)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native
from ._prototypes import AddNormArgs, DeltaArgs, LatentArgs, SimtGemmArgs, SinkAttnArgs

F16, BF16, F32 = 0, 1, 2


def code(dt: torch.dtype) -> int:
    try:
        return {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}[dt]
    except KeyError:
        raise ValueError(f"unsupported element type {dt}") from None


def _p(t: Optional[torch.Tensor]):
    return t.data_ptr() if t is not None else None


def _s():
    return native.current_stream_ptr()


def embed_f32(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, pdl: bool = False) -> torch.Tensor:
    assert ids.dtype == torch.int64 and out.dtype == torch.float32 and table.is_contiguous()
    T = ids.shape[0]
    native.check(native.lib().b200_embed_f32(ids.data_ptr(), table.data_ptr(), code(table.dtype), out.data_ptr(), T,
                                            table.shape[1], out.stride(0), table.shape[0], 1 if pdl else 0, _s()),
                 "b200_embed_f32")
    return out


def add_rms_norm(x: torch.Tensor, gain: Optional[torch.Tensor], out: Optional[torch.Tensor], eps: float,
                 gain_offset: float = 0.0, add_a: Optional[torch.Tensor] = None, add_b: Optional[torch.Tensor] = None,
                 pair_y: Optional[torch.Tensor] = None, pair_w: Optional[torch.Tensor] = None, top: int = 0,
                 add_scale: float = 1.0, pdl: bool = False) -> None:
    """x (fp32 [T, W], updated in place) += add_scale * (add_a + add_b + sum_k pair_w * pair_y);
    out = rms_norm(x) * (offset + gain)."""
    assert x.dtype == torch.float32 and x.stride(1) == 1
    a = AddNormArgs()
    a.x, a.add_a, a.add_b, a.pair_y, a.pair_w, a.gain, a.out = _p(x), _p(add_a), _p(add_b), _p(pair_y), _p(pair_w), _p(gain), _p(out)
    a.T, a.width, a.ldx = x.shape[0], x.shape[1], x.stride(0)
    a.lda = add_a.stride(0) if add_a is not None else 0
    a.ldb = add_b.stride(0) if add_b is not None else 0
    a.ldp = pair_y.stride(0) if pair_y is not None else 0
    a.top = top
    a.ldo = out.stride(0) if out is not None else 0
    a.out_dtype = code(out.dtype) if out is not None else F32
    a.eps, a.gain_offset, a.pdl, a.add_scale = eps, gain_offset, 1 if pdl else 0, add_scale
    for t in (add_a, add_b, pair_y, pair_w, gain):
        assert t is None or t.dtype == torch.float32
    native.check(native.lib().b200_add_rms_norm(ctypes.byref(a), _s()), "b200_add_rms_norm")


def glu_clamp(gate: torch.Tensor, up: torch.Tensor, act: torch.Tensor, limit: float, alpha: float, up_shift: float,
              pdl: bool = False) -> None:
    """gate / up: fp32 [T, ff] views with one row stride; act: [T, >= ff]."""
    assert gate.dtype == torch.float32 and up.dtype == torch.float32 and gate.stride(0) == up.stride(0)
    T, ff = gate.shape
    native.check(native.lib().b200_glu_clamp(gate.data_ptr(), up.data_ptr(), gate.stride(0), act.data_ptr(), act.stride(0),
                                            code(act.dtype), T, ff, limit, alpha, up_shift, 1 if pdl else 0, _s()),
                 "b200_glu_clamp")


def gemm_simt(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, T: Optional[int] = None, N: Optional[int] = None,
              K: Optional[int] = None, ldx: Optional[int] = None, ldw: Optional[int] = None, ldo: Optional[int] = None,
              w2: Optional[torch.Tensor] = None, batch: int = 1, x_bs: int = 0, w_bs: int = 0, o_bs: int = 0,
              group_off: Optional[torch.Tensor] = None, groups: int = 0, w_gs: int = 0,
              row_src: Optional[torch.Tensor] = None, row_dst: Optional[torch.Tensor] = None,
              row_scale: Optional[torch.Tensor] = None, pdl: bool = False) -> torch.Tensor:
    """out[r, n] = sum_k x[src(r), k] * w[n, k] on the CUDA cores (fp32 products); see ``b200_simt_gemm_args``."""
    a = SimtGemmArgs()
    a.x, a.w, a.w2, a.out = x.data_ptr(), w.data_ptr(), _p(w2), out.data_ptr()
    a.row_src, a.row_dst, a.group_off, a.row_scale = _p(row_src), _p(row_dst), _p(group_off), _p(row_scale)
    a.T = x.shape[0] if T is None else T
    a.N = w.shape[-2] if N is None else N
    a.K = w.shape[-1] if K is None else K
    a.ldx = x.stride(0) if ldx is None else ldx
    a.ldw = w.stride(-2) if ldw is None else ldw
    a.ldo = out.stride(0) if ldo is None else ldo
    a.x_dtype, a.w_dtype, a.out_dtype = code(x.dtype), code(w.dtype), code(out.dtype)
    a.batch, a.groups = batch, groups
    a.x_bs, a.w_bs, a.o_bs, a.w_gs = x_bs, w_bs, o_bs, w_gs
    a.pdl = 1 if pdl else 0
    native.check(native.lib().b200_gemm_simt(ctypes.byref(a), _s()), "b200_gemm_simt")
    return out


def latent_args(proj: torch.Tensor, q_off: int, kv_off: int, c_gain: Optional[torch.Tensor], inv_freq: torch.Tensor, *,
                heads: int, dim: int, rot: int, rot_dims: int, kv_rank: int, row_elems: int, cache_dtype: torch.dtype,
                eps: float, T: int, cache: Optional[torch.Tensor] = None, pos0: int = 0,
                kv_ptrs: Optional[torch.Tensor] = None, kv_ptr_stride: int = 0, pos: Optional[torch.Tensor] = None,
                q_abs: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, window: int = 0,
                scale: float = 1.0, pdl: bool = False) -> LatentArgs:
    assert proj.dtype == torch.float32 and inv_freq.dtype == torch.float64
    a = LatentArgs()
    a.proj, a.ldp, a.q_off, a.kv_off = proj.data_ptr(), proj.stride(0), q_off, kv_off
    a.c_gain, a.inv_freq = _p(c_gain), inv_freq.data_ptr()
    a.cache, a.kv_ptrs, a.pos = _p(cache), _p(kv_ptrs), _p(pos)
    a.kv_ptr_stride, a.pos0 = kv_ptr_stride, pos0
    a.T, a.heads, a.dim, a.rot, a.rot_dims, a.kv_rank = T, heads, dim, rot, rot_dims, kv_rank
    a.row_elems, a.cache_dtype, a.eps = row_elems, code(cache_dtype), eps
    a.q_abs, a.out = _p(q_abs), _p(out)
    a.ldqa = q_abs.stride(0) if q_abs is not None else 0
    a.ldout = out.stride(0) if out is not None else 0
    a.window, a.scale, a.pdl = window, scale, 1 if pdl else 0
    return a


def latent_rope_append(a: LatentArgs) -> None:
    native.check(native.lib().b200_latent_rope_append(ctypes.byref(a), _s()), "b200_latent_rope_append")


def latent_attn(a: LatentArgs, splits: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """splits > 1: the keys of every token's window are divided over that many blocks (``scratch``: fp32 tensor of
    at least T * heads * splits * (kv_rank + 2) elements)."""
    if splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32 and \
            scratch.numel() >= a.T * a.heads * splits * (a.kv_rank + 2)
        native.check(native.lib().b200_latent_attn_split(ctypes.byref(a), splits, scratch.data_ptr(), _s()), "b200_latent_attn")
    else:
        native.check(native.lib().b200_latent_attn(ctypes.byref(a), _s()), "b200_latent_attn")


def moe_route(logits: torch.Tensor, experts: int, groups: int, keep: int, top: int, ids: torch.Tensor, weights: torch.Tensor,
              renorm: bool = False, pdl: bool = False) -> None:
    """logits: fp32 [T, >= experts] view; ids int32 [T, top]; weights fp32 [T, top]."""
    assert logits.dtype == torch.float32 and ids.dtype == torch.int32 and weights.dtype == torch.float32
    native.check(native.lib().b200_moe_route(logits.data_ptr(), logits.stride(0), logits.shape[0], experts, groups, keep, top,
                                            1 if renorm else 0, ids.data_ptr(), weights.data_ptr(), 1 if pdl else 0, _s()),
                 "b200_moe_route")


def moe_plan(ids: torch.Tensor, T: int, top: int, experts: int, group_off: torch.Tensor, row_pair: torch.Tensor,
             row_token: torch.Tensor, pdl: bool = False) -> None:
    native.check(native.lib().b200_moe_plan(ids.data_ptr(), T, top, experts, group_off.data_ptr(), row_pair.data_ptr(),
                                           row_token.data_ptr(), 1 if pdl else 0, _s()), "b200_moe_plan")


def moe_scale(act: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int, ff: int, top: int,
              pdl: bool = False) -> None:
    """act: 16-bit [T, >= experts * ff], scaled in place by each token's routing weights (0 for experts not chosen)."""
    native.check(native.lib().b200_moe_scale(act.data_ptr(), act.stride(0), code(act.dtype), ids.data_ptr(), weights.data_ptr(),
                                            act.shape[0], experts, ff, top, 1 if pdl else 0, _s()), "b200_moe_scale")


def latent_attn_prefill(proj: torch.Tensor, q_off: int, kvx: torch.Tensor, v_off: int, cache: torch.Tensor, kv_rank: int,
                        out: torch.Tensor, *, T: int, heads: int, dim: int, rot: int, vdim: int, pos0: int, s0: int,
                        window: int, scale: float, pdl: bool = False) -> None:
    """Tensor-core attention of a chunk of one session over expanded keys / values (``b200_latent_attn_prefill``)."""
    assert proj.dtype == torch.float32 and kvx.dtype == cache.dtype == out.dtype and kvx.dtype in (torch.float16, torch.bfloat16)
    native.check(native.lib().b200_latent_attn_prefill(
        proj.data_ptr(), proj.stride(0), q_off, kvx.data_ptr(), kvx.stride(0), v_off, cache.data_ptr(), cache.stride(0),
        kv_rank, out.data_ptr(), out.stride(0), T, heads, dim, rot, vdim, pos0, s0, window, scale, code(out.dtype),
        1 if pdl else 0, _s()), "b200_latent_attn_prefill")


# ---------------------------------------------------------------- learned positions, piecewise activation
def embed_pos_f32(ids: torch.Tensor, table: torch.Tensor, pos_table: torch.Tensor, out: torch.Tensor,
                  pos: Optional[torch.Tensor] = None, pos0: int = 0, pdl: bool = False) -> torch.Tensor:
    """out[t] = table[ids[t]] + pos_table[p_t] in fp32; p_t = pos[t] (int32 device tensor) or pos0 + t."""
    assert ids.dtype == torch.int64 and out.dtype == torch.float32 and table.is_contiguous() and pos_table.is_contiguous()
    assert table.dtype == pos_table.dtype and table.shape[1] == pos_table.shape[1]
    native.check(native.lib().b200_embed_pos_f32(ids.data_ptr(), table.data_ptr(), pos_table.data_ptr(), code(table.dtype),
                                                _p(pos), pos0, out.data_ptr(), ids.shape[0], table.shape[1], out.stride(0),
                                                table.shape[0], pos_table.shape[0], 1 if pdl else 0, _s()), "b200_embed_pos_f32")
    return out


def xielu(z: torch.Tensor, params: torch.Tensor, act: torch.Tensor, lin: float = 0.5, neg_base: float = 0.5,
          pdl: bool = False) -> None:
    """z: fp32 [T, ff] view; params: fp32 [2] on the device; act: [T, >= ff]."""
    assert z.dtype == torch.float32 and params.dtype == torch.float32 and z.stride(1) == 1
    T, ff = z.shape
    native.check(native.lib().b200_xielu(z.data_ptr(), z.stride(0), params.data_ptr(), lin, neg_base, act.data_ptr(),
                                        act.stride(0), code(act.dtype), T, ff, 1 if pdl else 0, _s()), "b200_xielu")


def gated_head_norm(o: torch.Tensor, gate: torch.Tensor, gain: torch.Tensor, out: torch.Tensor, heads: int, vdim: int,
                    eps: float, pdl: bool = False) -> None:
    """out[t, h] = rms_norm(o[t, h]) * gain * silu(gate[t, h]); o / gate: fp32 [T, >= heads * vdim] views."""
    assert o.dtype == gate.dtype == gain.dtype == torch.float32
    native.check(native.lib().b200_gated_head_norm(o.data_ptr(), o.stride(0), gate.data_ptr(), gate.stride(0), gain.data_ptr(),
                                                  out.data_ptr(), out.stride(0), code(out.dtype), o.shape[0], heads, vdim, eps,
                                                  1 if pdl else 0, _s()), "b200_gated_head_norm")


# ---------------------------------------------------------------- attention with a sink
def sink_attn_args(proj: torch.Tensor, *, q_off: int, k_off: int, v_off: int, g_off: int, heads: int, kv_heads: int, dim: int,
                   vdim: int, row_elems: int, cache_dtype: torch.dtype, eps: float, scale: float, sink: float, T: int,
                   bias: Optional[torch.Tensor] = None, q_gain: Optional[torch.Tensor] = None,
                   k_gain: Optional[torch.Tensor] = None, temp: Optional[torch.Tensor] = None,
                   vmix: Optional[torch.Tensor] = None, v_first: Optional[torch.Tensor] = None, vmix_mode: int = 0,
                   k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None, pos0: int = 0,
                   kv_ptrs: Optional[torch.Tensor] = None, kv_ptr_stride: int = 0, pos: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, q16: Optional[torch.Tensor] = None, pdl: bool = False) -> SinkAttnArgs:
    assert proj.dtype == torch.float32
    for t in (bias, q_gain, k_gain, temp, vmix, v_first):
        assert t is None or t.dtype == torch.float32
    a = SinkAttnArgs()
    a.proj, a.ldp, a.q_off, a.k_off, a.v_off, a.g_off = proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, g_off
    a.bias, a.q_gain, a.k_gain, a.temp, a.vmix, a.v_first = _p(bias), _p(q_gain), _p(k_gain), _p(temp), _p(vmix), _p(v_first)
    a.ldvf = v_first.stride(0) if v_first is not None else 0
    a.vmix_mode = vmix_mode
    a.k_cache, a.v_cache, a.kv_ptrs, a.pos = _p(k_cache), _p(v_cache), _p(kv_ptrs), _p(pos)
    a.kv_ptr_stride, a.pos0 = kv_ptr_stride, pos0
    a.T, a.heads, a.kv_heads, a.dim, a.vdim, a.row_elems = T, heads, kv_heads, dim, vdim, row_elems
    a.cache_dtype, a.eps, a.scale, a.sink = code(cache_dtype), eps, scale, sink
    a.out = _p(out)
    a.ldo = out.stride(0) if out is not None else 0
    a.out_dtype = code(out.dtype) if out is not None else F32
    a.pdl = 1 if pdl else 0
    if q16 is not None:
        assert q16.dtype == cache_dtype and q16.dtype != torch.float32
        a.q16, a.ldq16 = q16.data_ptr(), q16.stride(0)
    return a


def head_gate(x: torch.Tensor, gate: torch.Tensor, heads: int, vdim: int, pdl: bool = False) -> None:
    """x[t, h, :] *= sigmoid(gate[t, h]) in place; gate: fp32 [T, >= heads] view."""
    assert gate.dtype == torch.float32
    native.check(native.lib().b200_head_gate(x.data_ptr(), x.stride(0), code(x.dtype), gate.data_ptr(), gate.stride(0), x.shape[0],
                                            heads, vdim, 1 if pdl else 0, _s()), "b200_head_gate")


def attn_prefill_rows_fits(dim: int, vdim: int, row_elems: int) -> bool:
    """Can the tcgen05 flash-attention kernel of the uniform families read these planes (equal key and value sizes of
    64 or 128, 16-byte rows)?"""
    return dim == vdim and dim in (64, 128) and row_elems % 8 == 0 and hasattr(native.lib(), "b200_attn_prefill_tc_rows")


def attn_prefill_rows(q16: torch.Tensor, out: torch.Tensor, k_plane: torch.Tensor, v_plane: torch.Tensor, *, heads: int,
                      kv_heads: int, dim: int, rows: int, pos0: int, scale: float, pdl: bool = False) -> None:
    """Causal attention of a chunk on the tcgen05 kernel over planes [rows, row] that keep the heads of a position side
    by side; query t sees rows 0 .. pos0 + t."""
    assert q16.dtype == out.dtype == k_plane.dtype == v_plane.dtype and k_plane.stride(1) == 1
    native.check(native.lib().b200_attn_prefill_tc_rows(
        q16.data_ptr(), out.data_ptr(), k_plane.data_ptr(), v_plane.data_ptr(), q16.shape[0], heads, kv_heads, dim, rows,
        q16.stride(0), out.stride(0), pos0, scale, code(out.dtype), k_plane.stride(0), dim, 1 if pdl else 0, _s()),
        "b200_attn_prefill_tc_rows")


def sink_attn_append(a: SinkAttnArgs) -> None:
    native.check(native.lib().b200_sink_attn_append(ctypes.byref(a), _s()), "b200_sink_attn_append")


def sink_attn(a: SinkAttnArgs, splits: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """splits > 1: ``scratch`` is an fp32 tensor of at least T * heads * splits * (vdim + 2) elements."""
    if splits > 1:
        assert scratch is not None and scratch.dtype == torch.float32 and \
            scratch.numel() >= a.T * a.heads * splits * (a.vdim + 2)
    native.check(native.lib().b200_sink_attn(ctypes.byref(a), splits, _p(scratch) if splits > 1 else None, _s()), "b200_sink_attn")


def sink_attn_prefill_fits(dim: int, vdim: int) -> bool:
    """Can the tensor-core kernel take heads of these sizes (its query tile, two key tiles and two value tiles must fit
    into shared memory)?"""
    if vdim > 256:
        return False
    dqp, nv = (dim + 15) // 16 * 16, (vdim + 7) // 8
    nv = 4 if nv <= 4 else 8 if nv <= 8 else 16 if nv <= 16 else 32
    return ((64 + 2 * 64) * (dqp + 8) + 2 * 64 * (nv * 8 + 8)) * 2 <= 200 * 1024


def sink_attn_prefill(a: SinkAttnArgs) -> None:
    native.check(native.lib().b200_sink_attn_prefill(ctypes.byref(a), _s()), "b200_sink_attn_prefill")


# ---------------------------------------------------------------- gated delta rule
def delta_args(proj: torch.Tensor, *, c_off: int, b_off: int, a_off: int, conv_w: torch.Tensor, A_log: torch.Tensor,
               dt_bias: torch.Tensor, work: torch.Tensor, o: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int,
               taps: int, unit_eps: float, n_seq: int, seq_len: int, state: Optional[torch.Tensor] = None,
               state_ptrs: Optional[torch.Tensor] = None, state_ptr_stride: int = 0, state_off: int = 0,
               pos: Optional[torch.Tensor] = None, pos0: int = 0, pdl: bool = False) -> DeltaArgs:
    for t in (proj, conv_w, A_log, dt_bias, work, o, state):
        assert t is None or t.dtype == torch.float32
    assert work.shape[1] >= 2 * kv_heads * dim + heads * vdim + 2 * heads + kv_heads
    a = DeltaArgs()
    a.proj, a.ldp, a.c_off, a.b_off, a.a_off = proj.data_ptr(), proj.stride(0), c_off, b_off, a_off
    a.conv_w, a.A_log, a.dt_bias = conv_w.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr()
    a.work, a.ldw = work.data_ptr(), work.stride(0)
    a.state, a.state_ptrs, a.state_ptr_stride, a.state_off = _p(state), _p(state_ptrs), state_ptr_stride, state_off
    a.pos, a.pos0 = _p(pos), pos0
    a.n_seq, a.seq_len, a.heads, a.kv_heads, a.dim, a.vdim, a.taps = n_seq, seq_len, heads, kv_heads, dim, vdim, taps
    a.unit_eps = unit_eps
    a.o, a.ldo, a.pdl = o.data_ptr(), o.stride(0), 1 if pdl else 0
    return a


def delta_prep(a: DeltaArgs) -> None:
    native.check(native.lib().b200_delta_prep(ctypes.byref(a), _s()), "b200_delta_prep")


def delta_rule(a: DeltaArgs) -> None:
    native.check(native.lib().b200_delta_rule(ctypes.byref(a), _s()), "b200_delta_rule")
