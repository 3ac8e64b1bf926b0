"""Python front-ends of the kernels for layer-list designs with an fp32 residual stream
(csrc/stream32.cu, csrc/gemm_simt.cu, csrc/latent_attention.cu, csrc/moe.cu)."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import native
from ._prototypes import AddNormArgs, LatentArgs, SimtGemmArgs

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
                 pdl: bool = False) -> None:
    """x (fp32 [T, W], updated in place) += add_a + add_b + sum_k pair_w * pair_y;  out = rms_norm(x) * (offset + gain)."""
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
    a.eps, a.gain_offset, a.pdl = eps, gain_offset, 1 if pdl else 0
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
