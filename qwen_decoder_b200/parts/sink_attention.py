"""Grouped-query attention with unit-normalised queries and keys, a sink in the softmax, values of their own size,
and values blended with an earlier layer's.

    q, k, v = Wq h, Wk h, Wv h (no biases); per head q <- unit(q) * wq, k <- unit(k) * wk with
    unit(y) = y / sqrt(mean(y^2) + eps) over the head's ``head_dim`` elements (one weight vector for all heads);
    the first ``rotary_dim`` elements of q and k turn by position (the ``position`` part's tables);
    s_ij = (q_i . k_j) * scale over the keys j <= i (or the last ``window``);
    p_ij = exp(s_ij) / (sum_j exp(s_ij) + exp(sink_h)): the sink is one learned number per query head that joins the
    denominator once, unscaled, and has no key and no value;  o_i = sum_j p_ij v_j;  out = Wo [o of all heads].
    Query head h reads key/value head h // (H / G).  Values have ``v_dim`` elements, keys ``head_dim``.

``value_mix`` names a family of layers that blend their values: the first layer of the family to run in a step
leaves its (unblended) values of the step's tokens on the step's context; every later layer of the family caches and
attends over (1 - lam) v + lam v_first, lam its learned number ``vmix`` (the first layer's own ``vmix`` is stored but
unused).  Only values of the same token are blended, so nothing but the blended value needs caching.

Each option is a constructor parameter (``qk_norm``, ``sink``, ``v_dim``, ``value_mix``); with all of them off this
is plain grouped-query attention.  Scores, softmax weights, the unit norms and the rotation are float32 in both
engine dtypes; the projections run in the engine's dtype with float32 sums.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from ..cache import PagedKV
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, PagedCacheView
from .linear import Linear

import os as _os
_TENSOR_CORES = _os.environ.get("QD_SINK_MMA", "1") != "0"       # 0: every dtype and size on the float32 kernel


@register_part("mixer", "sink_attention")
class SinkAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_dim: Optional[int] = None,
                 scale: Optional[float] = None, eps: float = 1e-6, qk_norm: bool = True, sink: bool = True,
                 value_mix: Optional[str] = None, value_mix_first: bool = False, position=None,
                 window: Optional[int] = None, prefix: str = "mix.", weight_suffix: str = "",
                 names=("q", "k", "v", "o")):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_kv_heads ({num_kv_heads}) must divide num_heads ({num_heads})")
        self.hidden_size, self.num_heads, self.num_kv_heads = hidden_size, num_heads, num_kv_heads
        self.head_dim, self.v_dim = head_dim, v_dim or head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.eps, self.qk_norm, self.sink = float(eps), bool(qk_norm), bool(sink)
        self.value_mix, self.value_mix_first = value_mix, bool(value_mix_first)
        self.position, self.window = position, window
        self.prefix, self.sfx = prefix, weight_suffix
        q, k, v, o = names
        self.names = tuple(names)
        self.qkv = Linear(hidden_size, [(f"{prefix}{q}", num_heads * head_dim), (f"{prefix}{k}", num_kv_heads * head_dim),
                                        (f"{prefix}{v}", num_kv_heads * self.v_dim)], bias=False,
                          weight_suffix=weight_suffix)
        self.out = Linear(num_heads * self.v_dim, [(f"{prefix}{o}", hidden_size)], bias=False,
                          weight_suffix=weight_suffix)
        self.w_q_norm = self.w_k_norm = self.sinks = self.lam = None

    def cache_need(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window, v_dim=self.v_dim)

    def tensor_specs(self) -> List[TensorSpec]:
        p = self.prefix
        q, k, _, _ = self.names
        specs = self.qkv.tensor_specs() + self.out.tensor_specs()
        if self.qk_norm:
            specs += [TensorSpec(f"{p}{q}.norm", (self.head_dim,), init="around_one"),
                      TensorSpec(f"{p}{k}.norm", (self.head_dim,), init="around_one")]
        if self.sink:
            specs.append(TensorSpec(f"{p}sink", (self.num_heads,), init="uniform:-1:1"))
        if self.value_mix is not None:
            specs.append(TensorSpec(f"{p}vmix", (), init="uniform:0.2:0.8"))
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.qkv.bind(source, dtype, device)
        self.out.bind(source, dtype, device)
        p = self.prefix
        q, k, _, _ = self.names
        f32 = lambda n: source.get(n).to(device=device, dtype=torch.float32).contiguous()
        if self.qk_norm:
            self.w_q_norm, self.w_k_norm = f32(f"{p}{q}.norm"), f32(f"{p}{k}.norm")
        if self.sink:
            self.sinks = f32(f"{p}sink")
        if self.value_mix is not None and not self.value_mix_first:
            self.lam = f32(f"{p}vmix").reshape(1)

    def forward(self, x: torch.Tensor, ctx, cache: PagedCacheView) -> torch.Tensor:
        H, G, d, vd = self.num_heads, self.num_kv_heads, self.head_dim, self.v_dim
        T = x.shape[0]
        pos = self.position
        rope = (pos.rotary_dim, pos.pairing_code, pos.cos, pos.sin) if pos is not None else (0, 0, None, None)
        qkv = self.qkv.forward(x, out_dtype=torch.float32)          # the norms and the rotation take unrounded sums
        v_source = None
        if self.value_mix is not None:
            key = ("value_mix", self.value_mix)
            if self.value_mix_first:
                ctx.shared[key] = qkv[:, (H + G) * d:]              # this step's tokens only; read by later layers
            else:
                v_source = ctx.shared.get(key)
                if v_source is None:
                    raise RuntimeError(f"value mix {self.value_mix!r}: no earlier layer of this step left its values")
        q = torch.empty((T, H * d), dtype=x.dtype, device=x.device)
        ps, window = cache.group.page_size, self.window or 0
        kernels.qk_norm_rope_write(qkv, H, G, d, vd, self.w_q_norm, self.w_k_norm, self.eps, *rope, ctx.positions, q,
                                   cache.kv, cache.group.slot_map, ps, cache.write, v_source, self.lam)
        attn = torch.empty((T, H * vd), dtype=x.dtype, device=x.device)
        if _TENSOR_CORES and kernels.sink_mma_supported(x.dtype, H, G, d, vd):
            # single tokens (all of the step, or the first ``num_decode`` of a mixed one) share their keys among CTAs
            args = (H, G, d, vd, ps, self.scale, window, self.sinks)
            nd = T if ctx.all_decode else getattr(ctx, "num_decode", 0)
            if nd:
                keys = ctx.max_context if ctx.all_decode else ctx.decode_max_context
                # a CTA of this kernel keeps two key tiles in flight and one warp busy per token: two CTAs on
                # every multiprocessor, about two tiles each
                splits = sink_decode_splits(nd * G, min(keys, window or keys))
                kernels.sink_attention_mma(q, attn, cache.kv, cache.group.block_table, ctx.cu_tokens, ctx.start_pos,
                                           nd, nd, *args, splits=splits)
            if nd < T:
                kernels.sink_attention_mma(q, attn, cache.kv, cache.group.block_table[nd:], ctx.cu_tokens[nd:],
                                           ctx.start_pos[nd:], ctx.num_requests - nd, T - nd, *args)
            return self.out.forward_partial(attn)
        kernels.sink_attention_generic(q, attn, cache.kv, cache.group.block_table, ctx.token_request, ctx.positions,
                                       H, G, d, vd, ps, self.scale, window, self.sinks)
        return self.out.forward_partial(attn)


def sink_decode_splits(ctas_without_split: int, max_keys: int) -> int:
    """CTAs per (token, KV head) of the tensor-core kernel for single tokens: as many as fill two CTAs on every
    multiprocessor and never one more (a CTA that waits for a free place doubles the launch's time), none with fewer
    than one tile of 64 keys, at most 64."""
    by_fill = max(1, 2 * kernels.sm_count() // max(1, ctas_without_split))
    by_work = max(1, (max_keys + 63) // 64)
    return max(1, min(by_fill, by_work, 64))
