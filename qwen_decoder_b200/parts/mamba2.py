"""The selective state-space mixer in its Mamba-2 form.

With h the mixer's input [T, D], ``num_heads`` heads of ``head_dim`` values (inner = heads * head_dim), a state
of ``state_size`` per value, ``groups`` groups of B and C shared by heads / groups heads each:

    Win h = [z (inner) | x (inner) | B (groups * N) | C (groups * N) | dt (heads)]
    (x, B, C) <- silu(causal convolution over ``conv_taps`` tokens per channel, with bias)
    dt <- softplus(dt + dt_bias);  S <- exp(-exp(A_log) dt) S + dt B x^T;  y = S^T C + D x       per head
    out = Wo (rms over each of ``norm_groups`` parts of (y * silu(z)) * w)

A request's state, one float32 row [S (heads * head_dim * N) | the last conv_taps - 1 convolution inputs], lives
in its state slot, starts at zero and is carried from step to step; a step may bring any number of a request's
tokens.  The projections' results are float32 and everything between them is float32 in both engine dtypes
(``csrc/mamba2.cu``).
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..cache import FixedState
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import Mixer, StateCacheView
from .linear import Linear


@register_part("mixer", "mamba2")
class Mamba2(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, state_size: int, groups: int, conv_taps: int,
                 norm_groups: int, eps: float, prefix: str = "mixer.", weight_suffix: str = ".weight"):
        if num_heads % groups or (num_heads * head_dim) % norm_groups:
            raise ValueError("mamba2: groups must divide heads, norm_groups must divide heads * head_dim")
        if state_size > 512:
            raise ValueError(f"mamba2: state_size {state_size} exceeds 512")
        self.hidden_size, self.num_heads, self.head_dim = hidden_size, num_heads, head_dim
        self.state_size, self.groups, self.conv_taps, self.norm_groups = state_size, groups, conv_taps, norm_groups
        self.eps = float(eps)
        self.inner = num_heads * head_dim
        self.channels = self.inner + 2 * groups * state_size
        self.prefix, self.sfx = prefix, weight_suffix
        self.inp = Linear(hidden_size, [(f"{prefix}in", 2 * self.inner + 2 * groups * state_size + num_heads)],
                          bias=False, weight_suffix=weight_suffix)
        self.out = Linear(self.inner, [(f"{prefix}o", hidden_size)], bias=False, weight_suffix=weight_suffix)
        self.ssm_floats = num_heads * head_dim * state_size

    def cache_need(self):
        return FixedState((self.ssm_floats + (self.conv_taps - 1) * self.channels,), torch.float32)

    def tensor_specs(self) -> List[TensorSpec]:
        p, nh = self.prefix, self.num_heads
        return self.inp.tensor_specs() + self.out.tensor_specs() + [
            TensorSpec(f"{p}conv", (self.channels, self.conv_taps), init="uniform:-0.5:0.5"),
            TensorSpec(f"{p}conv.b", (self.channels,), init="around_zero"),
            TensorSpec(f"{p}dt_bias", (nh,), init="uniform:-3.0:0.0"),
            TensorSpec(f"{p}A_log", (nh,), init="uniform:-1.0:1.5"),
            TensorSpec(f"{p}D", (nh,), init="around_one"),
            TensorSpec(f"{p}norm", (self.inner,), init="around_one")]

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        self.inp.bind(source, dtype, device)
        self.out.bind(source, dtype, device)
        p = self.prefix
        f32 = lambda n: source.get(n).to(device=device, dtype=torch.float32).contiguous()
        self.conv_w, self.conv_b = f32(f"{p}conv"), f32(f"{p}conv.b")
        self.dt_bias, self.A_log, self.D, self.norm_w = f32(f"{p}dt_bias"), f32(f"{p}A_log"), f32(f"{p}D"), f32(f"{p}norm")

    def forward(self, x: torch.Tensor, ctx, cache: StateCacheView) -> torch.Tensor:
        T, R = x.shape[0], ctx.num_requests
        inner, C, N, G = self.inner, self.channels, self.state_size, self.groups
        state = cache.state
        u = self.inp.forward(x, out_dtype=torch.float32)                    # [T, z | x B C | dt]
        xbc = torch.empty((T, C), dtype=torch.float32, device=x.device)
        kernels.mamba_conv(u, inner, C, self.conv_taps, self.conv_w, self.conv_b, state, self.ssm_floats,
                           ctx.token_request, ctx.cu_tokens, ctx.state_slots, xbc, R, cache.write)
        y = torch.empty((T, inner), dtype=torch.float32, device=x.device)
        kernels.mamba_scan(xbc, u, inner + C, self.dt_bias, self.A_log, self.D, state, ctx.cu_tokens, ctx.state_slots,
                           y, R, self.num_heads, self.head_dim, N, G, cache.write)
        h = torch.empty((T, inner), dtype=x.dtype, device=x.device)
        kernels.mamba_gate_norm(y, u, 0, self.norm_w, h, self.norm_groups, self.eps)
        return self.out.forward_partial(h)
