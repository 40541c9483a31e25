"""A feed-forward of routed experts with an optional shared expert.

    logits = Wr h + b (float32);  the ``top`` experts with the largest logits;  weights = softmax over those logits
    out = sum_k weight_k * expert_k(h)  +  sigmoid(wsg . h) * shared(h)
    expert(h) = Wdown (silu(Wgate h) * (Wup h)), no biases; the shared expert has the same form

Routing, ordering the (token, choice) pairs by expert, the grouped products and the weighted sum all stay on the
device (``csrc/moe.cu``): nothing is read back, so steps with routed experts replay as CUDA graphs.  The shared
expert is the dense gated feed-forward part with its own kernels.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from ..config.registry import register_part
from ..weights.loader import TensorSource, TensorSpec
from .base import FeedForward
from .mlp import SwiGLU


@register_part("feed_forward", "moe")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, expert_size: int, num_experts: int, top: int, shared_size: int = 0,
                 prefix: str = "mlp.", weight_suffix: str = ".weight", names=("gate", "up", "down")):
        if not (1 <= top <= num_experts) or top > kernels.MOE_MAX_TOP:
            raise ValueError(f"moe: top ({top}) must be between 1 and experts ({num_experts}), at most {kernels.MOE_MAX_TOP}")
        self.hidden_size, self.expert_size, self.num_experts, self.top = hidden_size, expert_size, num_experts, top
        self.prefix, self.sfx, self.names = prefix, weight_suffix, tuple(names)
        self.shared = SwiGLU(hidden_size, shared_size, prefix=f"{prefix}shared.", names=self.names,
                             weight_suffix=weight_suffix) if shared_size else None

    def tensor_specs(self) -> List[TensorSpec]:
        p, s, D, F = self.prefix, self.sfx, self.hidden_size, self.expert_size
        g, u, d = self.names
        specs = [TensorSpec(f"{p}router{s}", (self.num_experts, D), init="uniform:-0.5:0.5"),
                 TensorSpec(f"{p}router.b", (self.num_experts,), init="around_zero")]
        for e in range(self.num_experts):
            specs += [TensorSpec(f"{p}e{e}.{g}{s}", (F, D)), TensorSpec(f"{p}e{e}.{u}{s}", (F, D)),
                      TensorSpec(f"{p}e{e}.{d}{s}", (D, F))]
        if self.shared is not None:
            specs += self.shared.tensor_specs() + [TensorSpec(f"{p}shared.sg{s}", (1, D))]
        return specs

    def bind(self, source: TensorSource, dtype: torch.dtype, device: torch.device) -> None:
        p, s = self.prefix, self.sfx
        g, u, d = self.names
        get = lambda n: source.get(n).to(device=device, dtype=dtype)
        stack = lambda part: torch.stack([get(f"{p}e{e}.{part}{s}") for e in range(self.num_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack(g), stack(u), stack(d)          # [E, F, D], [E, F, D], [E, D, F]
        self.w_router = get(f"{p}router{s}").contiguous()
        self.b_router = source.get(f"{p}router.b").to(device=device, dtype=torch.float32).contiguous()
        self.w_sg = None
        if self.shared is not None:
            self.shared.bind(source, dtype, device)
            self.w_sg = get(f"{p}shared.sg{s}").reshape(-1).contiguous()

    def reset_after_fault(self) -> None:
        if self.shared is not None:
            self.shared.reset_after_fault()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        T, D = x.shape
        E, top, F = self.num_experts, self.top, self.expert_size
        n = T * top
        dev = x.device
        idx = torch.empty((T, top), dtype=torch.int32, device=dev)
        wt = torch.empty((T, top), dtype=torch.float32, device=dev)
        sgate = torch.empty((T,), dtype=torch.float32, device=dev) if self.shared is not None else None
        kernels.moe_route(x, self.w_router, self.b_router, self.w_sg, top, idx, wt, sgate)
        tile_rows = kernels.moe_tile_rows(n, E, D, F, x.dtype)   # rows of one expert a CTA takes
        max_tiles = n // tile_rows + E              # sum over experts of ceil(count / tile_rows) is at most this
        place = torch.empty((n,), dtype=torch.int32, device=dev)
        pair_at = torch.empty((n,), dtype=torch.int32, device=dev)
        meta = torch.empty((E + 2 + 3 * max_tiles,), dtype=torch.int32, device=dev)
        kernels.moe_sort(idx, E, tile_rows, max_tiles, place, pair_at, meta)
        act = torch.empty((n, F), dtype=x.dtype, device=dev)
        kernels.moe_gemm(x, pair_at, top, True, self.w_gate, self.w_up, act, meta, tile_rows, max_tiles)
        y = torch.empty((n, D), dtype=torch.float32, device=dev)
        kernels.moe_gemm(act, pair_at, top, False, self.w_down, None, y, meta, tile_rows, max_tiles)
        shared = self.shared.forward(x, ctx) if self.shared is not None else None
        out = torch.empty((T, D), dtype=torch.float32, device=dev)
        kernels.moe_combine(y, place, wt, shared, sgate, out)
        return out
