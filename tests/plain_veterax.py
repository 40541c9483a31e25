"""A plain, slow statement of the Veterax design: whole sequences, no cache, float64,
one function per mechanism.  It shares no code with the engine: it takes a plain
configuration dict and a dict of tensors by name.

Notation.  D width, T tokens of one sequence at positions 0..T-1.  A linear weight W is stored
[out, in] and applied as x @ W^T.

* unit(y)          = y / sqrt(mean(y^2) + eps)
* tanh norm:         n(x; w, b, a) = tanh(a x) * w + b            (a one number; no statistics)
* layer:             x += attention(n1(x)) + ff(n2(x))            (both branches read the same x)
                     then, with the layer's slice e of the token's row of the side table:
                     y = Wp (gelu(Wg x) * e);  x += unit(y) * ws
* attention:         q, k, v = Wq h, Wk h, Wv h per head; q <- unit(q) * wq, k <- unit(k) * wk (over the head);
                     the first ``dims`` elements of q and k turn in pairs (2i, 2i+1) by the angle p * f_i;
                     s_ij = (q_i . k_j) * scale for j <= i; p_ij = exp(s_ij) / (sum_j exp(s_ij) + exp(sink_h));
                     o_i = sum_j p_ij v_j; out = Wo o.  Query head h reads key/value head h // (H / G).
                     In layers that mix values, all but the first of them: v <- (1 - lam) v + lam v0, v0 the
                     first such layer's (unmixed) values of the same token.
* frequencies:       f_i = base^(-2i/dims); with scaling (factor, original, fast, slow):
                     c(t) = dims ln(original / (2 pi t)) / (2 ln base); lo = max(floor(c(fast)), 0);
                     hi = min(ceil(c(slow)), dims - 1); r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1);
                     f_i <- f_i / factor * r_i + f_i (1 - r_i); cos and sin times 0.1 ln(factor) + 1
* expert:            g = min(Wg h, L); u = clamp(Wu h, -L, L); Wd (g sigmoid(1.702 g) (u + 1))
* routed ff:         s = softmax(Wr h) over experts + identity outputs; the ``top`` largest of s + correction
                     are chosen; out = sum over the chosen of s_e * expert_e(h), where the last ``identity``
                     outputs stand for expert(h) = h; plus shared(h)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

F64 = torch.float64


def unit(y: torch.Tensor, eps: float) -> torch.Tensor:
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def tanh_norm(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    return torch.tanh(alpha * x) * w + b


def frequencies(rot: dict):
    """(f [dims / 2], magnitude): the turning rates of the pairs and what cos and sin are multiplied by."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor = float(sc["factor"])

    def c(t):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * t)) / (2.0 * math.log(base))
    lo = max(math.floor(c(float(sc["fast"]))), 0)
    hi = min(math.ceil(c(float(sc["slow"]))), dims - 1)
    r = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * r + f * (1.0 - r), 0.1 * math.log(factor) + 1.0


def turn(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, d]: pairs (2i, 2i+1) of the first ``dims`` elements turn by position * f_i."""
    dims = int(rot["dims"])
    f, mag = frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (torch.cos(ang) * mag)[:, None, :], (torch.sin(ang) * mag)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * cos - b * sin
    out[..., 1:dims:2] = b * cos + a * sin
    return out


def attention(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: dict, eps: float,
              v_first: Optional[torch.Tensor], mix: bool):
    """h [T, D] -> (out [T, D], the layer's own values before mixing [T, G, vdim])."""
    T = h.shape[0]
    H, G, d, vd = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v_raw = (h @ w[p + "v"].T).view(T, G, vd)
    q = unit(q, eps) * w[p + "q.norm"]
    k = unit(k, eps) * w[p + "k.norm"]
    pos = torch.arange(T)
    q, k = turn(q, pos, m["rot"]), turn(k, pos, m["rot"])
    v = v_raw
    if mix and v_first is not None:
        lam = w[p + "vmix"]
        v = (1.0 - lam) * v_raw + lam * v_first
    out = torch.zeros(T, H, vd, dtype=F64)
    causal = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * float(m["scale"])
        s = s.masked_fill(~causal, -math.inf)
        sink = w[p + "sink"][hq]
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        wts = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink - top))
        out[:, hq] = wts @ v[:, g]
    return out.reshape(T, H * vd) @ w[p + "o"].T, v_raw


def expert(h: torch.Tensor, wg, wu, wd, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ wg.T, max=limit)
    u = torch.clamp(h @ wu.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wd.T


def route(h: torch.Tensor, w_router, correction, top: int):
    """(chosen [T, top], their weights [T, top], all scores [T, outputs])."""
    s = torch.softmax(h @ w_router.T, dim=-1)
    chosen = torch.topk(s + correction, top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen), s


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, f: dict) -> torch.Tensor:
    E, ident, top = int(f["router"]["experts"]), int(f["router"].get("identity") or 0), int(f["router"]["top"])
    limit = float(f["expert"]["limit"])
    chosen, wt, _ = route(h, w[p + "router"], w[p + "correction"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(chosen[t, c])
            if e >= E:
                assert e < E + ident
                y = h[t]
            else:
                y = expert(h[t:t + 1], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], limit)[0]
            out[t] += wt[t, c] * y
    sh = f.get("shared")
    if sh:
        out = out + expert(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], float(sh["limit"]))
    return out


def side_input(x: torch.Tensor, tokens: torch.Tensor, w: Dict[str, torch.Tensor], layer: int, dim: int,
               eps: float) -> torch.Tensor:
    p = f"l{layer}.side."
    e = w["side.embed"][tokens][:, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return x + unit(y, eps) * w[p + "norm"]


def forward(cfg: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], return_layers: bool = False):
    """Logits [T, vocab] of one sequence (and, if asked, the residual sum after every layer [L, T, D])."""
    w = {n: t.to(F64) for n, t in weights.items() if t.dtype.is_floating_point}
    eps = float(cfg["norm"]["eps"])
    tok = torch.as_tensor(list(tokens), dtype=torch.long)
    x = w["embed"][tok]
    side = cfg.get("token_side")
    v_first = None
    after: List[torch.Tensor] = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        assert layer["type"] == "attention"
        h1 = tanh_norm(x, w[p + "norm1"], w[p + "norm1.b"], w[p + "norm1.alpha"])
        mix = bool(m.get("v_mix"))
        a, v_raw = attention(h1, w, p + "mix.", m, eps, v_first, mix)
        if mix and v_first is None:
            v_first = v_raw
        delta = a
        f = layer.get("mlp")
        if f is not None:
            h2 = tanh_norm(x, w[p + "norm2"], w[p + "norm2.b"], w[p + "norm2.alpha"])
            delta = delta + routed_ff(h2, w, p + "mlp.", f)
        x = x + delta
        if side:
            x = side_input(x, tok, w, i, int(side["dim"]), eps)
        after.append(x)
    hN = tanh_norm(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"])
    logits = hN @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
