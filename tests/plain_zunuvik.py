"""A plain, slow statement of the Zunuvik design: whole sequences, no cache, float64,
one function per mechanism.  It shares no code with the engine: it takes a plain
configuration dict and a dict of tensors by name.

Notation.  D width, T tokens of one sequence, positions 0..T-1.  A linear weight W is
stored [out, in] and applied as x @ W^T.

* offset norm:      n(x; w) = x / sqrt(mean(x^2) + eps) * (1 + w)
* plain norm:       m(x; w) = x / sqrt(mean(x^2) + eps) * w
* layer:            x += ls1 * mixer(n(x; norm1));  x += ls2 * ff(n(x; norm2))  (ff may be absent)
* latent attention: cq = m(Wdq h; dq.norm); q = Wuq cq, per head [dim | rot_dim];
                    Wdkv h = [c_raw (kv_rank) | kr (rot_dim)]; c = m(c_raw; dkv.norm);
                    k_h = Wuk_h c, v_h = Wuv_h c; rotation of q's rot part and of kr (pairs (2i, 2i+1),
                    angle p * base^(-2i/dims), the first ``dims`` elements only);
                    s_ij = (qn_i . k_j + qr_i . kr_j) * scale for j <= i; softmax; o = sum p v;
                    out = Wo (o * sigmoid(Wg h))
* mamba2:           Win h = [z | x | B | C | dt]; (x, B, C) <- silu(causal conv + bias);
                    dt <- softplus(dt + dt_bias); S <- exp(-exp(A_log) dt) S + dt B x^T; y = S^T C + D x;
                    y <- y * silu(z); grouped plain norm with '.norm'; out = Wo y
* dense ff:         Wdown (silu(Wgate h) * (Wup h))
* routed ff:        logits = Wr h + b; the ``top`` largest; weights = softmax over those; sum of the
                    chosen experts' outputs; + sigmoid(Wsg h) * shared(h) when a shared expert exists
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Sequence

import torch

F64 = torch.float64


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * (1.0 + w)


def plain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms_unit(x, eps) * w


def embed(table: torch.Tensor, tokens: Sequence[int], scale: float) -> torch.Tensor:
    return table[torch.as_tensor(list(tokens), dtype=torch.long)] * scale


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, ..., w]: the first ``dims`` elements of the last axis turn, pair (2i, 2i+1) by the
    angle position * base^(-2i/dims); the rest pass."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=F64)
    freq = torch.pow(torch.tensor(base, dtype=F64), -2.0 * i / dims)
    ang = positions.to(F64)[:, None] * freq[None, :]                # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = ang.cos().view(shape), ang.sin().view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                     positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h [T, D]; ``w`` holds the mixer's tensors by their short names (dq, dq.norm, uq, dkv, dkv.norm,
    uk, uv, g, o); ``m`` is the mixer's entry of the configuration."""
    T = h.shape[0]
    H, dn, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    cq = plain_norm(h @ w["dq"].t(), w["dq.norm"], eps)
    q = (cq @ w["uq"].t()).view(T, H, dn + dr)
    qn, qr = q[..., :dn], q[..., dn:]
    ckv = h @ w["dkv"].t()
    c = plain_norm(ckv[:, :r], w["dkv.norm"], eps)
    kr = ckv[:, r:]
    kn = (c @ w["uk"].t()).view(T, H, dn)
    v = (c @ w["uv"].t()).view(T, H, dv)
    base, dims = m["rot"]["base"], m["rot"]["dims"]
    qr = rotate_pairs(qr, pos, base, dims)
    kr = rotate_pairs(kr, pos, base, dims)
    s = (torch.einsum("ihd,jhd->hij", qn, kn) + torch.einsum("ihd,jd->hij", qr, kr)) * m["scale"]
    visible = pos[None, :] <= pos[:, None]
    s = s.masked_fill(~visible[None], -math.inf)
    p = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", p, v).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w["g"].t())
    return o @ w["o"].t()


def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h [T, D]; tensors by short name (in, conv, conv.b, dt_bias, A_log, D, norm, o)."""
    T = h.shape[0]
    nh, P, N, G, taps = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner = nh * P
    u = h @ w["in"].t()
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([torch.zeros(taps - 1, xbc.shape[1], dtype=h.dtype), xbc], dim=0)
    conv = torch.zeros_like(xbc)
    for k in range(taps):
        conv = conv + padded[k:k + T] * w["conv"][:, k][None, :]
    xbc = silu(conv + w["conv.b"][None, :])
    x = xbc[:, :inner].view(T, nh, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w["dt_bias"][None, :])                       # [T, nh]
    decay = torch.exp(-torch.exp(w["A_log"])[None, :] * dt)         # [T, nh]
    per_group = nh // G
    y = torch.zeros(T, nh, P, dtype=h.dtype)
    for hd in range(nh):
        g = hd // per_group
        S = torch.zeros(N, P, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.t() @ C[t, g] + w["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms_unit(y.view(T, ng, inner // ng), eps).reshape(T, inner) * w["norm"][None, :]
    return y @ w["o"].t()


def gated_ff(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor) -> torch.Tensor:
    return (silu(h @ gate.t()) * (h @ up.t())) @ down.t()


def routed_ff(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    """tensors by short name (router, router.b, e<i>.gate/up/down, shared.gate/up/down/sg)."""
    T = h.shape[0]
    E, top = f["router"]["experts"], f["router"]["top"]
    logits = h @ w["router"].t() + w["router.b"][None, :]
    val, idx = torch.topk(logits, top, dim=-1)
    wt = torch.softmax(val, dim=-1)
    out = torch.zeros(T, w["e0.down"].shape[0], dtype=h.dtype)
    for t in range(T):
        for k in range(top):
            e = int(idx[t, k])
            out[t] += wt[t, k] * gated_ff(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    if f.get("shared"):
        sg = torch.sigmoid(h @ w["shared.sg"].t())                  # [T, 1]
        out = out + sg * gated_ff(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


def _short(tensors: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[list] = None
            ) -> torch.Tensor:
    """float64 logits [T, vocab] of one sequence from position 0; ``layers_out`` (a list) takes the
    residual sum after every layer."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    eps = cfg["norm"]["eps"]
    x = embed(t["embed"], tokens, cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = offset_norm(x, t[p + "norm1"], eps)
        if layer["type"] == "latent_attention":
            d = latent_attention(h, _short(t, p + "mix."), layer["mixer"], eps)
        elif layer["type"] == "mamba2":
            d = mamba2(h, _short(t, p + "mix."), layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + d * t[p + "ls1"]
        f = layer.get("mlp")
        if f:
            h = offset_norm(x, t[p + "norm2"], eps)
            if f["kind"] == "dense":
                d = gated_ff(h, t[p + "mlp.gate"], t[p + "mlp.up"], t[p + "mlp.down"])
            elif f["kind"] == "moe":
                d = routed_ff(h, _short(t, p + "mlp."), f)
            else:
                raise ValueError(f["kind"])
            x = x + d * t[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return offset_norm(x, t["final.norm"], eps) @ t["head"].t()
