"""``Veterax``: a decoder whose ``config.json`` lists its layers one by one.

A layer runs two branches on the same residual sum, x += attention(n1(x)) + ff(n2(x)), where n is a norm without
statistics, tanh(alpha x) * w + b; then a per-layer token input joins: a slice of the token's row of a side table
gates a small projection of x, whose output is unit-normalised, scaled and added.  Attention is grouped-query
attention with unit-normalised queries and keys, rotary positions on the first ``rot.dims`` elements of a head
(adjacent pairs, frequencies stretched for long contexts by ``rot.scaling``), a sink in the softmax's denominator,
values of their own size, and, in layers that say ``v_mix``, values blended with those of the first such layer.  The
feed-forward is a mixture of experts with a clamped gate, a router that takes the softmax over all its outputs
(the last ``identity`` of which stand for the input itself), a correction that only the choice sees, and a shared
expert.  The output matrix is the embedding table.

Keys read from ``config.json``: ``architecture``, ``vocab``, ``width``, ``norm.eps``, ``token_side.dim`` (absent or
null: no token input), ``layers[i].type`` / ``.mixer`` / ``.mlp`` (and, optional, ``max_positions`` and
``eos_token_id``).  Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1|norm2`` (+ ``.b``, ``.alpha``),
``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.gate|proj|norm``, ``final.norm`` (+ ``.b``, ``.alpha``); linear weights
are [out, in] with no suffix.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DEFAULT_MAX_POSITIONS = 1 << 17        # the design has no position limit of its own: the engine's, unless 'max_positions' says otherwise
GATE_SLOPE = 1.702                     # the slope inside the sigmoid of an expert's gate: fixed by the design


def _need(d, key: str, where: str, kind=int):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where}: required key '{key}' is missing")
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
            raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
        return v
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
    return float(v)


def _check_layer(i: int, layer) -> None:
    where = f"layers[{i}]"
    kind = layer.get("type") if isinstance(layer, Mapping) else None
    if kind != "attention":
        raise ConfigError(f"config.json: {where}.type must be 'attention', got {kind!r}")
    m = layer.get("mixer")
    for k in ("heads", "kv_heads", "dim", "vdim"):
        _need(m, k, f"{where}.mixer")
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}.mixer.kv_heads ({m['kv_heads']}) must divide heads ({m['heads']})")
    _need(m, "scale", f"{where}.mixer", float)
    rot = m.get("rot")
    if rot is not None:
        dims = _need(rot, "dims", f"{where}.mixer.rot")
        if _need(rot, "base", f"{where}.mixer.rot", float) <= 0:
            raise ConfigError(f"config.json: {where}.mixer.rot.base must be positive")
        if dims % 2 or dims > m["dim"]:
            raise ConfigError(f"config.json: {where}.mixer.rot.dims ({dims}) must be even and at most dim")
        sc = rot.get("scaling")
        if sc is not None:
            for k in ("factor", "original", "fast", "slow"):
                if _need(sc, k, f"{where}.mixer.rot.scaling", float) <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.rot.scaling.{k} must be positive")
    f = layer.get("mlp")
    if f is None:
        return
    fk = f.get("kind") if isinstance(f, Mapping) else None
    if fk != "moe":
        raise ConfigError(f"config.json: {where}.mlp.kind must be 'moe', got {fk!r}")
    _need(f.get("expert"), "ff", f"{where}.mlp.expert")
    if _need(f.get("expert"), "limit", f"{where}.mlp.expert", float) <= 0:
        raise ConfigError(f"config.json: {where}.mlp.expert.limit must be positive")
    r = f.get("router")
    e, top = _need(r, "experts", f"{where}.mlp.router"), _need(r, "top", f"{where}.mlp.router")
    ident = r.get("identity") or 0
    if isinstance(ident, bool) or not isinstance(ident, int) or ident < 0:
        raise ConfigError(f"config.json: {where}.mlp.router.identity must be a non-negative integer, got {ident!r}")
    if top > e + ident:
        raise ConfigError(f"config.json: {where}.mlp.router.top ({top}) exceeds the router's outputs ({e + ident})")
    if f.get("shared"):                         # absent, null or empty: no shared expert
        _need(f["shared"], "ff", f"{where}.mlp.shared")
        if _need(f["shared"], "limit", f"{where}.mlp.shared", float) <= 0:
            raise ConfigError(f"config.json: {where}.mlp.shared.limit must be positive")


@dataclass(frozen=True)
class VeteraxConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    side_dim: int                       # 0: no per-layer token input
    layers: Tuple[dict, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VeteraxConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, layer in enumerate(layers):
            _check_layer(i, layer)
        mixing = [layer["mixer"] for layer in layers if layer["mixer"].get("v_mix")]
        if len({(m["kv_heads"], m["vdim"]) for m in mixing}) > 1:
            raise ConfigError("config.json: layers that say v_mix must agree on kv_heads and vdim (they blend values of one shape)")
        eps = _need(d.get("norm"), "eps", "norm", float)
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        side = d.get("token_side")
        side_dim = _need(side, "dim", "token_side") if side else 0
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        return cls(architecture=d.get("architecture") or d["architectures"][0],
                   vocab_size=_need(d, "vocab", "config"), hidden_size=_need(d, "width", "config"), norm_eps=eps,
                   side_dim=side_dim, layers=tuple(copy.deepcopy(layer) for layer in layers),
                   max_position_embeddings=d.get("max_positions") or DEFAULT_MAX_POSITIONS, eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "norm": {"eps": self.norm_eps}, "token_side": {"dim": self.side_dim} if self.side_dim else None,
             "layers": [copy.deepcopy(layer) for layer in self.layers]}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def describe_veterax(cfg: VeteraxConfig) -> ModelSpec:
    D, eps, L = cfg.hidden_size, cfg.norm_eps, len(cfg.layers)
    positions, layers = {}, []
    mix_seen = False
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        rot, pname = m.get("rot"), None
        if rot is not None:
            sc = rot.get("scaling")
            pname = f"rot{rot['dims']}of{m['dim']}b{rot['base']!r}" + \
                (f"s{sc['factor']!r}/{sc['original']!r}/{sc['fast']!r}/{sc['slow']!r}" if sc else "")
            positions.setdefault(pname, PartSpec("rotary", {
                "head_dim": m["dim"], "rotary_dim": rot["dims"], "base": rot["base"], "pairing": "adjacent",
                "scaling": dict(sc) if sc else None}))
        mixes = bool(m.get("v_mix"))
        mixer = PartSpec("sink_attention", {
            "hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
            "v_dim": m["vdim"], "scale": m["scale"], "eps": eps, "qk_norm": True, "sink": True,
            "value_mix": "v" if mixes else None, "value_mix_first": mixes and not mix_seen, "position": pname,
            "prefix": "mix.", "weight_suffix": ""})
        mix_seen = mix_seen or mixes
        f = layer.get("mlp")
        ff = None
        if f is not None:
            shared, r = f.get("shared"), f["router"]
            ff = PartSpec("moe", {
                "hidden_size": D, "expert_size": f["expert"]["ff"], "num_experts": r["experts"], "top": r["top"],
                "identity": r.get("identity") or 0, "routing": "softmax_all", "activation": "clamped",
                "limit": f["expert"]["limit"], "alpha": GATE_SLOPE, "shared_size": shared["ff"] if shared else 0,
                "shared_limit": shared["limit"] if shared else 0.0, "shared_gate": False, "prefix": "mlp.",
                "weight_suffix": ""})
        norms = {"input": PartSpec("dyntanh", {"size": D, "tensor": "norm1"})}
        if ff is not None:
            norms["post_mixer"] = PartSpec("dyntanh", {"size": D, "tensor": "norm2"})
        layers.append(LayerSpec(
            prefix=f"l{i}.", block="parallel_side", mixer=mixer, feed_forward=ff, norms=norms,
            block_params={"size": D, "eps": eps, "side_dim": cfg.side_dim, "side_index": i, "side_table": "side.embed",
                          "side_table_shape": (cfg.vocab_size, L * cfg.side_dim), "prefix": ""}))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding_tensor="embed", positions=positions, layers=layers,
        schedule=[ScheduleEntry(layer=i) for i in range(len(layers))],
        final_norm=PartSpec("dyntanh", {"size": D, "tensor": "norm"}), final_norm_prefix="final.",
        lm_head_tensor=None)


register_architecture("Veterax", VeteraxConfig, describe_veterax)
