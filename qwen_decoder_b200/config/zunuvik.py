"""``Zunuvik``: a hybrid decoder whose ``config.json`` lists its layers one by one.

Each entry of ``layers`` names a mixer (``latent_attention``: attention whose keys and values are
expanded from one cached low-rank row per token; ``mamba2``: a selective state-space recurrence with a
short causal convolution), the mixer's sizes, and a feed-forward (dense gated, a mixture of routed
experts with an optional always-on shared expert, or none).  Around them: an embedding times a
constant, pre-norm residual layers whose branches pass a per-channel layer scale, RMS norms whose
scales are stored around zero (the norm multiplies by 1 + w), a final norm and an output matrix.

Keys read from ``config.json``: ``architecture``, ``vocab``, ``width``, ``embedding.scale``,
``norm.eps``, ``layers[i].type`` / ``.mixer`` / ``.mlp`` (and, optional, ``max_positions`` and
``eos_token_id``).  Tensor names: ``embed``, ``l<i>.norm1|norm2|ls1|ls2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``; linear weights are [out, in] with no suffix.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping, Tuple

from .model_config import ConfigError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

DEFAULT_MAX_POSITIONS = 1 << 17        # the design has no position limit of its own: the engine's, unless 'max_positions' says otherwise

_MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"),
    "mamba2": ("heads", "vdim", "state", "groups", "conv", "norm_groups"),
}


def _need(d: Mapping[str, Any], key: str, where: str, kind=int):
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


def _check_layer(i: int, layer: Mapping[str, Any]) -> None:
    where = f"layers[{i}]"
    kind = layer.get("type") if isinstance(layer, Mapping) else None
    if kind not in _MIXER_KEYS:
        raise ConfigError(f"config.json: {where}.type must be one of {sorted(_MIXER_KEYS)}, got {kind!r}")
    m = layer.get("mixer")
    for k in _MIXER_KEYS[kind]:
        _need(m, k, f"{where}.mixer")
    if kind == "latent_attention":
        _need(m, "scale", f"{where}.mixer", float)
        rot = m.get("rot")
        dims = _need(rot, "dims", f"{where}.mixer.rot")
        if _need(rot, "base", f"{where}.mixer.rot", float) <= 0:
            raise ConfigError(f"config.json: {where}.mixer.rot.base must be positive")
        if dims % 2 or dims > m["rot_dim"]:
            raise ConfigError(f"config.json: {where}.mixer.rot.dims ({dims}) must be even and at most rot_dim")
    else:
        if m["heads"] % m["groups"]:
            raise ConfigError(f"config.json: {where}.mixer.groups must divide heads")
        if (m["heads"] * m["vdim"]) % m["norm_groups"]:
            raise ConfigError(f"config.json: {where}.mixer.norm_groups must divide heads * vdim")
    f = layer.get("mlp")
    if f is None:
        return
    fk = f.get("kind") if isinstance(f, Mapping) else None
    if fk == "dense":
        _need(f, "ff", f"{where}.mlp")
    elif fk == "moe":
        _need(f.get("expert"), "ff", f"{where}.mlp.expert")
        e = _need(f.get("router"), "experts", f"{where}.mlp.router")
        top = _need(f.get("router"), "top", f"{where}.mlp.router")
        if top > e:
            raise ConfigError(f"config.json: {where}.mlp.router.top ({top}) exceeds experts ({e})")
        if f.get("shared"):                     # absent, null or empty: no shared expert
            _need(f["shared"], "ff", f"{where}.mlp.shared")
    else:
        raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' or 'moe', got {fk!r}")


@dataclass(frozen=True)
class ZunuvikConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[dict, ...]
    max_position_embeddings: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "ZunuvikConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        for i, layer in enumerate(layers):
            _check_layer(i, layer)
        eps = _need(d.get("norm"), "eps", "norm", float)
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (eos,) if isinstance(eos, int) else tuple(eos)
        import copy
        return cls(architecture=d.get("architecture") or d["architectures"][0],
                   vocab_size=_need(d, "vocab", "config"), hidden_size=_need(d, "width", "config"),
                   embedding_scale=_need(d.get("embedding"), "scale", "embedding", float), norm_eps=eps,
                   layers=tuple(copy.deepcopy(layer) for layer in layers),
                   max_position_embeddings=d.get("max_positions") or DEFAULT_MAX_POSITIONS,
                   eos_token_ids=eos_ids)

    def to_dict(self) -> dict:
        import copy
        d = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "layers": [copy.deepcopy(layer) for layer in self.layers]}
        if self.max_position_embeddings != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_position_embeddings
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d


def describe_zunuvik(cfg: ZunuvikConfig) -> ModelSpec:
    D, eps = cfg.hidden_size, cfg.norm_eps
    norm = {"size": D, "eps": eps, "offset": 1.0}
    positions, layers = {}, []
    for i, layer in enumerate(cfg.layers):
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            rot = m["rot"]
            pname = f"rot{rot['dims']}of{m['rot_dim']}b{rot['base']!r}"
            positions.setdefault(pname, PartSpec("rotary", {
                "head_dim": m["rot_dim"], "rotary_dim": rot["dims"], "base": rot["base"], "pairing": "adjacent"}))
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "num_heads": m["heads"], "nope_dim": m["dim"], "rope_dim": m["rot_dim"],
                "v_dim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": m["scale"],
                "eps": eps, "position": pname, "prefix": "mix.", "weight_suffix": ""})
        else:
            mixer = PartSpec("mamba2", {
                "hidden_size": D, "num_heads": m["heads"], "head_dim": m["vdim"], "state_size": m["state"],
                "groups": m["groups"], "conv_taps": m["conv"], "norm_groups": m["norm_groups"], "eps": eps,
                "prefix": "mix.", "weight_suffix": ""})
        f = layer.get("mlp")
        if f is None:
            ff = None
        elif f["kind"] == "dense":
            ff = PartSpec("swiglu", {"hidden_size": D, "intermediate_size": f["ff"], "prefix": "mlp.",
                                     "names": ("gate", "up", "down"), "weight_suffix": ""})
        else:
            shared = f.get("shared")
            ff = PartSpec("moe", {"hidden_size": D, "expert_size": f["expert"]["ff"],
                                  "num_experts": f["router"]["experts"], "top": f["router"]["top"],
                                  "shared_size": shared["ff"] if shared else 0, "prefix": "mlp.",
                                  "weight_suffix": ""})
        norms = {"input": PartSpec("rmsnorm", dict(norm, tensor="norm1"))}
        if ff is not None:
            norms["post_mixer"] = PartSpec("rmsnorm", dict(norm, tensor="norm2"))
        layers.append(LayerSpec(prefix=f"l{i}.", block="pre_norm_scaled", mixer=mixer, feed_forward=ff,
                                norms=norms, block_params={"size": D, "prefix": ""}))
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab_size, max_positions=cfg.max_position_embeddings,
        embedding_tensor="embed", positions=positions, layers=layers,
        schedule=[ScheduleEntry(layer=i) for i in range(len(layers))],
        final_norm=PartSpec("rmsnorm", dict(norm, tensor="norm")), final_norm_prefix="final.",
        lm_head_tensor="head", embedding_scale=cfg.embedding_scale)


register_architecture("Zunuvik", ZunuvikConfig, describe_zunuvik)
