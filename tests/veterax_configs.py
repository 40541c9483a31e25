"""Small Veterax configurations for the tests: every size and option differs between them and from layer to layer;
values that a model may happen to make equal or 1 are unequal or not 1 somewhere (and equal or 1 somewhere else)."""
import json
import os

import torch


def attn(heads, kv_heads, dim, vdim, rot_dims=None, base=10000.0, scaling=None, scale=None, v_mix=False):
    return {"type": "attention", "mixer": {
        "heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "v_mix": v_mix,
        "rot": {"base": base, "dims": rot_dims or dim, "scaling": scaling},
        "scale": scale if scale is not None else dim ** -0.5}}


def yarn(factor, original, fast, slow):
    return {"factor": factor, "original": original, "fast": fast, "slow": slow}


def moe(experts, top, ff, limit, identity=0, shared=None):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "top": top, "identity": identity},
            "shared": {"ff": shared[0], "limit": shared[1]} if shared else None}


def config(vocab, width, eps, side, layers):
    return {"architecture": "Veterax", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "token_side": {"dim": side} if side else None, "layers": [dict(mix, mlp=mlp) for mix, mlp in layers]}


# values larger than keys, part of a head unrotated, stretched frequencies, identity experts, a layer without
# feed-forward, groups of one head, all experts chosen, the first mixing layer is not the first layer, a layer in
# between that does not mix, keys and values of one size
VA = config(300, 96, 1e-6, 8, [
    (attn(6, 3, 16, 24, rot_dims=8, base=500.0, scaling=yarn(4.0, 64, 16.0, 2.0), scale=0.3), moe(5, 2, 40, 1.0, identity=2, shared=(24, 0.7))),
    (attn(4, 4, 24, 16, v_mix=True), None),
    (attn(8, 4, 8, 16, base=77.0, scale=0.5, v_mix=True), moe(4, 4, 16, 2.5)),
    (attn(3, 1, 40, 8, rot_dims=16, scaling=yarn(2.0, 32, 8.0, 1.0)), moe(3, 1, 56, 0.8, identity=1, shared=(8, 3.0))),
    (attn(4, 4, 16, 16, base=1e6, v_mix=True), moe(6, 3, 24, 1.5, identity=3)),
])
# no token input, one key/value head for many query heads, head sizes that are no whole 16-byte pieces (the float32
# kernel serves them in bfloat16 too), heads of 128, every layer mixes
VB = config(515, 128, 2e-5, 0, [
    (attn(10, 1, 12, 20, rot_dims=4, base=300.0, v_mix=True), moe(7, 3, 32, 2.0, shared=(48, 1.0))),
    (attn(2, 1, 128, 20, scaling=yarn(6.0, 128, 24.0, 1.5), scale=0.1, v_mix=True), moe(2, 2, 64, 1.2, identity=2)),
    (attn(5, 1, 72, 20, rot_dims=36, v_mix=True), None),
])
CONFIGS = {"A": VA, "B": VB}


def one_layer(mix, mlp, vocab=200, width=64, eps=1e-5, side=0):
    return config(vocab, width, eps, side, [(mix, mlp)])


def make_folder(cfg: dict, path: str, seed: int, std: float = 0.12, edit=None) -> str:
    """A model folder with random bfloat16 weights, large enough that attention and routing are far from uniform.
    ``edit(tensors)`` may change tensors before they are written."""
    from qwen_decoder_b200.config import config_from_dict, describe_model
    from qwen_decoder_b200.parts.model import build_model
    from qwen_decoder_b200.weights import random_tensors
    from qwen_decoder_b200.weights.safetensors_io import save_safetensors
    typed = config_from_dict(cfg)
    model = build_model(describe_model(typed))
    tensors = random_tensors(model.tensor_specs(), seed, torch.bfloat16, "cpu", std, 0.1)
    if edit is not None:
        edit(tensors)
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(typed.to_dict(), f)
    save_safetensors(os.path.join(path, "model.safetensors"), tensors, {"format": "pt"})
    return path


def read_folder(path: str):
    """(config dict, {name: tensor}) with no code of the engine."""
    from safetensors import safe_open
    with open(os.path.join(path, "config.json")) as f:
        cfg = json.load(f)
    with safe_open(os.path.join(path, "model.safetensors"), framework="pt", device="cpu") as sf:
        tensors = {k: sf.get_tensor(k) for k in sf.keys()}
    return cfg, tensors


def steady_routing(tensors) -> None:
    """For runs in bfloat16: routers whose choice no rounding can flip.  The scores lie between 0 and 1; corrections
    that lie 1.5 apart decide the choice alone, so every token takes the same outputs (the last output, an identity
    one where there are any, then the first, then the last but one, ...), with weights that still depend on the token.  With random
    corrections a bfloat16 run meets, every few hundred tokens, two choice scores closer than its rounding, takes
    the other expert and differs from the plain statement by an expert's whole output: the float32 runs keep the
    random routers and check the choice."""
    for name in list(tensors):
        if name.endswith("mlp.correction"):
            n = tensors[name].numel()
            order = []                      # most preferred first: the last output, the first, the last but one, ...
            for j in range(n):
                order.append(n - 1 - j // 2 if j % 2 == 0 else j // 2)
            rank = torch.zeros(n)
            for j, e in enumerate(order):
                rank[e] = n - 1 - j
            tensors[name] = (rank * 1.5).to(torch.bfloat16)
