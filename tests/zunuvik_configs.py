"""Small Zunuvik configurations for the tests: every size and option differs between them, values that a
model may happen to make equal or 1 are unequal or not 1 somewhere (and 1 somewhere else)."""
import json
import os

import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, rot_dims=None, base=10000.0, scale=None):
    return {"type": "latent_attention", "mixer": {
        "heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
        "rot": {"base": base, "dims": rot_dims or rot_dim},
        "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}}


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": {"ff": shared} if shared else None}


def config(vocab, width, scale, eps, layers):
    return {"architecture": "Zunuvik", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps}, "layers": [dict(mix, mlp=mlp) for mix, mlp in layers]}


# attention first, a layer without feed-forward, experts without a shared one, part of the rotated key unrotated
ZP = config(300, 96, 6.0, 1e-6, [
    (latent(3, 24, 12, 16, 40, 56, rot_dims=8, base=500.0), moe(5, 2, 48)),
    (mamba(6, 16, 24, 3, 3, 1), None),
    (mamba(4, 20, 16, 1, 2, 4), dense(160)),
    (latent(5, 16, 8, 24, 32, 48), moe(4, 4, 40, shared=72)),
])
# state-space first, one expert per token, groups = heads, more heads than a CTA of the attention kernel has warps
ZQ = config(515, 128, 11.0, 2e-5, [
    (mamba(8, 8, 40, 8, 4, 2), moe(6, 1, 64, shared=32)),
    (latent(10, 8, 16, 8, 48, 64, base=100000.0, scale=0.3), dense(192)),
    (mamba(2, 64, 8, 2, 5, 1), dense(96)),
])
CONFIGS = {"P": ZP, "Q": ZQ}


def one_layer(mix, mlp, vocab=200, width=64, scale=4.0, eps=1e-5):
    return config(vocab, width, scale, eps, [(mix, mlp)])


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
    """For runs in bfloat16: routers whose choice no rounding can flip.  The biases lie 1.5 apart and the
    token-dependent part of the logits is small beside that, so every token takes the same experts (in an order
    and with weights that still depend on the token).  With random routers a bfloat16 run meets, every few
    hundred tokens, two logits closer than its rounding, takes the other expert, and differs from the plain
    statement by an expert's whole output: the float32 runs keep the random routers and check the choice."""
    for name in list(tensors):
        if name.endswith("mlp.router"):
            tensors[name] = (tensors[name].float() * 0.03).to(torch.bfloat16)
        elif name.endswith("mlp.router.b"):
            n = tensors[name].numel()
            order = torch.tensor([(3 * i + 1) % n if n % 3 else (i + 1) % n for i in range(n)])
            tensors[name] = (order.float() * 1.5).to(torch.bfloat16)
