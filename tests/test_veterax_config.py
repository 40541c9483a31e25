"""Veterax's configuration, description, cache layout and position tables (no GPU)."""
import copy
import math

import pytest
import torch

import plain_veterax as pv
import veterax_configs as vc
from qwen_decoder_b200.cache import CacheManager, PagedKV
from qwen_decoder_b200.config import ConfigError, config_from_dict, describe_model
from qwen_decoder_b200.parts.model import build_model
from qwen_decoder_b200.parts.rotary import Rotary


def test_round_trip_and_description():
    cfg = config_from_dict(vc.VA)
    assert cfg.architecture == "Veterax" and cfg.vocab_size == 300 and cfg.hidden_size == 96 and cfg.side_dim == 8
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = describe_model(cfg)
    assert spec.lm_head_tensor is None and len(spec.layers) == 5 and spec.embedding_scale == 1.0
    assert [l.block for l in spec.layers] == ["parallel_side"] * 5
    assert [l.mixer.name for l in spec.layers] == ["sink_attention"] * 5
    assert spec.layers[1].feed_forward is None and "post_mixer" not in spec.layers[1].norms
    # which layer blends its values, and which one is the source
    assert [l.mixer.params["value_mix"] for l in spec.layers] == [None, "v", "v", None, "v"]
    assert [l.mixer.params["value_mix_first"] for l in spec.layers] == [False, True, False, False, False]
    assert len(spec.positions) == 5          # five different rotations
    model = build_model(spec)
    names = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert names["l0.mix.q"] == (6 * 16, 96) and names["l0.mix.k"] == (3 * 16, 96) and names["l0.mix.v"] == (3 * 24, 96)
    assert names["l0.mix.o"] == (96, 6 * 24) and names["l0.mix.q.norm"] == (16,) and names["l0.mix.sink"] == (6,)
    assert "l0.mix.vmix" not in names and names["l1.mix.vmix"] == () and names["l4.mix.vmix"] == ()
    assert names["l0.mlp.router"] == (5 + 2, 96) and names["l0.mlp.correction"] == (7,) and "l0.mlp.router.b" not in names
    assert "l0.mlp.e4.gate" in names and "l0.mlp.e5.gate" not in names          # identity experts have no tensors
    assert names["l0.mlp.shared.down"] == (96, 24) and "l0.mlp.shared.sg" not in names and "l2.mlp.shared.gate" not in names
    assert "l1.norm2" not in names and names["l1.norm1.alpha"] == () and names["l1.norm1.b"] == (96,)
    assert names["side.embed"] == (300, 5 * 8) and names["l3.side.gate"] == (8, 96) and names["l3.side.proj"] == (96, 8)
    assert names["final.norm.alpha"] == () and "lm_head.weight" not in names and "head" not in names
    # without a token input nothing of it is declared
    names_b = {s.name for s in build_model(describe_model(config_from_dict(vc.VB))).tensor_specs()}
    assert not any("side" in n for n in names_b)


def test_cache_layout_keys_and_values_of_their_own_size():
    model = build_model(describe_model(config_from_dict(vc.VA)))
    layout = model.cache_layout()
    needs = [g.need for g in layout.groups]
    assert PagedKV(3, 16, None, v_dim=24) in needs and PagedKV(4, 16, None, v_dim=16) in needs and len(needs) == 5
    assert PagedKV(3, 16, None, v_dim=24).page_shape(8) == (3 * 8 * (16 + 24),)
    assert PagedKV(4, 16, None, v_dim=16).page_shape(8) == (2, 4, 8, 16) == PagedKV(4, 16).page_shape(8)
    assert CacheManager.bytes_per_page(layout, 16, torch.bfloat16) == \
        16 * 2 * (3 * (16 + 24) + 4 * (24 + 16) + 4 * (8 + 16) + 1 * (40 + 8) + 4 * (16 + 16))
    cm = CacheManager(layout, num_pages=8, page_size=16, max_requests=2)
    a = cm.open("a")
    cm.ensure(a, 40)
    cm.commit(a, 40)
    assert cm.free_pages() == [5] * 5
    cm.close(a)
    cm.check()


@pytest.mark.parametrize("scaling", [None, vc.yarn(4.0, 64, 16.0, 2.0), vc.yarn(5.0, 256, 20.0, 1.5)])
def test_position_tables_follow_the_stretched_frequencies(scaling):
    rot = {"base": 500.0, "dims": 24, "scaling": scaling}
    part = Rotary(head_dim=32, rotary_dim=24, base=500.0, pairing="adjacent", scaling=scaling)
    part.prepare(300, torch.device("cpu"))
    f, mag = pv.frequencies(rot)
    ang = torch.arange(300, dtype=torch.float64)[:, None] * f[None, :]
    assert torch.allclose(part.cos.double(), torch.cos(ang) * mag, atol=1e-6)
    assert torch.allclose(part.sin.double(), torch.sin(ang) * mag, atol=1e-6)
    if scaling is not None:
        assert mag == pytest.approx(0.1 * math.log(scaling["factor"]) + 1.0)
        plain, _ = pv.frequencies({"base": 500.0, "dims": 24, "scaling": None})
        assert f[0] == plain[0] and f[-1] == pytest.approx(float(plain[-1]) / scaling["factor"])   # fast pairs stay, slow ones stretch


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("vdim"), "vdim"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("fast"), "fast"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 8), "top"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][2]["mlp"].__setitem__("kind", "dense"), "kind"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("vdim", 24), "v_mix"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_errors_name_the_key(edit, word):
    cfg = copy.deepcopy(vc.VA)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)
