"""Zunuvik's configuration, description and cache layout (no GPU)."""
import copy

import pytest
import torch

import zunuvik_configs as zc
from qwen_decoder_b200.cache import CacheManager, FixedState, PagedRows
from qwen_decoder_b200.config import ConfigError, config_from_dict, describe_model
from qwen_decoder_b200.parts.model import build_model


def test_round_trip_and_description():
    cfg = config_from_dict(zc.ZP)
    assert cfg.architecture == "Zunuvik" and cfg.vocab_size == 300 and cfg.hidden_size == 96
    assert config_from_dict(cfg.to_dict()) == cfg
    spec = describe_model(cfg)
    assert spec.embedding_scale == 6.0 and spec.lm_head_tensor == "head" and len(spec.layers) == 4
    assert [l.mixer.name for l in spec.layers] == ["latent_attention", "mamba2", "mamba2", "latent_attention"]
    assert spec.layers[1].feed_forward is None and spec.layers[0].feed_forward.name == "moe"
    assert len(spec.positions) == 2          # two different rotations
    model = build_model(spec)
    names = {s.name: tuple(s.shape) for s in model.tensor_specs()}
    assert names["l0.mix.dkv"] == (40 + 12, 96) and names["l0.mix.uq"] == (3 * 36, 56)
    assert names["l1.mix.in"] == (2 * 96 + 2 * 3 * 24 + 6, 96) and names["l1.mix.conv"] == (96 + 144, 3)
    assert "l1.norm2" not in names and "l1.ls2" not in names and "l1.ls1" in names
    assert names["l3.mlp.shared.sg"] == (1, 96) and "l0.mlp.shared.sg" not in names
    assert names["l0.mlp.e4.down"] == (96, 48) and names["final.norm"] == (96,) and names["head"] == (300, 96)


def test_cache_layout_rows_and_states():
    model = build_model(describe_model(config_from_dict(zc.ZP)))
    layout = model.cache_layout()
    assert [g.need for g in layout.groups] == [PagedRows(52), PagedRows(40)]
    assert layout.fixed_needs[0] == FixedState((6 * 16 * 24 + 2 * 240,), torch.float32)
    cm = CacheManager(layout, num_pages=8, page_size=16, max_requests=2)
    assert CacheManager.bytes_per_page(layout, 16, torch.bfloat16) == 16 * (52 + 40) * 2
    a = cm.open("a")
    cm.ensure(a, 40)
    cm.commit(a, 40)
    assert cm.free_pages() == [5, 5]
    cm.close(a)
    cm.check()


@pytest.mark.parametrize("edit, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 14), "dims"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("groups", 4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][2]["mlp"].__setitem__("kind", "glu"), "kind"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_errors_name_the_key(edit, word):
    cfg = copy.deepcopy(zc.ZP)
    edit(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert word in str(e.value)
