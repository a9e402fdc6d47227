"""The Ripesun configuration reader on the CPU: what it builds from config.json, and what it refuses."""
import copy

import pytest

from aien_sovereign_core_mv_b200 import ConfigError, model_spec_for
from aien_sovereign_core_mv_b200.models.decoder import Decoder


def _latent(window, kv_from=None, kv_rank=24, rot_dim=8):
    m = {"heads": 3, "dim": 12, "rot_dim": rot_dim, "vdim": 10, "kv_rank": kv_rank, "q_rank": 20, "scale": 0.2,
         "rot": {"base": 10000.0, "dims": rot_dim}, "mask": {"size": window} if window else None}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


CONFIG = {"architecture": "Ripesun", "vocab": 101, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
          "residual_mult": 0.25, "logit_softcap": 9.0, "token_side": {"dim": 4}, "layers": [
              {"type": "mingru", "mixer": {"width": 40}, "mlp": {"kind": "dense", "ff": 64}},
              {"type": "latent_attention", "mixer": _latent(10), "mlp": None},
              {"type": "lightning", "mixer": {"heads": 2, "dim": 8, "vdim": 6, "decay": [0.5, 0.9]}, "mlp": {"kind": "dense", "ff": 32}},
              {"type": "latent_attention", "mixer": _latent(33, kv_from=1), "mlp": {"kind": "dense", "ff": 32}},
              {"type": "latent_attention", "mixer": _latent(10), "mlp": {"kind": "dense", "ff": 32}}]}


def test_spec_parts_run_list_and_tensor_names():
    cfg, spec = model_spec_for(CONFIG)
    assert cfg.num_hidden_layers == 5 and cfg.residual_mult == 0.25 and cfg.side_dim == 4
    assert [l.block for l in spec.layers] == ["sandwich", "sandwich_mixer", "sandwich", "sandwich", "sandwich"]
    assert [(r.cache, r.writes_cache) for r in spec.run_list] == [(0, True), (1, True), (2, True), (1, False), (4, True)]
    # the shared cache keeps the widest window of its readers; the layer's own mask stays its own
    assert spec.layers[1].mixer.params["window"] == 10 and spec.layers[1].mixer.params["cache_window"] == 33
    assert spec.layers[3].mixer.params["window"] == 33 and not spec.layers[3].mixer.params["own_cache"]
    assert spec.layers[4].mixer.params["cache_window"] == 10
    model = Decoder(spec)
    cat = model.catalog()
    assert cat["embed"][0] == (101, 48) and cat["side.embed"][0] == (101, 20) and cat["head"][0] == (101, 48)
    assert cat["l0.mix.z.b"][0] == (40,) and cat["l1.mix.dkv"][0] == (32, 48) and cat["l1.mix.dkv.norm"][0] == (24,)
    assert "l3.mix.dkv" not in cat and cat["l3.mix.uk"][0] == (36, 24) and cat["l3.mix.sink"][0] == (3,)
    assert "l1.mlp.up" not in cat and "l1.norm2" not in cat and cat["l1.side.gate"][0] == (4, 48)
    assert cat["l2.mix.norm"][0] == (12,) and cat["l2.norm1b"][0] == (48,)
    kinds = [(n.kind, n.window) for n in model.group_needs]
    assert ("state", 0) in kinds and ("window", 33) in kinds and ("window", 10) in kinds
    # layers 1 and 3 share planes; layer 4 has its own
    assert model.bindings[3].group == model.bindings[1].group and model.bindings[3].slot == model.bindings[1].slot
    assert not model.bindings[3].writes and model.bindings[4].group != model.bindings[1].group


def test_optional_keys_may_be_absent():
    raw = copy.deepcopy(CONFIG)
    for key in ("embedding", "residual_mult", "logit_softcap", "token_side"):
        del raw[key]
    cfg, spec = model_spec_for(raw)
    assert cfg.embedding_scale == 1.0 and cfg.residual_mult == 1.0 and cfg.logit_softcap == 0.0 and cfg.side_dim == 0
    assert "side.embed" not in Decoder(spec).catalog()


def test_config_errors_name_the_field():
    bad = copy.deepcopy(CONFIG); bad["layers"][0]["type"] = "conv"
    with pytest.raises(ConfigError, match=r"layers\[0\]\.type"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIG); del bad["layers"][1]["mixer"]["q_rank"]
    with pytest.raises(ConfigError, match=r"layers\[1\]\.mixer\.q_rank"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIG); bad["layers"][3]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError, match=r"layers\[3\]\.mixer\.kv_from"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIG); bad["layers"][3]["mixer"]["kv_rank"] = 16
    with pytest.raises(ConfigError, match="kv_rank"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIG); bad["layers"][2]["mixer"]["decay"] = [0.5]
    with pytest.raises(ConfigError, match=r"layers\[2\]\.mixer\.decay"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIG); bad["layers"][0]["mlp"]["kind"] = "moe"
    with pytest.raises(ConfigError, match=r"layers\[0\]\.mlp\.kind"):
        model_spec_for(bad)
    bad = copy.deepcopy(CONFIG); del bad["norm"]
    with pytest.raises(ConfigError, match="norm"):
        model_spec_for(bad)
