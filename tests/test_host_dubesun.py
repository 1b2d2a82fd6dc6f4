"""CPU tests of the Dubesun family's host side: configuration reader and model choice, checkpoint shapes, the distance buckets,
a cache manager whose paged layers keep state as well, and the slow reference against itself."""
import json

import pytest
import torch

from oracle import dubesun as orc


def test_config_reader_and_model_choice(tmp_path):
    import tgis_b200  # noqa: F401
    from tgis_b200.inference_engine import FLASH_TYPES, load_config
    from tgis_b200.models.custom_modeling.dubesun_modeling import DubesunConfig, tensor_shapes
    cfg = orc.random_config(order=("attention", "attention_2", "attention"), kv_from=(None, None, 0), with_mlp=(True, False, True))
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    c = load_config(str(tmp_path))
    assert c.model_type == "dubesun" and c.model_type in FLASH_TYPES
    assert (c.vocab_size, c.hidden_size, c.num_hidden_layers, c.max_position_embeddings) == (cfg["vocab"], cfg["width"], 3, cfg["max_positions"])
    assert c.layers[2]["mixer"]["kv_from"] == 0 and c.layers[1]["mlp"] is None
    # the product's table of checkpoint tensors is the reference's (the bucket count is a property of the rel tensor)
    assert tensor_shapes(cfg, rel_rows=12) == orc.tensor_shapes(cfg)
    assert "l2.mix.k" not in tensor_shapes(cfg) and "l0.mix.k" in tensor_shapes(cfg)
    for bad in (dict(cfg, layers=[{"type": "conv_only", "mixer": {}, "mlp": None}]),):
        with pytest.raises(NotImplementedError):
            DubesunConfig(bad)
    forward_ref = json.loads(json.dumps(cfg))
    forward_ref["layers"][0]["mixer"]["kv_from"] = 2          # a layer may only read an earlier one
    chained = json.loads(json.dumps(cfg))
    chained["layers"].append(json.loads(json.dumps(cfg["layers"][2])))
    chained["layers"][3]["mixer"]["kv_from"] = 2              # ... that has keys of its own
    other_sizes = json.loads(json.dumps(cfg))
    other_sizes["layers"][2]["mixer"]["vdim"] += 4
    not_keys = json.loads(json.dumps(cfg))
    not_keys["layers"][1]["mixer"]["vdim"] += 2               # attention_2 has no values of its own
    for bad in (forward_ref, chained, other_sizes, not_keys):
        with pytest.raises(ValueError):
            DubesunConfig(bad)


@pytest.mark.parametrize("rows,far", [(32, 240.0), (12, 40.0), (4, 9.0), (2, 5.0), (7, 100.0)])
def test_distance_buckets(rows, far):
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.mixers import log_distance_buckets
    tab = log_distance_buckets(rows, far)
    half = rows // 2
    assert tab[:half] == list(range(half)) and tab[half] == half           # one row per near distance, the log part starts on its own row
    assert all(b >= a for a, b in zip(tab, tab[1:])) and tab[-1] == rows - 1 and tab.count(rows - 1) == 1
    assert tab == [orc.distance_bucket(n, rows, far) for n in range(len(tab))]
    assert all(orc.distance_bucket(n, rows, far) == rows - 1 for n in (len(tab), len(tab) + 1, 10 * len(tab), int(far) + 1, 100000))
    assert len(tab) - 1 <= far                                             # the last row is reached at the far distance at the latest
    with pytest.raises(ValueError):
        log_distance_buckets(8, 4.0)


def test_cache_manager_paged_layers_with_state():
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.paged import HybridCacheManager, LayerCacheSpec
    specs = [LayerCacheSpec("paged", row_width=20, state={"conv": (2, 9)}), LayerCacheSpec("state", state={"conv": (2, 5)}),
             LayerCacheSpec("paged", row_width=6)]
    mgr = HybridCacheManager(specs, torch.float32, "cpu", total_num_gpu_blocks=5, num_state_slots=3)
    assert mgr.layer_pages(0).shape == (5, 16, 20) and mgr.layer_state(0)["conv"].shape == (3, 2, 9)
    assert mgr.layer_pages(1) is None and mgr.layer_state(1)["conv"].shape == (3, 2, 5)
    assert mgr.layer_pages(2).shape == (5, 16, 6) and mgr.layer_state(2) is None
    assert mgr.block_bytes() == 16 * 26 * 4 and mgr.state_bytes_per_slot() == (18 + 10) * 4
    a, b = mgr.allocate_tokens([17, 3])
    assert mgr.free_blocks == 2 and mgr.free_state_slots == 1
    mgr.free_sequences([a])
    (c,) = mgr.allocate_tokens([40])
    assert mgr.free_blocks == 1 and mgr.free_state_slots == 1 and mgr.state_slot(c) != mgr.state_slot(b)
    mgr.free_sequences([b, c])
    assert mgr.free_blocks == 5 and mgr.free_state_slots == 3


def test_reference_is_causal_and_its_mechanisms_are_live():
    cfg = orc.random_config()
    sd = orc.random_state_dict(cfg, seed=2)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(0)).tolist()
    full = orc.forward(cfg, sd, toks)
    assert torch.allclose(orc.forward(cfg, sd, toks[:25]), full[:25], atol=1e-9)
    assert set(orc.tensor_shapes(cfg)) == set(sd)
    # the convolution reaches taps - 1 rows back and not one more
    u, w = torch.randn(9, 4, dtype=torch.float64), torch.randn(4, 3, dtype=torch.float64)
    y = orc.short_conv(u, w)
    u2 = u.clone()
    u2[2] += 1.0
    d = (orc.short_conv(u2, w) - y).abs().sum(-1)
    assert all(d[i] > 0 for i in (2, 3, 4)) and all(d[i] == 0 for i in (0, 1, 5, 6))
    # the weights of the picked experts sum to one and only `top` experts contribute
    f = cfg["layers"][0]["mlp"]
    p = {k: v.double() for k, v in orc.sub(sd, "l0.mlp.").items()}
    h = torch.randn(6, cfg["width"], dtype=torch.float64)
    p1 = dict(p)
    z = h @ p["router"].T
    loser = int(z[0].argmin())
    p1[f"e{loser}.down"] = p[f"e{loser}.down"] * 3.0
    assert torch.allclose(orc.moe(h, p1, f)[0], orc.moe(h, p, f)[0])
