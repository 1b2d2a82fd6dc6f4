"""CPU tests of the hybrid families' host side: configuration reader and model choice, the block + state-slot manager, the
second library's build and binding table, and the slow reference against itself (prefix property of a causal model)."""
import os
import re

import pytest
import torch

from oracle import fetotar as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_config_reader_and_model_choice(tmp_path):
    import json
    import tgis_b200  # noqa: F401
    from tgis_b200.inference_engine import FLASH_TYPES, load_config
    cfg = orc.random_config(order=("mamba2", "latent_attention"), with_mlp=(True, False))
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    c = load_config(str(tmp_path))
    assert c.model_type == "fetotar" and c.model_type in FLASH_TYPES
    assert (c.vocab_size, c.hidden_size, c.num_hidden_layers) == (cfg["vocab"], cfg["width"], 2)
    assert c.layers[1]["mixer"]["mask"]["size"] == 9 and c.layers[0]["mlp"]["limit"] == 1.5
    bad = dict(cfg, layers=[{"type": "conv_only", "mixer": {}, "mlp": None}])
    from tgis_b200.models.custom_modeling.fetotar_modeling import FetotarConfig
    with pytest.raises(NotImplementedError):
        FetotarConfig(bad)


def test_seq_library_builds_and_exports_its_table():
    import tgis_b200  # noqa: F401
    from tgis_b200 import _lib
    lib = _lib.load_seq()
    for name in list(_lib.SEQ_SIGNATURES) + list(_lib._SEQ_SHARED):
        assert hasattr(lib, name), name
    header = open(os.path.join(ROOT, "include", "b200_seq.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(b200_seq_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.SEQ_SIGNATURES)


def test_hybrid_cache_manager_blocks_and_slots():
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.paged import HybridCacheManager, LayerCacheSpec, OutOfBlocks
    specs = [LayerCacheSpec("paged", row_width=20), LayerCacheSpec("state", state={"S": (2, 3, 4), "m": (2,)}), LayerCacheSpec("none")]
    mgr = HybridCacheManager(specs, torch.float32, "cpu", total_num_gpu_blocks=6, num_state_slots=2)
    assert mgr.layer_store(0).shape == (6, 16, 20) and mgr.layer_store(1)["S"].shape == (2, 2, 3, 4) and mgr.layer_store(2) is None
    assert mgr.block_bytes() == 16 * 20 * 4 and mgr.state_bytes_per_slot() == (24 + 2) * 4
    a, b = mgr.allocate_tokens([17, 1])
    assert mgr.free_blocks == 3 and mgr.free_state_slots == 0
    assert {mgr.state_slot(a), mgr.state_slot(b)} == {0, 1}
    with pytest.raises(OutOfBlocks):
        mgr.allocate_tokens([1])                      # no slot left; nothing is booked
    assert mgr.free_blocks == 3
    mgr.allocate_tokens([15, 15], [a, b])             # a: 32 tokens = 2 blocks (no new one), b: 16 tokens = 1 block
    assert mgr.free_blocks == 3 and mgr.sequence_length(a) == 32
    with pytest.raises(OutOfBlocks):
        mgr.allocate_tokens([16 * 3 + 1], [b])        # would need 4 more blocks
    assert mgr.sequence_length(b) == 16
    slots = mgr.slot_mapping_for([a], [15], [3]).tolist()
    blocks = mgr.sequence_blocks(a)
    assert slots == [blocks[0] * 16 + 15, blocks[1] * 16, blocks[1] * 16 + 1]
    slot_b = mgr.state_slot(b)
    mgr.free_sequences([b])
    assert mgr.free_state_slots == 1 and mgr.free_blocks == 4
    (c,) = mgr.allocate_tokens([40])
    assert mgr.state_slot(c) == slot_b and mgr.free_blocks == 1   # the freed slot and blocks are used again
    assert mgr.state_slots_tensor([c, a]).tolist() == [slot_b, mgr.state_slot(a)]
    mgr.free_sequences([a, c])
    assert mgr.free_blocks == 6 and mgr.free_state_slots == 2


def test_reference_is_causal_and_deterministic():
    cfg = orc.random_config()
    sd = orc.random_state_dict(cfg, seed=2)
    toks = torch.randint(0, cfg["vocab"], (40,), generator=torch.Generator().manual_seed(0)).tolist()
    full = orc.forward(cfg, sd, toks)
    assert torch.allclose(orc.forward(cfg, sd, toks[:25]), full[:25], atol=1e-9)
    assert set(orc.tensor_shapes(cfg)) == set(sd)
