"""Dubesun: a decoder with learned absolute positions whose layers are parallel - x += mixer(n) + experts(n) with one norm
n = rms(x) (1 + w) read by both - around an fp32 residual stream.  The mixer of a layer is differential attention (optionally over
the keys and values of an earlier layer) or attention with a distance-bucket bias; the feed-forward is a mixture of clamped gated
experts.

config.json: {"architecture": "Dubesun", "vocab", "width", "max_positions", "norm": {"eps"}, "layers": [{"type": "attention" |
"attention_2", "mixer": {...sizes and constants of that mixer...}, "mlp": null | {"kind": "moe", "expert": {"ff", "limit"},
"router": {"experts", "top"}}}, ...]}.
  attention:   heads, kv_heads, dim, vdim, conv (taps), diff, scale, q_temp {coef, every}, optional kv_from (index of the layer
               whose cache rows it reads)
  attention_2: heads, kv_heads, dim, vdim (= dim: the values are the keys), scale, bias_max
Checkpoint tensors: `embed`, `pos`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.router`, `l<i>.mlp.e<j>.{gate,up,down}`, `final.norm`,
`head`.

The mixers and the routed feed-forward (utils/mixers.py) and their kernels know nothing of this family; this file reads the
configuration, loads the tensors under the family's names and composes the layers.  Steps are ragged (ragged_decoder.py).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ... import ops_seq as ops
from ...utils.mixers import BucketBiasAttention, DifferentialAttention, RoutedExperts
from ...utils.paged import HybridCacheManager
from .ragged_decoder import RaggedDecoderForCausalLM

ARCHITECTURE = "Dubesun"
MIXER_TYPES = ("attention", "attention_2")


class DubesunConfig:
    """config.json of the family, with the attribute names the runtime reads on any model config."""
    model_type = "dubesun"

    def __init__(self, raw: Dict[str, Any]):
        if raw.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = raw
        self.architecture = ARCHITECTURE
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.max_position_embeddings = int(raw["max_positions"])
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.num_hidden_layers = len(self.layers)
        self.norm_eps = float(raw["norm"]["eps"])
        self.eos_token_id = raw.get("eos_token_id")
        self.pad_token_id = raw.get("pad_token_id")
        self.quantize = None
        for i, layer in enumerate(self.layers):
            m = layer["mixer"]
            if layer["type"] not in MIXER_TYPES:
                raise NotImplementedError(f"mixer type {layer['type']!r}")
            if layer.get("mlp") and layer["mlp"].get("kind") != "moe":
                raise NotImplementedError(f"mlp kind {layer['mlp'].get('kind')!r}")
            if layer["type"] == "attention_2" and int(m.get("vdim", m["dim"])) != int(m["dim"]):
                raise ValueError(f"layer {i}: the values of attention_2 are its keys, vdim must equal dim")
            src = m.get("kv_from")
            if src is not None:
                s = self.layers[int(src)]["mixer"] if 0 <= int(src) < i else None
                if layer["type"] != "attention" or s is None or self.layers[int(src)]["type"] != "attention" or s.get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier attention layer that has keys and values of its own")
                if any(int(s[k]) != int(m[k]) for k in ("kv_heads", "dim", "vdim")):
                    raise ValueError(f"layer {i}: kv_from layer {src} has other key / value sizes")

    @classmethod
    def from_pretrained(cls, model_path: str) -> "DubesunConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            return cls(json.load(f))


def tensor_shapes(raw: Dict[str, Any], rel_rows: int = 32) -> Dict[str, tuple]:
    """name -> shape of every checkpoint tensor of a configuration (synthetic checkpoints, load-time validation); the number of
    distance buckets is a property of the `rel` tensors, not of the configuration"""
    W, V = int(raw["width"]), int(raw["vocab"])
    out = {"embed": (V, W), "pos": (int(raw["max_positions"]), W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(raw["layers"]):
        m = layer["mixer"]
        H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
        if layer["type"] == "attention_2":
            mix = {"q": (H * d, W), "q.b": (H * d,), "k": (G * d, W), "k.b": (G * d,), "rel": (rel_rows, H), "g": (H * d, W), "o": (W, H * d)}
        else:
            dv, taps = int(m["vdim"]), int(m["conv"])
            mix = {"q": (H * 2 * d, W), "q.conv": (H * 2 * d, taps), "q.norm": (d,), "lq1": (d,), "lk1": (d,), "lq2": (d,), "lk2": (d,),
                   "o": (W, H * dv)}
            if m.get("kv_from") is None:
                mix.update({"k": (G * 2 * d, W), "k.conv": (G * 2 * d, taps), "k.norm": (d,), "v": (G * dv, W), "v.conv": (G * dv, taps)})
        out[f"l{i}.norm1"] = (W,)
        out.update({f"l{i}.mix.{k}": v for k, v in mix.items()})
        f = layer.get("mlp")
        if f:
            E, ff = int(f["router"]["experts"]), int(f["expert"]["ff"])
            out[f"l{i}.mlp.router"] = (E, W)
            for e in range(E):
                out.update({f"l{i}.mlp.e{e}.gate": (ff, W), f"l{i}.mlp.e{e}.up": (ff, W), f"l{i}.mlp.e{e}.down": (W, ff)})
    return out


def build_mixer(kind: str, prefix: str, m: Dict[str, Any], weights, eps: float) -> nn.Module:
    if kind == "attention":
        temp = m.get("q_temp") or {}
        return DifferentialAttention(prefix, weights, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                     conv=int(m["conv"]), scale=float(m["scale"]), diff=float(m["diff"]), temp_coef=float(temp.get("coef", 0.0)),
                                     temp_every=int(temp.get("every", 0)), eps=eps, own_kv=m.get("kv_from") is None)
    if kind == "attention_2":
        return BucketBiasAttention(prefix, weights, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), scale=float(m["scale"]),
                                   bias_max=float(m["bias_max"]), eps=eps)
    raise NotImplementedError(f"mixer type {kind!r}")


class _OnePlusNorm(nn.Module):
    """x / sqrt(mean(x^2) + eps) * (1 + w) of the fp32 stream, in the projections' element type"""

    def __init__(self, name: str, weights, eps: float):
        super().__init__()
        self.w, self.eps = weights.get_tensor(name).contiguous(), eps

    def forward(self, x):
        return ops.rmsnorm_rows(x, self.w, self.eps, w_offset=1.0)


class DubesunLayer(nn.Module):
    def __init__(self, index: int, config: DubesunConfig, weights):
        super().__init__()
        spec, pre, eps = config.layers[index], f"l{index}", config.norm_eps
        self.index = index
        self.norm1 = _OnePlusNorm(f"{pre}.norm1", weights, eps)
        self.mixer = build_mixer(spec["type"], f"{pre}.mix", spec["mixer"], weights, eps)
        src = spec["mixer"].get("kv_from")
        self.kv_layer = index if src is None else int(src)   # whose pool the mixer reads (and, when its own, writes)
        self.mlp = None
        f = spec.get("mlp")
        if f:
            self.mlp = RoutedExperts(f"{pre}.mlp", weights, experts=int(f["router"]["experts"]), top=int(f["router"]["top"]),
                                     limit=float(f["expert"]["limit"]))

    def forward(self, x: torch.Tensor, step: ops.RaggedStep, manager: HybridCacheManager, max_s: int) -> None:
        """advances the fp32 stream x in place: both sublayers read the same normed input"""
        n = self.norm1(x)
        mix = self.mixer(n, step, manager.layer_pages(self.kv_layer), manager.layer_state(self.index), max_s)
        y, routing = self.mlp(n) if self.mlp is not None else (None, None)
        ops.moe_combine_add(x, mix, y, routing)


class DubesunModel(nn.Module):
    def __init__(self, config: DubesunConfig, weights):
        super().__init__()
        self.config = config
        self.embed = weights.get_tensor("embed").contiguous()
        self.pos = weights.get_tensor("pos").contiguous()
        if self.pos.shape[0] != config.max_position_embeddings:
            raise ValueError("pos: one row per position of max_positions expected")
        self.layers = nn.ModuleList(DubesunLayer(i, config, weights) for i in range(config.num_hidden_layers))
        self.final_norm = _OnePlusNorm("final.norm", weights, config.norm_eps)
        self.kv_cache_manager: Optional[HybridCacheManager] = None
        self.residual_probe: Optional[list] = None  # when a list: receives a copy of the stream after every layer (tests)

    def forward(self, input_ids, step: ops.RaggedStep, max_s: int) -> torch.Tensor:
        if int(max_s) > self.config.max_position_embeddings + 1:  # the fused decode step passes one more than the longest sequence
            raise ValueError(f"a sequence of {max_s} tokens exceeds the {self.config.max_position_embeddings} learned positions")
        x = ops.embed_add_pos(self.embed, self.pos, input_ids, step.position_ids)
        for layer in self.layers:
            layer(x, step, self.kv_cache_manager, max_s)
            if self.residual_probe is not None:
                self.residual_probe.append(x.clone())
        return x


class DubesunForCausalLM(RaggedDecoderForCausalLM):
    def __init__(self, config: DubesunConfig, weights):
        super().__init__(config, weights, DubesunModel(config, weights))
