"""Fetotar: a hybrid decoder whose layers each pick one sequence mixer - matrix memory (mLSTM), latent attention with a sliding
window, or a selective state space (Mamba-2 form) - around an fp32 residual stream.

config.json: {"architecture": "Fetotar", "vocab", "width", "embedding": {"scale"}, "norm": {"eps"}, "token_side": {"dim"},
"layers": [{"type": "mlstm" | "latent_attention" | "mamba2", "mixer": {...sizes and constants of that mixer...},
"mlp": null | {"kind": "dense", "ff", "limit"}}, ...]}.  Checkpoint tensors: `embed`, `side.embed`, `l<i>.norm1[.b]`,
`l<i>.norm1b[.b]`, `l<i>.norm2[.b]`, `l<i>.norm2b[.b]`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`, `l<i>.side.{gate,proj,norm}`,
`final.norm[.b]`, `head`.

Graph of a layer (x is the fp32 stream, LN = layer norm with weight and bias):
    x += LN_1b(mixer(LN_1(x)));   x += LN_2b(mlp(LN_2(x)))  when the layer has an MLP;
    x += unit_rms(P (gelu_tanh(G x) * side_embed[token, layer's columns])) * w      (per-layer token input)
and x = embed[token] * scale before the first layer, logits = head LN_final(x) after the last.

The mixers (utils/mixers.py) and their kernels know nothing of this family; this file only reads the configuration, loads the
tensors under the family's names and composes the layers.  The model takes ragged steps (prompts, portions of prompts and single
decoded tokens in one batch): the forward has the flash families' signature and reads per-step indices from the batch's
`PagedKVState` (block table, slot mapping, state slots of utils/paged.py `HybridCacheManager`).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List, Optional

import torch
from torch import nn

from ... import ops_seq as ops
from ...utils.mixers import ClampedGatedMLP, LatentAttention, Mamba2Mixer, MLSTMMixer, ScaledRotaryTables
from ...utils.paged import HybridCacheManager
from .ragged_decoder import RaggedDecoderForCausalLM

ARCHITECTURE = "Fetotar"


class FetotarConfig:
    """config.json of the family, with the attribute names the runtime reads on any model config."""
    model_type = "fetotar"

    def __init__(self, raw: Dict[str, Any]):
        if raw.get("architecture") != ARCHITECTURE:
            raise ValueError(f"not a {ARCHITECTURE} configuration")
        self.raw = raw
        self.architecture = ARCHITECTURE
        self.vocab_size = int(raw["vocab"])
        self.hidden_size = int(raw["width"])
        self.layers: List[Dict[str, Any]] = list(raw["layers"])
        self.num_hidden_layers = len(self.layers)
        self.norm_eps = float(raw["norm"]["eps"])
        self.embedding_scale = float(raw["embedding"]["scale"])
        self.side_dim = int(raw["token_side"]["dim"])
        self.eos_token_id = raw.get("eos_token_id")
        self.pad_token_id = raw.get("pad_token_id")
        self.quantize = None
        for layer in self.layers:
            if layer["type"] not in ("mlstm", "latent_attention", "mamba2"):
                raise NotImplementedError(f"mixer type {layer['type']!r}")
            if layer.get("mlp") and layer["mlp"].get("kind", "dense") != "dense":
                raise NotImplementedError(f"mlp kind {layer['mlp']['kind']!r}")

    @classmethod
    def from_pretrained(cls, model_path: str) -> "FetotarConfig":
        with open(os.path.join(model_path, "config.json")) as f:
            return cls(json.load(f))


def tensor_shapes(raw: Dict[str, Any]) -> Dict[str, tuple]:
    """name -> shape of every checkpoint tensor of a configuration (synthetic checkpoints, load-time validation)"""
    W, V, side = int(raw["width"]), int(raw["vocab"]), int(raw["token_side"]["dim"])
    out = {"embed": (V, W), "side.embed": (V, side * len(raw["layers"])), "final.norm": (W,), "final.norm.b": (W,), "head": (V, W)}
    for i, layer in enumerate(raw["layers"]):
        m, mix = layer["mixer"], {}
        if layer["type"] == "mlstm":
            qk, vg = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            mix = {"q": (qk, W), "k": (qk, W), "v": (vg, W), "g": (vg, W), "i": (m["heads"], W), "i.b": (m["heads"],), "f": (m["heads"], W),
                   "f.b": (m["heads"],), "norm": (vg,), "o": (W, vg)}
        elif layer["type"] == "mamba2":
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            mix = {"in": (2 * inner + 2 * gn + m["heads"], W), "conv": (inner + 2 * gn, m["conv"]), "conv.b": (inner + 2 * gn,),
                   "dt_bias": (m["heads"],), "A_log": (m["heads"],), "D": (m["heads"],), "norm": (inner,), "o": (W, inner)}
        elif layer["type"] == "latent_attention":
            H = m["heads"]
            mix = {"dq": (m["q_rank"], W), "dq.norm": (m["q_rank"],), "uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                   "dkv": (m["kv_rank"] + m["rot_dim"], W), "dkv.norm": (m["kv_rank"],), "uk": (H * m["dim"], m["kv_rank"]),
                   "uv": (H * m["vdim"], m["kv_rank"]), "g": (H * m["vdim"], W), "o": (W, H * m["vdim"])}
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer.get("mlp") else [])
        for n in names:
            out[f"l{i}.{n}"] = (W,)
            out[f"l{i}.{n}.b"] = (W,)
        out.update({f"l{i}.mix.{k}": v for k, v in mix.items()})
        if layer.get("mlp"):
            ff = int(layer["mlp"]["ff"])
            out.update({f"l{i}.mlp.gate": (ff, W), f"l{i}.mlp.up": (ff, W), f"l{i}.mlp.down": (W, ff)})
        out.update({f"l{i}.side.gate": (side, W), f"l{i}.side.proj": (W, side), f"l{i}.side.norm": (W,)})
    return out


def build_mixer(kind: str, prefix: str, m: Dict[str, Any], weights, eps: float) -> nn.Module:
    if kind == "mlstm":
        return MLSTMMixer(prefix, weights, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), gate_cap=float(m["gate_cap"]), eps=eps)
    if kind == "mamba2":
        return Mamba2Mixer(prefix, weights, heads=int(m["heads"]), vdim=int(m["vdim"]), state=int(m["state"]), groups=int(m["groups"]),
                           conv=int(m["conv"]), norm_groups=int(m["norm_groups"]), eps=eps)
    rot = m["rot"]
    rotary = ScaledRotaryTables(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
    mask = m.get("mask") or {}
    return LatentAttention(prefix, weights, heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                           kv_rank=int(m["kv_rank"]), q_rank=int(m["q_rank"]), scale=float(m["scale"]), window=mask.get("size"),
                           rotary=rotary, eps=eps)


class _Norm(nn.Module):
    def __init__(self, name: str, weights, eps: float):
        super().__init__()
        self.w, self.b, self.eps = weights.get_tensor(name).contiguous(), weights.get_tensor(name + ".b").contiguous(), eps

    def forward(self, x):
        return ops.layernorm(x, self.w, self.b, self.eps)

    def add_into(self, y, residual, typed_copy: bool = False):
        return ops.layernorm_into_residual(y, self.w, self.b, self.eps, residual, typed_copy)


class FetotarLayer(nn.Module):
    def __init__(self, index: int, config: FetotarConfig, weights):
        super().__init__()
        spec, pre, eps = config.layers[index], f"l{index}", config.norm_eps
        self.index, self.eps, self.side_dim = index, eps, config.side_dim
        self.norm1, self.norm1b = _Norm(f"{pre}.norm1", weights, eps), _Norm(f"{pre}.norm1b", weights, eps)
        self.mixer = build_mixer(spec["type"], f"{pre}.mix", spec["mixer"], weights, eps)
        self.mlp = None
        if spec.get("mlp"):
            self.norm2, self.norm2b = _Norm(f"{pre}.norm2", weights, eps), _Norm(f"{pre}.norm2b", weights, eps)
            self.mlp = ClampedGatedMLP(f"{pre}.mlp", weights, limit=float(spec["mlp"]["limit"]))
        self.side_gate = weights.get_tensor(f"{pre}.side.gate").contiguous()
        self.side_proj = weights.get_tensor(f"{pre}.side.proj").contiguous()
        self.side_norm = weights.get_tensor(f"{pre}.side.norm").contiguous()

    def forward(self, x: torch.Tensor, input_ids, side_table, step: ops.RaggedStep, store, max_s: int) -> None:
        """advances the fp32 stream x in place"""
        x_t = self.norm1b.add_into(self.mixer(self.norm1(x), step, store, max_s), x, typed_copy=self.mlp is None)
        if self.mlp is not None:
            x_t = self.norm2b.add_into(self.mlp(self.norm2(x)), x, typed_copy=True)
        ops.token_side(x, x_t, input_ids, side_table, self.index * self.side_dim, self.side_dim, self.side_gate, self.side_proj,
                       self.side_norm, self.eps)


class FetotarModel(nn.Module):
    def __init__(self, config: FetotarConfig, weights):
        super().__init__()
        self.config = config
        self.embed = weights.get_tensor("embed").contiguous()
        self.side_table = weights.get_tensor("side.embed").contiguous()
        self.layers = nn.ModuleList(FetotarLayer(i, config, weights) for i in range(config.num_hidden_layers))
        self.final_norm = _Norm("final.norm", weights, config.norm_eps)
        self.kv_cache_manager: Optional[HybridCacheManager] = None
        self.residual_probe: Optional[list] = None  # when a list: receives a copy of the stream after every layer (tests)

    def forward(self, input_ids, step: ops.RaggedStep, max_s: int) -> torch.Tensor:
        x = ops.embed_scale(self.embed, input_ids, self.config.embedding_scale)
        for i, layer in enumerate(self.layers):
            layer(x, input_ids, self.side_table, step, self.kv_cache_manager.layer_store(i), max_s)
            if self.residual_probe is not None:
                self.residual_probe.append(x.clone())
        return x


class FetotarForCausalLM(RaggedDecoderForCausalLM):
    def __init__(self, config: FetotarConfig, weights):
        super().__init__(config, weights, FetotarModel(config, weights))
