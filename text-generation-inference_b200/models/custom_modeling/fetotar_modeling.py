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
from ...utils.paged import HybridCacheManager, PagedKVState
from .python_step import PythonStep, _NoScratch

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


class _HeadView:
    """what FlashCausalLM reads on a model's vocabulary head: `.linear.weight` and `.should_gather`"""

    def __init__(self, weight):
        self.linear, self.should_gather = self, False
        self.weight = weight


class FetotarForCausalLM(nn.Module):
    ragged_steps = True           # FlashCausalLM.step_ragged: any mix of prompts, portions and decoded tokens in one batch
    logits_dtype = torch.float32
    scratch = _NoScratch()        # nothing of the fused step is ever re-allocated

    @property
    def fused_greedy_enabled(self) -> bool:
        """plain greedy decode of a stable batch runs as one CUDA graph (decode_advance + this forward + arg-max + the batch's
        bookkeeping), as for the other Python-driven families; B200_PY_FUSED_STEP=0 keeps it op by op"""
        return os.environ.get("B200_PY_FUSED_STEP", "") != "0"

    def __init__(self, config: FetotarConfig, weights):
        super().__init__()
        self.config = config
        self.process_group = weights.process_group
        self.device = torch.device(weights.device)
        self.dtype = weights.dtype
        self.model = FetotarModel(config, weights)
        self.head = weights.get_tensor("head").contiguous()
        self.lm_head = _HeadView(self.head)

    @property
    def kv_cache_manager(self):
        return self.model.kv_cache_manager

    @kv_cache_manager.setter
    def kv_cache_manager(self, manager):
        self.model.kv_cache_manager = manager

    def get_input_embeddings(self):
        return None  # prompt-tuning prefixes are not defined for a model with a per-layer token input

    def make_cache_manager(self, dtype, device, num_blocks: Optional[int], num_state_slots: Optional[int]) -> HybridCacheManager:
        specs = [layer.mixer.cache_spec() for layer in self.model.layers]
        slots = int(num_state_slots or 64)
        if num_blocks is None:
            per_block = sum(16 * s.row_width for s in specs if s.kind == "paged") * torch.empty(0, dtype=dtype).element_size()
            free, _ = torch.cuda.mem_get_info(device)
            num_blocks = max(int(free * 0.6) // max(per_block, 1), 1) if per_block else 1
            num_blocks = min(num_blocks, 1 << 22)
        return HybridCacheManager(specs, dtype, device, int(num_blocks), slots)

    # ---- the fused greedy step protocol of FlashCausalLM._decode_fused_greedy (python_step.py)
    def make_step(self, *, T: int, B: int, is_prefill: bool, max_s: int, input_ids, position_ids, kv: PagedKVState, cu_seqlens=None,
                  head_rows=None, logits=None, next_ids=None, inputs_embeds=None) -> PythonStep:
        if is_prefill or head_rows is not None or inputs_embeds is not None or T != B:
            raise NotImplementedError("the fused step is decode-only")
        for layer in self.model.layers:  # angle tables for every position the batch can reach: nothing grows inside a captured graph
            if hasattr(layer.mixer, "rotary"):
                layer.mixer.rotary.tables(int(max_s) + 1, self.device)
        cu_q = torch.arange(B + 1, dtype=torch.int32, device=self.device)
        return PythonStep(T=T, B=B, max_s=int(max_s) + 1, input_ids=input_ids, position_ids=position_ids, kv=kv, logits=logits,
                          next_ids=next_ids, banned=None, decode_marker=cu_q)

    def run_step(self, s: PythonStep) -> None:
        logits, _ = self.forward(s.input_ids, s.position_ids, None, s.decode_marker, s.max_s, None, s.kv)
        s.logits.copy_(logits)
        if s.next_ids is not None:
            lg = s.logits
            if s.banned is not None:  # per-row banned id of the arg-max (min_new_tokens EOS mask); -1 bans nothing
                ids = torch.arange(lg.shape[1], device=lg.device)
                lg = lg.masked_fill(ids[None, :] == s.banned[:, None], float("-inf"))
            torch.argmax(lg, dim=-1, out=s.next_ids)

    def forward(self, input_ids, position_ids, cu_seqlens, cu_seqlens_q, max_s, inputs_embeds: Optional[torch.Tensor] = None,
                past_key_values: Optional[PagedKVState] = None, pre_allocate_past_size: Optional[int] = None,
                lm_head_indices: Optional[torch.Tensor] = None):
        """Flash-family signature.  `cu_seqlens_q` None: every sequence brings its whole prompt (`cu_seqlens` are the row
        boundaries); otherwise `cu_seqlens_q` are the row boundaries of this step and each sequence's rows continue at
        `position_ids`.  -> (fp32 logits of the rows `lm_head_indices` (all rows when None), past_key_values)."""
        if inputs_embeds is not None:
            raise NotImplementedError("inputs_embeds: the per-layer token input needs token ids")
        kv = past_key_values
        if kv is None or kv.state_slots is None:
            raise ValueError("past_key_values must be a PagedKVState of the model's HybridCacheManager")
        cu_q = (cu_seqlens if cu_seqlens_q is None else cu_seqlens_q).to(torch.int32)
        T, B = input_ids.shape[0], cu_q.shape[0] - 1
        if T == B:  # one row per sequence
            seq_of_token = torch.arange(B, dtype=torch.int32, device=cu_q.device)
        else:
            counts = cu_q[1:] - cu_q[:-1]
            seq_of_token = torch.repeat_interleave(torch.arange(B, dtype=torch.int32, device=cu_q.device), counts.to(torch.int64),
                                                   output_size=T)
        step = ops.RaggedStep(T=T, B=B, position_ids=position_ids.contiguous(), cu_q=cu_q.contiguous(), seq_of_token=seq_of_token.contiguous(),
                              slot_mapping=kv.slot_mapping[:T].contiguous(), block_table=kv.block_table, state_slots=kv.state_slots)
        x = self.model(input_ids.contiguous(), step, int(max_s))
        if lm_head_indices is not None:
            x = x[lm_head_indices].contiguous()
        logits = ops.linear(self.model.final_norm(x), self.head, out_dtype=torch.float32)
        return logits, kv
