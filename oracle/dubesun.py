"""Slow reference of the Dubesun decoder: plain PyTorch on the CPU, one function per mechanism, whole sequences at once.

Test infrastructure only.  It shares no code with the product path (no paged cache, no state slots, no kernels): every mixer
recomputes a sequence from its first token with a dense score matrix, so a test can compare any cut of a prompt, any batch and
any reuse of pages and slots in the product against it.  `dtype` is torch.float64 by default.

The model: x = embed[token] + pos[position]; every layer is parallel, x += mixer(n) + moe(n) with n = rms(x) * (1 + w); the
mixer is differential attention (two soft-max maps per head over the same values, short causal convolutions after the q / k / v
projections, a layer may read another layer's keys and values) or biased attention (values are the un-normed keys, a learned
bias per log-spaced distance bucket, sigmoid gate on the heads); logits = head (rms(x) * (1 + w_final)).

Checkpoint naming: `embed`, `pos`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.router`, `l<i>.mlp.e<j>.{gate,up,down}`, `final.norm`,
`head`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w)


def short_conv(u, w):
    """u [L, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the first row."""
    L, taps = u.shape[0], w.shape[1]
    pad = torch.cat([u.new_zeros(taps - 1, u.shape[1]), u], 0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + w[:, j] * pad[j:j + L]
    return y


def distance_bucket(n: int, rows: int, far: float) -> int:
    """row of the bias table for a key n positions back: one row per distance below rows/2, log-spaced rows from there to `far`"""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def causal_softmax(scores):
    """scores [H, L, L] (query, key) -> probabilities over keys j <= i"""
    L = scores.shape[-1]
    mask = torch.ones(L, L, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), -1)


def sub(sd: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


# ------------------------------------------------------------------------------------------------ mixers
def diff_attention_kv(h, p, m: dict, eps: float):
    """keys [L, G, 2, d] (after convolution and norm) and values [L, G, dv] (after convolution) of a layer that owns them"""
    L, G, d, dv = h.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = short_conv(h @ p["k"].T, p["k.conv"]).view(L, G, 2, d)
    v = short_conv(h @ p["v"].T, p["v.conv"]).view(L, G, dv)
    return unit_rms(k, eps) * p["k.norm"], v


def diff_attention(h, p, m: dict, eps: float, kv=None):
    """h [L, W] -> [L, W].  `kv`: (keys, values) of the layer this one shares with; None = its own."""
    L, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    k, v = kv if kv is not None else diff_attention_kv(h, p, m, eps)
    q = short_conv(h @ p["q"].T, p["q.conv"]).view(L, H, 2, d)
    q = unit_rms(q, eps) * p["q.norm"]
    pos = torch.arange(L, dtype=h.dtype)
    temp = 1.0 + float(m["q_temp"]["coef"]) * torch.log(torch.floor((pos + 1) / int(m["q_temp"]["every"])) + 1.0)
    q = q * temp[:, None, None, None]
    rep = H // G
    kh = k.repeat_interleave(rep, dim=1)    # [L, H, 2, d]
    vh = v.repeat_interleave(rep, dim=1)    # [L, H, dv]
    maps = []
    for mp in range(2):
        s = torch.einsum("ihd,jhd->hij", q[:, :, mp], kh[:, :, mp]) * float(m["scale"])
        maps.append(torch.einsum("hij,jhv->ihv", causal_softmax(s), vh))
    lam = torch.exp((p["lq1"] * p["lk1"]).sum()) - torch.exp((p["lq2"] * p["lk2"]).sum()) + float(m["diff"])
    o = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - float(m["diff"]))
    return o.reshape(L, H * dv) @ p["o"].T


def biased_attention(h, p, m: dict, eps: float):
    """h [L, W] -> [L, W]"""
    L, H, G, d = h.shape[0], m["heads"], m["kv_heads"], m["dim"]
    q = (h @ p["q"].T + p["q.b"]).view(L, H, d)
    k = (h @ p["k"].T + p["k.b"]).view(L, G, d)
    v = k
    q, kn = unit_rms(q, eps), unit_rms(k, eps)
    rep = H // G
    s = torch.einsum("ihd,jhd->hij", q, kn.repeat_interleave(rep, dim=1)) * float(m["scale"])
    rel = p["rel"]
    rows = rel.shape[0]
    bucket = torch.tensor([distance_bucket(n, rows, float(m["bias_max"])) for n in range(L)], dtype=torch.int64)
    dist = (torch.arange(L)[:, None] - torch.arange(L)[None, :]).clamp(min=0)
    s = s + rel[bucket[dist]].permute(2, 0, 1)
    o = torch.einsum("hij,jhv->ihv", causal_softmax(s), v.repeat_interleave(rep, dim=1)).reshape(L, H * d)
    return (o * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


def moe(h, p, f: dict, margins: Optional[list] = None):
    """h [L, W] -> [L, W]: the `top` experts with the largest router logits, weighted by the soft-max over those logits.
    `margins`, when a list, receives per row the gap between the last picked logit and the best one left out (inf when all are picked)"""
    E, top, limit = int(f["router"]["experts"]), int(f["router"]["top"]), float(f["expert"]["limit"])
    z = h @ p["router"].T
    val, idx = torch.topk(z, top, dim=-1)
    if margins is not None:
        margins.append(val[:, -1] - torch.topk(z, top + 1, dim=-1).values[:, -1] if top < E else torch.full_like(val[:, 0], float("inf")))
    wgt = torch.softmax(val, -1)
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0], dtype=h.dtype)
    for e in range(E):
        g = torch.clamp(h @ p[f"e{e}.gate"].T, max=limit)
        u = torch.clamp(h @ p[f"e{e}.up"].T, -limit, limit)
        y = (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p[f"e{e}.down"].T
        out = out + y * (wgt * (idx == e)).sum(-1, keepdim=True)
    return out


# ------------------------------------------------------------------------------------------------ the model
def forward(config: dict, sd: Dict[str, torch.Tensor], tokens: List[int], dtype=F64, residuals: Optional[list] = None,
            margins: Optional[list] = None):
    """logits [L, vocab] of one sequence; `residuals`, when a list, receives the stream after every layer, `margins` the routing
    margin of every position in every routed layer (a reduced-precision run may pick other experts where it is small)"""
    sd = {k: v.to(dtype) for k, v in sd.items()}
    eps = float(config["norm"]["eps"])
    ids = torch.tensor(tokens, dtype=torch.int64)
    L = ids.shape[0]
    x = sd["embed"][ids] + sd["pos"][:L]
    shared = {}
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], sub(sd, f"l{i}.mix.")
        n = norm_one_plus(x, sd[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                shared[i] = diff_attention_kv(n, p, m, eps)
            y = diff_attention(n, p, m, eps, shared[i if src is None else int(src)])
        elif layer["type"] == "attention_2":
            y = biased_attention(n, p, m, eps)
        else:
            raise NotImplementedError(layer["type"])
        if layer.get("mlp"):
            y = y + moe(n, sub(sd, f"l{i}.mlp."), layer["mlp"], margins)
        x = x + y
        if residuals is not None:
            residuals.append(x.clone())
    return norm_one_plus(x, sd["final.norm"], eps) @ sd["head"].T


# ------------------------------------------------------------------------------------------------ random models
def random_config(*, width: int = 40, vocab: int = 72, max_positions: int = 160, order=("attention_2", "attention", "attention"),
                  kv_from=(None, None, 1), heads=(6, 4), kv_heads=(2, 2), dim=(10, 12), vdim: int = 20, conv: int = 3, diff: float = 0.55,
                  every: int = 7, coef: float = 0.4, rel_rows: int = 12, bias_max: int = 40, experts: int = 5, top: int = 2, ff: int = 24,
                  limit: float = 1.25, with_mlp=None, eps: float = 1e-5) -> dict:
    """a small configuration; `heads`, `kv_heads`, `dim` are (biased attention, differential attention)"""
    layers = []
    for i, kind in enumerate(order):
        if kind == "attention_2":
            mixer = {"bias_max": bias_max, "dim": dim[0], "heads": heads[0], "kv_heads": kv_heads[0], "scale": dim[0] ** -0.5 * 1.7,
                     "vdim": dim[0], "rel_rows": rel_rows}
        else:
            mixer = {"conv": conv, "diff": diff, "dim": dim[1], "heads": heads[1], "kv_heads": kv_heads[1],
                     "q_temp": {"coef": coef, "every": every}, "scale": dim[1] ** -0.5 * 1.9, "vdim": vdim}
            if kv_from[i] is not None:
                mixer["kv_from"] = int(kv_from[i])
        has_mlp = True if with_mlp is None else with_mlp[i]
        mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}} if has_mlp else None
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    return {"architecture": "Dubesun", "layers": layers, "max_positions": max_positions, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V = int(config["width"]), int(config["vocab"])
    out = {"embed": (V, W), "pos": (int(config["max_positions"]), W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        m, pre = layer["mixer"], f"l{i}"
        out[f"{pre}.norm1"] = (W,)
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention_2":
            mix = {"q": (H * d, W), "q.b": (H * d,), "k": (G * d, W), "k.b": (G * d,), "rel": (int(m.get("rel_rows", 32)), H),
                   "g": (H * d, W), "o": (W, H * d)}
        else:
            taps = int(m["conv"])
            mix = {"q": (H * 2 * d, W), "q.norm": (d,), "q.conv": (H * 2 * d, taps), "lq1": (d,), "lk1": (d,), "lq2": (d,), "lk2": (d,),
                   "o": (W, H * dv)}
            if m.get("kv_from") is None:
                mix.update({"k": (G * 2 * d, W), "v": (G * dv, W), "k.norm": (d,), "k.conv": (G * 2 * d, taps), "v.conv": (G * dv, taps)})
        out.update({f"{pre}.mix.{k}": v for k, v in mix.items()})
        f = layer.get("mlp")
        if f:
            E, ff = int(f["router"]["experts"]), int(f["expert"]["ff"])
            out[f"{pre}.mlp.router"] = (E, W)
            for e in range(E):
                out.update({f"{pre}.mlp.e{e}.gate": (ff, W), f"{pre}.mlp.e{e}.up": (ff, W), f"{pre}.mlp.e{e}.down": (W, ff)})
    return out


def random_state_dict(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """weights that are exactly representable in bfloat16, so that every element type starts from the same numbers"""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".")[-1]
        if len(shape) == 2 and leaf not in ("conv", "rel"):
            t = torch.randn(shape, generator=g) * (1.5 / math.sqrt(shape[1]))
            if name in ("embed", "pos"):
                t = torch.randn(shape, generator=g) * 0.7
        elif leaf == "conv":
            t = torch.randn(shape, generator=g) * 0.6
        elif leaf == "rel":
            t = torch.randn(shape, generator=g) * 1.5
        elif leaf == "b":
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = torch.randn(shape, generator=g) * 0.3
        elif name.endswith(("q.norm", "k.norm")):
            t = 1.0 + torch.randn(shape, generator=g) * 0.3
        else:  # one-plus norm weights live around zero
            t = torch.randn(shape, generator=g) * 0.2
        sd[name] = t.to(torch.bfloat16).to(torch.float32)
    return sd
