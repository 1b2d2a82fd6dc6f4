"""Slow reference of the Fetotar decoder: plain PyTorch on the CPU, one function per mechanism, whole sequences at once.

Test infrastructure only.  It shares no code with the product path (no paged cache, no state slots, no kernels): every mixer here
recomputes a sequence from its first token, so a test can compare any cut of a prompt, any batch and any reuse of pages and
slots in the product against it.  `dtype` is torch.float64 by default: the product's 32-bit and bfloat16 results are both
compared with the same numbers.

Checkpoint naming: `embed`, `side.embed`, `l<i>.norm1[.b]`, `l<i>.norm1b[.b]`, `l<i>.norm2[.b]`, `l<i>.norm2b[.b]`,
`l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`, `l<i>.side.{gate,proj,norm}`, `final.norm[.b]`, `head`.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ small pieces
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def yarn_angles(n_pos: int, rot: dict, dtype=F64):
    """-> (cos, sin) [n_pos, dims/2], the YaRN attention factor already multiplied in."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    freq = base ** (-2.0 * i / dims)
    mscale = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def turn_dim(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
        hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        freq = freq / factor * ramp + freq * (1.0 - ramp)
        mscale = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(n_pos, dtype=dtype)[:, None] * freq[None, :]
    return torch.cos(ang) * mscale, torch.sin(ang) * mscale


def rotate_pairs(x, cos, sin):
    """x [L, ..., dims]: (x[2i], x[2i+1]) turned by the angle of (position, i).  cos / sin [L, dims/2]."""
    shape = x.shape
    a, b = x[..., 0::2], x[..., 1::2]
    while cos.dim() < a.dim():
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    return torch.stack((a * cos - b * sin, b * cos + a * sin), -1).reshape(shape)


# ------------------------------------------------------------------------------------------------ mixers
def latent_attention(h, p: Dict[str, torch.Tensor], m: dict, eps: float):
    """h [L, W] -> [L, W].  Low-rank queries, one shared latent per token for keys and values, one shared rotated key part,
    sliding window, gate on the concatenated heads."""
    L = h.shape[0]
    H, d, r, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = unit_rms(h @ p["dq"].T, eps) * p["dq.norm"]
    q = (cq @ p["uq"].T).view(L, H, d + r)
    kv = h @ p["dkv"].T
    c = unit_rms(kv[:, :R], eps) * p["dkv.norm"]
    k_rot = kv[:, R:]
    cos, sin = yarn_angles(L, m["rot"], h.dtype)
    nrot = int(m["rot"]["dims"])
    q_plain, q_rot = q[..., :d], q[..., d:].clone()
    q_rot[..., :nrot] = rotate_pairs(q_rot[..., :nrot], cos, sin)
    k_rot = k_rot.clone()
    k_rot[..., :nrot] = rotate_pairs(k_rot[..., :nrot], cos, sin)
    k_plain = (c @ p["uk"].T).view(L, H, d)
    v = (c @ p["uv"].T).view(L, H, dv)
    s = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * float(m["scale"])
    pos = torch.arange(L)
    dist = pos[:, None] - pos[None, :]
    hidden = (dist < 0) | (dist >= int(m["mask"]["size"]))
    s = s.masked_fill(hidden[None], float("-inf"))
    o = torch.einsum("hij,jhd->ihd", torch.softmax(s, -1), v).reshape(L, H * dv)
    return (o * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


def mamba2(h, p: Dict[str, torch.Tensor], m: dict, eps: float):
    """h [L, W] -> [L, W].  Selective state space, one decay per head and token, state [N, vdim] per head."""
    L = h.shape[0]
    H, P, N, G, taps, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner = H * P
    u = h @ p["in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    padded = torch.cat([xbc.new_zeros(taps - 1, xbc.shape[1]), xbc], 0)
    conv = p["conv.b"].expand(L, -1).clone()
    for j in range(taps):
        conv = conv + padded[j:j + L] * p["conv"][:, j]
    xbc = conv * torch.sigmoid(conv)
    x = xbc[:, :inner].view(L, H, P)
    Bm = xbc[:, inner:inner + G * N].view(L, G, N)
    Cm = xbc[:, inner + G * N:].view(L, G, N)
    dt = torch.nn.functional.softplus(dt + p["dt_bias"])
    decay = torch.exp(-torch.exp(p["A_log"]) * dt)  # [L, H]
    S = h.new_zeros(H, N, P)
    y = h.new_zeros(L, H, P)
    per_group = H // G
    grp = torch.arange(H) // per_group
    for t in range(L):
        Bt, Ct = Bm[t, grp], Cm[t, grp]  # [H, N]
        S = decay[t, :, None, None] * S + dt[t, :, None, None] * Bt[:, :, None] * x[t, :, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, Ct) + p["D"][:, None] * x[t]
    y = y.reshape(L, inner) * (z * torch.sigmoid(z))
    y = unit_rms(y.view(L, ng, inner // ng), eps).reshape(L, inner) * p["norm"]
    return y @ p["o"].T


def mlstm(h, p: Dict[str, torch.Tensor], m: dict, eps: float):
    """h [L, W] -> [L, W].  Matrix memory with exponential input gate, stabilised by a running maximum that starts at 0."""
    L = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ p["q"].T).view(L, H, d) * d ** -0.5
    k = (h @ p["k"].T).view(L, H, d)
    v = (h @ p["v"].T).view(L, H, dv)
    ig = cap * torch.tanh((h @ p["i"].T + p["i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ p["f"].T + p["f.b"]) / cap))
    S = h.new_zeros(H, d, dv)
    n = h.new_zeros(H, d)
    mx = h.new_zeros(H)
    out = h.new_zeros(L, H, dv)
    for t in range(L):
        m_new = torch.maximum(fg[t] + mx, ig[t])
        keep, take = torch.exp(fg[t] + mx - m_new), torch.exp(ig[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t, :, :, None] * v[t, :, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdp,hd->hp", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    o = unit_rms(out, eps).reshape(L, H * dv) * p["norm"]
    return (o * torch.sigmoid(h @ p["g"].T)) @ p["o"].T


def dense_ff(h, p: Dict[str, torch.Tensor], f: dict):
    lim = float(f["limit"])
    g = (h @ p["gate"].T).clamp(max=lim)
    u = (h @ p["up"].T).clamp(-lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T


def token_side(x, tokens, layer: int, table, p: Dict[str, torch.Tensor], dim: int, eps: float):
    e = table[tokens, layer * dim:(layer + 1) * dim]
    y = (gelu_tanh(x @ p["gate"].T) * e) @ p["proj"].T
    return x + unit_rms(y, eps) * p["norm"]


MIXERS = {"latent_attention": latent_attention, "mamba2": mamba2, "mlstm": mlstm}


# ------------------------------------------------------------------------------------------------ the model
def sub(sd: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in sd.items() if k.startswith(prefix)}


def forward(config: dict, sd: Dict[str, torch.Tensor], tokens: List[int], dtype=F64, residuals: Optional[list] = None):
    """-> logits [L, vocab] of one sequence.  `residuals`, when a list, receives the residual stream after every layer."""
    sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
    eps = float(config["norm"]["eps"])
    tok = torch.tensor(tokens, dtype=torch.long)
    x = sd["embed"][tok] * float(config["embedding"]["scale"])
    for i, layer in enumerate(config["layers"]):
        pre = f"l{i}."
        h = layer_norm(x, sd[pre + "norm1"], sd[pre + "norm1.b"], eps)
        mixed = MIXERS[layer["type"]](h, sub(sd, pre + "mix."), layer["mixer"], eps)
        x = x + layer_norm(mixed, sd[pre + "norm1b"], sd[pre + "norm1b.b"], eps)
        if layer.get("mlp"):
            h = layer_norm(x, sd[pre + "norm2"], sd[pre + "norm2.b"], eps)
            x = x + layer_norm(dense_ff(h, sub(sd, pre + "mlp."), layer["mlp"]), sd[pre + "norm2b"], sd[pre + "norm2b.b"], eps)
        x = token_side(x, tok, i, sd["side.embed"], sub(sd, pre + "side."), int(config["token_side"]["dim"]), eps)
        if residuals is not None:
            residuals.append(x.clone())
    x = layer_norm(x, sd["final.norm"], sd["final.norm.b"], eps)
    return x @ sd["head"].T


# ------------------------------------------------------------------------------------------------ random models for tests
def random_config(seed: int = 0, *, width: int = 64, vocab: int = 96, order=("mlstm", "latent_attention", "mamba2"), window: int = 9,
                  side_dim: int = 8, heads: int = 2, with_mlp=(False, True, False), yarn: bool = True) -> dict:
    """A small configuration whose sizes differ from one another wherever the design allows it."""
    layers = []
    for kind, has_mlp in zip(order, with_mlp):
        if kind == "mlstm":
            mixer = {"dim": 12, "gate_cap": 11.0, "heads": heads, "vdim": 20}
        elif kind == "mamba2":
            mixer = {"conv": 3, "groups": 1 if heads % 2 else 2, "heads": heads * 2, "norm_groups": 2, "state": 10, "vdim": 6}
        else:
            rot = {"base": 5000.0, "dims": 6}
            if yarn:
                rot["scaling"] = {"factor": 3.0, "fast": 24.0, "original": 64, "slow": 2.0}
            mixer = {"dim": 10, "heads": heads + 1, "kv_rank": 14, "mask": {"size": window}, "q_rank": 18, "rot": rot, "rot_dim": 6,
                     "scale": 0.21, "vdim": 12}
        layers.append({"type": kind, "mixer": mixer, "mlp": {"ff": 40, "kind": "dense", "limit": 1.5} if has_mlp else None})
    return {"architecture": "Fetotar", "embedding": {"scale": 3.0}, "layers": layers, "norm": {"eps": 1e-5},
            "token_side": {"dim": side_dim}, "vocab": vocab, "width": width}


def tensor_shapes(config: dict) -> Dict[str, tuple]:
    W, V, sd = config["width"], config["vocab"], config["token_side"]["dim"]
    shapes = {"embed": (V, W), "side.embed": (V, sd * len(config["layers"])), "final.norm": (W,), "final.norm.b": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        pre, m = f"l{i}.", layer["mixer"]
        names = ["norm1", "norm1b"] + (["norm2", "norm2b"] if layer.get("mlp") else [])
        for n in names:
            shapes[pre + n] = (W,)
            shapes[pre + n + ".b"] = (W,)
        if layer["type"] == "mlstm":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            mix = {"q": (H * d, W), "k": (H * d, W), "v": (H * dv, W), "g": (H * dv, W), "o": (W, H * dv), "norm": (H * dv,),
                   "i": (H, W), "i.b": (H,), "f": (H, W), "f.b": (H,)}
        elif layer["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            ch = H * P + 2 * G * N
            mix = {"in": (2 * H * P + 2 * G * N + H, W), "conv": (ch, m["conv"]), "conv.b": (ch,), "dt_bias": (H,), "A_log": (H,),
                   "D": (H,), "norm": (H * P,), "o": (W, H * P)}
        else:
            H, d, r, dv, R, Q = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            mix = {"dq": (Q, W), "dq.norm": (Q,), "uq": (H * (d + r), Q), "dkv": (R + r, W), "dkv.norm": (R,), "uk": (H * d, R),
                   "uv": (H * dv, R), "g": (H * dv, W), "o": (W, H * dv)}
        for n, s in mix.items():
            shapes[pre + "mix." + n] = s
        if layer.get("mlp"):
            ff = layer["mlp"]["ff"]
            shapes.update({pre + "mlp.gate": (ff, W), pre + "mlp.up": (ff, W), pre + "mlp.down": (W, ff)})
        shapes.update({pre + "side.gate": (sd, W), pre + "side.proj": (W, sd), pre + "side.norm": (W,)})
    return shapes


def random_state_dict(config: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors.  Matrices ~ N(0, 1/fan_in) scaled up a little so that gates and soft-max are not flat; norm weights
    around 1; decay parameters spread so that some heads forget fast and some keep long."""
    g = torch.Generator().manual_seed(seed)
    sd = {}
    for name, shape in tensor_shapes(config).items():
        leaf = name.split(".", 1)[1] if name.startswith("l") and name[1].isdigit() else name
        if len(shape) == 2 and not leaf.endswith("conv"):
            t = torch.randn(shape, generator=g) * (1.6 / math.sqrt(shape[1]))
            if name in ("embed", "side.embed"):
                t = torch.randn(shape, generator=g) * 0.5
        elif leaf.endswith("conv"):
            t = torch.randn(shape, generator=g) * 0.5
        elif leaf.endswith(".b") and "norm" in leaf:
            t = torch.randn(shape, generator=g) * 0.1
        elif leaf == "mix.i.b":
            t = torch.randn(shape, generator=g)
        elif leaf == "mix.f.b":
            t = torch.randn(shape, generator=g) + 3.0
        elif leaf == "mix.conv.b":
            t = torch.randn(shape, generator=g) * 0.2
        elif leaf == "mix.dt_bias":
            t = torch.randn(shape, generator=g) - 1.0
        elif leaf == "mix.A_log":
            t = torch.rand(shape, generator=g) * 2.0 - 1.5
        elif leaf == "mix.D":
            t = torch.randn(shape, generator=g) * 0.5 + 1.0
        else:  # norm weights
            t = 1.0 + torch.randn(shape, generator=g) * 0.1
        sd[name] = t.to(torch.bfloat16)
    return sd
