"""Dubesun on the GPU against the slow CPU reference (oracle/dubesun.py, float64): each mechanism alone, then the model through
the engine's step function and cache manager - whole prompts, token-by-token decoding, portions down to two tokens, ragged
batches, pages and state slots that are freed and used again - and greedy generation through FlashCausalLM.generate_token.

The configurations are small and uneven (key size != value size, head counts that differ between the two kinds of attention, one
and several query heads per key head, one to four convolution taps, one expert per token and all experts per token).  Where
random weights would hide a fault the test makes it show: a key that must win the soft-max from far away, at a page border or at
the first positions; a bias table with one loud row, so that a key on the wrong side of a bucket's edge moves the output; a query
temperature that changes inside the decoded tokens."""
import copy
import json
import os

import pytest
import torch

from oracle import dubesun as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL32, TOL16 = 2e-4, 0.3


# ------------------------------------------------------------------------------------------------ helpers
def _model(tmp_path, config, sd, dtype=torch.float32, blocks=64, slots=4):
    from safetensors.torch import save_file
    import tgis_b200  # noqa: F401
    from tgis_b200.inference_engine import InferenceEngine
    from tgis_b200.models.flash_causal_lm import FlashCausalLM
    from tgis_b200.utils.dist import FakeGroup
    from tgis_b200.utils.synthetic import make_tokenizer
    from tgis_b200.utils.weights import Weights

    d = str(tmp_path)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    path = os.path.join(d, "model.safetensors")
    save_file({k: v.contiguous() for k, v in sd.items()}, path)
    weights = Weights([path], device=DEV, dtype=dtype, process_group=FakeGroup(0, 1))
    engine = InferenceEngine(d, None, dtype, None, None, None, weights=weights, tokenizer=make_tokenizer(config["vocab"]))
    return FlashCausalLM(d, None, "tgis_native", dtype, None, None, engine=engine, num_kv_blocks=blocks, num_state_slots=slots)


def _tokens(seed, n, vocab):
    return torch.randint(4, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _rel(got, ref):
    """largest row error relative to the spread of the reference logits"""
    got, ref = got.double().cpu(), ref.double()
    return float(((got - ref).pow(2).mean(-1).sqrt() / ref.std()).max())


def _decided(config, sd, tokens, least=0.1):
    """positions whose routing is no close call in any layer: where bfloat16 must pick the reference's experts"""
    margins = []
    orc.forward(config, sd, tokens, margins=margins)
    return torch.stack(margins).min(0).values > least


def _run_cut(model, tokens, cuts):
    """one sequence in portions of the given sizes (the rest token by token) -> logits of every position"""
    sid, at, rows = None, 0, []
    sizes = list(cuts) + [1] * (len(tokens) - sum(cuts))
    for n in sizes:
        sids, lg = model.step_ragged([sid], [tokens[at:at + n]])
        sid, at = sids[0], at + n
        rows.append(lg)
    model.kv_cache_manager.free_sequences([sid])
    return torch.cat(rows)


class _DictWeights:
    def __init__(self, sd, dtype):
        from tgis_b200.utils.dist import FakeGroup
        self.sd, self.dtype, self.device, self.process_group = sd, dtype, DEV, FakeGroup(0, 1)

    def get_tensor(self, name):
        return self.sd[name].to(self.dtype).to(DEV)


def _step(starts_and_counts, tables):
    """RaggedStep for sequences (start, count) whose pages are given by `tables` (one list of block ids per sequence)"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq
    pos, seq, slots, cu = [], [], [], [0]
    for b, (start, n) in enumerate(starts_and_counts):
        for p in range(start, start + n):
            pos.append(p)
            seq.append(b)
            slots.append(tables[b][p // 16] * 16 + p % 16)
        cu.append(cu[-1] + n)
    width = max(len(t) for t in tables)
    bt = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    return ops_seq.RaggedStep(T=len(pos), B=len(tables), position_ids=torch.tensor(pos, dtype=torch.int64, device=DEV),
                              cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), seq_of_token=torch.tensor(seq, dtype=torch.int32, device=DEV),
                              slot_mapping=torch.tensor(slots, dtype=torch.int64, device=DEV), block_table=bt.to(DEV),
                              state_slots=torch.arange(len(tables), dtype=torch.int32, device=DEV))


# ------------------------------------------------------------------------------------------------ mechanisms alone
def test_row_kernels_match_reference():
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(0)
    T, W, V, P = 9, 50, 30, 40
    x = torch.randn(T, W, generator=g) * 3
    w = torch.randn(W, generator=g) * 0.2
    for offset in (1.0, 0.0):
        ref = orc.unit_rms(x.double(), 1e-5) * (w.double() + offset)
        got = ops.rmsnorm_rows(x.to(DEV), w.to(DEV), 1e-5, w_offset=offset)
        assert torch.allclose(got.cpu().double(), ref, atol=1e-5)
    # a bfloat16 weight near zero keeps its digits: the offset is added in fp32, not stored in the weight
    wb = w.bfloat16()
    got = ops.rmsnorm_rows(x.to(DEV), wb.to(DEV), 1e-5, w_offset=1.0).float().cpu()
    ref = (orc.unit_rms(x.double(), 1e-5) * (wb.double() + 1.0)).float()
    assert torch.allclose(got, ref.bfloat16().float(), atol=0.05) and float((got - ref).abs().max()) < 0.05
    table, ptab = torch.randn(V, W, generator=g), torch.randn(P, W, generator=g)
    ids, pos = torch.randint(0, V, (T,), generator=g), torch.randint(0, P, (T,), generator=g)
    got = ops.embed_add_pos(table.to(DEV), ptab.to(DEV), ids.to(DEV), pos.to(DEV))
    assert torch.equal(got.cpu(), table[ids] + ptab[pos])
    H, dv, lam = 3, 20, 0.37
    a = torch.randn(T, H * 2, dv, generator=g)
    a4 = a.view(T, H, 2, dv).double()
    ref = (orc.unit_rms(a4[:, :, 0] - lam * a4[:, :, 1], 1e-5) * 0.45).reshape(T, H * dv)
    got = ops.diff_combine(a.to(DEV), H, dv, lam, 0.45, 1e-5, torch.float32)
    assert torch.allclose(got.cpu().double(), ref, atol=1e-5)


@pytest.mark.parametrize("taps", [1, 2, 4])
def test_convolution_without_activation_any_cut(taps):
    """two sequences in unequal portions: the last taps - 1 rows of a sequence come back from its state slot"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(taps)
    C, lens = 37, [23, 9]
    us = [torch.randn(L, C + 5, generator=g) for L in lens]
    w = torch.randn(C, taps, generator=g)
    refs = [orc.short_conv(u[:, 3:3 + C].double(), w.double()) for u in us]
    tables = [[0, 1], [2]]
    for cuts in ([(23,), (9,)], [(1, 2, 16, 4), (3, 3, 3)], [(1,) * 23, (1,) * 9]):
        state = torch.full((2, max(taps - 1, 1), C), float("nan"), device=DEV)
        done, outs, k = [0, 0], [[], []], 0
        while any(d < L for d, L in zip(done, lens)):
            active = [(b, cuts[b][k]) for b in range(2) if k < len(cuts[b])]
            k += 1
            st = _step([(done[b], n) for b, n in active], [tables[b] for b, _ in active])
            st.state_slots = torch.tensor([b for b, _ in active], dtype=torch.int32, device=DEV)
            u = torch.cat([us[b][done[b]:done[b] + n] for b, n in active]).to(DEV)
            y = ops.causal_conv(u, 3, C, w.to(DEV), None, state, st)
            at = 0
            for b, n in active:
                outs[b].append(y[at:at + n])
                at += n
                done[b] += n
        for b in range(2):
            assert torch.allclose(torch.cat(outs[b]).cpu().double(), refs[b], atol=1e-5), (taps, cuts, b)


@pytest.mark.parametrize("E,top,ff", [(5, 2, 24), (3, 3, 70), (7, 1, 16), (40, 4, 8), (12, 10, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_match_reference(E, top, ff, dtype):
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    from tgis_b200.utils.mixers import RoutedExperts
    W = 64
    f = {"kind": "moe", "expert": {"ff": ff, "limit": 1.25}, "router": {"experts": E, "top": top}}
    cfg = orc.random_config(width=W, order=("attention_2",), kv_from=(None,), experts=E, top=top, ff=ff)
    sd = orc.random_state_dict(cfg, seed=3)
    sd["l0.mlp.router"] = (sd["l0.mlp.router"] * 4).bfloat16().float()  # well separated logits: the picks are not a close call
    mlp = RoutedExperts("l0.mlp", _DictWeights(sd, dtype), experts=E, top=top, limit=1.25)
    g = torch.Generator().manual_seed(1)
    for T in (1, 3, 150, 64 * E):   # the last one takes one dense product per expert when the type is bfloat16
        h = torch.randn(T, W, generator=g).to(dtype)
        ref = orc.moe(h.double(), {k: v.double() for k, v in orc.sub(sd, "l0.mlp.").items()}, f)
        y, routing = mlp(h.to(DEV))
        x = torch.ones(T, W, device=DEV)
        mix = torch.full((T, W), 2.0, device=DEV)
        ops.moe_combine_add(x, mix, y, routing)
        err = float((x.cpu().double() - 3.0 - ref).abs().max() / ref.abs().max())
        assert err < (2e-5 if dtype == torch.float32 else 0.05), (T, err)
        # every pick is a distinct expert, the weights of a token sum to one, compact rows map back to their tokens
        ids = routing.ids.cpu()
        assert all(len(set(r.tolist())) == top for r in ids) and torch.allclose(routing.weights.sum(-1).cpu(), torch.ones(T), atol=1e-5)
    x = torch.ones(2, W, device=DEV)
    ops.moe_combine_add(x, None, None, None)   # a layer with neither addend leaves the stream alone
    assert torch.equal(x.cpu(), torch.ones(2, W))
    # one row's result does not depend on what else the step holds
    h = torch.randn(40, W, generator=g).to(dtype).to(DEV)
    xa, xb = torch.zeros(40, W, device=DEV), torch.zeros(1, W, device=DEV)
    ya, ra = mlp(h)
    ops.moe_combine_add(xa, None, ya, ra)
    yb, rb = mlp(h[17:18].contiguous())
    ops.moe_combine_add(xb, None, yb, rb)
    assert torch.equal(xa[17], xb[0])


MIXER_CASES = [
    ("attention", {"conv": 3, "diff": 0.55, "dim": 12, "heads": 4, "kv_heads": 2, "q_temp": {"coef": 0.4, "every": 7}, "scale": 0.5, "vdim": 20}),
    ("attention", {"conv": 1, "diff": 0.2, "dim": 40, "heads": 3, "kv_heads": 3, "q_temp": {"coef": 0.9, "every": 16}, "scale": 0.3, "vdim": 8}),
    ("attention", {"conv": 4, "diff": 0.8, "dim": 8, "heads": 12, "kv_heads": 1, "q_temp": {"coef": 0.1, "every": 1}, "scale": 0.7, "vdim": 72}),
    ("attention_2", {"bias_max": 40, "dim": 10, "heads": 6, "kv_heads": 2, "scale": 0.5, "vdim": 10, "rel_rows": 12}),
    ("attention_2", {"bias_max": 30, "dim": 36, "heads": 2, "kv_heads": 2, "scale": 0.3, "vdim": 36, "rel_rows": 6}),
    ("attention_2", {"bias_max": 200, "dim": 16, "heads": 20, "kv_heads": 1, "scale": 0.4, "vdim": 16, "rel_rows": 32}),
    # shapes that take the tensor-core attention kernel when the cache is bfloat16 (sizes in 16s, group rows dividing 64)
    ("attention", {"conv": 3, "diff": 0.55, "dim": 16, "heads": 4, "kv_heads": 2, "q_temp": {"coef": 0.4, "every": 7}, "scale": 0.5, "vdim": 32}),
    ("attention", {"conv": 2, "diff": 0.3, "dim": 32, "heads": 2, "kv_heads": 2, "q_temp": {"coef": 0.2, "every": 3}, "scale": 0.3, "vdim": 144}),
    ("attention_2", {"bias_max": 40, "dim": 32, "heads": 8, "kv_heads": 2, "scale": 0.4, "vdim": 32, "rel_rows": 12}),
    ("attention_2", {"bias_max": 25, "dim": 16, "heads": 16, "kv_heads": 1, "scale": 0.4, "vdim": 16, "rel_rows": 10}),
    # ... and, with value sizes in 64s and a head group of at most 16 rows, its decode form for steps of few rows
    ("attention", {"conv": 3, "diff": 0.55, "dim": 16, "heads": 4, "kv_heads": 2, "q_temp": {"coef": 0.4, "every": 7}, "scale": 0.5, "vdim": 64}),
    ("attention", {"conv": 2, "diff": 0.4, "dim": 32, "heads": 8, "kv_heads": 1, "q_temp": {"coef": 0.3, "every": 5}, "scale": 0.3, "vdim": 128}),
    ("attention_2", {"bias_max": 40, "dim": 64, "heads": 6, "kv_heads": 2, "scale": 0.3, "vdim": 64, "rel_rows": 12}),
    ("attention_2", {"bias_max": 30, "dim": 64, "heads": 16, "kv_heads": 1, "scale": 0.3, "vdim": 64, "rel_rows": 8}),
]


@pytest.mark.parametrize("kind,m", MIXER_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixer_alone_any_cut(kind, m, dtype):
    """one mixer, two sequences of unequal length, fed whole / in ragged portions / token by token, pages out of order"""
    import tgis_b200  # noqa: F401
    from tgis_b200.models.custom_modeling.dubesun_modeling import build_mixer
    W, eps = 24, 1e-5
    cfg = {"architecture": "Dubesun", "layers": [{"type": kind, "mixer": m, "mlp": None}], "norm": {"eps": eps}, "max_positions": 64, "vocab": 8,
           "width": W}
    sd = orc.random_state_dict(cfg, seed=5)
    p64 = {k: v.double() for k, v in orc.sub(sd, "l0.mix.").items()}
    mixer = build_mixer(kind, "l0.mix", m, _DictWeights(sd, dtype), eps)
    spec = mixer.cache_spec()
    g = torch.Generator().manual_seed(1)
    lens = [45, 19]
    hs = [torch.randn(L, W, generator=g).to(dtype) for L in lens]
    fn = orc.diff_attention if kind == "attention" else orc.biased_attention
    refs = [fn(h.double(), p64, m, eps) for h in hs]
    tables = [[5, 0, 3], [7, 1]]
    for cuts in ([(45,), (19,)], [(16, 2, 27), (1, 18)], [(1,) * 45, (1,) * 19], [(7, 30, 8), (5, 5, 9)]):
        pages = torch.full((8, 16, spec.row_width), float("nan"), dtype=dtype, device=DEV)
        state = {n: torch.full((2, *s), float("nan"), dtype=torch.float32, device=DEV) for n, s in (spec.state or {}).items()}
        outs, done, k = [[], []], [0, 0], 0
        while any(d < L for d, L in zip(done, lens)):
            active = [(b, cuts[b][k]) for b in range(2) if k < len(cuts[b])]
            k += 1
            st = _step([(done[b], n) for b, n in active], [tables[b] for b, _ in active])
            st.state_slots = torch.tensor([b for b, _ in active], dtype=torch.int32, device=DEV)
            h = torch.cat([hs[b][done[b]:done[b] + n] for b, n in active]).to(DEV)
            y = mixer(h, st, pages, state, max(lens))
            at = 0
            for b, n in active:
                outs[b].append(y[at:at + n])
                at += n
                done[b] += n
        for b in range(2):
            got = torch.cat(outs[b]).double().cpu()
            err = float((got - refs[b]).abs().max() / refs[b].abs().max())
            assert err < (2e-5 if dtype == torch.float32 else 0.08), (kind, cuts, b, err)


def _fill_pool(cache, table, rows, kw, groups, kd, dv):
    """token rows [L, kw + groups * dv] (keys of all heads, then values) -> the pool as the kernels read it: inside a block of
    `page` tokens head-group-major - one group's keys of the block's tokens together, then the next group's, then the values"""
    page = cache.shape[1]
    host = cache.cpu().view(cache.shape[0], -1).clone()
    for j in range(rows.shape[0]):
        blk, tk = table[j // page], j % page
        for g in range(groups):
            o = g * page * kd + tk * kd
            host[blk, o:o + kd] = rows[j, g * kd:(g + 1) * kd]
            o = kw * page + g * page * dv + tk * dv
            host[blk, o:o + dv] = rows[j, kw + g * dv:kw + (g + 1) * dv]
    cache.copy_(host.view(cache.shape))


def _attn_reference(q, krows, vrows, q_pos, H, G, maps, scale, rel=None, rows=0, far=0.0):
    """q [n, H * maps, d]; krows [L, G * maps, d]; vrows [L, G, dv]: dense soft-max per query over keys 0 .. its position"""
    rep = H // G
    out = torch.zeros(q.shape[0], H * maps, vrows.shape[-1], dtype=torch.float64)
    for t, p in enumerate(q_pos):
        for qh in range(H * maps):
            h, mp = qh // maps, qh % maps
            g = h // rep
            s = (krows[:p + 1, g * maps + mp].double() @ q[t, qh].double()) * scale
            if rel is not None:
                s = s + torch.tensor([float(rel[orc.distance_bucket(p - j, rows, far), h]) for j in range(p + 1)], dtype=torch.float64)
            out[t, qh] = torch.softmax(s, 0) @ vrows[:p + 1, g].double()
    return out


@pytest.mark.parametrize("maps,H,G,d,dv", [(2, 4, 2, 12, 20), (1, 6, 2, 10, 10), (2, 5, 1, 8, 40), (2, 4, 2, 16, 48), (1, 8, 2, 32, 32),
                                          (2, 2, 1, 16, 160), (1, 64, 1, 16, 16), (2, 4, 2, 16, 64), (1, 16, 1, 32, 128), (2, 8, 1, 16, 64),
                                          (1, 3, 1, 16, 64), (2, 3, 1, 32, 256)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_paged_attention_far_keys_page_borders_first_tokens(dtype, maps, H, G, d, dv):
    """one key per query is made to dominate the soft-max of one map; it sits hundreds of tokens back, on either side of a page
    border, at the first positions or at the query itself - for single decoded tokens and for rows inside a prompt"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(3)
    L, scale = 420, 1.0
    KW, VW = G * maps * d, G * dv
    rows = (torch.randn(L, KW + VW, generator=g) * 0.3).to(dtype)
    krows, vrows = rows[:, :KW].float().view(L, G * maps, d), rows[:, KW:].float().view(L, G, dv)
    pairs = [(419, 0), (419, 1), (419, 15), (419, 16), (419, 17), (300, 31), (300, 32), (17, 16), (16, 16), (16, 15), (15, 15), (5, 0), (0, 0),
             (1, 0), (1, 1), (419, 419), (419, 418), (64, 63), (64, 64), (255, 128)]
    q = torch.randn(len(pairs), H * maps, d, generator=g) * 0.2
    for i, (p, j) in enumerate(pairs):
        qh = i % (H * maps)
        kh = ((qh // maps) // (H // G)) * maps + qh % maps
        q[i, qh] += 40.0 * krows[j, kh] / krows[j, kh].norm() ** 2
    q_pos = [p for p, _ in pairs]
    ref = _attn_reference(q, krows, vrows, q_pos, H, G, maps, scale)
    perm = torch.randperm(32, generator=g).tolist()   # the sequence's pages lie out of order in the pool
    table = perm[:(L + 15) // 16]
    cache = torch.full((32, 16, KW + VW), 1e4, dtype=dtype, device=DEV)  # rows that belong to nobody are loud but finite
    _fill_pool(cache, table, rows, KW, G, maps * d, dv)
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    for i, p in enumerate(q_pos):
        st = _step([(p, 1)], [table])
        got = ops.paged_attn(q[i:i + 1].to(DEV).contiguous(), cache, st, heads=H, kv_heads=G, maps=maps, vdim=dv, k_off=0, v_off=KW, scale=scale)
        assert torch.allclose(got.cpu().double(), ref[i:i + 1], atol=tol), ("decoded", pairs[i])
    qs = torch.randn(L, H * maps, d, generator=g) * 0.2
    for i, (p, j) in enumerate(pairs):
        qs[p] = q[i]
    got = ops.paged_attn(qs.to(DEV).contiguous(), cache, _step([(0, L)], [table]), heads=H, kv_heads=G, maps=maps, vdim=dv, k_off=0, v_off=KW,
                         scale=scale).cpu().double()
    for p, i in {p: i for i, p in enumerate(q_pos)}.items():
        assert torch.allclose(got[p], ref[i], atol=tol), ("prompt", pairs[i])


@pytest.mark.parametrize("dtype,d", [(torch.float32, 8), (torch.bfloat16, 16), (torch.bfloat16, 64)])
@pytest.mark.parametrize("rows,far", [(12, 40.0), (32, 200.0), (4, 9.0)])
def test_distance_bias_bucket_edges(rows, far, dtype, d):
    """one row of the bias table is loud: the keys of that bucket take the whole soft-max, so a key counted into the neighbouring
    bucket would show; queries sit so that the bucket's first and last distance, the last one-per-distance row and the saturated
    last row are all met, in decoding and inside a prompt"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    from tgis_b200.utils.mixers import log_distance_buckets
    H, G, L = 2, 1, 300
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    g = torch.Generator().manual_seed(rows)
    tab = log_distance_buckets(rows, far)
    assert tab == [orc.distance_bucket(n, rows, far) for n in range(len(tab))] and tab[-1] == rows - 1 and rows - 1 not in tab[:-1]
    tab_t = torch.tensor(tab, dtype=torch.int32, device=DEV)
    kv = (torch.randn(L, 2 * d, generator=g) * 0.3).to(dtype).float()
    cache = torch.zeros(20, 16, 2 * d, dtype=dtype, device=DEV)
    table = list(range(19))
    _fill_pool(cache, table, kv.to(dtype), d, 1, d, d)
    krows, vrows = kv[:, :d].view(L, 1, d), kv[:, d:].view(L, 1, d)
    for loud in sorted({0, rows // 2 - 1, rows // 2, rows - 2, rows - 1}):
        rel = torch.randn(rows, H, generator=g) * 0.2
        rel[loud] += 12.0
        q_pos = sorted({299, 150, len(tab) + 3, len(tab) - 1, len(tab) - 2, rows // 2, rows // 2 - 1, 1, 0}, reverse=True)
        q = torch.randn(len(q_pos), H, d, generator=g) * 0.2
        ref = _attn_reference(q, krows, vrows, q_pos, H, G, 1, 0.5, rel, rows, far)
        for i, p in enumerate(q_pos):
            got = ops.paged_attn(q[i:i + 1].to(DEV).contiguous(), cache, _step([(p, 1)], [table]), heads=H, kv_heads=G, maps=1, vdim=d, k_off=0,
                                 v_off=d, scale=0.5, rel=rel.to(DEV), bucket_tab=tab_t)
            assert torch.allclose(got.cpu().double(), ref[i:i + 1], atol=tol), (loud, p)
        qs = torch.zeros(L, H, d)
        for i, p in enumerate(q_pos):
            qs[p] = q[i]
        got = ops.paged_attn(qs.to(DEV).contiguous(), cache, _step([(0, L)], [table]), heads=H, kv_heads=G, maps=1, vdim=d, k_off=0, v_off=d,
                             scale=0.5, rel=rel.to(DEV), bucket_tab=tab_t).cpu().double()
        for i, p in enumerate(q_pos):
            assert torch.allclose(got[p], ref[i], atol=tol), (loud, "prompt", p)


# ------------------------------------------------------------------------------------------------ the model through the engine
def _sharp(config, factor=5.0):
    """soft-max sharp enough that single keys and the bias rows matter to the logits"""
    c = copy.deepcopy(config)
    for layer in c["layers"]:
        layer["mixer"]["scale"] *= factor
    return c


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_portions_and_decoding_agree_with_reference(tmp_path, dtype):
    # bfloat16 keeps the mechanisms live with a milder soft-max: its own rounding grows with the sharpness
    cfg = _sharp(orc.random_config(order=("attention", "attention_2", "attention", "attention"), kv_from=(None, None, 0, None),
                                   with_mlp=(True, True, False, True)), 5.0 if dtype == torch.float32 else 2.0)
    sd = orc.random_state_dict(cfg, seed=11)
    model = _model(tmp_path, cfg, sd, dtype)
    toks = _tokens(2, 75, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    tol = TOL32 if dtype == torch.float32 else TOL16
    sure = _decided(cfg, sd, toks) if dtype == torch.bfloat16 else torch.ones(75, dtype=torch.bool)
    assert int(sure.sum()) > 50
    whole = _run_cut(model, toks, [75])
    assert _rel(whole[sure], ref[sure]) < tol
    # the mechanisms are live in this configuration: a reference without the shared keys, with another temperature period or
    # with another far distance of the buckets is far outside the tolerance
    for path, wrong in ((("layers", 2, "mixer", "kv_from"), 3), (("layers", 0, "mixer", "q_temp", "every"), 8),
                        (("layers", 1, "mixer", "bias_max"), 30), (("layers", 3, "mixer", "diff"), 0.5)):
        c2 = copy.deepcopy(cfg)
        node = c2
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = wrong
        if path[-1] == "kv_from":   # layer 2 reads layer 3's tensors as if they were its own: just another set of keys
            sd2 = dict(sd)
            for n in ("k", "k.conv", "k.norm", "v", "v.conv"):
                sd2[f"l2.mix.{n}"] = sd[f"l3.mix.{n}"]
            del node["kv_from"]
            assert _rel(orc.forward(c2, sd2, toks), ref) > 20 * TOL32
        else:
            assert _rel(orc.forward(c2, sd, toks), ref) > 20 * TOL32, path
    for cuts in ([], [40], [2, 2, 2, 19, 3, 16, 17, 2], [16, 16, 16, 16], [7, 7, 7, 7, 7], [1, 20, 22, 31]):
        got = _run_cut(model, toks, cuts)
        assert _rel(got[sure], ref[sure]) < tol, cuts
        if dtype == torch.float32:
            assert _rel(got, whole.cpu()) < 1e-5, cuts  # the cut itself changes nothing beyond rounding
    assert model.kv_cache_manager.free_blocks == model.kv_cache_manager.total_num_gpu_blocks
    assert model.kv_cache_manager.free_state_slots == 4


def test_tensor_core_shapes_through_the_engine(tmp_path):
    """bfloat16 with head sizes in 16s: prompts, portions and decoded tokens take the tensor-core attention kernel; a step mixes
    a long portion (several query tiles) with single tokens"""
    cfg = _sharp(orc.random_config(width=64, order=("attention", "attention_2", "attention"), kv_from=(None, None, 0), heads=(8, 4),
                                   kv_heads=(2, 2), dim=(16, 16), vdim=64, max_positions=256), 3.0)
    sd = orc.random_state_dict(cfg, seed=12)
    model = _model(tmp_path, cfg, sd, torch.bfloat16)
    toks = _tokens(3, 150, cfg["vocab"])
    ref, sure = orc.forward(cfg, sd, toks), _decided(cfg, sd, toks)
    assert int(sure.sum()) > 100
    for cuts in ([150], [100, 2, 40], [1, 70, 33], [5]):
        assert _rel(_run_cut(model, toks, cuts)[sure], ref[sure]) < TOL16, cuts
    other = _tokens(4, 90, cfg["vocab"])
    ref_o, sure_o = orc.forward(cfg, sd, other), _decided(cfg, sd, other)
    (a,), la = model.step_ragged([None], [toks[:20]])
    (a, b), l2 = model.step_ragged([a, None], [toks[20:21], other[:80]])
    (b, a), l3 = model.step_ragged([b, a], [other[80:], toks[21:150]])
    model.kv_cache_manager.free_sequences([a, b])
    assert _rel(torch.cat([la, l2[:1], l3[10:]])[sure], ref[sure]) < TOL16
    assert _rel(torch.cat([l2[1:], l3[:10]])[sure_o], ref_o[sure_o]) < TOL16


def test_residual_stream_after_every_layer(tmp_path):
    cfg = orc.random_config(order=("attention_2", "attention", "attention"), kv_from=(None, None, 1), with_mlp=(True, False, True))
    sd = orc.random_state_dict(cfg, seed=4)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(5, 30, cfg["vocab"])
    want = []
    orc.forward(cfg, sd, toks, residuals=want)
    probe = []
    model.model.model.residual_probe = probe
    sids, _ = model.step_ragged([None], [toks])
    model.model.model.residual_probe = None
    model.kv_cache_manager.free_sequences(sids)
    assert len(probe) == len(want) == 3
    for i, (a, b) in enumerate(zip(probe, want)):
        assert float((a.cpu().double() - b).abs().max()) < 1e-4 * float(b.abs().max()), i


@pytest.mark.parametrize("variant", ["one_head_group", "equal_heads_top1", "all_experts_two_taps"])
def test_other_sizes(tmp_path, variant):
    """sizes that a usual configuration makes equal or 1: one key head, as many key heads as query heads, one expert per token,
    every expert per token, one and two taps, a value size below the key size"""
    kw = {"one_head_group": dict(heads=(5, 3), kv_heads=(1, 1), dim=(6, 16), vdim=8, conv=1, experts=4, top=3, rel_rows=8, bias_max=20),
          "equal_heads_top1": dict(heads=(3, 2), kv_heads=(3, 2), dim=(14, 6), vdim=36, conv=4, experts=6, top=1, rel_rows=20, bias_max=90),
          "all_experts_two_taps": dict(heads=(8, 6), kv_heads=(4, 2), dim=(8, 10), vdim=10, conv=2, experts=3, top=3, every=1, width=56)}[variant]
    cfg = _sharp(orc.random_config(order=("attention", "attention", "attention_2"), kv_from=(None, 0, None), **kw), 3.0)
    sd = orc.random_state_dict(cfg, seed=31)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(6, 60, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    for cuts in ([60], [3, 30, 2], [17]):
        assert _rel(_run_cut(model, toks, cuts), ref) < TOL32, (variant, cuts)


def test_ragged_batches_reused_pages_and_slots(tmp_path):
    """four requests of unequal length run as mixed steps (portions beside decoded tokens, requests joining and leaving) in a pool
    that is too small for all of them at once and is filled with garbage first: every request equals its run alone"""
    cfg = _sharp(orc.random_config(order=("attention", "attention_2", "attention"), kv_from=(None, None, 0), with_mlp=(True, False, True)))
    sd = orc.random_state_dict(cfg, seed=21)
    model = _model(tmp_path, cfg, sd, torch.float32, blocks=12, slots=2)
    mgr = model.kv_cache_manager
    for p in mgr.pages:
        if p is not None:
            p.fill_(float("nan"))
    for st in mgr.states:
        for t in (st or {}).values():
            t.fill_(float("nan"))
    lens = {"a": 70, "b": 33, "c": 1, "d": 50}
    toks = {k: _tokens(30 + i, n, cfg["vocab"]) for i, (k, n) in enumerate(lens.items())}
    refs = {k: orc.forward(cfg, sd, v) for k, v in toks.items()}
    plan = [[("a", 20), ("b", 2)], [("a", 1), ("b", 31)], [("a", 30)], [("a", 1)], [("a", 18), ("c", 1)],   # b ends at step 1, a at 4
            [("d", 17)], [("d", 2)], [("d", 1)], [("d", 30)]]
    got = {k: [] for k in lens}
    at = {k: 0 for k in lens}
    live = {}
    for step in plan:
        ids = [live.get(k) for k, _ in step]
        sids, lg = model.step_ragged(ids, [toks[k][at[k]:at[k] + n] for k, n in step])
        o = 0
        for (k, n), sid in zip(step, sids):
            live[k] = sid
            got[k].append(lg[o:o + n])
            o += n
            at[k] += n
            if at[k] == lens[k]:
                mgr.free_sequences([live.pop(k)])
        assert len(live) <= 2
    for k in lens:
        assert at[k] == lens[k]
        assert _rel(torch.cat(got[k]), refs[k]) < TOL32, k
    assert mgr.free_blocks == mgr.total_num_gpu_blocks and mgr.free_state_slots == 2


def test_long_decoding_and_first_tokens(tmp_path):
    """three prompt tokens, then 197 single steps: the temperature period (every 64) and the buckets' far distance pass inside the
    decoded tokens; the first tokens have fewer keys than taps"""
    cfg = orc.random_config(order=("attention", "attention_2", "attention"), kv_from=(None, None, 0), with_mlp=(False, True, True), every=64,
                            coef=0.8, max_positions=256, bias_max=100, rel_rows=16)
    sd = orc.random_state_dict(cfg, seed=8)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(9, 200, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    c2 = copy.deepcopy(cfg)
    c2["layers"][0]["mixer"]["q_temp"]["every"] = 65
    assert _rel(orc.forward(c2, sd, toks)[60:70], ref[60:70]) > 20 * TOL32   # the period's edge is live
    got = _run_cut(model, toks, [3])
    assert _rel(got[:8], ref[:8]) < TOL32
    assert _rel(got, ref) < TOL32
    one = _run_cut(model, toks[:1], [1])  # a request of a single token
    assert _rel(one, ref[:1]) < TOL32
    with pytest.raises(ValueError):
        model.step_ragged([None], [_tokens(1, 258, cfg["vocab"])])  # more tokens than learned positions


def test_greedy_generation_through_generate_token(tmp_path):
    """from_pb -> generate_token (prefill, decode steps, a second batch joined by concatenate, prune of a finished request):
    the engine's own scheduler path picks the reference's greedy tokens wherever the reference's top-2 gap is decisive"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import pb
    cfg = orc.random_config(order=("attention_2", "attention", "attention"), kv_from=(None, None, 1))
    sd = orc.random_state_dict(cfg, seed=13)
    model = _model(tmp_path, cfg, sd, torch.float32, blocks=64, slots=6)
    tok = model.tokenizer
    V = cfg["vocab"]

    def text(ids):
        return " ".join("test" if i == 3 else f"<tok{i}>" for i in ids)

    def batch_of(bid, prompts, n_new, first_id):
        reqs = [pb.Request(id=first_id + i, inputs=text(p), input_length=len(p), truncate=False, max_output_length=n_new,
                           parameters=pb.NextTokenChooserParameters(temperature=0.0, top_p=1.0, min_new_tokens=n_new))
                for i, p in enumerate(prompts)]
        return pb.Batch(id=bid, requests=reqs)

    def oracle_greedy(prompt, n_new):
        seq, out, sure = list(prompt), [], n_new
        for s in range(n_new):
            lg = orc.forward(cfg, sd, seq)[-1]
            lg[2] = float("-inf")  # min_new_tokens bans EOS
            top = lg.topk(2).values
            if float(top[0] - top[1]) < 1e-3 * float(lg[torch.isfinite(lg)].std()):
                sure = min(sure, s)
            out.append(int(lg.argmax()))
            seq.append(out[-1])
        return out, sure

    n_new = 7
    p1 = [_tokens(40, 9, V), _tokens(41, 23, V)]
    p2 = [_tokens(42, 5, V)]
    got = {0: [], 1: [], 2: []}
    with torch.inference_mode():
        b1, errs = model.batch_type.from_pb(batch_of(0, p1, n_new, 0), tok, model.dtype, model.device, None, None, True)
        assert not errs
        for t in model.generate_token(b1, first=True)[0]:
            got[t.request_id].append(t.token_id)
        for _ in range(2):
            for t in model.generate_token(b1)[0]:
                got[t.request_id].append(t.token_id)
        b2, errs = model.batch_type.from_pb(batch_of(1, p2, n_new, 2), tok, model.dtype, model.device, None, None, True)
        for t in model.generate_token(b2, first=True, for_concat=True)[0]:
            got[t.request_id].append(t.token_id)
        both = model.batch_type.concatenate([b1, b2])
        for _ in range(n_new - 3):
            for t in model.generate_token(both)[0]:
                got[t.request_id].append(t.token_id)
        assert len(got[0]) == n_new and len(got[1]) == n_new
        rest = model.batch_type.prune(both, [0, 1])
        assert len(rest) == 1
        while len(got[2]) < n_new:
            for t in model.generate_token(rest)[0]:
                got[t.request_id].append(t.token_id)
        model.kv_cache_manager.free_sequences(rest.sequence_ids)
    sure_total = 0
    for rid, prompt in enumerate(p1 + p2):
        ref, sure = oracle_greedy(prompt, n_new)
        assert got[rid][:sure] == ref[:sure], (rid, got[rid], ref)
        sure_total += sure
    assert sure_total >= 12
    mgr = model.kv_cache_manager
    assert mgr.free_blocks == mgr.total_num_gpu_blocks and mgr.free_state_slots == 6
