"""Fetotar on the GPU against the slow CPU reference (oracle/fetotar.py, float64): each mechanism alone, then the model through
the engine's step function and cache manager - whole prompts, token-by-token decoding, portions down to two tokens, ragged
batches, pages and state slots that are freed and used again - and greedy generation through FlashCausalLM.generate_token.

The configurations are small and deliberately uneven (key size != value size, rotated part smaller than the plain part, a state
size that is no multiple of the lane split, value sizes that need more than one column block, one and several groups).  Where
random weights would hide a fault the test makes it show: a key that must win the soft-max from far away, at a page border, or
exactly at the window's edge; a soft-max sharp enough that one key more or less in the window moves the logits."""
import copy
import json
import os

import pytest
import torch

from oracle import fetotar as orc

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


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


TOL32, TOL16 = 2e-4, 0.3


class _DictWeights:
    def __init__(self, sd, dtype):
        from tgis_b200.utils.dist import FakeGroup
        self.sd, self.dtype, self.device, self.process_group = sd, dtype, DEV, FakeGroup(0, 1)

    def get_tensor(self, name):
        return self.sd[name].to(self.dtype).to(DEV)


def _step(lens_and_starts, page_rows):
    """RaggedStep for sequences (start, count) laid out in consecutive blocks of their own"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq
    pos, seq, slots, cu, tables = [], [], [], [0], []
    blk = 0
    for b, (start, n) in enumerate(lens_and_starts):
        nblocks = (start + n + 15) // 16
        table = list(range(blk, blk + nblocks))
        blk += nblocks
        tables.append(table)
        for p in range(start, start + n):
            pos.append(p)
            seq.append(b)
            slots.append(table[p // 16] * 16 + p % 16)
        cu.append(cu[-1] + n)
    width = max(len(t) for t in tables)
    bt = torch.zeros(len(tables), width, dtype=torch.int32)
    for i, t in enumerate(tables):
        bt[i, :len(t)] = torch.tensor(t)
    assert blk <= page_rows
    return ops_seq.RaggedStep(T=len(pos), B=len(tables), position_ids=torch.tensor(pos, dtype=torch.int64, device=DEV),
                              cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV), seq_of_token=torch.tensor(seq, dtype=torch.int32, device=DEV),
                              slot_mapping=torch.tensor(slots, dtype=torch.int64, device=DEV), block_table=bt.to(DEV),
                              state_slots=torch.arange(len(tables), dtype=torch.int32, device=DEV))


# ------------------------------------------------------------------------------------------------ mechanisms alone
def test_row_kernels_match_reference():
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    g = torch.Generator().manual_seed(0)
    T, W, F, dim, V = 7, 50, 22, 5, 30
    x = torch.randn(T, W, generator=g) * 3
    w, b = torch.randn(W, generator=g), torch.randn(W, generator=g)
    ref = orc.layer_norm(x.double(), w.double(), b.double(), 1e-5)
    got = ops.layernorm(x.to(DEV), w.to(DEV), b.to(DEV), 1e-5)
    assert torch.allclose(got.cpu().double(), ref, atol=1e-5)
    res = torch.randn(T, W, generator=g)
    acc = res.clone().to(DEV)
    ops.layernorm_into_residual(x.to(DEV), w.to(DEV), b.to(DEV), 1e-5, acc)
    assert torch.allclose(acc.cpu().double(), res.double() + ref, atol=1e-5)
    gu = torch.randn(T, 2 * F, generator=g) * 3
    eye, zero = torch.eye(F).double(), torch.zeros(F, F).double()  # selector projections: the rows of gu pass straight into the activation
    ref = orc.dense_ff(gu.double(), {"gate": torch.cat([eye, zero], 1), "up": torch.cat([zero, eye], 1), "down": eye}, {"limit": 1.25})
    assert torch.allclose(ops.ff_clamped_gate(gu.to(DEV), 1.25).cpu().double(), ref, atol=1e-5)
    ids = torch.randint(0, V, (T,), generator=g)
    table = torch.randn(V, 3 * dim, generator=g)
    p = {"gate": torch.randn(dim, W, generator=g) * 0.3, "proj": torch.randn(W, dim, generator=g), "norm": torch.randn(W, generator=g)}
    ref = orc.token_side(x.double(), ids, 1, table.double(), {k: v.double() for k, v in p.items()}, dim, 1e-5)
    acc = x.clone().to(DEV)
    ops.token_side(acc, acc, ids.to(DEV), table.to(DEV), dim, dim, p["gate"].to(DEV), p["proj"].to(DEV), p["norm"].to(DEV), 1e-5)
    assert torch.allclose(acc.cpu().double(), ref, atol=1e-4)
    # the residual update that also hands out the typed copy for the next projection
    acc, xb = res.clone().to(DEV), x.to(DEV).bfloat16()
    copy = ops.layernorm_into_residual(xb, w.to(DEV).bfloat16(), b.to(DEV).bfloat16(), 1e-5, acc, typed_copy=True)
    assert copy.dtype == torch.bfloat16 and torch.equal(copy, acc.bfloat16())
    emb = ops.embed_scale(table.to(DEV), ids.to(DEV), 2.5)
    assert torch.equal(emb.cpu(), table[ids] * 2.5)
    # the product kernel in every type combination the mixers use, odd sizes, bias, per-head strides
    a, wt, bias = torch.randn(37, 29, generator=g), torch.randn(70, 29, generator=g), torch.randn(70, generator=g)
    assert torch.allclose(ops.linear(a.to(DEV), wt.to(DEV), bias.to(DEV)).cpu().double(), a.double() @ wt.double().T + bias.double(), atol=1e-4)
    got = ops.linear(a.to(DEV), wt.to(DEV).bfloat16(), out_dtype=torch.float32).cpu().double()
    assert torch.allclose(got, a.double() @ wt.bfloat16().double().T, atol=1e-4)
    xh, wh = torch.randn(9, 3, 11, generator=g), torch.randn(3, 6, 11, generator=g)
    out = torch.zeros(9, 3, 8, device=DEV)
    ops.linear_per_head(xh.to(DEV), wh.to(DEV), out[:, :, :6])
    assert torch.allclose(out[:, :, :6].cpu().double(), torch.einsum("mzk,znk->mzn", xh.double(), wh.double()), atol=1e-4)
    assert float(out[:, :, 6:].abs().max()) == 0.0


@pytest.mark.parametrize("dims,scaling", [(6, None), (6, {"factor": 3.0, "fast": 24.0, "original": 64, "slow": 2.0}),
                                          (32, {"factor": 4.0, "fast": 32.0, "original": 4096, "slow": 1.0})])
def test_rotary_tables_match_reference(dims, scaling):
    import tgis_b200  # noqa: F401
    from tgis_b200.utils.mixers import ScaledRotaryTables
    rot = {"dims": dims, "base": 5000.0}
    if scaling:
        rot["scaling"] = scaling
    cos, sin = ScaledRotaryTables(dims, 5000.0, scaling).tables(300, "cpu")
    rc, rs = orc.yarn_angles(300, rot)
    assert torch.allclose(cos[:300].double(), rc, atol=1e-6) and torch.allclose(sin[:300].double(), rs, atol=1e-6)


MIXER_CASES = [
    ("mlstm", {"dim": 12, "gate_cap": 11.0, "heads": 3, "vdim": 20}),
    ("mlstm", {"dim": 72, "gate_cap": 15.0, "heads": 1, "vdim": 40}),
    ("mamba2", {"conv": 3, "groups": 2, "heads": 4, "norm_groups": 2, "state": 10, "vdim": 6}),
    ("mamba2", {"conv": 2, "groups": 1, "heads": 3, "norm_groups": 3, "state": 70, "vdim": 36}),
    ("mamba2", {"conv": 4, "groups": 3, "heads": 3, "norm_groups": 1, "state": 16, "vdim": 8}),
    ("latent_attention", {"dim": 10, "heads": 3, "kv_rank": 14, "mask": {"size": 9}, "q_rank": 18, "rot_dim": 6, "scale": 0.4, "vdim": 12,
                          "rot": {"base": 5000.0, "dims": 6, "scaling": {"factor": 3.0, "fast": 24.0, "original": 64, "slow": 2.0}}}),
    ("latent_attention", {"dim": 24, "heads": 20, "kv_rank": 64, "mask": {"size": 70}, "q_rank": 16, "rot_dim": 16, "scale": 0.2, "vdim": 8,
                          "rot": {"base": 300.0, "dims": 16}}),
    ("latent_attention", {"dim": 8, "heads": 9, "kv_rank": 40, "mask": {"size": 33}, "q_rank": 12, "rot_dim": 8, "scale": 0.3, "vdim": 4,
                          "rot": {"base": 100.0, "dims": 4}}),
]


@pytest.mark.parametrize("kind,m", MIXER_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixer_alone_any_cut(kind, m, dtype):
    """one mixer, two sequences of unequal length, fed whole / in ragged portions / token by token: same as the reference"""
    import tgis_b200  # noqa: F401
    from tgis_b200.models.custom_modeling.fetotar_modeling import build_mixer
    W, eps = 24, 1e-5
    cfg = {"architecture": "Fetotar", "embedding": {"scale": 1.0}, "layers": [{"type": kind, "mixer": m, "mlp": None}], "norm": {"eps": eps},
           "token_side": {"dim": 4}, "vocab": 8, "width": W}
    sd = orc.random_state_dict(cfg, seed=5)
    p64 = {k: v.double() for k, v in orc.sub(sd, "l0.mix.").items()}
    mixer = build_mixer(kind, "l0.mix", m, _DictWeights(sd, dtype), eps)
    spec = mixer.cache_spec()
    g = torch.Generator().manual_seed(1)
    lens = [45, 19]
    hs = [torch.randn(L, W, generator=g).to(dtype) for L in lens]
    refs = [orc.MIXERS[kind](h.double(), p64, m, eps) for h in hs]
    for cuts in ([(45,), (19,)], [(16, 2, 27), (1, 18)], [(1,) * 45, (1,) * 19], [(7, 30, 8), (5, 5, 9)]):
        if spec.kind == "paged":
            store = torch.full((8, 16, spec.row_width), float("nan"), dtype=dtype, device=DEV)
        else:
            store = {n: torch.full((2, *s), float("nan"), dtype=torch.float32, device=DEV) for n, s in spec.state.items()}
        outs = [[], []]
        done = [0, 0]
        k = 0
        while any(d < L for d, L in zip(done, lens)):
            active = [(b, cuts[b][k]) for b in range(2) if k < len(cuts[b])]
            k += 1
            # a step holds the sequences that still have a portion; block tables and slots stay those of the full layout
            full = _step([(0, lens[0]), (0, lens[1])], 8)
            sub = _step([(done[b], n) for b, n in active], 8)
            sub.block_table = full.block_table[[b for b, _ in active]].contiguous()
            sub.state_slots = full.state_slots[[b for b, _ in active]].contiguous()
            slot_rows = []
            for b, n in active:
                for pp in range(done[b], done[b] + n):
                    slot_rows.append(int(full.block_table[b, pp // 16]) * 16 + pp % 16)
            sub.slot_mapping = torch.tensor(slot_rows, dtype=torch.int64, device=DEV)
            h = torch.cat([hs[b][done[b]:done[b] + n] for b, n in active]).to(DEV)
            y = mixer(h, sub, store, max(lens))
            at = 0
            for b, n in active:
                outs[b].append(y[at:at + n])
                at += n
                done[b] += n
        for b in range(2):
            got = torch.cat(outs[b]).double().cpu()
            err = float((got - refs[b]).abs().max() / refs[b].abs().max())
            assert err < (2e-5 if dtype == torch.float32 else 0.08), (kind, cuts, b, err)


def _attn_reference(q_abs, rows, pos_of_row, seq_of_row, q_pos, q_seq, R, window, scale):
    out = torch.zeros(q_abs.shape[0], q_abs.shape[1], R, dtype=torch.float64)
    for t in range(q_abs.shape[0]):
        vis = [i for i in range(rows.shape[0]) if seq_of_row[i] == q_seq[t] and 0 <= q_pos[t] - pos_of_row[i] < window]
        keys = rows[vis].double()
        p = torch.softmax(q_abs[t].double() @ keys.T * scale, -1)
        out[t] = p @ keys[:, :R]
    return out


@pytest.mark.parametrize("R,r", [(40, 8), (64, 16)])  # the second shape takes the tensor-core kernel when the cache is bfloat16
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_window_edges_page_borders_and_far_keys(dtype, R, r):
    """one key per query is made to dominate the soft-max; it sits just inside or just outside the window, on either side of a
    page border, at the first positions, or hundreds of tokens back - for query rows inside a prompt and for single decoded tokens"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import ops_seq as ops
    H, window, scale = 3, 48, 1.0
    D = R + r
    g = torch.Generator().manual_seed(3)
    L = 420
    rows = (torch.randn(L, D, generator=g) * 0.3).to(dtype)
    for far, win in ((False, window), (True, 0)):
        # (query position, position of the key that is made to stand out)
        pairs = [(100, 100 - win + 1), (101, 101 - win), (63, 16), (64, 17), (79, 32), (80, 32), (47, 0), (48, 0), (48, 1), (5, 0), (0, 0), (15, 15),
                 (16, 15), (16, 16), (419, 419 - win + 1), (419, 419 - win)] if not far else [(419, 0), (419, 15), (419, 16), (300, 1), (17, 16)]
        w = win if win else 1 << 30
        q_pos = [p for p, _ in pairs]
        q_abs = torch.randn(len(pairs), H, D, generator=g) * 0.2
        for i, (p, j) in enumerate(pairs):
            if 0 <= j <= p:
                q_abs[i, i % H] += 6.0 * rows[j].float() / rows[j].float().norm() ** 2 * 8.0
        ref = _attn_reference(q_abs, rows.float(), list(range(L)), [0] * L, q_pos, [0] * len(pairs), R, w, scale)
        cache = torch.zeros(32, 16, D, dtype=dtype, device=DEV)
        cache.view(-1, D)[:L] = rows.to(DEV)
        full = _step([(0, L)], 32)
        # as rows of one prompt portion: positions must be consecutive per sequence, so every query gets a step entry of its own
        for i, p in enumerate(q_pos):
            st = _step([(p, 1)], 32)
            st.block_table = full.block_table
            got = ops.latent_attn(q_abs[i:i + 1].to(DEV).contiguous(), cache, st, R, r, win, scale).cpu().double()
            assert torch.allclose(got, ref[i:i + 1], atol=1e-4 if dtype == torch.float32 else 3e-2), (far, pairs[i])
        # and all positions of the sequence as one prompt: row p is query p
        qs = torch.randn(L, H, D, generator=g) * 0.2
        for i, (p, j) in enumerate(pairs):
            qs[p] = q_abs[i]
        got = ops.latent_attn(qs.to(DEV).contiguous(), cache, full, R, r, win, scale).cpu().double()
        for p, i in {p: i for i, p in enumerate(q_pos)}.items():  # a position listed twice carries its last query
            assert torch.allclose(got[p], ref[i], atol=1e-4 if dtype == torch.float32 else 3e-2), (far, "prompt", pairs[i])


# ------------------------------------------------------------------------------------------------ the model through the engine
def _sharp(config, factor=6.0):
    """a soft-max sharp enough that a single key at the window's edge moves the logits"""
    c = copy.deepcopy(config)
    for layer in c["layers"]:
        if layer["type"] == "latent_attention":
            layer["mixer"]["scale"] *= factor
    return c


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prompt_portions_and_decoding_agree_with_reference(tmp_path, dtype):
    cfg = _sharp(orc.random_config(order=("mlstm", "latent_attention", "mamba2", "latent_attention"), with_mlp=(False, True, False, True),
                                   window=21))
    sd = orc.random_state_dict(cfg, seed=11)
    model = _model(tmp_path, cfg, sd, dtype)
    toks = _tokens(2, 75, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    tol = TOL32 if dtype == torch.float32 else TOL16
    whole = _run_cut(model, toks, [75])
    assert _rel(whole, ref) < tol
    # the window's edge is live in this configuration: a reference that sees one key more or fewer is far outside the tolerance
    for wrong in (20, 22):
        c2 = copy.deepcopy(cfg)
        for layer in c2["layers"]:
            if layer["type"] == "latent_attention":
                layer["mixer"]["mask"]["size"] = wrong
        assert _rel(orc.forward(c2, sd, toks), ref) > 20 * TOL32
    for cuts in ([], [40], [2, 2, 2, 19, 3, 16, 17, 2], [16, 16, 16, 16], [21, 21, 21], [1, 20, 22, 31]):
        got = _run_cut(model, toks, cuts)
        assert _rel(got, ref) < tol, cuts
        if dtype == torch.float32:
            assert _rel(got, whole.cpu()) < 1e-5, cuts  # the cut itself changes nothing beyond rounding
    assert model.kv_cache_manager.free_blocks == model.kv_cache_manager.total_num_gpu_blocks
    assert model.kv_cache_manager.free_state_slots == 4


def test_residual_stream_after_every_layer(tmp_path):
    cfg = orc.random_config(order=("mamba2", "mlstm", "latent_attention"), with_mlp=(True, False, False), heads=3, yarn=False)
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


def test_ragged_batches_reused_pages_and_slots(tmp_path):
    """four requests of unequal length run as mixed steps (portions beside decoded tokens, requests joining and leaving) in a pool
    that is too small for all of them at once and is filled with garbage first: every request equals its run alone"""
    cfg = _sharp(orc.random_config(order=("latent_attention", "mamba2", "mlstm"), with_mlp=(True, False, True), window=18, heads=2))
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
    for stepno, step in enumerate(plan):
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
    cfg = orc.random_config(order=("mlstm", "mamba2", "latent_attention"), with_mlp=(False, False, True), window=40, heads=1)
    sd = orc.random_state_dict(cfg, seed=8)
    model = _model(tmp_path, cfg, sd, torch.float32)
    toks = _tokens(9, 200, cfg["vocab"])
    ref = orc.forward(cfg, sd, toks)
    got = _run_cut(model, toks, [3])  # three prompt tokens, then 197 single steps
    assert _rel(got[:8], ref[:8]) < TOL32
    assert _rel(got, ref) < TOL32
    one = _run_cut(model, toks[:1], [1])  # a request of a single token
    assert _rel(one, ref[:1]) < TOL32


def test_greedy_generation_through_generate_token(tmp_path):
    """from_pb -> generate_token (prefill, decode steps, a second batch joined by concatenate, prune of a finished request):
    the engine's own scheduler path picks the reference's greedy tokens wherever the reference's top-2 gap is decisive"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import pb
    cfg = orc.random_config(order=("mlstm", "latent_attention", "mamba2"), with_mlp=(True, True, False), window=12)
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


def test_sampling_and_logprobs_through_generate_token(tmp_path):
    """requests that sample (temperature, top-k, a seed) and ask for log-probabilities take the chooser chain on the fp32 logits:
    the same seed draws the same tokens, ids stay inside the top-k set of the reference's logits, log-probabilities are finite"""
    import tgis_b200  # noqa: F401
    from tgis_b200 import pb
    cfg = orc.random_config(order=("mamba2", "latent_attention"), with_mlp=(False, True), window=10)
    sd = orc.random_state_dict(cfg, seed=17)
    model = _model(tmp_path, cfg, sd, torch.bfloat16, blocks=32, slots=4)
    tok, V = model.tokenizer, cfg["vocab"]
    prompt = _tokens(50, 11, V)
    text = " ".join(f"<tok{i}>" for i in prompt)
    n_new, top_k = 5, 4

    def run(batch_id):
        reqs = [pb.Request(id=i, inputs=text, input_length=len(prompt), truncate=False, max_output_length=n_new,
                           parameters=pb.NextTokenChooserParameters(temperature=0.9, top_k=top_k, top_p=1.0, seed=1234, min_new_tokens=n_new),
                           details=pb.RequestedDetails(logprobs=True)) for i in range(2)]
        out = [[], []]
        with torch.inference_mode():
            batch, errs = model.batch_type.from_pb(pb.Batch(id=batch_id, requests=reqs), tok, model.dtype, model.device, None, None, True)
            assert not errs
            infos = model.generate_token(batch, first=True)[0]
            for _ in range(n_new):
                for t in infos:
                    out[t.request_id].append((t.token_id, t.logprob))
                if len(out[0]) == n_new:
                    break
                infos = model.generate_token(batch)[0]
            model.kv_cache_manager.free_sequences(batch.sequence_ids)
        return out

    first, again = run(0), run(1)
    assert [t for t, _ in first[0]] == [t for t, _ in again[0]] and [t for t, _ in first[1]] == [t for t, _ in again[1]]
    assert [t for t, _ in first[0]] == [t for t, _ in first[1]]  # two requests with the same seed and prompt in one batch
    seq = list(prompt)
    for t, lp in first[0]:
        ref = orc.forward(cfg, sd, seq)[-1]
        ref[2] = float("-inf")
        assert t in ref.topk(top_k + 2).indices.tolist()  # bf16 may swap neighbours at the cut; it never reaches far down
        assert lp is not None and lp <= 0.0 and lp > -30.0
        seq.append(t)
