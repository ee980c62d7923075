"""Fezuzen on the engine against the plain oracle (oracle/fezuzen_oracle.py): every mechanism alone, prompts in one piece, in
portions down to two tokens and token by token, batched decode steps of unequal requests, slots that are freed and used
again, keys far away, at the edges of key tiles and just inside / outside every window and chunk (in prompts and in decode
steps), the first tokens of a sequence, long decoding, greedy generation through generate() and the continuous batcher.
Small configurations whose sizes differ from one another (and from multiples of the kernels' tiles), random weights, both
number formats; where random weights would hide a fault the weights are shaped so that it shows."""
import copy
import threading

import numpy as np
import pytest
import torch

from oracle import fezuzen_oracle as O

pytestmark = pytest.mark.gpu

YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}


def latent(heads, dim, rot_dim, vdim, rank, q_rank, window, base=500.0, scaling=None, scale=0.3, kv_from=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling:
        rot["scaling"] = dict(scaling)
    mix = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "q_rank": q_rank, "mask": {"size": window}, "rot": rot,
           "scale": scale}
    if kv_from is not None:
        mix["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mix}


def grouped(heads, kv_heads, dim, vdim, conv, chunk, rot_dims, base=100.0, scaling=None, scale=0.25):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(scaling)
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "mask": {"size": chunk},
                                           "rot": rot, "scale": scale}}


LAT = latent(3, 16, 8, 24, 40, 32, 7, scaling=YARN)
LAT_ODD = latent(5, 9, 7, 7, 21, 11, 33, base=10000.0)                    # nothing a multiple of 4, an odd rotated part (its last entry passes)
LAT_ONE = latent(1, 16, 2, 16, 16, 16, 1)                                  # one head, one pair, a window that holds the query alone
LAT_MANY = latent(40, 8, 4, 4, 24, 24, 50, scaling=YARN)                   # more heads than a CTA's pairs
LAT_WIDE = latent(2, 32, 16, 48, 288, 64, 19)                              # cached rows wider than 256
GQA = grouped(6, 2, 16, 24, 3, 11, 8, scaling=YARN)                        # part of a head rotated, keys with scaled frequencies
GQA_ODD = grouped(2, 2, 7, 9, 0, 5, 4)                                     # groups of one head, no convolution, odd head and value sizes
GQA_TAP = grouped(3, 1, 8, 4, 1, 1, 2)                                     # a convolution of ONE tap, chunks of one position, one rotated pair
GQA_ONE_KV = grouped(4, 1, 12, 10, 2, 64, 12, base=1.0e6)                  # one key/value head, all of a head rotated
GQA_BIG = grouped(3, 3, 40, 136, 5, 29, 40)                                # values wider than 128
MOE = {"kind": "moe", "expert": {"ff": 24}, "shared": {"ff": 40}, "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}}}
MOE_ONE = {"kind": "moe", "expert": {"ff": 10}, "router": {"experts": 6, "top": 1, "groups": {"count": 1, "keep": 1}}}      # no shared expert
MOE_SINGLES = {"kind": "moe", "expert": {"ff": 16}, "shared": {"ff": 8}, "router": {"experts": 4, "top": 3, "groups": {"count": 4, "keep": 3}}}
MOE_ALL = {"kind": "moe", "expert": {"ff": 32}, "shared": {"ff": 32}, "router": {"experts": 3, "top": 3}}                  # every expert chosen, no groups


def layer(mixer, mlp):
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def config(layers, width=72, vocab=150, eps=1e-5, taps=3, logit_scale=0.7):
    cfg = {"architecture": "Fezuzen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "canon": {"taps": taps}, "layers": copy.deepcopy(layers)}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    return cfg


CFG_MAIN = config([layer(LAT, MOE), layer(GQA, MOE_ALL), layer(latent(2, 24, 8, 8, 40, 16, 30, scaling=YARN, kv_from=0), None), layer(GQA_ONE_KV, MOE)], width=64)
CFG_ODD = config([layer(GQA_ODD, MOE_ONE), layer(LAT_ODD, MOE_SINGLES), layer(latent(3, 5, 7, 9, 21, 7, 4, base=10000.0, kv_from=1), MOE_ONE)],
                 width=50, vocab=77, eps=1e-3, taps=2, logit_scale=None)
CFG_ONE_TAP = config([layer(LAT_ONE, None), layer(GQA_BIG, MOE_SINGLES), layer(LAT_MANY, None), layer(GQA_TAP, MOE_ONE)], width=48, taps=1, logit_scale=2.5)
CFG_TAPS = config([layer(GQA_ONE_KV, None), layer(LAT_WIDE, MOE)], width=56, taps=6)


def build(cfg, dtype=torch.float32, seed=0, weights=None, **limits):
    from llava.model import FezuzenConfig, FezuzenForCausalLM

    w = weights if weights is not None else O.random_weights(cfg, seed=seed)
    limits = {"max_batch": 4, "max_seq": 256, **limits}
    model = FezuzenForCausalLM(FezuzenConfig(**cfg), {k: torch.from_numpy(np.asarray(v, np.float32)).bfloat16() for k, v in w.items()}, dtype=dtype, **limits)
    return model, w


def tokens_for(cfg, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def row_errors(a, b):
    a = torch.as_tensor(np.asarray(a.detach().cpu() if torch.is_tensor(a) else a), dtype=torch.float64)
    b = torch.as_tensor(np.asarray(b.detach().cpu() if torch.is_tensor(b) else b), dtype=torch.float64)
    return ((a - b) ** 2).mean(-1).sqrt() / (b.std(-1) + 1e-12)


def err(a, b):
    """rms difference over std of the reference, per row, worst row"""
    return float(row_errors(a, b).max())


def close(a, b, dtype, tight=False):
    """fp32: every row within rounding. bf16: nine rows in ten within the format's rounding (a router choice between two
    nearly equal scores may fall the other way for a row when its input is rounded to bf16)."""
    e = row_errors(a, b).flatten()
    if dtype == torch.float32:
        return float(e.max()) < (2e-5 if tight else 2e-4)
    return float(torch.quantile(e, 0.9)) < (2e-2 if tight else 6e-2)


def run_schedule(eng, kv, slot, toks, cuts, decode_single=True):
    """Feed toks in portions of the sizes `cuts` (the rest one by one); a single token of a running request takes the decode
    step when decode_single, else the portion call. Returns logits of every position."""
    out, at, first = [], 0, True
    sizes = list(cuts) + [1] * (len(toks) - sum(cuts))
    for n in sizes:
        part = toks[at:at + n]
        if n == 1 and not first and decode_single:
            out.append(eng.decode_step(kv, torch.tensor(part, dtype=torch.int32), slot0=slot))
        else:
            out.append(eng.append_tokens(kv, slot, part, list(range(n)), restart=first))
        at, first = at + n, False
    return torch.cat(out)


# ----------------------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["latent", "latent_odd", "latent_one", "latent_many", "latent_wide", "gqa", "gqa_odd", "gqa_one_kv", "gqa_big", "gqa_tap",
                                  "moe", "moe_top1", "moe_singles", "moe_all"])
def test_each_mechanism_alone(name, dtype):
    """One layer: the residual stream after it equals the oracle's x + norm_b(mechanism(u + conv(u))), u = norm(x), built here from
    the oracle's function for that mechanism."""
    mixers = {"latent": LAT, "latent_odd": LAT_ODD, "latent_one": LAT_ONE, "latent_many": LAT_MANY, "latent_wide": LAT_WIDE, "gqa": GQA,
              "gqa_odd": GQA_ODD, "gqa_one_kv": GQA_ONE_KV, "gqa_big": GQA_BIG, "gqa_tap": GQA_TAP}
    mlps = {"moe": MOE, "moe_top1": MOE_ONE, "moe_singles": MOE_SINGLES, "moe_all": MOE_ALL}
    lay = layer(mixers.get(name, GQA_ODD), mlps.get(name))
    cfg = config([lay], width=50 if name.endswith("odd") else 72, taps=4 if "gqa" in name else 3)
    model, w = build(cfg, dtype)
    toks = tokens_for(cfg, 75)
    _, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    eps = cfg["norm"]["eps"]
    x = np.asarray(w["embed"], np.float64)[toks]
    h = O.input_conv(O.rms_norm(x, w["l0.norm1"], eps), np.asarray(w["l0.canon1"], np.float64))
    p = O.layer_params(w, 0, "mix")
    y = O.latent_attention(h, p, lay["mixer"], eps) if lay["type"] == "latent_attention" else O.grouped_attention(h, p, lay["mixer"])
    x = x + O.rms_norm(y, w["l0.norm1b"], eps)
    if lay["mlp"]:
        h = O.input_conv(O.rms_norm(x, w["l0.norm2"], eps), np.asarray(w["l0.canon2"], np.float64))
        x = x + O.rms_norm(O.moe_ff(h, O.layer_params(w, 0, "mlp"), lay["mlp"]), w["l0.norm2b"], eps)
    assert close(hidden[0, 0], x, dtype)


def test_router_choices_and_weights():
    """The router alone: softmax scores, a group counted by its best expert, the raw scores as weights; three group layouts, fp32."""
    for mlp in (MOE, MOE_SINGLES, {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 12, "top": 4, "groups": {"count": 3, "keep": 1}}}):
        cfg = config([layer(GQA_ODD, mlp)], width=40)
        w = O.random_weights(cfg, seed=3)
        w["l0.mlp.router"] = O.bf16_round(w["l0.mlp.router"] * 4.0)      # spread scores: no choice is a close call
        model, _ = build(cfg, torch.float32, weights=w)
        toks = tokens_for(cfg, 60, seed=4)
        got = model.forward(torch.tensor([toks]))[0]
        assert err(got, O.forward(cfg, w, toks)) < 2e-4


# ----------------------------------------------------------------------------------------------------------- whole models
ALL_CFGS = [CFG_MAIN, CFG_ODD, CFG_ONE_TAP, CFG_TAPS]
ALL_IDS = ["main", "odd", "one_tap", "taps"]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", ALL_CFGS, ids=ALL_IDS)
def test_whole_prompt_against_the_oracle(cfg, dtype):
    model, w = build(cfg, dtype)
    toks = tokens_for(cfg, 150, seed=2)
    logits, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    ref, layers = O.forward(cfg, w, toks, return_layers=True)
    assert hidden.shape == (1, len(cfg["layers"]), len(toks), cfg["width"])
    for i in range(len(cfg["layers"])):
        assert close(hidden[0, i], layers[i], dtype), f"residual stream after layer {i}"
    assert close(logits[0], ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", ALL_CFGS, ids=ALL_IDS)
def test_portions_and_token_by_token_equal_the_whole_prompt(cfg, dtype):
    model, w = build(cfg, dtype)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    toks = tokens_for(cfg, 131, seed=3)
    whole = run_schedule(eng, kv, 0, toks, [len(toks)])
    assert close(whole, O.forward(cfg, w, toks), dtype)
    for cuts in ([1], [2] * 40, [9] * 6, [7, 2, 1, 13, 3, 2, 64, 2], [70, 2, 2, 3], [64, 64]):
        assert close(run_schedule(eng, kv, 1, toks, cuts), whole, dtype, tight=True), f"portions {cuts[:4]}.. then decode steps"
        assert close(run_schedule(eng, kv, 1, toks, cuts, decode_single=False), whole, dtype, tight=True), f"portions {cuts[:4]}.. then portions of one"


def test_the_first_tokens_of_a_sequence():
    """Prompts of one, two and three tokens (shorter than any convolution), alone and continued one token at a time."""
    cfg = CFG_TAPS
    model, w = build(cfg, torch.float32)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    toks = tokens_for(cfg, 12, seed=8)
    ref = O.forward(cfg, w, toks)
    for n in (1, 2, 3):
        assert err(run_schedule(eng, kv, 0, toks[:n], [n]), ref[:n]) < 2e-4
        assert err(run_schedule(eng, kv, 0, toks, [n]), ref) < 2e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_moves_windows_and_chunks_over_decoded_tokens(dtype):
    cfg = CFG_MAIN
    model, w = build(cfg, dtype)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    toks = tokens_for(cfg, 170, seed=5)
    got = run_schedule(eng, kv, 0, toks, [8])          # 162 decode steps: every window and chunk passes over decoded tokens many times
    ref = O.forward(cfg, w, toks)
    assert close(got[-40:], ref[-40:], dtype)
    assert close(got, ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batched_decode_of_unequal_requests_equals_each_alone(dtype):
    cfg = CFG_MAIN
    model, w = build(cfg, dtype, max_batch=6)
    eng = model._ensure_engine()
    kv = eng.new_kv(6, 256)
    reqs = [tokens_for(cfg, n, seed=10 + n) for n in (37, 14, 21, 50, 13)]
    steps = 12
    alone = [run_schedule(eng, kv, 5, r, [len(r) - steps]) for r in reqs]      # slot 5, one request after the other
    for b, r in enumerate(reqs):
        eng.append_tokens(kv, b, r[:len(r) - steps], [], restart=True)
    got = [[] for _ in reqs]
    for s in range(steps):                                                    # one decode step over the five slots
        col = torch.tensor([r[len(r) - steps + s] for r in reqs], dtype=torch.int32)
        lg = eng.decode_step(kv, col)
        for b in range(len(reqs)):
            got[b].append(lg[b])
    for b, r in enumerate(reqs):
        assert close(torch.stack(got[b]), alone[b][-steps:], dtype, tight=True), f"request {b}"
    assert close(torch.stack(got[1]), O.forward(cfg, w, reqs[1])[-steps:], dtype)


def test_a_slot_that_is_freed_and_used_again_starts_clean():
    cfg = CFG_MAIN
    model, w = build(cfg, torch.float32)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    a, b = tokens_for(cfg, 90, seed=21), tokens_for(cfg, 33, seed=22)
    fresh = run_schedule(eng, kv, 1, b, [20])
    run_schedule(eng, kv, 0, a, [50])                      # leaves cache rows and convolution tails of every kind behind
    kv.free_slot(0)
    assert kv.lengths(2)[0] == 0
    again = run_schedule(eng, kv, 0, b, [20])
    assert err(again, fresh) < 1e-6
    third = run_schedule(eng, kv, 0, b, [2, 2])            # restart on a slot that was not freed, shortest portions
    assert err(third, fresh) < 2e-5
    with pytest.raises(ValueError):
        eng.append_tokens(kv, 0, [0] * 300, [], restart=False)   # beyond the slot's capacity


# ----------------------------------------------------------------------------------------------------------- edges
def sharp_model(kind, size, seed=7):
    """One attention layer of either kind whose queries are scaled up until the softmax is almost an argmax: for most positions
    ONE visible key carries the output, as often the oldest visible one as any other. A key too many or too few at the edge of
    the window / chunk (or of a key tile of 32, a key split, a portion) then moves many rows by far more than the tolerance."""
    if kind == "window":
        lay = layer(latent(2, 16, 8, 12, 36, 24, size, base=50.0, scale=1.0), None)
    else:
        lay = layer(grouped(4, 2, 16, 12, 3, size, 16, base=50.0, scale=1.0), None)
    cfg = config([lay], width=48, vocab=400, taps=2)
    w = O.random_weights(cfg, seed=seed)
    name = "l0.mix.uq" if kind == "window" else "l0.mix.q"
    w[name] = O.bf16_round(w[name] * 14.0)
    return cfg, w


def with_mask(cfg, size):
    out = copy.deepcopy(cfg)
    out["layers"][0]["mixer"]["mask"]["size"] = size
    return out


@pytest.mark.parametrize("kind,size", [("window", 37), ("window", 64), ("window", 300), ("chunk", 37), ("chunk", 100), ("chunk", 256)])
def test_keys_just_inside_and_outside_the_mask_and_far_away(kind, size):
    T = 420
    cfg, w = sharp_model(kind, size)
    toks = tokens_for(cfg, T, seed=9)
    ref = O.forward(cfg, w, toks)
    # the test's premise: a mask that is one position larger or smaller changes many rows by much more than the tolerance (small masks:
    # every row has an edge close by), and keys further back than a third of the mask carry many rows (large masks: keys hundreds back)
    for other in (size - 1, size + 1) if size < 100 else (size // 3,):
        moved = row_errors(O.forward(with_mask(cfg, other), w, toks), ref)
        assert int((moved > 2e-2).sum()) >= (8 if size < 100 else 40), f"a mask of {other} instead of {size} would hardly show"
    model, _ = build(cfg, torch.float32, weights=w, max_batch=2, max_seq=1024, max_rows=512)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 1024)
    assert err(run_schedule(eng, kv, 0, toks, [T]), ref) < 2e-4, "whole prompt"
    assert err(run_schedule(eng, kv, 1, toks, [31, 2, 33, 64, 1, 5, 2, 2, 130]), ref) < 2e-4, "portions that end at and around tile edges, then decode steps"
    assert err(run_schedule(eng, kv, 1, toks, [size - 1, 2, 2, 64, 3]), ref) < 2e-4, "portions that end just inside and outside the first mask edge"
    assert err(run_schedule(eng, kv, 0, toks, [300]), ref) < 2e-4, "120 decode steps over split keys"
    assert err(run_schedule(eng, kv, 1, toks, [max(2, size - 2)]), ref) < 2e-4, "decode steps from just inside the first mask edge on"


def test_the_unit_in_the_softmax_denominator_shows():
    """With sharp scores every row whose best score is negative gives most of its weight to the extra 1 of the denominator (the
    first position of every chunk has one key only, and its score is negative half the time). Premise: leaving the term out moves many
    rows of the mixer's output; the engine agrees with the oracle that has it, in a prompt and in decode steps."""
    cfg, w = sharp_model("chunk", 9)
    toks = tokens_for(cfg, 150, seed=12)
    eps = cfg["norm"]["eps"]
    x = np.asarray(w["embed"], np.float64)[toks]
    h = O.input_conv(O.rms_norm(x, w["l0.norm1"], eps), np.asarray(w["l0.canon1"], np.float64))
    p, mix = O.layer_params(w, 0, "mix"), cfg["layers"][0]["mixer"]
    moved = row_errors(O.grouped_attention(h, p, mix, extra_one=False), O.grouped_attention(h, p, mix))
    assert int((moved > 0.3).sum()) >= 30
    ref = O.forward(cfg, w, toks)
    model, _ = build(cfg, torch.float32, weights=w)
    eng = model._ensure_engine()
    kv = eng.new_kv(1, 256)
    assert err(run_schedule(eng, kv, 0, toks, [150]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 0, toks, [20]), ref) < 2e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_absorbed_and_per_head_attention_agree(dtype, monkeypatch):
    """Long prompt portions make per-head keys and values from the cached rows (the rotated key part rides through an identity
    block); short ones and decode steps carry the query into the latent space instead. Both forms, forced on the same prompt and
    portions, give the same logits, also for a layer that reads another layer's rows."""
    cfg = config([layer(LAT, None), layer(LAT_WIDE, MOE), layer(latent(4, 8, 8, 12, 40, 16, 90, scaling=YARN, kv_from=0), None)], width=64)
    model, w = build(cfg, dtype, max_rows=32)     # a workspace of fewer rows than the prompt: keys and values are made in pieces
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    toks = tokens_for(cfg, 200, seed=31)
    ref = O.forward(cfg, w, toks)
    got = {}
    for name, rows in (("per head", "1"), ("absorbed", "100000")):
        monkeypatch.setenv("B2_LATENT_MATERIALISE_ROWS", rows)
        got[name] = run_schedule(eng, kv, 0, toks, [32, 32, 2, 30, 32, 32, 17])
        assert close(got[name], ref, dtype), name
    assert close(got["per head"], got["absorbed"], dtype, tight=True)


def test_experts_on_tensor_cores_equal_the_plain_products(monkeypatch):
    """Long bf16 prompt portions sort their (token, choice) pairs by expert into 128-row tiles for ONE grouped tensor-core
    product per projection; short ones and fp32 use plain grouped products. Uneven expert loads, experts without tokens."""
    mlp = {"kind": "moe", "expert": {"ff": 40}, "shared": {"ff": 32}, "router": {"experts": 10, "top": 3, "groups": {"count": 5, "keep": 3}}}
    cfg = config([layer(GQA_ODD, mlp)], width=64)
    w = O.random_weights(cfg, seed=6)
    w["l0.mlp.router"][7] = 0.0
    w["l0.mlp.router"][2] = O.bf16_round(w["l0.mlp.router"][2] * 3.0)
    model, _ = build(cfg, torch.bfloat16, weights=w, max_seq=512, max_rows=512)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 512)
    toks = tokens_for(cfg, 330, seed=23)
    ref = O.forward(cfg, w, toks)
    got = {}
    for name, flag in (("tensor cores", "1"), ("plain", "0")):
        monkeypatch.setenv("B2_SEQ_TC", flag)
        got[name] = run_schedule(eng, kv, 0, toks, [200, 65, 64])
        assert close(got[name], ref, torch.bfloat16), name
    assert close(got["tensor cores"], got["plain"], torch.bfloat16, tight=True)


def test_positions_far_along_keep_their_angles():
    """Rotations at positions in the thousands (angles of thousands of radians at the fastest pair) against the fp64 oracle."""
    cfg = config([layer(latent(2, 8, 8, 8, 16, 8, 6, base=20.0, scaling=YARN), None), layer(grouped(2, 1, 8, 8, 2, 8, 8, base=20.0), None)], width=32, vocab=60)
    model, w = build(cfg, torch.float32, max_seq=4096, max_rows=4096, max_batch=1)
    toks = tokens_for(cfg, 3500, seed=41)
    eng = model._ensure_engine()
    kv = eng.new_kv(1, 4096)
    got = run_schedule(eng, kv, 0, toks, [3490])
    ref = O.forward(cfg, w, toks)[-40:]        # windows and chunks of a few positions keep the oracle's loops short
    assert err(got[-40:], ref) < 2e-4


# ----------------------------------------------------------------------------------------------------------- generation
def greedy_matches_oracle(cfg, w, prompt, new_tokens, tol_margin=1e-3):
    """The generated ids, fed to the oracle, are its own greedy choices wherever its top-2 margin is not a rounding matter."""
    seq = list(prompt) + list(new_tokens)
    ref = torch.from_numpy(O.forward(cfg, w, seq))
    for i, t in enumerate(new_tokens):
        row = ref[len(prompt) - 1 + i]
        top = torch.topk(row, 2)
        if float(top.values[0] - top.values[1]) > tol_margin * float(row.std()):
            assert int(top.indices[0]) == int(t), f"token {i}"


def test_greedy_generation_through_generate():
    cfg = CFG_MAIN
    model, w = build(cfg, torch.float32)
    prompts = torch.tensor([tokens_for(cfg, 12, seed=51), tokens_for(cfg, 12, seed=52)])
    out = model.generate(prompts, max_new_tokens=24)       # past the first window and chunk edges
    assert out.shape == (2, 36) and torch.equal(out[:, :12], prompts)
    for b in range(2):
        greedy_matches_oracle(cfg, w, prompts[b].tolist(), out[b, 12:].tolist())
    solo = model.generate(prompts[1:2], max_new_tokens=24)
    assert torch.equal(solo[0], out[1])


def test_continuous_batching_of_unequal_requests():
    """Six generate() threads on three slots: requests join and leave between steps, slots are reused, and every request gets
    the ids it gets alone."""
    cfg = copy.deepcopy(CFG_MAIN)
    model, w = build(cfg, torch.float32)
    prompts = [torch.tensor([tokens_for(cfg, n, seed=60 + n)]) for n in (5, 19, 9, 30, 3, 14)]
    new = [6, 14, 9, 4, 12, 8]
    solo = [model.generate(p, max_new_tokens=n) for p, n in zip(prompts, new)]
    model.invalidate_engine()
    model.config.raw["b2_continuous_batching"] = 3
    results, errors = [None] * len(prompts), []

    def work(i):
        try:
            results[i] = model.generate(prompts[i], max_new_tokens=new[i])
        except BaseException as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(prompts))]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not errors, errors
    stats = model._batcher.stats
    for i in range(len(prompts)):
        assert torch.equal(results[i], solo[i]), f"request {i}"
    assert stats["admitted"] == 6 and stats["max_active"] <= 3 and stats["rows_stepped"] > stats["steps"]
    greedy_matches_oracle(cfg, w, prompts[1][0].tolist(), results[1][0, 19:].tolist())
    model.invalidate_engine()


def test_sampled_generation_repeats_with_the_seed_and_rejects_bad_input():
    cfg = CFG_ODD
    model, _ = build(cfg, torch.bfloat16)
    p = torch.tensor([tokens_for(cfg, 8, seed=71)])
    torch.manual_seed(5)
    a = model.generate(p, do_sample=True, temperature=0.9, top_k=20, top_p=0.95, max_new_tokens=12)
    torch.manual_seed(5)
    b = model.generate(p, do_sample=True, temperature=0.9, top_k=20, top_p=0.95, max_new_tokens=12)
    assert torch.equal(a, b) and int(a.max()) < cfg["vocab"]
    with pytest.raises(ValueError):
        model.generate(torch.tensor([[cfg["vocab"] + 3, 1, 2]]), max_new_tokens=2)
    with pytest.raises(ValueError):
        model.generate(p, max_new_tokens=4000)


# ----------------------------------------------------------------------------------------------------------- the replay program
def write_checkpoint(path, cfg, weights):
    import json
    import os
    import struct

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, at = {}, [], 0
    for k, v in weights.items():
        raw = torch.from_numpy(np.asarray(v, np.float32)).bfloat16().contiguous().view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": "BF16", "shape": list(np.asarray(v).shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program_on_a_written_checkpoint(dtype, tmp_path, repo_root):
    """bin/trace_run on a checkpoint directory: two requests one after the other on slots that are given back, portions down to two
    tokens, single tokens through the decode step, steps that want nothing; every written row against the oracle."""
    import json
    import subprocess
    import sys

    cfg = CFG_ODD
    w = O.random_weights(cfg, seed=13)
    write_checkpoint(str(tmp_path / "model"), cfg, w)
    a, b = tokens_for(cfg, 60, seed=31), tokens_for(cfg, 23, seed=32)
    steps, want_rows, at = [], [], 0
    for n in (17, 2, 30, 2):                                                   # request a in portions, the last one asks for nothing
        want = [] if n == 30 else list(range(0, n, 3))
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": a[at:at + n], "want": want}], "end": []})
        want_rows.append(("a", [at + i for i in want]))
        at += n
    for t in range(at, len(a)):                                                # then token by token
        steps.append({"step": len(steps), "entries": [{"id": "a", "tokens": [a[t]], "want": [0]}], "end": ["a"] if t == len(a) - 1 else []})
        want_rows.append(("a", [t]))
    steps.append({"step": len(steps), "entries": [{"id": "b", "tokens": b, "want": [0, len(b) - 1]}], "end": ["b"]})
    want_rows.append(("b", [0, len(b) - 1]))
    out = tmp_path / "out"
    run = subprocess.run([sys.executable, f"{repo_root}/bin/trace_run", "--model", str(tmp_path / "model"), "--dtype", dtype, "--out", str(out),
                          "--max-tokens", "64"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stderr[-2000:]
    assert [ln for ln in run.stdout.splitlines() if ln.startswith("done ")] == [f"done {i}" for i in range(len(steps))]
    ref = {"a": O.forward(cfg, w, a), "b": O.forward(cfg, w, b)}
    got, exp = [], []
    for i, (rid, rows) in enumerate(want_rows):
        path = out / f"{i}.f32"
        if not rows:
            assert not path.exists()
            continue
        got.append(np.fromfile(path, dtype="<f4").reshape(len(rows), cfg["vocab"]))
        exp.append(ref[rid][rows])
    assert close(torch.from_numpy(np.concatenate(got)), np.concatenate(exp), torch.float32 if dtype == "float32" else torch.bfloat16)
