"""Sofopel on the engine against the plain oracle (oracle/sofopel_oracle.py): every mechanism alone, prompts in one piece, in
portions down to two tokens and token by token, batched decode steps of unequal requests, slots that are freed and used again,
keys far away, at the edges of key tiles and just inside / outside every window, kept range and chunk (in prompts and in decode
steps), the first tokens of a sequence, long decoding, looped blocks, greedy generation through generate() and the continuous
batcher, the replay program. Small configurations whose sizes differ from one another (and from multiples of the kernels' tiles),
random weights, both number formats; where random weights would hide a fault the weights are shaped so that it shows."""
import copy
import threading

import numpy as np
import pytest
import torch

from oracle import sofopel_oracle as O

pytestmark = pytest.mark.gpu

YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}


def gla(heads, dim, vdim, tau=6.0):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}}


def diff(heads, kv_heads, dim, vdim, conv, chunk, rot_dims, lam0=0.7, base=100.0, scale=0.25):
    mix = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": lam0, "scale": scale}
    if conv is not None:
        mix["conv"] = conv
    if chunk is not None:
        mix["mask"] = {"size": chunk}
    if rot_dims:
        mix["rot"] = {"base": base, "dims": rot_dims}
    return {"type": "attention", "mixer": mix}


def win(heads, kv_heads, dim, vdim, size, keep, rot_dims, base=500.0, scaling=None, scale=0.3):
    mix = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        mix["mask"] = {"size": size} if keep is None else {"size": size, "keep_first": keep}
    if rot_dims:
        mix["rot"] = {"base": base, "dims": rot_dims}
        if scaling:
            mix["rot"]["scaling"] = dict(scaling)
    return {"type": "attention_2", "mixer": mix}


GLA = gla(3, 16, 24)
GLA_ODD = gla(5, 9, 7, tau=3.5)                      # nothing a multiple of 4
GLA_ONE = gla(1, 40, 136, tau=1.0)                   # one head, values wider than 128, tau 1: the plain sigmoid
GLA_WIDE = gla(2, 136, 12, tau=20.0)                 # keys beyond 128: sixteen keys of the state per thread
DIFF = diff(4, 2, 12, 20, 3, 13, 6)                  # two query heads per key/value head, half of every map rotated
DIFF_ODD = diff(3, 3, 7, 9, 0, 5, 4, lam0=0.35)      # no convolution, odd sizes
DIFF_TAP = diff(2, 1, 8, 4, 1, 1, 2, lam0=0.5)       # a convolution of ONE tap, chunks of one position, one rotated pair, one key/value head
DIFF_FREE = diff(6, 2, 16, 136, 5, None, 16, base=1.0e4)    # no mask, all of a map rotated, values wider than 128
WIN = win(6, 2, 16, 24, 11, 3, 8, scaling=YARN)      # part of a head rotated with scaled frequencies
WIN_ODD = win(2, 2, 9, 7, 4, 9, 4, base=10000.0)     # more kept positions than the window holds, odd sizes, a rotated part that ends inside the head
WIN_ONE = win(1, 1, 8, 8, 1, 1, 8)                   # one head, a window of the query alone plus position 0
WIN_PLAIN = win(4, 1, 12, 10, 64, None, 12, base=1.0e6)     # no kept positions, one key/value head, all of a head rotated
WIN_FREE = win(3, 3, 20, 40, None, None, 0)          # no mask and no rotation
DENSE = {"kind": "dense", "ff": 40, "limit": 1.25}
DENSE_ODD = {"kind": "dense", "ff": 27, "limit": 0.5}
DENSE_LOOSE = {"kind": "dense", "ff": 64, "limit": 100.0}


def layer(mixer, mlp):
    out = copy.deepcopy(mixer)
    out["mlp"] = copy.deepcopy(mlp)
    return out


def config(layers, width=72, vocab=150, eps=1e-5, scale=2.0, mult=0.6, loop=None):
    cfg = {"architecture": "Sofopel", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": copy.deepcopy(layers)}
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    if mult is not None:
        cfg["residual_mult"] = mult
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


CFG_MAIN = config([layer(WIN, DENSE), layer(GLA, DENSE_ODD), layer(DIFF, None), layer(WIN_PLAIN, DENSE)], width=64, loop=(1, 3, 2))
CFG_ODD = config([layer(DIFF_ODD, DENSE_ODD), layer(GLA_ODD, None), layer(WIN_ODD, DENSE_ODD)], width=50, vocab=77, eps=1e-3, scale=None, mult=None)
CFG_ONE = config([layer(WIN_ONE, None), layer(DIFF_TAP, DENSE_LOOSE), layer(GLA_ONE, DENSE)], width=48, mult=1.3, loop=(0, 3, 3))
CFG_WIDE = config([layer(GLA_WIDE, DENSE), layer(DIFF_FREE, DENSE), layer(WIN_FREE, None)], width=56, scale=0.5, loop=(2, 3, 1))
ALL_CFGS = [CFG_MAIN, CFG_ODD, CFG_ONE, CFG_WIDE]
ALL_IDS = ["main", "odd", "one", "wide"]
RANKS = {"main": {1: 8}, "odd": {1: 5}, "one": {2: 1}, "wide": {0: 40}}     # inner size of the decay projection, by layer


def ranks_of(cfg):
    for c, name in zip(ALL_CFGS, ALL_IDS):
        if c is cfg:
            return RANKS[name]
    return None


def build(cfg, dtype=torch.float32, seed=0, weights=None, **limits):
    from llava.model import SofopelConfig, SofopelForCausalLM

    w = weights if weights is not None else O.random_weights(cfg, seed=seed, ranks=ranks_of(cfg))
    limits = {"max_batch": 4, "max_seq": 256, **limits}
    model = SofopelForCausalLM(SofopelConfig(**cfg), {k: torch.from_numpy(np.asarray(v, np.float32)).bfloat16() for k, v in w.items()}, dtype=dtype, **limits)
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
    """fp32: every row within rounding. bf16: nine rows in ten within the format's rounding."""
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
MIXERS = {"gla": GLA, "gla_odd": GLA_ODD, "gla_one": GLA_ONE, "gla_wide": GLA_WIDE, "diff": DIFF, "diff_odd": DIFF_ODD, "diff_tap": DIFF_TAP,
          "diff_free": DIFF_FREE, "win": WIN, "win_odd": WIN_ODD, "win_one": WIN_ONE, "win_plain": WIN_PLAIN, "win_free": WIN_FREE}
MLPS = {"dense": DENSE, "dense_odd": DENSE_ODD, "dense_loose": DENSE_LOOSE}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", list(MIXERS) + list(MLPS))
def test_each_mechanism_alone(name, dtype):
    """One layer: the residual stream after it equals x + m * (mixer(u) + ff(u)), u = rms_w(x), built here from the oracle's function
    for that mechanism. A feed-forward is tested beside the smallest mixer."""
    lay = layer(MIXERS.get(name, WIN_ONE), MLPS.get(name))
    cfg = config([lay], width=50 if name.endswith("odd") else 72, mult=0.8)
    w = O.random_weights(cfg, seed=2, ranks={0: 3 if name.endswith("odd") else 16})
    model, _ = build(cfg, dtype, weights=w)
    toks = tokens_for(cfg, 75)
    _, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    eps = cfg["norm"]["eps"]
    x = np.asarray(w["embed"], np.float64)[toks] * 2.0
    u = O.rms_norm(x, w["l0.norm1"], eps)
    y = O.MIXERS[lay["type"]](u, O.layer_params(w, 0, "mix"), lay["mixer"], eps)
    if lay["mlp"]:
        y = y + O.clamped_glu(u, O.layer_params(w, 0, "mlp"), lay["mlp"])
    assert close(hidden[0, 0], x + 0.8 * y, dtype)


def test_the_bounds_of_the_gated_unit_show():
    """Inputs scaled until most gate and up values pass their limit: the engine follows the oracle, and an oracle without limit is far away."""
    cfg = config([layer(WIN_ONE, DENSE_ODD)], width=40)
    w = O.random_weights(cfg, seed=5)
    for n in ("l0.mlp.gate", "l0.mlp.up"):
        w[n] = O.bf16_round(w[n] * 4.0)
    toks = tokens_for(cfg, 40, seed=3)
    ref = O.forward(cfg, w, toks)
    loose = copy.deepcopy(cfg)
    loose["layers"][0]["mlp"]["limit"] = 1.0e9
    assert float(row_errors(O.forward(loose, w, toks), ref).median()) > 0.3
    model, _ = build(cfg, torch.float32, weights=w)
    eng = model._ensure_engine()
    kv = eng.new_kv(1, 256)
    assert err(run_schedule(eng, kv, 0, toks, [30]), ref) < 2e-4          # the prompt's unit and the decode step's fused one


# ----------------------------------------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", ALL_CFGS, ids=ALL_IDS)
def test_whole_prompt_against_the_oracle(cfg, dtype):
    model, w = build(cfg, dtype)
    toks = tokens_for(cfg, 150, seed=2)
    logits, hidden = model.forward(torch.tensor([toks]), output_hidden_states=True)
    ref, layers = O.forward(cfg, w, toks, return_layers=True)
    runs = len(O.layer_order(cfg))
    assert hidden.shape == (1, runs, len(toks), cfg["width"])          # a looped layer counts every time
    for i in range(runs):
        assert close(hidden[0, i], layers[i], dtype), f"residual stream after layer run {i}"
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
    """Prompts of one, two and three tokens (shorter than the convolution, inside the kept range), alone and continued one by one."""
    cfg = CFG_MAIN
    model, w = build(cfg, torch.float32)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 256)
    toks = tokens_for(cfg, 12, seed=8)
    ref = O.forward(cfg, w, toks)
    for n in (1, 2, 3):
        assert err(run_schedule(eng, kv, 0, toks[:n], [n]), ref[:n]) < 2e-4
        assert err(run_schedule(eng, kv, 0, toks, [n]), ref) < 2e-4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_moves_windows_chunks_and_state_over_decoded_tokens(dtype):
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
    run_schedule(eng, kv, 0, a, [50])                      # leaves cache rows, recurrent state and convolution tails of every pass behind
    kv.free_slot(0)
    assert kv.lengths(2)[0] == 0
    again = run_schedule(eng, kv, 0, b, [20])
    assert err(again, fresh) < 1e-6
    third = run_schedule(eng, kv, 0, b, [2, 2])            # restart on a slot that was not freed, shortest portions
    assert err(third, fresh) < 2e-5
    with pytest.raises(ValueError):
        eng.append_tokens(kv, 0, [0] * 300, [], restart=False)   # beyond the slot's capacity


def test_every_pass_of_a_looped_layer_has_its_own_state():
    """Three passes over all three layers against a model that lists the same tensors nine times: equal only if no pass shares a cache,
    a recurrent state or a convolution tail with another, in a prompt, in portions and in decode steps."""
    cfg = CFG_ONE
    w = O.random_weights(cfg, seed=0, ranks=RANKS["one"])
    flat = copy.deepcopy(cfg)
    del flat["loop"]
    flat["layers"] = [copy.deepcopy(cfg["layers"][i % 3]) for i in range(9)]
    wf = {k: v for k, v in w.items() if not k.startswith("l")}
    for i in range(9):
        wf.update({f"l{i}." + k.split(".", 1)[1]: v for k, v in w.items() if k.startswith(f"l{i % 3}.")})
    toks = tokens_for(cfg, 60, seed=6)
    ref = O.forward(cfg, w, toks)
    assert np.allclose(ref, O.forward(flat, wf, toks))
    model, _ = build(cfg, torch.float32, weights=w)
    eng = model._ensure_engine()
    kv = eng.new_kv(1, 256)
    for cuts in ([60], [13, 2, 20], [2]):
        assert err(run_schedule(eng, kv, 0, toks, cuts), ref) < 2e-4


# ----------------------------------------------------------------------------------------------------------- edges
def sharp_model(kind, size, keep=None, seed=7):
    """One attention layer of either kind whose scores are scaled up until the softmax is almost an argmax: for most positions ONE
    visible key carries the output, as often the oldest visible one as any other. A key too many or too few at the edge of the window,
    the kept range or the chunk (or of a key tile of 32, a key split, a portion) then moves many rows by far more than the tolerance."""
    if kind == "window":
        lay = layer(win(4, 2, 16, 12, size, keep, 8, base=50.0, scale=3.0), None)      # q and k are normed: the score's factor sharpens
    else:
        lay = layer(diff(4, 2, 16, 12, 3, size, 16, lam0=0.4, base=50.0, scale=1.0), None)
    cfg = config([lay], width=48, vocab=400)
    w = O.random_weights(cfg, seed=seed)
    if kind != "window":
        w["l0.mix.q"] = O.bf16_round(w["l0.mix.q"] * 14.0)
    return cfg, w


def with_mask(cfg, **mask):
    out = copy.deepcopy(cfg)
    out["layers"][0]["mixer"]["mask"].update(mask)
    return out


@pytest.mark.parametrize("kind,size,keep", [("window", 37, 5), ("window", 64, 33), ("window", 300, 0), ("window", 29, 70), ("chunk", 37, None),
                                            ("chunk", 100, None), ("chunk", 256, None)])
def test_keys_just_inside_and_outside_the_mask_and_far_away(kind, size, keep):
    T = 420
    cfg, w = sharp_model(kind, size, keep)
    toks = tokens_for(cfg, T, seed=9)
    ref = O.forward(cfg, w, toks)
    # the test's premise: a mask that is one position larger or smaller changes many rows by much more than the tolerance (small masks:
    # every row has an edge close by), keys further back than a third of a large mask carry many rows, and so do the kept first positions
    # (one more or one fewer of them shows, as does leaving them out)
    for other in (size - 1, size + 1) if size < 100 else (size // 3,):
        moved = row_errors(O.forward(with_mask(cfg, size=other), w, toks), ref)
        assert int((moved > 2e-2).sum()) >= (8 if size < 100 else 40), f"a mask of {other} instead of {size} would hardly show"
    if keep:
        for other, least in ((keep - 1, 3), (keep + 1, 3), (0, 20)):
            moved = row_errors(O.forward(with_mask(cfg, keep_first=other), w, toks), ref)
            assert int((moved > 2e-2).sum()) >= least, f"{other} kept positions instead of {keep} would hardly show"
    model, _ = build(cfg, torch.float32, weights=w, max_batch=2, max_seq=1024, max_rows=512)
    eng = model._ensure_engine()
    kv = eng.new_kv(2, 1024)
    assert err(run_schedule(eng, kv, 0, toks, [T]), ref) < 2e-4, "whole prompt"
    assert err(run_schedule(eng, kv, 1, toks, [31, 2, 33, 64, 1, 5, 2, 2, 130]), ref) < 2e-4, "portions that end at and around tile edges, then decode steps"
    assert err(run_schedule(eng, kv, 1, toks, [size - 1, 2, 2, 64, 3]), ref) < 2e-4, "portions that end just inside and outside the first mask edge"
    assert err(run_schedule(eng, kv, 0, toks, [300]), ref) < 2e-4, "120 decode steps over split keys"
    assert err(run_schedule(eng, kv, 1, toks, [max(2, size - 2)]), ref) < 2e-4, "decode steps from just inside the first mask edge on"
    if keep:
        assert err(run_schedule(eng, kv, 0, toks, [max(2, keep - 1), 2, 2]), ref) < 2e-4, "portions that end around the kept range, then decode steps"


def test_the_unit_in_the_softmax_denominator_shows():
    """With sharp scores every row whose best score is negative gives most of its weight to the extra 1 of the denominator. Premise:
    leaving the term out moves many rows of the mixer's output; the engine agrees with the oracle that has it, in a prompt and in
    decode steps over split keys."""
    cfg, w = sharp_model("window", 3, 1)
    toks = tokens_for(cfg, 150, seed=12)
    eps = cfg["norm"]["eps"]
    u = O.rms_norm(np.asarray(w["embed"], np.float64)[toks] * 2.0, w["l0.norm1"], eps)
    p, mix = O.layer_params(w, 0, "mix"), cfg["layers"][0]["mixer"]
    moved = row_errors(O.window_attention(u, p, mix, eps, extra_one=False), O.window_attention(u, p, mix, eps))
    assert int((moved > 0.3).sum()) >= 30
    ref = O.forward(cfg, w, toks)
    model, _ = build(cfg, torch.float32, weights=w)
    eng = model._ensure_engine()
    kv = eng.new_kv(1, 256)
    assert err(run_schedule(eng, kv, 0, toks, [150]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 0, toks, [20]), ref) < 2e-4


def test_the_second_map_and_its_factor_show():
    """Differential attention with a learned factor far from its constant: an oracle whose lambda is the constant alone, or whose maps
    are swapped, is far away; the engine follows the right one with three query heads per key/value head."""
    cfg = config([layer(diff(6, 2, 8, 10, 2, 40, 4, lam0=0.3), None)], width=40)
    w = O.random_weights(cfg, seed=3)
    w["l0.mix.lq1"], w["l0.mix.lk1"] = O.bf16_round(np.full(8, 0.5)), O.bf16_round(np.full(8, -0.4))
    w["l0.mix.lq2"], w["l0.mix.lk2"] = O.bf16_round(np.full(8, 0.3)), O.bf16_round(np.full(8, 0.45))
    toks = tokens_for(cfg, 90, seed=4)
    ref = O.forward(cfg, w, toks)
    flat = dict(w, **{"l0.mix." + n: np.zeros(8, np.float32) for n in ("lq1", "lk1", "lq2", "lk2")})
    assert float(row_errors(O.forward(cfg, flat, toks), ref).median()) > 0.1
    swapped = dict(w)
    for n, rows in (("q", 6), ("k", 2)):
        m = np.asarray(w[f"l0.mix.{n}"]).reshape(rows, 2, 8, -1)
        swapped[f"l0.mix.{n}"] = m[:, ::-1].reshape(rows * 16, -1).copy()
    assert float(row_errors(O.forward(cfg, swapped, toks), ref).median()) > 0.1
    model, _ = build(cfg, torch.float32, weights=w)
    eng = model._ensure_engine()
    kv = eng.new_kv(1, 256)
    assert err(run_schedule(eng, kv, 0, toks, [90]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 0, toks, [33, 2, 40]), ref) < 2e-4


def test_the_recurrent_state_remembers_far_tokens_and_forgets_by_its_decay():
    """Decay biases high enough that some channels keep hundreds of tokens and others a few: an oracle that starts its state 150
    tokens late, or whose tau is doubled, is far away from the last rows; the engine agrees with the right one in a prompt, in
    portions whose edges fall inside the scan's token tiles, and in decode steps."""
    cfg = config([layer(gla(2, 24, 20, tau=4.0), None)], width=40, vocab=300)
    w = O.random_weights(cfg, seed=8, ranks={0: 6})
    w["l0.mix.a2.b"] = O.bf16_round(np.linspace(0.0, 9.0, 48))
    T = 330
    toks = tokens_for(cfg, T, seed=9)
    ref = O.forward(cfg, w, toks)
    late = O.forward(cfg, w, toks[150:])
    assert float(row_errors(late[-40:], ref[-40:]).median()) > 0.01
    slow = copy.deepcopy(cfg)
    slow["layers"][0]["mixer"]["tau"] = 8.0
    assert float(row_errors(O.forward(slow, w, toks)[-40:], ref[-40:]).median()) > 0.01
    model, _ = build(cfg, torch.float32, weights=w, max_seq=512, max_rows=512)
    eng = model._ensure_engine()
    kv = eng.new_kv(1, 512)
    assert err(run_schedule(eng, kv, 0, toks, [T]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 0, toks, [15, 2, 16, 17, 1, 33, 2, 100]), ref) < 2e-4
    assert err(run_schedule(eng, kv, 0, toks, [200]), ref) < 2e-4


def test_positions_far_along_keep_their_angles():
    """Rotations at positions in the thousands (angles of thousands of radians at the fastest pair) in both pair layouts, fp64 oracle."""
    cfg = config([layer(win(2, 1, 8, 8, 6, 2, 8, base=20.0, scaling=YARN), None), layer(diff(2, 1, 8, 8, 2, 8, 8, base=20.0), None)], width=32, vocab=60)
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
    model, w = build(cfg, torch.float32, weights=O.random_weights(cfg, seed=0, ranks=RANKS["main"]))
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


def test_a_checkpoint_without_its_tensors_is_refused():
    cfg = CFG_ODD
    w = O.random_weights(cfg, seed=0, ranks=RANKS["odd"])
    for missing in ("l0.mix.lq2", "l1.mix.a2.b", "l2.mix.k.norm", "l2.mlp.gate", "final.norm"):
        model, _ = build(cfg, torch.float32, weights={k: v for k, v in w.items() if k != missing})
        with pytest.raises(Exception, match=missing.replace(".", r"\.")):
            model._ensure_engine()


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

    cfg = CFG_MAIN
    w = O.random_weights(cfg, seed=13, ranks=RANKS["main"])
    write_checkpoint(str(tmp_path / "model"), cfg, w)
    a, b = tokens_for(cfg, 60, seed=31), tokens_for(cfg, 23, seed=32)
    steps, want_rows, at = [], [], 0
    for n in (17, 2, 30, 2):                                                   # request a in portions, the last but one asks for nothing
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
