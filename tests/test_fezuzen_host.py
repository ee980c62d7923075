"""CPU checks around Fezuzen: the registry and configuration reader, and properties of the plain oracle that the GPU tests rely
on (causality, masks, rotations that undo themselves, scaled frequencies by hand, the router by hand, borrowed cache rows)."""
import json
import math

import numpy as np

from oracle import fezuzen_oracle as O

YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
LAT = {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 12, "q_rank": 10, "mask": {"size": 5},
                                             "rot": {"base": 500.0, "dims": 4, "scaling": YARN}, "scale": 0.5}}
LAT_B = {"type": "latent_attention", "mixer": {"heads": 3, "dim": 6, "rot_dim": 4, "vdim": 4, "kv_rank": 12, "q_rank": 7, "mask": {"size": 3}, "kv_from": 0,
                                               "rot": {"base": 500.0, "dims": 4, "scaling": YARN}, "scale": 0.4}}
GQA = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 8, "conv": 3, "mask": {"size": 4}, "rot": {"base": 100.0, "dims": 4},
                                      "scale": 0.3}}
MOE = {"kind": "moe", "expert": {"ff": 8}, "shared": {"ff": 12}, "router": {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 2}}}
CFG = {"architecture": "Fezuzen", "width": 32, "vocab": 50, "norm": {"eps": 1e-5}, "canon": {"taps": 3}, "logit_scale": 0.25,
       "layers": [dict(LAT, mlp=MOE), dict(GQA, mlp=None), dict(LAT_B, mlp=MOE)]}


def test_registry_and_configuration_reader(tmp_path):
    from llava._b2 import BLOCK_SANDWICH_RMS, FF_MOE, MASK_CHUNK, MASK_WINDOW, MIXER_GQA_ATTN, MIXER_LATENT_ATTN, MOE_ACT_RELU_SQ, MOE_GROUP_MAX, MOE_SCORE_SOFTMAX
    from llava.model import MODEL_REGISTRY, FezuzenConfig, model_class_for

    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert "Fezuzen" in MODEL_REGISTRY and model_class_for(str(tmp_path)).__name__ == "FezuzenForCausalLM"
    c = FezuzenConfig.from_pretrained(str(tmp_path))
    md = c.model_desc()
    assert md["block"] == BLOCK_SANDWICH_RMS and md["input_conv_taps"] == 3 and md["logit_scale"] == 0.25
    d = c.layer_descs({})
    assert [x["type"] for x in d] == [MIXER_LATENT_ATTN, MIXER_GQA_ATTN, MIXER_LATENT_ATTN]
    assert (d[0]["la_q_rank"], d[0]["la_rot_dim"], d[0]["la_rank"], d[0]["la_kv_from"], d[0]["mask_kind"], d[0]["mask_size"]) == (10, 4, 12, 0, MASK_WINDOW, 5)
    assert d[0]["la_no_sink"] == 1 and d[0]["la_no_gate"] == 1 and d[0]["rot_factor"] == 4.0 and d[0]["rot_original"] == 32.0
    assert d[2]["la_kv_from"] == 1 and d[2]["la_heads"] == 3                       # 1 + the layer it reads
    assert (d[1]["ga_heads"], d[1]["ga_kv_heads"], d[1]["ga_conv"], d[1]["mask_kind"], d[1]["rot_dims"]) == (4, 2, 3, MASK_CHUNK, 4)
    assert d[1]["ga_sink"] == 1 and d[1]["ga_sink_value"] == 0.0 and d[1]["ga_rot_values"] == 1 and "rot_factor" not in d[1] and d[1]["ff"] == 0
    assert d[0]["ff_kind"] == FF_MOE and (d[0]["moe_experts"], d[0]["moe_top"], d[0]["moe_groups"], d[0]["moe_keep"], d[0]["moe_shared_ff"]) == (6, 2, 3, 2, 12)
    assert (d[0]["moe_score"], d[0]["moe_group_score"], d[0]["moe_raw_weights"], d[0]["moe_act"]) == (MOE_SCORE_SOFTMAX, MOE_GROUP_MAX, 1, MOE_ACT_RELU_SQ)
    plain = {k: v for k, v in CFG.items() if k != "logit_scale"}
    assert FezuzenConfig(**plain).model_desc()["logit_scale"] == 1.0


def test_oracle_is_causal_and_keeps_its_masks():
    w = O.random_weights(CFG, seed=1)
    a = list(range(3, 23))
    b = a[:12] + [49 - t for t in a[12:]]
    la, sa = O.forward(CFG, w, a, return_layers=True)
    lb = O.forward(CFG, w, b)
    assert np.allclose(la[:12], lb[:12]) and not np.allclose(la[12:], lb[12:])
    assert sa.shape == (3, 20, 32)
    assert O.visible_keys(10, "window", 4) == [7, 8, 9, 10] and O.visible_keys(10, "chunk", 4) == [8, 9, 10]
    assert O.visible_keys(8, "chunk", 4) == [8] and O.visible_keys(2, "window", 4) == [0, 1, 2] and O.visible_keys(3, None, None) == [0, 1, 2, 3]
    # a one-layer attention model forgets what lies outside its chunk, convolutions aside: changing token 0 leaves position 9 alone
    # once the chunk (4) and the taps (3 + 3) no longer reach it
    one = dict(CFG, layers=[dict(GQA, mlp=None)])
    w1 = O.random_weights(one, seed=2)
    x, y = O.forward(one, w1, a), O.forward(one, w1, [a[0] + 1] + a[1:])
    assert not np.allclose(x[3], y[3]) and np.allclose(x[9:], y[9:])


def test_rotations():
    f, mag = O.rotary_frequencies({"base": 100.0, "dims": 4})
    assert np.allclose(f, [1.0, 0.1]) and mag == 1.0
    v = np.array([1.0, 2.0, 3.0, 4.0, 5.0])
    r = O.rotate_pairs(v, 3, f)
    assert np.allclose(r[0], math.cos(3) - 2 * math.sin(3)) and np.allclose(r[1], 2 * math.cos(3) + math.sin(3)) and r[4] == 5.0
    assert np.allclose(O.rotate_pairs(r, -3, f), v)
    # scaled frequencies by hand: dims 8, base 500, original 32, fast 8 -> lo 0, slow 1 -> hi 2; ramp 0, 1/2, 1, 1
    f, mag = O.rotary_frequencies({"base": 500.0, "dims": 8, "scaling": YARN})
    plain = np.array([500.0 ** (-2 * i / 8) for i in range(4)])
    assert np.allclose(f, [plain[0], plain[1] * (0.5 / 4 + 0.5), plain[2] / 4, plain[3] / 4]) and abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-12


def test_group_limited_softmax_routing():
    r = {"experts": 6, "top": 2, "groups": {"count": 3, "keep": 1}}
    logits = np.array([[1.0, -9.0, 1.2, 1.1, 0.5, -9.0]])          # the group of the best single expert wins, and both choices come from it
    chosen, weights = O.route(logits, np.eye(6), r)
    assert chosen[0] == [2, 3]
    s = np.exp(logits[0]) / np.exp(logits[0]).sum()
    assert np.allclose(weights[0], [s[2], s[3]]) and sum(weights[0]) < 1.0       # the scores as they are
    chosen, _ = O.route(logits, np.eye(6), dict(r, groups={"count": 3, "keep": 3}))
    assert chosen[0] == [2, 3]
    chosen, _ = O.route(logits, np.eye(6), dict(r, groups={"count": 3, "keep": 2}, top=3))
    assert chosen[0] == [2, 3, 0]
    h = np.array([[2.0, -1.0]])
    assert np.allclose(O.expert(h, np.array([[1.0, 0.0], [0.0, 1.0]]), np.array([[1.0, 1.0]])), [[4.0]])   # relu, then the square


def test_borrowed_cache_rows_are_the_owner_s():
    w = O.random_weights(CFG, seed=3)
    h = np.random.default_rng(0).standard_normal((9, 32))
    own = O.latent_kv(h, O.layer_params(w, 0, "mix"), LAT["mixer"], 1e-5)
    p = O.layer_params(w, 2, "mix")
    assert "dkv" not in p and "uk" in p
    a = O.latent_attention(h, p, LAT_B["mixer"], 1e-5, kv=own)
    b = O.latent_attention(h, p, LAT_B["mixer"], 1e-5, kv=(own[0] * 2.0, own[1]))
    assert a.shape == (9, 32) and not np.allclose(a, b)


def test_runner_help_names_the_replay_protocol(repo_root):
    import subprocess
    import sys

    out = subprocess.run([sys.executable, f"{repo_root}/bin/trace_run", "--help"], capture_output=True, text=True)
    assert out.returncode == 0 and "--max-tokens" in out.stdout and "done <step>" in out.stdout
