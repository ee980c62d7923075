"""CPU checks around Sofopel: the registry and configuration reader, and properties of the plain oracle that the GPU tests rely on
(causality, both masks, both pair layouts, scaled frequencies by hand, the decay and the recurrence by hand, the two maps, the bounded
gated unit, the order of looped layers)."""
import json
import math

import numpy as np

from oracle import sofopel_oracle as O

YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
GLA = {"type": "gla", "mixer": {"heads": 3, "dim": 4, "vdim": 6, "tau": 5.0}}
DIFF = {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 8, "conv": 3, "diff": 0.7, "mask": {"size": 4},
                                       "rot": {"base": 100.0, "dims": 4}, "scale": 0.3}}
WIN = {"type": "attention_2", "mixer": {"heads": 4, "kv_heads": 1, "dim": 8, "vdim": 6, "mask": {"size": 5, "keep_first": 2},
                                        "rot": {"base": 500.0, "dims": 6, "scaling": YARN}, "scale": 0.4}}
DENSE = {"kind": "dense", "ff": 20, "limit": 1.25}
CFG = {"architecture": "Sofopel", "width": 32, "vocab": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.5}, "residual_mult": 0.75,
       "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [dict(WIN, mlp=DENSE), dict(GLA, mlp=None), dict(DIFF, mlp=DENSE)]}


def test_registry_and_configuration_reader(tmp_path):
    from llava._b2 import BLOCK_PARALLEL_RMS, FF_CLAMP_GLU, GATE_HEAD, GATE_NONE, MASK_CAUSAL, MASK_CHUNK, MASK_WINDOW, MIXER_GLA, MIXER_GQA_ATTN
    from llava.model import MODEL_REGISTRY, SofopelConfig, model_class_for

    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert "Sofopel" in MODEL_REGISTRY and model_class_for(str(tmp_path)).__name__ == "SofopelForCausalLM"
    c = SofopelConfig.from_pretrained(str(tmp_path))
    md = c.model_desc()
    assert md["block"] == BLOCK_PARALLEL_RMS and md["embed_scale"] == 2.5 and md["residual_mult"] == 0.75
    assert (md["loop_start"], md["loop_stop"], md["loop_times"], md["loop_plain"]) == (1, 3, 2, 1)
    d = c.layer_descs({"l1.mix.a1": (7, 32)})
    assert [x["type"] for x in d] == [MIXER_GQA_ATTN, MIXER_GLA, MIXER_GQA_ATTN]
    assert (d[1]["gl_heads"], d[1]["gl_dim"], d[1]["gl_vdim"], d[1]["gl_rank"], d[1]["gl_tau"], d[1]["ff"]) == (3, 4, 6, 7, 5.0, 0)
    w, a = d[0], d[2]
    assert (w["ga_heads"], w["ga_kv_heads"], w["ga_dim"], w["ga_vdim"], w["mask_kind"], w["mask_size"], w["mask_keep"]) == (4, 1, 8, 6, MASK_WINDOW, 5, 2)
    assert w["ga_qk_norm"] == 1 and w["ga_rot_half"] == 1 and w["ga_sink"] == 1 and w["ga_sink_value"] == 0.0 and w["ga_gate"] == GATE_HEAD
    assert w["rot_dims"] == 6 and w["rot_factor"] == 4.0 and w["rot_original"] == 32.0 and "ga_maps" not in w and "ga_conv" not in w
    assert (w["ff_kind"], w["ff"], w["ff_limit"]) == (FF_CLAMP_GLU, 20, 1.25) and abs(w["ff_act_slope"] - 1.702) < 1e-12
    assert (a["ga_maps"], a["ga_diff"], a["ga_conv"], a["ga_gate"], a["mask_kind"], a["mask_size"]) == (2, 0.7, 3, GATE_NONE, MASK_CHUNK, 4)
    assert "mask_keep" not in a and "rot_factor" not in a and "ga_sink" not in a
    # what a configuration may leave out: loop, embedding scale, residual factor, masks, rotations, the convolution (read from the checkpoint)
    bare = {"architecture": "Sofopel", "width": 16, "vocab": 9, "norm": {"eps": 1e-6},
            "layers": [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 4, "vdim": 4, "diff": 0.5, "scale": 1.0}, "mlp": None},
                       {"type": "attention_2", "mixer": {"heads": 2, "dim": 4, "vdim": 4, "scale": 1.0}}]}
    b = SofopelConfig(**bare)
    assert b.model_desc() == dict(block=BLOCK_PARALLEL_RMS, residual_mult=1.0, embed_scale=1.0)
    bd = b.layer_descs({"l0.mix.q.conv": (16, 2)})
    assert bd[0]["ga_conv"] == 2 and bd[0]["mask_kind"] == MASK_CAUSAL and bd[0]["rot_dims"] == 0 and bd[1]["ga_kv_heads"] == 2
    assert b.layer_descs({})[0]["ga_conv"] == 0


def test_layer_order_of_a_looped_block():
    assert O.layer_order(CFG) == [0, 1, 2, 1, 2]
    assert O.layer_order(dict(CFG, loop={"start": 0, "stop": 1, "times": 3})) == [0, 0, 0, 1, 2]
    assert O.layer_order(dict(CFG, loop=None)) == [0, 1, 2]
    w = O.random_weights(CFG, seed=4)
    logits, layers = O.forward(CFG, w, [3, 4, 5, 6], return_layers=True)
    assert layers.shape == (5, 4, 32) and logits.shape == (4, 50)


def test_oracle_is_causal_and_keeps_its_masks():
    w = O.random_weights(CFG, seed=1)
    a = list(range(3, 23))
    b = a[:12] + [49 - t for t in a[12:]]
    la, lb = O.forward(CFG, w, a), O.forward(CFG, w, b)
    assert np.allclose(la[:12], lb[:12]) and not np.allclose(la[12:], lb[12:])
    assert [j for j in range(11) if O.sees_window(10, j, 4, 0)] == [7, 8, 9, 10]
    assert [j for j in range(11) if O.sees_window(10, j, 4, 2)] == [0, 1, 7, 8, 9, 10]
    assert [j for j in range(4) if O.sees_window(3, j, 2, 3)] == [0, 1, 2, 3]           # kept positions and window overlap
    assert [j for j in range(11) if O.sees_chunk(10, j, 4)] == [8, 9, 10] and [j for j in range(9) if O.sees_chunk(8, j, 4)] == [8]
    assert [j for j in range(4) if O.sees_chunk(3, j, None)] == [0, 1, 2, 3]
    # one window layer forgets what neither its window nor its kept positions hold: token 3 does not reach position 12, token 1 does
    one = dict(CFG, layers=[dict(WIN, mlp=None)], loop=None)
    w1 = O.random_weights(one, seed=2)
    x = O.forward(one, w1, a)
    assert np.allclose(x[12:], O.forward(one, w1, a[:3] + [a[3] + 1] + a[4:])[12:])
    assert not np.allclose(x[12], O.forward(one, w1, [a[0], a[1] + 1] + a[2:])[12])


def test_both_pair_layouts_turn_and_turn_back():
    f, mag = O.rotary_frequencies({"base": 100.0, "dims": 4})
    assert mag == 1.0 and np.allclose(f, [1.0, 0.1])
    x = np.arange(1.0, 7.0)
    y = O.rotate(x, 3, f, 1.0, "interleaved")
    assert np.allclose(y[0], 1 * math.cos(3) - 2 * math.sin(3)) and np.allclose(y[1], 2 * math.cos(3) + 1 * math.sin(3))
    assert np.allclose(y[2], 3 * math.cos(0.3) - 4 * math.sin(0.3)) and np.allclose(y[4:], x[4:])
    z = O.rotate(x, 3, f, 1.0, "half")
    assert np.allclose(z[0], 1 * math.cos(3) - 3 * math.sin(3)) and np.allclose(z[2], 3 * math.cos(3) + 1 * math.sin(3))
    assert np.allclose(z[1], 2 * math.cos(0.3) - 4 * math.sin(0.3)) and np.allclose(z[4:], x[4:])
    for layout in ("interleaved", "half"):
        assert np.allclose(O.rotate(O.rotate(x, 7, f, 1.0, layout), -7, f, 1.0, layout), x)
    # scaled frequencies by hand: dims 6, base 500: dim(t) = 6 ln(32 / (2 pi t)) / (2 ln 500)
    fs, mags = O.rotary_frequencies({"base": 500.0, "dims": 6, "scaling": YARN})
    lo = max(math.floor(6 * math.log(32 / (2 * math.pi * 8.0)) / (2 * math.log(500.0))), 0)
    hi = min(math.ceil(6 * math.log(32 / (2 * math.pi * 1.0)) / (2 * math.log(500.0))), 5)
    for i in range(3):
        plain = 500.0 ** (-2.0 * i / 6)
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        assert math.isclose(fs[i], plain / 4.0 * ramp + plain * (1 - ramp))
    assert math.isclose(mags, 0.1 * math.log(4.0) + 1.0)


def test_decay_and_recurrence_by_hand():
    mix = {"heads": 1, "dim": 2, "vdim": 2, "tau": 2.0}
    p = {"q": np.eye(2), "k": np.eye(2), "v": np.eye(2), "g": np.eye(2), "a1": np.eye(2), "a2": np.zeros((2, 2)), "a2.b": np.array([0.0, math.log(3.0)]),
         "norm": np.ones(2), "o": np.eye(2)}
    h = np.array([[1.0, 2.0], [3.0, -1.0]])
    alpha = O.gla_decay(h, p, mix)
    assert np.allclose(alpha, [[0.5 ** 0.5, 0.75 ** 0.5]] * 2)
    # S_0 = k_0 v_0^T; S_1 = diag(alpha) S_0 + k_1 v_1^T; o_t = S_t^T q_t with q = h / sqrt(2)
    S0 = np.outer(h[0], h[0])
    S1 = alpha[1][:, None] * S0 + np.outer(h[1], h[1])
    o = np.stack([S0.T @ h[0], S1.T @ h[1]]) / math.sqrt(2.0)
    want = O.rms_unit(o, 1e-5) * O.silu(h)
    assert np.allclose(O.gla(h, p, mix, 1e-5), want)


def test_two_maps_and_the_bounded_unit_by_hand():
    p = {"lq1": np.array([0.5, 1.0]), "lk1": np.array([1.0, 0.5]), "lq2": np.array([1.0, 0.0]), "lk2": np.array([-1.0, 3.0])}
    assert math.isclose(O.diff_lambda(p, {"diff": 0.2}), math.exp(1.0) - math.exp(-1.0) + 0.2)
    # one head, one position: both maps see one key, so a1 = a2 = v and o = unit_rms((1 - lambda) v) * (1 - diff)
    mix = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 2, "diff": 0.2, "scale": 1.0}
    pp = dict(p, q=np.ones((4, 2)), k=np.ones((4, 2)), v=np.eye(2), o=np.eye(2))
    h = np.array([[3.0, 4.0]])
    lam = O.diff_lambda(p, mix)
    assert np.allclose(O.diff_attention(h, pp, mix, 0.0), O.rms_unit((1 - lam) * h, 0.0) * 0.8)
    mlp = {"limit": 1.0}
    pm = {"gate": np.eye(3), "up": np.eye(3), "down": np.eye(3)}
    x = np.array([[0.5, 3.0, -2.0]])
    g, u = np.array([0.5, 1.0, -2.0]), np.array([0.5, 1.0, -1.0])      # the gate is bounded above only, the other branch on both sides
    assert np.allclose(O.clamped_glu(x, pm, mlp), g / (1 + np.exp(-1.702 * g)) * (u + 1))


def test_unit_in_the_denominator():
    s, v = np.array([-3.0, -4.0]), np.array([[1.0, 0.0], [0.0, 1.0]])
    e = np.exp(s)
    assert np.allclose(O.softmax_attend(s, v, True), e / (1 + e.sum())) and np.allclose(O.softmax_attend(s, v, False), e / e.sum())
    big = np.array([50.0, 49.0])
    assert np.allclose(O.softmax_attend(big, v, True), np.exp(big - 50) / (np.exp(-50.0) + np.exp(big - 50).sum()))


def test_runner_help_names_its_protocol(repo_root):
    import subprocess
    import sys

    out = subprocess.run([sys.executable, f"{repo_root}/bin/trace_run", "--help"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0 and "--max-tokens" in out.stdout and "done <step>" in out.stdout
