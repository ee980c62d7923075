"""Sofopel on the B200 engine: a layer-list decoder whose layers are PARALLEL blocks.

`config.json`: `architecture: "Sofopel"`, `width`, `vocab`, `norm.eps`, `embedding.scale`, `residual_mult`, `loop` and `layers`.
The token embedding is scaled; a layer is `x += residual_mult * (mixer(u) + ff(u))` with ONE weighted RMS norm `u = rms_w(x)` that
both sublayers read; `loop: {start, stop, times}` runs a block of layers several times in a row with the same tensors, every pass on
a cache / state of its own and with nothing added between the passes. Mixers: `gla` (gated linear attention: a [key, value] state per
head with a decay per key channel, `sigmoid(W_a2 W_a1 h + b)^(1 / tau)`; per-head RMS norm, SiLU gate), `attention` (differential
attention: every head holds two score maps over the same values and gives `unit_rms(a1 - lambda a2) * (1 - diff)`; a short
convolution on q / k / v; rotary pairs of neighbours; visibility limited to the query's chunk of positions) and `attention_2`
(grouped heads; weighted RMS norm of every q and k head; rotary pairs `(m, m + dims / 2)` with long-context frequency scaling; a
sliding window that keeps the sequence's first positions; a softmax with a 1 in its denominator; ONE sigmoid gate per head).
Feed-forward: `W_down (a(g) (u + 1))` with `g = min(W_gate h, limit)`, `u = clamp(W_up h, +-limit)`, `a(g) = g sigmoid(1.702 g)`.
This module only reads the configuration; tensors, engine, generation and replay are the layer-list decoders' common code
(layer_list.py).
"""
from ..._b2 import (BLOCK_PARALLEL_RMS, FF_CLAMP_GLU, GATE_HEAD, GATE_NONE, MASK_CAUSAL, MASK_CHUNK, MASK_WINDOW, MIXER_GLA,
                    MIXER_GQA_ATTN)
from .layer_list import LayerListConfig, LayerListForCausalLM

GLU_SLOPE = 1.702   # a(g) = g sigmoid(1.702 g): the sigmoid approximation of GELU, fixed by the design


def _rotation(rot, what):
    """Engine fields of a `rot` entry (absent: no rotation): rotated dimensions, base and, when present, the long-context scaling."""
    if not rot or not int(rot.get("dims", 0)):
        return dict(rot_dims=0, rot_base=10000.0)
    d = dict(rot_dims=int(rot["dims"]), rot_base=float(rot["base"]))
    sc = rot.get("scaling")
    if sc:
        if float(sc["factor"]) <= 0:
            raise ValueError(f"{what}: rot.scaling.factor must be positive")
        d.update(rot_factor=float(sc["factor"]), rot_original=float(sc["original"]), rot_fast=float(sc["fast"]), rot_slow=float(sc["slow"]))
    return d


def _mask(mix, kind):
    m = mix.get("mask")
    if not m or m.get("size") is None:
        return dict(mask_kind=MASK_CAUSAL, mask_size=0)
    d = dict(mask_kind=kind, mask_size=int(m["size"]))
    if kind == MASK_WINDOW:
        d["mask_keep"] = int(m.get("keep_first", 0) or 0)
    return d


class SofopelConfig(LayerListConfig):
    model_type = "Sofopel"

    def model_desc(self):
        c = self.raw
        d = dict(block=BLOCK_PARALLEL_RMS, residual_mult=float(c.get("residual_mult", 1.0)),
                 embed_scale=float((c.get("embedding") or {}).get("scale", 1.0)))
        loop = c.get("loop")
        if loop:
            d.update(loop_start=int(loop["start"]), loop_stop=int(loop["stop"]), loop_times=int(loop["times"]), loop_plain=1)
        return d

    def layer_descs(self, shapes):
        out = []
        for i, layer in enumerate(self.layers):
            mix, mlp, kind = layer["mixer"], layer.get("mlp"), layer["type"]
            d = dict(weights_of=-1, ff=0)
            if kind == "gla":
                a1 = shapes.get(f"l{i}.mix.a1")
                if a1 is None:
                    raise ValueError(f"layer {i}: the checkpoint has no l{i}.mix.a1 (its rows give the rank of the decay projection)")
                d.update(type=MIXER_GLA, gl_heads=int(mix["heads"]), gl_dim=int(mix["dim"]), gl_vdim=int(mix["vdim"]), gl_rank=int(a1[0]),
                         gl_tau=float(mix["tau"]))
            elif kind in ("attention", "attention_2"):
                d.update(type=MIXER_GQA_ATTN, ga_heads=int(mix["heads"]), ga_kv_heads=int(mix.get("kv_heads", mix["heads"])), ga_dim=int(mix["dim"]),
                         ga_vdim=int(mix["vdim"]), ga_scale=float(mix["scale"]), **_rotation(mix.get("rot"), f"layer {i}"))
                if kind == "attention":     # two maps, a convolution on q / k / v, neighbouring pairs, chunks, plain softmax, no gate
                    taps = mix.get("conv")
                    if taps is None:
                        shape = shapes.get(f"l{i}.mix.q.conv")
                        taps = shape[1] if shape else 0
                    d.update(ga_maps=2, ga_diff=float(mix["diff"]), ga_conv=int(taps), ga_gate=GATE_NONE, **_mask(mix, MASK_CHUNK))
                else:                       # q / k norm, half-layout pairs, window with kept first positions, a unit in the denominator, head gates
                    d.update(ga_qk_norm=1, ga_rot_half=1, ga_sink=1, ga_sink_value=0.0, ga_gate=GATE_HEAD, **_mask(mix, MASK_WINDOW))
            else:
                raise NotImplementedError(f"layer {i}: mixer type {kind!r}")
            if mlp:
                if mlp.get("kind", "dense") != "dense":
                    raise NotImplementedError(f"layer {i}: feed-forward kind {mlp.get('kind')!r}")
                d.update(ff_kind=FF_CLAMP_GLU, ff=int(mlp["ff"]), ff_limit=float(mlp.get("limit", 0.0) or 0.0), ff_act_slope=GLU_SLOPE)
            out.append(d)
        return out


class SofopelForCausalLM(LayerListForCausalLM):
    """Holds the checkpoint tensors (CPU) and builds the device engine on first use.

    dtype: torch.bfloat16 = bf16 matrix products with fp32 accumulation on bf16 weights (norms, convolutions, rotations, scores and
    softmax, decays and the recurrent state, the caches and the residual stream in fp32); torch.float32 = everything in true fp32."""
    config_class = SofopelConfig
