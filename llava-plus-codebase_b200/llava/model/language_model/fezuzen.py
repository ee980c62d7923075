"""Fezuzen on the B200 engine: a layer-list decoder whose sublayers are normed on both sides and read their input through a short
convolution over time.

`config.json`: `architecture: "Fezuzen"`, `width`, `vocab`, `norm.eps`, `canon.taps`, `logit_scale` and `layers`. A layer is
`x += rms_w1b(mixer(u + conv1(u)))`, `u = rms_w1(x)`, then the same around the feed-forward with `norm2 / canon2 / norm2b`; the
convolutions are causal and depthwise, and their last `taps - 1` inputs are part of a sequence's state. Mixers:
`latent_attention` (queries through a latent of their own; one cached row per token = a normed low-rank latent, from which
every head's keys and values are read, plus ONE rotary key part shared by the heads; YaRN-scaled frequencies; sliding window;
`kv_from: j` = the layer has no down-projection and reads layer j's cached rows) and `attention` (grouped key/value heads, a
short convolution on q / k / v, rotary q and k, values rotated by their own position and the output turned back by the
query's, visibility limited to the query's chunk of positions, a softmax with one extra 1 in the denominator, a per-channel
sigmoid output gate). Feed-forward: a mixture of `relu(.)^2` experts with softmax scores, group-limited top-k choice and the raw
scores as weights, plus a shared expert. This module only reads the configuration; tensors, engine, generation and replay are
the layer-list decoders' common code (layer_list.py).
"""
from ..._b2 import (BLOCK_SANDWICH_RMS, FF_MOE, MASK_CAUSAL, MASK_CHUNK, MASK_WINDOW, MIXER_GQA_ATTN, MIXER_LATENT_ATTN, MOE_ACT_RELU_SQ,
                    MOE_GROUP_MAX, MOE_SCORE_SOFTMAX)
from .layer_list import LayerListConfig, LayerListForCausalLM


def _rotation(rot, what):
    """Engine fields of a `rot` entry: rotated dimensions, base and, when present, the long-context scaling."""
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
    return dict(mask_kind=kind, mask_size=int(m["size"]))


class FezuzenConfig(LayerListConfig):
    model_type = "Fezuzen"

    def model_desc(self):
        c = self.raw
        return dict(block=BLOCK_SANDWICH_RMS, logit_scale=float(c.get("logit_scale", 1.0)),
                    input_conv_taps=int((c.get("canon") or {}).get("taps", 0)))

    @staticmethod
    def _conv_taps(i, mix, shapes):
        """Taps of the short convolution on q / k / v: `mixer.conv`, or what the checkpoint's tensor says when the key is absent."""
        if mix.get("conv") is not None:
            return int(mix["conv"])
        shape = shapes.get(f"l{i}.mix.q.conv")
        return int(shape[1]) if shape else 0

    def layer_descs(self, shapes):
        out = []
        for i, layer in enumerate(self.layers):
            mix, mlp = layer["mixer"], layer.get("mlp")
            d = dict(weights_of=-1, ff=0)
            if layer["type"] == "latent_attention":
                src = mix.get("kv_from")
                d.update(type=MIXER_LATENT_ATTN, la_heads=int(mix["heads"]), la_dim=int(mix["dim"]), la_vdim=int(mix["vdim"]),
                         la_rank=int(mix["kv_rank"]), la_scale=float(mix["scale"]), la_q_rank=int(mix["q_rank"]),
                         la_rot_dim=int(mix["rot_dim"]), la_no_sink=1, la_no_gate=1, la_kv_from=0 if src is None else int(src) + 1,
                         **_rotation(mix["rot"], f"layer {i}"), **_mask(mix, MASK_WINDOW))
            elif layer["type"] == "attention":
                d.update(type=MIXER_GQA_ATTN, ga_heads=int(mix["heads"]), ga_kv_heads=int(mix["kv_heads"]), ga_dim=int(mix["dim"]),
                         ga_vdim=int(mix["vdim"]), ga_conv=self._conv_taps(i, mix, shapes), ga_rot_values=1, ga_sink=1, ga_sink_value=0.0,
                         ga_scale=float(mix["scale"]), **_rotation(mix["rot"], f"layer {i}"), **_mask(mix, MASK_CHUNK))
            else:
                raise NotImplementedError(f"layer {i}: mixer type {layer['type']!r}")
            if mlp:
                kind = mlp.get("kind", "moe")
                if kind != "moe":
                    raise NotImplementedError(f"layer {i}: feed-forward kind {kind!r}")
                r = mlp["router"]
                groups = r.get("groups") or {"count": 1, "keep": 1}
                d.update(ff_kind=FF_MOE, ff=int(mlp["expert"]["ff"]), moe_experts=int(r["experts"]), moe_top=int(r["top"]),
                         moe_groups=int(groups["count"]), moe_keep=int(groups["keep"]), moe_scale=1.0,
                         moe_shared_ff=int(mlp["shared"]["ff"]) if mlp.get("shared") else 0,
                         moe_score=MOE_SCORE_SOFTMAX, moe_group_score=MOE_GROUP_MAX, moe_raw_weights=1, moe_act=MOE_ACT_RELU_SQ)
            out.append(d)
        return out


class FezuzenForCausalLM(LayerListForCausalLM):
    """Holds the checkpoint tensors (CPU) and builds the device engine on first use.

    dtype: torch.bfloat16 = bf16 matrix products with fp32 accumulation on bf16 weights (norms, convolutions, rotations, router,
    scores and softmax, the caches and the residual stream in fp32); torch.float32 = everything in true fp32."""
    config_class = FezuzenConfig
