"""Plain restatement of the Sofopel decoder, one function per mechanism, in float64, position by position, without any cache.

Nothing here is shared with the engine: the tests compare the engine's kernels, caches and schedules with these loops.
A model is (cfg, w): `cfg` the dictionary of config.json, `w` a dictionary name -> numpy array with the checkpoint's names
(`embed`, `l<i>.norm1`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head`).

The design: x = embed[token] * embedding.scale; every layer is PARALLEL, x += m * (mixer(u) + ff(u)) with ONE weighted RMS norm
u = rms_w(x) read by both sublayers (a layer without feed-forward adds the mixer alone); a block of layers may run several times in
a row with the same tensors and nothing else between the passes; weighted RMS norm and head at the end. Mixers: `gla` (gated linear
attention with a low-rank per-channel decay), `attention` (differential attention: two softmax maps over the same values, the
second subtracted with a learned factor; a short convolution on q / k / v; interleaved rotary pairs; chunked visibility) and
`attention_2` (grouped heads, weighted q / k norm, rotate-half rotary pairs with long-context scaling, a sliding window that keeps
the sequence's first tokens, a softmax with a unit in its denominator, a sigmoid gate per head).

Notation: h is a sublayer's input [T, width]; every Linear weight is [out, in] and applied as h @ W.T; t, i, j are positions
of one sequence, counted from 0.
"""
import math

import numpy as np

F = np.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ------------------------------------------------------------------------------------------------- convolution over time
def causal_conv(u, taps_w):
    """y_t = sum_j w[:, j] * u_(t - taps + 1 + j) per channel, zeros in front of the sequence. u [T, C], taps_w [C, taps]."""
    T, C = u.shape
    taps = taps_w.shape[1]
    y = np.zeros((T, C), F)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += taps_w[:, j] * u[s]
    return y


# ------------------------------------------------------------------------------------------------- rotations
def rotary_frequencies(rot):
    """Angle per position of every rotated pair, and the factor on cos and sin (1 without long-context scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], F)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2, dtype=F) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, pos, freq, mag, layout):
    """Turns len(freq) pairs of the leading entries of x's last axis by pos * freq_i; the rest passes. layout "interleaved": pair i is
    (2i, 2i+1); "half": pair i is (i, i + len(freq))."""
    n = len(freq)
    out = np.array(x, F, copy=True)
    if n == 0:
        return out
    a = pos * freq
    c, s = np.cos(a) * mag, np.sin(a) * mag
    if layout == "interleaved":
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2] = u * c - v * s
        out[..., 1:2 * n:2] = v * c + u * s
    else:
        u, v = x[..., 0:n], x[..., n:2 * n]
        out[..., 0:n] = u * c - v * s
        out[..., n:2 * n] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------- visibility
def sees_chunk(i, j, size):
    """Chunks of `size` positions counted from 0 (size None: plain causal)."""
    return j <= i and (size is None or i // size == j // size)


def sees_window(i, j, size, keep_first):
    """The last `size` positions and, whatever their distance, the first `keep_first` of the sequence (size None: plain causal)."""
    return j <= i and (size is None or i - j < size or j < keep_first)


def softmax_attend(scores, values, extra_one):
    """Weights exp(s_j) / (sum exp(s) [+ 1]) over the given keys, applied to their values."""
    m = max(scores.max(), 0.0) if extra_one else scores.max()
    e = np.exp(scores - m)
    den = e.sum() + (math.exp(-m) if extra_one else 0.0)
    return (e / den) @ values


# ------------------------------------------------------------------------------------------------- mixers
def gla_decay(h, p, mix):
    """alpha [T, heads * dim] = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau)."""
    z = (h @ p["a1"].T) @ p["a2"].T + p["a2.b"]
    return np.exp(-np.logaddexp(0.0, -z) / float(mix["tau"]))


def gla(h, p, mix, eps):
    H, dk, dv = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
    T = h.shape[0]
    q = (h @ p["q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ p["k"].T).reshape(T, H, dk)
    v = (h @ p["v"].T).reshape(T, H, dv)
    alpha = gla_decay(h, p, mix).reshape(T, H, dk)
    gate = silu(h @ p["g"].T)
    out = np.zeros((T, H, dv), F)
    S = np.zeros((H, dk, dv), F)
    for t in range(T):
        for a in range(H):
            S[a] = alpha[t, a][:, None] * S[a] + np.outer(k[t, a], v[t, a])
            out[t, a] = rms_norm(S[a].T @ q[t, a], p["norm"], eps)
    return (out.reshape(T, H * dv) * gate) @ p["o"].T


def diff_lambda(p, mix):
    return math.exp(float(p["lq1"] @ p["lk1"])) - math.exp(float(p["lq2"] @ p["lk2"])) + float(mix["diff"])


def diff_attention(h, p, mix, eps):
    H, G, dk, dv = int(mix["heads"]), int(mix["kv_heads"]), int(mix["dim"]), int(mix["vdim"])
    T = h.shape[0]
    q, k, v = h @ p["q"].T, h @ p["k"].T, h @ p["v"].T
    if "q.conv" in p:
        q, k, v = causal_conv(q, p["q.conv"]), causal_conv(k, p["k.conv"]), causal_conv(v, p["v.conv"])
    q, k, v = q.reshape(T, H, 2, dk), k.reshape(T, G, 2, dk), v.reshape(T, G, dv)
    rot = mix.get("rot")
    if rot:
        f, mag = rotary_frequencies(rot)
        q = np.stack([rotate(q[t], t, f, mag, "interleaved") for t in range(T)])
        k = np.stack([rotate(k[t], t, f, mag, "interleaved") for t in range(T)])
    size = (mix.get("mask") or {}).get("size")
    lam, d0, scale = diff_lambda(p, mix), float(mix["diff"]), float(mix["scale"])
    out = np.zeros((T, H, dv), F)
    for i in range(T):
        js = [j for j in range(i + 1) if sees_chunk(i, j, size)]
        for a in range(H):
            g = a // (H // G)
            maps = [softmax_attend(k[js, g, m] @ q[i, a, m] * scale, v[js, g], False) for m in range(2)]
            out[i, a] = rms_unit(maps[0] - lam * maps[1], eps) * (1.0 - d0)
    return out.reshape(T, H * dv) @ p["o"].T


def window_attention(h, p, mix, eps, extra_one=True):
    H, G, dk, dv = int(mix["heads"]), int(mix["kv_heads"]), int(mix["dim"]), int(mix["vdim"])
    T = h.shape[0]
    q = rms_norm((h @ p["q"].T).reshape(T, H, dk), p["q.norm"], eps)
    k = rms_norm((h @ p["k"].T).reshape(T, G, dk), p["k.norm"], eps)
    v = (h @ p["v"].T).reshape(T, G, dv)
    rot = mix.get("rot")
    if rot:
        f, mag = rotary_frequencies(rot)
        q = np.stack([rotate(q[t], t, f, mag, "half") for t in range(T)])
        k = np.stack([rotate(k[t], t, f, mag, "half") for t in range(T)])
    mask = mix.get("mask") or {}
    size, keep, scale = mask.get("size"), int(mask.get("keep_first", 0)), float(mix["scale"])
    gate = sigmoid(h @ p["g"].T)
    out = np.zeros((T, H, dv), F)
    for i in range(T):
        js = [j for j in range(i + 1) if sees_window(i, j, size, keep)]
        for a in range(H):
            g = a // (H // G)
            out[i, a] = softmax_attend(k[js, g] @ q[i, a] * scale, v[js, g], extra_one) * gate[i, a]
    return out.reshape(T, H * dv) @ p["o"].T


MIXERS = {"gla": gla, "attention": diff_attention, "attention_2": window_attention}


# ------------------------------------------------------------------------------------------------- feed-forward
def clamped_glu(h, p, mlp):
    limit = float(mlp["limit"])
    g = np.minimum(h @ p["gate"].T, limit)
    u = np.clip(h @ p["up"].T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ p["down"].T


# ------------------------------------------------------------------------------------------------- the model
def layer_params(w, i, part):
    pre = f"l{i}.{part}."
    return {k[len(pre):]: np.asarray(v, F) for k, v in w.items() if k.startswith(pre)}


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer run)."""
    eps, m = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = np.asarray(w["embed"], F)[np.asarray(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    layers = []
    for i in layer_order(cfg):
        layer = cfg["layers"][i]
        u = rms_norm(x, np.asarray(w[f"l{i}.norm1"], F), eps)
        y = MIXERS[layer["type"]](u, layer_params(w, i, "mix"), layer["mixer"], eps)
        if layer.get("mlp"):
            if layer["mlp"].get("kind", "dense") != "dense":
                raise NotImplementedError(layer["mlp"]["kind"])
            y = y + clamped_glu(u, layer_params(w, i, "mlp"), layer["mlp"])
        x = x + m * y
        layers.append(x.copy())
    logits = rms_norm(x, np.asarray(w["final.norm"], F), eps) @ np.asarray(w["head"], F).T
    return (logits, np.stack(layers)) if return_layers else logits


# ------------------------------------------------------------------------------------------------- random models
def bf16_round(a):
    """Nearest bfloat16 (ties to even) of float32 values, returned as float32."""
    b = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    b = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) << 16
    return b.astype(np.uint32).view(np.float32)


def tensor_shapes(cfg, ranks=None):
    """name -> shape of every tensor of a model of this configuration. ranks: decay rank of a gla layer by index (default 8)."""
    W, V = int(cfg["width"]), int(cfg["vocab"])
    s = {"embed": (V, W), "head": (V, W), "final.norm": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        mix, t, pre = layer["mixer"], layer["type"], f"l{i}."
        s[pre + "norm1"] = (W,)
        H, dk, dv = int(mix["heads"]), int(mix["dim"]), int(mix["vdim"])
        if t == "gla":
            r = (ranks or {}).get(i, 8)
            s.update({pre + "mix.q": (H * dk, W), pre + "mix.k": (H * dk, W), pre + "mix.v": (H * dv, W), pre + "mix.g": (H * dv, W),
                      pre + "mix.o": (W, H * dv), pre + "mix.norm": (dv,), pre + "mix.a1": (r, W), pre + "mix.a2": (H * dk, r),
                      pre + "mix.a2.b": (H * dk,)})
        elif t == "attention":
            G = int(mix["kv_heads"])
            s.update({pre + "mix.q": (2 * H * dk, W), pre + "mix.k": (2 * G * dk, W), pre + "mix.v": (G * dv, W), pre + "mix.o": (W, H * dv)})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                s[pre + "mix." + n] = (dk,)
            if mix.get("conv"):
                for n, c in (("q", 2 * H * dk), ("k", 2 * G * dk), ("v", G * dv)):
                    s[pre + f"mix.{n}.conv"] = (c, int(mix["conv"]))
        elif t == "attention_2":
            G = int(mix["kv_heads"])
            s.update({pre + "mix.q": (H * dk, W), pre + "mix.k": (G * dk, W), pre + "mix.v": (G * dv, W), pre + "mix.g": (H, W),
                      pre + "mix.o": (W, H * dv), pre + "mix.q.norm": (dk,), pre + "mix.k.norm": (dk,)})
        else:
            raise NotImplementedError(t)
        if layer.get("mlp"):
            ff = int(layer["mlp"]["ff"])
            s.update({pre + "mlp.gate": (ff, W), pre + "mlp.up": (ff, W), pre + "mlp.down": (W, ff)})
    return s


def random_weights(cfg, seed=0, gain=1.0, ranks=None):
    """Random bfloat16-representable tensors: matrices ~ N(0, gain^2 / fan_in), norm weights near 1, decay biases that spread the decays
    between fast and slow channels."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg, ranks).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm") or name == "final.norm":
            a = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            a = 0.3 * rng.standard_normal(shape)
        elif leaf == "b":
            a = rng.uniform(-1.0, 5.0, shape)
        elif leaf == "conv":
            a = rng.standard_normal(shape) * 0.5
        elif name == "embed":
            a = rng.standard_normal(shape)
        else:
            a = rng.standard_normal(shape) * gain / math.sqrt(shape[-1])
        w[name] = bf16_round(a.astype(np.float32))
    return w
