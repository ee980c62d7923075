"""Plain restatement of the Fezuzen decoder, one function per mechanism, in float64, position by position, without any cache.

Nothing here is shared with the engine: the tests compare the engine's kernels, caches and schedules with these loops.
A model is (cfg, w): `cfg` the dictionary of config.json, `w` a dictionary name -> numpy array with the checkpoint's names
(`embed`, `l<i>.norm1`, `l<i>.norm1b`, `l<i>.canon1`, `l<i>.mix.*`, `l<i>.norm2`, `l<i>.norm2b`, `l<i>.canon2`, `l<i>.mlp.*`,
`final.norm`, `head`).

Notation: h is a sublayer's input [T, width]; every Linear weight is [out, in] and applied as h @ W.T; t, i, j are positions
of one sequence, counted from 0.
"""
import math

import numpy as np

F = np.float64


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * weight


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# ------------------------------------------------------------------------------------------------- convolutions over time
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


def input_conv(h, taps_w):
    """What a sublayer reads: its input plus the causal convolution of its input (taps_w None: the input itself)."""
    return h if taps_w is None else h + causal_conv(h, taps_w)


# ------------------------------------------------------------------------------------------------- rotations
def rotary_frequencies(rot):
    """Angle per position of every pair of the rotated part, and the factor on cos and sin (1 without long-context scaling)."""
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


def rotate_pairs(x, pos, freq, mag=1.0, n=None):
    """Turns the pairs (2i, 2i+1), i < len(freq), of the first n (= 2 len(freq)) entries of x's last axis by pos * freq_i; the
    rest passes. x [..., D]; pos a number."""
    n = 2 * len(freq) if n is None else n
    out = np.array(x, F, copy=True)
    a = pos * freq
    c, s = np.cos(a) * mag, np.sin(a) * mag
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * c - v * s
    out[..., 1:n:2] = v * c + u * s
    return out


# ------------------------------------------------------------------------------------------------- mixers
def visible(i, j, kind, size):
    """Whether position i sees position j <= i: a sliding window of `size` positions, or chunks of `size` counted from 0."""
    if j > i:
        return False
    if size is None:
        return True
    if kind == "window":
        return i - j < size
    return i // size == j // size


def visible_keys(i, kind, size):
    """Positions that position i sees (under either mask nothing further back than `size` positions can be visible)."""
    first = 0 if size is None else max(0, i - size)
    return [j for j in range(first, i + 1) if visible(i, j, kind, size)]


def mask_size(mix):
    m = mix.get("mask")
    return int(m["size"]) if m and m.get("size") is not None else None


def latent_kv(h, p, mix, eps):
    """What a latent-attention layer leaves per position: the normed latent c [T, kv_rank] and the rotated shared key part
    [T, rot_dim]."""
    rank, rd = int(mix["kv_rank"]), int(mix["rot_dim"])
    freq, mag = rotary_frequencies(mix["rot"])
    d = h @ p["dkv"].T
    c = rms_norm(d[:, :rank], p["dkv.norm"], eps)
    kr = np.stack([rotate_pairs(d[t, rank:rank + rd], t, freq, mag) for t in range(h.shape[0])])
    return c, kr


def latent_attention(h, p, mix, eps, kv=None):
    """Attention whose per-head keys and values are read off a low-rank latent, plus one rotated key part shared by all heads;
    queries through a latent of their own; sliding window; ordinary softmax. kv: (c, kr) of the layer it borrows them from."""
    T = h.shape[0]
    H, dk, rd, dv = int(mix["heads"]), int(mix["dim"]), int(mix["rot_dim"]), int(mix["vdim"])
    scale, size = float(mix["scale"]), mask_size(mix)
    freq, mag = rotary_frequencies(mix["rot"])
    cq = rms_norm(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).reshape(T, H, dk + rd)
    c, kr = kv if kv is not None else latent_kv(h, p, mix, eps)
    k = (c @ p["uk"].T).reshape(T, H, dk)
    v = (c @ p["uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv), F)
    for i in range(T):
        js = visible_keys(i, "window", size)
        for hd in range(H):
            qn, qr = q[i, hd, :dk], rotate_pairs(q[i, hd, dk:], i, freq, mag)
            s = (k[js, hd] @ qn + kr[js] @ qr) * scale
            e = np.exp(s - s.max())
            out[i, hd] = (e / e.sum()) @ v[js, hd]
    return out.reshape(T, H * dv) @ p["o"].T


def grouped_attention(h, p, mix, extra_one=True):
    """Attention with grouped key/value heads: short convolutions on q, k, v; rotary q, k; values rotated by their own position
    and the head's output turned back by the query's; chunked mask; a softmax whose denominator holds one extra 1 (extra_one False
    leaves it out: what a test compares with to see that the term matters); sigmoid output gate."""
    T = h.shape[0]
    H, G, dk, dv = int(mix["heads"]), int(mix["kv_heads"]), int(mix["dim"]), int(mix["vdim"])
    scale, size = float(mix["scale"]), mask_size(mix)
    freq, mag = rotary_frequencies(mix["rot"])
    vfreq = np.array([float(mix["rot"]["base"]) ** (-2.0 * m / dv) for m in range(dv // 2)], F)
    conv = (lambda u, n: causal_conv(u, p[n + ".conv"])) if int(mix.get("conv", 0) or 0) >= 1 else (lambda u, n: u)
    q = conv(h @ p["q"].T, "q").reshape(T, H, dk)
    k = conv(h @ p["k"].T, "k").reshape(T, G, dk)
    v = conv(h @ p["v"].T, "v").reshape(T, G, dv)
    gate = sigmoid(h @ p["g"].T).reshape(T, H, dv)
    q = np.stack([rotate_pairs(q[t], t, freq, mag) for t in range(T)])
    k = np.stack([rotate_pairs(k[t], t, freq, mag) for t in range(T)])
    v = np.stack([rotate_pairs(v[t], t, vfreq) for t in range(T)])
    out = np.zeros((T, H, dv), F)
    for i in range(T):
        js = visible_keys(i, "chunk", size)
        for hd in range(H):
            g = hd // (H // G)
            s = (k[js, g] @ q[i, hd]) * scale
            m = max(s.max(), 0.0)
            e = np.exp(s - m)
            o = (e / ((math.exp(-m) if extra_one else 0.0) + e.sum())) @ v[js, g]
            out[i, hd] = rotate_pairs(o, -i, vfreq) * gate[i, hd]
    return out.reshape(T, H * dv) @ p["o"].T


# ------------------------------------------------------------------------------------------------- feed-forward
def expert(h, up, down):
    """W_down relu(W_up h)^2."""
    a = np.maximum(h @ up.T, 0.0)
    return (a * a) @ down.T


def route(h, router_w, r):
    """Chosen experts and their weights for every row: softmax scores; experts in equal groups of neighbours, a group scored by
    its best expert, only the best `keep` groups compete; the `top` largest scores win and are the weights as they are."""
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {"count": 1, "keep": 1}
    G, keep = int(groups["count"]), int(groups["keep"])
    z = h @ router_w.T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z)
    s = s / s.sum(-1, keepdims=True)
    idx, wgt = [], []
    for t in range(h.shape[0]):
        gs = s[t].reshape(G, E // G).max(-1)
        alive = sorted(range(G), key=lambda g: (-gs[g], g))[:keep]
        cand = [e for e in range(E) if e // (E // G) in alive]
        chosen = sorted(cand, key=lambda e: (-s[t, e], e))[:top]
        idx.append(chosen)
        wgt.append([s[t, e] for e in chosen])
    return idx, wgt


def moe_ff(h, p, mlp):
    idx, wgt = route(h, p["router"], mlp["router"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(idx[t], wgt[t]):
            out[t] += g * expert(h[t:t + 1], p[f"e{e}.up"], p[f"e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + expert(h, p["shared.up"], p["shared.down"])
    return out


# ------------------------------------------------------------------------------------------------- the model
def layer_params(w, i, part):
    pre = f"l{i}.{part}."
    return {k[len(pre):]: np.asarray(v, F) for k, v in w.items() if k.startswith(pre)}


def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence (and the residual stream after every layer)."""
    eps = float(cfg["norm"]["eps"])
    x = np.asarray(w["embed"], F)[list(tokens)]
    kept, per_layer = {}, []
    for i, layer in enumerate(cfg["layers"]):
        mix, mlp = layer["mixer"], layer.get("mlp")
        g = lambda n: np.asarray(w[f"l{i}.{n}"], F) if f"l{i}.{n}" in w else None  # noqa: E731
        h = input_conv(rms_norm(x, g("norm1"), eps), g("canon1"))
        p = layer_params(w, i, "mix")
        if layer["type"] == "latent_attention":
            src = mix.get("kv_from")
            if src is None:
                kept[i] = latent_kv(h, p, mix, eps)
                y = latent_attention(h, p, mix, eps)
            else:
                y = latent_attention(h, p, mix, eps, kv=kept[int(src)])
        elif layer["type"] == "attention":
            y = grouped_attention(h, p, mix)
        else:
            raise NotImplementedError(layer["type"])
        x = x + rms_norm(y, g("norm1b"), eps)
        if mlp:
            h = input_conv(rms_norm(x, g("norm2"), eps), g("canon2"))
            x = x + rms_norm(moe_ff(h, layer_params(w, i, "mlp"), mlp), g("norm2b"), eps)
        per_layer.append(x.copy())
    logits = rms_norm(x, np.asarray(w["final.norm"], F), eps) @ np.asarray(w["head"], F).T * float(cfg.get("logit_scale", 1.0))
    return (logits, np.stack(per_layer)) if return_layers else logits


def bf16_round(a):
    """Round float32 values to the nearest bfloat16 (ties to even), returned as float32."""
    u = np.asarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def tensor_shapes(cfg):
    """name -> shape of every tensor a checkpoint of this configuration holds."""
    width, vocab, ct = int(cfg["width"]), int(cfg["vocab"]), int((cfg.get("canon") or {}).get("taps", 0))
    out = {"embed": (vocab, width), "head": (vocab, width), "final.norm": (width,)}
    for i, layer in enumerate(cfg["layers"]):
        mix, mlp = layer["mixer"], layer.get("mlp")
        a = f"l{i}."
        out[a + "norm1"] = out[a + "norm1b"] = (width,)
        if ct >= 1:
            out[a + "canon1"] = (width, ct)
        if layer["type"] == "latent_attention":
            H, dk, rd, dv, rank, qr = (int(mix[k]) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank"))
            out[a + "mix.dq"], out[a + "mix.dq.norm"], out[a + "mix.uq"] = (qr, width), (qr,), (H * (dk + rd), qr)
            if mix.get("kv_from") is None:
                out[a + "mix.dkv"], out[a + "mix.dkv.norm"] = (rank + rd, width), (rank,)
            out[a + "mix.uk"], out[a + "mix.uv"], out[a + "mix.o"] = (H * dk, rank), (H * dv, rank), (width, H * dv)
        else:
            H, G, dk, dv = (int(mix[k]) for k in ("heads", "kv_heads", "dim", "vdim"))
            taps = int(mix.get("conv", 0) or 0)
            for n, rows in (("q", H * dk), ("k", G * dk), ("v", G * dv)):
                out[a + "mix." + n] = (rows, width)
                if taps >= 1:
                    out[a + "mix." + n + ".conv"] = (rows, taps)
            out[a + "mix.g"], out[a + "mix.o"] = (H * dv, width), (width, H * dv)
        if mlp:
            out[a + "norm2"] = out[a + "norm2b"] = (width,)
            if ct >= 1:
                out[a + "canon2"] = (width, ct)
            ff = int(mlp["expert"]["ff"])
            out[a + "mlp.router"] = (int(mlp["router"]["experts"]), width)
            for e in range(int(mlp["router"]["experts"])):
                out[a + f"mlp.e{e}.up"], out[a + f"mlp.e{e}.down"] = (ff, width), (width, ff)
            if mlp.get("shared"):
                sf = int(mlp["shared"]["ff"])
                out[a + "mlp.shared.up"], out[a + "mlp.shared.down"] = (sf, width), (width, sf)
    return out


def random_weights(cfg, seed=0, gain=1.0):
    """Random tensors (values exactly representable in bfloat16) for any configuration: Linear weights ~ N(0, gain^2 / in), norm
    weights near 1, convolution taps ~ N(0, 0.3^2)."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if len(shape) == 1:
            t = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf in ("canon1", "canon2", "conv"):
            t = 0.3 * rng.standard_normal(shape)
        elif leaf == "embed":
            t = rng.standard_normal(shape)
        elif leaf == "router":
            t = 2.0 * rng.standard_normal(shape) / math.sqrt(shape[1])
        else:
            t = gain * rng.standard_normal(shape) / math.sqrt(shape[1])
        w[name] = bf16_round(t.astype(np.float32))
    return w
