"""Plain, slow implementation of the Vokelix decoder in float64 numpy.

The oracle of the Vokelix tests: whole sequences, no cache, no chunks, one function per
mechanism, and no code shared with the `inferllm_b200` package (it reads the raw
`config.json` dictionary and a dictionary of numpy arrays keyed by tensor name).

Notation: T tokens, width D; a linear map is `y = x @ W.T` with W stored [out, in].
Every recurrence is written as the literal token-by-token loop.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


# --------------------------------------------------------------------------- small pieces


def linear(x, w, b=None):
    y = np.asarray(x, F64) @ np.asarray(w, F64).T
    return y if b is None else y + np.asarray(b, F64)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, F64)
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """RMS norm whose stored weight is the offset from one."""
    return rms(x, eps) * (1.0 + np.asarray(w, F64))


def norm_plain(x, w, eps):
    return rms(x, eps) * np.asarray(w, F64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F64)))


def silu(z):
    z = np.asarray(z, F64)
    return z * sigmoid(z)


# --------------------------------------------------------------------------- rotations


def base_frequencies(base, dims):
    i = np.arange(dims // 2, dtype=F64)
    return np.power(F64(base), -2.0 * i / dims)


def yarn_frequencies(base, dims, scaling):
    """Frequencies blended between the plain and the stretched ones by a linear ramp over the pair
    index, and the factor that cos and sin are multiplied with."""
    f = base_frequencies(base, dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    i = np.arange(dims // 2, dtype=F64)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, mag, dims, layout):
    """x [T, heads, d]; the first `dims` channels of each head are rotated.  layout "pairs": channel
    2i goes with 2i+1; "half": channel i goes with i + dims/2."""
    x = np.asarray(x, F64)
    ang = np.asarray(positions, F64)[:, None] * freqs[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    out = x.copy()
    if layout == "pairs":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        h = dims // 2
        u, v = x[..., :h], x[..., h:dims]
        out[..., :h] = u * c - v * s
        out[..., h:dims] = v * c + u * s
    return out


# --------------------------------------------------------------------------- mixers


def attention_keys_values(h, w, pre, m, eps, positions):
    """Keys (normed over the whole projection, rotated) and values of an attention layer:
    [T, G, dim], [T, G, vdim]."""
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k = norm_plain(linear(h, w[pre + "k"], w[pre + "k.b"]), w[pre + "k.norm"], eps).reshape(T, G, d)
    v = linear(h, w[pre + "v"], w[pre + "v.b"]).reshape(T, G, dv)
    rot = m["rot"]
    f, mag = yarn_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
    return rotate(k, positions, f, mag, rot["dims"], "pairs"), v


def sink_softmax_attention(q, k, v, scale, sink):
    """q [T, H, d], k [T, G, d], v [T, G, dv], causal; the softmax denominator holds one more term
    exp(sink[h]) that has no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]), F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd, :] @ k[:, g, :].T) * scale
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
        top = np.maximum(s.max(-1), sink[hd])
        e = np.exp(s - top[:, None])
        den = e.sum(-1) + np.exp(sink[hd] - top)
        out[:, hd, :] = (e / den[:, None]) @ v[:, g, :]
    return out


def attention_mixer(h, w, pre, m, eps, positions, shared_kv=None):
    H, d = m["heads"], m["dim"]
    T = h.shape[0]
    q = norm_plain(linear(h, w[pre + "q"], w[pre + "q.b"]), w[pre + "q.norm"], eps).reshape(T, H, d)
    rot = m["rot"]
    f, mag = yarn_frequencies(rot["base"], rot["dims"], rot.get("scaling"))
    q = rotate(q, positions, f, mag, rot["dims"], "pairs")
    k, v = shared_kv if shared_kv is not None else attention_keys_values(h, w, pre, m, eps, positions)
    o = sink_softmax_attention(q, k, v, m["scale"], np.asarray(w[pre + "sink"], F64))
    o = o * sigmoid(linear(h, w[pre + "g"]))[:, :, None]
    return linear(o.reshape(T, -1), w[pre + "o"]), (k, v)


def decayed_state_scan(q, k, v, decay):
    """S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t; q, k [T, H, d], v [T, H, dv]."""
    T, H, d = q.shape
    o = np.zeros((T, H, v.shape[2]), F64)
    S = np.zeros((H, d, v.shape[2]), F64)
    dec = np.asarray(decay, F64)[:, None, None]
    for t in range(T):
        S = dec * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    return o


def lightning_mixer(h, w, pre, m, eps):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(linear(h, w[pre + "q"])).reshape(T, H, d)
    k = silu(linear(h, w[pre + "k"])).reshape(T, H, d)
    v = silu(linear(h, w[pre + "v"])).reshape(T, H, dv)
    o = decayed_state_scan(q, k, v, m["decay"]).reshape(T, H * dv)
    o = norm_plain(o, w[pre + "norm"], eps) * sigmoid(linear(h, w[pre + "g"]))
    return linear(o, w[pre + "o"])


def retention_mixer(h, w, pre, m, eps, positions):
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    rot = m["rot"]
    f = base_frequencies(rot["base"], rot["dims"])
    q = rotate(linear(h, w[pre + "q"]).reshape(T, H, d), positions, f, 1.0, rot["dims"], "half")
    k = rotate(linear(h, w[pre + "k"]).reshape(T, H, d), positions, f, 1.0, rot["dims"], "half") * d ** -0.5
    v = linear(h, w[pre + "v"]).reshape(T, H, dv)
    o = rms(decayed_state_scan(q, k, v, m["decay"]), eps).reshape(T, H * dv)
    return linear(o * silu(linear(h, w[pre + "g"])), w[pre + "o"])


def gated_feed_forward(h, w, pre):
    return linear(silu(linear(h, w[pre + "gate"])) * linear(h, w[pre + "up"]), w[pre + "down"])


# --------------------------------------------------------------------------- the model


def forward(cfg, w, ids, return_layers=False):
    """Logits [T, vocab] of one whole sequence (positions 0..T-1)."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    ids = np.asarray(ids, np.int64)
    pos = np.arange(len(ids))
    x = np.asarray(w["embed"], F64)[ids]
    kept, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        m, pre = layer["mixer"], f"l{i}.mix."
        if layer["type"] == "attention":
            src = m.get("kv_from")
            y, kv = attention_mixer(x, w, pre, m, eps, pos, kept[src] if src is not None else None)
            kept[i] = kv
        elif layer["type"] == "lightning":
            y = lightning_mixer(x, w, pre, m, eps)
        elif layer["type"] == "retention":
            y = retention_mixer(x, w, pre, m, eps, pos)
        else:
            raise ValueError(layer["type"])
        x = norm_one_plus(alpha * x + y, w[f"l{i}.norm1"], eps)
        if layer.get("mlp") is not None:
            x = norm_one_plus(alpha * x + gated_feed_forward(x, w, f"l{i}.mlp."), w[f"l{i}.norm2"], eps)
        elif f"l{i}.norm2" in w:        # a file that holds a second norm for a layer without feed-forward
            x = norm_one_plus(alpha * x, w[f"l{i}.norm2"], eps)
        after.append(x)
    logits = linear(norm_one_plus(x, w["final.norm"], eps), w["head"])
    return (logits, np.stack(after)) if return_layers else logits


def greedy_generate(cfg, w, prompt, n_new):
    ids, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(np.argmax(forward(cfg, w, ids)[-1]))
        out.append(nxt)
        ids.append(nxt)
    return out


def random_config(rng, layer_types=("lightning", "attention", "retention"), width=48, vocab=97, share_from=None, **over):
    """A small configuration dictionary with the design's keys; `over` replaces mixer sizes."""
    layers = []
    for n, t in enumerate(layer_types):
        if t == "attention":
            m = dict(heads=over.get("heads", 4), kv_heads=over.get("kv_heads", 2), dim=over.get("dim", 16), vdim=over.get("vdim", 24),
                     scale=over.get("scale", 0.3), rot=dict(base=over.get("base", 5000.0), dims=over.get("rot_dims", 8),
                                                             scaling=over.get("scaling", dict(factor=4.0, original=64, fast=16.0, slow=2.0))))
            if share_from is not None and n in share_from:
                m["kv_from"] = share_from[n]
        elif t == "lightning":
            m = dict(heads=over.get("lin_heads", 3), dim=over.get("lin_dim", 8), vdim=over.get("lin_vdim", 16),
                     decay=over.get("decay", [0.5, 0.9, 0.995])[:over.get("lin_heads", 3)])
        else:
            m = dict(heads=over.get("lin_heads", 3), dim=over.get("lin_dim", 8), vdim=over.get("lin_vdim", 16),
                     decay=over.get("decay", [0.7, 0.95, 0.999])[:over.get("lin_heads", 3)],
                     rot=dict(base=over.get("ret_base", 300.0), dims=over.get("ret_rot_dims", over.get("lin_dim", 8))))
        mlp = None if (over.get("no_mlp") is not None and n in over["no_mlp"]) else dict(kind="dense", ff=over.get("ff", 80))
        layers.append(dict(type=t, mixer=m, mlp=mlp))
    return dict(architecture="Vokelix", layers=layers, norm=dict(eps=over.get("eps", 1e-5)), postln_alpha=over.get("alpha", 1.5),
                vocab=vocab, width=width)


def tensor_shapes(cfg, norm2_always=False):
    """name -> shape of every tensor of a configuration, in file order.  norm2_always: also for layers
    without a feed-forward."""
    D, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], f"l{i}."
        out[p + "norm1"] = (D,)
        if layer.get("mlp") is not None or norm2_always:
            out[p + "norm2"] = (D,)
        H, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m["kv_heads"]
            out[p + "mix.q"], out[p + "mix.q.b"], out[p + "mix.q.norm"] = (H * d, D), (H * d,), (H * d,)
            if m.get("kv_from") is None:
                out[p + "mix.k"], out[p + "mix.k.b"], out[p + "mix.k.norm"] = (G * d, D), (G * d,), (G * d,)
                out[p + "mix.v"], out[p + "mix.v.b"] = (G * dv, D), (G * dv,)
            out[p + "mix.sink"], out[p + "mix.g"], out[p + "mix.o"] = (H,), (H, D), (D, H * dv)
        else:
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = (H * d, D), (H * d, D), (H * dv, D)
            out[p + "mix.g"], out[p + "mix.o"] = (H * dv, D), (D, H * dv)
            if layer["type"] == "lightning":
                out[p + "mix.norm"] = (H * dv,)
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            out[p + "mlp.gate"], out[p + "mlp.up"], out[p + "mlp.down"] = (ff, D), (ff, D), (D, ff)
    out["final.norm"], out["head"] = (D,), (cfg["vocab"], D)
    return out
