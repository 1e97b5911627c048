"""Plain, slow implementation of the Vizosun decoder in float64 numpy.

The oracle of the Vizosun tests: whole sequences, no cache, no chunks, one function per mechanism,
and no code shared with the `inferllm_b200` package (it reads the raw `config.json` dictionary and
a dictionary of numpy arrays keyed by tensor name).

Notation: T tokens, width D; a linear map is `y = x @ W.T` with W stored [out, in].  Every
recurrence is the literal token-by-token loop.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def linear(x, w, b=None):
    y = np.asarray(x, F64) @ np.asarray(w, F64).T
    return y if b is None else y + np.asarray(b, F64)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis (w None: no weight)."""
    x = np.asarray(x, F64)
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)
    return y if w is None else y * np.asarray(w, F64)


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-np.asarray(z, F64)))


def silu(z):
    z = np.asarray(z, F64)
    return z * sigmoid(z)


def softplus(z):
    z = np.asarray(z, F64)
    return np.logaddexp(0.0, z)


# --------------------------------------------------------------------------- embedding


def bigram_rows(ids, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous, current); the row behind the
    hashed ones for a sequence's first token."""
    rows = []
    for t, tok in enumerate(ids):
        rows.append(buckets if t == 0 else (int(ids[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return rows


def embed(cfg, w, ids):
    x = np.asarray(w["embed"], F64)[list(ids)]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        x = x + np.asarray(w["bigram"], F64)[bigram_rows(ids, bg["buckets"], bg["mul_prev"], bg["mul_cur"])]
    return x


# --------------------------------------------------------------------------- mixers


def causal_conv(x, taps):
    """x [T, C], taps [C, K]: y[t, c] = sum_j taps[c, K-1-j] x[t-j, c], zeros before the start."""
    x, taps = np.asarray(x, F64), np.asarray(taps, F64)
    T, K = x.shape[0], taps.shape[1]
    y = np.zeros_like(x)
    for t in range(T):
        for j in range(K):
            if t - j >= 0:
                y[t] += taps[:, K - 1 - j] * x[t - j]
    return y


def unit(x):
    """Every head's vector divided by sqrt(sum of squares + 1e-6)."""
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def delta_recurrence(q, k, v, g, beta):
    """q, k, g [T, H, d]; v [T, H, dv]; beta [T, H].  Per head, S [d, dv] from zero:
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T, H, d = q.shape
    dv = v.shape[-1]
    o = np.zeros((T, H, dv), F64)
    for h in range(H):
        S = np.zeros((d, dv), F64)
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            o[t, h] = S.T @ q[t, h]
    return o


def channel_delta(m, w, p, h, eps):
    """The gated delta rule with a decay per head and key channel.  m: the mixer's sizes; p: prefix."""
    H, KV, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(causal_conv(linear(h, w[p + "q"]), w[p + "q.conv"])).reshape(T, KV, d)
    k = silu(causal_conv(linear(h, w[p + "k"]), w[p + "k.conv"])).reshape(T, KV, d)
    v = silu(causal_conv(linear(h, w[p + "v"]), w[p + "v.conv"])).reshape(T, H, dv)
    q = unit(q) * d ** -0.5
    k = unit(k)
    rep = H // KV
    q = np.repeat(q, rep, axis=1)          # head j reads q/k head j // rep
    k = np.repeat(k, rep, axis=1)
    beta = sigmoid(linear(h, w[p + "b"]))
    a = linear(linear(h, w[p + "a1"]), w[p + "a2"]) + np.asarray(w[p + "dt_bias"], F64)
    rate = np.exp(np.asarray(w[p + "A_log"], F64))
    g = np.exp(-rate[None, :, None] * softplus(a).reshape(T, H, d))
    o = delta_recurrence(q, k, v, g, beta)
    o = rms_norm(o, w[p + "norm"], eps)
    gate = sigmoid(linear(linear(h, w[p + "g1"]), w[p + "g2"])).reshape(T, H, dv)
    return linear((o * gate).reshape(T, H * dv), w[p + "o"])


def window_softmax_attention(q, k, v, scale, window):
    """q, k [T, H, d]; v [T, H, dv]; token i sees j with 0 <= i - j < window (window None: all before)."""
    T, H, _ = q.shape
    o = np.zeros((T, H, v.shape[-1]), F64)
    for i in range(T):
        lo = 0 if not window else max(0, i - window + 1)
        for h in range(H):
            s = (k[lo:i + 1, h] @ q[i, h]) * scale
            e = np.exp(s - s.max())
            o[i, h] = (e / e.sum()) @ v[lo:i + 1, h]
    return o


def latent_attention(m, w, p, h, eps):
    """Attention whose queries and whose keys and values come out of normed low-rank latents."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    cq = rms_norm(linear(h, w[p + "dq"]), w[p + "dq.norm"], eps)
    q = linear(cq, w[p + "uq"]).reshape(T, H, d)
    c = rms_norm(linear(h, w[p + "dkv"]), w[p + "dkv.norm"], eps)
    k = linear(c, w[p + "uk"]).reshape(T, H, d)
    v = linear(c, w[p + "uv"]).reshape(T, H, dv)
    window = (m.get("mask") or {}).get("size")
    o = window_softmax_attention(q, k, v, m["scale"], window)
    return linear(o.reshape(T, H * dv), w[p + "o"])


# --------------------------------------------------------------------------- feed-forward


def dense_ff(w, p, h):
    return linear(np.maximum(linear(h, w[p + "gate"]), 0.0) * linear(h, w[p + "up"]), w[p + "down"])


def routed_ff(mlp, w, p, h):
    """Every token goes through its `top` experts with the largest router logits; their weights are
    the softmax over those logits alone."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = linear(h, w[p + "router"], w[p + "router.b"])
    out = np.zeros((h.shape[0], np.asarray(w[p + "e0.down"]).shape[0]), F64)
    for t in range(h.shape[0]):
        chosen = np.argsort(-z[t], kind="stable")[:top]
        e = np.exp(z[t, chosen] - z[t, chosen].max())
        for j, wt in zip(chosen, e / e.sum()):
            pe = f"{p}e{j}."
            out[t] += wt * linear(silu(linear(h[t], w[pe + "gate"])) * linear(h[t], w[pe + "up"]), w[pe + "down"])
    assert E == z.shape[1]
    return out


# --------------------------------------------------------------------------- the model


def layer_runs(cfg):
    """The layers in the order they run: (layer index, first of a pass?)."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return runs + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, w, ids, return_layers=False):
    """float64 logits [T, vocab] of one sequence (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x0 = embed(cfg, w, ids)
    x = x0
    streams = []
    for i, first in layer_runs(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if first:
            x = linear(np.concatenate([x, x0], axis=-1), w["loop.in"])
        h = rms_norm(x, w[p + "norm1"], eps)
        if L["type"] == "channel_delta":
            y = channel_delta(L["mixer"], w, p + "mix.", h, eps)
        elif L["type"] == "latent_attention":
            y = latent_attention(L["mixer"], w, p + "mix.", h, eps)
        else:
            raise ValueError(L["type"])
        mlp = L.get("mlp")
        if mlp:
            y = y + (dense_ff(w, p + "mlp.", h) if mlp["kind"] == "dense" else routed_ff(mlp, w, p + "mlp.", h))
        x = x + y
        streams.append(x)
    logits = linear(rms_norm(x, w["final.norm"], eps), w["embed"])
    return (logits, np.stack(streams)) if return_layers else logits


def greedy_generate(cfg, w, prompt, n_new):
    ids = list(prompt)
    for _ in range(n_new):
        ids.append(int(np.argmax(forward(cfg, w, ids)[-1])))
    return ids[len(prompt):]


# --------------------------------------------------------------------------- weights


def tensor_shapes(cfg):
    """name -> (shape, kind) of every tensor a model of this configuration has; kind is "matrix",
    "norm" (around one), "conv", "vector" or "decay"."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": ((V, D), "matrix")}
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = ((bg["buckets"] + 1, D), "matrix")
    if cfg.get("loop"):
        out["loop.in"] = ((D, 2 * D), "matrix")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = ((D,), "norm")
        if L["type"] == "channel_delta":
            H, KV, d, dv, K = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            ra, rg = m.get("a_rank", 8), m.get("g_rank", 8)
            for n, rows in (("q", KV * d), ("k", KV * d), ("v", H * dv)):
                out[p + "mix." + n] = ((rows, D), "matrix")
                out[p + "mix." + n + ".conv"] = ((rows, K), "conv")
            out[p + "mix.b"] = ((H, D), "matrix")
            out[p + "mix.A_log"] = ((H,), "decay")
            out[p + "mix.norm"] = ((dv,), "norm")
            out[p + "mix.a1"] = ((ra, D), "matrix")
            out[p + "mix.a2"] = ((H * d, ra), "matrix")
            out[p + "mix.dt_bias"] = ((H * d,), "vector")
            out[p + "mix.g1"] = ((rg, D), "matrix")
            out[p + "mix.g2"] = ((H * dv, rg), "matrix")
            out[p + "mix.o"] = ((D, H * dv), "matrix")
        else:
            H, d, dv, R, Q = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            out[p + "mix.dq"] = ((Q, D), "matrix")
            out[p + "mix.dq.norm"] = ((Q,), "norm")
            out[p + "mix.uq"] = ((H * d, Q), "matrix")
            out[p + "mix.dkv"] = ((R, D), "matrix")
            out[p + "mix.dkv.norm"] = ((R,), "norm")
            out[p + "mix.uk"] = ((H * d, R), "matrix")
            out[p + "mix.uv"] = ((H * dv, R), "matrix")
            out[p + "mix.o"] = ((D, H * dv), "matrix")
        mlp = L.get("mlp")
        if mlp and mlp["kind"] == "dense":
            out[p + "mlp.gate"] = ((mlp["ff"], D), "matrix")
            out[p + "mlp.up"] = ((mlp["ff"], D), "matrix")
            out[p + "mlp.down"] = ((D, mlp["ff"]), "matrix")
        elif mlp:
            E, F = mlp["router"]["experts"], mlp["expert"]["ff"]
            out[p + "mlp.router"] = ((E, D), "matrix")
            out[p + "mlp.router.b"] = ((E,), "vector")
            for e in range(E):
                out[f"{p}mlp.e{e}.gate"] = ((F, D), "matrix")
                out[f"{p}mlp.e{e}.up"] = ((F, D), "matrix")
                out[f"{p}mlp.e{e}.down"] = ((D, F), "matrix")
    out["final.norm"] = ((D,), "norm")
    return out


def random_weights(cfg, seed, scale=1.0):
    """Random weights rounded to bfloat16 values (as float32 arrays), sized so that activations stay
    of order one through the layers."""
    rng = np.random.default_rng(seed)
    w = {}
    for name, (shape, kind) in tensor_shapes(cfg).items():
        if name in ("embed", "bigram"):
            a = rng.standard_normal(shape)
        elif kind == "matrix":
            a = rng.standard_normal(shape) * scale / math.sqrt(shape[-1])
        elif kind == "norm":
            a = 1.0 + 0.1 * rng.standard_normal(shape)
        elif kind == "conv":
            a = rng.standard_normal(shape) * 0.5
        elif kind == "decay":
            a = rng.uniform(-2.0, 0.5, shape)
        else:
            a = rng.standard_normal(shape) * 0.5
        w[name] = bf16_round(a.astype(np.float32))
    return w


def bf16_round(a):
    """float32 array rounded to the nearest bfloat16 value (ties to even), still float32."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32).astype(np.uint64)
    u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
    return u.astype(np.uint32).view(np.float32).reshape(np.shape(a))


def write_safetensors(path, w):
    """Write float arrays as bfloat16 (their values must be bfloat16 already) and integer arrays as int32."""
    import json
    import struct
    header, blobs, off = {}, [], 0
    for name, a in w.items():
        a = np.asarray(a)
        if a.dtype.kind in "iu":
            blob, dt = a.astype("<i4").tobytes(), "I32"
        else:
            blob, dt = (np.ascontiguousarray(a, np.float32).view(np.uint32) >> 16).astype("<u2").tobytes(), "BF16"
        header[name] = {"dtype": dt, "shape": list(a.shape), "data_offsets": [off, off + len(blob)]}
        blobs.append(blob)
        off += len(blob)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)


def read_safetensors(path):
    import json
    import struct
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        raw = data[a:b]
        if rec["dtype"] == "BF16":
            arr = (np.frombuffer(raw, "<u2").astype(np.uint32) << 16).view(np.float32)
        elif rec["dtype"] == "F32":
            arr = np.frombuffer(raw, "<f4")
        elif rec["dtype"] == "I32":
            arr = np.frombuffer(raw, "<i4")
        else:
            raise ValueError(rec["dtype"])
        out[name] = arr.reshape(rec["shape"])
    return out


def random_config(layer_types, width=48, vocab=97, heads=4, kv_heads=2, dim=16, vdim=8, conv=3, a_rank=8, g_rank=4, att_heads=3, att_dim=16,
                  att_vdim=24, q_rank=24, kv_rank=32, window=20, scale=0.5, experts=5, top=2, expert_ff=24, ff=64, mlps=None, loop=None,
                  bigram=(53, 31, 7), eps=1e-5, max_positions=1024):
    """A small configuration: `layer_types` names the mixers, `mlps` the feed-forwards ("dense", "moe" or None) of the
    layers (dense and moe in turn if not given)."""
    layers = []
    for i, t in enumerate(layer_types):
        kind = mlps[i] if mlps is not None else ("dense", "moe")[i % 2]
        if t == "channel_delta":
            m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "a_rank": a_rank, "g_rank": g_rank}
        else:
            m = {"heads": att_heads, "dim": att_dim, "vdim": att_vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
            if window:
                m["mask"] = {"size": window}
        mlp = None
        if kind == "dense":
            mlp = {"kind": "dense", "ff": ff}
        elif kind == "moe":
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top}}
        layers.append({"type": t, "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Vizosun", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers, "max_positions": max_positions}
    if bigram:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg
