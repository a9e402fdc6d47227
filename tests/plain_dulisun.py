"""A plain, slow implementation of the Dulisun decoder in numpy float64, one function per
mechanism, written from the design's equations.  It shares no code with the engine: the tests
hold the engine's parts and whole models to it.

Notation: x [T, D] residual stream; positions p_t count from 0; weights W are [out, in] and
act as W x.  ``tensors`` maps checkpoint names to numpy arrays; ``config`` is the parsed
``config.json``.
"""
import math

import numpy as np

_ERF = np.vectorize(math.erf, otypes=[np.float64])


# ------------------------------------------------------------------ elementwise pieces
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def offset_rmsnorm(x, w, eps):
    """RMS norm whose stored weight lies around zero: unit_rms(x) * (1 + w)."""
    return unit_rms(x, eps) * (1.0 + np.asarray(w, dtype=np.float64))


def gelu_erf(z):
    z = np.asarray(z, dtype=np.float64)
    return 0.5 * z * (1.0 + _ERF(z / math.sqrt(2.0)))


def gelu_tanh(z):
    z = np.asarray(z, dtype=np.float64)
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


ACTIVATIONS = {"gelu": gelu_erf, "gelu_erf": gelu_erf, "gelu_tanh": gelu_tanh}


def rotate_interleaved(v, positions, base, dims):
    """v [T, heads, d].  Dimension 2i is paired with 2i+1 for i < dims/2; the pair (a, b) at
    position p becomes (a cos t - b sin t, b cos t + a sin t), t = p * base^(-2i/dims).  The
    dimensions from ``dims`` on pass unchanged."""
    v = np.array(v, dtype=np.float64)
    out = v.copy()
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        ang = np.asarray(positions, dtype=np.float64) * f
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        a, b = v[:, :, 2 * i], v[:, :, 2 * i + 1]
        out[:, :, 2 * i] = a * c - b * s
        out[:, :, 2 * i + 1] = b * c + a * s
    return out


# ------------------------------------------------------------------ attention
def chunk_sink_attention(q, k, v, q_pos, k_pos, scale, chunk, sink):
    """q [Tq, H, d], k [Tk, G, d], v [Tk, G, dv]; query at position i sees the key at position j
    iff j <= i and floor(i / chunk) == floor(j / chunk) (``chunk`` None or 0: every j <= i).  Per head the softmax denominator also
    holds exp(sink[h]), which has no key and no value.  Returns [Tq, H, dv]."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    out = np.zeros((Tq, H, v.shape[2]))
    for t in range(Tq):
        i = int(q_pos[t])
        vis = [n for n, j in enumerate(k_pos) if j <= i and (not chunk or (int(j) // chunk) == (i // chunk))]
        for h in range(H):
            g = h // rep
            s = np.array([float(np.dot(q[t, h], k[n, g])) * scale for n in vis] + [float(sink[h])])
            m = s.max()
            e = np.exp(s - m)
            w = e[:-1] / e.sum()
            for wn, n in zip(w, vis):
                out[t, h] += wn * v[n, g]
    return out


def attention_mixer(h, positions, W, mc, eps, past=None):
    """The mixer on its input h [T, D].  ``W`` holds q, k, sink, o.  ``past`` = (k_rows, v_rows,
    their positions) of earlier tokens of the sequence, or None.  Returns (y, (k, v, positions))
    so that a caller can feed tokens one by one."""
    H, G, d, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    T = h.shape[0]
    q = (h @ W["q"].T.astype(np.float64)).reshape(T, H, d)
    kp = (h @ W["k"].T.astype(np.float64)).reshape(T, G, d)
    v = kp[:, :, :dv].copy()                                    # the values are the keys as projected
    rot = mc.get("rot") or {"base": 1.0, "dims": 0}
    q = unit_rms(rotate_interleaved(q, positions, rot["base"], rot["dims"]), eps)
    k = unit_rms(rotate_interleaved(kp, positions, rot["base"], rot["dims"]), eps)
    pos = np.asarray(positions)
    if past is not None:
        k = np.concatenate([past[0], k], axis=0)
        v = np.concatenate([past[1], v], axis=0)
        kpos = np.concatenate([past[2], pos])
    else:
        kpos = pos
    a = chunk_sink_attention(q, k, v, pos, kpos, mc["scale"], (mc.get("mask") or {}).get("size"), W["sink"].astype(np.float64))
    y = a.reshape(T, H * dv) @ W["o"].T.astype(np.float64)
    return y, (k, v, kpos)


# ------------------------------------------------------------------ feed-forward
def expert_ff(h, up, down, act="gelu"):
    return ACTIVATIONS[act](h @ up.T.astype(np.float64)) @ down.T.astype(np.float64)


def route(z, top, group_count, group_keep):
    """z [E] router logits -> (chosen experts, their weights).  Scores are the softmax over all
    experts; a group (E / group_count neighbours) scores its best expert; only experts of the
    best ``group_keep`` groups can be chosen; the ``top`` best of those are taken with their
    scores as weights, not renormalised."""
    z = np.asarray(z, dtype=np.float64)
    s = np.exp(z - z.max())
    s = s / s.sum()
    E = s.shape[0]
    per = E // group_count
    gscore = s.reshape(group_count, per).max(axis=1)
    kept = sorted(range(group_count), key=lambda g: (-gscore[g], g))[:group_keep]
    allowed = [e for e in range(E) if e // per in kept]
    chosen = sorted(allowed, key=lambda e: (-s[e], e))[:top]
    return chosen, [s[e] for e in chosen]


def moe_ff(h, W, mlp):
    """Routed experts plus the shared expert.  ``W``: router, e<i>.up/down, shared.up/down."""
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    act = (mlp.get("expert") or {}).get("act", "gelu")
    out = np.zeros((h.shape[0], W["e0.down"].shape[0]))
    z = h @ W["router"].T.astype(np.float64)
    for t in range(h.shape[0]):
        chosen, weights = route(z[t], r["top"], groups["count"], groups["keep"])
        for e, w in zip(chosen, weights):
            out[t] += w * expert_ff(h[t:t + 1], W[f"e{e}.up"], W[f"e{e}.down"], act)[0]
    if mlp.get("shared"):
        out += expert_ff(h, W["shared.up"], W["shared.down"], mlp["shared"].get("act", "gelu"))
    return out


# ------------------------------------------------------------------ the model
def _sub(tensors, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config, tensors, token_ids, keep_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the residual stream after every
    layer when asked)."""
    eps = config["norm"]["eps"]
    T = len(token_ids)
    positions = np.arange(T)
    x = tensors["embed"].astype(np.float64)[np.asarray(token_ids)]
    x = offset_rmsnorm(x, tensors["embed.norm"], eps)
    streams = []
    for i, layer in enumerate(config["layers"]):
        assert layer["type"] == "attention"
        p = f"l{i}."
        y, _ = attention_mixer(x, positions, _sub(tensors, p + "mix."), layer["mixer"], eps)
        x = x + offset_rmsnorm(y, tensors[p + "norm1"], eps)
        if layer.get("mlp"):
            f = moe_ff(x, _sub(tensors, p + "mlp."), layer["mlp"])
            x = x + offset_rmsnorm(f, tensors[p + "norm2"], eps)
        streams.append(x.copy())
    hn = offset_rmsnorm(x, tensors["final.norm"], eps)
    logits = hn @ tensors["embed"].T.astype(np.float64)
    return (logits, np.stack(streams)) if keep_layers else logits
