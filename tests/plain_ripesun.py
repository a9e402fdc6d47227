"""A plain, slow implementation of the Ripesun design in numpy float64, one function per mechanism.

It shares no code with the engine: every recurrence is a loop over tokens, attention builds every head's keys and
values from the latent and walks the keys of one query at a time, and masks are written as comparisons of positions.
``forward`` runs a whole sequence from position 0 and returns the logits of every position.

Notation: x the stream [T, D]; N(x, w) = x / sqrt(mean(x^2) + eps) * w over the last axis.
"""
import math

import numpy as np


def rms_norm(x, w, eps):
    x = np.asarray(x, dtype=np.float64)
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rotate_pairs(v, positions, base, dims):
    """v [T, ..., n]: the pair (v[2i], v[2i+1]), i < dims/2, of the token at position p turns by p * base^(-2i/dims)."""
    out = np.array(v, dtype=np.float64, copy=True)
    for t, p in enumerate(positions):
        for i in range(dims // 2):
            a = p * base ** (-2.0 * i / dims)
            u, w = v[t, ..., 2 * i], v[t, ..., 2 * i + 1]
            out[t, ..., 2 * i] = u * math.cos(a) - w * math.sin(a)
            out[t, ..., 2 * i + 1] = w * math.cos(a) + u * math.sin(a)
    return out


def latent_rows(h, positions, w_dkv, w_norm, kv_rank, rot_dim, base, dims, eps):
    """What a layer with its own key/value projection keeps per token: (c [T, kv_rank], k_rot [T, rot_dim])."""
    d = h @ w_dkv.T
    c = rms_norm(d[:, :kv_rank], w_norm, eps)
    k_rot = d[:, kv_rank:kv_rank + rot_dim]
    return c, (rotate_pairs(k_rot, positions, base, dims) if dims else k_rot.copy())


def latent_attention(h, positions, c, k_rot, p, heads, dim, rot_dim, vdim, base, dims, scale, window, eps):
    """Queries of the tokens in h (at ``positions``) against the rows (c, k_rot) of positions 0 .. len(c) - 1."""
    T = h.shape[0]
    cq = rms_norm(h @ p["dq"].T, p["dq.norm"], eps)
    q = (cq @ p["uq"].T).reshape(T, heads, dim + rot_dim)
    q_rot = rotate_pairs(q[:, :, dim:], positions, base, dims) if dims else q[:, :, dim:]
    keys = (c @ p["uk"].T).reshape(len(c), heads, dim)
    vals = (c @ p["uv"].T).reshape(len(c), heads, vdim)
    out = np.zeros((T, heads, vdim))
    for t, pos in enumerate(positions):
        seen = [j for j in range(len(c)) if 0 <= pos - j and (window == 0 or pos - j < window)]
        for hd in range(heads):
            s = np.array([(q[t, hd, :dim] @ keys[j, hd] + q_rot[t, hd] @ k_rot[j]) * scale for j in seen])
            m = max(s.max(), p["sink"][hd])
            e = np.exp(s - m)
            den = e.sum() + math.exp(p["sink"][hd] - m)
            out[t, hd] = sum((e[n] / den) * vals[j, hd] for n, j in enumerate(seen))
    return out.reshape(T, heads * vdim) @ p["o"].T


def lightning(h, p, heads, dim, vdim, decay, eps, state=None):
    """Token by token: S = decay_h S + k v^T; o = S^T q.  Returns (output [T, D], state [heads, dim, vdim])."""
    T = h.shape[0]
    q = silu(h @ p["q"].T).reshape(T, heads, dim)
    k = silu(h @ p["k"].T).reshape(T, heads, dim)
    v = silu(h @ p["v"].T).reshape(T, heads, vdim)
    S = np.zeros((heads, dim, vdim)) if state is None else state.copy()
    o = np.zeros((T, heads, vdim))
    for t in range(T):
        for hd in range(heads):
            S[hd] = decay[hd] * S[hd] + np.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    o = rms_norm(o.reshape(T, heads * vdim), p["norm"], eps) * sigmoid(h @ p["g"].T)
    return o @ p["o"].T, S


def mingru(h, p, state=None):
    """Token by token: S = (1 - z) S + z c.  Returns (output [T, D], state [width])."""
    z = sigmoid(h @ p["z"].T + p["z.b"])
    u = h @ p["x"].T + p["x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(z.shape[1]) if state is None else state.copy()
    o = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        o[t] = S
    return (o * silu(h @ p["g"].T)) @ p["o"].T, S


def dense(h, p):
    return gelu_tanh(h @ p["up"].T) @ p["down"].T


def side_input(x, tokens, table, layer, dim, p):
    e = table[tokens][:, layer * dim:(layer + 1) * dim]
    return (gelu_tanh(x @ p["gate"].T) * e) @ p["proj"].T


def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, layers_out=None):
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    tokens = list(tokens)
    positions = list(range(len(tokens)))
    x = tensors["embed"][tokens] * (cfg.get("embedding") or {}).get("scale", 1.0)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        mx, lp = layer["mixer"], _sub(tensors, f"l{i}.")
        mp = _sub(lp, "mix.")
        h = rms_norm(x, lp["norm1"], eps)
        if layer["type"] == "latent_attention":
            rot = mx.get("rot") or {}
            base, dims = rot.get("base", 1.0), int(rot.get("dims") or 0)
            if mx.get("kv_from") is None:
                kept[i] = latent_rows(h, positions, mp["dkv"], mp["dkv.norm"], mx["kv_rank"], mx["rot_dim"], base, dims, eps)
            c, k_rot = kept[i if mx.get("kv_from") is None else mx["kv_from"]]
            a = latent_attention(h, positions, c, k_rot, mp, mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], base, dims,
                                 mx["scale"], int((mx.get("mask") or {}).get("size") or 0), eps)
        elif layer["type"] == "lightning":
            a, _ = lightning(h, mp, mx["heads"], mx["dim"], mx["vdim"], mx["decay"], eps)
        elif layer["type"] == "mingru":
            a, _ = mingru(h, mp)
        else:
            raise ValueError(layer["type"])
        x = x + m * rms_norm(a, lp["norm1b"], eps)
        if layer.get("mlp"):
            x = x + m * rms_norm(dense(rms_norm(x, lp["norm2"], eps), _sub(lp, "mlp.")), lp["norm2b"], eps)
        if (cfg.get("token_side") or {}).get("dim"):
            sp = _sub(lp, "side.")
            x = x + m * rms_norm(side_input(x, tokens, tensors["side.embed"], i, cfg["token_side"]["dim"], sp), sp["norm"], eps)
        if layers_out is not None:
            layers_out.append(x.copy())
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    cap = cfg.get("logit_softcap")
    return cap * np.tanh(logits / cap) if cap else logits
