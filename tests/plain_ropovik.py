"""Plain, slow Ropovik decoder: the oracle of the numerics tests of that design.

Ropovik is a decoder-only model whose layers are listed one by one in its
config.json: each is either grouped-query attention whose values are the keys
as projected (no value projection), with partial rotary positions under YaRN
frequency scaling, or a Mamba-2 recurrence (a selective state space with a
scalar decay per head), each optionally followed by a dense feed-forward with a
squared-relu activation.  A stretch of the layers may run several times with
the same weights; before every such pass the hidden state is mixed with the
embedding output by a projection of the two side by side.  Layer norms with
bias, a soft cap on the logits.

Whole sequences, no cache, one function per mechanism, NumPy in float64.  It
shares no code with the package (the safetensors reader is the one of
plain_llama.py, which is also test code).

Notation: W is stored [out, in] and applied as x W^T for row vectors x.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


# --------------------------------------------------------------------------
# norms
# --------------------------------------------------------------------------
def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b; var is the mean squared deviation."""
    x = np.asarray(x, F64)
    mu = x.mean(axis=-1, keepdims=True)
    d = x - mu
    var = (d * d).mean(axis=-1, keepdims=True)
    return d / np.sqrt(var + eps) * w + b


def rms_norm_parts(x, w, parts, eps):
    """The last axis is cut into `parts` equal pieces; every piece is divided by
    its own root mean square (eps inside the root); then the weight."""
    x = np.asarray(x, F64)
    n = x.shape[-1]
    y = x.reshape(x.shape[:-1] + (parts, n // parts))
    y = y / np.sqrt((y * y).mean(axis=-1, keepdims=True) + eps)
    return y.reshape(x.shape) * w


# --------------------------------------------------------------------------
# activations
# --------------------------------------------------------------------------
def silu(x):
    return x / (1.0 + np.exp(-x))


def softplus(x):
    return np.maximum(x, 0.0) + np.log1p(np.exp(-np.abs(x)))


def relu_squared(x):
    r = np.maximum(x, 0.0)
    return r * r


# --------------------------------------------------------------------------
# rotary positions with YaRN scaling
# --------------------------------------------------------------------------
def rotary_frequencies(dims, base, scaling):
    """(frequencies [dims/2], amplitude).  Without scaling: base^(-2i/dims), 1.
    With {factor, original, fast, slow}: a ramp over the pair index i between the
    pairs that turn `fast` and `slow` times within `original` positions blends
    f_i (ramp 0) into f_i / factor (ramp 1); cos and sin grow by 0.1 ln(factor) + 1."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], F64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2, dtype=F64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, dims, freqs, amplitude):
    """x: [T, heads, dim].  Channel i < dims/2 pairs with i + dims/2; channels from
    `dims` on pass unchanged."""
    x = np.asarray(x, F64)
    half = dims // 2
    ang = np.asarray(positions, F64)[:, None] * freqs[None, :]          # [T, half]
    c, s = np.cos(ang)[:, None, :] * amplitude, np.sin(ang)[:, None, :] * amplitude
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# --------------------------------------------------------------------------
# attention whose values are the unrotated keys
# --------------------------------------------------------------------------
def attention_mixer(h, wq, wk, wo, m, positions=None):
    """h: [T, width] -> [T, width].  m: the layer's 'mixer' block of config.json."""
    T = h.shape[0]
    H, G, dim = m["heads"], m["kv_heads"], m["dim"]
    positions = np.arange(T) if positions is None else positions
    q = (h @ wq.T).reshape(T, H, dim)
    k = (h @ wk.T).reshape(T, G, dim)
    v = k                                                   # as projected, before rotation
    rot = m.get("rot")
    if rot:
        freqs, amp = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = rotate(q, positions, rot["dims"], freqs, amp)
        k = rotate(k, positions, rot["dims"], freqs, amp)
    out = np.zeros((T, H, dim), F64)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head, :] @ k[:, g, :].T) * m["scale"]     # [T, T]
        s = np.where(np.tril(np.ones((T, T), bool)), s, -np.inf)
        p = np.exp(s - s.max(axis=-1, keepdims=True))
        p /= p.sum(axis=-1, keepdims=True)
        out[:, head, :] = p @ v[:, g, :]
    return out.reshape(T, H * dim) @ wo.T


# --------------------------------------------------------------------------
# Mamba-2
# --------------------------------------------------------------------------
def causal_conv(x, w, b):
    """x: [T, C]; w: [C, taps], the last tap is the current token's; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), F64), np.asarray(x, F64)], axis=0)
    out = np.zeros((T, C), F64) + b
    for j in range(taps):
        out += padded[j:j + T] * w[:, j]
    return out


def selective_scan(x, dt, a_log, B, C, D):
    """x: [T, heads, P], dt: [T, heads] (after softplus), B, C: [T, groups, N].
    S_t = exp(-exp(a_log) dt_t) S_{t-1} + dt_t B_t x_t^T;  y_t = S_t^T C_t + D x_t."""
    T, heads, P = x.shape
    groups, N = B.shape[1], B.shape[2]
    y = np.zeros((T, heads, P), F64)
    for head in range(heads):
        g = head // (heads // groups)
        S = np.zeros((N, P), F64)
        for t in range(T):
            S = math.exp(-math.exp(a_log[head]) * dt[t, head]) * S + dt[t, head] * np.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + D[head] * x[t, head]
    return y


def mamba2_mixer(h, w, m, eps):
    """h: [T, width]; w: the mixer's tensors by short name (in, conv, conv.b,
    dt_bias, A_log, D, norm, o)."""
    T = h.shape[0]
    heads, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * P
    proj = h @ w["in"].T                                     # [z | x | B | C | dt]
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = selective_scan(x, dt, w["A_log"], B, C, w["D"]).reshape(T, inner)
    y = rms_norm_parts(y * silu(z), w["norm"], m["norm_groups"], eps)
    return y @ w["o"].T


# --------------------------------------------------------------------------
# feed-forward, loop input, head
# --------------------------------------------------------------------------
def dense_feed_forward(h, up, down):
    return relu_squared(h @ up.T) @ down.T


def loop_input(x, x0, w_in):
    """[x | x0] W_in^T: the hidden state and the embedding output side by side."""
    return np.concatenate([x, x0], axis=-1) @ w_in.T


def soft_cap(logits, cap):
    return cap * np.tanh(logits / cap) if cap else logits


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def layer_runs(cfg):
    """The order in which layers run: [('in',) | ('layer', i)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [("layer", i) for i in range(n)]
    runs = [("layer", i) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        runs.append(("in",))
        runs += [("layer", i) for i in range(loop["start"], loop["stop"])]
    runs += [("layer", i) for i in range(loop["stop"], n)]
    return runs


def forward(cfg, W, tokens, return_layers=False):
    """tokens: [T] -> logits [T, vocab] (float64); with return_layers also the
    hidden state after every layer run, [runs, T, width]."""
    W = {k: np.asarray(v, F64) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x0 = W["embed"][np.asarray(tokens)]
    x = x0.copy()
    after = []
    for run in layer_runs(cfg):
        if run[0] == "in":
            x = loop_input(x, x0, W["loop.in"])
            continue
        i = run[1]
        layer, p = cfg["layers"][i], f"l{i}."
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(h, W[p + "mix.q"], W[p + "mix.k"], W[p + "mix.o"], layer["mixer"])
        elif layer["type"] == "mamba2":
            short = {k[len(p) + 4:]: v for k, v in W.items() if k.startswith(p + "mix.")}
            x = x + mamba2_mixer(h, short, layer["mixer"], eps)
        else:
            raise ValueError(f"plain Ropovik: layer type {layer['type']!r}")
        if layer.get("mlp"):
            h = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            x = x + dense_feed_forward(h, W[p + "mlp.up"], W[p + "mlp.down"])
        after.append(x.copy())
    h = layer_norm(x, W["final.norm"], W["final.norm.b"], eps)
    logits = soft_cap(h @ W["head"].T, cfg.get("logit_softcap"))
    return (logits, np.stack(after)) if return_layers else logits


def greedy(cfg, W, prompt, n_new):
    """Greedy generation by running the whole sequence again for each token."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(np.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
