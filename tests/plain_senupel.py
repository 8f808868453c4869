"""Plain, slow Senupel decoder: the oracle of the numerics tests of that design.

Senupel is a decoder-only model whose config.json lists its layers one by one.
Every layer adds the *normed output* of its sublayers to the hidden state, and
the sublayers read the hidden state itself:

    x <- x + rms(mixer(x)) w1,      x <- x + rms(ff(x)) w2.

The mixer is attention through a latent: one down projection gives a short
latent vector per token (normed) and one small rotated key shared by all heads;
every head's unrotated key and its value are up projections of the latent.  A
layer may have no down projection and read the latents and rotated keys of an
earlier layer.  Keys are visible inside a sliding window; the heads are gated
by a sigmoid of a projection of the mixer's input.  The feed-forward is a gated
silu layer with biases, or a mixture of such experts without biases, the
chosen ones weighted by a softmax over their own router logits.

Whole sequences, no cache, one function per mechanism, NumPy in float64.  It
shares no code with the package.

Notation: W is stored [out, in]; rows of x are tokens, so a projection is x W^T.
"""
from __future__ import annotations

import math

import numpy as np

F64 = np.float64


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    x = np.asarray(x, F64)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * np.asarray(w, F64)


def silu(z):
    return z / (1.0 + np.exp(-z))


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


# --------------------------------------------------------------------------
# rotary positions, interleaved pairs, YaRN scaling
# --------------------------------------------------------------------------
def rotary_frequencies(dims, base, scaling=None):
    """(f [dims/2], amplitude).  f_i = base^(-2i/dims).  With scaling {factor,
    original, fast, slow}: pair i makes original f_i / (2 pi) turns in `original`
    positions; from the pair that makes `fast` turns (its index rounded down) to
    the one that makes `slow` turns (rounded up) a ramp rises from 0 to 1, and
    f_i becomes f_i (1 - ramp_i) + f_i / factor ramp_i.  Cosines and sines are
    multiplied by the amplitude 0.1 ln(factor) + 1."""
    f = np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], F64)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(dims // 2, dtype=F64) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, amplitude):
    """x [..., T, d] with d = 2 len(freqs): channels (2i, 2i+1) of token t turn by
    the angle positions[t] f_i; cos and sin carry the amplitude."""
    x = np.asarray(x, F64)
    angle = np.asarray(positions, F64)[:, None] * freqs[None, :]
    c, s = np.cos(angle) * amplitude, np.sin(angle) * amplitude
    u, v = x[..., 0::2], x[..., 1::2]
    out = np.empty_like(x)
    out[..., 0::2] = u * c - v * s
    out[..., 1::2] = v * c + u * s
    return out


# --------------------------------------------------------------------------
# the mixer
# --------------------------------------------------------------------------
def latent_and_rotated_key(h, w_dkv, w_norm, kv_rank, eps, positions, freqs, amplitude):
    """The two things a layer with a down projection leaves for attention:
    the normed latent [T, kv_rank] and the rotated shared key part [T, rot_dim]."""
    d = np.asarray(h, F64) @ np.asarray(w_dkv, F64).T
    latent = rms_norm(d[:, :kv_rank], w_norm, eps)
    return latent, rotate_pairs(d[:, kv_rank:], positions, freqs, amplitude)


def windowed_softmax_attention(q, k, v, window, scale):
    """q, k [H, T, dk], v [H, T, dv]: token i sees j with 0 <= i - j < window."""
    T = q.shape[1]
    scores = np.einsum("hid,hjd->hij", q, k) * scale
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    seen = (j <= i) & (i - j < window)
    scores = np.where(seen[None], scores, -np.inf)
    scores -= scores.max(axis=-1, keepdims=True)
    p = np.exp(scores)
    p /= p.sum(axis=-1, keepdims=True)
    return np.einsum("hij,hjd->hid", p, v)


def latent_attention(h, m, w, eps, latent, key_rot, positions, freqs, amplitude):
    """h [T, width]; m: the mixer's sizes; w: its tensors by short name (q, uk,
    uv, g, o); latent, key_rot: this layer's own or an earlier layer's."""
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    h = np.asarray(h, F64)
    T = h.shape[0]
    q = (h @ np.asarray(w["q"], F64).T).reshape(T, H, dim + rot).transpose(1, 0, 2)
    q = np.concatenate([q[..., :dim], rotate_pairs(q[..., dim:], positions, freqs, amplitude)], axis=-1)
    k_plain = (latent @ np.asarray(w["uk"], F64).T).reshape(T, H, dim).transpose(1, 0, 2)
    k = np.concatenate([k_plain, np.broadcast_to(key_rot[None], (H, T, rot))], axis=-1)
    v = (latent @ np.asarray(w["uv"], F64).T).reshape(T, H, vdim).transpose(1, 0, 2)
    heads = windowed_softmax_attention(q, k, v, int(m["mask"]["size"]), float(m["scale"]))
    mixed = heads.transpose(1, 0, 2).reshape(T, H * vdim) * sigmoid(h @ np.asarray(w["g"], F64).T)
    return mixed @ np.asarray(w["o"], F64).T


# --------------------------------------------------------------------------
# feed-forwards
# --------------------------------------------------------------------------
def gated_ff(h, gate, up, down, gate_b=None, up_b=None, down_b=None):
    """down(silu(gate h) * (up h)), each projection with its bias if it has one."""
    h = np.asarray(h, F64)
    g = h @ np.asarray(gate, F64).T + (0.0 if gate_b is None else np.asarray(gate_b, F64))
    u = h @ np.asarray(up, F64).T + (0.0 if up_b is None else np.asarray(up_b, F64))
    return (silu(g) * u) @ np.asarray(down, F64).T + (0.0 if down_b is None else np.asarray(down_b, F64))


def route(h, router, router_b, top):
    """(chosen [T, top], weights [T, top]): the `top` largest router logits of
    each token and the softmax over those alone."""
    z = np.asarray(h, F64) @ np.asarray(router, F64).T + np.asarray(router_b, F64)
    chosen = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    zc = np.take_along_axis(z, chosen, axis=-1)
    e = np.exp(zc - zc.max(axis=-1, keepdims=True))
    return chosen, e / e.sum(axis=-1, keepdims=True)


def expert_mixture(h, experts, router, router_b, top, chosen=None):
    """experts: list of (gate, up, down).  `chosen` [T, top], if given, replaces the
    router's choice (the weights are still the softmax over the chosen logits): a
    test follows an implementation's choices where two logits were too close to call."""
    h = np.asarray(h, F64)
    if chosen is None:
        chosen, weights = route(h, router, router_b, top)
    else:
        z = h @ np.asarray(router, F64).T + np.asarray(router_b, F64)
        zc = np.take_along_axis(z, np.asarray(chosen), axis=-1)
        e = np.exp(zc - zc.max(axis=-1, keepdims=True))
        weights = e / e.sum(axis=-1, keepdims=True)
    out = np.zeros((h.shape[0], np.asarray(experts[0][2]).shape[0]), F64)
    for t in range(h.shape[0]):
        for e, p in zip(chosen[t], weights[t]):
            gate, up, down = experts[int(e)]
            out[t] += p * gated_ff(h[t:t + 1], gate, up, down)[0]
    return out


# --------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------
def forward(config, weights, tokens, keep_layers=False, routing=None):
    """Logits [T, vocab] of one whole sequence (and, if asked, the hidden state
    after every layer [L, T, width]).  `routing`: {layer: chosen [T, top]} to use
    instead of the routers' own choices."""
    eps = float(config["norm"]["eps"])
    tokens = np.asarray(tokens)
    T = tokens.shape[0]
    positions = np.arange(T)
    x = np.asarray(weights["embed"], F64)[tokens]
    kept = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        m, p = layer["mixer"], f"l{i}."
        rot = m["rot"]
        freqs, amplitude = rotary_frequencies(int(rot["dims"]), float(rot["base"]), rot.get("scaling"))
        if m.get("kv_from") is None:
            kept[i] = latent_and_rotated_key(x, weights[p + "mix.dkv"], weights[p + "mix.dkv.norm"],
                                             int(m["kv_rank"]), eps, positions, freqs, amplitude)
            latent, key_rot = kept[i]
        else:
            latent, key_rot = kept[int(m["kv_from"])]
        w = {k: weights[p + "mix." + k] for k in ("q", "uk", "uv", "g", "o")}
        x = x + rms_norm(latent_attention(x, m, w, eps, latent, key_rot, positions, freqs, amplitude),
                         weights[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            if mlp["kind"] == "dense":
                y = gated_ff(x, weights[p + "mlp.gate"], weights[p + "mlp.up"], weights[p + "mlp.down"],
                             weights[p + "mlp.gate.b"], weights[p + "mlp.up.b"], weights[p + "mlp.down.b"])
            else:
                n, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                experts = [tuple(weights[f"{p}mlp.e{e}.{k}"] for k in ("gate", "up", "down")) for e in range(n)]
                y = expert_mixture(x, experts, weights[p + "mlp.router"], weights[p + "mlp.router.b"], top,
                                   None if routing is None else routing.get(i))
            x = x + rms_norm(y, weights[p + "norm2"], eps)
        if keep_layers:
            after.append(x.copy())
    logits = rms_norm(x, weights["final.norm"], eps) @ np.asarray(weights["head"], F64).T
    return (logits, np.stack(after)) if keep_layers else logits


def greedy(config, weights, prompt, n_new):
    """n_new tokens, each the first maximum of the logits after everything before it."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(np.argmax(forward(config, weights, seq)[-1])))
    return seq[len(prompt):]
