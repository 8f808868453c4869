"""The Ropovik design in the engine against its plain implementation
(plain_ropovik.py): every mechanism alone, then whole models of two small
configurations that differ in every size and option, under every way of
cutting the same requests into steps."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import go_tinygrad_b200 as lib
import plain_llama
import plain_ropovik as plain
from go_tinygrad_b200.cache import Cache
from go_tinygrad_b200.engine import Model, StepEntry, step
from go_tinygrad_b200.kernels import ops
from go_tinygrad_b200.parts import PartSpec, ResidualStream, Runtime, build_part, walk
from conftest import ROOT, assert_close
from test_parts_gpu import context

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda" if torch.cuda.is_available() and torch.cuda.device_count() else "cpu")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def attention_layer(heads, kv_heads, dim, scale, rot, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}}


def mamba_layer(heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                      "norm_groups": norm_groups}}


# P: a stretch in the middle runs three times; part of a head rotates, under yarn scaling; a head
# size the tiled attention kernels do not take (24); one group, one norm piece; two and three taps.
CONFIG_P = {
    "architecture": "Ropovik", "vocab": 211, "width": 64, "logit_softcap": 9.0, "norm": {"eps": 1e-4},
    "loop": {"start": 1, "stop": 4, "times": 3},
    "layers": [
        mamba_layer(4, 16, 16, 1, 3, 1, {"kind": "dense", "ff": 72}),
        attention_layer(4, 1, 32, 0.21, {"dims": 16, "base": 50.0, "scaling": {"factor": 3.0, "original": 24, "fast": 3.0, "slow": 0.5}},
                        {"kind": "dense", "ff": 96}),
        mamba_layer(6, 8, 24, 3, 2, 3, None),
        attention_layer(2, 2, 24, 0.3, None, None),
        attention_layer(3, 3, 16, 0.25, {"dims": 16, "base": 1000.0, "scaling": None}, {"kind": "dense", "ff": 40}),
    ],
}
# Q: no loop, no cap; whole heads of 64 rotate without scaling (the layout the decode attention
# rotates itself); state of 64, heads of 32, five taps; every layer with a feed-forward.
CONFIG_Q = {
    "architecture": "Ropovik", "vocab": 160, "width": 128, "logit_softcap": None, "norm": {"eps": 1e-6},
    "loop": None,
    "layers": [
        attention_layer(4, 2, 64, 0.125, {"dims": 64, "base": 10000.0, "scaling": None}, {"kind": "dense", "ff": 256}),
        mamba_layer(4, 32, 64, 2, 5, 4, {"kind": "dense", "ff": 128}),
        attention_layer(2, 1, 64, 0.11, {"dims": 64, "base": 300.0, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}},
                        {"kind": "dense", "ff": 64}),
    ],
}
CONFIGS = {"P": (CONFIG_P, 3, 0.15, 0.1), "Q": (CONFIG_Q, 4, 0.08, 0.05)}     # configuration, seed, std, norm std


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, seed, std, norm_std) in CONFIGS.items():
        folder = str(tmp_path_factory.mktemp(f"ropovik_{name}"))
        lib.write_random_model(folder, cfg, seed=seed, dtype="bfloat16", std=std, norm_std=norm_std)
        out[name] = folder
    return out


_models, _weights, _memo = {}, {}, {}


def get_model(folders, name, dtype):
    if (name, dtype) not in _models:
        _models[(name, dtype)] = Model.load(folders[name], dtype=dtype, device="cuda")
    return _models[(name, dtype)]


def weights_of(folders, name):
    if name not in _weights:
        _weights[name] = plain_llama.read_safetensors(os.path.join(folders[name], "model.safetensors"))
    return _weights[name]


def want_logits(folders, name, tokens):
    key = (name, tuple(tokens))
    if key not in _memo:
        _memo[key] = plain.forward(CONFIGS[name][0], weights_of(folders, name), list(tokens))
    return _memo[key]


def prompts_of(name, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, CONFIGS[name][0]["vocab"], n).tolist() for n in lengths]


def run_cut(model, cache, tokens, portions):
    """Feed `tokens` in portions of the given sizes (the last size repeats), logits everywhere."""
    slot = cache.open_sequence()
    out, at, i = [], 0, 0
    while at < len(tokens):
        n = min(portions[min(i, len(portions) - 1)], len(tokens) - at)
        out.append(step(model, cache, [StepEntry(slot, tokens[at:at + n], list(range(n)))]).float().cpu().numpy())
        at += n
        i += 1
    cache.close_sequence(slot)
    return np.concatenate(out)


# ---------------------------------------------------------------- mechanisms alone
def t32(a):
    return torch.tensor(np.asarray(a, np.float32), device=DEV)


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_with_pending_update_and_chosen_rows(dtype):
    rng = np.random.default_rng(0)
    for H in (24, 200, 1031):
        x, upd = rng.standard_normal((9, H)) * 3 + 1.5, rng.standard_normal((9, H))
        w, b = rng.standard_normal(H), rng.standard_normal(H)
        pend = t32(upd).to(TORCH[dtype])
        res, out = t32(x), torch.empty(9, H, dtype=TORCH[dtype], device=DEV)
        ops.add_layernorm(res, pend, t32(w), t32(b), 1e-3, out)
        summed = np.asarray(x, np.float32) + pend.float().cpu().numpy()
        np.testing.assert_array_equal(res.cpu().numpy(), summed)
        want = plain.layer_norm(summed, np.float32(w), np.float32(b), 1e-3)
        lim = 2e-5 if dtype == "float32" else 2e-2
        assert np.abs(out.float().cpu().numpy() - want).max() <= lim * np.abs(want).max()
        rows = i32([7, 0, 7])
        out3 = torch.empty(3, H, dtype=TORCH[dtype], device=DEV)
        ops.add_layernorm(res, None, t32(w), None, 1e-3, out3, rows)
        want3 = plain.layer_norm(summed[[7, 0, 7]], np.float32(w), 0.0, 1e-3)
        assert np.abs(out3.float().cpu().numpy() - want3).max() <= lim * np.abs(want3).max()


def test_rotary_table_under_yarn_scaling():
    rt = Runtime(DEV, torch.float32)
    for dims, base, scaling in ((16, 50.0, {"factor": 3.0, "original": 24, "fast": 3.0, "slow": 0.5}),
                                (64, 10000.0, {"factor": 4.0, "original": 512, "fast": 32.0, "slow": 1.0}),
                                (8, 7.0, {"factor": 2.0, "original": 5, "fast": 1.0, "slow": 1.0}),     # lo == hi: a step
                                (32, 100.0, None)):
        spec = PartSpec("rotary", {"head_dim": 2 * dims, "rotary_dim": dims, "theta": base,
                                   "scaling": dict(scaling, rope_type="yarn") if scaling else None})
        pos = build_part("position", spec)
        pos.load({}, rt)
        positions = [0, 1, 2, 63, 64, 700, 5000]
        ctx = context(rt, [len(positions)], [0], [0])
        ctx.positions = i32(positions)
        table = pos.rotation(ctx).cpu().numpy()
        freqs, amp = plain.rotary_frequencies(dims, base, scaling)
        ang = np.array(positions, np.float64)[:, None] * freqs[None, :]
        np.testing.assert_allclose(table[..., 0], np.cos(ang) * amp, rtol=0, atol=2e-7 * amp)
        np.testing.assert_allclose(table[..., 1], np.sin(ang) * amp, rtol=0, atol=2e-7 * amp)
        if scaling:
            assert amp > 1.0 and not np.allclose(freqs, plain.rotary_frequencies(dims, base, None)[0])


@pytest.mark.parametrize("dtype", DTYPES)
def test_convolution_carries_its_last_inputs_across_portions(dtype):
    rng = np.random.default_rng(1)
    for C, taps in ((40, 4), (130, 2), (16, 1), (24, 6), (48, 4), (64, 3), (32, 2)):
        T = 37
        x = t32(rng.standard_normal((2 * T, C))).to(TORCH[dtype])
        w, b = np.float32(rng.standard_normal((C, taps))), np.float32(rng.standard_normal(C))
        xs = x.float().cpu().numpy()
        want = np.concatenate([plain.silu(plain.causal_conv(xs[:T], w, b)), plain.silu(plain.causal_conv(xs[T:], w, b))])
        state = torch.zeros(5, max(taps - 1, 0), C, device=DEV)
        state[1] = 99.0                                    # a slot nobody uses stays as it is
        got = torch.zeros(2 * T, C, dtype=TORCH[dtype], device=DEV)
        # two sequences in slots 3 and 0, cut into portions of 1, 2, 5, 1, ... tokens
        at = 0
        for n in (1, 2, 5, 1, 1, 3, 24):
            rows = list(range(at, at + n)) + list(range(T + at, T + at + n))
            xin, out = x[rows].contiguous(), torch.empty(2 * n, C, dtype=TORCH[dtype], device=DEV)
            seq, cu, slots = i32([0] * n + [1] * n), i32([0, n, 2 * n]), i32([3, 0])
            if n == 1:                                      # one token each: convolution and state in one kernel
                ops.causal_conv_silu(xin, t32(w.T.copy()), t32(b), state, out, seq, cu, slots, update_state=True, one_token_each=True)
            else:
                ops.causal_conv_silu(xin, t32(w.T.copy()), t32(b), state, out, seq, cu, slots)
                ops.conv_state_update(xin, state, cu, slots, 2)
            got[rows] = out
            at += n
        lim = 1e-5 if dtype == "float32" else 1e-2
        assert np.abs(got.float().cpu().numpy() - want).max() <= lim * max(1.0, np.abs(want).max())
        # both sequences whole in one step (a prompt-sized step: a thread walks a run of tokens, and the
        # second sequence begins inside a run)
        whole = torch.empty(2 * T, C, dtype=TORCH[dtype], device=DEV)
        ops.causal_conv_silu(x, t32(w.T.copy()), t32(b), torch.zeros(5, max(taps - 1, 0), C, device=DEV), whole,
                             i32([0] * T + [1] * T), i32([0, T, 2 * T]), i32([3, 0]))
        assert np.abs(whole.float().cpu().numpy() - want).max() <= lim * max(1.0, np.abs(want).max())
        if C % 4 == 0:                                     # the last half of the channels as float pairs (U_q, V_q)
            q, n_all = C // 4, 2 * T
            plain_out = torch.empty(n_all, C - 2 * q, dtype=TORCH[dtype], device=DEV)
            pairs = torch.empty(n_all, q, 2, device=DEV)
            fresh = torch.zeros(5, max(taps - 1, 0), C, device=DEV)
            ops.causal_conv_silu(x, t32(w.T.copy()), t32(b), fresh, plain_out, i32([0] * T + [1] * T), i32([0, T, 2 * T]),
                                 i32([3, 0]), pairs=pairs)
            got_pairs = pairs.cpu().numpy()
            assert np.abs(plain_out.float().cpu().numpy() - want[:, :C - 2 * q]).max() <= lim * max(1.0, np.abs(want).max())
            assert np.abs(got_pairs[:, :, 0] - want[:, C - 2 * q:C - q]).max() <= 1e-5 * max(1.0, np.abs(want).max())
            assert np.abs(got_pairs[:, :, 1] - want[:, C - q:]).max() <= 1e-5 * max(1.0, np.abs(want).max())
        if taps > 1:
            np.testing.assert_array_equal(state[3].cpu().numpy(), xs[T - taps + 1:T])
            np.testing.assert_array_equal(state[0].cpu().numpy(), xs[2 * T - taps + 1:])
            assert (state[1] == 99.0).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,groups,N,P", [(4, 2, 16, 8), (3, 1, 40, 24), (2, 2, 128, 64), (6, 3, 24, 5), (1, 1, 7, 3)])
def test_recurrence_keeps_its_state_across_portions_and_remembers_far_tokens(dtype, heads, groups, N, P):
    rng = np.random.default_rng(2)
    T, inner = 150, heads * P
    xbc = t32(rng.standard_normal((T, inner + 2 * groups * N))).to(TORCH[dtype])
    dt_raw = t32(rng.standard_normal((T, heads))).to(TORCH[dtype])
    dt_bias = np.float32(rng.standard_normal(heads) - 1.0)
    a_log = np.float32(rng.standard_normal(heads))
    a_log[0] = -9.0                                        # head 0 forgets almost nothing: token 0 is felt at token 149
    skip = np.float32(rng.standard_normal(heads))
    xs, ds = xbc.float().cpu().numpy().astype(np.float64), dt_raw.float().cpu().numpy().astype(np.float64)
    xs[0, :P] *= 30.0                                      # ... and token 0 of head 0 stands out
    xbc[0, :P] = t32(xs[0, :P]).to(TORCH[dtype])
    xs = xbc.float().cpu().numpy().astype(np.float64)
    want = plain.selective_scan(xs[:, :inner].reshape(T, heads, P), plain.softplus(ds + dt_bias), a_log,
                                xs[:, inner:inner + groups * N].reshape(T, groups, N),
                                xs[:, inner + groups * N:].reshape(T, groups, N), skip).reshape(T, inner)
    forgot = plain.selective_scan(xs[1:, :inner].reshape(T - 1, heads, P), plain.softplus(ds[1:] + dt_bias), a_log,
                                  xs[1:, inner:inner + groups * N].reshape(T - 1, groups, N),
                                  xs[1:, inner + groups * N:].reshape(T - 1, groups, N), skip).reshape(T - 1, inner)
    assert np.abs(want[-1, :P] - forgot[-1, :P]).max() > 0.05 * np.abs(want[-1, :P]).max()   # the test can see token 0
    x_in = xbc[:, :inner].contiguous()
    bc_in = torch.stack([xbc[:, inner:inner + groups * N], xbc[:, inner + groups * N:]], dim=2).float().contiguous()
    for portions in ([T], [1], [15, 16, 17, 1, 2, 33], [100, 1]):
        state = torch.zeros(3, heads, N, P, device=DEV)
        got = torch.zeros(T, inner, device=DEV)
        at, i = 0, 0
        while at < T:
            n = min(portions[min(i, len(portions) - 1)], T - at)
            y = torch.empty(n, inner, device=DEV)
            ops.ssm_scan(x_in[at:at + n], bc_in[at:at + n], dt_raw[at:at + n], t32(dt_bias), t32(a_log), t32(skip), state, y,
                         i32([0, n]), i32([2]), 1, heads, groups, N, P, one_token_each=(n == 1 and portions != [1]))
            got[at:at + n] = y
            at += n
            i += 1
        assert np.abs(got.cpu().numpy() - want).max() <= 2e-5 * np.abs(want).max(), portions
        assert (state[:2] == 0).all()


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_then_norm_in_pieces(dtype):
    rng = np.random.default_rng(3)
    for width, parts in ((48, 1), (48, 3), (640, 2), (96, 96), (1024, 2), (768, 3), (2048, 1)):
        y, z, w = rng.standard_normal((7, width)) * 4, rng.standard_normal((7, width)), rng.standard_normal(width)
        zt = t32(z).to(TORCH[dtype])
        out = torch.empty(7, width, dtype=TORCH[dtype], device=DEV)
        ops.gated_rmsnorm(t32(y), zt, t32(w), 1e-3, out, parts)
        gated = np.float32(y).astype(np.float64) * plain.silu(zt.float().cpu().numpy().astype(np.float64))
        want = plain.rms_norm_parts(gated, np.float32(w), parts, 1e-3)
        lim = 2e-5 if dtype == "float32" else 2e-2
        assert np.abs(out.float().cpu().numpy() - want).max() <= lim * np.abs(want).max()
        if parts == 3:                                    # the gate comes before the norm, not after it
            after = plain.rms_norm_parts(np.float32(y), np.float32(w), parts, 1e-3) * plain.silu(z)
            assert np.abs(after - want).max() > 0.1


@pytest.mark.parametrize("dtype", DTYPES)
def test_activations_cap_and_the_projection_beside_a_kept_tensor(dtype):
    rng = np.random.default_rng(4)
    x = rng.standard_normal((5, 33)) * 3
    for kind, fn in (("relu2", plain.relu_squared), ("silu", plain.silu),
                     ("gelu_tanh", lambda v: 0.5 * v * (1 + np.tanh(np.sqrt(2 / np.pi) * (v + 0.044715 * v ** 3))))):
        t = t32(x).to(TORCH[dtype])
        want = fn(t.float().cpu().numpy().astype(np.float64))
        ops.activation(t, kind)
        lim = 1e-6 if dtype == "float32" else 1e-2
        assert np.abs(t.float().cpu().numpy() - want).max() <= lim * np.abs(want).max()
    logits = t32(x * 10)
    ops.softcap(logits, 7.5)
    np.testing.assert_allclose(logits.cpu().numpy(), plain.soft_cap(np.float32(x * 10).astype(np.float64), 7.5), rtol=2e-6, atol=1e-6)
    # x <- W [x + pending | kept]
    H = 24
    rt = Runtime(DEV, TORCH[dtype])
    block = build_part("block", PartSpec("concat_projection", {"hidden_size": H, "weight": "w"}))
    w = t32(rng.standard_normal((H, 2 * H)) * 0.3).to(torch.bfloat16)
    block.load({"w": w.cpu()}, rt)
    res, pend, kept = rng.standard_normal((6, H)), rng.standard_normal((6, H)), rng.standard_normal((6, H))
    pend_t = t32(pend).to(TORCH[dtype])
    ctx = context(rt, [6], [0], [0])
    ctx.shared["embedding_output"] = t32(kept)
    stream = ResidualStream(t32(res), pend_t)
    block.forward(stream, ctx, None)
    assert stream.pending is None
    want = plain.loop_input(np.float32(res) + pend_t.float().cpu().numpy(), np.float32(kept), w.float().cpu().numpy())
    lim = 2e-5 if dtype == "float32" else 2e-2
    assert np.abs(stream.residual.cpu().numpy() - want).max() <= lim * np.abs(want).max()
    with pytest.raises(ValueError):
        block.forward(stream, context(rt, [6], [0], [0]), None)      # nothing was kept in that step


@pytest.mark.parametrize("rows", [3, 16, 40, 128, 300])
def test_activation_in_the_epilogue_of_every_product(rows):
    """The dense feed-forward's activation applied to the float sums inside the product (one kernel per
    range of row counts), against the product followed by the activation kernel and against float64."""
    rng = np.random.default_rng(rows)
    for K, N in ((64, 72), (256, 1000)):
        x = t32(rng.standard_normal((rows, K))).to(torch.bfloat16)
        w = t32(rng.standard_normal((N, K)) * 0.2).to(torch.bfloat16)
        ref = x.float().cpu().numpy().astype(np.float64) @ w.float().cpu().numpy().astype(np.float64).T
        for kind, fn in (("relu2", plain.relu_squared), ("silu", plain.silu),
                         ("gelu_tanh", lambda v: 0.5 * v * (1 + np.tanh(np.sqrt(2 / np.pi) * (v + 0.044715 * v ** 3))))):
            fused = torch.empty(rows, N, dtype=torch.bfloat16, device=DEV)
            ops.linear(x, w, fused, epilogue=kind)
            want = fn(ref)
            assert np.abs(fused.float().cpu().numpy() - want).max() <= 1e-2 * max(1.0, np.abs(want).max()), (kind, K, N)
    # float32 and unaligned operands take the product and then the activation kernel: same answer
    x32, w32 = t32(rng.standard_normal((rows, 20))), t32(rng.standard_normal((9, 20)))
    out = torch.empty(rows, 9, device=DEV)
    ops.linear(x32, w32, out, epilogue="relu2")
    want = plain.relu_squared(x32.cpu().numpy().astype(np.float64) @ w32.cpu().numpy().astype(np.float64).T)
    assert np.abs(out.cpu().numpy() - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


def _attention_part(dtype, heads, kv_heads, dim, rot, scale, hidden, wq, wk, wo):
    position = PartSpec("none", {}) if rot is None else PartSpec("rotary", {
        "head_dim": dim, "rotary_dim": rot["dims"], "theta": rot["base"],
        "scaling": dict(rot["scaling"], rope_type="yarn") if rot.get("scaling") else None})
    spec = PartSpec("gqa_attention", {"hidden_size": hidden, "n_heads": heads, "n_kv_heads": kv_heads, "head_dim": dim,
                                      "scale": scale, "position": position, "values": "keys", "q": "q", "k": "k", "o": "o"})
    rt = Runtime(DEV, TORCH[dtype])
    mixer = build_part("mixer", spec)
    assert [s.name for s in mixer.weight_specs()] == ["q", "k", "o"]           # no value projection
    for part in walk(mixer):
        part.load({"q": wq, "k": wk, "o": wo}, rt)
    return rt, mixer


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dim,rot", [(32, {"dims": 8, "base": 100.0, "scaling": {"factor": 4.0, "original": 16, "fast": 2.0, "slow": 1.0}}),
                                     (64, {"dims": 64, "base": 10000.0}), (24, None), (96, {"dims": 48, "base": 500.0})])
@pytest.mark.parametrize("needle", [0, 3, 63, 64, 65, 127, 128, 290])
def test_attention_finds_one_far_key_and_returns_its_unrotated_key(dtype, dim, rot, needle):
    """One key among 300 is made to stand out for the last query, through channels
    that do not rotate where there are some.  Its value is the key as projected:
    with an identity output projection the mixer's answer is that key itself."""
    if needle % 64 not in (0, 63) and (dim, needle) not in ((32, 3), (64, 65), (24, 290), (96, 290), (64, 290)):
        pytest.skip("one head size per place away from a page border")
    heads, kv_heads, T = 2, 1, 300
    hidden = heads * dim
    rng = np.random.default_rng(needle)
    eye, none = torch.eye(dim), torch.zeros(dim, dim)
    wq = torch.cat([torch.cat([none, eye], dim=1)] * heads).to(torch.bfloat16)      # queries read channels dim..2dim-1
    wk = torch.cat([eye, none], dim=1).to(torch.bfloat16)                            # keys read channels 0..dim-1
    wo = torch.eye(hidden).to(torch.bfloat16)
    x = rng.standard_normal((T, hidden)) * 0.1
    # the marked channel does not rotate; where every channel does, it is the slowest pair's
    # (300 positions turn it by a few hundredths of a radian)
    mark = dim - 1 if (rot is None or rot["dims"] < dim) else dim // 2 - 1
    x[needle, mark] = 9.0                                   # the key that stands out ...
    x[needle, 1] = 5.0                                      # ... whose value differs from every other
    x[-1, dim + mark] = 9.0                                 # the last query asks for it
    xt = t32(x).to(TORCH[dtype])
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "scale": 1.0, "rot": rot}
    w64 = lambda t: t.float().numpy().astype(np.float64)
    want = plain.attention_mixer(xt.float().cpu().numpy().astype(np.float64), w64(wq), w64(wk), w64(wo), m)
    rt, mixer = _attention_part(dtype, heads, kv_heads, dim, rot, 1.0, hidden, wq, wk, wo)
    lim = 1e-4 if dtype == "float32" else 3e-2
    for cut in (T, T - 1, T - 40):                            # the last query in the prompt, alone, and after 39 decoded tokens
        cache = Cache([mixer.cache_requests()], [None], max_tokens=64 * 6, max_slots=2, dtype=TORCH[dtype], device=DEV)
        cache.open_sequence()
        slot = cache.open_sequence()
        at, got = 0, []
        for n in [cut] + [1] * (T - cut):
            cache.reserve_many([(slot, at + n)]); cache.flush_tables()
            ctx = context(rt, [n], [at], [slot])
            ctx.total_kv_len = at + n
            got.append(mixer.forward(xt[at:at + n].contiguous(), ctx, cache.handles[0]).float().cpu().numpy())
            cache.advance(slot, n)
            at += n
        got = np.concatenate(got)
        assert np.abs(got - want).max() <= lim * max(1.0, np.abs(want).max()), (cut, np.abs(got - want).argmax())
    # the answer at the last place is the needle's key as projected, not its rotated form
    key = xt[needle, :dim].float().cpu().numpy()
    assert np.abs(want[-1, :dim] - key).max() < 0.02 and np.abs(got[-1, :dim] - key).max() < (1e-3 if dtype == "float32" else 0.1)


# ------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_whole_prompts_of_many_lengths(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    for p in prompts_of(name, [1, 2, 3, 17, 63, 64, 65, 129, 230]):
        got = run_cut(model, cache, p, [len(p)])
        assert_close(got, want_logits(folders, name, p), dtype, f"{name} {dtype} whole prompt of {len(p)}")
    assert cache.open_slots() == []


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_portions_down_to_two_tokens_and_token_by_token_from_the_start(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    p = prompts_of(name, [150], seed=5)[0]
    want = want_logits(folders, name, p)
    rows = {}
    for portions in ([150], [1], [2], [3, 2, 1, 16, 15, 17, 64], [63, 1, 1, 64, 2], [100, 1]):
        rows[tuple(portions)] = run_cut(model, cache, p, portions)
        assert_close(rows[tuple(portions)], want, dtype, f"{name} {dtype} portions {portions}")
    if dtype == "float32":
        # sums walk keys and tokens in one order whatever the cut: the float32 answers agree to the last bits
        for portions, got in rows.items():
            np.testing.assert_allclose(got, rows[(150,)], rtol=0, atol=2e-5 * np.abs(want).max(), err_msg=str(portions))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_long_decoding_across_page_borders(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 6)
    p = prompts_of(name, [5 + 280], seed=6)[0]
    got = run_cut(model, cache, p, [5, 1])
    assert_close(got, want_logits(folders, name, p), dtype, f"{name} {dtype} 280 tokens decoded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_unequal_batches_against_each_alone_with_slots_and_pages_used_again(folders, name, dtype):
    """Three batches through a cache too small for two of them: the slots and pages
    of finished requests, with their old keys and states, go to new ones.  In a
    batch every request is decoded to its own length and leaves when it ends."""
    model = get_model(folders, name, dtype)
    cache = model.new_cache(max_tokens=64 * 7, max_slots=4)
    batches = [[(5, 9), (70, 3), (17, 20), (1, 12)], [(64, 1), (130, 6), (3, 33)], [(40, 8), (128, 2), (9, 9), (2, 2)]]
    for bi, batch in enumerate(batches):
        prompts = prompts_of(name, [a + b for a, b in batch], seed=20 + bi)
        want = [want_logits(folders, name, p) for p in prompts]
        slots = [cache.open_sequence() for _ in batch]
        got = [[] for _ in batch]
        entries = [StepEntry(slots[i], p[:plen], list(range(plen))) for i, ((plen, _), p) in enumerate(zip(batch, prompts))]
        flat = step(model, cache, entries).float().cpu().numpy()
        o = 0
        for i, e in enumerate(entries):
            got[i].append(flat[o:o + len(e.want)])
            o += len(e.want)
        live, t = list(range(len(batch))), 0
        while True:
            live = [i for i in live if t < batch[i][1]]
            if not live:
                break
            flat = step(model, cache, [StepEntry(slots[i], [prompts[i][batch[i][0] + t]], [0]) for i in live]).float().cpu().numpy()
            for j, i in enumerate(live):
                got[i].append(flat[j:j + 1])
                if t + 1 >= batch[i][1]:
                    cache.close_sequence(slots[i])
            t += 1
        for i in range(len(batch)):
            assert_close(np.concatenate(got[i]), want[i], dtype, f"{name} {dtype} batch {bi} request {i}")
        assert cache.open_slots() == []
    assert cache.free_pages() == [7] * len(cache.free_pages())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype):
    model = get_model(folders, name, dtype)
    prompts = prompts_of(name, [5, 17, 40, 1], seed=7)
    cfg, w = CONFIGS[name][0], weights_of(folders, name)
    for use_graph in (True, False):
        results = lib.generate(model, prompts, [12, 6, 9, 12], stop=[], use_graph=use_graph)
        assert [len(r.tokens) for r in results] == [12, 6, 9, 12]
        for p, r in zip(prompts, results):
            seq = list(p)
            for tok in r.tokens:                          # each token is one the plain model could have chosen there
                logits = plain.forward(cfg, w, seq)[-1]
                slack = (1e-4 if dtype == "float32" else 5e-2) * max(1.0, np.abs(logits).max())
                assert logits[tok] >= logits.max() - slack
                seq.append(tok)
    if dtype == "float32":
        assert results[1].tokens == plain.greedy(cfg, w, prompts[1], 6)


def test_trace_replay_and_command_line(folders, tmp_path):
    """bin/trace_run with a batch that starts together and shrinks, and llmgen with token ids."""
    name = "P"
    a, b = prompts_of(name, [30, 9], seed=8)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": a[:20], "want": [0, 19]}, {"id": "y", "tokens": b[:7], "want": [6]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": a[20:21], "want": [0]}, {"id": "y", "tokens": b[7:8], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "x", "tokens": a[21:22], "want": []}, {"id": "y", "tokens": b[8:9], "want": [0]}], "end": ["y"]},
             {"step": 3, "entries": [{"id": "x", "tokens": a[22:], "want": [7]}], "end": ["x"]}]
    out = str(tmp_path / "out")
    proc = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders[name], "--dtype", "float32",
                           "--out", out, "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    wa, wb = want_logits(folders, name, a), want_logits(folders, name, b)
    V = CONFIGS[name][0]["vocab"]
    read = lambda i: np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, V)
    assert_close(read(0), np.stack([wa[0], wa[19], wb[6]]), "float32", "step 0")
    assert_close(read(1), wa[20:21], "float32", "step 1")
    assert_close(read(2), wb[8:9], "float32", "step 2")
    assert_close(read(3), wa[29:30], "float32", "step 3")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "llmgen"), "-model", folders[name], "-ids",
                           ",".join(str(t) for t in b), "-tokens", "5", "-dtype", "float32"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    want = plain.greedy(CONFIGS[name][0], weights_of(folders, name), b, 5)
    assert " ".join(str(t) for t in want) in proc.stdout.replace(",", " ").replace("[", " ").replace("]", " ")
