"""Recurrent mixers: per-sequence state of fixed size instead of keys and values.

``mamba2``: the state-space mixer with a scalar decay per head.  With
inner = n_heads * head_dim, N = state_size, G = n_groups, the input projection
gives [z: inner | x: inner | B: G*N | C: G*N | dt: n_heads] per token.  x, B and
C pass a causal convolution over the last `conv_taps` tokens, per channel, and
silu.  Per head h (which reads B and C of group h // (n_heads / G)):

    dt_t = softplus(dt_t + dt_bias[h])
    S_t  = exp(-exp(a_log[h]) dt_t) S_{t-1} + dt_t B_t x_t^T        (S: N x head_dim)
    y_t  = S_t^T C_t + d[h] x_t

then y * silu(z), an RMS norm over `norm_parts` equal pieces of the row (each
piece by its own root mean square) with a weight, and the output projection.
What a sequence keeps between steps is S (float32) and the last
conv_taps - 1 inputs of the convolution; both live in the cache as
`StateRequest`s, are zero when a slot is opened, and are read and left by
every step, so a prompt, a portion of one and a single token are one code path.
Step sizes, decays, the state, the recurrence's sums and the norm are float32
in both compute dtypes, and so are B and C from the convolution on; the
projections and the x the convolution leaves are in the compute dtype.  The reference has no recurrent mixer.

Parameters: ``hidden_size``, ``n_heads``, ``head_dim``, ``state_size``,
``n_groups``, ``conv_taps``, ``norm_parts``, ``eps`` and the tensor names
``in``, ``conv``, ``conv_bias``, ``dt_bias``, ``a_log``, ``d``, ``norm``, ``o``.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..cache import CacheHandle, Request, StateRequest
from ..kernels import ops
from ..weights.binder import WeightSpec
from .base import Mixer, Runtime, StepContext, emit_update, register_part


@register_part("mixer", "mamba2")
class Mamba2(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(self.param("hidden_size"))
        self.n_heads = int(self.param("n_heads"))
        self.head_dim = int(self.param("head_dim"))
        self.n_state = int(self.param("state_size"))
        self.n_groups = int(self.param("n_groups"))
        self.taps = int(self.param("conv_taps"))
        self.norm_parts = int(self.p.get("norm_parts") or 1)
        self.eps = float(self.param("eps"))
        if self.n_heads % self.n_groups:
            raise ValueError(f"{self.n_heads} heads cannot share {self.n_groups} groups of B and C")
        self.inner = self.n_heads * self.head_dim
        if self.inner % self.norm_parts:
            raise ValueError(f"a row of {self.inner} cannot be normed in {self.norm_parts} equal pieces")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.conv_dim = self.inner + 2 * self.n_groups * self.n_state
        self.proj_dim = self.inner + self.conv_dim + self.n_heads
        self.names = {k: str(self.param(k)) for k in ("in", "conv", "conv_bias", "dt_bias", "a_log", "d", "norm", "o")}
        self.w_in: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        n = self.names
        return [WeightSpec(n["in"], (self.proj_dim, self.hidden)),
                WeightSpec(n["conv"], (self.conv_dim, self.taps), role="parameter", std=0.3),
                WeightSpec(n["conv_bias"], (self.conv_dim,), role="parameter", std=0.1),
                WeightSpec(n["dt_bias"], (self.n_heads,), role="parameter", mean=-1.5, std=0.7),
                WeightSpec(n["a_log"], (self.n_heads,), role="parameter", mean=-0.5, std=0.7),
                WeightSpec(n["d"], (self.n_heads,), role="parameter", mean=1.0, std=0.3),
                WeightSpec(n["norm"], (self.inner,), role="vector", mean=1.0),
                WeightSpec(n["o"], (self.hidden, self.inner))]

    def cache_requests(self) -> List[Request]:
        return [StateRequest("ssm", (self.n_heads, self.n_state, self.head_dim), "float32"),
                StateRequest("conv", (self.taps - 1, self.conv_dim), "float32")]

    def load(self, tensors: Mapping[str, torch.Tensor], rt: Runtime) -> None:
        n = self.names
        self.w_in = rt.matrix(tensors[n["in"]])
        self.w_o = rt.matrix(tensors[n["o"]])
        self.conv_w = rt.vector(tensors[n["conv"]].t().contiguous())      # tap by tap: [taps, channels]
        self.conv_b = rt.vector(tensors[n["conv_bias"]])
        self.dt_bias = rt.vector(tensors[n["dt_bias"]])
        self.a_log = rt.vector(tensors[n["a_log"]])
        self.d = rt.vector(tensors[n["d"]])
        self.norm_w = rt.vector(tensors[n["norm"]])

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheHandle) -> torch.Tensor:
        rt = ctx.rt
        n = x.shape[0]
        if not cache.writes:
            raise ValueError("a recurrent mixer cannot read another run's state: every run advances its own")
        # rows padded to a multiple of 8 elements, which the products' stores want
        proj = rt.empty(n, (self.proj_dim + 7) // 8 * 8)[:, : self.proj_dim]
        ops.linear(x, self.w_in, proj)
        z = proj[:, : self.inner]
        conv_in = proj[:, self.inner: self.inner + self.conv_dim]
        dt_raw = proj[:, self.inner + self.conv_dim:]
        conv_state, ssm_state = cache.state("conv"), cache.state("ssm")
        # x in the compute dtype; B and C as float pairs, the form the recurrence reads
        xs = rt.empty(n, self.inner)
        bc = rt.empty(n, self.n_groups * self.n_state, 2, dtype=torch.float32)
        ops.causal_conv_silu(conv_in, self.conv_w, self.conv_b, conv_state, xs,
                             ctx.token_seq, ctx.cu_seqlens, ctx.slots, n_seqs=ctx.n_seqs, update_state=True,
                             one_token_each=ctx.is_decode, pairs=bc)
        ctx.trace("conv", xs)
        y = rt.empty(n, self.inner, dtype=torch.float32)
        ops.ssm_scan(xs, bc, dt_raw, self.dt_bias, self.a_log, self.d, ssm_state, y, ctx.cu_seqlens, ctx.slots,
                     ctx.n_seqs, self.n_heads, self.n_groups, self.n_state, self.head_dim,
                     one_token_each=ctx.is_decode)
        ctx.trace("scan", y)
        gated = rt.empty(n, self.inner)
        ops.gated_rmsnorm(y, z, self.norm_w, self.eps, gated, self.norm_parts)
        ctx.trace("attn", gated)
        return emit_update(gated, self.w_o, ctx)
