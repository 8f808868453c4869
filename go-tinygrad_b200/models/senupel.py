"""The Senupel decoder as a plan of parts.

Every layer is an ``output_norm`` block (x += rmsnorm(sublayer(x)) w; the
sublayers read x itself) around attention through a latent
(``latent_attention``: a normed latent and one shared rotated key part per
token in the cache, interleaved rotary pairs under yarn scaling, a causal
window, a sigmoid gate on the heads) and a gated silu feed-forward with biases
(``swiglu``) or a mixture of such experts without biases (``routed_experts``).
A layer with ``kv_from`` has no down projection: its schedule entry reads the
cache of the named layer's entry.  A final RMS norm and the head close the
model.  Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``,
``l<i>.mix.q|dkv|dkv.norm|uk|uv|g|o``, ``l<i>.mlp.gate|up|down[.b]``,
``l<i>.mlp.router[.b]``, ``l<i>.mlp.e<j>.gate|up|down``, ``final.norm``,
``head``.  The reference has no such architecture.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.senupel import DenseMlp, SenupelConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


def _norm(cfg: SenupelConfig, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name})


def _mixer(cfg: SenupelConfig, i: int) -> PartSpec:
    m, p = cfg.layers[i].mixer, f"l{i}.mix."
    scaling = dict(m.rot.scaling.to_json(), rope_type="yarn") if m.rot.scaling else None
    position = PartSpec("rotary", {"head_dim": m.rot_dim, "rotary_dim": m.rot.dims, "theta": m.rot.base,
                                   "scaling": scaling, "pairing": "interleaved"})
    return PartSpec("latent_attention", {
        "hidden_size": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_dim": m.vdim,
        "kv_rank": m.kv_rank, "window": m.window, "scale": m.scale, "eps": cfg.norm_eps, "position": position,
        "own_kv": m.kv_from is None, "q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm",
        "uk": p + "uk", "uv": p + "uv", "gate": p + "g", "o": p + "o"})


def _feed_forward(cfg: SenupelConfig, i: int) -> PartSpec:
    mlp, p = cfg.layers[i].mlp, f"l{i}.mlp."
    if isinstance(mlp, DenseMlp):
        return PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": mlp.ff,
                                   "gate": p + "gate", "up": p + "up", "down": p + "down",
                                   "gate_bias": p + "gate.b", "up_bias": p + "up.b", "down_bias": p + "down.b"})
    return PartSpec("routed_experts", {"hidden_size": cfg.width, "intermediate_size": mlp.ff,
                                       "n_experts": mlp.experts, "top": mlp.top,
                                       "router": p + "router", "router_bias": p + "router.b",
                                       "gate": p + "e{e}.gate", "up": p + "e{e}.up", "down": p + "e{e}.down"})


def senupel_plan(cfg: SenupelConfig) -> ModelPlan:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, i),
                 "feed_forward_norm": None, "feed_forward": None}
        if layer.mlp is not None:
            parts["feed_forward_norm"] = _norm(cfg, p + "norm2")
            parts["feed_forward"] = _feed_forward(cfg, i)
        layers.append(LayerSpec(PartSpec("output_norm", parts)))
    # one schedule entry per layer, in order: a layer's index is its entry's
    schedule = tuple(ScheduleEntry(layer=i, cache=layer.mixer.kv_from) for i, layer in enumerate(cfg.layers))
    plan = ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed"}),
        layers=tuple(layers),
        schedule=schedule,
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "head"}),
        stop_tokens=(),
        max_position=None,
    )
    plan.check()
    return plan


SENUPEL = register_architecture(Architecture(
    names=("Senupel", "senupel"),
    read_config=SenupelConfig.from_json,
    plan=senupel_plan,
))
