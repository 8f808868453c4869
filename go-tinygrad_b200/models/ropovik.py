"""The Ropovik decoder as a plan of parts.

Its layers differ one from the next: each is a pre-norm block (layer norms with
bias) around either attention whose values are the unrotated keys, with
partial rotary positions under yarn scaling, or a Mamba-2 recurrence; a dense
squared-relu feed-forward follows where the layer has one.  A stretch of
layers may run several times with the same weights; every pass has cache and
state of its own (one schedule entry per run) and is entered through a
projection of the hidden state beside the embedding output (the
``concat_projection`` block, one more layer of the plan that the schedule names
once per pass).  The final layer norm, the head and a soft cap on the logits
close the model.  Tensor names: ``embed``, ``loop.in``, ``l<i>.norm1[.b]``,
``l<i>.norm2[.b]``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``final.norm[.b]``,
``head``.  The reference has no such architecture.
"""
from __future__ import annotations

from ..config.registry import Architecture, register_architecture
from ..config.ropovik import RopovikConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry


def _norm(cfg: RopovikConfig, name: str) -> PartSpec:
    return PartSpec("layernorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight": name, "bias": name + ".b"})


def _mixer(cfg: RopovikConfig, i: int) -> PartSpec:
    layer, p = cfg.layers[i], f"l{i}.mix."
    m = layer.mixer
    if layer.type == "attention":
        if m.rot is None:
            position = PartSpec("none", {})
        else:
            scaling = dict(m.rot.scaling.to_json(), rope_type="yarn") if m.rot.scaling else None
            position = PartSpec("rotary", {"head_dim": m.dim, "rotary_dim": m.rot.dims, "theta": m.rot.base,
                                           "scaling": scaling, "pairing": "half"})
        return PartSpec("gqa_attention", {
            "hidden_size": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
            "window": None, "scale": m.scale, "position": position, "values": "keys",
            "q": p + "q", "k": p + "k", "o": p + "o"})
    return PartSpec("mamba2", {
        "hidden_size": cfg.width, "n_heads": m.heads, "head_dim": m.vdim, "state_size": m.state,
        "n_groups": m.groups, "conv_taps": m.conv, "norm_parts": m.norm_groups, "eps": cfg.norm_eps,
        "in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
        "a_log": p + "A_log", "d": p + "D", "norm": p + "norm", "o": p + "o"})


def ropovik_plan(cfg: RopovikConfig) -> ModelPlan:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": _norm(cfg, p + "norm1"), "mixer": _mixer(cfg, i),
                 "feed_forward_norm": None, "feed_forward": None}
        if layer.mlp is not None:
            parts["feed_forward_norm"] = _norm(cfg, p + "norm2")
            parts["feed_forward"] = PartSpec("dense", {
                "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "relu2",
                "up": p + "mlp.up", "down": p + "mlp.down"})
        layers.append(LayerSpec(PartSpec("pre_norm", parts)))
    n = len(cfg.layers)
    if cfg.loop is None:
        schedule = [ScheduleEntry(layer=i) for i in range(n)]
    else:
        # the projection that opens every pass is one more layer of the plan
        layers.append(LayerSpec(PartSpec("concat_projection", {
            "hidden_size": cfg.width, "weight": "loop.in", "source": "embedding_output"})))
        schedule = [ScheduleEntry(layer=i) for i in range(cfg.loop.start)]
        for _ in range(cfg.loop.times):
            schedule.append(ScheduleEntry(layer=n))
            schedule += [ScheduleEntry(layer=i) for i in range(cfg.loop.start, cfg.loop.stop)]
        schedule += [ScheduleEntry(layer=i) for i in range(cfg.loop.stop, n)]
    plan = ModelPlan(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                               "weight": "embed", "keep_output": cfg.loop is not None}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(cfg, "final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "head",
                                  "softcap": cfg.logit_softcap}),
        stop_tokens=(),
        max_position=None,
    )
    plan.check()
    return plan


ROPOVIK = register_architecture(Architecture(
    names=("Ropovik", "ropovik"),
    read_config=RopovikConfig.from_json,
    plan=ropovik_plan,
))
