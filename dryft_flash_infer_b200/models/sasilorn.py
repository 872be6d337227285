"""The Sasilorn decoder as a ``ModelSpec``.

A float32 residual stream between pre-norm layers whose norm is Dynamic Tanh.  A layer's mixer is
either RWKV-style time mixing (``wkv``) or two mixers side by side (``parallel``): softmax attention
without positions, with per-head query/key norm, values of a size of their own and a sigmoid gate
per head, beside gated linear attention; their sum is weighted by two constants.  A layer may have
a dense feed-forward with the squared relu, or none.  A layer with ``weights_of`` appears in the
schedule as a second application of another layer's tensors with a cache entry and a state of its own.

Tensor names: ``embed``, ``head``, ``final.norm[.b|.alpha]``, and per layer ``l<i>.norm1``,
``l<i>.norm2`` (each with ``.b`` and ``.alpha``), ``l<i>.mix.*`` and ``l<i>.mlp.{up,down}``.
"""

from __future__ import annotations

from ..config.sasilorn import DEFAULT_RANK, SasilornConfig
from ..config import register_architecture
from ..parts import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm_names(local: str, file_name: str) -> dict[str, str]:
    return {f"{local}.weight": file_name, f"{local}.bias": file_name + ".b", f"{local}.alpha": file_name + ".alpha"}


def _time_mix(config: SasilornConfig, sizes: dict, prefix: str):
    spec = PartSpec("time_mix", {"n_heads": sizes["heads"], "key_dim": sizes["dim"],
                                 "value_dim": sizes.get("vdim", sizes["dim"]),
                                 "decay_rank": sizes.get("rank", DEFAULT_RANK), "norm_eps": config.norm_eps})
    names = {f"mixer.mu_{s}": f"{prefix}mu.{s}" for s in "rkvgw"}
    names.update({f"mixer.{s}_proj": prefix + s for s in ("r", "k", "v", "g", "w1", "w2", "o")})
    names.update({"mixer.w0": prefix + "w0", "mixer.u": prefix + "u", "mixer.norm": prefix + "norm"})
    return spec, names


def _parallel(config: SasilornConfig, sizes: dict, prefix: str):
    left, right = sizes["left"], sizes["right"]
    attention = PartSpec("gated_attention", {
        "n_heads": left["heads"], "n_kv_heads": left["kv_heads"], "head_dim": left["dim"], "v_head_dim": left["vdim"],
        "scale": left["scale"], "qk_norm": True, "qk_norm_eps": config.norm_eps})
    linear = PartSpec("gated_linear_attention", {
        "n_heads": right["heads"], "key_dim": right["dim"], "value_dim": right["vdim"],
        "decay_rank": right.get("rank", DEFAULT_RANK), "tau": right["tau"], "norm_eps": config.norm_eps})
    spec = PartSpec("parallel", {"branches": (("left", attention, sizes["left_scale"]),
                                              ("right", linear, sizes["right_scale"]))})
    names = {f"mixer.left.{s}_proj": f"{prefix}left.{s}" for s in ("q", "k", "v", "g", "o")}
    names.update({"mixer.left.q_norm": prefix + "left.q.norm", "mixer.left.k_norm": prefix + "left.k.norm"})
    names.update({f"mixer.right.{s}_proj": f"{prefix}right.{s}" for s in ("q", "k", "v", "g", "o", "a1", "a2")})
    names.update({"mixer.right.a2_bias": prefix + "right.a2.b", "mixer.right.norm": prefix + "right.norm"})
    return spec, names


def build_sasilorn(config: SasilornConfig) -> ModelSpec:
    norm = PartSpec("dynamic_tanh", {})
    layers, place, schedule = [], {}, []
    for index, entry in enumerate(config.layers):
        if "weights_of" not in entry:
            p = f"l{index}."
            mixer, names = (_time_mix if entry["type"] == "wkv" else _parallel)(config, entry["mixer"], p + "mix.")
            names.update(_norm_names("mixer_norm", p + "norm1"))
            norms = {"mixer_norm": norm}
            feed_forward = None
            if entry["mlp"] is not None:
                feed_forward = PartSpec("dense_mlp", {"intermediate_size": entry["mlp"]["ff"], "activation": "relu2"})
                names.update({"feed_forward.up_proj": p + "mlp.up", "feed_forward.down_proj": p + "mlp.down"})
                names.update(_norm_names("ffn_norm", p + "norm2"))
                norms["ffn_norm"] = norm
            place[index] = len(layers)
            layers.append(LayerSpec("pre_norm", mixer, feed_forward, norms, names))
    for index in range(len(config.layers)):
        # a layer that runs another one's tensors: the same LayerSpec once more, cache and state of its own
        schedule.append(ScheduleEntry(layer=place[config.source_of(index)], cache=index))
    return ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        max_positions=1 << 30,                      # no layer reads a position
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm,
        embedding_name="embed",
        final_norm_names={"weight": "final.norm", "bias": "final.norm.b", "alpha": "final.norm.alpha"},
        head_name="head",
        residual_float32=True,
    )


register_architecture(SasilornConfig.architecture, SasilornConfig, build_sasilorn)
