"""Configuration of the Sasilorn decoder.

``config.json`` names the architecture in ``architecture`` and gives ``vocab``, ``width``,
``norm.eps`` and ``layers``: one entry per layer with its ``type`` (``wkv`` or ``parallel``), the
sizes of its mixer under ``mixer``, its feed-forward under ``mlp`` (``{"kind": "dense", "ff": n}``
or null for a layer without one) and optionally ``weights_of: j`` for a layer that runs layer
``j``'s tensors with a cache and state of its own.

Sizes that the file does not state are read from the shapes of the model's tensors
(``with_tensor_shapes``): the narrow middle of the decay projections and the value size of a
``wkv`` mixer.  A configuration for random weights states them itself (``rank``, ``vdim``).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, ClassVar

from .base import ConfigError, ModelConfig, take

MIXER_TYPES = ("wkv", "parallel")
DEFAULT_RANK = 32


def _positive(raw: dict, key: str, where: str) -> int:
    try:
        value = take(raw, key, int)
    except ConfigError as exc:
        raise ConfigError(f"{exc} (in {where})") from None
    if value <= 0:
        raise ConfigError(f"config.json: '{key}' must be positive in {where}, got {value}")
    return value


@dataclass(frozen=True)
class SasilornConfig(ModelConfig):
    vocab_size: int
    hidden_size: int
    norm_eps: float
    #: the entries of ``layers`` as the file gives them (plus ``rank``/``vdim`` once known)
    layers: tuple = field(default_factory=tuple)

    architecture: ClassVar[str] = "Sasilorn"
    model_type: ClassVar[str] = "sasilorn"

    @classmethod
    def from_dict(cls, raw: dict[str, Any]) -> "SasilornConfig":
        norm = raw.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: missing key 'norm' (an object with 'eps')")
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab_size=take(raw, "vocab", int), hidden_size=take(raw, "width", int),
                  norm_eps=take(norm, "eps", float), layers=tuple(copy.deepcopy(layers)))
        cfg.validate()
        return cfg

    def to_dict(self) -> dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def source_of(self, index: int) -> int:
        """The layer whose tensors layer ``index`` runs (itself unless it says ``weights_of``)."""
        seen = set()
        while "weights_of" in self.layers[index] and index not in seen:
            seen.add(index)
            index = self.layers[index]["weights_of"]
        return index

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0:
            raise ConfigError("config.json: 'vocab' and 'width' must be positive")
        if not self.norm_eps > 0:
            raise ConfigError("config.json: 'norm.eps' must be positive")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, dict) or layer.get("type") not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type must be one of {MIXER_TYPES}")
            mixer = layer.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"config.json: {where}.mixer must be an object")
            if layer["type"] == "wkv":
                _positive(mixer, "heads", where), _positive(mixer, "dim", where)
            else:
                left, right = mixer.get("left"), mixer.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    raise ConfigError(f"config.json: {where}.mixer needs 'left' and 'right'")
                heads, kv = _positive(left, "heads", where), _positive(left, "kv_heads", where)
                if heads % kv:
                    raise ConfigError(f"config.json: {where}: {heads} heads are not a multiple of {kv} kv_heads")
                _positive(left, "dim", where), _positive(left, "vdim", where)
                take(left, "scale", float)
                _positive(right, "heads", where), _positive(right, "dim", where), _positive(right, "vdim", where)
                if not take(right, "tau", float) > 0:
                    raise ConfigError(f"config.json: {where}.mixer.right.tau must be positive")
                take(mixer, "left_scale", float), take(mixer, "right_scale", float)
            mlp = layer.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind must be 'dense' (or mlp null)")
                _positive(mlp, "ff", where)
            source = layer.get("weights_of")
            if source is not None:
                if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < len(self.layers) \
                        or source == index or "weights_of" in self.layers[self.source_of(index)]:
                    raise ConfigError(f"config.json: {where}.weights_of must name another layer that has tensors of its own")
                other = self.layers[self.source_of(index)]
                if other.get("type") != layer["type"] or (other.get("mlp") is None) != (mlp is None):
                    raise ConfigError(f"config.json: {where} runs layer {source}'s tensors but is of another kind")

    def with_tensor_shapes(self, shapes: dict[str, tuple[int, ...]]) -> "SasilornConfig":
        """The configuration with the sizes that only the model's tensors give: ``rank`` (rows of the
        first decay projection) and, for ``wkv``, ``vdim`` (rows of the value projection over heads)."""
        layers = copy.deepcopy(list(self.layers))
        for index, layer in enumerate(layers):
            p = f"l{self.source_of(index)}.mix."
            if layer["type"] == "wkv":
                mixer = layer["mixer"]
                if p + "w1" in shapes:
                    mixer["rank"] = int(shapes[p + "w1"][0])
                if p + "v" in shapes and shapes[p + "v"][0] % mixer["heads"] == 0:
                    mixer["vdim"] = int(shapes[p + "v"][0]) // mixer["heads"]
            elif p + "right.a1" in shapes:
                layer["mixer"]["right"]["rank"] = int(shapes[p + "right.a1"][0])
        return SasilornConfig(self.vocab_size, self.hidden_size, self.norm_eps, tuple(layers))
