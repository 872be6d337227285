"""Small Sasilorn configurations for the tests, and how a model folder is written from one."""

from __future__ import annotations

import copy

import torch

import plain_sasilorn
from dryft_flash_infer_b200.config import SasilornConfig
from dryft_flash_infer_b200.weights import write_safetensors


def _parallel(left, right, left_scale, right_scale, ff, **more):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale,
                                          "right_scale": right_scale},
            "mlp": {"kind": "dense", "ff": ff} if ff else None, **more}


def _wkv(heads, dim, ff, **more):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": {"kind": "dense", "ff": ff} if ff else None, **more}


_LEFT_A = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25}
_RIGHT_A = {"heads": 2, "dim": 16, "vdim": 8, "tau": 8.0}
#: a parallel layer first, a layer run twice, layers with and without a feed-forward
CASE_A = {"architecture": "Sasilorn", "vocab": 96, "width": 64, "norm": {"eps": 1e-5}, "layers": [
    _parallel(_LEFT_A, _RIGHT_A, 0.7, 1.1, 96),
    _wkv(2, 32, 0),
    _parallel(_LEFT_A, _RIGHT_A, 0.7, 1.1, 96, weights_of=0),
    _wkv(4, 16, 80),
]}
#: sizes that are no multiples of 8, as many key/value heads as heads, one head, values wider than keys, a
#: time-mixing layer first and run twice, scales that are 1 and not
CASE_B = {"architecture": "Sasilorn", "vocab": 75, "width": 72, "norm": {"eps": 1e-6}, "layers": [
    _wkv(3, 24, 0),
    _parallel({"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 12, "scale": 0.3},
              {"heads": 1, "dim": 24, "vdim": 40, "tau": 1.0}, 1.0, 0.5, 0),
    _wkv(3, 24, 0, weights_of=0),
    _parallel({"heads": 4, "kv_heads": 1, "dim": 8, "vdim": 36, "scale": 0.5},
              {"heads": 3, "dim": 36, "vdim": 20, "tau": 3.5}, 0.4, 1.0, 50),
]}
#: no layer keeps keys and values; a width that is no multiple of 8
CASE_C = {"architecture": "Sasilorn", "vocab": 50, "width": 44, "norm": {"eps": 1e-5}, "layers": [
    _wkv(2, 16, 60), _wkv(1, 40, 0)]}
#: sizes in steps of 16, which the bfloat16 engine runs on its tensor-core attention, and heads of 64 key channels
CASE_D = {"architecture": "Sasilorn", "vocab": 120, "width": 128, "norm": {"eps": 1e-5}, "layers": [
    _parallel({"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 64, "scale": 0.2},
              {"heads": 2, "dim": 64, "vdim": 32, "tau": 12.0}, 0.75, 1.25, 160),
    _wkv(2, 64, 0),
    _parallel({"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 64, "scale": 0.2},
              {"heads": 2, "dim": 64, "vdim": 32, "tau": 12.0}, 0.75, 1.25, 160, weights_of=0),
]}
CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D}


def one_layer(kind: str) -> dict:
    """A model of one layer that shows one mechanism: ``left`` / ``right`` (a parallel mixer with the other
    side's weight 0), ``wkv``, or ``mlp`` (a time-mixing layer whose feed-forward is the larger part)."""
    base = {"architecture": "Sasilorn", "vocab": 64, "width": 48, "norm": {"eps": 1e-5}}
    left = {"heads": 6, "kv_heads": 2, "dim": 24, "vdim": 40, "scale": 0.2}
    right = {"heads": 2, "dim": 24, "vdim": 16, "tau": 4.0}
    layer = {"left": _parallel(left, right, 1.3, 0.0, 0), "right": _parallel(left, right, 0.0, 0.9, 0),
             "wkv": _wkv(3, 16, 0), "mlp": _wkv(1, 8, 200)}[kind]
    return {**base, "layers": [layer]}


def sharpened(config: dict, factor: float = 6.0) -> dict:
    """The same model with attention scores ``factor`` times larger: the softmax then rests on a few keys,
    wherever they are, so that a key that is lost or one too many shows in the logits."""
    out = copy.deepcopy(config)
    for layer in out["layers"]:
        if layer["type"] == "parallel":
            layer["mixer"]["left"]["scale"] *= factor
    return out


def long_memory(tensors: dict) -> dict:
    """The same weights with decays close to 1, so that tokens hundreds of places back still matter."""
    out = dict(tensors)
    for name, t in tensors.items():
        if name.endswith(".right.a2.b"):
            out[name] = (t.float() + 5.0).to(t.dtype)
        if name.endswith(".mix.w0"):
            out[name] = (t.float() - 4.0).to(t.dtype)
    return out


def write_model(folder, config: dict, tensors: dict):
    SasilornConfig.from_dict(config).save(folder)
    write_safetensors(folder / "model.safetensors", tensors.items())
    return folder


def make(folder, config: dict, seed: int, change=None):
    """Writes a model of bfloat16-valued random weights and returns ``(folder, config, tensors)``."""
    tensors = plain_sasilorn.random_tensors(config, seed)
    if change is not None:
        tensors = change(tensors)
    return write_model(folder, config, tensors), config, tensors


def prompts(config: dict, lengths, seed: int):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, config["vocab"], (n,), generator=g).tolist() for n in lengths]


def plain_logits(config, tensors, tokens):
    return plain_sasilorn.forward(config, tensors, tokens).float()
