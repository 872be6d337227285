"""A plain, slow implementation of the Sasilorn decoder, token by token where a layer has a state.

It works from the dictionary of ``config.json`` and a dictionary of tensors by their file names, on
the CPU, in float64 unless told otherwise, with one function per mechanism.  It shares no code with the
package: the tests compare the engine with it.

Notation: ``h`` is a mixer's input (one sequence, ``[tokens, width]``); matrices are stored
``[out, in]`` and applied as ``h @ W.T``.
"""

from __future__ import annotations

import math

import torch


def dynamic_tanh(x, weight, bias, alpha):
    """``tanh(alpha x) * weight + bias``, element by element: no mean, no variance."""
    return torch.tanh(alpha * x) * weight + bias


def unit_rms(x, eps):
    """``x`` divided by its root mean square over the last axis, ``eps`` inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def squared_relu_mlp(h, up, down):
    return torch.relu(h @ up.T).square() @ down.T


def gated_softmax_attention(h, p, sizes, eps):
    """Causal softmax attention without positions: grouped key/value heads, query and key heads
    normalised to unit rms and weighted, values of a size of their own, one sigmoid gate per head."""
    T = h.shape[0]
    H, G, D, V, scale = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"], sizes["scale"]
    q = (h @ p["q"].T).view(T, H, D)
    k = (h @ p["k"].T).view(T, G, D)
    v = (h @ p["v"].T).view(T, G, V)
    q = unit_rms(q, eps) * p["q.norm"]
    k = unit_rms(k, eps) * p["k.norm"]
    gate = torch.sigmoid(h @ p["g"].T)                       # [T, H]
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for head in range(H):
        kv = head // (H // G)
        for t in range(T):
            scores = (k[: t + 1, kv] @ q[t, head]) * scale
            weights = torch.softmax(scores, 0)
            out[t, head] = (weights[:, None] * v[: t + 1, kv]).sum(0) * gate[t, head]
    return out.reshape(T, H * V) @ p["o"].T


def gated_linear_attention(h, p, sizes, eps):
    """``S_t = diag(a_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head, with the decay
    ``a = sigmoid(z)^(1/tau)`` per key channel from a two-step projection; each head's output is
    normalised over its values, gated by ``silu`` of a projection and projected."""
    T = h.shape[0]
    H, D, V, tau = sizes["heads"], sizes["dim"], sizes["vdim"], sizes["tau"]
    q = (h @ p["q"].T).view(T, H, D) * D ** -0.5
    k = (h @ p["k"].T).view(T, H, D)
    v = (h @ p["v"].T).view(T, H, V)
    z = ((h @ p["a1"].T) @ p["a2"].T + p["a2.b"]).view(T, H, D)
    decay = torch.sigmoid(z) ** (1.0 / tau)
    state = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        state = decay[t][:, :, None] * state + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state, q[t])
    out = unit_rms(out, eps) * p["norm"]
    gate = torch.nn.functional.silu(h @ p["g"].T)
    return (out.reshape(T, H * V) * gate) @ p["o"].T


def parallel_mixer(h, p, sizes, eps):
    left = gated_softmax_attention(h, {k[5:]: v for k, v in p.items() if k.startswith("left.")}, sizes["left"], eps)
    right = gated_linear_attention(h, {k[6:]: v for k, v in p.items() if k.startswith("right.")}, sizes["right"], eps)
    return sizes["left_scale"] * left + sizes["right_scale"] * right


def wkv_mixer(h, p, sizes, eps):
    """Time mixing with a matrix state per head: every projection reads its own blend of the token's
    row and the row before it; the token itself enters its own output through the bonus ``u``, the
    state decays by ``exp(-exp(.))`` per key channel."""
    T, _ = h.shape
    H, D = sizes["heads"], sizes["dim"]
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]])

    def blend(which):
        return h + (before - h) * p["mu." + which]

    r = (blend("r") @ p["r"].T).view(T, H, D)
    k = (blend("k") @ p["k"].T).view(T, H, D)
    v = (blend("v") @ p["v"].T).view(T, H, -1)
    gate = torch.nn.functional.silu(blend("g") @ p["g"].T)
    w = torch.exp(-torch.exp(torch.tanh(blend("w") @ p["w1"].T) @ p["w2"].T + p["w0"])).view(T, H, D)
    u = p["u"]
    V = v.shape[-1]
    state = torch.zeros(H, D, V, dtype=h.dtype)
    out = torch.zeros(T, H, V, dtype=h.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", state + u[:, :, None] * kv, r[t])
        state = w[t][:, :, None] * state + kv
    out = unit_rms(out, eps).reshape(T, H * V) * p["norm"] * gate
    return out @ p["o"].T


_MIXERS = {"parallel": parallel_mixer, "wkv": wkv_mixer}


def layer_tensors(tensors, index):
    prefix = f"l{index}."
    return {name[len(prefix):]: t for name, t in tensors.items() if name.startswith(prefix)}


def forward(config, tensors, tokens, dtype=torch.float64, residuals=None):
    """Logits ``[tokens, vocab]`` of one sequence from its first token on.  ``residuals``: a list that
    receives the residual stream after every layer."""
    tensors = {name: t.to(dtype) for name, t in tensors.items()}
    eps = config["norm"]["eps"]
    x = tensors["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    for index, layer in enumerate(config["layers"]):
        p = layer_tensors(tensors, layer.get("weights_of", index))

        def norm(name):
            return dynamic_tanh(x, p[name], p[name + ".b"], p[name + ".alpha"])

        mixer = {k[4:]: v for k, v in p.items() if k.startswith("mix.")}
        x = x + _MIXERS[layer["type"]](norm("norm1"), mixer, layer["mixer"], eps)
        if layer["mlp"] is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(layer["mlp"]["kind"])
            x = x + squared_relu_mlp(norm("norm2"), p["mlp.up"], p["mlp.down"])
        if residuals is not None:
            residuals.append(x.clone())
    x = dynamic_tanh(x, tensors["final.norm"], tensors["final.norm.b"], tensors["final.norm.alpha"])
    return x @ tensors["head"].T


def random_tensors(config, seed, dtype=torch.bfloat16):
    """Random weights for ``config`` under the file's names, rounded to ``dtype``.  The scales are chosen
    so that every mechanism matters: decays spread between fast and slow, norms away from 1 and 0."""
    g = torch.Generator().manual_seed(seed)
    width, vocab = config["width"], config["vocab"]

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(tuple(shape), generator=g) * std + mean).to(dtype)

    def matrix(out, inner, gain=1.0):
        return normal(out, inner, std=gain / math.sqrt(inner))

    out = {"embed": normal(vocab, width), "head": matrix(vocab, width)}

    def norm(name):
        out[name] = normal(width, std=0.2, mean=1.0)
        out[name + ".b"] = normal(width, std=0.1)
        out[name + ".alpha"] = normal(std=0.1, mean=0.7)

    norm("final.norm")
    for index, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        p = f"l{index}."
        norm(p + "norm1")
        m, s = p + "mix.", layer["mixer"]
        if layer["type"] == "wkv":
            H, D = s["heads"], s["dim"]
            for which in "rkvgw":
                out[m + "mu." + which] = torch.rand(width, generator=g).to(dtype)
            for which in "rkvg":
                out[m + which] = matrix(H * D, width)
            rank = max(4, width // 8)
            out[m + "w1"] = matrix(rank, width)
            out[m + "w2"] = matrix(H * D, rank)
            out[m + "w0"] = normal(H * D, std=1.0, mean=-1.5)
            out[m + "u"] = normal(H, D, std=0.5)
            out[m + "norm"] = normal(H * D, std=0.2, mean=1.0)
            out[m + "o"] = matrix(width, H * D)
        elif layer["type"] == "parallel":
            left, right = s["left"], s["right"]
            H, G, D, V = left["heads"], left["kv_heads"], left["dim"], left["vdim"]
            out[m + "left.q"] = matrix(H * D, width)
            out[m + "left.k"] = matrix(G * D, width)
            out[m + "left.v"] = matrix(G * V, width)
            out[m + "left.q.norm"] = normal(D, std=0.2, mean=1.0)
            out[m + "left.k.norm"] = normal(D, std=0.2, mean=1.0)
            out[m + "left.g"] = matrix(H, width)
            out[m + "left.o"] = matrix(width, H * V)
            H, D, V = right["heads"], right["dim"], right["vdim"]
            rank = max(4, width // 8)
            for which, cols in (("q", D), ("k", D), ("v", V), ("g", V)):
                out[m + "right." + which] = matrix(H * cols, width)
            out[m + "right.a1"] = matrix(rank, width)
            out[m + "right.a2"] = matrix(H * D, rank)
            out[m + "right.a2.b"] = normal(H * D, std=1.5, mean=2.0)
            out[m + "right.norm"] = normal(V, std=0.2, mean=1.0)
            out[m + "right.o"] = matrix(width, H * V)
        else:
            raise ValueError(layer["type"])
        if layer["mlp"] is not None:
            norm(p + "norm2")
            out[p + "mlp.up"] = matrix(layer["mlp"]["ff"], width)
            out[p + "mlp.down"] = matrix(width, layer["mlp"]["ff"])
    return out
