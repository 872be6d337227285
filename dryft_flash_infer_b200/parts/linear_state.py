"""Mixers that carry a matrix state per head from token to token instead of keys and values."""

from __future__ import annotations

import torch

from ..ops import kernels
from .base import Mixer, StateNeed, TensorDecl, register_part


class GatedLinearAttention(Mixer):
    """Linear attention with a decay per key channel.

    Per head, with ``q = W_q h * key_dim^-0.5``, ``k = W_k h``, ``v = W_v h``:
    ``S_t = diag(a_t) S_(t-1) + k_t v_t^T`` and ``o_t = S_t^T q_t``, where the decay is
    ``a = sigmoid(z)^(1/tau)`` with ``z = W_a2 (W_a1 h) + b`` (a projection through a narrow middle,
    laid out heads x key_dim).  Each head's ``o`` is divided by its root mean square over
    ``value_dim`` and multiplied by a weight the heads share; the heads, side by side, are
    multiplied by ``silu(W_g h)`` and projected by ``W_o``.

    q, k, v, g and the narrow projection come from one fused matrix.  ``z`` is computed as a float32
    product and everything after it (the bias, the decay, the state, the reads, the norm) is float32
    in either engine dtype.  The state ``[heads, key_dim, value_dim]`` float32 starts at zero.
    """

    kind = "gated_linear_attention"
    graph_safe = True
    output_tensor = "o_proj"

    def __init__(self, hidden_size: int, n_heads: int, key_dim: int, value_dim: int, decay_rank: int, tau: float,
                 norm_eps: float = 1e-6):
        if not tau > 0:
            raise ValueError(f"tau must be positive, got {tau}")
        self.hidden_size, self.n_heads, self.key_dim, self.value_dim = hidden_size, n_heads, key_dim, value_dim
        self.decay_rank, self.tau, self.norm_eps = int(decay_rank), float(tau), float(norm_eps)
        self.qkvga = self.a2 = self.a2_bias = self.o = self.norm = None

    @property
    def inner_size(self) -> int:
        return self.n_heads * self.value_dim

    def tensors(self):
        hk, hv, hidden = self.n_heads * self.key_dim, self.n_heads * self.value_dim, self.hidden_size
        return {
            "q_proj": TensorDecl((hk, hidden), "qkvga", 0),
            "k_proj": TensorDecl((hk, hidden), "qkvga", hk),
            "v_proj": TensorDecl((hv, hidden), "qkvga", 2 * hk),
            "g_proj": TensorDecl((hv, hidden), "qkvga", 2 * hk + hv),
            "a1_proj": TensorDecl((self.decay_rank, hidden), "qkvga", 2 * hk + 2 * hv),
            "a2_proj": TensorDecl((hk, self.decay_rank), "a2"),
            "a2_bias": TensorDecl((hk,), "a2_bias", precision="float32"),
            "norm": TensorDecl((self.value_dim,), "norm", init="norm", precision="float32"),
            "o_proj": TensorDecl((hidden, hv), "o"),
        }

    def state_need(self):
        return StateNeed((self.n_heads * self.key_dim * self.value_dim,), "float32", 0.0)

    def first_weights(self):
        return kernels.next_weights(self.qkvga)

    def forward_inner(self, x, ctx, cache, state, out=None, scale: float = 1.0):
        hk, hv = self.n_heads * self.key_dim, self.n_heads * self.value_dim
        proj = kernels.linear(x, self.qkvga)
        narrow = proj[:, 2 * hk + 2 * hv:]
        z = kernels.linear(narrow.contiguous(), self.a2, out_dtype=torch.float32)
        if out is None:
            out = torch.empty((proj.shape[0], hv), dtype=proj.dtype, device=proj.device)
        return kernels.linear_scan(
            kernels.SCAN_DECAY_THEN_READ, proj[:, :hk], proj[:, hk:2 * hk], proj[:, 2 * hk:2 * hk + hv],
            proj[:, 2 * hk + hv:2 * hk + 2 * hv], z, self.a2_bias, None, self.tau, self.key_dim ** -0.5, state, ctx,
            self.n_heads, self.key_dim, self.value_dim, self.norm, False, self.norm_eps, out, out_scale=scale)

    def forward(self, x, ctx, cache, state):
        return kernels.linear(self.forward_inner(x, ctx, cache, state), self.o, then=getattr(ctx, "upcoming", None))


class TimeMix(Mixer):
    """RWKV-style time mixing with a data-dependent decay.

    With ``h'`` the row of the token before (zeros for a sequence's first token), each of r, k, v, g
    and w reads its own blend ``h + (h' - h) * mu_s``.  ``r, k, v`` are projections of their blends
    (heads x key_dim; values heads x value_dim), ``gate = silu(W_g blend_g)``, and the decay is
    ``w = exp(-exp(W_w2 tanh(W_w1 blend_w) + w0))`` per head and key channel.  Per head
    ``o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t`` (the bonus ``u`` lets the token read itself), then
    ``S_t = diag(w_t) S_(t-1) + k_t v_t^T``.  Each head's ``o`` is divided by its root mean square; the
    heads, side by side, are multiplied by a weight, by the gate, and projected by ``W_o``.

    The decay's second product gives float32 and everything after it is float32 in either engine
    dtype.  The state per sequence is ``S [heads, key_dim, value_dim]`` followed by the last row
    ``h`` the sequence has seen, all float32, all zero at the start.
    """

    kind = "time_mix"
    graph_safe = True
    output_tensor = "o_proj"
    BLENDS = ("r", "k", "v", "g", "w")

    def __init__(self, hidden_size: int, n_heads: int, key_dim: int, value_dim: int | None = None,
                 decay_rank: int = 64, norm_eps: float = 1e-5):
        self.hidden_size, self.n_heads, self.key_dim = hidden_size, n_heads, key_dim
        self.value_dim = key_dim if value_dim is None else int(value_dim)
        self.decay_rank, self.norm_eps = int(decay_rank), float(norm_eps)
        self.mu = self.r = self.k = self.v = self.g = self.w1 = self.w2 = self.w0 = self.u = self.norm = self.o = None

    @property
    def inner_size(self) -> int:
        return self.n_heads * self.value_dim

    @property
    def _matrix_floats(self) -> int:
        return self.n_heads * self.key_dim * self.value_dim

    def tensors(self):
        hk, hv, hidden = self.n_heads * self.key_dim, self.n_heads * self.value_dim, self.hidden_size
        out = {f"mu_{s}": TensorDecl((hidden,), "mu", i * hidden, init="norm", precision="float32")
               for i, s in enumerate(self.BLENDS)}
        out.update({
            "r_proj": TensorDecl((hk, hidden), "r"),
            "k_proj": TensorDecl((hk, hidden), "k"),
            "v_proj": TensorDecl((hv, hidden), "v"),
            "g_proj": TensorDecl((hv, hidden), "g"),
            "w1_proj": TensorDecl((self.decay_rank, hidden), "w1"),
            "w2_proj": TensorDecl((hk, self.decay_rank), "w2"),
            "w0": TensorDecl((hk,), "w0", precision="float32"),
            "u": TensorDecl((self.n_heads, self.key_dim), "u", precision="float32"),
            "norm": TensorDecl((hv,), "norm", init="norm", precision="float32"),
            "o_proj": TensorDecl((hidden, hv), "o"),
        })
        return out

    def state_need(self):
        return StateNeed((self._matrix_floats + self.hidden_size,), "float32", 0.0)

    def first_weights(self):
        return kernels.next_weights(self.r)

    def forward_inner(self, x, ctx, cache, state, out=None, scale: float = 1.0):
        hv = self.n_heads * self.value_dim
        blends = kernels.token_shift(x, self.mu.view(len(self.BLENDS), self.hidden_size), state, self._matrix_floats, ctx)
        r = kernels.linear(blends[0], self.r, then=kernels.next_weights(self.k))
        k = kernels.linear(blends[1], self.k, then=kernels.next_weights(self.v))
        v = kernels.linear(blends[2], self.v, then=kernels.next_weights(self.g))
        g = kernels.linear(blends[3], self.g)
        narrow = kernels.linear_act(blends[4], self.w1, "tanh")
        z = kernels.linear(narrow, self.w2, out_dtype=torch.float32)
        if out is None:
            out = torch.empty((x.shape[0], hv), dtype=x.dtype, device=x.device)
        return kernels.linear_scan(
            kernels.SCAN_READ_THEN_DECAY, r, k, v, g, z, self.w0, self.u, 0.0, 1.0, state, ctx, self.n_heads,
            self.key_dim, self.value_dim, self.norm, True, self.norm_eps, out, out_scale=scale, carry_rows=x,
            carry_offset=self._matrix_floats)

    def forward(self, x, ctx, cache, state):
        return kernels.linear(self.forward_inner(x, ctx, cache, state), self.o, then=getattr(ctx, "upcoming", None))


register_part("mixer", GatedLinearAttention.kind, GatedLinearAttention)
register_part("mixer", TimeMix.kind, TimeMix)
