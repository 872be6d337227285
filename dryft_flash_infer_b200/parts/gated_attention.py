"""Softmax attention without positions whose heads are gated: the left half of a parallel mixer."""

from __future__ import annotations

from ..ops import kernels
from .base import KVNeed, Mixer, TensorDecl, register_part


class GatedAttention(Mixer):
    """``o_proj(concat_h(sigmoid(g_h) * attend_h))`` over the paged cache, causal, no biases, no rotation.

    q, k, v and the gates come from one fused matrix (q rows, then k, then v, then one gate row per
    query head).  Keys have ``head_dim`` elements, values ``v_head_dim`` of their own; query head ``h``
    reads key/value head ``h // (n_heads / n_kv_heads)``.  With ``qk_norm`` every query and key head is
    divided by its root mean square (``qk_norm_eps`` inside the root) and multiplied by a weight that
    all heads share.  Scores are ``q . k * scale`` in float32, ordinary softmax over the visible keys.
    Every head's output is multiplied by the sigmoid of its own gate, a projection of the mixer's
    input, before the output projection.

    ``forward_inner`` stops before the output projection and writes the gated heads, times
    ``scale``, where it is told: a mixer that runs beside another one sums both projections in one
    product (``parts/parallel.py``).
    """

    kind = "gated_attention"
    graph_safe = True
    #: the local name of the output projection, which a parallel mixer fuses with its neighbours'
    output_tensor = "o_proj"

    def __init__(self, hidden_size: int, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int | None = None,
                 scale: float | None = None, qk_norm: bool = True, qk_norm_eps: float = 1e-6, window: int = 0):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads are not a multiple of {n_kv_heads} key/value heads")
        v_head_dim = head_dim if v_head_dim is None else int(v_head_dim)
        if not (0 < head_dim <= 256 and 0 < v_head_dim <= 256):
            raise ValueError(f"gated attention takes head sizes up to 256, got {head_dim} and {v_head_dim}")
        self.hidden_size, self.n_heads, self.n_kv_heads = hidden_size, n_heads, n_kv_heads
        self.head_dim, self.v_head_dim = head_dim, v_head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.qk_norm, self.qk_norm_eps, self.window = qk_norm, float(qk_norm_eps), int(window)
        self.qkvg = self.o = self.q_norm = self.k_norm = None

    @property
    def inner_size(self) -> int:
        return self.n_heads * self.v_head_dim

    def tensors(self):
        q_rows, k_rows, v_rows = self.n_heads * self.head_dim, self.n_kv_heads * self.head_dim, self.n_kv_heads * self.v_head_dim
        out = {
            "q_proj": TensorDecl((q_rows, self.hidden_size), "qkvg", 0),
            "k_proj": TensorDecl((k_rows, self.hidden_size), "qkvg", q_rows),
            "v_proj": TensorDecl((v_rows, self.hidden_size), "qkvg", q_rows + k_rows),
            "g_proj": TensorDecl((self.n_heads, self.hidden_size), "qkvg", q_rows + k_rows + v_rows),
            "o_proj": TensorDecl((self.hidden_size, self.inner_size), "o"),
        }
        if self.qk_norm:
            out["q_norm"] = TensorDecl((self.head_dim,), "q_norm", init="norm", precision="float32")
            out["k_norm"] = TensorDecl((self.head_dim,), "k_norm", init="norm", precision="float32")
        return out

    @property
    def _used_rows(self) -> int:
        return (self.n_heads + self.n_kv_heads) * self.head_dim + self.n_kv_heads * self.v_head_dim + self.n_heads

    def buffer_shapes(self):
        # the fused projection's rows are rounded up to eight, so that a row of its result starts on 16 bytes
        # (what the tensor-core attention's copies of the query rows need); the spare rows are zeros
        shapes = super().buffer_shapes()
        (rows, cols), precision = shapes["qkvg"]
        shapes["qkvg"] = ((-(-rows // 8) * 8, cols), precision)
        return shapes

    def bind(self, buffers) -> None:
        super().bind(buffers)
        self.qkvg[self._used_rows:].zero_()

    def cache_need(self):
        return KVNeed(self.n_kv_heads, self.head_dim, self.window,
                      self.v_head_dim if self.v_head_dim != self.head_dim else 0)

    def first_weights(self):
        return kernels.next_weights(self.qkvg)

    def forward_inner(self, x, ctx, cache, state, out=None, scale: float = 1.0):
        H, G, D, V = self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim
        proj = kernels.linear(x, self.qkvg)
        q = kernels.head_norm_write(proj, H, G, D, V, self.q_norm, self.k_norm, self.qk_norm_eps, ctx.row_pos,
                                    ctx.row_seq, cache)
        gates = proj[:, self._used_rows - H: self._used_rows]
        if ctx.all_decode:
            return kernels.attention_split_decode(q, cache, ctx, H, G, D, self.scale, self.window, gate=gates,
                                                  out_scale=scale, out=out)
        if kernels.split_prefill_takes(q, D, V):
            return kernels.attention_split_prefill(q, cache, ctx, H, G, D, self.scale, self.window, gate=gates,
                                                   out_scale=scale, out=out)
        return kernels.attention_generic(q, cache, ctx.row_seq, ctx.row_pos, H, G, D, self.scale, self.window,
                                         gate=gates, out_scale=scale, out=out)

    def forward(self, x, ctx, cache, state):
        return kernels.linear(self.forward_inner(x, ctx, cache, state), self.o, then=getattr(ctx, "upcoming", None))


register_part("mixer", GatedAttention.kind, GatedAttention)
