"""Two or more mixers side by side: all read the same rows, and their results are summed with weights."""

from __future__ import annotations

import dataclasses

import torch

from ..ops import kernels
from .base import Mixer, build_part, register_part
from .spec import PartSpec


class ParallelMixer(Mixer):
    """``sum_i scale_i * branch_i(h)`` for branches that are mixers of any kind with an output
    projection of their own (they say which tensor it is in ``output_tensor`` and stop before it in
    ``forward_inner``).

    The output projections stand side by side in one matrix ``[hidden, sum of inner sizes]`` and every
    branch writes its inner rows, already times its scale, into its columns of one buffer: the sum
    of the branches is then a single product, with no pass for the weights.  At most one branch may
    keep keys and values and at most one a state (the cache hands a mixer one of each).

    ``branches``: a sequence of ``(name, PartSpec, scale)``; a branch's tensors are called
    ``<name>.<its local name>``.
    """

    kind = "parallel"

    def __init__(self, hidden_size: int, branches):
        self.hidden_size = hidden_size
        self.names = [name for name, _, _ in branches]
        self.scales = [float(scale) for _, _, scale in branches]
        self.branches = [build_part("mixer", spec if isinstance(spec, PartSpec) else PartSpec(*spec), hidden_size)
                         for _, spec, _ in branches]
        if len(set(self.names)) != len(self.names) or not self.branches:
            raise ValueError("a parallel mixer needs branches with names of their own")
        for name, branch in zip(self.names, self.branches):
            if not hasattr(branch, "forward_inner") or not getattr(branch, "output_tensor", None):
                raise ValueError(f"branch '{name}' ({branch.kind}) cannot stop before its output projection")
        if sum(b.cache_need() is not None for b in self.branches) > 1 or \
                sum(b.state_need() is not None for b in self.branches) > 1:
            raise ValueError("at most one branch of a parallel mixer keeps keys and values, and at most one a state")
        self.offsets, total = [], 0
        for branch in self.branches:
            self.offsets.append(total)
            total += branch.inner_size
        self.inner_size = total
        self.o = None

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.branches)

    def set_compute_dtype(self, dtype) -> None:
        self.compute_dtype = dtype
        for branch in self.branches:
            branch.set_compute_dtype(dtype)

    def tensors(self):
        out = {}
        for name, branch, offset in zip(self.names, self.branches, self.offsets):
            for local, decl in branch.tensors().items():
                if local == branch.output_tensor:
                    if decl.shape != (self.hidden_size, branch.inner_size):
                        raise ValueError(f"branch '{name}': an output projection of shape {decl.shape}")
                    out[f"{name}.{local}"] = dataclasses.replace(decl, buffer="o", row_start=0, col_start=offset)
                else:
                    out[f"{name}.{local}"] = dataclasses.replace(decl, buffer=f"{name}.{decl.buffer}")
        return out

    def buffer_shapes(self):
        out = {"o": ((self.hidden_size, self.inner_size), "compute")}
        for name, branch in zip(self.names, self.branches):
            joint = branch.tensors()[branch.output_tensor].buffer
            for buffer, shape in branch.buffer_shapes().items():
                if buffer != joint:
                    out[f"{name}.{buffer}"] = shape         # a branch may ask for more than its tensors fill
        return out

    def bind(self, buffers) -> None:
        self.o = buffers["o"]
        for name, branch in zip(self.names, self.branches):
            prefix = name + "."
            branch.bind({key[len(prefix):]: t for key, t in buffers.items() if key.startswith(prefix)})

    def cache_need(self):
        return next((n for n in (b.cache_need() for b in self.branches) if n is not None), None)

    def state_need(self):
        return next((n for n in (b.state_need() for b in self.branches) if n is not None), None)

    def prepare(self, max_positions: int, device) -> None:
        for branch in self.branches:
            branch.prepare(max_positions, device)

    def first_weights(self):
        return self.branches[0].first_weights()

    def forward(self, x, ctx, cache, state):
        rows = x.shape[0]
        inner = torch.empty((rows, self.inner_size), dtype=x.dtype, device=x.device)
        after = getattr(ctx, "upcoming", None)
        for index, (branch, offset, scale) in enumerate(zip(self.branches, self.offsets, self.scales)):
            # what the step streams after a branch: the next branch's first matrix, at the end the joint projection
            ctx.upcoming = self.branches[index + 1].first_weights() if index + 1 < len(self.branches) \
                else kernels.next_weights(self.o)
            branch.forward_inner(x, ctx, cache if branch.cache_need() is not None else None,
                                 state if branch.state_need() is not None else None,
                                 out=inner[:, offset: offset + branch.inner_size], scale=scale)
        ctx.upcoming = after
        return kernels.linear(inner, self.o, then=after)


register_part("mixer", ParallelMixer.kind, ParallelMixer)
