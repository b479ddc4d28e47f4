"""Mixers side by side: every branch reads the same input.  ``combine`` says how their outputs
meet:

* ``mean_of_normed`` (the default): each branch's output is divided by its root mean square over
  the width and multiplied by a weight of its own (``<name_i>.out``), and the results are averaged,

      out = ( rms_norm(branch_0(x)) * w_0 + rms_norm(branch_1(x)) * w_1 ) / 2

* ``weighted_sum``: out = scales[0] * branch_0(x) + scales[1] * branch_1(x) with fixed numbers; the
  branches' outputs stay float32 until they are summed.

The branches are projected mixers (``parts.recurrent.ProjectedMixer``): their input matrices are
stacked, so the layer's input goes through one product for all of them.  The mixer's cache spec is
the tuple of its branches' specs; its run gets one binding per branch.  Branch i's tensors live
under ``<name_i>.``.
"""

from __future__ import annotations

import torch

from ..config.model import PartSpec
from ..kernels import ops
from ..kernels import recurrent as rk
from .base import Mixer, build_mixer, compute_matrix, register_mixer
from .context import CacheBinding, StepContext, StepPrep, UnscaledRows
from .recurrent import ProjectedMixer, stack_segments, vector32


class ParallelMixer(Mixer):
    def __init__(self, width: int, eps: float, branches, dtype: torch.dtype,
                 device: torch.device, combine: str = "mean_of_normed", scales=None) -> None:
        """``branches``: ((name, PartSpec), (name, PartSpec))."""
        super().__init__(dtype, device)
        if len(branches) != 2:
            raise ValueError("parallel: two branches side by side are implemented")
        if combine not in ("mean_of_normed", "weighted_sum"):
            raise ValueError(f"parallel: combine '{combine}' is not implemented")
        if combine == "weighted_sum" and (scales is None or len(scales) != 2):
            raise ValueError("parallel: a weighted sum needs one scale for each branch")
        self.width, self.eps, self.combine = width, eps, combine
        self.scales = None if scales is None else tuple(float(x) for x in scales)
        self.names = [name for name, _ in branches]
        self.branches = [build_mixer(spec, dtype, device) for _, spec in branches]
        for branch in self.branches:
            if not isinstance(branch, ProjectedMixer):
                raise ValueError("parallel: a branch must be a projected mixer")
        self.graph_safe = all(branch.graph_safe for branch in self.branches)
        self.prepare_key = "parallel/" + "+".join(str(getattr(b, "prepare_key", b.kind))
                                                  for b in self.branches)

    def tensors(self):
        out = {}
        for name, branch in zip(self.names, self.branches):
            for local, what in branch.tensors().items():
                out[f"{name}.{local}"] = what
            if self.combine == "mean_of_normed":
                out[f"{name}.out"] = ((self.width,), "vector")
        return out

    def load(self, tensors):
        mats = []
        for name, branch in zip(self.names, self.branches):
            branch.load({local: tensors[f"{name}.{local}"] for local in branch.tensors()})
            mats.append(branch.input_matrix())
        stacked, self.offsets = stack_segments(mats)
        self.rows = [m.shape[0] for m in mats]
        self.w_in = compute_matrix(stacked, self.dtype, self.device)
        for branch in self.branches:
            branch.finish_load()
        if self.combine == "mean_of_normed":
            self.out_weights = [vector32(tensors[f"{name}.out"], self.device)
                                for name in self.names]

    def cache_spec(self):
        return tuple(branch.cache_spec() for branch in self.branches)

    def kernel_modules(self):
        own = ("recurrent",) if self.combine == "mean_of_normed" else ()
        return tuple(m for branch in self.branches for m in branch.kernel_modules()) + own

    def prepare(self, prep: StepPrep) -> None:
        for branch in self.branches:
            branch.prepare(prep)

    def takes_unscaled(self, n_rows: int) -> bool:
        """The norm before the mixer can ride on the one input product (``NormRider``); the
        mixer's last operation is no product, so the norm after it runs itself."""
        return ops.norm_ride_parts(n_rows, self.w_in, self.dtype) > 0

    def forward(self, x: "torch.Tensor | UnscaledRows", ctx: StepContext,
                cache: "CacheBinding | None") -> torch.Tensor:
        if cache is None or cache.kind != "parts" or len(cache.parts) != len(self.branches):
            raise ValueError("parallel: one cache binding per branch is needed")
        before = None
        if isinstance(x, UnscaledRows):
            before, x = x, x.rows
        n = x.shape[0]
        proj = ctx.buffer("parallel.proj", (n, self.w_in.shape[0]))
        ops.linear(x, self.w_in, out=proj, status=ctx.status, before=before)
        out = ctx.buffer("parallel.out", (n, self.width))
        if self.combine == "weighted_sum":
            outs = [branch.run(proj[:, at: at + rows], ctx, binding, out_dtype=torch.float32)
                    for branch, at, rows, binding in zip(self.branches, self.offsets, self.rows,
                                                         cache.parts)]
            ops.scaled_sum(outs[0], outs[1], self.scales[0], self.scales[1], out)
            return out
        outs = [branch.run(proj[:, at: at + rows], ctx, binding)
                for branch, at, rows, binding in zip(self.branches, self.offsets, self.rows,
                                                     cache.parts)]
        rk.mean_of_normed(outs[0], outs[1], self.out_weights[0], self.out_weights[1], out,
                          self.eps)
        return out


register_mixer("parallel", ParallelMixer)
