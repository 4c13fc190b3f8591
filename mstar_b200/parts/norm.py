"""RMSNorm part, fused with the residual add that precedes it.

out = x * rsqrt(mean(x^2) + eps) * (weight + weight_offset), x the float residual
after adding the pending part output.  Llama mode multiplies by ``weight``
(mstar/model/components/norm.py:45-59); ``weight_offset=1`` gives the ``1 + weight``
form the reference calls gemma_mode (norm.py:46-52).  The reference down-casts
float input to bfloat16 before the library norm (mstar/utils/flashinfer_utils.py:
38-40); here sums and the scale are float in both dtypes.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import ResidualStream, Runtime
from .registry import register_part


class RMSNorm:
    graph_safe = True       # nothing per-step is read from the host

    @classmethod
    def param_specs(cls, spec) -> dict:
        # a weight stored as an offset from one starts at zero
        return {"weight": ParamSpec(shape=(spec.size,), role="vector",
                                    init="zeros" if spec.weight_offset else "ones")}

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime
        self.weight = params["weight"]
        if tuple(self.weight.shape) != (spec.size,):
            raise ValueError(f"rmsnorm weight has shape {tuple(self.weight.shape)}, "
                             f"expected ({spec.size},)")

    def _float_weight(self) -> torch.Tensor:
        if getattr(self, "_weight_f32", None) is None:
            self._weight_f32 = self.weight.float().contiguous()
        return self._weight_f32

    def add_normed(self, resid: torch.Tensor, delta: torch.Tensor, scale: float = 1.0,
                   rows_dtype=None):
        """resid += scale * norm(delta): this norm applied to a part's output on its way into
        the float residual (the norm after a sublayer).  With ``rows_dtype`` the new residual
        is returned as rows of that dtype, from the same kernel."""
        return ops.add_postnorm_rmsnorm(resid, delta, self._float_weight(), self.spec.eps,
                                        self.spec.weight_offset, post_scale=scale,
                                        out_dtype=rows_dtype, plain_out=rows_dtype is not None)

    def add_norm(self, stream: ResidualStream) -> torch.Tensor:
        """Fold the pending delta into the residual and return the normed rows."""
        scale = stream.post_scale
        delta, post = stream.take_pending()
        if post is None and hasattr(delta, "materialize"):
            # a part's output that is not computed yet and carries no norm of its own
            delta = ops.convert(delta.materialize(), self.runtime.dtype)
        if post is not None:
            if isinstance(post, RMSNorm):
                # the sublayer's own norm, the residual sum and this norm as one kernel
                return ops.add_postnorm_rmsnorm(
                    stream.h, delta, post._float_weight(), post.spec.eps, post.spec.weight_offset,
                    self.weight, self.spec.eps, self.spec.weight_offset, self.runtime.dtype,
                    post_scale=scale)
            post.add_normed(stream.h, delta, scale)
            delta = None
        # a pending delta is the output of the part before: its kernels lie between this
        # norm and whatever wrote the residual last
        return ops.add_rmsnorm(stream.h, delta, self.weight, self.spec.eps, self.runtime.dtype,
                               self.spec.weight_offset, resid_static=delta is not None)

    def norm_rows(self, rows_f32: torch.Tensor) -> torch.Tensor:
        """Norm of float rows that carry no pending delta (the final norm on the
        gathered rows)."""
        return ops.add_rmsnorm(rows_f32, None, self.weight, self.spec.eps, self.runtime.dtype,
                               self.spec.weight_offset)


register_part("norm", "rmsnorm", RMSNorm)
