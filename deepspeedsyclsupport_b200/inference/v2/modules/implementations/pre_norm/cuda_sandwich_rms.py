"""RMS norms of a block that norms every sublayer on both sides, on an fp32 residual stream:

    x <- x + mult * rms_norm(branch) * (w_branch + offset)     (the sublayer's output, normed before it joins the stream)
    out = rms_norm(x) * (w + offset)                           (the next sublayer's input, in the activation dtype)
    out = x                                                    (`emit_stream`: designs whose sublayers read the stream unnormed)

Both happen in one pass over the token's row (csrc/ragged/latent_ops.cu `sandwich_norm`).  `offset` is 1 for weights stored around
zero.  The statistics, the weights and the stream itself are fp32 whatever the activation dtype is."""
from typing import Any, Dict, Optional, Tuple

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum, NormTypeEnum
from ...configs import DSNormConfig
from ...interfaces import DSPreNormBase, DSPreNormRegistry


@DSPreNormRegistry.register_module
class DSSandwichRMSNorm(DSPreNormBase):

    @staticmethod
    def name() -> str:
        return "cuda_sandwich_rms"

    @staticmethod
    def supports_config(config: DSNormConfig) -> bool:
        return (NormTypeEnum(config.type) == NormTypeEnum.RMSNorm and config.sandwich and DtypeEnum(config.residual_dtype) == DtypeEnum.fp32 and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32) and DtypeEnum(config.output_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def transform_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, residual: torch.Tensor, hidden_states: Optional[torch.Tensor], gamma: Optional[torch.Tensor],
                beta: Optional[torch.Tensor] = None, branch_gamma: Optional[torch.Tensor] = None, fp32_copy: bool = False,
                emit_stream: bool = False):
        """residual: fp32 stream (updated in place).  hidden_states: the finished sublayer's output or None; branch_gamma: the weight
        of the norm applied to it.  gamma: weight of the norm that feeds the next sublayer, None when nothing follows.
        Returns (residual, normed input of the next sublayer or None); with `fp32_copy` a third value: the same normed input before
        its rounding to the activation dtype (what an fp32 router should decide on).  `emit_stream` (with gamma None): the second value
        is the updated stream itself in the activation dtype (the stream tensor when that is fp32)."""
        c = self._config
        assert beta is None, "RMS norms have no shift"
        out_dtype = DtypeEnum(c.output_dtype).value
        plain = emit_stream and gamma is None and out_dtype != torch.float32
        out = K.sandwich_norm(residual, hidden_states, branch_gamma, c.weight_offset, gamma, c.weight_offset, c.eps,
                              out_dtype=out_dtype, fp32_copy=fp32_copy, y_mult=c.branch_mult, plain_out=plain)
        if emit_stream and gamma is None and not plain:
            out = residual
        if fp32_copy:
            return residual, out[0], out[1]
        return residual, out
