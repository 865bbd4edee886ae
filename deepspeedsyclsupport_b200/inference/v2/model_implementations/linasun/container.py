"""Containers of the Linasun family: tensor names of its checkpoints -> parameters of the inference model.

A layer's tensors are `l<i>.norm1 / norm1b / norm2 / norm2b`, `l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o}` and,
when the layer has a feed-forward, `l<i>.mlp.{router, correction, e<j>.gate, e<j>.up, e<j>.down}`; outside the layers `embed`,
`final.norm` and `head`.  Linear weights have shape [out, in]."""
from typing import Optional

import torch

from ..common_parameters import (EmbeddingParameter, MoEGatingWeightParameter, NormParameter, UnembedParameter, UnfusedMoEGatedMLPParameter,
                                 UnfusedMoEMLP2Parameter)
from ..layer_container_base import LayerContainer
from ..parameter_base import ParameterBase


class FusedInputProjectionParameter(ParameterBase):
    """Everything a latent-attention mixer projects straight from its input, stacked into one weight so that one GEMM serves all
    of it: (query down-projection | key/value down-projection | output gate)."""
    dq: torch.Tensor
    dkv: torch.Tensor
    gate: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.dq, self.dkv, self.gate], dim=0))


class DenseParameter(ParameterBase):
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(self.params)


class LatentNormParameter(ParameterBase):
    """Plain weight of the RMS norm of a latent (fp32)."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_latent_norm_param(self.params)


class KeyUpParameter(ParameterBase):
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_key_up_param(self.params, self.layer_index)


class ValueUpParameter(ParameterBase):
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_value_up_param(self.params, self.layer_index)


class RouterCorrectionParameter(ParameterBase):
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_moe_gate_param(self.params)


class LinasunTransformerContainer(LayerContainer):
    norm1_w: NormParameter
    norm1b_w: NormParameter
    norm2_w: Optional[NormParameter]
    norm2b_w: Optional[NormParameter]
    in_w: FusedInputProjectionParameter
    dq_norm_w: LatentNormParameter
    dkv_norm_w: LatentNormParameter
    uq_w: DenseParameter
    uk_w: KeyUpParameter
    uv_w: ValueUpParameter
    o_w: DenseParameter
    router_w: Optional[MoEGatingWeightParameter]
    correction: Optional[RouterCorrectionParameter]
    experts_gu: Optional[UnfusedMoEGatedMLPParameter]
    experts_dn: Optional[UnfusedMoEMLP2Parameter]

    PARAM_MAPPING = {
        "norm1": "norm1_w.params",
        "norm1b": "norm1b_w.params",
        "norm2": "norm2_w.params",
        "norm2b": "norm2b_w.params",
        "mix.dq": "in_w.dq",
        "mix.dkv": "in_w.dkv",
        "mix.g": "in_w.gate",
        "mix.dq.norm": "dq_norm_w.params",
        "mix.dkv.norm": "dkv_norm_w.params",
        "mix.uq": "uq_w.params",
        "mix.uk": "uk_w.params",
        "mix.uv": "uv_w.params",
        "mix.o": "o_w.params",
        "mlp.router": "router_w.params",
        "mlp.correction": "correction.params",
        "mlp.e*.gate": "experts_gu.gating_experts",
        "mlp.e*.up": "experts_gu.up_experts",
        "mlp.e*.down": "experts_dn.experts",
    }

    def __init__(self, model, layer_index: int) -> None:
        self.layer_index = layer_index  # the expert lists and the reshapes below are sized per layer
        model._loading_layer = layer_index
        super().__init__(model)
        for p in self._params.values():
            p.layer_index = layer_index


class LinasunNonTransformerContainer(LayerContainer):
    embed: EmbeddingParameter
    final_norm_w: NormParameter
    lm_head: UnembedParameter

    PARAM_MAPPING = {"embed": "embed.params", "final.norm": "final_norm_w.params", "head": "lm_head.params"}
