"""Containers of the Kulanex family: tensor names of its checkpoints -> parameters of the inference model.

Every layer has `l<i>.norm1` and, with a feed-forward, `l<i>.norm2` and `l<i>.mlp.{router, e<j>.gate, e<j>.up, e<j>.down}`.  A 'parallel'
layer's mixer is `l<i>.mix.left.{q, k, q.conv, k.conv, q.norm, k.norm, o}` (windowed attention) and
`l<i>.mix.right.{q, k, v, g, o, norm, i, i.b, f, f.b}` (matrix memory); a 'channel_delta' layer's is
`l<i>.mix.{q, k, v, q.conv, k.conv, v.conv, b, a1, a2, dt_bias, A_log, g1, g2, norm, o}`.  Outside the layers: `embed`, `final.norm`,
`head`.  Linear weights have shape [out, in]."""
from typing import Optional

import torch

from ..common_parameters import (EmbeddingParameter, MoEGatingWeightParameter, NormParameter, UnembedParameter, UnfusedMoEGatedMLPParameter,
                                 UnfusedMoEMLP2Parameter)
from ..layer_container_base import LayerContainer
from ..parameter_base import ParameterBase


class DenseParameter(ParameterBase):
    """A linear weight in the activation dtype."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(self.params)


class Fp32Parameter(ParameterBase):
    """Small tensors that enter norms, gates, decays or convolutions: kept fp32."""
    params: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_fp32_param(self.params)


class ParallelInputProjectionParameter(ParameterBase):
    """Everything the two halves of a 'parallel' mixer project straight from the layer input, stacked so that one GEMM serves all of it:
    (attention queries | attention keys | memory queries | memory keys | memory values | memory output gate)."""
    lq: torch.Tensor
    lk: torch.Tensor
    rq: torch.Tensor
    rk: torch.Tensor
    rv: torch.Tensor
    rg: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.lq, self.lk, self.rq, self.rk, self.rv, self.rg], dim=0))


class MemoryGateProjectionParameter(ParameterBase):
    """(input gate | forget gate) projections of the matrix memory, fp32: the gates are formed from the fp32 stream."""
    i: torch.Tensor
    f: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_fp32_param(torch.cat([self.i, self.f], dim=0))


class ParallelOutputProjectionParameter(ParameterBase):
    """(attention output | memory output) projections side by side along their input axis: the weighted sum of the two halves is one GEMM
    over their concatenated outputs (the weights of the sum are applied to the halves' outputs before they are rounded)."""
    left: torch.Tensor
    right: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.left, self.right], dim=1))


class DeltaInputProjectionParameter(ParameterBase):
    """(queries | keys | values | low-rank output-gate latent) of a delta-rule mixer as one weight."""
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    g1: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_dense_param(torch.cat([self.q, self.k, self.v, self.g1], dim=0))


class DeltaControlProjectionParameter(ParameterBase):
    """(write strength beta | low-rank decay latent) projections, fp32: both feed the recurrence."""
    b: torch.Tensor
    a1: torch.Tensor

    def finalize(self) -> torch.Tensor:
        return self.inference_model.transform_fp32_param(torch.cat([self.b, self.a1], dim=0))


class _KulanexLayerContainer(LayerContainer):

    def __init__(self, model, layer_index: int) -> None:
        self.layer_index = layer_index
        model._loading_layer = layer_index  # the expert lists are sized per layer
        super().__init__(model)
        for p in self._params.values():
            p.layer_index = layer_index


class KulanexParallelContainer(_KulanexLayerContainer):
    norm1_w: NormParameter
    norm2_w: Optional[NormParameter]
    in_w: ParallelInputProjectionParameter
    gates_w: MemoryGateProjectionParameter
    bias_i: Fp32Parameter
    bias_f: Fp32Parameter
    conv_q: Fp32Parameter
    conv_k: Fp32Parameter
    norm_q: Fp32Parameter
    norm_k: Fp32Parameter
    memory_norm: Fp32Parameter
    o_w: ParallelOutputProjectionParameter
    router_w: Optional[MoEGatingWeightParameter]
    experts_gu: Optional[UnfusedMoEGatedMLPParameter]
    experts_dn: Optional[UnfusedMoEMLP2Parameter]

    PARAM_MAPPING = {
        "norm1": "norm1_w.params",
        "norm2": "norm2_w.params",
        "mix.left.q": "in_w.lq",
        "mix.left.k": "in_w.lk",
        "mix.right.q": "in_w.rq",
        "mix.right.k": "in_w.rk",
        "mix.right.v": "in_w.rv",
        "mix.right.g": "in_w.rg",
        "mix.right.i": "gates_w.i",
        "mix.right.f": "gates_w.f",
        "mix.right.i.b": "bias_i.params",
        "mix.right.f.b": "bias_f.params",
        "mix.left.q.conv": "conv_q.params",
        "mix.left.k.conv": "conv_k.params",
        "mix.left.q.norm": "norm_q.params",
        "mix.left.k.norm": "norm_k.params",
        "mix.right.norm": "memory_norm.params",
        "mix.left.o": "o_w.left",
        "mix.right.o": "o_w.right",
        "mlp.router": "router_w.params",
        "mlp.e*.gate": "experts_gu.gating_experts",
        "mlp.e*.up": "experts_gu.up_experts",
        "mlp.e*.down": "experts_dn.experts",
    }


class KulanexDeltaContainer(_KulanexLayerContainer):
    norm1_w: NormParameter
    norm2_w: Optional[NormParameter]
    in_w: DeltaInputProjectionParameter
    control_w: DeltaControlProjectionParameter
    a2_w: Fp32Parameter
    dt_bias: Fp32Parameter
    A_log: Fp32Parameter
    g2_w: DenseParameter
    conv_q: Fp32Parameter
    conv_k: Fp32Parameter
    conv_v: Fp32Parameter
    mix_norm: Fp32Parameter
    o_w: DenseParameter
    router_w: Optional[MoEGatingWeightParameter]
    experts_gu: Optional[UnfusedMoEGatedMLPParameter]
    experts_dn: Optional[UnfusedMoEMLP2Parameter]

    PARAM_MAPPING = {
        "norm1": "norm1_w.params",
        "norm2": "norm2_w.params",
        "mix.q": "in_w.q",
        "mix.k": "in_w.k",
        "mix.v": "in_w.v",
        "mix.g1": "in_w.g1",
        "mix.b": "control_w.b",
        "mix.a1": "control_w.a1",
        "mix.a2": "a2_w.params",
        "mix.dt_bias": "dt_bias.params",
        "mix.A_log": "A_log.params",
        "mix.g2": "g2_w.params",
        "mix.q.conv": "conv_q.params",
        "mix.k.conv": "conv_k.params",
        "mix.v.conv": "conv_v.params",
        "mix.norm": "mix_norm.params",
        "mix.o": "o_w.params",
        "mlp.router": "router_w.params",
        "mlp.e*.gate": "experts_gu.gating_experts",
        "mlp.e*.up": "experts_gu.up_experts",
        "mlp.e*.down": "experts_dn.experts",
    }


class KulanexNonTransformerContainer(LayerContainer):
    embed: EmbeddingParameter
    final_norm_w: NormParameter
    lm_head: UnembedParameter

    PARAM_MAPPING = {"embed": "embed.params", "final.norm": "final_norm_w.params", "head": "lm_head.params"}
