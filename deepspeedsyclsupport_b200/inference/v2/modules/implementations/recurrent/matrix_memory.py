"""Matrix memory with exponential gating (one d x dv matrix, a normaliser vector and a running log-maximum per head and sequence).

Per layer and step: the scan kernel walks every sequence's new tokens in order with the state in registers (prompt portions and decode
tokens alike; csrc/ragged/recurrent_ops.cu `matrix_memory_scan`), then one pass applies the per-head RMS norm, the weight, the sigmoid
output gate and the mixer's constant (`head_norm_gate`).  Gates, state and read-out are fp32 whatever the activation dtype."""
from typing import Any, Dict, List, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ....ragged.state_slots import StateBufferSpec
from ...configs import DSMatrixMemoryConfig
from ...interfaces import DSRecurrentMixerBase, DSRecurrentRegistry


@DSRecurrentRegistry.register_module
class DSMatrixMemory(DSRecurrentMixerBase):

    @staticmethod
    def name() -> str:
        return "matrix_memory"

    @staticmethod
    def config_class() -> Type[DSMatrixMemoryConfig]:
        return DSMatrixMemoryConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSMatrixMemoryConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32) and min(config.n_heads, config.key_size, config.value_size) >= 1 and
                config.key_size <= 2048 and config.gate_cap > 0)

    def __init__(self, config: DSMatrixMemoryConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value

    def state_specs(self, prefix: str) -> List[StateBufferSpec]:
        c = self._config
        return [StateBufferSpec(prefix + ".S", (c.n_heads, K.scan_state_floats(c.key_size, c.value_size)), torch.float32),
                StateBufferSpec(prefix + ".n", (c.n_heads, c.key_size), torch.float32),
                StateBufferSpec(prefix + ".m", (c.n_heads, ), torch.float32)]

    def transform_fp32_param(self, param: torch.Tensor) -> InferenceParameter:
        """Gate biases and the read-out norm's weight stay fp32."""
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, proj: torch.Tensor, cols, gates: torch.Tensor, bias_i: torch.Tensor, bias_f: torch.Tensor, norm_w: torch.Tensor, batch,
                state_manager, prefix: str, out: torch.Tensor) -> torch.Tensor:
        """proj [T, N]: the fused projection; cols = (q, k, v, output gate) column offsets in it.  gates fp32 [T, 2 heads] (input | forget
        pre-activations, without biases).  out: [T, heads * value_size] view that receives the result."""
        c = self._config
        q0, k0, v0, g0 = cols
        o = K.matrix_memory_scan(proj, q0, k0, v0, gates, bias_i, bias_f, c.gate_cap, batch.seq_desc(), batch.current_sequences,
                                 state_manager.get_state(prefix + ".S"), state_manager.get_state(prefix + ".n"),
                                 state_manager.get_state(prefix + ".m"), c.n_heads, c.key_size, c.value_size)
        n = c.n_heads * c.value_size
        return K.head_norm_gate(o, norm_w, proj[:, g0:g0 + n], out, c.n_heads, c.value_size, c.eps, mult=c.out_scale)
