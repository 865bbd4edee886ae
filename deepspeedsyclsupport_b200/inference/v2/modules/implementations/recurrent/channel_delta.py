"""Gated delta rule with one decay per head and key channel (one d x dv matrix per head and sequence, plus the tails of three short
convolutions).

Per layer and step: `delta_prepare` (convolutions + silu, unit-length q and k, decays and betas; all tokens in parallel),
`conv_state_update`, the scan kernel (`delta_rule_scan`: the state stays in registers over a sequence's new tokens, inputs are prefetched a
chunk ahead), `head_norm_gate`.  csrc/ragged/recurrent_ops.cu.  Everything that enters the recurrence is fp32 whatever the activation dtype."""
from typing import Any, Dict, List, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ....ragged.state_slots import StateBufferSpec
from ...configs import DSDeltaRuleConfig
from ...interfaces import DSRecurrentMixerBase, DSRecurrentRegistry


@DSRecurrentRegistry.register_module
class DSChannelDeltaRule(DSRecurrentMixerBase):

    @staticmethod
    def name() -> str:
        return "channel_delta_rule"

    @staticmethod
    def config_class() -> Type[DSDeltaRuleConfig]:
        return DSDeltaRuleConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSDeltaRuleConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32) and config.n_heads >= 1 and config.n_heads_qk >= 1 and
                config.n_heads % config.n_heads_qk == 0 and config.key_size >= 1 and config.key_size <= 2048 and config.value_size >= 1 and
                config.conv_taps >= 1)

    def __init__(self, config: DSDeltaRuleConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value

    @property
    def conv_channels(self) -> int:
        c = self._config
        return 2 * c.n_heads_qk * c.key_size + c.n_heads * c.value_size

    def state_specs(self, prefix: str) -> List[StateBufferSpec]:
        c = self._config
        specs = [StateBufferSpec(prefix + ".S", (c.n_heads, K.scan_state_floats(c.key_size, c.value_size)), torch.float32)]
        if c.conv_taps > 1:
            specs.append(StateBufferSpec(prefix + ".conv", (c.conv_taps - 1, self.conv_channels), self._dtype))
        return specs

    def transform_fp32_param(self, param: torch.Tensor) -> InferenceParameter:
        """Convolution taps, decay rates, step biases and the read-out norm's weight stay fp32."""
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, proj: torch.Tensor, cols, beta_pre: torch.Tensor, a_pre: torch.Tensor, gate: torch.Tensor, conv_q: torch.Tensor,
                conv_k: torch.Tensor, conv_v: torch.Tensor, A_log: torch.Tensor, dt_bias: torch.Tensor, norm_w: torch.Tensor, batch,
                state_manager, prefix: str, out: torch.Tensor) -> torch.Tensor:
        """proj [T, N]: the fused projection with q | k | v side by side from column cols[0] (cols = their three offsets).  beta_pre fp32
        [T, heads], a_pre fp32 [T, heads * key_size] (before bias and softplus; both are overwritten), gate [T, heads * value_size] (before the
        sigmoid).
        out: [T, heads * value_size] view that receives the result."""
        c = self._config
        q0, k0, v0 = cols
        nqk = c.n_heads_qk * c.key_size
        assert k0 == q0 + nqk and v0 == k0 + nqk, "the convolved projections sit side by side (q | k | v)"
        desc, n_seqs = batch.seq_desc(), batch.current_sequences
        conv_state = state_manager.get_state(prefix + ".conv") if c.conv_taps > 1 else None
        qn, kn, v = K.delta_prepare(proj, q0, k0, v0, conv_q, conv_k, conv_v, conv_state, desc, batch.tok_seq(), a_pre, beta_pre, A_log, dt_bias,
                                    c.n_heads_qk, c.n_heads, c.key_size, c.value_size, c.conv_taps)  # a_pre -> decays, beta_pre -> betas, in place
        if conv_state is not None:
            K.conv_state_update(proj, q0, self.conv_channels, conv_state, 0, desc, n_seqs, c.conv_taps)
        o = K.delta_rule_scan(qn, kn, v, beta_pre, a_pre, desc, n_seqs, state_manager.get_state(prefix + ".S"), c.n_heads, c.n_heads_qk, c.key_size,
                              c.value_size)
        return K.head_norm_gate(o, norm_w, gate, out, c.n_heads, c.value_size, c.eps, mult=c.out_scale, shared_weight=True)
