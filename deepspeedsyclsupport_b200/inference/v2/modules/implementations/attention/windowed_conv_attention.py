"""Sliding-window attention with kept first tokens over a paged cache, for mixers whose queries and keys pass a short causal convolution,
a whole-projection RMS norm and an interleaved partial rotation, and whose values are the convolved keys.

Per layer and step: `window_qk_prepare` (convolution from the batch rows and the sequence's kept rows; values into cache plane 1; norms;
rotation with angles formed in double precision; keys into plane 0), `conv_state_update`, then the attention kernel over the visible keys
[0, keep_first) + the last `window`.  The cache is [blocks, 2, block_size, kv_heads, head_size], the layout of the dense attention's
cache, so both kinds of layer share the block ids of a sequence.  csrc/ragged/recurrent_ops.cu.

Two attention kernels.  bf16 with head size 64 / 128: the tcgen05 paged flash kernels (csrc/attn/paged_flash.cu) with the window, the kept
keys and a page list that skips what lies between them.  Everything else (fp32, other head sizes): `window_attention`, a CUDA-core kernel
with fp32 scores and accumulation that takes any size."""
import math
from typing import Any, Dict, List, Type

import torch

from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ....ragged.state_slots import StateBufferSpec
from ...configs import DSWindowedAttentionConfig
from ...interfaces import DSSelfAttentionBase, DSSelfAttentionRegistry


def scaled_rotary_frequencies(rotate_dim, theta_base, scaling=None):
    """float64 [rotate_dim / 2]: f_i = theta_base^(-2i / rotate_dim), long wavelengths slowed down as `RotaryScalingConfig` describes."""
    out = []
    for i in range(rotate_dim // 2):
        f = float(theta_base) ** (-2.0 * i / rotate_dim)
        if scaling is not None:
            wavelength = 2.0 * math.pi / f
            if wavelength > scaling.original / scaling.low:
                f = f / scaling.factor
            elif wavelength >= scaling.original / scaling.high:
                s = (scaling.original / wavelength - scaling.low) / (scaling.high - scaling.low)
                f = (1.0 - s) * f / scaling.factor + s * f
        out.append(f)
    return torch.tensor(out, dtype=torch.float64)


def windowed_attention(q, kv_cache, tok_seq, tok_pos, block_table, out, H, G, d, window, keep_first, scale, out_scale=1.0, decode=False):
    """Attention of q [T, H d] over the paged cache with the sliding window and the kept first keys, into `out` (a [T, H d] view)."""
    if K.paged_flash_window_ok(q, kv_cache, out, H, G, d):
        return K.paged_flash_window(q, kv_cache, tok_seq, tok_pos, block_table, out, H, G, d, window, keep_first, scale, out_scale=out_scale, decode=decode)
    return K.window_attention(q, kv_cache, tok_seq, tok_pos, block_table, out, H, G, d, window, keep_first, scale, out_scale=out_scale)


@DSSelfAttentionRegistry.register_module
class DSWindowedConvAttention(DSSelfAttentionBase):

    @staticmethod
    def name() -> str:
        return "windowed_conv_attention"

    @staticmethod
    def config_class() -> Type[DSWindowedAttentionConfig]:
        return DSWindowedAttentionConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSWindowedAttentionConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def __init__(self, config: DSWindowedAttentionConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value
        self._freq_host = scaled_rotary_frequencies(config.rotate_dim, config.theta_base, config.rotary_scaling)
        self._freq = None

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    @property
    def conv_channels(self) -> int:
        c = self._config
        return (c.n_heads_q + c.n_heads_kv) * c.head_size

    def state_specs(self, prefix: str) -> List[StateBufferSpec]:
        c = self._config
        return [StateBufferSpec(prefix + ".conv", (c.conv_taps - 1, self.conv_channels), self._dtype)] if c.conv_taps > 1 else []

    def transform_fp32_param(self, param: torch.Tensor) -> InferenceParameter:
        """Convolution taps and the norm weights stay fp32."""
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def forward(self, proj: torch.Tensor, cols, kv_cache: torch.Tensor, batch, conv_q: torch.Tensor, conv_k: torch.Tensor, norm_q: torch.Tensor,
                norm_k: torch.Tensor, state_manager, prefix: str, out: torch.Tensor) -> torch.Tensor:
        """proj [T, N]: the fused projection with queries at column cols[0] and keys right behind them at cols[1].  kv_cache
        [blocks, 2, block_size, kv_heads, head_size].  out: [T, heads * head_size] view that receives out_scale * attention."""
        c = self._config
        q0, k0 = cols
        H, G, d = c.n_heads_q, c.n_heads_kv, c.head_size
        assert k0 == q0 + H * d, "the convolved projections sit side by side (q | k)"
        if self._freq is None or self._freq.device != proj.device:
            self._freq = self._freq_host.to(proj.device)
        desc = batch.seq_desc()
        conv_state = state_manager.get_state(prefix + ".conv") if c.conv_taps > 1 else None
        q = torch.empty(proj.shape[0], H * d, dtype=proj.dtype, device=proj.device)
        K.window_qk_prepare(proj, q0, k0, conv_q, conv_k, norm_q, norm_k, conv_state, desc, batch.tok_seq(), batch.tok_pos(), batch.block_table(),
                            kv_cache, q, self._freq, H, G, d, c.conv_taps, c.rotate_dim, c.eps)
        if conv_state is not None:
            K.conv_state_update(proj, q0, self.conv_channels, conv_state, 0, desc, batch.current_sequences, c.conv_taps)
        return windowed_attention(q, kv_cache, batch.tok_seq(), batch.tok_pos(), batch.block_table(), out, H, G, d, c.window, c.keep_first, c.scale,
                                  out_scale=c.out_scale, decode=batch.current_tokens <= 2 * batch.current_sequences)
