"""Attention over a paged cache of low-rank latents (one row of `kv_rank` values per token and layer instead of per-head keys
and values).

With k_h = U_h c and v_h = V_h c for the cached latent c, the score q_h . k_h equals (U_h^T q_h) . c and the head's output is
V_h (sum_j p_j c_j): the queries are mapped into the latent space once per token, all heads of a token then share the cached rows
as keys AND values, and the value up-projection is applied to the attended latent.  Nothing but c is ever cached or expanded,
for prompt chunks and decode steps alike.

Per layer: fused norm-of-both-latents + cache append, query up-projection, per-head map into the latent space (batched GEMM),
`latent_attention` (causal softmax in fp32; split along the keys when the batch is small), per-head value up-projection
(batched GEMM), optional elementwise output gate sigmoid(g)."""
from typing import Any, Dict, Optional, Type

import torch

from ......ops.gemm import dense_matmul
from .... import kernels as K
from ....inference_parameter import InferenceParameter
from ....inference_utils import DtypeEnum
from ...configs import DSLatentAttentionConfig
from ...interfaces import DSSelfAttentionBase, DSSelfAttentionRegistry


def _bmm(a, b, out_dtype):
    """Batched a @ b with fp32 accumulation; fp32 operands in true fp32."""
    if a.dtype == torch.float32:
        keep = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            return torch.bmm(a, b)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = keep
    if out_dtype == torch.float32:
        try:
            return torch.bmm(a, b, out_dtype=torch.float32)
        except (TypeError, RuntimeError):
            return torch.bmm(a, b).float()
    return torch.bmm(a, b)


@DSSelfAttentionRegistry.register_module
class DSLatentBlockedAttention(DSSelfAttentionBase):

    @staticmethod
    def name() -> str:
        return "latent_blocked_attention"

    @staticmethod
    def config_class() -> Type[DSLatentAttentionConfig]:
        return DSLatentAttentionConfig

    @staticmethod
    def supports_config(config) -> bool:
        return (isinstance(config, DSLatentAttentionConfig) and config.input_dtype == config.output_dtype and
                DtypeEnum(config.input_dtype) in (DtypeEnum.bf16, DtypeEnum.fp32))

    def __init__(self, config: DSLatentAttentionConfig, implementation_config: Dict[str, Any] = None) -> None:
        super().__init__(config, implementation_config)
        self._dtype = DtypeEnum(config.input_dtype).value

    @property
    def kv_block_size(self) -> int:
        return 64

    @property
    def q_block_size(self) -> int:
        return 1

    # ---- parameter layouts
    def transform_norm_param(self, param: torch.Tensor) -> InferenceParameter:
        return InferenceParameter.initialize(param.to(torch.float32).contiguous())

    def transform_key_up_param(self, param: torch.Tensor) -> InferenceParameter:
        """[heads * qk_dim, kv_rank] -> [heads, qk_dim, kv_rank]: right operand of the per-head query map q_h -> U_h^T q_h."""
        c = self._config
        return InferenceParameter.initialize(param.to(self._dtype).reshape(c.n_heads, c.qk_dim, c.kv_rank).contiguous())

    def transform_value_up_param(self, param: torch.Tensor) -> InferenceParameter:
        """[heads * v_dim, kv_rank] -> [heads, kv_rank, v_dim]: right operand of the per-head value up-projection."""
        c = self._config
        return InferenceParameter.initialize(param.to(self._dtype).reshape(c.n_heads, c.v_dim, c.kv_rank).transpose(1, 2).contiguous())

    # ---- forward
    def forward(self, latents: torch.Tensor, kv_cache: torch.Tensor, batch, q_norm_w: torch.Tensor, kv_norm_w: torch.Tensor,
                q_up_w: torch.Tensor, key_up_w: torch.Tensor, value_up_w: torch.Tensor, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """latents [T, >= q_rank + kv_rank]: (query latent | key/value latent) before their norms, unit column stride.
        kv_cache [blocks, block_size, 1, kv_rank].  gate [T, heads * v_dim] (optional, any row stride): the result is multiplied by
        sigmoid(gate).  Returns [T, heads * v_dim]."""
        c = self._config
        T, H = latents.shape[0], c.n_heads
        cache = kv_cache.view(kv_cache.shape[0], kv_cache.shape[1], c.kv_rank)
        tok_seq, tok_pos, bt = batch.tok_seq(), batch.tok_pos(), batch.block_table()
        cq = K.latent_norm_append(latents, q_norm_w, kv_norm_w, cache, tok_seq, tok_pos, bt, c.q_rank, c.kv_rank, c.eps)
        q = dense_matmul(cq, q_up_w)  # [T, H * qk_dim]
        q_abs = _bmm(q.view(T, H, c.qk_dim).transpose(0, 1), key_up_w, torch.float32)  # [H, T, kv_rank]
        att = torch.empty(H, T, c.kv_rank, dtype=torch.float32, device=latents.device)
        K.latent_attention(q_abs.transpose(0, 1), cache, tok_seq, tok_pos, bt, c.scale, out=att.transpose(0, 1))
        o = _bmm(att if self._dtype == torch.float32 else att.to(self._dtype), value_up_w, self._dtype)  # [H, T, v_dim]
        o = o.transpose(0, 1).reshape(T, H * c.v_dim)
        if gate is not None:
            K.sigmoid_gate_mul(o, gate)
        return o
