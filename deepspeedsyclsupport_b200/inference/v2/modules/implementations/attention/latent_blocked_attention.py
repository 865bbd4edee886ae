"""Attention over a paged cache of low-rank latents (one row of `kv_rank` values per token and layer instead of per-head keys
and values).

With k_h = U_h c and v_h = V_h c for the cached latent c, the score q_h . k_h equals (U_h^T q_h) . c and the head's output is
V_h (sum_j p_j c_j): the queries are mapped into the latent space once per token, all heads of a token then share the cached rows
as keys AND values, and the value up-projection is applied to the attended latent.  Nothing but c is ever cached or expanded,
for prompt chunks and decode steps alike.

Per layer: fused norm-of-both-latents + cache append, query up-projection, per-head map into the latent space (batched GEMM),
the attention kernel, per-head value up-projection (batched GEMM), optional elementwise output gate sigmoid(g).

Two attention kernels.  bf16 with kv_rank <= 128: the tcgen05 paged flash kernels in their one-plane mode (the cached row is key and
value; TMA pages, S / P / O in TMEM) -- cache rows are padded with zeros to 64 or 128 values and the query heads with zero heads to a
divisor of 128, which changes neither scores nor outputs.  Everything else (fp32, larger ranks): `latent_attention`, a CUDA-core
kernel with fp32 scores and accumulation that takes any size (split along the keys when the batch is small)."""
import os
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
        c = config
        self._flash = (self._dtype == torch.bfloat16 and c.kv_rank <= 128 and c.n_heads <= 128 and os.environ.get("DSB200_LATENT_FLASH", "1") != "0")
        self._rank = (64 if c.kv_rank <= 64 else 128) if self._flash else c.kv_rank  # width of a cached row
        self._heads_p = 1
        while self._heads_p < c.n_heads:
            self._heads_p *= 2

    @property
    def cache_rank(self) -> int:
        """Values per cached row (kv_rank, or its padding to what the tensor-core kernel takes)."""
        return self._rank

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
        w = param.to(self._dtype).reshape(c.n_heads, c.qk_dim, c.kv_rank)
        if self._rank > c.kv_rank:  # zero columns: the padded part of a latent-space query is zero
            w = torch.nn.functional.pad(w, (0, self._rank - c.kv_rank))
        return InferenceParameter.initialize(w.contiguous())

    def transform_value_up_param(self, param: torch.Tensor) -> InferenceParameter:
        """[heads * v_dim, kv_rank] -> [heads, kv_rank, v_dim]: right operand of the per-head value up-projection."""
        c = self._config
        w = param.to(self._dtype).reshape(c.n_heads, c.v_dim, c.kv_rank).transpose(1, 2)
        if self._rank > c.kv_rank:  # zero rows: the padded part of an attended latent contributes nothing
            w = torch.nn.functional.pad(w, (0, 0, 0, self._rank - c.kv_rank))
        return InferenceParameter.initialize(w.contiguous())

    # ---- forward
    def forward(self, latents: torch.Tensor, kv_cache: torch.Tensor, batch, q_norm_w: torch.Tensor, kv_norm_w: torch.Tensor,
                q_up_w: torch.Tensor, key_up_w: torch.Tensor, value_up_w: torch.Tensor, gate: Optional[torch.Tensor] = None) -> torch.Tensor:
        """latents [T, >= q_rank + kv_rank]: (query latent | key/value latent) before their norms, unit column stride.
        kv_cache [blocks, block_size, 1, kv_rank].  gate [T, heads * v_dim] (optional, any row stride): the result is multiplied by
        sigmoid(gate).  Returns [T, heads * v_dim]."""
        c = self._config
        T, H, R = latents.shape[0], c.n_heads, self._rank
        cache = kv_cache.view(kv_cache.shape[0], kv_cache.shape[1], R)
        tok_seq, tok_pos, bt = batch.tok_seq(), batch.tok_pos(), batch.block_table()
        cq = K.latent_norm_append(latents, q_norm_w, kv_norm_w, cache, tok_seq, tok_pos, bt, c.q_rank, c.kv_rank, c.eps)
        q = dense_matmul(cq, q_up_w).reshape(T, H, c.qk_dim).transpose(0, 1)  # [H, T, qk_dim]
        bs = cache.shape[1]
        if self._flash and bs >= 8 and 128 % bs == 0:
            qa = torch.bmm(q, key_up_w)  # [H, T, R]; the kernel reads it head-major through its TMA strides, missing heads as zeros
            att = K.paged_latent_flash(qa.transpose(0, 1), cache, tok_seq, tok_pos, bt, c.scale, heads=self._heads_p,
                                       decode=batch.current_tokens <= 2 * batch.current_sequences)
            o = torch.bmm(att[:, :H].transpose(0, 1), value_up_w)  # [H, T, v_dim]
        else:
            q_abs = _bmm(q, key_up_w, torch.float32)  # [H, T, R]
            att = torch.empty(H, T, R, dtype=torch.float32, device=latents.device)
            K.latent_attention(q_abs.transpose(0, 1), cache, tok_seq, tok_pos, bt, c.scale, out=att.transpose(0, 1))
            o = _bmm(att if self._dtype == torch.float32 else att.to(self._dtype), value_up_w, self._dtype)  # [H, T, v_dim]
        if gate is not None:
            return K.gate_heads(o.contiguous(), gate)  # heads side by side per token and the gate, one pass
        return o.transpose(0, 1).reshape(T, H * c.v_dim)
