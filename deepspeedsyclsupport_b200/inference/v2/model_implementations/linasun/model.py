"""Linasun: a decoder-only family built from
  * an fp32 residual stream that starts as token embedding + sinusoidal position vector,
  * blocks that RMS-norm every sublayer on both sides, x += norm_b(sublayer(norm_a(x))), with zero-centred weights (applied as 1 + w),
  * a latent-attention mixer: queries through a normed low-rank latent, keys and values as per-head up-projections of ONE cached
    normed latent per token, no positional rotation, causal softmax, a sigmoid output gate computed from the mixer's input,
  * an optional mixture-of-experts feed-forward with a grouped, correction-biased top-k router and a clamped gated activation,
  * a loop: a contiguous range of layers may run several times in a row with the same weights, every pass with a cache of its own,
  * a final norm, the unembedding and a tanh soft cap on the logits.
Every size may differ from layer to layer; all of them, the layer order, the loop and the constants come from config.json.

The class reuses the ragged engine's plumbing from `RaggedTransformer` (containers and streamed loading, decode-step CUDA graphs,
the state manager's paged cache and block tables) and replaces the module set and the layer loop.  One cache layer exists per layer
RUN (a looped layer counts once per pass), each holding one row of that layer's `kv_rank` values per token."""
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ...inference_utils import ActivationType, DtypeEnum, NormTypeEnum
from ...modules import heuristics
from ...modules.configs import (DSEmbeddingsConfig, DSLatentAttentionConfig, DSLinearConfig, DSMoEConfig, DSNormConfig, DSUnembedConfig)
from ...ragged.manager_configs import KVCacheConfig
from ..inference_model_base import DSInferenceModelBase
from ..ragged_transformer import RaggedTransformer

SINUSOID_BASE = 10000.0  # fixed by the design
SWISH_ALPHA = 1.702  # fixed by the design: experts compute g * sigmoid(1.702 g) * (u + 1)
UP_SHIFT = 1.0
NORM_WEIGHT_OFFSET = 1.0  # block norms and the final norm keep a zero-centred weight; the latent norms store it plainly


@dataclass
class LinasunMixerSpec:
    heads: int
    dim: int  # query / key size per head
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float


@dataclass
class LinasunMoESpec:
    experts: int
    top: int
    groups: int
    keep: int
    ff: int
    limit: float


@dataclass
class LinasunLayerSpec:
    mixer: LinasunMixerSpec
    mlp: Optional[LinasunMoESpec]


@dataclass
class LinasunSpec:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    logit_softcap: float
    layers: List[LinasunLayerSpec] = field(default_factory=list)
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    family: str = "linasun"

    @property
    def num_layers(self):
        return len(self.layers)

    def run_order(self):
        """Layer index of every layer run, in execution order: layers before the loop, the looped range `times` times, the rest."""
        n = len(self.layers)
        a, b = self.loop_start, self.loop_stop
        return list(range(a)) + list(range(a, b)) * self.loop_times + list(range(b, n))

    @classmethod
    def from_config(cls, c: dict) -> "LinasunSpec":
        layers = []
        for i, lc in enumerate(c["layers"]):
            if lc["type"] != "latent_attention":
                raise ValueError(f"layer {i}: unknown mixer type '{lc['type']}'")
            m = lc["mixer"]
            mixer = LinasunMixerSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]),
                                     q_rank=int(m["q_rank"]), scale=float(m["scale"]))
            mlp = None
            if lc.get("mlp") is not None:
                f = lc["mlp"]
                if f.get("kind") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind '{f.get('kind')}'")
                r = f["router"]
                g = r.get("groups") or {"count": 1, "keep": 1}
                mlp = LinasunMoESpec(experts=int(r["experts"]), top=int(r["top"]), groups=int(g["count"]), keep=int(g["keep"]),
                                     ff=int(f["expert"]["ff"]), limit=float(f["expert"]["limit"]))
            layers.append(LinasunLayerSpec(mixer, mlp))
        loop = c.get("loop") or {}
        start, stop = int(loop.get("start", 0)), int(loop.get("stop", loop.get("start", 0)))
        times = int(loop.get("times", 1))
        if not (0 <= start <= stop <= len(layers)) or times < 0:
            raise ValueError(f"loop {loop} does not fit {len(layers)} layers")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]), norm_eps=float(c["norm"]["eps"]),
                   logit_softcap=float(c.get("logit_softcap", 0.0) or 0.0), layers=layers, loop_start=start, loop_stop=stop, loop_times=times)


class LinasunInferenceModel(RaggedTransformer, DSInferenceModelBase):
    describes_own_cache = True  # the engine builds its paged cache from `kv_cache_config` below

    def __init__(self, spec: LinasunSpec, tp_group=None, dtype=torch.bfloat16, device=None, engine_config=None, layer_container_cls=None,
                 non_transformer_container_cls=None, quantization_mode=""):
        from .container import LinasunNonTransformerContainer, LinasunTransformerContainer
        assert dtype in (torch.bfloat16, torch.float32), "Linasun runs with bf16 or fp32 activations"
        assert not quantization_mode, "Linasun has no quantised linears"
        self._loading_layer = 0
        self._init_plumbing(spec, tp_group, dtype, device, engine_config)
        assert self.tp == 1, "Linasun is served on one GPU per replica (no tensor-parallel sharding of the latent mixers yet)"
        self.hq = self.hkv = 0
        self.vocab_padded = spec.vocab_size
        self._build_modules()
        lc = layer_container_cls or LinasunTransformerContainer
        self.layers = [lc(self, i) for i in range(spec.num_layers)]
        self.non_transformer = (non_transformer_container_cls or LinasunNonTransformerContainer)(self)
        self._order = spec.run_order()
        self._layer_hook = None  # debugging aid: called as hook(run index, fp32 residual) after every layer run

    # ---- facts the parameter classes ask for
    @property
    def n_experts(self):
        mlp = self.spec.layers[self._loading_layer].mlp
        return mlp.experts if mlp is not None else 0

    # ---- cache: one single-plane layer of kv_rank values per token for every layer run
    def kv_cache_config(self, block_size: int = 64):
        name = {torch.bfloat16: "bf16", torch.float32: "fp32"}[self.dtype]
        shapes = [(1, 1, self.attn_mods[li].cache_rank) for li in self._order]  # kv_rank, padded where the tensor-core kernel wants it
        return KVCacheConfig(block_size=block_size, cache_shape=(len(shapes), 1, max([s[2] for s in shapes] + [1])), cache_dtype=name,
                             layer_shapes=shapes)

    # ---- building blocks
    def _build_modules(self):
        s, ec, dt = self.spec, self.engine_config, DtypeEnum(self.dtype)
        sm = getattr(ec, "state_manager", None)
        max_tokens = getattr(sm, "max_ragged_batch_size", 768)
        max_seqs = getattr(sm, "max_ragged_sequence_count", 512)
        D = s.hidden_size
        self.embed_mod = heuristics.instantiate_embed(DSEmbeddingsConfig(max_tokens=max_tokens, residual_dtype=dt, embedding_dim=D,
                                                                         sinusoidal_base=SINUSOID_BASE), ec)
        self.norm_mod = heuristics.instantiate_pre_norm(DSNormConfig(max_tokens=max_tokens, type=NormTypeEnum.RMSNorm, channels=D,
                                                                      residual_dtype=DtypeEnum.fp32, input_dtype=dt, output_dtype=dt,
                                                                      eps=s.norm_eps, weight_offset=NORM_WEIGHT_OFFSET, sandwich=True), ec)
        self.lin_mod = heuristics.instantiate_linear(DSLinearConfig(max_tokens=max_tokens, in_channels=D, out_channels=D, input_dtype=dt,
                                                                    output_dtype=dt), None)
        self.attn_mods, self.moe_mods = [], []
        for L in s.layers:
            m = L.mixer
            self.attn_mods.append(heuristics.instantiate_attention(
                DSLatentAttentionConfig(max_tokens=max_tokens, n_heads=m.heads, qk_dim=m.dim, v_dim=m.vdim, kv_rank=m.kv_rank, q_rank=m.q_rank,
                                        scale=m.scale, eps=s.norm_eps, max_sequences=max_seqs, input_dtype=dt, output_dtype=dt), ec))
            f = L.mlp
            self.moe_mods.append(None if f is None else heuristics.instantiate_moe(
                DSMoEConfig(max_tokens=max_tokens, model_dim=D, intermediate_features=f.ff, n_experts=f.experts, top_k=f.top,
                            activation=ActivationType.ClampedSwiGLU, normalize_scores=False, n_groups=f.groups, keep_groups=f.keep,
                            use_correction=True, act_alpha=SWISH_ALPHA, act_limit=f.limit, act_shift=UP_SHIFT, input_dtype=dt, output_dtype=dt), ec))
        self.unembed_mod = heuristics.instantiate_unembed(DSUnembedConfig(max_tokens=max_tokens, dtype=dt, norm_type=NormTypeEnum.RMSNorm, model_dim=D,
                                                                          max_sequences=max_seqs, vocab_size=s.vocab_size, eps=s.norm_eps,
                                                                          norm_weight_offset=NORM_WEIGHT_OFFSET, logit_softcap=s.logit_softcap,
                                                                          residual_fp32=True), ec)

    # ---- parameter transforms
    def transform_embedding_param(self, param):
        return self._dev(self.embed_mod.transform_param(param))

    def transform_norm_param(self, param):
        return self._dev(self.norm_mod.transform_param(param))

    def transform_latent_norm_param(self, param):
        return self._dev(self.attn_mods[0].transform_norm_param(param))

    def transform_dense_param(self, param):
        return self._dev(self.lin_mod.transform_param(param))

    def transform_key_up_param(self, param, layer):
        return self._dev(self.attn_mods[layer].transform_key_up_param(param))

    def transform_value_up_param(self, param, layer):
        return self._dev(self.attn_mods[layer].transform_value_up_param(param))

    def transform_unembed_param(self, param):
        return self._dev(param.to(self.dtype).contiguous())

    def _any_moe(self):
        mods = [m for m in self.moe_mods if m is not None]
        assert mods, "a feed-forward tensor arrived for a model without feed-forward layers"
        return mods[0]

    def transform_moe_gate_param(self, param):
        return self._dev(self._any_moe().transform_gate_param(param))

    def transform_moe_mlp_1_param(self, param, gated=True):
        return self._dev(self._any_moe().transform_moe_mlp_1_param(param))

    def transform_moe_mlp_2_param(self, param):
        return self._dev(self._any_moe().transform_moe_mlp_2_param(param))

    def load_canonical(self, sd):
        """State dict with the family's own tensor names."""
        import re
        rx = re.compile(r"^l(\d+)\.(.*)$")
        for name, tensor in sd.items():
            m = rx.match(name)
            ok = self.layers[int(m.group(1))].set_dependency(m.group(2), tensor) if m else self.non_transformer.set_dependency(name, tensor)
            if not ok:
                raise KeyError(f"unexpected parameter '{name}' for family linasun")
        self.check_populated()

    def check_populated(self):
        super().check_populated()
        for i, (L, c) in enumerate(zip(self.spec.layers, self.layers)):
            if L.mlp is not None and any(k not in c for k in ("norm2_w", "norm2b_w", "router_w", "correction", "experts_gu", "experts_dn")):
                raise RuntimeError(f"layer {i}: feed-forward tensors are missing")

    # ---- forward
    def forward(self, batch, state_manager):
        """batch: finalized RaggedBatchWrapper.  Returns fp32 logits [batch.n_logit_rows, vocab]."""
        s, nt = self.spec, self.non_transformer
        x = self.embed_mod(batch, nt.embed)  # fp32 residual stream [T, width]
        order = self._order
        if not order:
            return self.unembed_mod(x, nt.lm_head, batch, gamma=nt.final_norm_w)
        _, h = self.norm_mod(x, None, self.layers[order[0]]["norm1_w"])
        for run, li in enumerate(order):
            L, m = self.layers[li], s.layers[li].mixer
            nxt = self.layers[order[run + 1]]["norm1_w"] if run + 1 < len(order) else None
            fused = self.lin_mod(h, L["in_w"])  # (query latent | key/value latent | gate)
            a = self.attn_mods[li](fused, state_manager.get_cache(run), batch, L["dq_norm_w"], L["dkv_norm_w"], L["uq_w"], L["uk_w"], L["uv_w"],
                                   gate=fused[:, m.q_rank + m.kv_rank:m.q_rank + m.kv_rank + m.heads * m.vdim])
            y = self.lin_mod(a, L["o_w"])
            if self.moe_mods[li] is None:
                _, h = self.norm_mod(x, y, nxt, branch_gamma=L["norm1b_w"])
            else:
                # the router decides on the normed activations before their rounding (same pass, no separate conversion)
                _, h, h32 = self.norm_mod(x, y, L["norm2_w"], branch_gamma=L["norm1b_w"], fp32_copy=True)
                y = self.moe_mods[li](h, L["router_w"], L["experts_gu"], L["experts_dn"], correction=L["correction"], router_input=h32)
                _, h = self.norm_mod(x, y, nxt, branch_gamma=L["norm2b_w"])
            if self._layer_hook is not None:
                self._layer_hook(run, x)
        return self.unembed_mod(x, nt.lm_head, batch, gamma=nt.final_norm_w)
