"""Kulanex: a decoder-only family built from
  * an fp32 residual stream that starts as the token embedding; sublayers read the stream itself (no norm in front) and their OUTPUT is
    RMS-normed with a zero-centred weight (applied as 1 + w) and scaled by a constant before it joins: x += mult * norm(f(x)),
  * 'parallel' layers: a weighted sum of two mixers that read the same input -- sliding-window attention that keeps the first tokens
    visible (queries and keys pass a short causal convolution, a whole-projection RMS norm and an interleaved partial rotation with
    scaled frequencies; the values are the convolved keys) and a matrix memory with exponential gating,
  * 'channel_delta' layers: a gated delta rule with one decay per head and key channel behind short convolutions,
  * an optional mixture-of-experts feed-forward whose router scores are sigmoids that multiply the chosen experts' INPUT,
  * a final norm and the unembedding.
Every size may differ from layer to layer; all of them, the order of layers and the constants come from config.json.

The class reuses the ragged engine's plumbing from `RaggedTransformer` (containers and streamed loading, decode-step CUDA graphs, the state
manager's paged cache and block tables) and replaces the module set and the layer loop.  Attention layers get one (key, value) cache layer
each, all sharing a sequence's block ids; what the mixers carry besides (matrix memories, convolution tails) lives in the state manager's
per-sequence state slots, described by `state_config`."""
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .....ops.gemm import dense_matmul
from ...inference_utils import ActivationType, DtypeEnum, NormTypeEnum
from ...modules import heuristics
from ...modules.configs import (DSDeltaRuleConfig, DSEmbeddingsConfig, DSLinearConfig, DSMatrixMemoryConfig, DSMoEConfig, DSNormConfig,
                                DSUnembedConfig, DSWindowedAttentionConfig, RotaryScalingConfig)
from ...ragged.manager_configs import KVCacheConfig
from ..inference_model_base import DSInferenceModelBase
from ..ragged_transformer import RaggedTransformer

NORM_WEIGHT_OFFSET = 1.0  # block norms and the final norm keep a zero-centred weight; the norms inside the mixers store theirs plainly


@dataclass
class KulanexWindowSpec:
    heads: int
    kv_heads: int
    dim: int
    conv: int
    window: int
    keep_first: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[dict]


@dataclass
class KulanexMemorySpec:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass
class KulanexDeltaSpec:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass
class KulanexMoESpec:
    experts: int
    top: int
    ff: int


@dataclass
class KulanexLayerSpec:
    kind: str  # "parallel" | "channel_delta"
    left: Optional[KulanexWindowSpec] = None
    right: Optional[KulanexMemorySpec] = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    delta: Optional[KulanexDeltaSpec] = None
    mlp: Optional[KulanexMoESpec] = None


@dataclass
class KulanexSpec:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    residual_mult: float
    layers: List[KulanexLayerSpec] = field(default_factory=list)
    family: str = "kulanex"

    @property
    def num_layers(self):
        return len(self.layers)

    @classmethod
    def from_config(cls, c: dict) -> "KulanexSpec":
        layers = []
        for i, lc in enumerate(c["layers"]):
            m = lc["mixer"]
            mlp = None
            if lc.get("mlp") is not None:
                f = lc["mlp"]
                if f.get("kind") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind '{f.get('kind')}'")
                mlp = KulanexMoESpec(experts=int(f["router"]["experts"]), top=int(f["router"]["top"]), ff=int(f["expert"]["ff"]))
            if lc["type"] == "parallel":
                a, r = m["left"], m["right"]
                if int(a["vdim"]) != int(a["dim"]):
                    raise ValueError(f"layer {i}: the attention's values are its keys, so vdim ({a['vdim']}) must equal dim ({a['dim']})")
                rot = a.get("rot") or {}
                left = KulanexWindowSpec(heads=int(a["heads"]), kv_heads=int(a["kv_heads"]), dim=int(a["dim"]), conv=int(a["conv"]),
                                         window=int(a["mask"]["size"]), keep_first=int(a["mask"].get("keep_first", 0)), scale=float(a["scale"]),
                                         rot_dims=int(rot.get("dims", 0)), rot_base=float(rot.get("base", 10000.0)),
                                         rot_scaling=dict(rot["scaling"]) if rot.get("scaling") else None)
                right = KulanexMemorySpec(heads=int(r["heads"]), dim=int(r["dim"]), vdim=int(r["vdim"]), gate_cap=float(r["gate_cap"]))
                layers.append(KulanexLayerSpec("parallel", left=left, right=right, left_scale=float(m.get("left_scale", 1.0)),
                                               right_scale=float(m.get("right_scale", 1.0)), mlp=mlp))
            elif lc["type"] == "channel_delta":
                delta = KulanexDeltaSpec(heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                         conv=int(m["conv"]))
                layers.append(KulanexLayerSpec("channel_delta", delta=delta, mlp=mlp))
            else:
                raise ValueError(f"layer {i}: unknown mixer type '{lc['type']}'")
        return cls(vocab_size=int(c["vocab"]), hidden_size=int(c["width"]), norm_eps=float(c["norm"]["eps"]),
                   residual_mult=float(c.get("residual_mult", 1.0)), layers=layers)


class KulanexInferenceModel(RaggedTransformer, DSInferenceModelBase):
    describes_own_cache = True  # the engine builds its paged cache from `kv_cache_config` below

    def __init__(self, spec: KulanexSpec, tp_group=None, dtype=torch.bfloat16, device=None, engine_config=None, quantization_mode=""):
        from .container import KulanexDeltaContainer, KulanexNonTransformerContainer, KulanexParallelContainer
        assert dtype in (torch.bfloat16, torch.float32), "Kulanex runs with bf16 or fp32 activations"
        assert not quantization_mode, "Kulanex has no quantised linears"
        self._loading_layer = 0
        self._init_plumbing(spec, tp_group, dtype, device, engine_config)
        assert self.tp == 1, "Kulanex is served on one GPU per replica (its recurrent mixers are not sharded for tensor parallelism)"
        self.hq = self.hkv = 0
        self.vocab_padded = spec.vocab_size
        self._build_modules()
        self.layers = [(KulanexParallelContainer if L.kind == "parallel" else KulanexDeltaContainer)(self, i) for i, L in enumerate(spec.layers)]
        self.non_transformer = KulanexNonTransformerContainer(self)
        # cache layer of every attention layer (the delta layers have none)
        self._cache_index, n = {}, 0
        for i, L in enumerate(spec.layers):
            if L.kind == "parallel":
                self._cache_index[i] = n
                n += 1
        self._layer_hook = None  # debugging aid: called as hook(layer index, fp32 residual) after every layer

    # ---- facts the parameter classes ask for
    @property
    def n_experts(self):
        mlp = self.spec.layers[self._loading_layer].mlp
        return mlp.experts if mlp is not None else 0

    # ---- cache and state
    def kv_cache_config(self, block_size: int = 64):
        name = {torch.bfloat16: "bf16", torch.float32: "fp32"}[self.dtype]
        shapes = [(2, L.left.kv_heads, L.left.dim) for L in self.spec.layers if L.kind == "parallel"]
        if not shapes:
            shapes = [(1, 1, 1)]  # a model without attention layers caches nothing per token; the block bookkeeping stays uniform
        return KVCacheConfig(block_size=block_size, cache_shape=(len(shapes), max(s[1] for s in shapes), max(s[2] for s in shapes)),
                             cache_dtype=name, layer_shapes=shapes)

    def state_config(self):
        """What a sequence carries between steps besides its cache blocks, per layer: `l<i>.attn.conv`, `l<i>.mem.{S, n, m}`,
        `l<i>.delta.{S, conv}`."""
        specs = []
        for i, L in enumerate(self.spec.layers):
            if L.kind == "parallel":
                specs += self.attn_mods[i].state_specs(f"l{i}.attn") + self.mem_mods[i].state_specs(f"l{i}.mem")
            else:
                specs += self.delta_mods[i].state_specs(f"l{i}.delta")
        return specs

    # ---- building blocks
    def _build_modules(self):
        s, ec, dt = self.spec, self.engine_config, DtypeEnum(self.dtype)
        sm = getattr(ec, "state_manager", None)
        max_tokens = getattr(sm, "max_ragged_batch_size", 768)
        max_seqs = getattr(sm, "max_ragged_sequence_count", 512)
        D = s.hidden_size
        common = dict(max_tokens=max_tokens, input_dtype=dt, output_dtype=dt)
        self.embed_mod = heuristics.instantiate_embed(DSEmbeddingsConfig(max_tokens=max_tokens, residual_dtype=dt, embedding_dim=D, fp32_stream=True), ec)
        self.norm_mod = heuristics.instantiate_pre_norm(DSNormConfig(type=NormTypeEnum.RMSNorm, channels=D, residual_dtype=DtypeEnum.fp32,
                                                                      eps=s.norm_eps, weight_offset=NORM_WEIGHT_OFFSET, sandwich=True,
                                                                      branch_mult=s.residual_mult, **common), ec)
        self.lin_mod = heuristics.instantiate_linear(DSLinearConfig(in_channels=D, out_channels=D, **common), None)
        self.attn_mods, self.mem_mods, self.delta_mods, self.moe_mods = [], [], [], []
        for L in s.layers:
            attn = mem = delta = None
            if L.kind == "parallel":
                a, r = L.left, L.right
                attn = heuristics.instantiate_attention(DSWindowedAttentionConfig(
                    n_heads_q=a.heads, n_heads_kv=a.kv_heads, head_size=a.dim, conv_taps=a.conv, window=a.window, keep_first=a.keep_first,
                    scale=a.scale, rotate_dim=a.rot_dims, theta_base=a.rot_base,
                    rotary_scaling=RotaryScalingConfig(**a.rot_scaling) if a.rot_scaling else None, eps=s.norm_eps, out_scale=L.left_scale,
                    max_sequences=max_seqs, **common), ec)
                mem = heuristics.instantiate_recurrent(DSMatrixMemoryConfig(n_heads=r.heads, key_size=r.dim, value_size=r.vdim, gate_cap=r.gate_cap,
                                                                            eps=s.norm_eps, out_scale=L.right_scale, max_sequences=max_seqs, **common), ec)
            else:
                d = L.delta
                delta = heuristics.instantiate_recurrent(DSDeltaRuleConfig(n_heads=d.heads, n_heads_qk=d.kv_heads, key_size=d.dim, value_size=d.vdim,
                                                                           conv_taps=d.conv, eps=s.norm_eps, max_sequences=max_seqs, **common), ec)
            self.attn_mods.append(attn)
            self.mem_mods.append(mem)
            self.delta_mods.append(delta)
            f = L.mlp
            self.moe_mods.append(None if f is None else heuristics.instantiate_moe(
                DSMoEConfig(model_dim=D, intermediate_features=f.ff, n_experts=f.experts, top_k=f.top, activation=ActivationType.SiGLU,
                            normalize_scores=False, score_function="sigmoid", scale_input=True, **common), ec))
        self.unembed_mod = heuristics.instantiate_unembed(DSUnembedConfig(max_tokens=max_tokens, dtype=dt, norm_type=NormTypeEnum.RMSNorm, model_dim=D,
                                                                          max_sequences=max_seqs, vocab_size=s.vocab_size, eps=s.norm_eps,
                                                                          norm_weight_offset=NORM_WEIGHT_OFFSET, residual_fp32=True), ec)

    # ---- parameter transforms
    def transform_embedding_param(self, param):
        return self._dev(self.embed_mod.transform_param(param))

    def transform_norm_param(self, param):
        return self._dev(self.norm_mod.transform_param(param))

    def transform_dense_param(self, param):
        return self._dev(self.lin_mod.transform_param(param))

    def transform_fp32_param(self, param):
        return self._dev(param.to(torch.float32).contiguous())

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
                raise KeyError(f"unexpected parameter '{name}' for family kulanex")
        self.check_populated()

    def check_populated(self):
        super().check_populated()
        for i, (L, c) in enumerate(zip(self.spec.layers, self.layers)):
            if L.mlp is not None and any(k not in c for k in ("norm2_w", "router_w", "experts_gu", "experts_dn")):
                raise RuntimeError(f"layer {i}: feed-forward tensors are missing")

    # ---- forward
    def _parallel_mixer(self, li, L, W, h, x, batch, state_manager):
        a, r = L.left, L.right
        nq, nk = a.heads * a.dim, a.kv_heads * a.dim
        nrk, nrv = r.heads * r.dim, r.heads * r.vdim
        proj = self.lin_mod(h, W["in_w"])  # (attn q | attn k | mem q | mem k | mem v | mem gate)
        gates = dense_matmul(x, W["gates_w"])  # fp32 from the fp32 stream: (input | forget) gate pre-activations
        mixed = torch.empty(h.shape[0], nq + nrv, dtype=h.dtype, device=h.device)  # the two halves' outputs side by side, already weighted
        self.attn_mods[li](proj, (0, nq), state_manager.get_cache(self._cache_index[li]), batch, W["conv_q"], W["conv_k"], W["norm_q"], W["norm_k"],
                           state_manager, f"l{li}.attn", mixed[:, :nq])
        c0 = nq + nk
        self.mem_mods[li](proj, (c0, c0 + nrk, c0 + 2 * nrk, c0 + 2 * nrk + nrv), gates, W["bias_i"], W["bias_f"], W["memory_norm"], batch,
                          state_manager, f"l{li}.mem", mixed[:, nq:])
        return self.lin_mod(mixed, W["o_w"])

    def _delta_mixer(self, li, L, W, h, x, batch, state_manager):
        d = L.delta
        nqk, nv = d.kv_heads * d.dim, d.heads * d.vdim
        proj = self.lin_mod(h, W["in_w"])  # (q | k | v | gate latent)
        ctl = dense_matmul(x, W["control_w"])  # fp32: (beta pre-activation [heads] | decay latent)
        beta_pre = ctl[:, :d.heads].contiguous()
        a_pre = dense_matmul(ctl[:, d.heads:], W["a2_w"])
        gate = self.lin_mod(proj[:, 2 * nqk + nv:], W["g2_w"])
        out = torch.empty(h.shape[0], nv, dtype=h.dtype, device=h.device)
        self.delta_mods[li](proj, (0, nqk, 2 * nqk), beta_pre, a_pre if a_pre.is_contiguous() else a_pre.contiguous(), gate, W["conv_q"], W["conv_k"],
                            W["conv_v"], W["A_log"], W["dt_bias"], W["mix_norm"], batch, state_manager, f"l{li}.delta", out)
        return self.lin_mod(out, W["o_w"])

    def forward(self, batch, state_manager):
        """batch: finalized RaggedBatchWrapper.  Returns fp32 logits [batch.n_logit_rows, vocab]."""
        s, nt = self.spec, self.non_transformer
        x = self.embed_mod(batch, nt.embed)  # fp32 residual stream [T, width]
        _, h = self.norm_mod(x, None, None, emit_stream=True)  # the stream in the activation dtype: what the sublayers read
        last = len(s.layers) - 1
        for li, L in enumerate(s.layers):
            W = self.layers[li]
            y = (self._parallel_mixer if L.kind == "parallel" else self._delta_mixer)(li, L, W, h, x, batch, state_manager)
            more = L.mlp is not None or li < last
            _, h = self.norm_mod(x, y, None, branch_gamma=W["norm1_w"], emit_stream=more)
            if L.mlp is not None:
                y = self.moe_mods[li](h, W["router_w"], W["experts_gu"], W["experts_dn"], router_input=x)  # the router reads the fp32 stream
                _, h = self.norm_mod(x, y, None, branch_gamma=W["norm2_w"], emit_stream=li < last)
            if self._layer_hook is not None:
                self._layer_hook(li, x)
        return self.unembed_mod(x, nt.lm_head, batch, gamma=nt.final_norm_w)
