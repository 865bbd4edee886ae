"""Kulanex on the ragged engine against the plain float64 oracle of tests/kulanex_oracle.py: every mechanism alone (kernels of
csrc/ragged/recurrent_ops.cu and the router / norm extensions of csrc/ragged/latent_ops.cu), then whole models of several small random
configurations through the engine factory, the paged cache, the state slots, the scheduler and the decode-step graphs."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import kulanex_oracle as O  # noqa: E402

F64 = torch.float64
SCALING = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}


# ------------------------------------------------------------------------------------------------------------------ CPU: plumbing
def test_spec_reads_every_size_from_the_config():
    from deepspeedsyclsupport_b200.inference.v2.model_implementations.kulanex import KulanexSpec
    cfg = O.make_config([O.parallel_layer(heads=6, kv_heads=3, dim=10, conv=2, window=7, keep_first=3, rot_dims=4, base=500.0, scaling=SCALING, scale=0.3,
                                          r_heads=5, r_dim=6, r_vdim=14, gate_cap=9.0, left_scale=0.7, right_scale=1.3, mlp=O.moe(5, 2, 12)),
                         O.delta_layer(heads=6, kv_heads=2, dim=12, vdim=10, conv=5)], vocab=77, width=40, eps=3e-5, residual_mult=0.25)
    s = KulanexSpec.from_config(cfg)
    assert (s.vocab_size, s.hidden_size, s.norm_eps, s.residual_mult, s.num_layers) == (77, 40, 3e-5, 0.25, 2)
    a, r, d = s.layers[0].left, s.layers[0].right, s.layers[1].delta
    assert (a.heads, a.kv_heads, a.dim, a.conv, a.window, a.keep_first, a.rot_dims, a.rot_base, a.scale) == (6, 3, 10, 2, 7, 3, 4, 500.0, 0.3)
    assert a.rot_scaling == SCALING and (r.heads, r.dim, r.vdim, r.gate_cap) == (5, 6, 14, 9.0)
    assert (s.layers[0].left_scale, s.layers[0].right_scale) == (0.7, 1.3) and s.layers[0].mlp.top == 2 and s.layers[1].mlp is None
    assert (d.heads, d.kv_heads, d.dim, d.vdim, d.conv) == (6, 2, 12, 10, 5)
    with pytest.raises(ValueError):
        KulanexSpec.from_config(dict(cfg, layers=[dict(cfg["layers"][0], type="other")]))


def test_family_is_registered_and_chosen_by_the_config():
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import model_type_of
    from deepspeedsyclsupport_b200.inference.v2.model_implementations import KulanexPolicy, policy_for
    assert model_type_of({"architecture": "Kulanex"}) == "kulanex" and policy_for("kulanex") is KulanexPolicy


def test_rotary_frequencies_with_scaling():
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import RotaryScalingConfig
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.windowed_conv_attention import scaled_rotary_frequencies
    for dims, base, sc in ((16, 10000.0, None), (40, 5e5, {"factor": 6.0, "low": 1.0, "high": 3.0, "original": 256}), (24, 300.0, SCALING), (2, 7.0, SCALING)):
        got = scaled_rotary_frequencies(dims, base, RotaryScalingConfig(**sc) if sc else None)
        want = O.rotary_frequencies(dims, base, sc)
        assert torch.allclose(got, want, rtol=1e-14, atol=0)
    f = O.rotary_frequencies(24, 300.0, SCALING)  # the three regimes all occur in this table
    plain = O.rotary_frequencies(24, 300.0)
    ratio = (f / plain).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 1 / 8) < 1e-12 and any(1 / 8 + 1e-9 < r < 1 - 1e-9 for r in ratio)


def test_state_slots_are_handed_out_and_taken_back():
    from deepspeedsyclsupport_b200.inference.v2.ragged.state_slots import StateBufferSpec, StateSlotPool
    pool = StateSlotPool(3, [StateBufferSpec("a.S", (2, 5), torch.float32), StateBufferSpec("a.conv", (3, 7), torch.bfloat16)], device="cpu")
    assert pool.buffer("a.S").shape == (3, 2, 5) and pool.buffer("a.conv").dtype == torch.bfloat16 and pool.bytes_per_slot == 40 + 42
    s = [pool.allocate() for _ in range(3)]
    assert sorted(s) == [0, 1, 2] and pool.free_slots == 0
    with pytest.raises(RuntimeError):
        pool.allocate()
    pool.free(1)
    assert pool.allocate() == 1
    with pytest.raises(ValueError):
        pool.free(7)


def test_manager_gives_every_sequence_a_slot_and_the_batch_ships_it():
    from deepspeedsyclsupport_b200.inference.v2.ragged.manager_configs import AllocationMode, DSStateManagerConfig, KVCacheConfig, MemoryConfig
    from deepspeedsyclsupport_b200.inference.v2.ragged.ragged_manager import DSStateManager
    from deepspeedsyclsupport_b200.inference.v2.ragged.ragged_wrapper import RaggedBatchWrapper
    from deepspeedsyclsupport_b200.inference.v2.ragged.state_slots import StateBufferSpec
    cfg = DSStateManagerConfig(max_ragged_batch_size=32, max_ragged_sequence_count=3, max_tracked_sequences=3, max_context=64,
                               memory_config=MemoryConfig(mode=AllocationMode.ALLOCATE, size=4), kv_block_size=16)
    kv = KVCacheConfig(block_size=16, cache_shape=(1, 1, 4), cache_dtype="fp32", layer_shapes=[(2, 1, 4)])
    sm = DSStateManager(cfg, kv, state_specs=[StateBufferSpec("l0.S", (2, 3), torch.float32)])
    assert sm.get_state("l0.S").shape == (3, 2, 3) and sm.get_cache(0).shape == (4, 2, 16, 1, 4)
    a, b = sm.get_or_create_sequence(10), sm.get_or_create_sequence(11)
    assert {a.state_slot, b.state_slot} == {0, 1}
    sm.flush_sequence(10)
    c = sm.get_or_create_sequence(12)
    assert c.state_slot == a.state_slot and sm.state_slots.free_slots == 1  # the freed slot is used again
    batch = RaggedBatchWrapper(cfg)
    batch.set_block_table_shape(sm.max_blocks_per_seq)
    for seq, n in ((b, 5), (c, 1)):
        seq.extend_kv_cache(sm.allocate_blocks(seq.kv_blocks_needed(n)))
        seq.pre_forward(n)
        batch.insert_sequence(seq, torch.arange(n))
    batch.finalize()
    assert batch.seq_desc().tolist() == [[0, 5, 0, b.state_slot], [5, 1, 0, c.state_slot]]
    b.post_forward()
    batch.clear()
    b.pre_forward(2)
    batch.insert_sequence(b, torch.arange(2))
    batch.finalize()
    assert batch.seq_desc().tolist() == [[0, 2, 5, b.state_slot]]


def test_cache_and_state_layout_of_a_model():
    from deepspeedsyclsupport_b200.inference.v2.checkpoint import InMemoryModelEngine
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import build_model_from_checkpoint
    cfg = O.make_config([O.delta_layer(heads=4, kv_heads=2, dim=8, vdim=6, conv=3), O.parallel_layer(heads=4, kv_heads=2, dim=6, conv=4, rot_dims=4, mlp=O.moe(3, 1, 10)),
                         O.parallel_layer(heads=2, kv_heads=1, dim=12, conv=1)], width=24)
    w = O.random_weights(cfg)
    m = build_model_from_checkpoint("kulanex", cfg, InMemoryModelEngine(w), None, device=torch.device("cpu"), dtype=torch.float32)
    kc = m.kv_cache_config(block_size=32)
    assert kc.layer_shapes == [(2, 2, 6), (2, 1, 12)] and kc.cache_dtype == "fp32"  # the delta layer caches nothing per token
    assert m.layers[1]["in_w"].shape == (4 * 6 + 2 * 6 + 2 * 8 + 2 * 8 + 2 * 16 + 2 * 16, 24) and m.layers[1]["o_w"].shape == (24, 4 * 6 + 2 * 16)
    assert m.layers[1]["experts_gu"].shape == (3, 20, 24) and m.layers[0].get("experts_gu") is None and m.layers[1]["gates_w"].dtype == torch.float32
    assert m.layers[0]["in_w"].shape == (2 * 8 * 2 + 4 * 6 + 8, 24) and m.layers[0]["control_w"].shape == (4 + 8, 24)
    with pytest.raises(Exception):  # a missing tensor is reported, not ignored
        w2 = dict(w)
        w2.pop("l1.mlp.router")
        build_model_from_checkpoint("kulanex", cfg, InMemoryModelEngine(w2), None, device=torch.device("cpu"), dtype=torch.float32)


# ------------------------------------------------------------------------------------------------------------- GPU: mechanisms
gpu = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def _K():
    from deepspeedsyclsupport_b200.inference.v2 import kernels
    return kernels


class _Batch:
    """Ragged metadata of a step, built by hand: seqs = [(slot, seen, new tokens, block ids)]."""

    def __init__(self, seqs, block, max_blocks=8):
        tok_seq, tok_pos, desc, at = [], [], [], 0
        bt = torch.zeros(len(seqs), max_blocks, dtype=torch.int32)
        for i, (slot, seen, n, blocks) in enumerate(seqs):
            tok_seq += [i] * n
            tok_pos += list(range(seen, seen + n))
            desc.append([at, n, seen, slot])
            bt[i, :len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
            at += n
        self.current_sequences, self.current_tokens = len(seqs), at
        self._ts, self._tp = torch.tensor(tok_seq, dtype=torch.int32).cuda(), torch.tensor(tok_pos, dtype=torch.int32).cuda()
        self._bt, self._desc = bt.cuda(), torch.tensor(desc, dtype=torch.int32).cuda()

    def tok_seq(self):
        return self._ts

    def tok_pos(self):
        return self._tp

    def block_table(self):
        return self._bt

    def seq_desc(self):
        return self._desc


class _State:
    """Stand-in for the state manager: named per-slot buffers (filled with garbage: a sequence at position 0 must not read them)."""

    def __init__(self, specs, slots):
        self.buf = {s.name: torch.full((slots, ) + tuple(s.shape), 7.5, dtype=s.dtype, device="cuda") for s in specs}

    def get_state(self, name):
        return self.buf[name]


def _rel(got, want):
    return float((got.cpu().double() - want).norm() / want.norm())


def _cuts(total, sizes):
    out, at = [], 0
    for n in sizes:
        out.append((at, min(n, total - at)))
        at += n
        if at >= total:
            break
    if at < total:
        out.append((at, total - at))
    return out


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("dim", [6, 328])
def test_post_norm_with_multiplier_and_plain_stream(dt, dim):
    K = _K()
    x0 = torch.randn(7, dim).cuda() * 2
    y = (torch.randn(7, dim) * 4).to(dt).cuda()
    wb = (torch.randn(dim) * 0.3).cuda()
    want = x0.cpu().double() + 0.3 * O.zero_centred_norm(y.cpu().double(), wb.cpu(), 1e-5)
    x = x0.clone()
    out = K.sandwich_norm(x, y, wb, 1.0, None, 0.0, 1e-5, out_dtype=dt, y_mult=0.3, plain_out=True)
    assert torch.allclose(x.cpu().double(), want, rtol=1e-6, atol=1e-5)
    assert out.dtype == dt and torch.equal(out, x.to(dt))  # the stream itself, rounded once
    x = x0.clone()
    assert K.sandwich_norm(x, y, wb, 1.0, None, 0.0, 1e-5, out_dtype=dt, y_mult=0.3) is None and torch.allclose(x.cpu().double(), want, rtol=1e-6, atol=1e-5)
    assert torch.equal(K.sandwich_norm(x0.clone(), out_dtype=dt, plain_out=True), x0.to(dt))


@gpu
def test_embedding_without_position_vector():
    K = _K()
    table = torch.randn(30, 37).bfloat16().cuda()
    ids = torch.tensor([3, 29, 0, 7, 7], device="cuda")
    got = K.embed_sinusoid(ids, table, None, None)
    assert got.dtype == torch.float32 and torch.equal(got, table[ids].float())


@gpu
@pytest.mark.parametrize("E,top", [(8, 3), (5, 1), (16, 16), (33, 4)])
def test_sigmoid_router(E, top):
    K = _K()
    logits = (torch.randn(50, E) * 2).cuda()
    counts, scores, asg, off = K.grouped_topk_gating(logits, top, sigmoid_scores=True)
    s = torch.sigmoid(logits.cpu().double())
    ws, wi = s.topk(top, dim=-1)
    assert torch.equal(asg.cpu().long().sort(-1).values, wi.sort(-1).values)
    assert torch.allclose(scores.cpu().double().sort(-1).values, ws.sort(-1).values, rtol=1e-6, atol=1e-7)  # plain scores, not renormalised
    assert counts.cpu().tolist() == torch.bincount(wi.reshape(-1), minlength=E).tolist()


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("D,E,top,ff", [(24, 4, 2, 10), (64, 8, 1, 32), (40, 3, 3, 7)])
def test_experts_that_weigh_their_input(dt, D, E, top, ff):
    """The whole feed-forward module against the oracle: sigmoid scores, top-k, score times the expert's input, plain sum."""
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import ActivationType, DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSMoEConfig
    g = torch.Generator().manual_seed(E)
    w = {"m.router": (torch.randn(E, D, generator=g) * 0.5).bfloat16()}
    for e in range(E):
        w[f"m.e{e}.gate"], w[f"m.e{e}.up"] = (torch.randn(ff, D, generator=g) * D ** -0.5).bfloat16(), (torch.randn(ff, D, generator=g) * D ** -0.5).bfloat16()
        w[f"m.e{e}.down"] = (torch.randn(D, ff, generator=g) * ff ** -0.5).bfloat16()
    x = torch.randn(33, D, generator=g)
    h = x.to(dt)
    want = O.sigmoid_moe(h.double(), w, "m", {"router": {"experts": E, "top": top}})
    mod = heuristics.instantiate_moe(DSMoEConfig(max_tokens=64, model_dim=D, intermediate_features=ff, n_experts=E, top_k=top, activation=ActivationType.SiGLU,
                                                 score_function="sigmoid", scale_input=True, input_dtype=DtypeEnum(dt), output_dtype=DtypeEnum(dt)), None)
    assert type(mod).__name__ == "DSGroupedTopKMoE"
    gu = mod.transform_moe_mlp_1_param(torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(E)])).cuda()
    dn = mod.transform_moe_mlp_2_param(torch.stack([w[f"m.e{e}.down"] for e in range(E)])).cuda()
    got = mod(h.cuda(), mod.transform_gate_param(w["m.router"]).cuda(), gu, dn, router_input=h.float().cuda())
    assert got.dtype == torch.float32 and _rel(got, want) < (2e-5 if dt == torch.float32 else 2e-2)


def _attention_module(m, dt, eps=1e-5, out_scale=1.0):
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSWindowedAttentionConfig, RotaryScalingConfig
    sc = m["rot"].get("scaling")
    return heuristics.instantiate_attention(DSWindowedAttentionConfig(
        max_tokens=512, n_heads_q=m["heads"], n_heads_kv=m["kv_heads"], head_size=m["dim"], conv_taps=m["conv"], window=m["mask"]["size"],
        keep_first=m["mask"]["keep_first"], scale=m["scale"], rotate_dim=m["rot"]["dims"], theta_base=m["rot"]["base"],
        rotary_scaling=RotaryScalingConfig(**sc) if sc else None, eps=eps, out_scale=out_scale, max_sequences=8, input_dtype=DtypeEnum(dt),
        output_dtype=DtypeEnum(dt)), None)


def _attention_weights(m, D, seed):
    g = torch.Generator().manual_seed(seed)
    nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
    return {"a.q": (torch.randn(nq, D, generator=g) * D ** -0.5).bfloat16(), "a.k": (torch.randn(nk, D, generator=g) * D ** -0.5).bfloat16(),
            "a.q.conv": (torch.randn(nq, m["conv"], generator=g) * 0.6 + 0.2).bfloat16(), "a.k.conv": (torch.randn(nk, m["conv"], generator=g) * 0.6 + 0.2).bfloat16(),
            "a.q.norm": (torch.randn(nq, generator=g) * 0.3 + 1.1).bfloat16(), "a.k.norm": (torch.randn(nk, generator=g) * 0.3 + 1.1).bfloat16(),
            "a.o": torch.eye(nq).bfloat16()}


def _run_attention(mod, m, w, h, cuts, dt, block, blocks, slot=1, total_blocks=16):
    """Feed h [T, D] of ONE sequence through the module in the given portions; returns [T, heads * dim]."""
    nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
    cache = torch.zeros(total_blocks, 2, block, m["kv_heads"], m["dim"], dtype=dt, device="cuda")
    state = _State(mod.state_specs("a"), 3)
    W = torch.cat([w["a.q"], w["a.k"]]).double()
    f32 = lambda t: t.float().cuda()  # noqa: E731
    outs = []
    for at, n in cuts:
        proj = (h[at:at + n].double() @ W.T).to(dt).cuda()
        out = torch.empty(n, nq, dtype=dt, device="cuda")
        mod(proj, (0, nq), cache, _Batch([(slot, at, n, blocks)], block, max_blocks=len(blocks)), f32(w["a.q.conv"]), f32(w["a.k.conv"]), f32(w["a.q.norm"]),
            f32(w["a.k.norm"]), state, "a", out)
        outs.append(out)
    return torch.cat(outs)


ATTN = {
    # kv heads shared by 3 query heads, partial rotation with all three scaling regimes, window inside a page, kept tokens
    "grouped": O.parallel_layer(heads=6, kv_heads=2, dim=10, conv=4, window=11, keep_first=3, rot_dims=6, base=300.0, scaling=SCALING, scale=0.4)["mixer"]["left"],
    # one head, every entry rotated, no kept tokens, no convolution memory (one tap), window longer than the sequence
    "plain": O.parallel_layer(heads=1, kv_heads=1, dim=8, conv=1, window=500, keep_first=0, rot_dims=8, scale=0.35)["mixer"]["left"],
    # no rotation at all, more kept tokens than the window is long, two taps
    "sinks": O.parallel_layer(heads=4, kv_heads=4, dim=16, conv=2, window=5, keep_first=9, rot_dims=0, scale=0.25)["mixer"]["left"],
    # an odd head size: the last entry of every head has no partner and is never rotated
    "odd_head": O.parallel_layer(heads=3, kv_heads=1, dim=7, conv=3, window=9, keep_first=1, rot_dims=6, scale=0.4)["mixer"]["left"],
    # head sizes the tensor-core kernels take in bf16: grouped heads, a window that ends inside a 128-key page, kept keys
    "tc64": O.parallel_layer(heads=4, kv_heads=2, dim=64, conv=3, window=21, keep_first=2, rot_dims=32, scale=0.125)["mixer"]["left"],
    "tc128": O.parallel_layer(heads=8, kv_heads=1, dim=128, conv=4, window=50, keep_first=5, rot_dims=64, base=1e5, scale=0.09)["mixer"]["left"],
}


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name", list(ATTN))
@pytest.mark.parametrize("sizes", [[200], [1] * 70, [2, 3, 31, 1, 1, 16, 2, 40]])
def test_windowed_attention_mixer(name, sizes, dt):
    """Convolution with its carried rows, whole-projection norms, rotation, cache append and masked attention, whole and in portions
    (cut inside pages, inside the window and inside the convolution's reach), pages in shuffled order."""
    m, D, T = ATTN[name], 20, 70
    w = _attention_weights(m, D, len(name))
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(3)).bfloat16().float()
    want = O.windowed_attention(h.double(), w, "a", m, 1e-5)
    got = _run_attention(_attention_module(m, dt), m, w, h, _cuts(T, sizes), dt, block=16, blocks=[9, 2, 11, 5, 0])
    assert _rel(got, want) < (3e-5 if dt == torch.float32 else 3e-2)


@gpu
def test_output_constant_of_the_attention():
    m = ATTN["grouped"]
    w = _attention_weights(m, 20, 1)
    h = torch.randn(20, 20, generator=torch.Generator().manual_seed(4)).bfloat16().float()
    a = _run_attention(_attention_module(m, torch.float32), m, w, h, [(0, 20)], torch.float32, 16, [1, 2])
    b = _run_attention(_attention_module(m, torch.float32, out_scale=1.7), m, w, h, [(0, 20)], torch.float32, 16, [1, 2])
    assert torch.allclose(b, a * 1.7, rtol=1e-6, atol=1e-7)


@gpu
@pytest.mark.parametrize("d,dt", [(8, torch.float32), (8, torch.bfloat16), (64, torch.bfloat16), (128, torch.bfloat16)])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("window,keep", [(40, 4), (64, 1), (17, 0), (300, 2), (130, 3)])
def test_window_and_kept_edges_decide_what_is_seen(window, keep, decode, d, dt):
    """One key is made to dominate its row's softmax (its direction is planted in key and query, its value is a marker): the output shows
    the marker exactly when the key is visible -- the last key inside the window, the first outside, the last kept token, the first not
    kept, keys at both sides of block and 128-key page borders and a far one; in a prompt portion and for a single decoded token; on the
    CUDA-core kernel (head size 8) and on the tensor-core kernels (64, 128: the decode kernel too)."""
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.windowed_conv_attention import windowed_attention
    K = _K()
    H, G, block, T = 2, 1, 16, 300
    blocks = [3, 7, 1, 12, 5, 9, 0, 4, 8, 2, 19, 14, 11, 17, 6, 10, 13, 15, 16]
    g = torch.Generator().manual_seed(window)
    kk = torch.randn(T, d, generator=g) * 0.1
    vv = torch.randn(T, d, generator=g) * 0.1
    query_pos = T - 1
    targets = {query_pos - window + 1, query_pos - window, keep - 1, keep, 15, 16, 127, 128, 255, 256, 60, query_pos}
    for target in sorted(t for t in targets if 0 <= t < T):
        k2, v2 = kk.clone(), vv.clone()
        k2[target] = torch.tensor([6.0] + [0.0] * (d - 1))
        v2[target] = 50.0
        cache = torch.zeros(20, 2, block, G, d, dtype=dt, device="cuda")
        pages = torch.tensor(blocks)[torch.arange(T) // block]
        cache[pages, 0, torch.arange(T) % block, 0] = k2.to(dt).cuda()
        cache[pages, 1, torch.arange(T) % block, 0] = v2.to(dt).cuda()
        n_new = 1 if decode else 23
        q = torch.zeros(n_new, H * d)
        q[:, 0] = q[:, d] = 6.0
        out = torch.empty(n_new, H * d, dtype=dt, device="cuda")
        b = _Batch([(0, T - n_new, n_new, blocks)], block, len(blocks))
        qd = q.to(dt).cuda()
        if d == 8:
            K.window_attention(qd, cache, b.tok_seq(), b.tok_pos(), b.block_table(), out, H, G, d, window, keep, 1.0)
        else:
            assert K.paged_flash_window_ok(qd, cache, out, H, G, d)
            windowed_attention(qd, cache, b.tok_seq(), b.tok_pos(), b.block_table(), out, H, G, d, window, keep, 1.0, decode=decode)
        visible = target <= query_pos and (query_pos - target < window or target < keep)
        row = out[-1].float().cpu()
        assert bool((row > 40).all()) == visible and bool((row.abs() < 1).all()) == (not visible), (target, visible, row)
        ks, vs = k2.to(dt).double(), v2.to(dt).double()
        s = (ks[:T] @ q[-1, :d].to(dt).double()).masked_fill(~O.window_visible(T, window, keep)[query_pos], float("-inf"))
        assert torch.allclose(row[:d].double(), torch.softmax(s, -1) @ vs, rtol=2e-2 if dt == torch.bfloat16 else 1e-4, atol=2e-2 if dt == torch.bfloat16 else 1e-5)


@gpu
@pytest.mark.parametrize("d,G", [(64, 2), (128, 1)])
def test_tensor_core_and_cuda_core_attention_agree_on_a_mixed_batch(d, G):
    """Portions of unequal sequences beside single tokens, strided output with a constant: both kernels give the same rows."""
    from deepspeedsyclsupport_b200.inference.v2.modules.implementations.attention.windowed_conv_attention import windowed_attention
    K = _K()
    H, block, window, keep = 4, 32, 70, 3
    seqs = [(0, 150, 40, [5, 1, 9, 3, 7, 11]), (1, 0, 9, [0]), (2, 99, 1, [2, 4, 6, 8]), (3, 255, 1, [10, 12, 13, 14, 15, 16, 17, 18])]
    b = _Batch(seqs, block, 8)
    g = torch.Generator().manual_seed(d)
    cache = (torch.randn(20, 2, block, G, d, generator=g) * 0.5).bfloat16().cuda()
    q = torch.randn(b.current_tokens, H * d, generator=g).bfloat16().cuda()
    wide = torch.zeros(b.current_tokens, H * d + 24, dtype=torch.bfloat16, device="cuda")
    ref = torch.empty(b.current_tokens, H * d, dtype=torch.bfloat16, device="cuda")
    K.window_attention(q, cache, b.tok_seq(), b.tok_pos(), b.block_table(), ref, H, G, d, window, keep, d ** -0.5, out_scale=1.3)
    for decode in (False, True):
        wide.zero_()
        windowed_attention(q, cache, b.tok_seq(), b.tok_pos(), b.block_table(), wide[:, :H * d], H, G, d, window, keep, d ** -0.5, out_scale=1.3, decode=decode)
        assert _rel(wide[:, :H * d], ref.cpu().double()) < 1.5e-2 and float(wide[:, H * d:].abs().max()) == 0


def _memory_module(m, dt, out_scale=1.0):
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSMatrixMemoryConfig
    return heuristics.instantiate_recurrent(DSMatrixMemoryConfig(max_tokens=512, n_heads=m["heads"], key_size=m["dim"], value_size=m["vdim"], gate_cap=m["gate_cap"],
                                                                 eps=1e-5, out_scale=out_scale, max_sequences=8, input_dtype=DtypeEnum(dt), output_dtype=DtypeEnum(dt)), None)


def _memory_weights(m, D, seed, forget_bias=3.0):
    g = torch.Generator().manual_seed(seed)
    hd, hv, H = m["heads"] * m["dim"], m["heads"] * m["vdim"], m["heads"]
    r = lambda *s, std=1.0, mean=0.0: (torch.randn(*s, generator=g) * std + mean).bfloat16()  # noqa: E731
    return {"r.q": r(hd, D, std=D ** -0.5), "r.k": r(hd, D, std=D ** -0.5), "r.v": r(hv, D, std=D ** -0.5), "r.g": r(hv, D, std=D ** -0.5),
            "r.i": r(H, D, std=2 * D ** -0.5), "r.i.b": r(H, std=0.5), "r.f": r(H, D, std=2 * D ** -0.5), "r.f.b": r(H, std=1.5, mean=forget_bias),
            "r.norm": r(hv, std=0.2, mean=1.0), "r.o": torch.eye(hv).bfloat16()}


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,cap", [(3, 8, 16, 15.0), (1, 5, 3, 2.0), (2, 32, 48, 11.0), (2, 72, 40, 30.0), (1, 130, 300, 8.0)])
@pytest.mark.parametrize("sizes", [[90], [1] * 60, [2, 5, 1, 33, 2, 9]])
def test_matrix_memory_mixer(heads, dim, vdim, cap, sizes, dt):
    """Whole, token by token and in portions, with the state carried in a slot that held something else before; sizes that are not powers
    of two, one head, more rows than a thread group holds at once, several column tiles, a tight and a loose gate cap."""
    m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    D, T = 24, 60
    w = _memory_weights(m, D, heads * dim, forget_bias=1.0 if cap < 5 else 3.0)
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(5)).bfloat16().float()
    want = O.matrix_memory(h.double(), w, "r", m, 1e-5)
    mod = _memory_module(m, dt)
    state = _State(mod.state_specs("r"), 3)
    Win = torch.cat([w["r.q"], w["r.k"], w["r.v"], w["r.g"]]).double()
    Wg = torch.cat([w["r.i"], w["r.f"]]).double()
    hd, hv = heads * dim, heads * vdim
    outs = []
    for at, n in _cuts(T, sizes):
        proj = (h[at:at + n].double() @ Win.T).to(dt).cuda()
        gates = (h[at:at + n].double() @ Wg.T).float().cuda()
        out = torch.empty(n, hv, dtype=dt, device="cuda")
        mod(proj, (0, hd, 2 * hd, 2 * hd + hv), gates, w["r.i.b"].float().cuda(), w["r.f.b"].float().cuda(), w["r.norm"].float().cuda(),
            _Batch([(2, at, n, [])], 16), state, "r", out)
        outs.append(out)
    assert _rel(torch.cat(outs), want) < (5e-5 if dt == torch.float32 else 3e-2)


def _delta_module(m, dt):
    from deepspeedsyclsupport_b200.inference.v2.inference_utils import DtypeEnum
    from deepspeedsyclsupport_b200.inference.v2.modules import heuristics
    from deepspeedsyclsupport_b200.inference.v2.modules.configs import DSDeltaRuleConfig
    return heuristics.instantiate_recurrent(DSDeltaRuleConfig(max_tokens=512, n_heads=m["heads"], n_heads_qk=m["kv_heads"], key_size=m["dim"], value_size=m["vdim"],
                                                              conv_taps=m["conv"], eps=1e-5, max_sequences=8, input_dtype=DtypeEnum(dt), output_dtype=DtypeEnum(dt)), None)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("heads,kv,dim,vdim,conv", [(4, 2, 8, 16, 3), (1, 1, 5, 3, 1), (2, 2, 32, 48, 4), (6, 2, 72, 24, 2), (1, 1, 130, 300, 5)])
@pytest.mark.parametrize("sizes", [[90], [1] * 60, [2, 5, 1, 33, 2, 9]])
def test_channel_delta_mixer(heads, kv, dim, vdim, conv, sizes, dt):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "_low_rank": 6}
    D, T = 24, 60
    cfg = O.make_config([O.delta_layer(heads, kv, dim, vdim, conv)], width=D)
    cfg["layers"][0]["mixer"]["_low_rank"] = 6
    w = O.random_weights(cfg, seed=heads + dim)
    w["l0.mix.o"] = torch.eye(heads * vdim).bfloat16()
    h = torch.randn(T, D, generator=torch.Generator().manual_seed(6)).bfloat16().float()
    want = O.channel_delta(h.double(), w, "l0.mix", m, 1e-5)
    mod = _delta_module(m, dt)
    state = _State(mod.state_specs("d"), 3)
    P = lambda n: w["l0.mix." + n]  # noqa: E731
    Win = torch.cat([P("q"), P("k"), P("v")]).double()
    nqk, nv = kv * dim, heads * vdim
    f32 = lambda t: t.float().cuda()  # noqa: E731
    outs = []
    for at, n in _cuts(T, sizes):
        hh = h[at:at + n].double()
        proj = (hh @ Win.T).to(dt).cuda()
        beta_pre = (hh @ P("b").double().T).float().cuda()
        a_pre = ((hh @ P("a1").double().T) @ P("a2").double().T).float().cuda()
        gate = ((hh @ P("g1").double().T) @ P("g2").double().T).to(dt).cuda()
        out = torch.empty(n, nv, dtype=dt, device="cuda")
        mod(proj, (0, nqk, 2 * nqk), beta_pre, a_pre, gate, f32(P("q.conv")), f32(P("k.conv")), f32(P("v.conv")), f32(P("A_log")), f32(P("dt_bias")),
            f32(P("norm")), _Batch([(1, at, n, [])], 16), state, "d", out)
        outs.append(out)
    assert _rel(torch.cat(outs), want) < (5e-5 if dt == torch.float32 else 3e-2)


@gpu
def test_sequences_of_a_batch_keep_their_own_state():
    """Three sequences advance side by side with unequal portions; each equals the sequence run alone, and a new sequence that takes over a
    used slot starts from nothing."""
    m = {"heads": 2, "dim": 8, "vdim": 16, "gate_cap": 15.0}
    D = 24
    w = _memory_weights(m, D, 3)
    mod = _memory_module(m, torch.float32)
    state = _State(mod.state_specs("r"), 4)
    Win, Wg = torch.cat([w["r.q"], w["r.k"], w["r.v"], w["r.g"]]).double(), torch.cat([w["r.i"], w["r.f"]]).double()
    hs = {u: torch.randn(n, D, generator=torch.Generator().manual_seed(u)).bfloat16().double() for u, n in ((0, 30), (1, 7), (2, 19), (3, 12))}
    want = {u: O.matrix_memory(h, w, "r", m, 1e-5) for u, h in hs.items()}
    slot = {0: 3, 1: 0, 2: 2, 3: 0}  # sequence 3 reuses the slot of sequence 1
    steps = [[(0, 10), (1, 6), (2, 1)], [(0, 1), (1, 1), (2, 17)], [(0, 19), (2, 1), (3, 5)], [(3, 7)]]
    at, got = {u: 0 for u in hs}, {u: [] for u in hs}
    for step in steps:
        hcat = torch.cat([hs[u][at[u]:at[u] + n] for u, n in step])
        proj, gates = (hcat @ Win.T).float().cuda(), (hcat @ Wg.T).float().cuda()
        out = torch.empty(hcat.shape[0], 32, dtype=torch.float32, device="cuda")
        mod(proj, (0, 16, 32, 64), gates, w["r.i.b"].float().cuda(), w["r.f.b"].float().cuda(), w["r.norm"].float().cuda(),
            _Batch([(slot[u], at[u], n, []) for u, n in step], 16), state, "r", out)
        r = 0
        for u, n in step:
            got[u].append(out[r:r + n])
            r += n
            at[u] += n
    for u in hs:
        assert at[u] == hs[u].shape[0] and _rel(torch.cat(got[u]), want[u]) < 5e-5, u


# ------------------------------------------------------------------------------------------------------------ GPU: whole models
CONFIGS = {
    # odd sizes that differ per layer; grouped kv heads; kept tokens and none; one / two / four taps; rotation of all, some and no entries;
    # a layer without feed-forward; top 1 and top 3
    "odd": O.make_config([
        O.parallel_layer(heads=6, kv_heads=2, dim=10, conv=4, window=19, keep_first=3, rot_dims=6, base=300.0, scaling=SCALING, scale=0.4, r_heads=3, r_dim=6, r_vdim=14,
                         gate_cap=10.0, left_scale=1.3, right_scale=0.8, mlp=O.moe(5, 3, 18)),
        O.delta_layer(heads=4, kv_heads=2, dim=6, vdim=10, conv=3, mlp=O.moe(3, 1, 9)),
        O.delta_layer(heads=3, kv_heads=3, dim=12, vdim=5, conv=1),
        O.parallel_layer(heads=2, kv_heads=2, dim=8, conv=1, window=7, keep_first=0, rot_dims=8, scale=0.3, r_heads=1, r_dim=9, r_vdim=7, gate_cap=4.0, left_scale=0.5,
                         right_scale=2.0),
        O.parallel_layer(heads=3, kv_heads=1, dim=14, conv=2, window=40, keep_first=20, rot_dims=0, scale=0.2, r_heads=2, r_dim=4, r_vdim=4, mlp=O.moe(4, 4, 6)),
    ], vocab=61, width=44, eps=1e-5, residual_mult=0.35),
    # aligned sizes (tensor-core GEMMs in bf16), head size 64, window across pages
    "aligned": O.make_config([
        O.delta_layer(heads=4, kv_heads=4, dim=32, vdim=32, conv=4, mlp=O.moe(8, 2, 32)),
        O.parallel_layer(heads=4, kv_heads=2, dim=64, conv=4, window=33, keep_first=2, rot_dims=32, base=1e5, scaling={"factor": 5.0, "low": 1.0, "high": 3.0, "original": 128},
                         scale=0.11, r_heads=2, r_dim=32, r_vdim=48, mlp=O.moe(8, 2, 32)),
        O.parallel_layer(heads=2, kv_heads=1, dim=128, conv=2, window=140, keep_first=3, rot_dims=128, scale=0.09, r_heads=1, r_dim=16, r_vdim=32),
    ], vocab=96, width=128, eps=1e-6, residual_mult=1.0),
    # no attention layer at all: nothing is cached per token, everything lives in the state slots
    "recurrent": O.make_config([O.delta_layer(heads=2, kv_heads=1, dim=8, vdim=8, conv=2), O.delta_layer(heads=2, kv_heads=2, dim=4, vdim=12, conv=3, mlp=O.moe(2, 1, 8))],
                               vocab=40, width=24, residual_mult=0.7),
}
_MODELS = {}


def _model(name, tmp_path_factory, dt=torch.float32):
    """fp32 runs keep the configured top-k (every selection is compared tightly).  bf16 runs let every token use ALL experts of a layer,
    weighted by their scores: a top-k choice between two close scores flips under rounding and the flipped token then colours the rest of
    its sequence through the recurrent state, which says nothing about the engine (the bf16 selection itself is checked on equal inputs in
    test_experts_that_weigh_their_input)."""
    import copy
    every = dt == torch.bfloat16
    if (name, every) not in _MODELS:
        cfg = copy.deepcopy(CONFIGS[name])
        if every:
            for L in cfg["layers"]:
                if L["mlp"] is not None:
                    L["mlp"]["router"]["top"] = L["mlp"]["router"]["experts"]
        w = O.random_weights(cfg, seed=len(name))
        _MODELS[(name, every)] = (cfg, w, O.write_model(str(tmp_path_factory.mktemp(name)), cfg, w))
    return _MODELS[(name, every)]


def _engine(path, dt, pool_tokens=256, block=16, max_seqs=4):
    from deepspeedsyclsupport_b200.inference.v2.config_v2 import RaggedInferenceEngineConfig
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import build_hf_engine
    from deepspeedsyclsupport_b200.inference.v2.ragged.manager_configs import AllocationMode, DSStateManagerConfig, MemoryConfig
    mgr = DSStateManagerConfig(max_tracked_sequences=max_seqs, max_ragged_sequence_count=max_seqs, max_ragged_batch_size=pool_tokens, max_context=pool_tokens,
                               memory_config=MemoryConfig(mode=AllocationMode.ALLOCATE, size=pool_tokens // block), kv_block_size=block)
    return build_hf_engine(path, RaggedInferenceEngineConfig(state_manager=mgr), dtype=dt)


def _close(got, want, dt):
    """Every logit row agrees up to a per-row shift, relative to the spread of the logits.  fp32: tightly.  bf16: within a few times what
    rounding of the matrix products does to these small random models, far below what a wrong key, a lost state or a wrong expert causes
    (order 1)."""
    d = got.cpu().double() - want
    d = d - d.mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std()
    if dt == torch.float32:
        return float(err.max()) < 5e-5, float(err.max())
    return float(err.max()) < 0.2 and float(err.median()) < 0.05, (float(err.median()), float(err.max()))


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n, ), generator=torch.Generator().manual_seed(seed))


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_every_layer(name, dt, tmp_path_factory):
    cfg, w, path = _model(name, tmp_path_factory, dt)
    eng = _engine(path, dt)
    toks = _tokens(cfg, 75, 1)
    want, res = O.forward(cfg, w, toks.tolist(), collect_layers=True)
    got_res = []
    eng.model()._layer_hook = lambda li, x: got_res.append(x.clone())
    got = eng.put([7], [toks], logit_positions=[list(range(75))])
    assert got.shape == (75, cfg["vocab"]) and len(got_res) == len(res)
    for r, (a, b) in enumerate(zip(got_res, res)):
        if dt == torch.float32:
            assert torch.allclose(a.cpu().double(), b, rtol=1e-4, atol=1e-4), f"layer {r}"
        else:
            row = (a.cpu().double() - b).norm(dim=-1) / b.norm(dim=-1)
            assert float(row.max()) < 0.2 and float(row.median()) < 0.04, f"layer {r}"
    ok, err = _close(got, want, dt)
    assert ok, err
    assert got[0].isfinite().all()


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name,cuts", [("odd", [1] * 60), ("odd", [2, 2, 15, 1, 17, 3, 2, 18]), ("aligned", [16, 16, 1, 1, 6, 2, 30]), ("aligned", [31, 2, 7, 32]),
                                       ("recurrent", [3, 33, 2, 2, 1, 1, 9])])
def test_portions_and_token_by_token_equal_the_whole_prompt(name, cuts, dt, tmp_path_factory):
    """Prefill against decoding token by token, and portions cut inside pages (block 16), windows and convolutions, down to two tokens."""
    cfg, w, path = _model(name, tmp_path_factory, dt)
    eng = _engine(path, dt)
    toks = _tokens(cfg, sum(cuts), 2)
    want = O.forward(cfg, w, toks.tolist())
    rows, at = [], 0
    for n in cuts:
        rows.append(eng.put([3], [toks[at:at + n]], logit_positions=[list(range(n))]))
        at += n
    ok, err = _close(torch.cat(rows), want, dt)
    assert ok, err


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name", ["odd", "aligned"])
def test_unequal_requests_in_one_batch_and_reused_pages_and_slots(name, dt, tmp_path_factory):
    """Four requests of unequal length share steps (portions beside single tokens), one pauses for a step, they finish at different
    times, and two more take over their state slots and pages: every logit row equals the request run alone."""
    cfg, w, path = _model(name, tmp_path_factory, dt)
    eng = _engine(path, dt, pool_tokens=160, block=16)
    prompts = {u: _tokens(cfg, n, 10 + u) for u, n in ((0, 50), (1, 17), (2, 33), (3, 1), (4, 48), (5, 31))}
    want = {u: O.forward(cfg, w, p.tolist()) for u, p in prompts.items()}
    schedule = [[(0, 20), (1, 16), (3, 1)], [(0, 1), (2, 30)], [(0, 1), (1, 1), (2, 1)], [(0, 28), (2, 1)], [(2, 1), (4, 15)], [(4, 33), (5, 2)], [(5, 29)]]
    at, got = {u: 0 for u in prompts}, {u: [] for u in prompts}
    free0 = eng.free_blocks
    for step in schedule:
        uids = [u for u, _ in step]
        out = eng.put(uids, [prompts[u][at[u]:at[u] + n] for u, n in step], logit_positions=[list(range(n)) for _, n in step])
        r = 0
        for u, n in step:
            got[u].append(out[r:r + n])
            r += n
            at[u] += n
            if at[u] == len(prompts[u]):
                eng.flush(u)
    assert eng.free_blocks == free0 and all(at[u] == len(p) for u, p in prompts.items())
    assert eng._state_manager.state_slots.free_slots == 4
    for u in prompts:
        ok, err = _close(torch.cat(got[u]), want[u], dt)
        assert ok, (u, err)


@gpu
@pytest.mark.parametrize("name", ["aligned", "odd"])
def test_long_decoding_through_the_step_graphs(name, tmp_path_factory):
    """A prompt, then 150 single-token steps (the steady-state ones replay a captured graph) that carry the window over decoded tokens and
    past the kept ones; some steps ask for no logits."""
    cfg, w, path = _model(name, tmp_path_factory)
    eng = _engine(path, torch.float32, pool_tokens=256, block=16)
    toks = _tokens(cfg, 200, 5)
    want = O.forward(cfg, w, toks.tolist())
    got = [eng.put([1], [toks[:50]], logit_positions=[[49]])]
    keep = [49]
    for i in range(50, 200):
        wanted = i % 7 != 0
        out = eng.put([1], [toks[i:i + 1]], logit_positions=[[0] if wanted else []])
        assert out.shape[0] == int(wanted)
        if wanted:
            got.append(out)
            keep.append(i)
    ok, err = _close(torch.cat(got), want[keep], torch.float32)
    assert ok, err
    graphs = eng.model()._graphs
    assert 1 in graphs and (1, 0) in graphs, list(graphs)


@gpu
def test_greedy_generation_through_the_scheduler(tmp_path_factory):
    from deepspeedsyclsupport_b200.inference.v2.scheduler import SplitFuseScheduler
    cfg, w, path = _model("odd", tmp_path_factory)
    eng = _engine(path, torch.float32, pool_tokens=192, block=16)
    sched = SplitFuseScheduler(eng, token_budget=24)  # prompts are split into portions and fused with running decodes
    prompts = {0: _tokens(cfg, 37, 20), 1: _tokens(cfg, 5, 21), 2: _tokens(cfg, 21, 22)}
    for u, p in prompts.items():
        sched.add_request(u, p, max_new_tokens=6)
    done = sched.run_to_completion()
    for u, p in prompts.items():
        assert done[u] == O.greedy(cfg, w, p.tolist(), 6), u


@gpu
def test_trace_runner_replays_steps(tmp_path_factory):
    """bin/trace_run as a process: portions of three requests beside single tokens, a request that pauses for a step, wanted positions
    anywhere in a portion, requests ending at different steps with their pages and slots reused by a later one (pool of 3 pages)."""
    import json
    import subprocess
    cfg, w, path = _model("odd", tmp_path_factory)
    out_dir = str(tmp_path_factory.mktemp("trace_out"))
    reqs = {"a": _tokens(cfg, 70, 31).tolist(), "b": _tokens(cfg, 9, 32).tolist(), "c": _tokens(cfg, 64, 33).tolist(), "d": _tokens(cfg, 100, 34).tolist()}
    want = {k: O.forward(cfg, w, v) for k, v in reqs.items()}
    plan = [[("a", 30, [0, 29]), ("b", 8, [3])], [("a", 2, [1]), ("c", 64, [63])], [("a", 37, [36]), ("b", 1, [0])], [("a", 1, [0]), ("d", 64, [])],
            [("d", 2, [0, 1])], [("d", 1, [])], [("d", 33, [32])]]
    at = {k: 0 for k in reqs}
    lines, expect = [], []
    for n, step in enumerate(plan):
        entries, end, rows = [], [], []
        for k, cnt, wanted in step:
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + cnt], "want": wanted})
            rows += [want[k][at[k] + p] for p in wanted]
            at[k] += cnt
            if at[k] == len(reqs[k]):
                end.append(k)
        lines.append(json.dumps({"step": n, "entries": entries, "end": end}))
        expect.append(torch.stack(rows) if rows else None)
    assert all(at[k] == len(v) for k, v in reqs.items())
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", out_dir, "--max-tokens", "192"],
                       input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == [f"done {n}" for n in range(len(plan))]
    for n, e in enumerate(expect):
        f = os.path.join(out_dir, f"{n}.f32")
        if e is None:
            assert not os.path.exists(f)
            continue
        got = torch.frombuffer(bytearray(open(f, "rb").read()), dtype=torch.float32).view(len(e), cfg["vocab"])
        ok, err = _close(got, e, torch.float32)
        assert ok, (n, err)
