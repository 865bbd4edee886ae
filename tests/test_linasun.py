"""Linasun on the ragged engine against the plain float64 oracle of tests/linasun_oracle.py: every mechanism alone (kernels of
csrc/ragged/latent_ops.cu), then whole models of several small random configurations through the engine factory, the paged cache,
the scheduler and the decode-step graphs."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import linasun_oracle as O  # noqa: E402

F64 = torch.float64


# ------------------------------------------------------------------------------------------------------------------ CPU: plumbing
def test_spec_reads_every_size_from_the_config():
    from deepspeedsyclsupport_b200.inference.v2.model_implementations.linasun import LinasunSpec
    cfg = O.make_config(48, 70, [O.layer_cfg(3, 8, 6, 12, 10, 0.3, (6, 2, 3, 2, 12, 1.5)), O.layer_cfg(5, 16, 4, 20, 7, 0.11), O.layer_cfg(2, 4, 4, 8, 8, 0.5, (4, 1, 1, 1, 6, 3.0))],
                        loop={"start": 1, "stop": 3, "times": 3}, eps=3e-5, softcap=11.0)
    s = LinasunSpec.from_config(cfg)
    assert (s.vocab_size, s.hidden_size, s.norm_eps, s.logit_softcap) == (70, 48, 3e-5, 11.0)
    assert s.run_order() == [0, 1, 2, 1, 2, 1, 2] == O.run_order(cfg)
    assert s.layers[1].mlp is None and s.layers[1].mixer.kv_rank == 20 and s.layers[0].mlp.groups == 3 and s.layers[2].mlp.limit == 3.0
    assert LinasunSpec.from_config(O.make_config(8, 9, [O.layer_cfg(1, 2, 2, 2, 2, 1.0)] * 2, loop={"start": 1, "stop": 1, "times": 5})).run_order() == [0, 1]
    with pytest.raises(ValueError):
        LinasunSpec.from_config(dict(cfg, layers=[dict(cfg["layers"][0], type="other")]))


def test_family_is_registered_and_chosen_by_the_config():
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import model_type_of
    from deepspeedsyclsupport_b200.inference.v2.model_implementations import LinasunPolicy, policy_for
    assert model_type_of({"architecture": "Linasun"}) == "linasun" and policy_for("linasun") is LinasunPolicy
    assert model_type_of({"model_type": "llama", "architecture": "x"}) == "llama"


def test_cache_has_one_latent_plane_per_layer_run():
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import build_model_from_checkpoint
    from deepspeedsyclsupport_b200.inference.v2.checkpoint import InMemoryModelEngine
    cfg = O.make_config(16, 20, [O.layer_cfg(2, 4, 4, 6, 5, 0.5), O.layer_cfg(1, 4, 2, 10, 3, 0.5, (4, 2, 2, 1, 6, 2.0))], loop={"start": 0, "stop": 2, "times": 2})
    m = build_model_from_checkpoint("linasun", cfg, InMemoryModelEngine(O.random_weights(cfg)), None, device=torch.device("cpu"), dtype=torch.float32)
    kc = m.kv_cache_config(block_size=32)
    assert kc.layer_shapes == [(1, 1, 6), (1, 1, 10), (1, 1, 6), (1, 1, 10)] and kc.block_size == 32 and kc.cache_dtype == "fp32"
    assert m.layers[1]["experts_gu"].shape == (4, 12, 16) and m.layers[0].get("experts_gu") is None and m.layers[0]["in_w"].shape == (5 + 6 + 8, 16)
    with pytest.raises(Exception):  # a missing tensor is reported, not ignored
        w = O.random_weights(cfg)
        w.pop("l1.mlp.correction")
        build_model_from_checkpoint("linasun", cfg, InMemoryModelEngine(w), None, device=torch.device("cpu"), dtype=torch.float32)


def test_logit_positions_of_a_batch():
    from deepspeedsyclsupport_b200.inference.v2.ragged.manager_configs import DSStateManagerConfig
    from deepspeedsyclsupport_b200.inference.v2.ragged.ragged_wrapper import RaggedBatchWrapper
    from deepspeedsyclsupport_b200.inference.v2.ragged.sequence_descriptor import DSSequenceDescriptor
    b = RaggedBatchWrapper(DSStateManagerConfig(max_ragged_batch_size=32, max_ragged_sequence_count=4, max_tracked_sequences=4, max_context=64))
    b.set_block_table_shape(4)
    for uid, n in ((0, 5), (1, 1), (2, 3)):
        d = DSSequenceDescriptor(uid, 4, 16)
        d.extend_kv_cache([uid])
        b.insert_sequence(d, torch.arange(n))
    assert b.n_logit_rows == 3
    b.set_logit_positions([[0, 4], [], [2]])
    b.finalize()
    assert b.logit_rows().tolist() == [0, 4, 8] and b.n_logit_rows == 3
    with pytest.raises(ValueError):
        b.set_logit_positions([[5], [], []])


def test_builder_selects_components():
    from deepspeedsyclsupport_b200.ops.op_builder import builder as B
    rel = [os.path.relpath(s, B.CSRC).replace(os.sep, "/") for s in B.device_sources(["ragged", "gemm/gemm_bf16.cu"])]
    assert "ragged/latent_ops.cu" in rel and "gemm/gemm_bf16.cu" in rel and "common/host.cu" in rel
    assert not any(r.startswith(("optim/", "comm/")) or r == "gemm/gemm_fp8.cu" for r in rel)
    assert "--use_fast_math" not in B._flags_for(os.path.join(B.CSRC, "ragged", "latent_ops.cu")) and "--use_fast_math" in B._flags_for(os.path.join(B.CSRC, "norm", "norm.cu"))


# ------------------------------------------------------------------------------------------------------------- GPU: mechanisms
gpu = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def _tol(dt):
    return dict(rtol=2e-5, atol=2e-5) if dt == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def _K():
    from deepspeedsyclsupport_b200.inference.v2 import kernels
    return kernels


@gpu
@pytest.mark.parametrize("dim", [7, 64, 322])
def test_embedding_with_sinusoid(dim):
    K = _K()
    table = torch.randn(30, dim).bfloat16().cuda()
    ids = torch.tensor([3, 29, 0, 7, 7], device="cuda")
    pos = torch.tensor([0, 1, 4097, 63, 64], dtype=torch.int32, device="cuda")
    got = K.embed_sinusoid(ids, table, pos, K.sinusoid_frequencies(dim, device="cuda"))
    want = table.cpu().to(F64)[ids.cpu()] + O.sinusoid(pos.tolist(), dim)
    assert got.dtype == torch.float32 and torch.allclose(got.cpu().double(), want, rtol=0, atol=3e-6)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("dim", [5, 328, 1030])
def test_sandwich_norm_modes(dt, dim):
    K = _K()
    T, eps = 9, 1e-4
    x0 = torch.randn(T, dim).cuda() * 3
    y = (torch.randn(T, dim) * 5).to(dt).cuda()
    wb, w = (torch.randn(dim) * 0.3).cuda(), (torch.randn(dim) * 0.3).cuda()
    x1 = x0.double().cpu() + O.block_norm(y.cpu().double(), wb.cpu().double(), eps)
    x = x0.clone()
    out, out32 = K.sandwich_norm(x, y, wb, 1.0, w, 1.0, eps, out_dtype=dt, fp32_copy=True)
    assert torch.allclose(x.cpu().double(), x1, rtol=1e-6, atol=1e-5)
    assert torch.allclose(out.cpu().double(), O.block_norm(x1, w.cpu().double(), eps), **_tol(dt))
    assert out32.dtype == torch.float32 and torch.allclose(out32.cpu().double(), O.block_norm(x1, w.cpu().double(), eps), rtol=2e-5, atol=2e-5)
    assert torch.equal(out32.to(dt), out)  # the unrounded copy rounds to the activation-dtype output
    x = x0.clone()  # branch only
    assert K.sandwich_norm(x, y, wb, 1.0, None, 0.0, eps) is None and torch.allclose(x.cpu().double(), x1, rtol=1e-6, atol=1e-5)
    x = x0.clone()  # norm only, plain weight, gathered rows
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    out = K.sandwich_norm(x, w=w, o=0.0, eps=eps, out_dtype=torch.float32, rows=rows)
    assert torch.equal(x, x0) and torch.allclose(out.cpu().double(), O.latent_norm(x0.cpu().double()[rows.cpu().long()], w.cpu().double(), eps), rtol=1e-5, atol=1e-5)


def _paged(c_rows, block, perm_seed=0):
    """Latents of several sequences -> (cache [blocks, block, R], block table, tok_seq, tok_pos for ALL tokens) with shuffled pages."""
    R = c_rows[0].shape[1]
    need = [-(-len(c) // block) for c in c_rows]
    g = torch.Generator().manual_seed(perm_seed)
    ids = torch.randperm(sum(need) + 3, generator=g).tolist()
    cache = torch.full((sum(need) + 3, block, R), float("nan"), dtype=c_rows[0].dtype)
    bt = torch.zeros(len(c_rows), max(need), dtype=torch.int32)
    for s, c in enumerate(c_rows):
        for b in range(need[s]):
            bt[s, b] = ids.pop()
            chunk = c[b * block:(b + 1) * block]
            cache[bt[s, b], :len(chunk)] = chunk
    return cache, bt


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("H,R,block,splits", [(1, 24, 16, 1), (5, 64, 64, 3), (9, 96, 32, 1), (20, 200, 8, 7), (6, 33, 64, None)])
def test_latent_attention_over_pages(dt, H, R, block, splits):
    """Every query position of three ragged sequences (lengths around page borders) against the oracle's softmax over latents."""
    K = _K()
    torch.manual_seed(H * 1000 + R)
    lens = [block * 2 + 1, 1, block]
    c_rows = [torch.randn(n, R).to(dt) for n in lens]
    cache, bt = _paged(c_rows, block)
    tok_seq = torch.tensor(sum([[s] * n for s, n in enumerate(lens)], []), dtype=torch.int32)
    tok_pos = torch.tensor(sum([list(range(n)) for n in lens], []), dtype=torch.int32)
    q = (torch.randn(len(tok_seq), H, R) * 0.5).to(dt)
    scale = 0.37
    got = K.latent_attention(q.cuda(), cache.cuda(), tok_seq.cuda(), tok_pos.cuda(), bt.cuda(), scale, n_splits=splits)
    for t in range(len(tok_seq)):
        c = c_rows[int(tok_seq[t])][:int(tok_pos[t]) + 1].double()
        p = torch.softmax((q[t].double() @ c.T) * scale, -1)
        assert torch.allclose(got[t].cpu().double(), p @ c, rtol=1e-4, atol=1e-4), t


@gpu
@pytest.mark.parametrize("H,R,block,decode", [(4, 64, 16, False), (8, 128, 64, False), (16, 128, 128, True), (2, 128, 32, True), (32, 64, 64, False)])
def test_tensor_core_latent_attention(H, R, block, decode):
    """The one-plane mode of the paged flash kernels against the oracle's softmax over latents (bf16 operands)."""
    K = _K()
    torch.manual_seed(H + R)
    lens = [block * 2 + 1, 1, 300] if not decode else [block * 2 + 1, 1, 300, 129]
    c_rows = [torch.randn(n, R).bfloat16() for n in lens]
    cache, bt = _paged(c_rows, block)
    cache = torch.nan_to_num(cache, nan=0.0)  # rows past a sequence's end are read (and masked) by the kernel: they must be finite
    if decode:  # the last token of every sequence
        tok_seq = torch.arange(len(lens), dtype=torch.int32)
        tok_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    else:
        tok_seq = torch.tensor(sum([[s] * n for s, n in enumerate(lens)], []), dtype=torch.int32)
        tok_pos = torch.tensor(sum([list(range(n)) for n in lens], []), dtype=torch.int32)
    q = (torch.randn(len(tok_seq), H, R) * 0.5).bfloat16()
    got = K.paged_latent_flash(q.cuda(), cache.cuda(), tok_seq.cuda(), tok_pos.cuda(), bt.cuda(), 0.2, decode=decode)
    for t in range(len(tok_seq)):
        c = c_rows[int(tok_seq[t])][:int(tok_pos[t]) + 1].double()
        p = torch.softmax((q[t].double() @ c.T) * 0.2, -1)
        assert torch.allclose(got[t].cpu().double(), p @ c, rtol=3e-2, atol=3e-2), t


@gpu
def test_tensor_core_latent_attention_finds_one_far_key():
    K = _K()
    n, R, H, block = 2048, 64, 8, 64
    for far in (0, 63, 64, 1500, 2047):
        c = (torch.randn(n, R) * 0.1).bfloat16()
        c[far] = (torch.randn(R).sign() * 2.0).bfloat16()
        q = (c[far].float().repeat(H, 1)[None] * 4.0).bfloat16()
        cache, bt = _paged([c], block, perm_seed=far)
        cache = torch.nan_to_num(cache, nan=0.0)
        z = torch.zeros(1, dtype=torch.int32).cuda()
        got = K.paged_latent_flash(q.cuda(), cache.cuda(), z, torch.tensor([n - 1], dtype=torch.int32).cuda(), bt.cuda(), 1.0)
        assert torch.allclose(got.cpu()[0].float(), c[far].float().expand(H, R), atol=2e-2), far
        if far > 0:
            got = K.paged_latent_flash(q.cuda(), cache.cuda(), z, torch.tensor([far - 1], dtype=torch.int32).cuda(), bt.cuda(), 1.0)
            assert (got.cpu()[0].float() - c[far].float()).abs().max() > 1.0, far
        lo, hi = max(far - 2, 0), min(far + 3, n)  # a prompt portion across the key
        pos = torch.arange(lo, hi, dtype=torch.int32)
        got = K.paged_latent_flash(q.expand(len(pos), H, R).contiguous().cuda(), cache.cuda(), torch.zeros(len(pos), dtype=torch.int32).cuda(), pos.cuda(),
                                   bt.cuda(), 1.0)
        for i, p_ in enumerate(pos.tolist()):
            seen = torch.allclose(got.cpu()[i].float(), c[far].float().expand(H, R), atol=2e-2)
            assert seen == (p_ >= far), (far, p_)


@gpu
def test_bf16_model_on_the_cuda_core_attention_too(tmp_path_factory, monkeypatch):
    """bf16 normally takes the tensor-core attention; with it switched off the general kernel serves the same model."""
    monkeypatch.setenv("DSB200_LATENT_FLASH", "0")
    cfg, w, path = _model("aligned", tmp_path_factory, torch.bfloat16)
    eng = _engine(path, torch.bfloat16)
    assert not eng.model().attn_mods[0]._flash and eng.model().attn_mods[1].cache_rank == 96
    toks = _tokens(cfg, 40, 3)
    want = O.forward(cfg, w, toks.tolist())
    got = torch.cat([eng.put([1], [toks[:33]], logit_positions=[list(range(33))])] + [eng.put([1], [toks[i:i + 1]]) for i in range(33, 40)])
    ok, err = _close(got, want, torch.bfloat16)
    assert ok, err


@gpu
@pytest.mark.parametrize("far", [0, 63, 64, 700, 1023])
def test_latent_attention_finds_one_far_key(far):
    """One latent far back (also at a page's first and last row) is made to dominate: the output must be that row."""
    K = _K()
    n, R, H, block = 1024, 48, 3, 64
    c = torch.randn(n, R) * 0.1
    c[far] = torch.randn(R).sign() * 2.0
    q = c[far].repeat(H, 1)[None] * 4.0  # score of the far key = 4 * |c|^2 = 768, all others ~ 0
    cache, bt = _paged([c], block, perm_seed=far)
    for pos in (n - 1, max(far, 1)):
        got = K.latent_attention(q.cuda(), cache.cuda(), torch.zeros(1, dtype=torch.int32).cuda(), torch.tensor([pos], dtype=torch.int32).cuda(), bt.cuda(), 1.0)
        assert torch.allclose(got.cpu()[0], c[far].expand(H, R), atol=1e-5)
    if far > 0:  # the key just after the last visible position must not be seen
        got = K.latent_attention(q.cuda(), cache.cuda(), torch.zeros(1, dtype=torch.int32).cuda(), torch.tensor([far - 1], dtype=torch.int32).cuda(), bt.cuda(), 1.0)
        assert (got.cpu()[0] - c[far]).abs().max() > 1.0
    # the same inside a prompt portion that starts before the key and runs past it: rows before it do not see it, rows from it on do
    lo, hi = max(far - 2, 0), min(far + 3, n)
    pos = torch.arange(lo, hi, dtype=torch.int32)
    got = K.latent_attention(q.expand(len(pos), H, R).contiguous().cuda(), cache.cuda(), torch.zeros(len(pos), dtype=torch.int32).cuda(), pos.cuda(), bt.cuda(), 1.0)
    for i, p_ in enumerate(pos.tolist()):
        seen = torch.allclose(got.cpu()[i], c[far].expand(H, R), atol=1e-5)
        assert seen == (p_ >= far), (far, p_)


@gpu
@pytest.mark.parametrize("dt", DTYPES)
def test_latent_norm_and_append(dt):
    K = _K()
    T, nq, nkv, block, eps = 11, 10, 12, 4, 1e-5
    lat = torch.randn(T, nq + nkv + 5).to(dt).cuda()  # wider rows: the gate columns follow the latents
    wq, wkv = torch.rand(nq).cuda() + 0.5, torch.rand(nkv).cuda() + 0.5
    cache = torch.zeros(9, block, nkv, dtype=dt, device="cuda")
    bt = torch.tensor([[7, 2, 5], [1, 0, 0]], dtype=torch.int32, device="cuda")
    tok_seq = torch.tensor([0] * 9 + [1] * 2, dtype=torch.int32, device="cuda")
    tok_pos = torch.tensor(list(range(3, 12)) + [0, 1], dtype=torch.int32, device="cuda")  # sequence 0 continues at position 3
    cq = K.latent_norm_append(lat, wq, wkv, cache, tok_seq, tok_pos, bt, nq, nkv, eps)
    L = lat.cpu().double()
    assert torch.allclose(cq.cpu().double(), O.latent_norm(L[:, :nq], wq.cpu().double(), eps), **_tol(dt))
    want = O.latent_norm(L[:, nq:nq + nkv], wkv.cpu().double(), eps)
    for t in range(T):
        s, p = int(tok_seq[t]), int(tok_pos[t])
        assert torch.allclose(cache[int(bt[s, p // block]), p % block].cpu().double(), want[t], **_tol(dt))
    assert float(cache[3].abs().max()) == 0 and float(cache[7, :3].abs().max()) == 0  # untouched pages / rows stay untouched


@gpu
@pytest.mark.parametrize("E,top,G,keep", [(8, 3, 2, 1), (6, 2, 3, 2), (12, 1, 1, 1), (16, 5, 4, 4), (9, 3, 3, 1), (64, 8, 8, 3)])
def test_grouped_router(E, top, G, keep):
    K = _K()
    torch.manual_seed(E + top)
    z = (torch.randn(40, E) * 2).cuda()
    corr = torch.randn(E).cuda() * 0.5 - 0.6  # mostly negative selection scores: an excluded group must count as -inf, not 0
    counts, scores, asg, off = K.grouped_topk_gating(z, top, corr, G, keep)
    chosen, weights = O.route(z.cpu().double(), corr.cpu().double(), top, G, keep)
    assert torch.equal(asg.cpu().long(), chosen) and torch.allclose(scores.cpu().double(), weights, rtol=1e-5, atol=1e-7)
    assert torch.equal(counts.cpu().long(), torch.bincount(chosen.flatten(), minlength=E))
    for e in range(E):  # offsets number the rows of an expert
        assert sorted(off[asg == e].tolist()) == list(range(int(counts[e])))


@gpu
@pytest.mark.parametrize("dt", DTYPES)
def test_expert_pieces(dt):
    K = _K()
    torch.manual_seed(3)
    T, D, E, top, ff = 37, 24, 5, 2, 16
    h = torch.randn(T, D).to(dt).cuda()
    z = torch.randn(T, E).cuda()
    counts, scores, asg, off = K.grouped_topk_gating(z, top, None, 1, 1)
    moe_in, cumsum, slots = K.moe_scatter_rows(h, counts, asg, off)
    assert cumsum.tolist() == torch.cumsum(counts.long(), 0).tolist()
    for k in range(top):
        assert torch.equal(moe_in[slots[:, k].long()], h)
    w1, w2 = (torch.randn(E, 2 * ff, D) / 4).to(dt).cuda(), (torch.randn(E, D, ff) / 3).to(dt).cuda()
    gu = K.moe_gemm_rows(moe_in, w1, cumsum)
    act = K.clamped_swish_gate(gu, 1.702, 1.5, 1.0)
    out = K.moe_gemm_rows(act, w2, cumsum)
    y = K.moe_gather_rows(out, scores, slots)
    want = torch.zeros(T, D, dtype=F64)
    for t in range(T):
        for k in range(top):
            e = int(asg[t, k])
            want[t] += float(scores[t, k]) * O.expert(h[t:t + 1].cpu().double(), w1[e, :ff].cpu().double(), w1[e, ff:].cpu().double(), w2[e].cpu().double(), 1.5)[0]
    assert y.dtype == torch.float32 and torch.allclose(y.cpu().double(), want, **(dict(rtol=1e-4, atol=1e-4) if dt == torch.float32 else dict(rtol=5e-2, atol=5e-2)))
    if dt == torch.bfloat16:  # the tensor-core grouped GEMM agrees with the CUDA-core one where it applies
        from deepspeedsyclsupport_b200.ops.gemm import moe_gemm
        assert torch.allclose(moe_gemm(moe_in, w1, cumsum).float(), gu.float(), rtol=2e-2, atol=2e-2)


@gpu
def test_gate_and_softcap():
    K = _K()
    a, g = torch.randn(6, 10).cuda(), torch.randn(6, 14).cuda()
    want = a.cpu().double() * torch.sigmoid(g[:, 3:13].cpu().double())
    K.sigmoid_gate_mul(a, g[:, 3:13])
    assert torch.allclose(a.cpu().double(), want, rtol=1e-6, atol=1e-6)
    x = (torch.randn(4, 9) * 40).cuda()
    want = 15.0 * torch.tanh(x.cpu().double() / 15.0)
    assert torch.allclose(K.softcap_(x[:, :7], 15.0).cpu().double(), want[:, :7], rtol=1e-6, atol=1e-5) and torch.allclose(x[:, 7:].cpu().double(), (want * 0 + x.cpu().double())[:, 7:])


# ------------------------------------------------------------------------------------------------------------ GPU: whole models
CONFIGS = {
    # odd sizes everywhere, layers that differ, a loop over a dense-only and a MoE layer, groups > kept, top 1
    "odd": O.make_config(44, 61, [O.layer_cfg(3, 12, 10, 20, 14, 0.31, (6, 2, 3, 2, 18, 1.5)), O.layer_cfg(5, 6, 9, 33, 9, 0.2),
                                  O.layer_cfg(2, 16, 8, 16, 24, 0.25, (4, 1, 1, 1, 7, 2.5))], loop={"start": 1, "stop": 3, "times": 2}, eps=1e-5, softcap=9.0),
    # aligned sizes (tensor-core GEMMs in bf16), more heads than one head group, no loop, one group
    "aligned": O.make_config(64, 96, [O.layer_cfg(10, 32, 16, 64, 48, 0.18, (8, 3, 1, 1, 32, 2.0)), O.layer_cfg(4, 16, 32, 96, 32, 0.25, (8, 4, 4, 2, 16, 1.0))],
                             eps=1e-6, softcap=30.0),
    # a single dense layer run three times
    "looped": O.make_config(24, 40, [O.layer_cfg(2, 8, 8, 8, 8, 0.35)], loop={"start": 0, "stop": 1, "times": 3}, eps=1e-5, softcap=50.0),
}
_MODELS = {}


def _model(name, tmp_path_factory, dt=torch.float32):
    """fp32 runs get an informative router (every selection is compared tightly); bf16 runs get well separated selections."""
    sep = dt == torch.bfloat16
    if (name, sep) not in _MODELS:
        cfg = CONFIGS[name]
        w = O.random_weights(cfg, seed=len(name), separated_router=sep)
        _MODELS[(name, sep)] = (cfg, w, O.write_model(str(tmp_path_factory.mktemp(name)), cfg, w))
    return _MODELS[(name, sep)]


def _engine(path, dt, pool_tokens=256, block=16, max_seqs=4):
    from deepspeedsyclsupport_b200.inference.v2.config_v2 import RaggedInferenceEngineConfig
    from deepspeedsyclsupport_b200.inference.v2.engine_factory import build_hf_engine
    from deepspeedsyclsupport_b200.inference.v2.ragged.manager_configs import AllocationMode, DSStateManagerConfig, MemoryConfig
    mgr = DSStateManagerConfig(max_tracked_sequences=max_seqs, max_ragged_sequence_count=max_seqs, max_ragged_batch_size=pool_tokens, max_context=pool_tokens,
                               memory_config=MemoryConfig(mode=AllocationMode.ALLOCATE, size=pool_tokens // block), kv_block_size=block)
    return build_hf_engine(path, RaggedInferenceEngineConfig(state_manager=mgr), dtype=dt)


def _close(got, want, dt):
    """Every logit row agrees up to a per-row shift, relative to the spread of the logits.  fp32: tightly.  bf16: within what rounding
    alone does to these random models (a plain pipeline with bf16-rounded matrix products lands at a median of ~0.02 and rows up to
    ~0.09 of the spread), far below what a wrong key, a lost page or a wrong expert would cause (order 1)."""
    d = got.cpu().double() - want
    d = d - d.mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std()
    if dt == torch.float32:
        return float(err.max()) < 2e-5, float(err.max())
    return float(err.max()) < 0.15 and float(err.median()) < 0.04, (float(err.median()), float(err.max()))


def _tokens(cfg, n, seed):
    return torch.randint(0, cfg["vocab"], (n, ), generator=torch.Generator().manual_seed(seed))


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_and_every_layer(name, dt, tmp_path_factory):
    cfg, w, path = _model(name, tmp_path_factory, dt)
    eng = _engine(path, dt)
    toks = _tokens(cfg, 45, 1)
    res, got_res = [], []
    want = O.forward(cfg, w, toks.tolist(), res)
    eng.model()._layer_hook = lambda run, x: got_res.append(x.clone())
    got = eng.put([7], [toks], logit_positions=[list(range(45))])
    assert got.shape == (45, cfg["vocab"]) and len(got_res) == len(res)
    for r, (a, b) in enumerate(zip(got_res, res)):
        if dt == torch.float32:
            assert torch.allclose(a.cpu().double(), b, rtol=1e-4, atol=1e-4), f"layer run {r}"
        else:
            row = (a.cpu().double() - b).norm(dim=-1) / b.norm(dim=-1)
            assert float(row.max()) < 0.15 and float(row.median()) < 0.03, f"layer run {r}"
    ok, err = _close(got, want, dt)
    assert ok, err
    assert got[0].isfinite().all()  # the first token attends to itself only


@gpu
@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("name,cuts", [("odd", [1] * 40), ("odd", [2, 2, 15, 1, 17, 3]), ("aligned", [16, 16, 1, 1, 6]), ("aligned", [31, 2, 7]), ("looped", [3, 33, 2, 2])])
def test_portions_and_token_by_token_equal_the_whole_prompt(name, cuts, dt, tmp_path_factory):
    """Prefill against decoding token by token, and portions cut inside pages (block 16) down to two tokens."""
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
def test_unequal_requests_in_one_batch_and_reused_pages(dt, tmp_path_factory):
    """Four requests of unequal length share steps (portions beside single tokens), finish at different times, and two more
    take over their sequence slots and pages: every logit row equals the request run alone."""
    cfg, w, path = _model("odd", tmp_path_factory, dt)
    eng = _engine(path, dt, pool_tokens=160, block=16)
    prompts = {u: _tokens(cfg, n, 10 + u) for u, n in ((0, 50), (1, 17), (2, 33), (3, 1), (4, 48), (5, 31))}
    want = {u: O.forward(cfg, w, p.tolist()) for u, p in prompts.items()}
    schedule = [[(0, 20), (1, 16), (3, 1)], [(0, 1), (1, 1), (2, 30)], [(0, 29), (2, 1)], [(2, 2), (4, 15)], [(4, 33), (5, 2)], [(5, 29)]]
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
    for u in prompts:
        ok, err = _close(torch.cat(got[u]), want[u], dt)
        assert ok, (u, err)


@gpu
def test_long_decoding_through_the_step_graphs(tmp_path_factory):
    """A prompt, then 150 single-token steps (the steady-state ones replay a captured graph); some steps ask for no logits."""
    cfg, w, path = _model("aligned", tmp_path_factory)
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
    graphs = eng.model()._graphs  # both kinds of step (one logit row, none) were captured and replayed
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
    """bin/trace_run as a process: portions of three requests beside single tokens, a request that pauses for a step, wanted
    positions anywhere in a portion, requests ending at different steps with their pages reused by a later one (pool of 3 pages)."""
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
    # live tokens never exceed 192 = three 64-token pages: a (70 -> 2 pages) + b (1 page), then a + c, then d alone (2 pages)
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
