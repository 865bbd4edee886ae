"""Plain, slow float64 statement of the Linasun design, one function per mechanism, used as the oracle of tests/test_linasun.py.
Nothing here imports the package under test.

Notation: x is the residual stream [n, width]; a linear weight has shape [out, in] and acts as x @ W.T; position indices are zero-based."""
import json
import math
import os

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x scaled to unit RMS; eps joins the mean square before the square root is taken."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def block_norm(x, w, eps):
    """Norm of the blocks and of the output: zero-centred weight (applied as 1 + w)."""
    return rms_unit(x, eps) * (1.0 + w)


def latent_norm(x, w, eps):
    """Norm of the two latents: plain weight."""
    return rms_unit(x, eps) * w


def sinusoid(positions, width):
    """[n, width]: entry 2i = sin(p * 10000^(-2i/width)), entry 2i+1 = cos(p * 10000^(-2i/width))."""
    out = torch.zeros(len(positions), width, dtype=F64)
    for r, p in enumerate(positions):
        for e in range(width):
            i = e // 2
            ang = float(p) * 10000.0 ** (-2.0 * i / width)
            out[r, e] = math.sin(ang) if e % 2 == 0 else math.cos(ang)
    return out


def latent_attention_mixer(h, W, pre, m, eps):
    """h [n, width] (positions 0 .. n-1 of one sequence).  Returns the mixer output before norm1b and the cached latents."""
    n = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = latent_norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps)
    q = (cq @ W[pre + "uq"].T).view(n, H, d)
    c = latent_norm(h @ W[pre + "dkv"].T, W[pre + "dkv.norm"], eps)  # the only thing a cache needs
    k = (c @ W[pre + "uk"].T).view(n, H, d)
    v = (c @ W[pre + "uv"].T).view(n, H, dv)
    out = torch.zeros(n, H, dv, dtype=F64)
    for i in range(n):
        for hh in range(H):
            s = (k[:i + 1, hh] @ q[i, hh]) * m["scale"]  # causal: keys 0 .. i
            p = torch.softmax(s, 0)
            out[i, hh] = p @ v[:i + 1, hh]
    gate = torch.sigmoid(h @ W[pre + "g"].T)
    return (out.reshape(n, H * dv) * gate) @ W[pre + "o"].T, c


def route(z, correction, top, groups, keep):
    """z [n, E] router logits.  Returns (chosen experts [n, top], their weights [n, top])."""
    n, E = z.shape
    s = torch.softmax(z, -1)
    choice = s + correction
    per = E // groups
    chosen, weights = [], []
    for t in range(n):
        gscore = [max(float(choice[t, g * per + j]) for j in range(per)) for g in range(groups)]
        best_groups = sorted(range(groups), key=lambda g: (-gscore[g], g))[:keep]
        allowed = [e for e in range(E) if e // per in best_groups]
        picks = sorted(allowed, key=lambda e: (-float(choice[t, e]), e))[:top]
        chosen.append(picks)
        weights.append([float(s[t, e]) for e in picks])  # uncorrected, not renormalised
    return torch.tensor(chosen), torch.tensor(weights, dtype=F64)


def expert(h, Wg, Wu, Wd, limit):
    g = torch.clamp(h @ Wg.T, max=limit)
    u = torch.clamp(h @ Wu.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ Wd.T


def moe(h, W, pre, f):
    r = f["router"]
    gr = r.get("groups") or {"count": 1, "keep": 1}
    chosen, weights = route(h @ W[pre + "router"].T, W[pre + "correction"], r["top"], gr["count"], gr["keep"])
    y = torch.zeros(h.shape[0], W[pre + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, wgt in zip(chosen[t].tolist(), weights[t].tolist()):
            y[t] += wgt * expert(h[t:t + 1], W[pre + f"e{e}.gate"], W[pre + f"e{e}.up"], W[pre + f"e{e}.down"], f["expert"]["limit"])[0]
    return y


def run_order(cfg):
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    return list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"] + list(range(lp["stop"], n))


def forward(cfg, weights, tokens, residuals=None):
    """Logits [n, vocab] of a whole sequence.  `residuals`: list that receives the stream after every layer run."""
    W = {k: v.to(F64) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens)] + sinusoid(range(len(tokens)), cfg["width"])
    for li in run_order(cfg):
        L, pre = cfg["layers"][li], f"l{li}."
        assert L["type"] == "latent_attention"
        y, _ = latent_attention_mixer(block_norm(x, W[pre + "norm1"], eps), W, pre + "mix.", L["mixer"], eps)
        x = x + block_norm(y, W[pre + "norm1b"], eps)
        if L["mlp"] is not None:
            y = moe(block_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.", L["mlp"])
            x = x + block_norm(y, W[pre + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    z = block_norm(x, W["final.norm"], eps) @ W["head"].T
    cap = cfg.get("logit_softcap", 0.0)
    return cap * torch.tanh(z / cap) if cap else z


def greedy(cfg, weights, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]


# ------------------------------------------------------------------------------------------------ random models for the tests
def layer_cfg(heads, dim, vdim, kv_rank, q_rank, scale, moe=None):
    """moe: None or (experts, top, group count, groups kept, ff, limit)."""
    mlp = None
    if moe is not None:
        E, top, G, keep, ff, limit = moe
        mlp = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
               "router": {"experts": E, "top": top, "groups": {"count": G, "keep": keep}}}
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale},
            "mlp": mlp}


def make_config(width, vocab, layers, loop=None, eps=1e-5, softcap=20.0):
    return {"architecture": "Linasun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_softcap": softcap,
            "layers": layers, "loop": loop or {"start": 0, "stop": 0, "times": 1}}


def random_weights(cfg, seed=0, dtype=torch.bfloat16, separated_router=False):
    """Weights in the checkpoint's naming, rounded to `dtype` (the oracle then uses the same rounded values).
    `separated_router`: the per-expert correction terms are a permutation of 0, 2, 4, ...: the selection then never hangs on a
    close call (a 16-bit run of a random model otherwise picks another expert for a few tokens, and that spreads through attention),
    while the combine weights stay the informative softmax scores."""
    g = torch.Generator().manual_seed(seed)
    D, V = cfg["width"], cfg["vocab"]

    def lin(o, i, gain=1.0):
        return (torch.randn(o, i, generator=g) * gain / math.sqrt(i)).to(dtype)

    def small(n, s=0.2):
        return (torch.randn(n, generator=g) * s).to(dtype)

    W = {"embed": (torch.randn(V, D, generator=g)).to(dtype), "final.norm": small(D), "head": lin(V, D, 2.0)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, d, dv, R, Q = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        for nm in ("norm1", "norm1b", "norm2", "norm2b"):
            if L["mlp"] is not None or nm in ("norm1", "norm1b"):
                W[p + nm] = small(D)
        W[p + "mix.dq"], W[p + "mix.dq.norm"] = lin(Q, D), (1.0 + small(Q)).to(dtype)
        W[p + "mix.uq"] = lin(H * d, Q, 2.0)
        W[p + "mix.dkv"], W[p + "mix.dkv.norm"] = lin(R, D), (1.0 + small(R)).to(dtype)
        W[p + "mix.uk"], W[p + "mix.uv"] = lin(H * d, R, 2.0), lin(H * dv, R)
        W[p + "mix.g"], W[p + "mix.o"] = lin(H * dv, D), lin(D, H * dv)
        if L["mlp"] is not None:
            f = L["mlp"]
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            W[p + "mlp.router"] = lin(E, D, 3.0)
            W[p + "mlp.correction"] = (2.0 * torch.randperm(E, generator=g).float()).to(dtype) if separated_router else small(E, 0.3)
            for e in range(E):
                W[p + f"mlp.e{e}.gate"], W[p + f"mlp.e{e}.up"], W[p + f"mlp.e{e}.down"] = lin(ff, D, 2.0), lin(ff, D, 2.0), lin(D, ff)
    return W


def write_model(folder, cfg, weights):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw little-endian data)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
    header, blobs, off = {}, [], 0
    for k, t in weights.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 else t.view(torch.int16).numpy().tobytes()
        header[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(len(hj).to_bytes(8, "little"))
        f.write(hj)
        for b in blobs:
            f.write(b)
    return folder
