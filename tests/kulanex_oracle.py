"""Plain, slow float64 statement of the Kulanex design, one function per mechanism, token by token where the design is recurrent.
It shares no code with the engine: tests compare the engine's kernels, cache and state handling against these functions.

A model is (config dict, weights dict).  Weights are keyed by the checkpoint's tensor names (`l<i>.mix...`, `l<i>.mlp...`, `embed`,
`final.norm`, `head`); linear weights are [out, in].  Everything here works on one sequence at a time: [T, ...] tensors, positions 0 .. T-1.
"""
import math

import torch

F64 = torch.float64


def f64(t):
    return t.to(F64)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def logsigmoid(z):
    return -softplus(-z)


def short_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the first token (the last column weighs the
    current token)."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` (factor, low, high, original) long wavelengths are slowed down: wavelengths
    above original/low are divided by factor, below original/high kept, and blended linearly in between."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if scaling:
        factor, low, high, orig = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"]), float(scaling["original"])
        out = []
        for fi in f:
            wl = 2.0 * math.pi / fi
            if wl < orig / high:
                out.append(fi)
            elif wl > orig / low:
                out.append(fi / factor)
            else:
                s = (orig / wl - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate_interleaved(x, pos, freqs):
    """x [T, H, dim], pos [T]: pairs (2i, 2i+1) of the first 2 * len(freqs) entries of each head are rotated by pos * f_i."""
    out = x.clone()
    n = freqs.numel()
    ang = pos.to(F64)[:, None] * freqs[None, :]  # [T, n]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


def window_visible(T, size, keep_first):
    """[T, T] bool: query i sees key j iff j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def windowed_attention(h, w, pre, m, eps):
    """The attention half of a 'parallel' mixer.  h [T, width]; w weights; pre = tensor-name prefix ('l0.mix.left'); m its config."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    assert m["vdim"] == d, "the values are the keys: vdim equals dim"
    q = short_conv(h @ f64(w[pre + ".q"]).T, f64(w[pre + ".q.conv"]))
    k = short_conv(h @ f64(w[pre + ".k"]).T, f64(w[pre + ".k.conv"]))
    v = k.clone().reshape(T, G, d)  # as it leaves the convolution
    q = (rms(q, eps) * f64(w[pre + ".q.norm"])).reshape(T, H, d)
    k = (rms(k, eps) * f64(w[pre + ".k.norm"])).reshape(T, G, d)
    fr = rotary_frequencies(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    pos = torch.arange(T)
    q, k = rotate_interleaved(q, pos, fr), rotate_interleaved(k, pos, fr)
    vis = window_visible(T, m["mask"]["size"], m["mask"]["keep_first"])
    out = torch.zeros(T, H, d, dtype=F64)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~vis, float("-inf"))
        out[:, hh] = torch.softmax(s, -1) @ v[:, g]
    return out.reshape(T, H * d) @ f64(w[pre + ".o"]).T


def matrix_memory(h, w, pre, m, eps):
    """The recurrent half of a 'parallel' mixer: a matrix memory per head with exponential input gate, sigmoid forget gate in log space
    and a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (h @ f64(w[pre + ".q"]).T * d ** -0.5).reshape(T, H, d)
    k = (h @ f64(w[pre + ".k"]).T).reshape(T, H, d)
    v = (h @ f64(w[pre + ".v"]).T).reshape(T, H, dv)
    ig = cap * torch.tanh((h @ f64(w[pre + ".i"]).T + f64(w[pre + ".i.b"])) / cap)  # [T, H]
    fg = logsigmoid(cap * torch.tanh((h @ f64(w[pre + ".f"]).T + f64(w[pre + ".f.b"])) / cap))
    S = torch.zeros(H, d, dv, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(fg[t] + mx, ig[t])
        a, b = torch.exp(fg[t] + mx - m_new), torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = num / den[:, None]
    o = rms(o, eps).reshape(T, H * dv) * f64(w[pre + ".norm"])
    o = o * torch.sigmoid(h @ f64(w[pre + ".g"]).T)
    return o @ f64(w[pre + ".o"]).T


def parallel_mixer(h, w, pre, m, eps):
    return m["left_scale"] * windowed_attention(h, w, pre + ".left", m["left"], eps) + \
        m["right_scale"] * matrix_memory(h, w, pre + ".right", m["right"], eps)


def channel_delta(h, w, pre, m, eps):
    """Gated delta rule with one decay per head and key channel."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ f64(w[pre + ".q"]).T, f64(w[pre + ".q.conv"]))).reshape(T, G, d)
    k = silu(short_conv(h @ f64(w[pre + ".k"]).T, f64(w[pre + ".k.conv"]))).reshape(T, G, d)
    v = silu(short_conv(h @ f64(w[pre + ".v"]).T, f64(w[pre + ".v.conv"]))).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ f64(w[pre + ".b"]).T)  # [T, H]
    a = (h @ f64(w[pre + ".a1"]).T) @ f64(w[pre + ".a2"]).T + f64(w[pre + ".dt_bias"])
    decay = torch.exp(-torch.exp(f64(w[pre + ".A_log"]))[None, :, None] * softplus(a).reshape(T, H, d))  # [T, H, d]
    S = torch.zeros(H, d, dv, dtype=F64)
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            g = hh // (H // G)
            Sh = decay[t, hh][:, None] * S[hh]
            u = beta[t, hh] * (v[t, hh] - Sh.T @ k[t, g])
            Sh = Sh + k[t, g][:, None] * u[None, :]
            S[hh] = Sh
            o[t, hh] = Sh.T @ q[t, g]
    o = rms(o, eps) * f64(w[pre + ".norm"])[None, None, :]
    o = o.reshape(T, H * dv) * torch.sigmoid((h @ f64(w[pre + ".g1"]).T) @ f64(w[pre + ".g2"]).T)
    return o @ f64(w[pre + ".o"]).T


def sigmoid_moe(h, w, pre, f):
    """Experts chosen by the largest sigmoid scores; the score scales the expert's INPUT; no renormalisation."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ f64(w[pre + ".router"]).T)  # [T, E]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(s[t], top).indices.tolist():
            x = s[t, e] * h[t]
            p = pre + ".e%d" % e
            out[t] += f64(w[p + ".down"]) @ (silu(f64(w[p + ".gate"]) @ x) * (f64(w[p + ".up"]) @ x))
    return out


def zero_centred_norm(x, weight, eps):
    return rms(x, eps) * (1.0 + f64(weight))


def forward(cfg, w, tokens, collect_layers=False):
    """Logits [T, vocab] of one sequence (float64); with `collect_layers` also the residual stream after every layer."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = f64(w["embed"])[torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    for i, L in enumerate(cfg["layers"]):
        p = "l%d" % i
        if L["type"] == "parallel":
            y = parallel_mixer(x, w, p + ".mix", L["mixer"], eps)
        elif L["type"] == "channel_delta":
            y = channel_delta(x, w, p + ".mix", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + mult * zero_centred_norm(y, w[p + ".norm1"], eps)
        if L.get("mlp") is not None:
            x = x + mult * zero_centred_norm(sigmoid_moe(x, w, p + ".mlp", L["mlp"]), w[p + ".norm2"], eps)
        streams.append(x.clone())
    logits = zero_centred_norm(x, w["final.norm"], eps) @ f64(w["head"]).T
    return (logits, torch.stack(streams)) if collect_layers else logits


# ---- random models for the tests
def random_weights(cfg, seed=0, router_gain=1.0):
    """Weights of the right shapes, drawn so that every mechanism matters (gates neither saturated nor dead); values are bf16-exact."""
    g = torch.Generator().manual_seed(seed)
    D = cfg["width"]
    w = {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16)

    w["embed"] = rnd(cfg["vocab"], D)
    w["head"] = rnd(cfg["vocab"], D, std=D ** -0.5)
    w["final.norm"] = rnd(D, std=0.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d" % i, L["mixer"]
        w[p + ".norm1"] = rnd(D, std=0.2)
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            nq, nk = a["heads"] * a["dim"], a["kv_heads"] * a["dim"]
            for nm, n in (("q", nq), ("k", nk)):
                w[f"{p}.mix.left.{nm}"] = rnd(n, D, std=D ** -0.5)
                w[f"{p}.mix.left.{nm}.conv"] = rnd(n, a["conv"], std=0.6, mean=0.2)
                w[f"{p}.mix.left.{nm}.norm"] = rnd(n, std=0.3, mean=1.1)
            w[p + ".mix.left.o"] = rnd(D, a["heads"] * a["vdim"], std=(a["heads"] * a["vdim"]) ** -0.5)
            hd, hv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            w[p + ".mix.right.q"] = rnd(hd, D, std=D ** -0.5)
            w[p + ".mix.right.k"] = rnd(hd, D, std=D ** -0.5)
            w[p + ".mix.right.v"] = rnd(hv, D, std=D ** -0.5)
            w[p + ".mix.right.g"] = rnd(hv, D, std=D ** -0.5)
            w[p + ".mix.right.o"] = rnd(D, hv, std=hv ** -0.5)
            w[p + ".mix.right.norm"] = rnd(hv, std=0.2, mean=1.0)
            w[p + ".mix.right.i"] = rnd(r["heads"], D, std=D ** -0.5)
            w[p + ".mix.right.i.b"] = rnd(r["heads"], std=0.3)
            w[p + ".mix.right.f"] = rnd(r["heads"], D, std=D ** -0.5)
            w[p + ".mix.right.f.b"] = rnd(r["heads"], std=1.5, mean=3.0)
        else:
            nqk, nv, lr = m["kv_heads"] * m["dim"], m["heads"] * m["vdim"], m.get("_low_rank", 8)
            for nm, n in (("q", nqk), ("k", nqk), ("v", nv)):
                w[f"{p}.mix.{nm}"] = rnd(n, D, std=D ** -0.5)
                w[f"{p}.mix.{nm}.conv"] = rnd(n, m["conv"], std=0.6, mean=0.25)
            w[p + ".mix.b"] = rnd(m["heads"], D, std=D ** -0.5)
            w[p + ".mix.A_log"] = rnd(m["heads"], std=0.8, mean=-2.5)
            w[p + ".mix.norm"] = rnd(m["vdim"], std=0.2, mean=1.0)
            w[p + ".mix.a1"] = rnd(lr, D, std=D ** -0.5)
            w[p + ".mix.a2"] = rnd(m["heads"] * m["dim"], lr, std=lr ** -0.5)
            w[p + ".mix.dt_bias"] = rnd(m["heads"] * m["dim"], std=0.8, mean=-2.0)
            w[p + ".mix.g1"] = rnd(lr, D, std=D ** -0.5)
            w[p + ".mix.g2"] = rnd(nv, lr, std=lr ** -0.5)
            w[p + ".mix.o"] = rnd(D, nv, std=nv ** -0.5)
        f = L.get("mlp")
        if f is not None:
            w[p + ".norm2"] = rnd(D, std=0.2)
            w[p + ".mlp.router"] = rnd(f["router"]["experts"], D, std=router_gain * D ** -0.5)
            ff = f["expert"]["ff"]
            for e in range(f["router"]["experts"]):
                w[f"{p}.mlp.e{e}.gate"] = rnd(ff, D, std=D ** -0.5)
                w[f"{p}.mlp.e{e}.up"] = rnd(ff, D, std=D ** -0.5)
                w[f"{p}.mlp.e{e}.down"] = rnd(D, ff, std=ff ** -0.5)
    return w


def parallel_layer(heads=4, kv_heads=2, dim=16, conv=4, window=24, keep_first=2, rot_dims=8, base=10000.0, scaling=None, scale=0.25,
                   r_heads=2, r_dim=8, r_vdim=16, gate_cap=15.0, left_scale=1.0, right_scale=1.0, mlp=None):
    return {"type": "parallel",
            "mixer": {"left": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "mask": {"keep_first": keep_first, "size": window},
                               "rot": {"base": base, "dims": rot_dims, "scaling": scaling}, "scale": scale, "vdim": dim},
                      "left_scale": left_scale, "right": {"dim": r_dim, "gate_cap": gate_cap, "heads": r_heads, "vdim": r_vdim},
                      "right_scale": right_scale},
            "mlp": mlp}


def delta_layer(heads=4, kv_heads=2, dim=8, vdim=16, conv=3, mlp=None):
    return {"type": "channel_delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}, "mlp": mlp}


def moe(experts=4, top=2, ff=16):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def make_config(layers, vocab=96, width=48, eps=1e-5, residual_mult=0.5):
    return {"architecture": "Kulanex", "layers": layers, "norm": {"eps": eps}, "residual_mult": residual_mult, "vocab": vocab, "width": width}


def greedy(cfg, w, prompt, n_new):
    """Greedy continuation, recomputing the whole sequence for every new token."""
    toks, out = list(prompt), []
    for _ in range(n_new):
        nxt = int(forward(cfg, w, toks)[-1].argmax())
        out.append(nxt)
        toks.append(nxt)
    return out


def write_model(folder, cfg, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw little-endian data) -> folder."""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
    header, blobs, at = {}, [], 0
    for k, t in w.items():
        t = t.contiguous()
        raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
        header[k] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    return folder
