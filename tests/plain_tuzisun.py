"""A plain, slow statement of the Tuzisun decoder, one function per mechanism, in float64 on the CPU.

It shares no code with the engine: every function takes plain tensors and the numbers of its own
section of config.json and walks the tokens of ONE sequence one after the other.  `forward` returns the
logits of every position and the sum of the streams after every layer.

Notation: T tokens, W the model width, h [T, W] a sub-layer's input.  Linear weights are [out, in].
"""
from __future__ import annotations

import math

import torch

F = torch.float64


def lin(w, h, b=None):
    y = h @ w.to(F).t()
    return y if b is None else y + b.to(F)


def dyn_tanh(x, w, b, alpha):
    return torch.tanh(alpha.to(F) * x) * w.to(F) + b.to(F)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def short_conv(x, w, b=None):
    """x [T, C]; w [C, taps], the last column multiplies the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), x], 0)
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y = y + pad[j:j + T] * w[:, j].to(F)
    return y if b is None else y + b.to(F)


def rotate_pairs(x, dims, base, first_position=0):
    """x [T, heads, dim]; neighbours (2i, 2i+1) of the first `dims` features turn by position * base^(-2i/dims)."""
    T = x.shape[0]
    out = x.clone()
    pos = torch.arange(first_position, first_position + T, dtype=F)
    for i in range(dims // 2):
        a = pos * (float(base) ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - v * s
        out[:, :, 2 * i + 1] = v * c + u * s
    return out


def window_attention(h, p, m, eps):
    """p: tensors of the mixer (q, q.b, k, k.b, v, v.b, q.norm, k.norm, o, o.b); m: its sizes."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = lin(p["q"], h, p["q.b"]).view(T, H, D)
    k = lin(p["k"], h, p["k.b"]).view(T, G, D)
    v = lin(p["v"], h, p["v.b"]).view(T, G, Dv)
    q = unit_rms(q, eps) * p["q.norm"].to(F)
    k = unit_rms(k, eps) * p["k.norm"].to(F)
    q = rotate_pairs(q, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_pairs(k, m["rot"]["dims"], m["rot"]["base"])
    out = torch.zeros(T, H, Dv, dtype=F)
    window = m["mask"]["size"]
    for t in range(T):
        lo = max(0, t - window + 1)
        for hd in range(H):
            g = hd // (H // G)
            s = (k[lo:t + 1, g] @ q[t, hd]) * m["scale"]
            w = torch.softmax(s, 0)
            out[t, hd] = w @ v[lo:t + 1, g]
    return lin(p["o"], out.reshape(T, H * Dv), p["o.b"])


def state_space(h, p, m, eps):
    """Selective state space with a scalar decay per head (p: in, conv, conv.b, dt_bias, A_log, D, norm, o)."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    y = lin(p["in"], h)
    z, xbc, dt = y[:, :inner], y[:, inner:2 * inner + 2 * G * N], y[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, p["conv"], p["conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + p["dt_bias"].to(F))
    A = torch.exp(p["A_log"].to(F))
    S = torch.zeros(H, N, P, dtype=F)
    out = torch.zeros(T, H, P, dtype=F)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = torch.exp(-A[hd] * dt[t, hd]) * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            out[t, hd] = S[hd].t() @ C[t, g] + p["D"].to(F)[hd] * x[t, hd]
    y = out.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * p["norm"].to(F)
    return lin(p["o"], y)


def parallel_mixer(h, p, m, eps):
    left = window_attention(h, {k[5:]: v for k, v in p.items() if k.startswith("left.")}, m["left"], eps)
    right = state_space(h, {k[6:]: v for k, v in p.items() if k.startswith("right.")}, m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def matrix_memory(h, p, m, eps):
    """Matrix memory with exponential input gate and a running maximum (p: q, k, v, g, o, norm, i, i.b, f, f.b)."""
    T = h.shape[0]
    H, D, P, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    q = (lin(p["q"], h) * D ** -0.5).view(T, H, D)
    k = lin(p["k"], h).view(T, H, D)
    v = lin(p["v"], h).view(T, H, P)
    ig = cap * torch.tanh(lin(p["i"], h, p["i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh(lin(p["f"], h, p["f.b"]) / cap))
    S = torch.zeros(H, D, P, dtype=F)
    n = torch.zeros(H, D, dtype=F)
    mx = torch.zeros(H, dtype=F)
    out = torch.zeros(T, H, P, dtype=F)
    for t in range(T):
        for hd in range(H):
            new = torch.maximum(fg[t, hd] + mx[hd], ig[t, hd])
            keep, put = torch.exp(fg[t, hd] + mx[hd] - new), torch.exp(ig[t, hd] - new)
            S[hd] = keep * S[hd] + put * torch.outer(k[t, hd], v[t, hd])
            n[hd] = keep * n[hd] + put * k[t, hd]
            mx[hd] = new
            den = torch.maximum((n[hd] @ q[t, hd]).abs(), torch.exp(-new)) + 1e-6
            out[t, hd] = (S[hd].t() @ q[t, hd]) / den
    o = unit_rms(out, eps).reshape(T, H * P) * p["norm"].to(F)
    return lin(p["o"], o * torch.sigmoid(lin(p["g"], h)))


def channel_delta(h, p, m, eps):
    """Delta rule with one decay per head and key channel (p: q, q.conv, k, k.conv, v, v.conv, b, A_log, norm,
    a1, a2, dt_bias, g1, g2, o)."""
    T = h.shape[0]
    H, G, D, P = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(lin(p["q"], h), p["q.conv"])).view(T, G, D)
    k = silu(short_conv(lin(p["k"], h), p["k.conv"])).view(T, G, D)
    v = silu(short_conv(lin(p["v"], h), p["v.conv"])).view(T, H, P)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin(p["b"], h))
    A = torch.exp(p["A_log"].to(F))
    step = softplus(lin(p["a2"], lin(p["a1"], h)) + p["dt_bias"].to(F)).view(T, H, D)
    decay = torch.exp(-A[None, :, None] * step)
    S = torch.zeros(H, D, P, dtype=F)
    out = torch.zeros(T, H, P, dtype=F)
    for t in range(T):
        for hd in range(H):
            g = hd // (H // G)
            S[hd] = decay[t, hd][:, None] * S[hd]
            u = beta[t, hd] * (v[t, hd] - S[hd].t() @ k[t, g])
            S[hd] = S[hd] + torch.outer(k[t, g], u)
            out[t, hd] = S[hd].t() @ q[t, g]
    o = unit_rms(out, eps) * p["norm"].to(F)
    gate = torch.sigmoid(lin(p["g2"], lin(p["g1"], h))).view(T, H, P)
    return lin(p["o"], (o * gate).reshape(T, H * P))


MIXERS = {"parallel": parallel_mixer, "mlstm": matrix_memory, "channel_delta": channel_delta}


def dense_ff(h, p, m):
    L = float(m["limit"])
    g = torch.clamp(lin(p["gate"], h), max=L)
    u = torch.clamp(lin(p["up"], h), -L, L)
    return lin(p["down"], g * torch.sigmoid(1.702 * g) * (u + 1))


def routed_ff(h, p, m):
    T = h.shape[0]
    r = m["router"]
    E, top = r["experts"], r["top"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    s = torch.softmax(lin(p["router"], h), -1)
    out = torch.zeros(T, p["e0.down"].shape[0], dtype=F)
    per = E // groups["count"]
    for t in range(T):
        best = s[t].view(groups["count"], per).max(-1).values
        kept = torch.topk(best, groups["keep"]).indices.tolist()
        allowed = [e for e in range(E) if e // per in kept]
        chosen = sorted(allowed, key=lambda e: (-float(s[t, e]), e))[:top]
        for e in chosen:
            x = h[t:t + 1]
            y = lin(p[f"e{e}.down"], silu(lin(p[f"e{e}.gate"], x)) * lin(p[f"e{e}.up"], x))
            out[t] += s[t, e] * y[0]
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(config, weights, tokens):
    """(logits [T, vocab], [sum of the streams after each layer]) for one sequence from its first token."""
    eps = float(config["norm"]["eps"])
    S = int(config.get("streams", 1))
    x = weights["embed"].to(F)[torch.as_tensor(tokens, dtype=torch.long)]
    streams = [x.clone() for _ in range(S)]
    after = []
    for i, layer in enumerate(config["layers"]):
        w = sub(weights, f"l{i}.")
        subs = [(1, lambda h: MIXERS[layer["type"]](h, sub(w, "mix."), layer["mixer"], eps))]
        if layer.get("mlp") is not None:
            ff = dense_ff if layer["mlp"]["kind"] == "dense" else routed_ff
            subs.append((2, lambda h, ff=ff: ff(h, sub(w, "mlp."), layer["mlp"])))
        for n, fn in subs:
            a, o, mix = w[f"hc{n}.in"].to(F), w[f"hc{n}.out"].to(F), w[f"hc{n}.mix"].to(F)
            u = sum(a[s] * streams[s] for s in range(S))
            y = fn(dyn_tanh(u, w[f"norm{n}"], w[f"norm{n}.b"], w[f"norm{n}.alpha"]))
            streams = [sum(mix[s, t] * streams[s] for s in range(S)) + o[t] * y for t in range(S)]
        after.append(sum(streams))
    x = sum(streams)
    h = dyn_tanh(x, weights["final.norm"], weights["final.norm.b"], weights["final.norm.alpha"])
    return h @ weights["embed"].to(F).t(), after


def read_model_dir(folder):
    """(config.json as a dict, {name: tensor}) of a model folder; a reader of its own: 8 bytes of length, a JSON
    header name -> (dtype, shape, data_offsets), then the data."""
    import json
    import struct
    from pathlib import Path
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    raw = (folder / "model.safetensors").read_bytes()
    n = struct.unpack("<Q", raw[:8])[0]
    header = json.loads(raw[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
    weights = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        t = torch.frombuffer(bytearray(raw[8 + n + lo:8 + n + hi]), dtype=kinds[info["dtype"]])
        weights[name] = t.reshape(info["shape"]).clone()
    return config, weights
