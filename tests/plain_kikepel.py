"""Plain, slow implementation of the Kikepel decoder, whole sequences, no cache.

The oracle of the Kikepel tests.  It shares no code with the product path: it
reads config.json and model.safetensors itself, works on the CPU in float64 (or
float32), materialises every key and value, and has one function per mechanism.

The design in this file's notation (x_t: the residual stream at position t):

  layer     x <- x + LN_1(mixer(x));  x <- x + LN_2(ff(x))      (ff may be absent)
            LN(y) = (y - mean y) / sqrt(var y + eps) * w          (no bias)
  mixer     cq = RMS(W_dq x; w_dq, eps); q = W_uq cq
            c  = RMS(W_dkv x; w_dkv, eps); k_h = W_uk[h] c; v_h = W_uv[h] c
            s_tj = scale * <q_t,h , k_j,h>  for  0 <= t - j < window
            p = exp(s) / (sum_j exp(s_tj) [+ exp(sink_h)]);  out = W_o concat_h(sum_j p_tj v_j,h)
  dense ff  W_d (relu(W_g x + b_g) * (W_u x + b_u)) + b_d
  experts   z = W_r x; s = sigmoid(z); the `top` largest s pick experts e with weight s_e;
            ff(x) = sum_e E_e(s_e x);  E(y): g = min(W_g y, L), u = clamp(W_u y, -L, L),
            W_d (g * sigmoid(1.702 g) * (u + 1))
  output    LN_final(x) -> W_head * logit_scale -> cap * tanh(. / cap)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_ST_DTYPES = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "I32": torch.int32}


def read_safetensors(path, dtype=torch.float64) -> dict:
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        t = torch.frombuffer(bytearray(raw[base + lo:base + hi]), dtype=dt).reshape(meta["shape"])
        out[name] = t.to(dtype) if dt.is_floating_point else t
    return out


def read_model_dir(model_dir, dtype=torch.float64):
    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    return cfg, read_safetensors(Path(model_dir) / "model.safetensors", dtype)


# --------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------

def layer_norm(y, weight, eps):
    mean = y.mean(dim=-1, keepdim=True)
    dev = y - mean
    var = (dev * dev).mean(dim=-1, keepdim=True)
    return dev / torch.sqrt(var + eps) * weight


def rms_norm(y, weight, eps):
    return y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps) * weight


def window_mask(T, window):
    """[T, T] bool: query t sees key j iff 0 <= t - j < window."""
    t = torch.arange(T).view(T, 1)
    j = torch.arange(T).view(1, T)
    return (t - j >= 0) & (t - j < window)


def softmax_with_sink(scores, mask, sink=None):
    """scores [H, T, T]; sink [H] or None: one more term exp(sink_h) in the denominator only."""
    s = scores.masked_fill(~mask, -math.inf)
    m = s.max(dim=-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.view(-1, 1, 1))
    e = torch.exp(s - m)
    denom = e.sum(dim=-1, keepdim=True)
    if sink is not None:
        denom = denom + torch.exp(sink.view(-1, 1, 1) - m)
    return e / denom


def latent_attention(x, w, m, eps, with_sink):
    """x [T, width]; w: the mixer's tensors by their short names; m: the mixer's sizes."""
    T = x.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(x @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, D)
    c = rms_norm(x @ w["dkv"].T, w["dkv.norm"], eps)
    k = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, V)
    scores = torch.einsum("thd,jhd->htj", q, k) * m["scale"]
    p = softmax_with_sink(scores, window_mask(T, m["mask"]["size"]), w["sink"] if with_sink else None)
    out = torch.einsum("htj,jhv->thv", p, v).reshape(T, H * V)
    return out @ w["o"].T


def dense_ff(x, w):
    g = torch.relu(x @ w["gate"].T + w["gate.b"])
    u = x @ w["up"].T + w["up.b"]
    return (g * u) @ w["down"].T + w["down.b"]


def expert(y, w, e, limit):
    g = torch.clamp(y @ w[f"e{e}.gate"].T, max=limit)
    u = torch.clamp(y @ w[f"e{e}.up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[f"e{e}.down"].T


def route(x, router, top):
    """(experts [T, top], weights [T, top]): the largest sigmoid scores, not renormalised."""
    s = torch.sigmoid(x @ router.T)
    val, idx = torch.topk(s, top, dim=-1)
    return idx, val


def moe_ff(x, w, mlp):
    top, limit = mlp["router"]["top"], mlp["expert"]["limit"]
    idx, val = route(x, w["router"], top)
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for j in range(top):
            out[t] += expert(val[t, j] * x[t], w, int(idx[t, j]), limit)
    return out


def feed_forward(x, w, mlp):
    return dense_ff(x, w) if mlp["kind"] == "dense" else moe_ff(x, w, mlp)


def sub(weights, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x, weights, i, spec, eps):
    w = sub(weights, f"l{i}.")
    mix = latent_attention(x, sub(w, "mix."), spec["mixer"], eps, with_sink=spec["type"] == "latent_attention")
    x = x + layer_norm(mix, w["norm1"], eps)
    if spec.get("mlp") is not None:
        x = x + layer_norm(feed_forward(x, sub(w, "mlp."), spec["mlp"]), w["norm2"], eps)
    return x


def output(x, weights, cfg):
    h = layer_norm(x, weights["final.norm"], cfg["norm"]["eps"])
    z = h @ weights["head"].T * cfg["logit_scale"]
    cap = cfg["logit_softcap"]
    return cap * torch.tanh(z / cap)


def forward(cfg, weights, tokens, streams=None):
    """Logits [T, vocab] of a whole sequence.  `streams`, a list, receives x after every layer."""
    x = weights["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    eps = cfg["norm"]["eps"]
    for i, spec in enumerate(cfg["layers"]):
        x = layer(x, weights, i, spec, eps)
        if streams is not None:
            streams.append(x.clone())
    return output(x, weights, cfg)
