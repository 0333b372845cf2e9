"""The Kikepel decoder in the engine against the plain implementation (tests/plain_kikepel.py).

Small configurations of their own (three, which differ in every size, in the order and kinds of layers, in
windows, routing and constants), seeded random weights with edits where random numbers would hide a fault:
sharp attention (a large `scale`) so that one key more or less in a window moves the logits, large sinks,
a router with wide gaps.  Each mechanism alone; then whole prompts, token-by-token decoding, portions down
to two tokens, mixed batches with pages used again, and greedy generation through the engine's entry point.
Where a test claims to be sensitive to a fault (a window that is one key off, a sink left out), it first
shows that the plain implementation WITH that fault differs from the right one by far more than the tolerance.
"""
import copy
import functools
import math

import numpy as np
import pytest
import torch

import helpers as H
import plain_kikepel as P

DEV = "cuda:0"


def mixer(heads, dim, vdim, q_rank, kv_rank, window, scale=None):
    return dict(heads=heads, dim=dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, mask=dict(size=window),
                scale=dim ** -0.5 if scale is None else scale)


def moe(ff, experts, top, limit):
    return dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, top=top))


def dense(ff):
    return dict(kind="dense", ff=ff)


def layer(typ, mix, mlp):
    return dict(type=typ, mixer=mix, mlp=mlp)


# U: ranks that are no multiple of 16, a window shorter than a page and one that spans pages, top 2 of 4, a layer
# without a feed-forward.  V: twelve heads on the latent, window 1 (a token sees itself only), top = all experts
# and top 1, a window longer than most prompts.  W: latent rows of 128 numbers and pages of 64 positions, the size
# class of the tcgen05 and TMA attention kernels.
CONFIGS = {
    "U": dict(architecture="Kikepel", vocab=160, width=64, norm=dict(eps=1e-5), logit_scale=1.5, logit_softcap=9.0,
              layers=[layer("latent_attention", mixer(4, 16, 24, 32, 40, 7), dense(96)),
                      layer("latent_attention_2", mixer(3, 32, 16, 24, 32, 20), moe(48, 4, 2, 0.5)),
                      layer("latent_attention", mixer(2, 24, 8, 20, 24, 11), None)]),
    "V": dict(architecture="Kikepel", vocab=211, width=96, norm=dict(eps=3e-6), logit_scale=0.7, logit_softcap=30.0,
              layers=[layer("latent_attention_2", mixer(12, 16, 16, 48, 64, 33), moe(40, 6, 1, 2.0)),
                      layer("latent_attention", mixer(5, 48, 40, 40, 112, 100), moe(64, 3, 3, 1.0)),
                      layer("latent_attention", mixer(2, 16, 32, 16, 16, 1), dense(72)),
                      layer("latent_attention_2", mixer(20, 16, 8, 32, 48, 150), dense(40))]),
    "W": dict(architecture="Kikepel", vocab=301, width=128, norm=dict(eps=1e-6), logit_scale=2.5, logit_softcap=12.0,
              layers=[layer("latent_attention", mixer(8, 32, 48, 64, 128, 200), moe(64, 8, 2, 1.5)),
                      layer("latent_attention_2", mixer(4, 64, 64, 96, 128, 70), dense(160))]),
}
# X: the smallest and the largest sizes the kernels take side by side: one head of 8 numbers, a cached row of 256, a
# window longer than any prompt, an expert width that is no multiple of 8, a vocabulary and a width that are no powers of two
CONFIGS["X"] = dict(architecture="Kikepel", vocab=97, width=72, norm=dict(eps=2e-5), logit_scale=1.0, logit_softcap=20.0,
                    layers=[layer("latent_attention", mixer(1, 8, 8, 8, 256, 300), moe(20, 5, 2, 3.0)),
                            layer("latent_attention_2", mixer(3, 8, 40, 56, 8, 5, scale=0.9), dense(24))])
PAGE = {"U": 8, "V": 16, "W": 64, "X": 4}
SEED = {"U": 11, "V": 12, "W": 13, "X": 14}
TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def sharpened(cfg, factor):
    """The same model with every attention scale multiplied: near one-hot attention weights."""
    cfg = copy.deepcopy(cfg)
    for l in cfg["layers"]:
        l["mixer"]["scale"] *= factor
    return cfg


def with_window(cfg, delta):
    cfg = copy.deepcopy(cfg)
    for l in cfg["layers"]:
        l["mixer"]["mask"]["size"] = max(1, l["mixer"]["mask"]["size"] + delta)
    return cfg


@functools.lru_cache(maxsize=None)
def model_dir(which, store="bfloat16", sharp=1.0):
    """A folder with the configuration and seeded weights, edited so that no test rests on a close call
    between two experts, and with sinks spread over [-1, 3].
    float32: the routers are widened (times 12).  bfloat16, where rounding of the stream could still turn a
    near tie: the first E coordinates of the stream are kept exact and carry the routing: the layers' norm
    weights are zero there, so these coordinates hold the token's embedding for good, the embedding puts E
    distinct multiples of 1/8 there (in an order that depends on the token), and router row e reads
    coordinate e with weight 4 beside a small random rest.  The experts' logits then lie 0.5 apart, in
    [-1.25, 1.25], so that the weights (the sigmoid scores) differ from token to token."""
    from vllm_lite_b200.weights import write_model_dir
    from vllm_lite_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = sharpened(CONFIGS[which], sharp)
    d = H.tmp_root() / f"kikepel_{which}_{store}_{sharp}"
    write_model_dir(d, cfg, SEED[which], std=0.08, dtype=torch.float32 if store == "float32" else torch.bfloat16)
    f = SafetensorsFile(d / "model.safetensors")
    tensors = {n: f.read(n).clone() for n in f.names()}
    f.close()
    experts = [l["mlp"]["router"]["experts"] for l in cfg["layers"] if l["mlp"] and l["mlp"]["kind"] == "moe"]
    emax = max(experts)
    for name, t in tensors.items():
        if name.endswith(".mix.sink"):
            tensors[name] = torch.linspace(-1.0, 3.0, t.numel()).to(t.dtype)
        if name.endswith(".mlp.router") and store == "float32":
            tensors[name] = (t.float() * 12.0).to(t.dtype)
        if store != "float32":
            if name.endswith(".mlp.router"):
                r = t.float() * 0.1
                r[:, :emax] = 0.0
                r[torch.arange(r.shape[0]), torch.arange(r.shape[0])] = 4.0
                tensors[name] = r.to(t.dtype)
            if name.endswith(".norm1") or name.endswith(".norm2"):
                t[:emax] = 0.0
            if name == "embed":
                tok, c = torch.arange(t.shape[0]).view(-1, 1), torch.arange(emax).view(1, -1)
                t[:, :emax] = ((((tok + c) % emax).float() - (emax - 1) / 2) * 0.125).to(t.dtype)
    write_safetensors(d / "model.safetensors", tensors, metadata={"format": "pt"})
    return d


def store_of(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@functools.lru_cache(maxsize=None)
def plain_model(which, store, sharp=1.0):
    return P.read_model_dir(model_dir(which, store, sharp))


_logits = {}


def plain_logits(which, tokens, dtype, sharp=1.0, cfg_edit=None):
    key = (which, store_of(dtype), sharp, tuple(tokens), cfg_edit)
    if key not in _logits:
        cfg, w = plain_model(which, store_of(dtype), sharp)
        if cfg_edit is not None:
            cfg = cfg_edit[1](cfg)
        _logits[key] = P.forward(cfg, w, list(tokens)).float()
    return _logits[key]


def tokens_for(which, length, seed):
    rng = np.random.default_rng(7000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[which]["vocab"], size=length)]


def make_runner(which, dtype, num_pages, sharp=1.0, page_size=None, **kw):
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    _, plan, weights = load_model_dir(model_dir(which, store_of(dtype), sharp), dtype, DEV)
    return ModelRunner(plan, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV,
                       page_size=page_size or PAGE[which], num_pages=num_pages, max_requests=8, max_context=1024, **kw)


def assert_rows(rows, which, requests, dtype, what, sharp=1.0):
    """Every compared row within the tolerance (as a fraction of the row's largest logit)."""
    assert rows, "nothing was compared"
    bad, worst = [], 0.0
    for (rid, pos), row in rows.items():
        ref = plain_logits(which, requests[rid], dtype, sharp)[pos]
        err = float((row - ref).abs().max()) / max(float(ref.abs().max()), 1e-12)
        if err > TOL[dtype]:
            bad.append((rid, pos, err))
        else:
            worst = max(worst, err)
    assert not bad, f"{what} {which}/{dtype}: {len(bad)} of {len(rows)} rows differ, e.g. {bad[:4]}"
    key = ("kikepel " + what, which, dtype)
    H.WORST[key] = max(H.WORST.get(key, 0.0), worst)


def pages_for(which, tokens):
    return -(-tokens // PAGE[which])


# ----------------------------------------------------------------------------------------------
# without a GPU: configuration, plan, cache layout, and the plain implementation's own behaviour
# ----------------------------------------------------------------------------------------------

def test_config_reads_every_size_and_constant():
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import declare_model
    cfg, plan = plan_from_config_json(CONFIGS["U"])
    assert cfg.vocab_size == 160 and cfg.hidden_size == 64 and cfg.eps == 1e-5 and cfg.logit_scale == 1.5
    assert [l.mixer.window for l in cfg.layers] == [7, 20, 11]
    assert plan.layers[0].mixer.sink and not plan.layers[1].mixer.sink and plan.layers[2].ffn is None
    assert plan.layers[1].ffn.top == 2 and plan.layers[1].ffn.limit == 0.5 and plan.layers[1].ffn.scale_input
    assert plan.head.softcap == 9.0 and plan.head.scale == 1.5
    names = declare_model(plan)
    assert names["embed"].shape == (160, 64) and names["head"].shape == (160, 64) and names["final.norm"].shape == (64,)
    assert names["l0.mix.uv"].shape == (4 * 24, 40) and names["l0.mix.sink"].shape == (4,) and "l1.mix.sink" not in names
    assert names["l0.mlp.gate.b"].shape == (96,) and names["l1.mlp.e3.down"].shape == (64, 48)
    assert names["l1.mlp.router"].shape == (4, 64) and "l2.norm2" not in names and "l2.norm1" in names


def test_config_errors_name_the_field():
    from vllm_lite_b200.config import InvalidField, MissingField, plan_from_config_json
    bad = copy.deepcopy(CONFIGS["U"])
    del bad["layers"][1]["mixer"]["kv_rank"]
    with pytest.raises(MissingField, match=r"layers\[1\]\.mixer\.kv_rank"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["U"])
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(InvalidField, match=r"layers\[0\]\.type"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["U"])
    bad["layers"][1]["mlp"]["router"]["top"] = 5
    with pytest.raises(InvalidField, match="top"):
        plan_from_config_json(bad)


def test_latent_layers_share_pools_by_width_and_window():
    from vllm_lite_b200.cache import CacheManager, PagedLatent
    from vllm_lite_b200.cache.manager import CacheLayout
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import cache_needs
    cfg = copy.deepcopy(CONFIGS["U"])
    cfg["layers"].append(copy.deepcopy(cfg["layers"][0]))             # a fourth layer equal to the first
    _, plan = plan_from_config_json(cfg)
    needs = cache_needs(plan)
    assert needs[0] == PagedLatent(48, 7) and needs[1] == PagedLatent(32, 20)       # 40 -> rows of 48
    layout = CacheLayout.from_needs(needs, [None] * 4)
    assert layout.paged_members == [[0, 3], [1], [2]]
    mgr = CacheManager(layout, page_size=8, num_pages=6, max_requests=2)
    mgr.admit("a")
    mgr.append("a", 40)
    mgr.release_behind_window("a")
    held = [sum(p >= 0 for p in t) for t in mgr.requests["a"].block_tables]
    assert held == [1, 3, 2]           # windows 7, 20, 11 behind position 40: first read 34, 21, 30
    mgr.check_invariants()


def test_cache_sized_from_memory_for_latent_groups():
    """The arithmetic of `kv_blocks=None` on a plan of latent layers and experts: groups are capped by what their
    window lets a request hold, and a latent page costs one plane of its row width."""
    from vllm_lite_b200.cache.manager import CacheLayout
    from vllm_lite_b200.cache.sizing import activation_reserve, page_bytes, pages_from_memory
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import cache_needs
    _, plan = plan_from_config_json(CONFIGS["V"])
    layout = CacheLayout.from_needs(cache_needs(plan), [None] * 4)
    assert page_bytes(layout, 16, 2) == [16 * 64 * 2, 16 * 112 * 2, 16 * 16 * 2, 16 * 48 * 2]
    reserve = activation_reserve(plan, 512, 4, 1024, 2)
    assert reserve > 0
    pages = pages_from_memory(layout, 16, 2, 8 << 30, 0.9, reserve, 4, 1024, 512)
    # windows 33, 100, 1, 150 and steps of up to 512 tokens: a request holds at most ceil((window + 512) / 16) + 1 pages
    assert pages == [4 * (-(-(w + 512) // 16) + 1) + 1 for w in (33, 100, 1, 150)]


def test_plain_softmax_sink_and_window():
    s = torch.tensor([[[0.3, -1.0, 2.0], [0.1, 0.2, 0.3], [1.0, 1.0, 1.0]]], dtype=torch.float64)
    mask = P.window_mask(3, 2)
    assert mask.tolist() == [[True, False, False], [True, True, False], [False, True, True]]
    p = P.softmax_with_sink(s, mask)
    assert torch.allclose(p.sum(-1), torch.ones(1, 3, dtype=torch.float64))
    ps = P.softmax_with_sink(s, mask, torch.tensor([0.5], dtype=torch.float64))
    z = math.exp(1.0) + math.exp(1.0) + math.exp(0.5)
    assert abs(float(ps[0, 2, 1]) - math.exp(1.0) / z) < 1e-12 and float(ps[0, 2, 0]) == 0.0
    far = P.softmax_with_sink(s, mask, torch.tensor([-80.0], dtype=torch.float64))
    assert torch.allclose(far, p)


def test_plain_layer_norm_and_routing():
    y = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    out = P.layer_norm(y, torch.full((4,), 2.0, dtype=torch.float64), 0.0)
    assert abs(float(out.mean())) < 1e-12 and abs(float((out / 2).pow(2).mean()) - 1.0) < 1e-12
    x = torch.eye(3, dtype=torch.float64)
    router = torch.tensor([[1.0, 0.0, -1.0], [0.5, 2.0, 0.0]], dtype=torch.float64)
    idx, val = P.route(x, router, 1)
    assert idx.view(-1).tolist() == [0, 1, 1] and abs(float(val[0, 0]) - 1 / (1 + math.exp(-1.0))) < 1e-12


# ----------------------------------------------------------------------------------------------
# each mechanism alone, against one function of the plain implementation
# ----------------------------------------------------------------------------------------------

def ops():
    from vllm_lite_b200.csrc import ops as o
    return o


def rand(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, dtype, what):
    tol = 2e-5 if dtype == torch.float32 else 2.5e-2
    err = float((got.double().cpu() - want.double().cpu()).abs().max()) / max(float(want.abs().max()), 1e-12)
    assert err <= tol, f"{what} ({dtype}): {err:.3e}"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H_", [24, 100, 1000])
def test_layer_norm_kernels(dtype, H_):
    y, w = rand((9, H_), 1, dtype, 3.0) + 1.5, rand((H_,), 2) + 1.0
    x = rand((9, H_), 3)
    want = x.double() + P.layer_norm(y.double(), w.double(), 1e-5)
    x_new, cast = x.clone(), torch.empty((9, H_), dtype=dtype, device=DEV)
    ops().layernorm_add(y, w, 1e-5, x_new, cast)
    close(x_new, want, torch.float32 if dtype == torch.float32 else dtype, "layernorm_add")
    assert torch.equal(cast, x_new.to(dtype))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    out = torch.empty((3, H_), dtype=dtype, device=DEV)
    ops().layernorm_rows(x, rows, w, 1e-5, out)
    close(out, P.layer_norm(x.double()[rows.long()], w.double(), 1e-5), dtype, "layernorm_rows")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("q_rank,kv_rank,width", [(24, 40, 48), (96, 128, 128), (7, 5, 16)])
def test_latent_norms_and_cache_write(dtype, q_rank, kv_rank, width):
    T, page, pages = 6, 4, 5
    proj = rand((T, q_rank + kv_rank + 3), 4, dtype, 2.0)
    wq, wkv = rand((q_rank,), 5) + 1.0, rand((kv_rank,), 6) + 1.0
    cache = torch.full((pages, 1, page, width), 9.0, dtype=dtype, device=DEV)
    slots = torch.tensor([17, 3, -1, 0, 19, 8], dtype=torch.int32, device=DEV)
    cq = torch.empty((T, q_rank), dtype=dtype, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().latent_norm_write(proj, q_rank, kv_rank, wq, wkv, 1e-6, cq, slots, cache, err)
    p = proj.double()
    close(cq, P.rms_norm(p[:, :q_rank], wq.double(), 1e-6), dtype, "query latent")
    c = P.rms_norm(p[:, q_rank:q_rank + kv_rank], wkv.double(), 1e-6)
    flat = cache.view(pages * page, width)
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            close(flat[s, :kv_rank], c[t], dtype, "cached latent")
            assert float(flat[s, kv_rank:].abs().sum()) == 0.0          # the padding of a row is zero
    untouched = [s for s in range(pages * page) if s not in slots.tolist()]
    assert bool((flat[untouched] == 9.0).all()) and int(err.item()) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,heads,N,K", [(1, 3, 48, 16), (13, 5, 20, 33), (150, 2, 130, 64), (70, 12, 16, 128)])
def test_products_per_head(dtype, T, heads, N, K, monkeypatch):
    """K = 33 takes the FFMA kernel in both dtypes; the other bfloat16 cases the tensor cores, and once more the FFMA
    kernel (the switch that keeps bfloat16 products off the tensor cores): both against the same sums."""
    a, w = rand((T, heads * K), 7, dtype), rand((heads, N, K), 8, dtype)
    out = torch.empty((T, heads * N), dtype=dtype, device=DEV)
    ops().gemm_heads(a, w, out)
    want = torch.einsum("thk,hnk->thn", a.double().view(T, heads, K), w.double()).reshape(T, heads * N)
    close(out, want, dtype, "per-head product")
    monkeypatch.setenv("VLLM_LITE_B200_BATCHED_SIMT", "1")
    again = torch.empty_like(out)
    ops().gemm_heads(a, w, again)
    close(again, want, dtype, "per-head product, FFMA kernel")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_activations_and_capped_logits(dtype):
    gu = rand((5, 2 * 37), 9, dtype, 2.0)
    g, u = gu.double()[:, :37], gu.double()[:, 37:]
    out = torch.empty((5, 37), dtype=dtype, device=DEV)
    close(ops().gated_act(gu, out, "relu"), torch.relu(g) * u, dtype, "relu gate")
    lim = 0.75
    gc, uc = torch.clamp(g, max=lim), torch.clamp(u, -lim, lim)
    close(ops().gated_act(gu, out, "capped_swish", 0, 1.702, lim, 1.0), gc * torch.sigmoid(1.702 * gc) * (uc + 1.0), dtype,
          "capped swish gate")
    close(ops().gated_act(gu, out, "silu"), g * torch.sigmoid(g) * u, dtype, "silu gate")
    bias = rand((74,), 12)
    close(ops().gated_act(gu, out, "relu", bias=bias), torch.relu(g + bias.double()[:37]) * (u + bias.double()[37:]), dtype,
          "relu gate with the projections' biases")
    z = rand((4, 50), 10, torch.float32, 10.0)
    want = 6.0 * torch.tanh(z.double() * 1.7 / 6.0)
    close(ops().scale_softcap(z.clone(), 1.7, 6.0), want, torch.float32, "capped logits")
    close(ops().scale_softcap(z.clone(), 1.7, None), z.double() * 1.7, torch.float32, "scaled logits")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,ff", [(1, 4, 1, 24), (9, 5, 2, 40), (150, 8, 3, 17), (33, 3, 3, 64), (600, 4, 2, 136),
                                        (700, 8, 3, 40)])
def test_routed_experts_part(dtype, T, E, top, ff):
    """The whole feed-forward part (router, sort, grouped products, activation, sum) against the plain loop
    over tokens; router weights are wide apart so that both sides choose the same experts."""
    from vllm_lite_b200.parts.base import BuildContext, Workspace
    from vllm_lite_b200.parts.experts import RoutedExperts
    from vllm_lite_b200.parts.spec import RoutedExpertsSpec
    from types import SimpleNamespace
    Hd = 48
    spec = RoutedExpertsSpec(Hd, ff, E, top, limit=0.8)
    names = RoutedExperts.declare(spec)
    w = {n: rand(d.shape, 20 + i, dtype, 0.3 if n == "router" else 0.15) for i, (n, d) in enumerate(sorted(names.items()))}
    part = RoutedExperts(spec, w, BuildContext(torch.device(DEV), dtype))
    h = rand((T, Hd), 11, dtype)
    step = SimpleNamespace(workspace=Workspace(torch.device(DEV)), tag="", err=None)
    got = part(h, step)
    wd = {k: v.double().cpu() for k, v in w.items()}
    mlp = dict(kind="moe", expert=dict(ff=ff, limit=0.8), router=dict(experts=E, top=top))
    want = P.moe_ff(h.double().cpu(), wd, mlp)
    idx, val = P.route(h.double().cpu(), wd["router"], top)
    ids = step.workspace.get("moe.ids", (T, top), torch.int32).cpu()
    assert torch.equal(ids.long(), idx), "the router chose other experts"
    close(got, want, dtype, "routed experts")
    # the same row alone: the same bits where both steps run on the same kernels (a row's arithmetic does not
    # depend on its place among the sorted rows); steps of many rows take the tcgen05 products, whose sums
    # are rounded alike but not added in the same order
    alone = part(h[T // 2:T // 2 + 1].contiguous(), step).clone()
    again = part(h, step)[T // 2]
    if T * top < 1024 or dtype == torch.float32:
        assert torch.equal(alone[0], again)
    else:
        close(alone[0], again.double(), dtype, "a row alone against the row in a long step")


def reference_attention(q, c, pos, window, scale, sinks):
    """q [H, R] of one token at position `pos`, c [n, R] its request's latents: out [H, R]."""
    lo = max(0, pos - window + 1) if window else 0
    keys = c[lo:pos + 1].double()
    s = (q.double() @ keys.T) * scale
    m = s.max(dim=-1, keepdim=True).values
    if sinks is not None:
        m = torch.maximum(m, sinks.double().view(-1, 1))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sinks is not None:
        den = den + torch.exp(sinks.double().view(-1, 1) - m)
    return (e / den) @ keys


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("with_sinks", [False, True])
@pytest.mark.parametrize("rank,heads,page,window", [(48, 3, 8, 7), (128, 8, 64, 100), (64, 12, 16, 0), (16, 20, 4, 33)])
def test_attention_over_latent_pages(dtype, with_sinks, rank, heads, page, window):
    """Every attention kernel that the dispatcher may pick for a latent group (one shared head whose keys are its
    values) on prompt portions, single tokens and both together, with and without sinks, pages in shuffled order."""
    from vllm_lite_b200.parts import attention_dispatch
    from vllm_lite_b200.parts.base import CallCache, GroupView, Workspace, QUERY_TILE
    from vllm_lite_b200.parts.latent_attention import HeadLayout
    from types import SimpleNamespace
    lens = [150, 1, 37, 90]                       # cached tokens of four requests after the step
    news = [150, 1, 1, 70]                        # tokens each brings in this step: a whole prompt, a first token, a decoded one, a portion
    n_pages = sum(-(-n // page) for n in lens) + 3
    order = torch.randperm(n_pages, generator=torch.Generator().manual_seed(5)).tolist()
    cache = torch.zeros((n_pages, 1, page, rank), dtype=dtype, device=DEV)
    max_blocks = max(-(-n // page) for n in lens)
    table = torch.full((len(lens), max_blocks), -1, dtype=torch.int32)
    latents = []
    for b, n in enumerate(lens):
        c = rand((n, rank), 30 + b, dtype)
        latents.append(c)
        for blk in range(-(-n // page)):
            pg = order.pop()
            table[b, blk] = pg
            rows = c[blk * page:(blk + 1) * page]
            cache[pg, 0, :rows.shape[0]] = rows
    pos, req, tiles, singles = [], [], [], []
    for b, (n, k) in enumerate(zip(lens, news)):
        t0 = len(pos)
        pos += list(range(n - k, n))
        req += [b] * k
        if k > 1:
            tiles += [(b, t0 + lo, min(QUERY_TILE, k - lo), n - k + lo) for lo in range(0, k, QUERY_TILE)]
        else:
            singles.append(t0)
    T = len(pos)
    q = rand((T, heads * rank), 40, dtype, 0.5)
    sinks = torch.linspace(-1.0, 2.5, heads, device=DEV) if with_sinks else None
    dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    scale = 0.2
    step = SimpleNamespace(req_index=dev(req), positions=dev(pos), err=torch.zeros(1, dtype=torch.int32, device=DEV),
                           workspace=Workspace(torch.device(DEV)), tag="", max_query_len=max(news),
                           query_tiles=dev(tiles).view(-1, 4), single_tokens=dev(singles), single_context=max(lens))
    group = GroupView(page_size=page, block_table=table.to(DEV), slots=None, max_context=max(lens))
    cc = CallCache(group=0, k=cache, v=cache)
    out = torch.full((T, heads * rank), 7.0, dtype=dtype, device=DEV)
    attention_dispatch.run(q, out, cc, group, step, HeadLayout(heads, 1, rank, window or None), scale, sinks=sinks)
    assert int(step.err.item()) == 0
    for t in range(T):
        want = reference_attention(q[t].view(heads, rank).cpu(), latents[req[t]].cpu(), pos[t], window, scale,
                                   None if sinks is None else sinks.cpu())
        close(out[t].view(heads, rank), want, dtype, f"attention of token {t} (request {req[t]}, position {pos[t]})")
    # a decode-only step: every request brings one token
    pos1 = [n - 1 for n in lens]
    q1 = rand((4, heads * rank), 41, dtype, 0.5)
    step1 = SimpleNamespace(req_index=dev([0, 1, 2, 3]), positions=dev(pos1), err=step.err, workspace=step.workspace,
                            tag="d.", max_query_len=1, query_tiles=None, single_tokens=None, single_context=0)
    out1 = torch.empty((4, heads * rank), dtype=dtype, device=DEV)
    attention_dispatch.run(q1, out1, cc, group, step1, HeadLayout(heads, 1, rank, window or None), scale, sinks=sinks)
    for t in range(4):
        want = reference_attention(q1[t].view(heads, rank).cpu(), latents[t].cpu(), pos1[t], window, scale,
                                   None if sinks is None else sinks.cpu())
        close(out1[t].view(heads, rank), want, dtype, f"decode attention of request {t}")
    assert int(step.err.item()) == 0


@pytest.mark.gpu
def test_a_sink_and_a_far_key_show_in_the_attention():
    """One key far back whose score stands out among hundreds carries the output; a large sink takes it away."""
    from vllm_lite_b200.csrc import ops as o
    rank, heads, page, n = 32, 2, 8, 400
    c = rand((n, rank), 50, torch.float32, 0.1)
    c[13] = 0.0
    c[13, 5] = 4.0                                # the far key
    q = torch.zeros((1, heads * rank), device=DEV)
    q[0, 5] = 6.0
    q[0, rank + 5] = 6.0
    cache = c.view(n // page, 1, page, rank).contiguous()
    table = torch.arange(n // page, dtype=torch.int32, device=DEV).view(1, -1)
    zero = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    o.paged_attention(q, out, cache, cache, table, zero, pos, heads, 1, rank, 1.0, None, err)
    assert float(out[0, 5]) > 3.9                                      # all of the weight on key 13
    o.paged_attention(q, out, cache, cache, table, zero, pos, heads, 1, rank, 1.0, n - 14, err)
    assert float(out[0, 5]) < 0.5                                      # the window ends one key short of it
    o.paged_attention(q, out, cache, cache, table, zero, pos, heads, 1, rank, 1.0, n - 13, err)
    assert float(out[0, 5]) > 3.9                                      # ... and just reaches it
    sinks = torch.tensor([24.0 + math.log(3.0), -50.0], device=DEV)   # head 0: a sink three times the key's weight
    o.paged_attention(q, out, cache, cache, table, zero, pos, heads, 1, rank, 1.0, None, err, sinks=sinks)
    assert abs(float(out[0, 5]) - 1.0) < 0.02 and float(out[0, rank + 5]) > 3.9
    assert int(err.item()) == 0


# ----------------------------------------------------------------------------------------------
# the model in the engine
# ----------------------------------------------------------------------------------------------

CASES = [(w, d) for w in ("U", "V", "W", "X") for d in ("float32", "bfloat16")]
LENGTHS = {"U": [1, 6, 8, 9, 40, 75], "V": [2, 17, 33, 120, 170], "W": [65, 230, 300], "X": [1, 3, 50, 131]}


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_whole_prompts(which, dtype):
    runner = make_runner(which, dtype, num_pages=pages_for(which, 320))
    for n, length in enumerate(LENGTHS[which]):
        toks = tokens_for(which, length, n)
        rows = H.run_schedule(runner, [([("r", toks, list(range(length)))], ["r"])])
        assert_rows(rows, which, {"r": toks}, dtype, "whole")
    assert set(runner.cache.free_pages()) == {pages_for(which, 320)}


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["U", "V", "W"])
def test_residual_stream_after_every_layer(which):
    """float32: the stream after each layer against the plain implementation's."""
    toks = tokens_for(which, 50, 3)
    runner = make_runner(which, "float32", num_pages=pages_for(which, 64))
    batch = runner.prepare([__import__("vllm_lite_b200.engine", fromlist=["StepEntry"]).StepEntry("r", toks, [49])])
    from vllm_lite_b200.parts.base import Residual
    x = runner.workspace.get("residual", (50, runner.plan.hidden_size), torch.float32)
    runner.model.embedding(batch, x)
    res = Residual(x)
    cfg, w = plain_model(which, "float32")
    streams = []
    P.forward(cfg, w, toks, streams)
    for i, (layer_, cache) in enumerate(zip(runner.model.layers, runner.storage.call_caches)):
        layer_(res, batch, cache)
        close(res.x, streams[i], torch.float32, f"stream after layer {i}")
    runner.check_device_errors()


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_prompt_then_token_by_token(which, dtype):
    """Most of a request in one step, then single tokens until every window has passed over decoded tokens."""
    length, tail = {"U": (90, 40), "V": (260, 170), "W": (300, 90), "X": (60, 20)}[which]
    toks = tokens_for(which, length, 7)
    runner = make_runner(which, dtype, num_pages=pages_for(which, length + PAGE[which]))
    head = length - tail
    schedule = [([("r", toks[:head], [head - 1])], [])]
    schedule += [([("r", [toks[p]], [0])], []) for p in range(head, length)]
    rows = H.run_schedule(runner, schedule)
    assert len(rows) == tail + 1
    assert_rows(rows, which, {"r": toks}, dtype, "decode")


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_first_tokens_one_by_one(which, dtype):
    toks = tokens_for(which, 12, 3)
    runner = make_runner(which, dtype, num_pages=4)
    rows = H.run_schedule(runner, [([("r", [t], [0])], []) for t in toks])
    assert_rows(rows, which, {"r": toks}, dtype, "first tokens")


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_portions_of_changing_size(which, dtype):
    length = {"U": 120, "V": 200, "W": 330, "X": 90}[which]
    toks = tokens_for(which, length, 11)
    runner = make_runner(which, dtype, num_pages=pages_for(which, length + PAGE[which]))
    sizes = [7, 2, 13, 3, 2, 16, 5, 2, 31, 8, 2, 17, 2, 2, 3] if which != "W" else [70, 2, 129, 3, 64, 2, 40, 2, 2, 16]
    schedule, p, k = [], 0, 0
    while p < length:
        n = min(sizes[k % len(sizes)], length - p)
        k += 1
        schedule.append(([("r", toks[p:p + n], list(range(n)))], []))
        p += n
    rows = H.run_schedule(runner, schedule)
    assert len(rows) == length
    assert_rows(rows, which, {"r": toks}, dtype, "portions")


def mixed_schedule(which, scale=1):
    lens = {k: n * scale for k, n in {"a": 50, "b": 37, "c": 64, "d": 21, "e": 45, "f": 30}.items()}
    reqs = {k: tokens_for(which, n, 20 + i) for i, (k, n) in enumerate(lens.items())}
    fed = {k: 0 for k in reqs}

    def take(k, n, want="all"):
        n = n * scale if n > 4 else n
        t = reqs[k][fed[k]:fed[k] + n]
        fed[k] += len(t)
        return (k, t, list(range(len(t))) if want == "all" else ([len(t) - 1] if want == "last" else []))
    S = [([take("a", 20), take("b", 30)], []),
         ([take("a", 30, "last"), take("c", 9), take("b", 1)], []),
         ([take("c", 2), take("d", 21), take("b", 1)], ["a"]),
         ([take("c", 23, "none"), take("e", 13), take("b", 1)], ["d"]),
         ([take("c", 1), take("e", 1), take("f", 2), take("b", 2)], []),
         ([take("c", 1), take("e", 7), take("f", 11), take("b", 1)], [])]
    S.append(([(k, reqs[k][fed[k]:], list(range(len(reqs[k]) - fed[k]))) for k in ("b", "c", "e", "f") if fed[k] < lens[k]],
              ["b", "c", "e", "f"]))
    return reqs, S


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_mixed_batches_with_pages_used_again(which, dtype):
    """Up to four live requests, portions beside single tokens; so few pages that freed ones are taken again,
    by other requests and at other places.  Every row against the request alone in the plain implementation."""
    reqs, schedule = mixed_schedule(which, 3 if which == "W" else 1)
    ps = PAGE[which]
    live_peak, live = 0, {}
    for entries, end in schedule:
        for k, t, _ in entries:
            live[k] = live.get(k, 0) + len(t)
        live_peak = max(live_peak, sum(-(-n // ps) for n in live.values()))
        for k in end:
            live.pop(k)
    assert live_peak < sum(-(-len(t) // ps) for t in reqs.values())
    runner = make_runner(which, dtype, num_pages=live_peak)
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, reqs, dtype, "mixed")
    assert set(runner.cache.free_pages()) == {live_peak}
    # the same requests once more through the same runner: every page and slot is used a second time
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, reqs, dtype, "mixed, second round")


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["U", "V"])
def test_cuts_and_batches_agree_bitwise_in_float32(which):
    toks = tokens_for(which, 60, 5)
    other = tokens_for(which, 23, 6)
    runner = make_runner(which, "float32", num_pages=pages_for(which, 192))
    whole = H.run_schedule(runner, [([("w", toks, list(range(60)))], ["w"])])
    cut = H.run_schedule(runner, [
        ([("o", other[:20], [])], []),
        ([("x", toks[:17], list(range(17))), ("o", other[20:21], [0])], []),
        ([("o", other[21:22], [0]), ("x", toks[17:19], [0, 1])], []),
        ([("x", toks[19:60], list(range(41)))], ["x", "o"])])
    for p in range(60):
        assert torch.equal(whole[("w", p)], cut[("x", p)]), f"position {p} differs between cuts"


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["U", "V"])
def test_window_edges_and_sinks_show_in_the_logits(which):
    """Sharp attention (scales times 24, float32).  First the test's own sensitivity: the plain implementation
    with every window one key longer or shorter, or without the sinks, is far outside the tolerance at many
    positions.  Then the engine matches the right one, in a whole prompt, in portions and decoded alone."""
    sharp = 24.0
    length = 140
    toks = tokens_for(which, length, 17)
    ref = plain_logits(which, toks, "float32", sharp)

    def moved(edit_name, edit):
        other = plain_logits(which, toks, "float32", sharp, (edit_name, edit))
        return ((other - ref).abs().amax(1) / ref.abs().amax(1) > 50 * TOL["float32"]).float().mean().item()
    assert moved("longer", lambda c: with_window(c, 1)) > 0.5
    assert moved("shorter", lambda c: with_window(c, -1)) > 0.5

    def without_sinks(c):
        c = copy.deepcopy(c)
        for l in c["layers"]:
            l["type"] = "latent_attention_2"
        return c
    assert moved("no sinks", without_sinks) > 0.5
    runner = make_runner(which, "float32", num_pages=pages_for(which, 160), sharp=sharp)
    rows = H.run_schedule(runner, [([("r", toks, list(range(length)))], ["r"])])
    assert_rows(rows, which, {"r": toks}, "float32", "sharp, whole", sharp)
    schedule = [([("r", toks[:9], list(range(9)))], []), ([("r", toks[9:40], list(range(31)))], []),
                ([("r", toks[40:42], [0, 1])], []), ([("r", toks[42:100], list(range(58)))], [])]
    schedule += [([("r", [toks[p]], [0])], []) for p in range(100, length)]
    rows = H.run_schedule(runner, schedule)
    assert len(rows) == length
    assert_rows(rows, which, {"r": toks}, "float32", "sharp, portions and decode", sharp)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    which, length = "V", 400
    toks = tokens_for(which, length, 31)
    runner = make_runner(which, dtype, num_pages=pages_for(which, length + 16))
    schedule = [([("r", toks[:4], [3])], [])] + [([("r", [toks[p]], [0])], []) for p in range(4, length)]
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks}, dtype, "long decode")
    # windowed groups gave back what lies behind their windows: 33, 100, 1, 150 positions of 400
    held = [sum(p >= 0 for p in t) for t in runner.cache.requests["r"].block_tables]
    assert max(held) <= pages_for(which, 150) + 1 and min(held) <= 1


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["U", "V"])
def test_greedy_generation_through_the_engine(which):
    """LLMEngine with its scheduler (prompts cut into portions, requests batched): greedy tokens equal the plain
    implementation's, float32."""
    from vllm_lite_b200 import LLMEngine
    prompts = [tokens_for(which, n, 50 + i) for i, n in enumerate([5, 17, 33, 64])]
    eng = LLMEngine(str(model_dir(which, "float32")), dtype="float32", kv_blocks=64, block_size=PAGE[which],
                    max_batch_size=4, max_num_batched_tokens=48, prefill_chunk_size=13, max_model_len=256)
    outs = eng.generate(prompts, max_tokens=24)
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o:
            row = plain_logits(which, toks, "float32")[-1]
            assert int(row.argmax()) == t or float(row.max() - row[t]) < 1e-4 * float(row.abs().max())
            toks.append(t)
    st = eng.stats()
    assert set(st["free_pages"]) == {64} and st["finished"] == len(prompts)


@pytest.mark.gpu
def test_greedy_generation_bfloat16_follows_the_plain_logits():
    from vllm_lite_b200 import LLMEngine
    which = "W"
    prompts = [tokens_for(which, n, 60 + i) for i, n in enumerate([9, 140])]
    # kv_blocks=None: the cache is sized from the GPU's free memory (capped by what 4 requests of 512 tokens can hold)
    eng = LLMEngine(str(model_dir(which, "bfloat16")), dtype="bfloat16", kv_blocks=None, block_size=64, max_batch_size=4,
                    max_model_len=512)
    outs = eng.generate(prompts, max_tokens=12)
    far = 0
    for p, o in zip(prompts, outs):
        toks = list(p)
        for t in o:
            row = plain_logits(which, toks, "bfloat16")[-1]
            far += float(row.max() - row[t]) > 2 * TOL["bfloat16"] * float(row.abs().max())
            toks.append(t)
    assert far <= 1


@pytest.mark.gpu
def test_command_line_and_replay_program(tmp_path):
    """`python -m vllm_lite_b200 init` writes a Kikepel folder from its config.json, the command line generates from it
    (greedy, float32: the plain implementation's tokens), and bin/trace_run replays steps on it."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(CONFIGS["U"]))
    folder = tmp_path / "model"
    run = lambda *a, **k: subprocess.run([sys.executable, *a], capture_output=True, text=True, cwd=root, timeout=900, **k)
    made = run("-m", "vllm_lite_b200", "init", "--config", str(cfg), "--out", str(folder), "--seed", "5", "--std", "0.08")
    assert made.returncode == 0, made.stderr[-2000:]
    prompt = tokens_for("U", 14, 77)
    out = run("-m", "vllm_lite_b200", "--model", str(folder), "--dtype", "float32", "--kv-blocks", "32", "--max-tokens", "6",
              "--prompt-ids", ",".join(map(str, prompt)), "--log-level", "warn")
    assert out.returncode == 0, out.stderr[-2000:]
    got = [int(t) for t in out.stdout.strip().split(",")]
    pc, pw = P.read_model_dir(folder)
    toks = list(prompt)
    for t in got:
        row = P.forward(pc, pw, toks)[-1]
        assert int(row.argmax()) == t or float(row.max() - row[t]) < 1e-4 * float(row.abs().max())
        toks.append(t)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": prompt[:9], "want": [8]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": prompt[9:], "want": [0, 4]}, {"id": "b", "tokens": [3, 1], "want": []}],
              "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": [4], "want": [0]}], "end": ["b"]}]
    outdir = tmp_path / "logits"
    rep = run(str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(outdir),
              "--max-tokens", "64", "--page-size", "8", input="".join(json.dumps(x) + "\n" for x in steps))
    assert rep.returncode == 0, rep.stderr[-2000:]
    assert [l for l in rep.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = P.forward(pc, pw, prompt).float()
    rows = np.fromfile(outdir / "1.f32", dtype="<f4").reshape(2, CONFIGS["U"]["vocab"])
    for row, pos in zip(rows, (9, 13)):
        assert float(np.abs(row - ref[pos].numpy()).max()) <= TOL["float32"] * float(ref[pos].abs().max())
    last = np.fromfile(outdir / "2.f32", dtype="<f4")
    refb = P.forward(pc, pw, [3, 1, 4]).float()[2].numpy()
    assert float(np.abs(last - refb).max()) <= TOL["float32"] * float(np.abs(refb).max())
