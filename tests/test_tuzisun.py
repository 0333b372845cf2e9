"""The Tuzisun decoder in the engine against the plain implementation (tests/plain_tuzisun.py).

Small configurations of their own that differ in every size, in the order and kinds of layers, in windows, taps,
groups and constants (also values that are 1: one stream, one group, a window of one page, a layer without a
feed-forward), seeded random weights with edits where random numbers would hide a fault (sharp attention so that one
key more or less in a window moves the logits; a router with wide gaps).  Each mechanism alone against one function
of the plain implementation, state carried across steps and slots; then whole prompts, the stream after every layer,
token-by-token decoding, portions down to two tokens, mixed batches with pages and slots used again, long decoding,
and greedy generation through the engine's entry point.
"""
import copy
import functools
import json

import numpy as np
import pytest
import torch

import helpers as H
import plain_tuzisun as P

DEV = "cuda:0"


def parallel(heads, kv, dim, vdim, window, rot, base, scale, r_heads, r_vdim, state, groups, conv, norm_groups, ls, rs):
    return dict(left=dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, mask=dict(size=window), rot=dict(dims=rot, base=base),
                          scale=scale),
                right=dict(heads=r_heads, vdim=r_vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups),
                left_scale=ls, right_scale=rs)


def mlstm(heads, dim, vdim, cap):
    return dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap)


def delta(heads, kv, dim, vdim, conv, decay_rank, gate_rank):
    return dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, conv=conv, decay_rank=decay_rank, gate_rank=gate_rank)


def dense(ff, limit):
    return dict(kind="dense", ff=ff, limit=limit)


def moe(ff, experts, top, count=None, keep=None):
    router = dict(experts=experts, top=top)
    if count is not None:
        router["groups"] = dict(count=count, keep=keep)
    return dict(kind="moe", expert=dict(ff=ff), router=router)


def layer(typ, mix, mlp):
    return dict(type=typ, mixer=mix, mlp=mlp)


# A: three streams; value heads wider than key heads (padded to 32 for the kernels), a partial rotation, a window shorter
#    than a page, three expert groups of which two are kept, a layer without a feed-forward, sizes that are no powers of two.
# B: ONE stream, one expert chosen, no expert groups, as many key heads as query heads, value heads narrower than key heads,
#    two taps, one norm part, a window that spans pages.
# C: four streams, pages of 64 positions, heads of 64 (the tensor-core attention's size class), a state of 128 rows (eight
#    lanes to a column), a window of 70 that crosses a page border, five taps.
CONFIGS = {
    "A": dict(architecture="Tuzisun", vocab=150, width=64, streams=3, norm=dict(eps=1e-5),
              layers=[layer("channel_delta", delta(4, 2, 16, 24, 4, 8, 12), dense(96, 0.7)),
                      layer("parallel", parallel(4, 2, 16, 24, 7, 8, 10000.0, 0.6, 3, 16, 24, 1, 3, 3, 0.7, 1.2), moe(40, 6, 2, 3, 2)),
                      layer("mlstm", mlstm(2, 24, 40, 8.0), None)]),
    "B": dict(architecture="Tuzisun", vocab=211, width=96, streams=1, norm=dict(eps=3e-6),
              layers=[layer("mlstm", mlstm(3, 16, 16, 15.0), moe(48, 4, 1)),
                      layer("parallel", parallel(6, 6, 32, 16, 33, 32, 500000.0, 0.4, 4, 8, 16, 4, 2, 1, 1.0, 0.5), dense(72, 2.0)),
                      layer("channel_delta", delta(2, 2, 40, 8, 2, 5, 7), dense(40, 1.5)),
                      layer("parallel", parallel(2, 1, 48, 48, 100, 16, 777.0, 0.3, 2, 24, 8, 2, 4, 2, 0.5, 0.5), moe(24, 8, 3, 2, 1))]),
    "C": dict(architecture="Tuzisun", vocab=301, width=128, streams=4, norm=dict(eps=1e-6),
              layers=[layer("parallel", parallel(8, 1, 64, 64, 70, 64, 300000.0, 0.25, 4, 32, 128, 2, 5, 4, 0.75, 0.95), dense(160, 1.0)),
                      layer("channel_delta", delta(4, 1, 128, 32, 3, 16, 16), moe(64, 8, 2, 4, 2)),
                      layer("mlstm", mlstm(4, 64, 96, 10.0), dense(136, 1.25))]),
}
# D: sizes that are multiples of two at best: key heads of 20 and value heads of 12 numbers (padded to 32 for the kernels),
#    three rotated pairs, a state of 10 rows, ONE tap (a convolution without memory), every expert chosen, two streams.
# E: no attention anywhere (the engine then keeps no pages at all), and F: nothing but attention layers.
CONFIGS["D"] = dict(architecture="Tuzisun", vocab=97, width=72, streams=2, norm=dict(eps=2e-5),
                    layers=[layer("parallel", parallel(6, 3, 20, 12, 5, 6, 50.0, 0.9, 2, 6, 10, 2, 1, 2, 1.1, 0.3), moe(20, 5, 5)),
                            layer("mlstm", mlstm(1, 10, 14, 3.0), dense(52, 0.5)),
                            layer("channel_delta", delta(3, 3, 12, 10, 1, 3, 2), None)])
CONFIGS["E"] = dict(architecture="Tuzisun", vocab=120, width=48, streams=2, norm=dict(eps=1e-6),
                    layers=[layer("mlstm", mlstm(2, 16, 16, 10.0), dense(64, 1.0)),
                            layer("channel_delta", delta(2, 1, 16, 24, 3, 4, 4), moe(16, 4, 2, 2, 1))])
CONFIGS["F"] = dict(architecture="Tuzisun", vocab=120, width=48, streams=5, norm=dict(eps=1e-6),
                    layers=[layer("parallel", parallel(2, 2, 16, 16, 1, 16, 10000.0, 0.25, 2, 8, 16, 1, 4, 1, 1.0, 1.0), None),
                            layer("parallel", parallel(4, 1, 32, 32, 300, 8, 123.0, 0.2, 1, 16, 32, 1, 2, 2, 0.0, 1.0), dense(40, 3.0))])
PAGE = {"A": 8, "B": 16, "C": 64, "D": 4, "E": 8, "F": 16}
SEED = {"A": 21, "B": 22, "C": 23, "D": 24, "E": 25, "F": 26}
TOL = {"float32": 3e-5, "bfloat16": 4e-2}
# C (sums over 128 and more products, a matrix memory whose denominator cancels): the plain implementation run in
# float32 already differs from itself in float64 by 4e-5 of the largest logit, three times what A shows
# (bfloat16 in the same proportion: 6e-2 of the largest logit was seen on C, 4.8e-2 on A, 2.6e-2 on B)
TOL_OF = {("C", "float32"): 1.5e-4, ("A", "bfloat16"): 6e-2, ("C", "bfloat16"): 1e-1}


def tol(which, dtype):
    return TOL_OF.get((which, dtype), TOL[dtype])
CASES = [(w, d) for w in ("A", "B", "C", "D", "E", "F") for d in ("float32", "bfloat16")]


def edited(cfg, scale=1.0, window=0):
    """The same model with every attention scale multiplied (near one-hot weights) and every window moved."""
    cfg = copy.deepcopy(cfg)
    for l in cfg["layers"]:
        if l["type"] == "parallel":
            l["mixer"]["left"]["scale"] *= scale
            l["mixer"]["left"]["mask"]["size"] = max(1, l["mixer"]["left"]["mask"]["size"] + window)
    return cfg


@functools.lru_cache(maxsize=None)
def model_dir(which, store="bfloat16", sharp=1.0):
    """A folder with the configuration and seeded weights; the routers are widened so that no test rests on a close
    call between two experts."""
    from vllm_lite_b200.weights import write_model_dir
    from vllm_lite_b200.weights.safetensors_io import SafetensorsFile, write_safetensors
    cfg = edited(CONFIGS[which], sharp)
    d = H.tmp_root() / f"tuzisun_{which}_{store}_{sharp}"
    write_model_dir(d, cfg, SEED[which], std=0.08, dtype=torch.float32 if store == "float32" else torch.bfloat16)
    f = SafetensorsFile(d / "model.safetensors")
    tensors = {n: f.read(n).clone() for n in f.names()}
    f.close()
    for name, t in tensors.items():
        if name.endswith(".mlp.router"):
            tensors[name] = (t.float() * 15.0).to(t.dtype)
    write_safetensors(d / "model.safetensors", tensors, metadata={"format": "pt"})
    return d


def store_of(dtype):
    return "float32" if dtype == "float32" else "bfloat16"


@functools.lru_cache(maxsize=None)
def plain_model(which, store, sharp=1.0):
    return P.read_model_dir(model_dir(which, store, sharp))


_plain = {}


def plain_run(which, tokens, dtype, sharp=1.0, window=0):
    key = (which, store_of(dtype), sharp, window, tuple(tokens))
    if key not in _plain:
        cfg, w = plain_model(which, store_of(dtype), sharp)
        logits, after = P.forward(edited(cfg, 1.0, window), w, list(tokens))
        _plain[key] = (logits.float(), [a.float() for a in after])
    return _plain[key]


def tokens_for(which, length, seed):
    rng = np.random.default_rng(9000 + seed)
    return [int(t) for t in rng.integers(0, CONFIGS[which]["vocab"], size=length)]


def make_runner(which, dtype, num_pages, sharp=1.0, page_size=None, max_requests=4, **kw):
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    _, plan, weights = load_model_dir(model_dir(which, store_of(dtype), sharp), dtype, DEV)
    return ModelRunner(plan, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV,
                       page_size=page_size or PAGE[which], num_pages=num_pages, max_requests=max_requests, max_context=1024, **kw)


def assert_rows(rows, which, requests, dtype, what, sharp=1.0, loosen=1.0):
    assert rows, "nothing was compared"
    bad, worst = [], 0.0
    for (rid, pos), row in rows.items():
        ref = plain_run(which, requests[rid], dtype, sharp)[0][pos]
        err = float((row - ref).abs().max()) / max(float(ref.abs().max()), 1e-12)
        if err > loosen * tol(which, dtype):
            bad.append((rid, pos, err))
        else:
            worst = max(worst, err)
    # bfloat16: a head of the matrix memory whose k.q is near zero at a sequence's first tokens turns its (normed) output
    # round under rounding, and a row of logits with it; float32 shows none of this and is held to every row.  So in
    # bfloat16 a few rows may lie outside, as long as most lie well inside.
    allowed = 0 if dtype == "float32" else int(0.2 * len(rows))
    assert len(bad) <= allowed, f"{what} {which}/{dtype}: {len(bad)} of {len(rows)} rows differ, e.g. {bad[:4]}"
    key = ("tuzisun " + what, which, dtype)
    H.WORST[key] = max(H.WORST.get(key, 0.0), worst)


def pages_for(which, tokens):
    return -(-tokens // PAGE[which])


# ----------------------------------------------------------------------------------------------
# without a GPU: configuration, plan, cache layout, the plain implementation's own behaviour
# ----------------------------------------------------------------------------------------------

def test_config_reads_every_size_and_constant():
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import declare_model
    cfg, plan = plan_from_config_json(CONFIGS["A"])
    assert (cfg.vocab_size, cfg.hidden_size, cfg.streams, cfg.eps) == (150, 64, 3, 1e-5)
    d, p, m = (b.mixer for b in plan.layers)
    assert (d.num_heads, d.num_kv_heads, d.dim, d.vdim, d.conv, d.decay_rank, d.gate_rank) == (4, 2, 16, 24, 4, 8, 12)
    assert (p.left.window, p.left.scale, p.left.v_head_dim, p.left.position.dim, p.left.position.theta) == (7, 0.6, 24, 8, 10000.0)
    assert p.left.position.interleaved and p.left.bias and p.left.out_bias and (p.left_scale, p.right_scale) == (0.7, 1.2)
    assert (p.right.state, p.right.groups, p.right.conv, p.right.norm_groups) == (24, 1, 3, 3)
    assert m.gate_cap == 8.0 and plan.layers[2].ffn is None and plan.layers[0].ffn.limit == 0.7
    f = plan.layers[1].ffn
    assert (f.num_experts, f.top, f.groups, f.keep_groups, f.score, f.scale_input, f.renormalize) == (6, 2, 3, 2, "softmax", False, False)
    names = declare_model(plan)
    assert names["embed"].shape == (150, 64) and names["final.norm.alpha"].shape == () and "head" not in names
    assert names["l0.mix.a2"].shape == (64, 8) and names["l0.mix.q.conv"].shape == (32, 4) and names["l0.hc2.mix"].shape == (3, 3)
    assert names["l1.mix.left.o.b"].shape == (64,) and names["l1.mix.right.in"].shape == (2 * 48 + 2 * 24 + 3, 64)
    assert names["l1.mix.right.conv"].shape == (48 + 48, 3) and names["l2.mix.i.b"].shape == (2,)
    assert "l2.hc2.in" not in names and "l2.norm2" not in names and names["l1.mlp.e5.down"].shape == (64, 40)


def test_config_errors_name_the_field_and_ranks_come_from_shapes():
    from vllm_lite_b200.config import InvalidField, MissingField, plan_from_config_json
    bad = copy.deepcopy(CONFIGS["A"])
    del bad["layers"][1]["mixer"]["right"]["state"]
    with pytest.raises(MissingField, match=r"layers\[1\]\.mixer\.right\.state"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["A"])
    bad["layers"][2]["type"] = "something_else"
    with pytest.raises(InvalidField, match=r"layers\[2\]\.type"):
        plan_from_config_json(bad)
    bad = copy.deepcopy(CONFIGS["A"])
    bad["layers"][1]["mlp"]["router"]["groups"]["keep"] = 1           # one group of two experts cannot give top 2... it can; top 3 cannot
    bad["layers"][1]["mlp"]["router"]["top"] = 3
    with pytest.raises(InvalidField, match="router"):
        plan_from_config_json(bad)
    bare = copy.deepcopy(CONFIGS["A"])
    for key in ("decay_rank", "gate_rank"):
        del bare["layers"][0]["mixer"][key]
    with pytest.raises(MissingField, match="decay_rank"):
        plan_from_config_json(bare)
    _, plan = plan_from_config_json(bare, shapes={"l0.mix.a1": (5, 64), "l0.mix.g1": (9, 64)})
    assert (plan.layers[0].mixer.decay_rank, plan.layers[0].mixer.gate_rank) == (5, 9)


def test_a_layer_with_two_mixers_holds_pages_and_a_state_slot():
    from vllm_lite_b200.cache import CacheManager, FixedState, PagedKV, Several
    from vllm_lite_b200.cache.manager import CacheLayout
    from vllm_lite_b200.config import plan_from_config_json
    from vllm_lite_b200.parts.model import cache_needs
    _, plan = plan_from_config_json(CONFIGS["B"])
    needs = cache_needs(plan)
    assert isinstance(needs[0], FixedState) and isinstance(needs[1], Several) and isinstance(needs[2], FixedState)
    assert needs[1].parts[0] == PagedKV(6, 32, 33) and needs[3].parts[0] == PagedKV(1, 48, 100)
    layout = CacheLayout.from_needs(needs, [None] * 4)
    assert layout.paged_members == [[1], [3]] and len(layout.state_groups) == 4
    assert layout.call_place[1][0] == "several" and layout.call_place[1][1][0] == ("paged", 0, 0, True)
    mgr = CacheManager(layout, page_size=16, num_pages=9, max_requests=2)
    mgr.admit("a")
    mgr.append("a", 130)
    mgr.release_behind_window("a")
    assert [sum(p >= 0 for p in t) for t in mgr.requests["a"].block_tables] == [3, 8]     # first read 98 and 31: six pages and one given back
    mgr.check_invariants()


def test_plain_pieces_behave():
    x = torch.arange(12, dtype=torch.float64).view(6, 2) + 1
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=torch.float64)
    y = P.short_conv(x, w)
    assert torch.equal(y[:, 0], x[:, 0]) and y[:2, 1].tolist() == [0.0, 0.0] and torch.equal(y[2:, 1], x[:-2, 1])
    q = torch.randn(5, 2, 8, dtype=torch.float64)
    r = P.rotate_pairs(q, 4, 100.0)
    assert torch.allclose(r[0], q[0]) and torch.equal(r[:, :, 4:], q[:, :, 4:])
    assert torch.allclose((r[:, :, :4] ** 2).sum(-1), (q[:, :, :4] ** 2).sum(-1))
    # two experts per group, one group kept: the other group's larger second score does not count
    h = torch.eye(4, dtype=torch.float64)[:1]
    p = {"router": torch.tensor([[3.0, 0, 0, 0], [0.0, 0, 0, 0], [2.5, 0, 0, 0], [2.0, 0, 0, 0]])}
    for e in range(4):
        p[f"e{e}.gate"] = torch.full((2, 4), 1.0)
        p[f"e{e}.up"] = torch.full((2, 4), float(e + 1))
        p[f"e{e}.down"] = torch.ones(4, 2)
    s = torch.softmax(torch.tensor([3.0, 0.0, 2.5, 2.0], dtype=torch.float64), 0)
    out = P.routed_ff(h, p, dict(router=dict(experts=4, top=2, groups=dict(count=2, keep=1))))
    act = float(P.silu(torch.tensor(1.0, dtype=torch.float64)))
    assert abs(float(out[0, 0]) - 2 * act * (float(s[0]) * 1 + float(s[1]) * 2)) < 1e-12


# ----------------------------------------------------------------------------------------------
# each mechanism alone, against one function of the plain implementation
# ----------------------------------------------------------------------------------------------

def ops():
    from vllm_lite_b200.csrc import ops as o
    return o


def rand(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(DEV)


def close(got, want, dtype, what, tol=None):
    tol = tol or (2e-5 if dtype in (torch.float32, "float32") else 2.5e-2)
    err = float((got.double().cpu() - want.double().cpu()).abs().max()) / max(float(want.abs().max()), 1e-12)
    assert err <= tol, f"{what} ({dtype}): {err:.3e}"


def mini_step(lengths, slots):
    """A step's description for parts that keep a state: request b brings lengths[b] tokens and owns state row slots[b]."""
    from vllm_lite_b200.parts.base import StepBatch, Workspace
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lengths)]), dtype=torch.int32, device=DEV)
    T = int(sum(lengths))
    z = torch.zeros(T, dtype=torch.int32, device=DEV)
    return StepBatch(tokens=z, positions=z, req_index=z, cu_seqlens=cu, state_slots=torch.tensor(slots, dtype=torch.int32, device=DEV),
                     logit_rows=z[:0], groups=[], entries=[], err=torch.zeros(1, dtype=torch.int32, device=DEV),
                     workspace=Workspace(torch.device(DEV)), num_tokens=T, num_entries=len(lengths), max_query_len=max(lengths))


def build_part(spec, dtype, seed, registry="MIXERS"):
    """(part, its tensors as the plain implementation reads them) with seeded random weights."""
    from vllm_lite_b200.parts import registry as R
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.weights import random_tensors
    cls = getattr(R, registry).get(spec.kind)
    tensors = random_tensors(cls.declare(spec), seed, 0.15, 0.1, dtype=dtype)
    part = cls(spec, {k: v.to(DEV) for k, v in tensors.items()}, BuildContext(torch.device(DEV), dtype))
    return part, tensors


def run_recurrent(part, spec, h, cuts, dtype):
    """Two requests of unequal length fed in portions `cuts` (lists of per-step lengths), in swapped slots, one of
    the slots holding another request's leftovers first: the output of every token, per request."""
    from vllm_lite_b200.parts.base import CallCache
    need = type(part).cache_need(spec)
    state = torch.zeros((3,) + tuple(need.shape), dtype=torch.float32, device=DEV)
    state[2].normal_()                                                  # a used slot: handed out again after zeroing
    state[2].zero_()
    cache = CallCache(state=state)
    outs = [[], []]
    at = [0, 0]
    for lens in cuts:
        live = [b for b in (0, 1) if lens[b] > 0]
        step = mini_step([lens[b] for b in live], [2 - b for b in live])
        x = torch.cat([h[b][at[b]:at[b] + lens[b]] for b in live]).to(dtype).to(DEV).contiguous()
        y = part(x, step, cache).float()
        o = 0
        for b in live:
            outs[b].append(y[o:o + lens[b]].clone())
            o += lens[b]
            at[b] += lens[b]
    return [torch.cat(o) for o in outs]


RECURRENT = [
    ("state_space", dict(num_heads=3, vdim=16, state=24, groups=1, conv=3, norm_groups=3)),
    ("state_space", dict(num_heads=4, vdim=40, state=130, groups=2, conv=4, norm_groups=1)),
    ("matrix_memory", dict(num_heads=2, dim=24, vdim=40, gate_cap=8.0)),
    ("matrix_memory", dict(num_heads=3, dim=72, vdim=136, gate_cap=15.0)),
    ("delta_rule", dict(num_heads=4, num_kv_heads=2, dim=16, vdim=24, conv=4, decay_rank=8, gate_rank=12)),
    ("delta_rule", dict(num_heads=2, num_kv_heads=1, dim=136, vdim=8, conv=2, decay_rank=5, gate_rank=7)),
    # columns of more than 256 rows: sixteen rows a lane; of 512: the most the kernels take
    ("state_space", dict(num_heads=2, vdim=12, state=264, groups=2, conv=2, norm_groups=2)),
    ("matrix_memory", dict(num_heads=1, dim=300, vdim=20, gate_cap=10.0)),
    ("delta_rule", dict(num_heads=2, num_kv_heads=2, dim=512, vdim=24, conv=3, decay_rank=4, gate_rank=4)),
]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind,sizes", RECURRENT)
def test_recurrent_mixers_alone(dtype, kind, sizes):
    """One mixer, two requests: whole, in portions down to one token, and batched beside each other, against the
    plain function on each request alone."""
    from vllm_lite_b200.parts import spec as S
    W, eps = 48, 1e-5
    cls = {"state_space": S.StateSpaceSpec, "matrix_memory": S.MatrixMemorySpec, "delta_rule": S.DeltaRuleSpec}[kind]
    spec = cls(hidden_size=W, eps=eps, **sizes)
    part, tensors = build_part(spec, dtype, 5)
    fn = {"state_space": P.state_space, "matrix_memory": P.matrix_memory, "delta_rule": P.channel_delta}[kind]
    keys = {"state_space": {"num_heads": "heads"}, "matrix_memory": {"num_heads": "heads"},
            "delta_rule": {"num_heads": "heads", "num_kv_heads": "kv_heads"}}[kind]
    m = {keys.get(k, k): v for k, v in sizes.items()}
    n = [19, 11]
    h = [rand((n[b], W), 30 + b, dtype, 1.5).cpu() for b in (0, 1)]
    want = [fn(h[b].double(), tensors, m, eps) for b in (0, 1)]
    whole = run_recurrent(part, spec, h, [n], dtype)
    cut = run_recurrent(part, spec, h, [[7, 0], [1, 3], [2, 1], [9, 7]], dtype)
    for b in (0, 1):
        close(whole[b], want[b], dtype, f"{kind} whole")
        close(cut[b], want[b], dtype, f"{kind} in portions")
        if dtype == torch.float32:
            assert torch.equal(whole[b], cut[b]), "float32 results depend on how the tokens were cut"


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S_,H_", [(1, 24), (3, 100), (4, 256), (8, 40)])
def test_streams_and_tanh_norm(dtype, S_, H_):
    T = 7
    x = rand((T, H_), 1)
    y1, y2 = rand((T, H_), 2, dtype), rand((T, H_), 3, dtype)
    mix1, mix2 = rand((S_, S_), 4) + torch.eye(S_, device=DEV), rand((S_, S_), 5)
    out1, out2, in1, in2 = rand((S_,), 6), rand((S_,), 7), rand((S_,), 8), rand((S_,), 9)
    alpha, w, b = rand((1,), 10) + 1.0, rand((H_,), 11) + 1.0, rand((H_,), 12)
    streams = torch.empty((T, S_, H_), device=DEV)
    h1, h2 = torch.empty((T, H_), dtype=dtype, device=DEV), torch.empty((T, H_), dtype=dtype, device=DEV)
    total = torch.empty((T, H_), device=DEV)
    o = ops()
    o.hc_step(streams, single=x, in_w=in1, norm=(alpha, w, b), h=h1)                 # spread + read
    o.hc_step(streams, y=y1, mix=mix1, out_w=out1, in_w=in2, h=h2)                   # write back + plain read
    o.hc_step(streams, y=y2, mix=mix2, out_w=out2, total=total)                      # write back + sum
    xs = [x.double()] * S_
    u1 = sum(in1[s].double() * xs[s] for s in range(S_))
    close(h1, P.dyn_tanh(u1, w.double(), b.double(), alpha.double()), dtype, "spread and read")
    xs = [sum(mix1[s, t].double() * xs[s] for s in range(S_)) + out1[t].double() * y1.double() for t in range(S_)]
    close(h2, sum(in2[s].double() * xs[s] for s in range(S_)), dtype, "write back and read")
    xs = [sum(mix2[s, t].double() * xs[s] for s in range(S_)) + out2[t].double() * y2.double() for t in range(S_)]
    close(total, sum(xs), torch.float32, "sum of the streams")
    close(streams[:, S_ - 1], xs[S_ - 1], torch.float32, "last stream")
    rows = torch.tensor([5, 0], dtype=torch.int32, device=DEV)
    out = torch.empty((2, H_), dtype=dtype, device=DEV)
    o.dyt_rows(total, None, rows, alpha, w, b, out)
    close(out, P.dyn_tanh(total.double()[rows.long()], w.double(), b.double(), alpha.double()), dtype, "tanh norm on rows")


@pytest.mark.gpu
@pytest.mark.parametrize("taps,C", [(1, 5), (2, 40), (4, 33), (6, 128)])
def test_short_convolution_carries_its_inputs(taps, C):
    """A request fed in portions shorter than the taps, beside another one: every output equals the whole sequence's."""
    n = [13, 6]
    x = [rand((n[b], C + 3), 40 + b) for b in (0, 1)]
    w, bias = rand((C, taps), 42), rand((C,), 43)
    want = [P.silu(P.short_conv(x[b][:, 2:2 + C].double().cpu(), w.cpu(), bias.cpu())) for b in (0, 1)]
    state = torch.zeros((2, 7 + (taps - 1) * C), device=DEV)
    got, at = [[], []], [0, 0]
    for lens in ([1, 2], [1, 0], [2, 1], [1, 3], [8, 0]):
        live = [b for b in (0, 1) if lens[b]]
        step = mini_step([lens[b] for b in live], [1 - b for b in live])
        xin = torch.cat([x[b][at[b]:at[b] + lens[b]] for b in live]).contiguous()
        out = torch.empty((xin.shape[0], C), device=DEV)
        ops().short_conv(xin, 2, C, w, bias, state, 7, step.cu_seqlens, step.state_slots, out)
        o = 0
        for b in live:
            got[b].append(out[o:o + lens[b]].clone())
            o += lens[b]
            at[b] += lens[b]
    for b in (0, 1):
        close(torch.cat(got[b]), want[b], torch.float32, "short convolution")
    assert float(state[:, :7].abs().max()) == 0.0


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,count,keep,ff", [(6, 2, 3, 2, 40), (8, 3, 2, 1, 24), (4, 1, 1, 1, 17), (16, 4, 4, 2, 64), (12, 6, 6, 3, 8)])
def test_routed_experts_with_groups(dtype, E, top, count, keep, ff):
    from vllm_lite_b200.parts import spec as S
    W, T = 64, 37
    spec = S.RoutedExpertsSpec(W, ff, E, top, activation="silu", score="softmax", renormalize=False, scale_input=False,
                               groups=count, keep_groups=keep)
    part, tensors = build_part(spec, dtype, 8, "FEED_FORWARDS")
    tensors["router"] = (tensors["router"].float() * 40).to(dtype)             # wide gaps between the experts' scores
    part, _ = build_part(spec, dtype, 8, "FEED_FORWARDS")
    part.router.copy_(tensors["router"].to(part.router.dtype))
    h = rand((T, W), 9, dtype)
    got = part(h, mini_step([T], [0]))
    want = P.routed_ff(h.double().cpu(), tensors, dict(router=dict(experts=E, top=top, groups=dict(count=count, keep=keep))))
    close(got, want, dtype, "routed experts")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_group_that_is_not_kept_hides_its_experts(dtype):
    """Logits (3, 0, 2.5, 2) over two groups of two, one group kept, top 2: experts 0 and 1 are chosen although 2 and 3
    score higher than 1; scores are still taken over all four.  Experts answer with different constants, so a router
    that forgot the groups would be far off."""
    from vllm_lite_b200.parts import spec as S
    W, T, ff = 16, 5, 8
    spec = S.RoutedExpertsSpec(W, ff, 4, 2, activation="silu", score="softmax", renormalize=False, scale_input=False,
                               groups=2, keep_groups=1)
    part, tensors = build_part(spec, dtype, 3, "FEED_FORWARDS")
    router = torch.zeros(4, W)
    router[:, 0] = torch.tensor([3.0, 0.0, 2.5, 2.0])
    tensors["router"] = router.to(dtype)
    for e in range(4):
        tensors[f"e{e}.gate"] = torch.full((ff, W), 0.25).to(dtype)
        tensors[f"e{e}.up"] = torch.full((ff, W), 0.125 * (e + 1)).to(dtype)
        tensors[f"e{e}.down"] = torch.full((W, ff), 0.5).to(dtype)
    from vllm_lite_b200.parts.base import BuildContext
    from vllm_lite_b200.parts.registry import FEED_FORWARDS
    part = FEED_FORWARDS.get(spec.kind)(spec, {k: v.to(DEV) for k, v in tensors.items()}, BuildContext(torch.device(DEV), dtype))
    h = torch.zeros(T, W)
    h[:, 0] = torch.tensor([1.0, 1.0, -1.0, 0.5, 2.0])                   # token 2: the order turns round, the other group wins
    h[:, 1] = 0.5
    h = h.to(dtype).to(DEV)
    want = P.routed_ff(h.double().cpu(), tensors, dict(router=dict(experts=4, top=2, groups=dict(count=2, keep=1))))
    free = P.routed_ff(h.double().cpu(), tensors, dict(router=dict(experts=4, top=2)))
    assert float((free - want).abs().max()) > 0.05 * float(want.abs().max())
    close(part(h, mini_step([T], [0])), want, dtype, "grouped routing")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_feed_forward(dtype):
    from vllm_lite_b200.parts import spec as S
    spec = S.GatedMlpSpec(48, 72, activation="capped_swish", alpha=1.702, limit=0.4, up_shift=1.0, names=("gate", "up", "down"))
    part, tensors = build_part(spec, dtype, 12, "FEED_FORWARDS")
    h = rand((9, 48), 13, dtype, 3.0)
    want = P.dense_ff(h.double().cpu(), tensors, dict(limit=0.4))
    close(part(h, mini_step([9], [0])), want, dtype, "dense feed-forward")
    loose = P.dense_ff(h.double().cpu(), tensors, dict(limit=40.0))
    assert float((loose - want).abs().max()) > 1e-2 * float(want.abs().max())             # the limit matters here


# ----------------------------------------------------------------------------------------------
# the model in the engine
# ----------------------------------------------------------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_whole_prompts(which, dtype):
    reqs = {f"r{i}": tokens_for(which, n, i) for i, n in enumerate([1, 2, 37, 150])}
    runner = make_runner(which, dtype, num_pages=pages_for(which, 150) + 1)
    rows = {}
    for rid, toks in reqs.items():
        rows.update(H.run_schedule(runner, [([(rid, toks, list(range(len(toks))))], [rid])]))
    assert_rows(rows, which, reqs, dtype, "whole")


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E", "F"])
def test_stream_after_every_layer(which):
    from vllm_lite_b200.engine import StepEntry
    toks = tokens_for(which, 29, 5)
    runner = make_runner(which, "float32", num_pages=pages_for(which, 64))
    seen = []
    batch = runner.prepare([StepEntry("a", toks, [])])
    runner.model.forward(batch, runner.storage.call_caches, watch=lambda i, x: seen.append(x.clone().cpu()))
    runner.finish(batch)
    runner.check_device_errors()
    want = plain_run(which, toks, "float32")[1]
    assert len(seen) == len(want)
    for i, (a, b) in enumerate(zip(seen, want)):
        close(a, b, "float32", f"stream after layer {i}", tol=2e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_prompt_then_token_by_token(which, dtype):
    """Most of a prompt in one step, then single tokens (replayed from a graph), far enough for the windows to pass over
    decoded tokens; and a request fed one token at a time from its first."""
    toks, first = tokens_for(which, 140, 11), tokens_for(which, 12, 12)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 140) + 2)
    cut = 140 - 60
    schedule = [([("r", toks[:cut], [0, cut - 1])], [])] + [([("r", [toks[p]], [0])], []) for p in range(cut, 140)]
    schedule += [([("s", [first[p]], [0])], []) for p in range(12)]
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks, "s": first}, dtype, "decode")


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_portions_of_changing_size(which, dtype):
    toks = tokens_for(which, 171, 21)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 171) + 1)
    sizes, schedule, at = [2, 37, 3, 2, 64, 1, 5, 33, 2, 22], [], 0
    for n in sizes:
        schedule.append(([("r", toks[at:at + n], [0, n - 1] if n > 1 else [0])], []))
        at += n
    assert at == 171
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks}, dtype, "portions")


def mixed_schedule(which):
    """Up to three live requests in three state slots: portions beside single tokens, requests that pause, end and are
    replaced, so that pages and slots change hands."""
    reqs = {k: tokens_for(which, n, 60 + i) for i, (k, n) in enumerate([("a", 90), ("b", 41), ("c", 7), ("d", 66), ("e", 30)])}
    fed = {k: 0 for k in reqs}
    plan = [[("a", 30), ("b", 2)], [("a", 1), ("b", 17), ("c", 3)], [("a", 29), ("c", 1)], [("b", 1), ("c", 3)],
            [("a", 2), ("b", 21), ("d", 40)], [("a", 28), ("d", 1)], [("d", 2), ("e", 9)], [("d", 23), ("e", 1)], [("e", 20)]]
    schedule = []
    for step in plan:
        entries, end = [], []
        for k, n in step:
            lo = fed[k]
            entries.append((k, reqs[k][lo:lo + n], sorted({0, n - 1})))
            fed[k] += n
            if fed[k] == len(reqs[k]):
                end.append(k)
        schedule.append((entries, end))
    assert all(fed[k] == len(v) for k, v in reqs.items())
    return reqs, schedule


@pytest.mark.gpu
@pytest.mark.parametrize("which,dtype", CASES)
def test_mixed_batches_with_pages_and_slots_used_again(which, dtype):
    reqs, schedule = mixed_schedule(which)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 90) + pages_for(which, 66) + pages_for(which, 41) + 1, max_requests=3)
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, reqs, dtype, "mixed")
    assert runner.cache.slots.free_count == 3


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C", "D", "E", "F"])
def test_cuts_and_batches_agree_bitwise_in_float32(which):
    reqs, schedule = mixed_schedule(which)
    runner = make_runner(which, "float32", num_pages=4 * pages_for(which, 90), max_requests=3)
    mixed = H.run_schedule(runner, schedule)
    for rid, toks in reqs.items():
        alone = H.run_schedule(runner, [([(rid, toks, list(range(len(toks))))], [rid])])
        for (r, pos), row in mixed.items():
            if r == rid:
                assert torch.equal(row, alone[(r, pos)]), f"{rid} position {pos} depends on the batch or the cut"


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "B", "C"])
def test_window_edges_show_in_the_logits(which):
    """Sharp attention: a window that is one key too long or too short moves the logits by far more than the tolerance in
    the plain implementation, and the engine agrees with the right one, in prompts and in decoding."""
    sharp = 40.0
    toks = tokens_for(which, 150, 33)
    right = plain_run(which, toks, "float32", sharp)[0]
    for off in (-1, 1):
        wrong = plain_run(which, toks, "float32", sharp, window=off)[0]
        gap = float((wrong - right).abs().max()) / float(right.abs().max())
        assert gap > 100 * tol(which, "float32"), f"a window off by {off} would not show ({gap:.2e})"
    runner = make_runner(which, "float32", num_pages=pages_for(which, 150) + 1, sharp=sharp)
    schedule = [([("r", toks[:60], list(range(60)))], [])] + [([("r", [toks[p]], [0])], []) for p in range(60, 150)]
    # scores forty times as large carry forty times the rounding of q.k into the exponentials: three times the tolerance,
    # which the gap shown above still exceeds thirty times over
    assert_rows(H.run_schedule(runner, schedule), which, {"r": toks}, "float32", "window edges", sharp, loosen=3.0)


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["B", "C"])
def test_long_prompt_whole_against_portions(which):
    """A prompt of 2,300 tokens in one step (the products, the experts and the attention of many rows run on their
    tensor-core kernels for long steps, the convolution is cut among blocks, the scans walk thousands of tokens) against
    the same prompt in portions of a few hundred tokens (the kernels of short steps): bfloat16 both, so they agree to rounding;
    float32 bit for bit."""
    from vllm_lite_b200.engine import ModelRunner, load_model_dir
    n = 2300
    toks = tokens_for(which, n, 71)
    want = sorted(set(range(0, n, 97)) | set(range(n - 8, n)))
    for dtype in ("bfloat16", "float32"):
        _, plan, weights = load_model_dir(model_dir(which, store_of(dtype)), dtype, DEV)
        runner = ModelRunner(plan, weights, dtype=torch.bfloat16 if dtype == "bfloat16" else torch.float32, device=DEV,
                             page_size=PAGE[which], num_pages=pages_for(which, n) + 2, max_requests=2, max_context=4096)
        whole = H.run_schedule(runner, [([("w", toks, want)], ["w"])])
        cuts, schedule, at = [300, 411, 2, 600, 87, 900], [], 0
        for c in cuts:
            schedule.append(([("p", toks[at:at + c], [p - at for p in want if at <= p < at + c])], []))
            at += c
        assert at == n
        parts = H.run_schedule(runner, schedule)
        errs = []
        for p in want:
            a, b = whole[("w", p)], parts[("p", p)]
            if dtype == "float32":
                assert torch.equal(a, b), f"{which}: position {p} depends on the cut"
            errs.append(float((a - b).abs().max()) / max(float(b.abs().max()), 1e-12))
        if dtype == "bfloat16":
            errs.sort()
            assert errs[len(errs) // 2] <= tol(which, dtype) and errs[int(0.8 * len(errs))] <= 2 * tol(which, dtype), errs[-5:]
        del runner


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(dtype):
    which, length = "B", 420
    toks = tokens_for(which, length, 31)
    runner = make_runner(which, dtype, num_pages=pages_for(which, 140))
    schedule = [([("r", toks[:4], [3])], [])] + [([("r", [toks[p]], [0])], []) for p in range(4, length)]
    rows = H.run_schedule(runner, schedule)
    assert_rows(rows, which, {"r": toks}, dtype, "long decode")
    held = [sum(p >= 0 for p in t) for t in runner.cache.requests["r"].block_tables]
    assert held[0] <= pages_for(which, 33) + 1 and held[1] <= pages_for(which, 100) + 1


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["A", "C"])
def test_greedy_generation_through_the_engine(which):
    from vllm_lite_b200 import LLMEngine
    prompts = [tokens_for(which, n, 50 + i) for i, n in enumerate([5, 17, 33, 64])]
    eng = LLMEngine(str(model_dir(which, "float32")), dtype="float32", kv_blocks=64, block_size=PAGE[which],
                    max_batch_size=3, max_num_batched_tokens=48, prefill_chunk_size=13, max_model_len=256)
    outs = eng.generate(prompts, max_tokens=20)
    for p, o in zip(prompts, outs):
        toks = list(p)
        assert len(o) == 20
        for t in o:
            row = plain_run(which, toks, "float32")[0][-1]
            assert int(row.argmax()) == t or float(row.max() - row[t]) < 1e-4 * float(row.abs().max())
            toks.append(t)
    assert eng.stats()["finished"] == len(prompts)


@pytest.mark.gpu
@pytest.mark.parametrize("which", ["C", "E"])
def test_greedy_generation_bfloat16_with_the_cache_sized_from_memory(which):
    """kv_blocks=None: pools (none at all for a model without attention) and state slots are sized from the GPU's free
    memory; the tokens the bfloat16 engine picks lie at or near the plain implementation's maximum."""
    from vllm_lite_b200 import LLMEngine
    prompts = [tokens_for(which, n, 80 + i) for i, n in enumerate([9, 70])]
    eng = LLMEngine(str(model_dir(which, "bfloat16")), dtype="bfloat16", kv_blocks=None, block_size=PAGE[which], max_batch_size=4,
                    max_model_len=256)
    outs = eng.generate(prompts, max_tokens=10)
    far = 0
    for p, o in zip(prompts, outs):
        toks = list(p)
        assert len(o) == 10
        for t in o:
            row = plain_run(which, toks, "bfloat16")[0][-1]
            far += float(row.max() - row[t]) > 2 * tol(which, "bfloat16") * float(row.abs().max())
            toks.append(t)
    assert far <= 2


@pytest.mark.gpu
def test_command_line_and_replay_program(tmp_path):
    """The command line writes a folder from config.json and generates from it (greedy, float32: the plain implementation's
    tokens); bin/trace_run replays steps on the folder after the two low ranks were taken out of its config.json (the
    tensors' shapes give them)."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(CONFIGS["A"]))
    folder = tmp_path / "model"
    run = lambda *a, **k: subprocess.run([sys.executable, *a], capture_output=True, text=True, cwd=root, timeout=900, **k)
    made = run("-m", "vllm_lite_b200", "init", "--config", str(cfg), "--out", str(folder), "--seed", "5", "--std", "0.08")
    assert made.returncode == 0, made.stderr[-2000:]
    prompt = tokens_for("A", 14, 77)
    out = run("-m", "vllm_lite_b200", "--model", str(folder), "--dtype", "float32", "--kv-blocks", "32", "--max-tokens", "6",
              "--prompt-ids", ",".join(map(str, prompt)), "--log-level", "warn")
    assert out.returncode == 0, out.stderr[-2000:]
    got = [int(t) for t in out.stdout.strip().split(",")]
    pc, pw = P.read_model_dir(folder)
    toks = list(prompt)
    for t in got:
        row = P.forward(pc, pw, toks)[0][-1]
        assert int(row.argmax()) == t or float(row.max() - row[t]) < 1e-4 * float(row.abs().max())
        toks.append(t)
    bare = copy.deepcopy(CONFIGS["A"])
    for key in ("decay_rank", "gate_rank"):
        del bare["layers"][0]["mixer"][key]
    (folder / "config.json").write_text(json.dumps(bare))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": prompt[:9], "want": [8]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": prompt[9:], "want": [0, 4]}, {"id": "b", "tokens": [3, 1], "want": []}],
              "end": ["a"]},
             {"step": 2, "entries": [{"id": "b", "tokens": [4], "want": [0]}], "end": ["b"]}]
    outdir = tmp_path / "logits"
    rep = run(str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(outdir),
              "--max-tokens", "64", "--page-size", "8", input="".join(json.dumps(x) + "\n" for x in steps))
    assert rep.returncode == 0, rep.stderr[-2000:]
    assert [l for l in rep.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = P.forward(pc, pw, prompt)[0].float()
    rows = np.fromfile(outdir / "1.f32", dtype="<f4").reshape(2, CONFIGS["A"]["vocab"])
    for row, pos in zip(rows, (9, 13)):
        assert float(np.abs(row - ref[pos].numpy()).max()) <= TOL["float32"] * float(ref[pos].abs().max())
    last = np.fromfile(outdir / "2.f32", dtype="<f4")
    refb = P.forward(pc, pw, [3, 1, 4])[0].float()[2].numpy()
    assert float(np.abs(last - refb).max()) <= TOL["float32"] * float(np.abs(refb).max())
