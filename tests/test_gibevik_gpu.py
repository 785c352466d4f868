"""Gibevik on the GPU against the plain restatement in tests/gibevik_ref.py: each mechanism alone (as a kernel and as a
one-layer model), whole prompts against token-by-token decoding, portions down to two tokens, unequal batches against
each request alone, pages and slots that are used again, keys far back and at page borders with inputs made so that
one key stands out, the causal edge, the steps of the query temperature, routers whose bias, groups and identity
experts decide the choice, the first tokens of a sequence, long decoding, several sizes, and greedy generation through
LLMEngine.  fp32 runs are held to 2e-4 of the logits' spread, bf16 runs to 6e-2; models with routed experts are judged
at the 0.9 quantile of their rows in bf16, where 16-bit operands can flip a near-tied expert choice at single rows."""
import math

import numpy as np
import pytest
import torch

import gibevik_ref as R
from fidasun_util import Driver, rel_err
from gibevik_util import (attn_cfg, dense_cfg, full_cfg, latent_cfg, layer, make_cfg, moe_cfg, random_layers,
                          random_tensors)
from zalalix_util import random_schedule

pytestmark = pytest.mark.gpu
F32_TOL, BF16_TOL = 2e-4, 6e-2


def ref_logits(cfg, tensors, tokens):
    return R.forward(cfg, tensors, tokens, torch.float64).numpy()


def toks(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def _i32(a):
    return torch.tensor(a, dtype=torch.int32, device="cuda")


def judge(dtype, routed=True):
    """(tolerance, quantile of the rows it applies to)."""
    if dtype == torch.float32:
        return F32_TOL, 1.0
    return BF16_TOL, 0.9 if routed else 1.0


# ------------------------------------------------------------------ each mechanism alone (one-layer models)
@pytest.mark.parametrize("kind,mlp,kw", [
    ("attention", None, {}),
    ("attention", None, dict(heads=5, kv_heads=5, dim=24, q_temp=None)),                   # no grouping, no temperature
    ("attention", None, dict(heads=3, kv_heads=1, dim=32, q_temp={"coef": 2.0, "every": 1})),   # tensor-core forms
    ("attention", None, dict(heads=34, kv_heads=2, dim=16)),                               # a group wider than an MMA tile
    ("latent_attention", None, {}),
    ("latent_attention", None, dict(heads=1, dim=1, vdim=1, kv_rank=3)),
    ("latent_attention", None, dict(heads=18, dim=16, vdim=24, kv_rank=64)),               # tensor-core forms
    ("attention", dense_cfg(), {}),
    ("latent_attention", moe_cfg(), {}),
    ("latent_attention", moe_cfg(shared=None, router=dict(experts=4, identity=0, top=1)), {}),
    ("attention", moe_cfg(router=dict(experts=1, identity=5, top=3, groups={"count": 2, "keep": 1})), {}),
])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_layer_alone(lib, kind, mlp, kw, dtype):
    if dtype == torch.bfloat16 and kw.get("vdim") == 1:
        pytest.skip("one-element heads: a single 16-bit rounding is the whole value, nothing averages out")
    cfg = make_cfg([layer(kind, mlp, **kw)])
    w = random_tensors(cfg, seed=3)
    t = toks(90, cfg["vocab"], 1)
    d = Driver(cfg, w, dtype, trace=True)
    d.step([("a", t)])
    tr = []
    want = R.forward(cfg, w, t, torch.float64, tr).numpy()
    resid = d.runner.trace[0, :len(t)].cpu().numpy()
    tol, q = judge(dtype, routed=bool(mlp) and mlp["kind"] == "moe")
    row_err = np.abs(resid - tr[0].numpy()).max(-1)
    assert np.quantile(row_err, q) <= tol * np.abs(tr[0].numpy()).max()
    assert rel_err(d.result("a"), want, q) <= tol


def test_position_vector_joins_the_embedding(lib):
    """A model whose only layer is switched off by zero output weights: the logits are the final norm of embedding
    row + position vector, at positions up to 700 and across portions."""
    cfg = make_cfg([layer("latent_attention", None)], width=36, vocab=40)
    w = random_tensors(cfg, seed=1)
    w["l0.norm1"] = torch.zeros_like(w["l0.norm1"])
    t = toks(700, cfg["vocab"], 2)
    d = Driver(cfg, w, torch.float32)
    d.step([("a", t[:333])]), d.step([("a", t[333:699])]), d.step([("a", t[699:])])
    x = w["embed"].double()[torch.tensor(t)] + R.position_vector(len(t), 36, torch.float64)
    want = (R.norm(x, w["final.norm"].double(), 1e-5) @ w["head"].double().T).numpy()
    assert rel_err(d.result("a"), want) <= F32_TOL


# ------------------------------------------------------------------ attention: distance bias, gate, causal edge, far keys
def _plain_biased_attention(q, k, v, gate, rows_pos, scale, slopes):
    """q [T, H, dk] at positions rows_pos; k [n, G, dk], v [n, G, dv]; gate [T, H * dv] logits."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for r, i in enumerate(rows_pos):
        for h in range(H):
            a = h // (H // G)
            s = (k[:i + 1, a] @ q[r, h]) * scale
            if slopes is not None:
                s = s - slopes[h] * torch.tensor([float(i - j) for j in range(i + 1)], dtype=torch.float64)
            e = torch.exp(s - s.max())
            out[r, h] = (e[:, None] * v[:i + 1, a]).sum(0) / e.sum()
            if gate is not None:
                out[r, h] *= torch.sigmoid(gate[r, h * dv:(h + 1) * dv])
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("split", [True, False])
@pytest.mark.parametrize("dk,H,G", [(12, 4, 2), (32, 3, 1), (16, 34, 2), (96, 2, 2)])
def test_attention_op_bias_gate_and_edges(lib, dtype, split, dk, H, G):
    """Keys carry a position tag u and its square, so a query can put a sharp peak on any position.  Queries per row: a
    peak on the FIRST key (hundreds of places back), one on the key just before a page border, one on the row's own
    position and one on the key just AFTER it (not visible: had the kernel seen it, it would take most of the weight).
    The distance bias is checked with slopes steep enough to move the weights.  Prompt rows and single decoded rows, on
    a shuffled block table, with a gate per output element."""
    from vllm_rs_b200 import ops
    n = 330
    pages = [5, 2, 7, 0, 3, 6]
    g = torch.Generator().manual_seed(0)
    u = (torch.arange(n) - 160.0) / 256.0
    k = torch.randn(n, G, dk, generator=g) * 0.05
    k[:, :, 0], k[:, :, 1] = u[:, None], (u * u)[:, None]
    v = torch.randn(n, G, dk, generator=g)
    kc = torch.zeros(8, 64, G, dk, dtype=dtype, device="cuda")
    vc = torch.zeros(8, 64, G, dk, dtype=dtype, device="cuda")
    for j in range(n):
        kc[pages[j // 64], j % 64], vc[pages[j // 64], j % 64] = k[j].to(dtype).cuda(), v[j].to(dtype).cuda()
    kr, vr = k.to(dtype).double(), v.to(dtype).double()
    bt = _i32([pages])
    tol = 3e-3 if dtype == torch.float32 else 4e-2
    sharp = 16384.0
    slopes = torch.tensor([2.0 ** (-3.0 * (h + 1) / H) for h in range(H)])
    for rows_pos in ([329], [64], [63], [0], list(range(200, 329)), list(range(0, 70)), list(range(250, 260))):
        T = len(rows_pos)
        pos = torch.tensor(rows_pos, dtype=torch.float32)
        for form, sl in (("first", None), ("border", None), ("self", slopes), ("next", None), ("flat", slopes)):
            q = torch.randn(T, H, dk, generator=g) * 0.1
            if form != "flat":
                target = {"first": torch.zeros(T), "border": torch.full((T,), 127.0).minimum(pos), "self": pos,
                          "next": pos + 1}[form]
                ut = (target - 160.0) / 256.0
                q[:, :, 0], q[:, :, 1] = (2.0 * sharp * ut)[:, None], -sharp
            q = q.to(dtype).float()
            gate = torch.randn(T, H * dk, generator=g)
            out = ops.window_attn(q.cuda().contiguous(), kc, vc, None, gate.cuda(), _i32([0, T]), _i32([rows_pos[-1] + 1]),
                                  bt, window=0, keep_first=0, scale=1.0, split=split,
                                  dist_slopes=None if sl is None else sl.cuda()).float().cpu()
            want = _plain_biased_attention(q.double(), kr, vr, gate.double(), rows_pos, 1.0,
                                           None if sl is None else sl.double())
            assert (out.double() - want).abs().max() <= tol * max(1.0, want.abs().max().item()), (rows_pos[0], T, form)


def test_attention_prep_op(lib):
    """Per-head norms with one shared weight, raw key rows as values, and the query temperature at the places
    where its floor steps (position = every - 2, every - 1, 2 every - 1), against the plain formulas."""
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(3)
    H, G, dk, every, coef = 6, 2, 10, 6, 0.75
    pos = torch.tensor([0, 4, 5, 6, 10, 11, 12, 1000, 63, 64])
    T = len(pos)
    slots = torch.tensor([3, 64, 2, 0, 130, 191, 1, 70, 5, 6])
    proj = torch.randn(T, H * dk + G * dk + H * dk, generator=g) * 3        # gate logits ride along, untouched
    qn, kn = torch.randn(dk, generator=g), torch.randn(dk, generator=g)
    kc, vc = torch.zeros(3, 64, G, dk, device="cuda"), torch.zeros(3, 64, G, dk, device="cuda")
    q = ops.window_attn_prep(proj.cuda(), None, qn.cuda(), kn.cuda(), None, pos.cuda(), slots.cuda(), kc, vc, heads=H,
                             rot_dims=0, eps=1e-4, head_norm=True, v_from_k=True, q_temp=(coef, every)).cpu()
    x = proj.double()
    for t in range(T):
        f = R.query_temperature(int(pos[t]), coef, every)
        assert f == 1.0 + coef * math.log((int(pos[t]) + 1) // every + 1)
        for h in range(H):
            want = R.norm(x[t, h * dk:(h + 1) * dk], qn.double(), 1e-4) * f
            assert torch.allclose(q[t, h].double(), want, atol=3e-5, rtol=1e-5), (t, h)
        s = int(slots[t])
        for a in range(G):
            raw = x[t, H * dk + a * dk:H * dk + (a + 1) * dk]
            assert torch.allclose(kc.cpu()[s // 64, s % 64, a].double(), R.norm(raw, kn.double(), 1e-4), atol=3e-5)
            assert torch.allclose(vc.cpu()[s // 64, s % 64, a].double(), raw, atol=1e-6)
    assert R.query_temperature(4, coef, every) == 1.0 and R.query_temperature(5, coef, every) > 1.0


@pytest.mark.parametrize("where", ["prompt", "decoded"])
def test_query_temperature_steps_show_in_logits(lib, where):
    """A one-layer model with a large temperature coefficient: the plain model's logits at the position where the floor
    steps differ from those of a model whose step lies one position later by far more than the tolerance, and the
    framework follows the right one, in a prompt portion and for a token decoded alone."""
    every = 9
    cfg = make_cfg([layer("attention", None, q_temp={"coef": 4.0, "every": every})])
    late = make_cfg([layer("attention", None, q_temp={"coef": 4.0, "every": every + 1})])
    w = random_tensors(cfg, seed=4)
    t = toks(2 * every + 3, cfg["vocab"], 5)
    want, other = ref_logits(cfg, w, t), ref_logits(late, w, t)
    edge = every - 1                                               # floor((p + 1) / every) becomes 1 here
    assert rel_err(want[edge:edge + 1], other[edge:edge + 1]) > 50 * F32_TOL
    assert rel_err(want[:edge], other[:edge]) < 1e-12
    d = Driver(cfg, w, torch.float32)
    if where == "prompt":
        d.step([("a", t[:edge - 1])]), d.step([("a", t[edge - 1:])])
    else:
        d.step([("a", t[:edge])])
        for x in t[edge:]:
            d.step([("a", [x])])
    assert rel_err(d.result("a"), want) <= F32_TOL


# ------------------------------------------------------------------ latent attention: gate, shared cache
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R_", [(3, 24), (18, 64)])
def test_latent_attention_op_with_gate_on_a_shared_cache(lib, dtype, H, R_):
    """The attention kernel alone on a cache that another call filled: absorbed queries against cached latents, a far
    latent made to stand out, the per-head gate, prompt rows and a decoded row."""
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(2)
    n, pages = 200, [3, 0, 2, 1]
    c = torch.randn(n, R_, generator=g).to(dtype)
    cache = torch.zeros(4, 64, R_, dtype=dtype, device="cuda")
    for j in range(n):
        cache[pages[j // 64], j % 64] = c[j].cuda()
    cr = c.double()
    tol = 2e-3 if dtype == torch.float32 else 4e-2
    for rows_pos in ([199], [64], list(range(100, 200)), list(range(0, 66))):
        T = len(rows_pos)
        q = torch.randn(T, H, R_, generator=g)
        q[-1, 0] = 40.0 * cr[0].float()                            # the last row's first head asks for the first token
        gate = torch.randn(T, H, generator=g) * 2
        out = ops.latent_attn(q.cuda().contiguous(), cache, None, _i32([0, T]), _i32([rows_pos[-1] + 1]), _i32([pages]),
                              kv_rank=R_, rot_dim=0, window=0, scale=0.2, gate=gate.cuda()).float().cpu()
        for r, i in enumerate(rows_pos):
            for h in range(H):
                s = (cr[:i + 1] @ q[r, h].double()) * 0.2
                p = torch.softmax(s, 0)
                want = (p[:, None] * cr[:i + 1]).sum(0) * torch.sigmoid(gate[r, h].double())
                assert (out[r, h].double() - want).abs().max() <= tol * max(1.0, want.abs().max().item()), (i, h)
        if rows_pos[-1] > 0:
            assert (out[-1, 0].double() - cr[0] * torch.sigmoid(gate[-1, 0].double())).abs().max() <= 3e-2 * cr[0].abs().max()


def test_layers_that_share_a_latent_cache(lib):
    """Two layers read the cache of a third (one of them with other head counts and sizes): the plain model with the
    shared latents agrees, and it differs from a model in which the reading layer sees the latents one layer late."""
    cfg = make_cfg([layer("latent_attention", dense_cfg()),
                    layer("latent_attention", None, kv_from=0, heads=2, dim=20, vdim=8),
                    layer("attention", None),
                    layer("latent_attention", dense_cfg(24), kv_from=0)])
    w = random_tensors(cfg, seed=6)
    t = toks(140, cfg["vocab"], 7)
    want = ref_logits(cfg, w, t)
    for dtype in (torch.float32, torch.bfloat16):
        d = Driver(cfg, w, dtype)
        d.step([("a", t[:70])]), d.step([("a", t[70:72])])
        for x in t[72:]:
            d.step([("a", [x])])
        assert rel_err(d.result("a"), want) <= judge(dtype, routed=False)[0]


# ------------------------------------------------------------------ router and experts
def test_router_op_bias_groups_and_negative_scores(lib):
    """The router alone: choice by softmax + bias inside the kept groups only, weights without the bias.  With a bias of
    -5 everywhere every choice score is negative: members of dropped groups must still not win (a dropped member must
    not be treated as a score of zero).  A bias that lifts one group's best member decides which groups stay."""
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, E = 50, 12
    z = torch.randn(T, E, generator=g) * 2
    for bias, groups, keep, top in ((None, 0, 0, 3), (torch.full((E,), -5.0), 4, 2, 3), (torch.randn(E, generator=g), 3, 1, 4),
                                    (torch.tensor([0.0] * 11 + [3.0]), 6, 2, 2), (torch.randn(E, generator=g) * 0.1, 1, 1, 12),
                                    (torch.randn(E, generator=g), 12, 5, 5)):
        idx, wt = ops.moe_route_ex(z.cuda(), None if bias is None else bias.cuda(), top, 1.0, groups, keep)
        idx, wt = idx.cpu(), wt.cpu()
        for t in range(T):
            want_idx, want_w = R.route(z[t].double(), None if bias is None else bias.double(), top, groups, keep)
            assert idx[t].tolist() == want_idx, (t, groups)
            assert torch.allclose(wt[t].double(), torch.stack(want_w), atol=1e-6)
    idx, _ = ops.moe_route_ex(z.cuda(), torch.tensor([0.0] * 11 + [3.0]).cuda(), 2, 1.0, 6, 2)
    assert (idx[:, 0] == 11).all()                                    # the lifted expert, through its group


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_op_squared_relu_and_identity(lib, dtype):
    from vllm_rs_b200 import ops
    g = torch.Generator().manual_seed(8)
    T, D, F, E, ident, top = 70, 40, 24, 5, 2, 3
    h = torch.randn(T, D, generator=g).to(dtype)
    wu = (torch.randn(E, F, D, generator=g) / D ** 0.5).to(dtype)
    wd = (torch.randn(E, D, F, generator=g) / F ** 0.5).to(dtype)
    idx = torch.stack([torch.randperm(E + ident, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    idx[0] = torch.tensor([E, E + 1, 0])                              # both identity experts at once
    wt = torch.rand(T, top, generator=g)
    out = torch.full((T, D), 7.0, device="cuda")
    ops.moe_experts_ex(out, h.cuda(), idx.cuda(), wt.cuda(), wu.cuda(), wd.cuda(), act="relu2", identity=ident,
                       accumulate=False)
    want = torch.zeros(T, D, dtype=torch.float64)
    for t in range(T):
        for j in range(top):
            e = int(idx[t, j])
            y = h[t].double() if e >= E else (torch.relu(wu[e].double() @ h[t].double()) ** 2) @ wd[e].double().T
            want[t] += wt[t, j].double() * y
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert (out.cpu().double() - want).abs().max() <= tol * want.abs().max()


def test_identity_experts_and_groups_decide_the_logits(lib):
    """A correction that always selects the identity experts, and one that always drops their group: both agree with
    the plain model and differ from each other by far more than the tolerance."""
    mlp = moe_cfg(router=dict(experts=4, identity=2, top=2, groups={"count": 3, "keep": 2}), shared=None)
    cfg = make_cfg([layer("latent_attention", mlp)])
    w = random_tensors(cfg, seed=9)
    t = toks(60, cfg["vocab"], 3)
    outs = []
    for corr in ([0, 0, 0, 0, 9.0, 9.0], [0, 0, 0, 0, -9.0, -9.0]):
        w["l0.mlp.correction"] = torch.tensor(corr).to(torch.bfloat16)
        d = Driver(cfg, w, torch.float32)
        d.step([("a", t)])
        assert rel_err(d.result("a"), ref_logits(cfg, w, t)) <= F32_TOL
        outs.append(d.result("a"))
    assert rel_err(outs[0], outs[1]) > 50 * F32_TOL


# ------------------------------------------------------------------ schedules
def test_a_far_token_and_the_causal_edge_show_in_logits(lib):
    """Replacing the very first token of a 300-token prompt changes the last row's logits of the plain model by far
    more than the tolerance (the flattest head's slope is 2^-8), and the framework follows, the last row decoded alone
    after portions that end at and just after a page border."""
    cfg = make_cfg([layer("attention", None, heads=2, kv_heads=1, dim=16, scale=1.0, q_temp=None)])
    w = random_tensors(cfg, seed=11)
    n = 300
    base = toks(n, cfg["vocab"] - 1, 5)
    t = list(base)
    t[0] = cfg["vocab"] - 1
    want, other = ref_logits(cfg, w, t), ref_logits(cfg, w, base)
    assert rel_err(want[-1:], other[-1:]) > 5 * F32_TOL
    d = Driver(cfg, w, torch.float32)
    d.step([("a", t[:64])]), d.step([("a", t[64:129])]), d.step([("a", t[129:n - 1])]), d.step([("a", t[n - 1:])])
    assert rel_err(d.result("a"), want) <= F32_TOL


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_decode_and_portions_agree_with_the_plain_model(lib, dtype):
    cfg = full_cfg()
    w = random_tensors(cfg, seed=7)
    t = toks(150, cfg["vocab"], 3)
    want = ref_logits(cfg, w, t)
    tol, q = judge(dtype)
    d = Driver(cfg, w, dtype)
    d.step([("whole", t)])
    assert rel_err(d.result("whole"), want, q) <= tol
    d.close("whole")
    d.step([("dec", t[:60])])
    for x in t[60:]:
        d.step([("dec", [x])])
    assert rel_err(d.result("dec"), want, q) <= tol
    d.close("dec")
    cuts = [2, 1, 2, 61, 2, 3, 64, 2, 13]                            # 150 tokens; cuts inside and at the ends of pages
    at = 0
    for c in cuts:
        d.step([("cut", t[at:at + c])])
        at += c
    assert at == len(t)
    assert rel_err(d.result("cut"), want, q) <= tol
    if dtype == torch.float32:                                       # the cut must not matter beyond rounding
        assert rel_err(d.result("cut"), d.result("dec")) <= 2e-5


def test_unequal_batches_and_reuse_of_pages_and_slots(lib):
    cfg = full_cfg()
    w = random_tensors(cfg, seed=9)
    V = cfg["vocab"]
    reqs = {"a": toks(130, V, 1), "b": toks(3, V, 2), "c": toks(70, V, 3), "d": toks(65, V, 4), "e": toks(40, V, 5),
            "f": toks(129, V, 6)}
    want = {k: ref_logits(cfg, w, v) for k, v in reqs.items()}
    d = Driver(cfg, w, torch.float32, num_blocks=7, max_seqs=4, slots=4)      # 7 pages: a(3) + c(2) + d(2) fill it
    at = {k: 0 for k in reqs}

    def portion(k, n):
        p = (k, reqs[k][at[k]:at[k] + n])
        at[k] += n
        return p

    d.step([portion("a", 64), portion("b", 2)])
    d.step([portion("a", 1), portion("b", 1), portion("c", 30)])
    d.close("b")                                                      # its page and slot go back
    d.step([portion("c", 40), portion("a", 2), portion("d", 65)])
    d.step([portion("a", 63)])
    d.close("a"), d.close("c")
    assert d.sched.num_free_blocks == 5 and d.sched.num_free_state_slots == 3
    d.step([portion("e", 39), portion("f", 128)])                     # reuses a's and c's pages and slots
    d.step([portion("f", 1), portion("e", 1)])
    for k in "abcdef":
        assert at[k] == len(reqs[k])
        assert rel_err(d.result(k), want[k]) <= F32_TOL, k


def test_first_tokens_and_long_decoding(lib):
    cfg = full_cfg()
    w = random_tensors(cfg, seed=13)
    t = toks(260, cfg["vocab"], 8)
    want = ref_logits(cfg, w, t)
    d = Driver(cfg, w, torch.float32)
    for x in t:                                                       # every token alone, from the very first
        d.step([("a", [x])])
    got = d.result("a")
    assert rel_err(got[:6], want[:6]) <= F32_TOL
    assert rel_err(got, want) <= F32_TOL


def test_other_sizes(lib):
    """Sizes of one and values that coincide elsewhere: one head, one key / value head per query head, a temperature
    that steps at every position, a latent of rank one, one expert with top one, one group that is always kept, a
    router made of identity experts but for one, no feed-forward at all."""
    cfg = make_cfg([layer("attention", dense_cfg(7), heads=1, kv_heads=1, dim=2, scale=1.0, q_temp={"coef": 0.01, "every": 1}),
                    layer("latent_attention", moe_cfg(expert={"ff": 1}, shared={"ff": 1},
                                                      router=dict(experts=1, identity=0, top=1, groups={"count": 1, "keep": 1})),
                          heads=1, dim=3, vdim=130, kv_rank=1, scale=2.0),
                    layer("latent_attention", None, kv_from=1, heads=7, dim=1, vdim=5, kv_rank=1),
                    layer("attention", moe_cfg(expert={"ff": 130}, shared=None, router=dict(experts=1, identity=3, top=4)),
                          heads=7, kv_heads=7, dim=8)],
                   width=24, vocab=50, eps=1e-3)
    w = random_tensors(cfg, seed=17)
    t = toks(80, cfg["vocab"], 9)
    want = ref_logits(cfg, w, t)
    d = Driver(cfg, w, torch.float32)
    d.step([("a", t[:7])]), d.step([("a", t[7:9])]), d.step([("a", t[9:])])
    assert rel_err(d.result("a"), want) <= F32_TOL


def test_greedy_generation_through_the_engine(lib):
    """LLMEngine (schedule -> chunked prefill -> decode, state slots from the scheduler) against greedy decoding with
    the plain model."""
    from vllm_rs_b200 import engine, models
    cfg = full_cfg()
    w = random_tensors(cfg, seed=21)
    V = cfg["vocab"]
    prompts = [toks(75, V, 1), toks(5, V, 2), toks(40, V, 3)]
    new = 12
    runner = models.build_runner(cfg, w, dtype=torch.float32, device="cuda", num_blocks=12, max_blocks_per_seq=4,
                                 max_seqs=5, max_tokens=64, num_state_slots=5)
    eng = engine.LLMEngine(runner, 12, 3, chunk_size=32)              # prompts longer than a chunk are cut
    sids = [eng.add_request(p, new) for p in prompts]
    out = eng.run_to_completion()
    for sid, p in zip(sids, prompts):
        seq, want = list(p), []
        for _ in range(new):
            lg = ref_logits(cfg, w, seq)[-1]
            top2 = np.sort(lg)[-2:]
            nxt = int(lg.argmax())
            want.append(nxt)
            seq.append(nxt)
            if top2[1] - top2[0] < 1e-3:                              # a near tie may flip in fp32: stop comparing there
                break
        assert out[sid][:len(want)] == want
    assert eng.sched.num_free_state_slots == 5


# ------------------------------------------------------------------ random configurations under random schedules
@pytest.mark.parametrize("seed", [11, 12, 13, 14, 15, 16])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_random_configurations_under_random_schedules(lib, seed, dtype):
    """Sizes, layer orders and constants drawn at random (odd sizes, groups wider than an MMA tile, temperatures that
    step at every position, routers with and without groups and identity experts, layers that read an earlier layer's
    latents); five requests of 5 .. 420 tokens share four state slots and just enough pages, so both are used again.
    bf16 runs are judged at the 0.9 quantile of all requests' rows together: with 16-bit operands a near-tied expert
    choice can flip at single rows."""
    rng = np.random.default_rng(seed)
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]              # noqa: E731
    cfg = make_cfg(random_layers(rng, int(rng.integers(2, 6))), width=pick(64, 128, 200), vocab=pick(300, 512),
                   eps=pick(1e-6, 1e-5))
    w = random_tensors(cfg, seed=seed)
    reqs = {f"r{i}": toks(pick(5, 40, 150, 260, 420), cfg["vocab"], seed + i) for i in range(5)}
    pages = sum(sorted((len(v) + 63) // 64 for v in reqs.values())[-4:])
    d = Driver(cfg, w, dtype, num_blocks=pages, max_seqs=4, slots=4)
    for st, ends in random_schedule(rng, reqs):
        d.step(st)
        for k in ends:
            d.close(k)
    tol, q = judge(dtype)
    want = {k: ref_logits(cfg, w, v) for k, v in reqs.items()}
    got, ref = np.concatenate([d.result(k) for k in reqs]), np.concatenate([want[k] for k in reqs])
    assert rel_err(got, ref, q) <= tol, [L["type"] for L in cfg["layers"]]
    if dtype == torch.float32:
        for k in reqs:
            assert rel_err(d.result(k), want[k]) <= tol, k


# ------------------------------------------------------------------ a model folder through the command line
def _write_model_folder(path, cfg, tensors):
    """config.json and model.safetensors (8-byte little-endian header length, JSON header, raw data), bf16 tensors."""
    import json
    import struct
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        raw = t.contiguous().view(torch.uint8).numpy().tobytes() if t.dtype != torch.bfloat16 else \
            t.contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    with open(path / "config.json", "w") as f:
        json.dump(cfg, f)


def test_model_folder_through_trace_runner_and_generate(lib, tmp_path):
    """The registry picks the model by config.json; the trace runner replays two interleaved requests on a pool of
    three pages (the second request reuses the first one's page and slot), `generate` decodes greedily."""
    import json
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    cfg = full_cfg()
    w = random_tensors(cfg, seed=23)
    assert all(t.dtype == torch.bfloat16 for t in w.values())
    _write_model_folder(tmp_path, cfg, w)
    V = cfg["vocab"]
    a, b, c = toks(70, V, 1), toks(9, V, 2), toks(64, V, 3)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:40], "want": [0, 39]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[2:], "want": [6]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[40:69], "want": [28]}, {"id": "c", "tokens": c, "want": [63]}], "end": ["c"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[69:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    r = subprocess.run([str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps), text=True,
                       capture_output=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb, rc = ref_logits(cfg, w, a), ref_logits(cfg, w, b), ref_logits(cfg, w, c)
    want = {0: ra[[0, 39]], 1: rb[[8]], 2: np.stack([ra[68], rc[63]]), 3: ra[[69]]}
    for i, ref in want.items():
        got = np.fromfile(out / f"{i}.f32", dtype="<f4").reshape(-1, V)
        assert rel_err(got, ref) <= 2 * F32_TOL, i
    r = subprocess.run([sys.executable, "-m", "vllm_rs_b200", "generate", "--model", str(tmp_path), "--dtype", "float32",
                        "--prompt-ids", ",".join(map(str, b)), "--max-new-tokens", "5"], cwd=root, text=True,
                       capture_output=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = json.loads(r.stdout.strip().split("\n")[-1])["output_ids"]
    seq = list(b)
    for k in range(5):
        lg = ref_logits(cfg, w, seq)[-1]
        top2 = np.sort(lg)[-2:]
        if top2[1] - top2[0] < 1e-3:
            break
        assert got[k] == int(lg.argmax()), k
        seq.append(int(lg.argmax()))
