"""Host-side pieces behind the Tasadra decoder: the model registry, the arrangement of weights for the launch plan, the
config reader's checks, and the plain restatement's own invariants."""
import math

import numpy as np
import pytest
import torch

import tasadra_ref as R
from tasadra_util import full_cfg, layer, make_cfg, random_layers, random_tensors


def test_registry_knows_the_family():
    from vllm_rs_b200 import models
    assert "Tasadra" in models.registered() and "Tasadra" in models.HYBRID_ARCHITECTURES
    assert models.architecture_of({"architecture": "Tasadra"}) == "Tasadra"


def test_command_line_lists_the_architecture(capsys):
    from vllm_rs_b200.__main__ import main
    assert main(["models"]) == 0
    assert "Tasadra" in capsys.readouterr().out.split()


def test_maps_are_laid_out_one_after_the_other():
    from vllm_rs_b200.models.tasadra import map_major
    H, dk, D = 3, 4, 5
    w = torch.arange(H * 2 * dk * D, dtype=torch.float32).reshape(H * 2 * dk, D)
    m = map_major(w, H, 2, dk).reshape(2, H, dk, D)
    for h in range(H):
        for j in range(2):
            assert torch.equal(m[j, h], w.reshape(H, 2, dk, D)[h, j])


def test_lambda_of_differential_attention():
    from vllm_rs_b200.models.tasadra import differential_lambda
    g = torch.Generator().manual_seed(0)
    v = [torch.randn(9, generator=g).to(torch.bfloat16) for _ in range(4)]
    W = {"lq1": v[0].double(), "lk1": v[1].double(), "lq2": v[2].double(), "lk2": v[3].double()}
    assert math.isclose(differential_lambda(*v, 0.3), float(R.differential_lambda(W, "", 0.3)), rel_tol=1e-12)


def test_frequency_tables_agree_with_the_plain_formulas():
    from vllm_rs_b200.rotary import rotary_frequencies
    for n, base, sc in ((16, 10000.0, None), (12, 300.0, {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}),
                        (40, 1000000.0, {"factor": 8.0, "original": 1024, "fast": 16.0, "slow": 2.0}), (2, 2.0, None)):
        f, fac = rotary_frequencies(n, base, sc)
        rf, rfac = R.pair_frequencies(n, base, sc)
        assert np.allclose(f, rf.numpy(), rtol=1e-14) and math.isclose(fac, rfac, rel_tol=1e-14)


def test_config_reader_rejects_what_the_design_excludes():
    from vllm_rs_b200.models import build_runner
    kw = dict(dtype=torch.float32, device="cpu", num_blocks=2, max_blocks_per_seq=2, max_seqs=1, max_tokens=64)
    later = make_cfg([layer("attention_2", 0, kv_from=1), layer("attention_2", 0)])
    with pytest.raises(ValueError):
        build_runner(later, random_tensors(later), **kw)
    chain = make_cfg([layer("attention_2", 0), layer("attention_2", 0, kv_from=0), layer("attention_2", 0, kv_from=1)])
    with pytest.raises(ValueError):                                   # the source must have projections of its own
        build_runner(chain, random_tensors(chain), **kw)
    other = make_cfg([layer("attention", 0), layer("attention_2", 0, kv_from=0)])
    with pytest.raises(ValueError):
        build_runner(other, random_tensors(other), **kw)
    odd = make_cfg([layer("attention", 0, vdim=7)])                   # rotated values come in pairs
    with pytest.raises(ValueError):
        build_runner(odd, random_tensors(odd), **kw)
    short = make_cfg([layer("attention", 0), layer("attention", 0)])
    w = random_tensors(short)
    w["l1.dwa"] = w["l1.dwa"][:2]                                     # one weight per earlier result and the embedding
    with pytest.raises(ValueError):
        build_runner(short, w, **kw)
    unknown = make_cfg([layer("attention", 0)])
    unknown["layers"][0]["type"] = "attention_3"
    with pytest.raises(ValueError):
        build_runner(unknown, random_tensors(make_cfg([layer("attention", 0)])), **kw)


def test_plain_model_invariants():
    """The restatement itself: causal; a later token cannot change an earlier row; equal tokens are told apart by the
    rotation and the token shift; the depth weights matter."""
    cfg = full_cfg()
    w = random_tensors(cfg, seed=1)
    t = np.random.default_rng(0).integers(0, cfg["vocab"], size=90).tolist()
    full = R.forward(cfg, w, t).numpy()
    part = R.forward(cfg, w, t[:47]).numpy()
    assert np.abs(full[:47] - part).max() < 1e-9
    same = R.forward(cfg, w, [t[0]] * 5).numpy()
    assert np.abs(same[0] - same[4]).max() > 1e-3
    w2 = dict(w)
    w2["l2.dwa"] = torch.flip(w["l2.dwa"], [0])
    assert np.abs(R.forward(cfg, w2, t).numpy() - full).max() > 1e-3


def test_plain_mechanisms():
    g = torch.Generator().manual_seed(2)
    h = torch.randn(6, 4, generator=g, dtype=torch.float64)
    s = torch.tensor([0.0, 1.0, 0.5, 0.25], dtype=torch.float64)
    out = R.token_shift(h, s)
    assert torch.equal(out[:, 0], h[:, 0])                            # a weight of 0 keeps the token's own value
    assert torch.allclose(out[1:, 1], h[:-1, 1], atol=1e-15) and abs(out[0, 1]) < 1e-15   # a weight of 1: the previous token's
    cut = torch.cat([R.token_shift(h[:2], s), R.token_shift(h[2:], s, h[1])], 0)
    assert torch.allclose(cut, out)
    x = torch.randn(5, 3, 8, generator=g, dtype=torch.float64)
    ang = torch.randn(5, 4, generator=g, dtype=torch.float64)
    back = R.turn_halves(R.turn_halves(x, ang), -ang)
    assert torch.allclose(back, x, atol=1e-12)
    # a value turned by its position j and the sum turned back by i: what arrives is the value turned by j - i
    f = R.pair_frequencies(8, 100.0)[0]
    v = x[:1]
    a = R.turn_halves(R.turn_halves(v, 7.0 * f[None]), -3.0 * f[None])
    assert torch.allclose(a, R.turn_halves(v, 4.0 * f[None]), atol=1e-12)
    y = R.short_conv_silu(h, torch.tensor([[0.0, 0.0, 1.0]] * 4, dtype=torch.float64))
    assert torch.allclose(y, h * torch.sigmoid(h))


def test_random_layers_are_consistent():
    for seed in range(30):
        rng = np.random.default_rng(seed)
        layers = random_layers(rng, 6)
        for i, L in enumerate(layers):
            m = L["mixer"]
            assert m["heads"] % m["kv_heads"] == 0
            if m.get("kv_from") is not None:
                src = layers[m["kv_from"]]
                assert m["kv_from"] < i and src["type"] == "attention_2" and src["mixer"].get("kv_from") is None
                assert all(src["mixer"][n] == m[n] for n in ("heads", "kv_heads", "dim", "vdim"))
            if L["type"] == "attention":
                assert m["vdim"] % 2 == 0 and m["rot"]["dims"] % 2 == 0 and 2 <= m["rot"]["dims"] <= m["dim"]
