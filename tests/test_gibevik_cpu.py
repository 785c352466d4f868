"""Host-side pieces behind the Gibevik decoder: the model registry, the heads' slopes, the config reader's checks, and
the plain restatement's own invariants."""
import math

import numpy as np
import pytest
import torch

import gibevik_ref as R
from gibevik_util import dense_cfg, full_cfg, layer, make_cfg, moe_cfg, random_layers, random_tensors


def test_registry_knows_the_family():
    from vllm_rs_b200 import models
    assert "Gibevik" in models.registered() and "Gibevik" in models.HYBRID_ARCHITECTURES
    assert models.architecture_of({"architecture": "Gibevik"}) == "Gibevik"


def test_command_line_lists_the_architecture(capsys):
    from vllm_rs_b200.__main__ import main
    assert main(["models"]) == 0
    assert "Gibevik" in capsys.readouterr().out.split()


@pytest.mark.parametrize("heads", [1, 3, 8, 12])
def test_head_slopes(heads):
    from vllm_rs_b200.models.gibevik import head_slopes
    s = head_slopes(heads)
    assert s.dtype == torch.float32 and s.shape == (heads,)
    for h in range(heads):
        assert math.isclose(s[h].item(), R.head_slope(h, heads), rel_tol=1e-7)
    assert math.isclose(s[-1].item(), 2.0 ** -8, rel_tol=1e-7)        # the last head always has the flattest slope


def test_config_reader_rejects_what_the_design_excludes():
    from vllm_rs_b200.models import build_runner
    kw = dict(dtype=torch.float32, device="cpu", num_blocks=2, max_blocks_per_seq=2, max_seqs=1, max_tokens=64)
    bad = make_cfg([layer("attention", None, dim=16, vdim=8)])        # raw key rows serve as values: vdim must equal dim
    with pytest.raises(ValueError):
        build_runner(bad, random_tensors(make_cfg([layer("attention", None)])), **kw)
    later = make_cfg([layer("latent_attention", None, kv_from=1), layer("latent_attention", None)])
    with pytest.raises(ValueError):
        build_runner(later, random_tensors(later), **kw)
    chain = make_cfg([layer("latent_attention", None), layer("latent_attention", None, kv_from=0),
                      layer("latent_attention", None, kv_from=1)])    # the source must write latents of its own
    with pytest.raises(ValueError):
        build_runner(chain, random_tensors(chain), **kw)
    rank = make_cfg([layer("latent_attention", None), layer("latent_attention", None, kv_from=0, kv_rank=8)])
    with pytest.raises(ValueError):
        build_runner(rank, random_tensors(rank), **kw)


def test_plain_model_invariants():
    """The restatement itself: causal; position-dependent although nothing is rotated; a later token cannot change an
    earlier row."""
    cfg = full_cfg()
    w = random_tensors(cfg, seed=1)
    t = np.random.default_rng(0).integers(0, cfg["vocab"], size=30).tolist()
    full = R.forward(cfg, w, t).numpy()
    part = R.forward(cfg, w, t[:17]).numpy()
    assert np.abs(full[:17] - part).max() < 1e-9
    same = R.forward(cfg, w, [t[0]] * 5).numpy()
    assert np.abs(same[0] - same[4]).max() > 1e-3                     # the position vector tells equal tokens apart


def test_plain_router():
    z = torch.tensor([2.0, 1.0, 0.0, -1.0, 3.0, -2.0], dtype=torch.float64)
    s = torch.softmax(z, -1)
    idx, wt = R.route(z, None, 2, 0, 0)
    assert idx == [4, 0] and torch.allclose(torch.stack(wt), s[[4, 0]])
    idx, _ = R.route(z, None, 2, 3, 1)                                # groups {0,1} {2,3} {4,5}: only the last one stays
    assert idx == [4, 5]
    idx, wt = R.route(z, torch.tensor([0.0, 0.0, 5.0, 0.0, 0.0, 0.0], dtype=torch.float64), 2, 3, 1)
    assert idx == [2, 3] and torch.allclose(torch.stack(wt), s[[2, 3]])    # the weights carry no correction
    idx, _ = R.route(z, torch.full((6,), -7.0, dtype=torch.float64), 3, 3, 2)   # all choice scores negative
    assert sorted(idx) == [0, 1, 4]


def test_random_layers_are_consistent():
    for seed in range(30):
        rng = np.random.default_rng(seed)
        for i, L in enumerate(random_layers(rng, 5)):
            m, mlp = L["mixer"], L["mlp"]
            if m.get("kv_from") is not None:
                assert m["kv_from"] < i
            if mlp and mlp["kind"] == "moe":
                r = mlp["router"]
                n_all = r["experts"] + r["identity"]
                g = r.get("groups")
                assert r["experts"] >= 1 and r["top"] <= (n_all // g["count"] * g["keep"] if g else n_all)
                assert not g or n_all % g["count"] == 0
