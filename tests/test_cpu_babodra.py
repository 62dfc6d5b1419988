"""Babodra without a GPU: configuration reader, registry, weight layout helpers, and the plain restatement's own
mechanisms checked against hand-made cases (the GPU tests compare the served model with that restatement)."""
import math

import pytest
import torch

import babodra_oracle as O
from proxy_inference_engine_b200.babodra import BabodraArgs, interleave_pairs, random_weights
from proxy_inference_engine_b200.checkpoint import MODEL_REGISTRY, model_kind


def test_registry_and_config_reader():
    cfg = O.random_config()
    assert model_kind(cfg) == "Babodra" and "Babodra" in MODEL_REGISTRY
    args = BabodraArgs.from_dict(cfg)
    assert args.to_dict()["layers"] == cfg["layers"] and args.norm_eps == 1e-5
    for key in ("vocab", "width", "layers", "max_positions"):
        with pytest.raises(ValueError):
            BabodraArgs.from_dict({k: v for k, v in cfg.items() if k != key})
    bad = O.random_config()
    bad["layers"][0]["mixer"]["vdim"] = 8
    with pytest.raises(ValueError):
        BabodraArgs.from_dict(bad)
    bad = O.random_config(experts=6, top=5, groups=(3, 2))
    with pytest.raises(ValueError):
        BabodraArgs.from_dict(bad)
    bad = O.random_config()
    bad["layers"][0]["type"] = "delta"
    with pytest.raises(ValueError):
        BabodraArgs.from_dict(bad)


def test_random_weights_cover_every_tensor_the_oracle_reads():
    cfg = O.random_config()
    w = random_weights(BabodraArgs.from_dict(cfg), seed=2)
    out = O.forward(cfg, w, [1, 5, 9, 2])
    assert out.shape == (4, cfg["vocab"]) and torch.isfinite(out).all()
    assert "l2.norm2" not in w and "l1.mlp.shared.sg" in w


def test_interleaved_pairs():
    g, u = torch.arange(6.).view(3, 2), -torch.arange(6.).view(3, 2)
    w = interleave_pairs(g, u)
    assert torch.equal(w[0::2], g) and torch.equal(w[1::2], u)


def test_sink_takes_its_share():
    """One key, score s: the weight is e^s / (1 + e^s), not 1."""
    q = torch.tensor([[[2.0, 0.0]]], dtype=torch.float64)
    k = torch.tensor([[[1.5, 0.0]]], dtype=torch.float64)
    v = torch.tensor([[[1.0, 3.0]]], dtype=torch.float64)
    out = O.sink_attention(q, k, v, 0.5, torch.zeros(1, dtype=torch.float64), 1)
    assert torch.allclose(out[0, 0], v[0, 0] * math.exp(1.5) / (1 + math.exp(1.5)))


def test_distance_bias_counts_back_from_the_query():
    """Equal keys: the weights of key j seen from query i fall off as exp(-slope (i - j))."""
    T = 5
    q = torch.zeros((T, 1, 2), dtype=torch.float64)
    k = torch.zeros((T, 1, 2), dtype=torch.float64)
    v = torch.eye(T, dtype=torch.float64).view(T, 1, T)
    slope = O.head_slopes(1)
    assert float(slope[0]) == 2.0 ** -8
    out = O.sink_attention(q, k, v, 1.0, torch.tensor([0.7], dtype=torch.float64), 1)
    e = torch.exp(-0.7 * torch.arange(T - 1, -1, -1, dtype=torch.float64))
    assert torch.allclose(out[T - 1, 0], e / (1 + e.sum()))
    assert float(out[1, 0, 2:].abs().sum()) == 0.0      # causal


def test_query_temperature_steps():
    t = O.query_temperature(torch.tensor([0., 22., 23., 46., 47.]), 0.5, 24)
    assert torch.allclose(t, 1 + 0.5 * torch.log(torch.tensor([1., 1., 2., 2., 3.])))


def test_group_limited_routing():
    """Group 0 holds the single best expert but group 1 has the better pair: with keep = 1 the choice comes from group 1."""
    r = {"experts": 4, "top": 2, "scale": 2.0, "groups": {"count": 2, "keep": 1}}
    z = torch.tensor([[3.0, -3.0, 1.0, 1.2]], dtype=torch.float64)
    idx, wt = O.route(z, torch.eye(4, dtype=torch.float64), r)
    assert sorted(idx[0].tolist()) == [2, 3]
    assert torch.allclose(wt[0].sort().values, 2.0 * torch.sigmoid(torch.tensor([1.0, 1.2], dtype=torch.float64)))
    r["groups"] = {"count": 2, "keep": 2}
    idx, _ = O.route(z, torch.eye(4, dtype=torch.float64), r)
    assert sorted(idx[0].tolist()) == [0, 3]


def test_dense_unit_clamps_before_the_gate():
    w = {"gate": torch.tensor([[10.0]], dtype=torch.float64), "up": torch.tensor([[-10.0]], dtype=torch.float64),
         "down": torch.tensor([[1.0]], dtype=torch.float64)}
    y = O.dense_ff(torch.tensor([[1.0]], dtype=torch.float64), w, "", {"limit": 0.8})
    g, u = 0.8, -0.8
    assert torch.allclose(y, torch.tensor([[g / (1 + math.exp(-1.702 * g)) * (u + 1)]], dtype=torch.float64))
