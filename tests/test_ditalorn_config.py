"""Ditalorn without a device: its configuration, its plan, its tensors, what it asks of the cache manager, and the plain model's own pieces."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_ditalorn as P
import tiny_ditalorn as td
from inference_bench_b200.config import ConfigError
from inference_bench_b200.engine.model import plan_from_config
from inference_bench_b200.parts.base import FixedState, PagedKV, PagedRows, Several
from inference_bench_b200.parts.decoder import Decoder


@pytest.mark.parametrize("name", list(td.CONFIGS))
def test_configuration_plan_and_tensors(name):
    raw = td.CONFIGS[name]["config"]
    cfg, plan = plan_from_config(raw)
    assert plan.architecture == "Ditalorn" and len(plan.layers) == len(raw["layers"]) and plan.root == "" and plan.max_positions == raw["max_positions"]
    again = type(cfg).from_dict(cfg.to_dict())
    assert again == cfg and cfg.embedding_scale == (raw.get("embedding") or {}).get("scale", 1.0)
    d = Decoder(plan)
    made = td.tensors(raw, 1)
    specs = {s.name: tuple(s.shape) for s in d.weight_specs()}
    assert specs == {n: tuple(t.shape) for n, t in made.items()}
    for need, l in zip(d.cache_needs(), raw["layers"]):
        m = l["mixer"]
        if l["type"] == "latent_attention":
            assert need == PagedRows(m["kv_rank"], (m.get("mask") or {}).get("size"))
            continue
        G, taps = m.get("kv_heads") or m["heads"], m.get("conv") or 0
        pages = PagedKV(G, max(m["dim"], m["vdim"]))
        channels = (m["heads"] + G) * m["dim"] + G * m["vdim"]
        assert need == (Several((pages, FixedState((taps - 1, channels), torch.float32))) if taps > 1 else pages)


def test_cache_manager_keeps_windows_apart_and_state_beside_pages():
    from inference_bench_b200.cache.manager import CacheManager
    d = Decoder(plan_from_config(td.CONFIGS["A"]["config"])[1])
    cache = CacheManager(d.cache_needs(), 16, 8, 2, 64, sources=d.cache_sources())
    assert sorted(g.window or 0 for g in cache.groups) == [0, 0, 9, 1000]       # two sigmoid layers of different rows, two windows
    assert set(cache.states) == {(0, 1), (3, 1)}
    cache.admit("a")
    cache.extend("a", 40)
    cache.commit("a", 40)
    assert sorted(cache.used_pages()) == [1, 3, 3, 3]      # the short window let the pages that passed go
    cache.release("a")
    cache.check()


@pytest.mark.parametrize("change,why", [
    (lambda c: c["layers"][0].update(type="conv"), "not supported"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(dim=300), "at most 256"),
    (lambda c: c["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda c: c["layers"][1]["mixer"].update(q_rank=0), "q_rank"),
    (lambda c: c["layers"][1]["mixer"]["mask"].update(size=0), "mask.size"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top 9"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "equal groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(keep=1, count=6), "cannot come"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not supported"),
    (lambda c: c.pop("max_positions"), "max_positions"),
    (lambda c: c["norm"].update(eps=0.0), "positive"),
])
def test_refusals(change, why):
    raw = copy.deepcopy(td.CONFIGS["A"]["config"])
    change(raw)
    with pytest.raises(ConfigError, match=why):
        plan_from_config(raw)


def test_route_by_hand():
    """Six experts in three groups of two, two groups stay, two experts a token. The correction makes a group with small scores win, choice
    scores of a kept group may all be negative, and the weights are the scores without the correction."""
    s = torch.tensor([[0.9, 0.1, 0.2, 0.3, 0.6, 0.5]], dtype=torch.float64)
    corr = torch.tensor([-2.0, -2.0, 0.5, 0.4, -0.7, -0.8], dtype=torch.float64)
    # choice: [-1.1, -1.9 | 0.7, 0.7 | -0.1, -0.3]; group sums -3.0, 1.4, -0.4: groups 1 and 2 stay; the two largest choices are experts 2 and 3
    idx, wt = P.choose(s, corr, 2, 3, 2)
    assert sorted(idx[0].tolist()) == [2, 3] and sorted(wt[0].tolist()) == [0.2, 0.3]
    # three experts a token: the third comes from group 2 although its choice score is negative, and never from the dropped group 0
    idx, wt = P.choose(s, corr, 3, 3, 2)
    assert sorted(idx[0].tolist()) == [2, 3, 4] and math.isclose(sum(wt[0].tolist()), 1.1)
    # one group stays: a group's score is the sum of its two largest, not its largest
    s2 = torch.tensor([[0.9, 0.0, 0.5, 0.5]], dtype=torch.float64)
    idx, _ = P.choose(s2, torch.zeros(4, dtype=torch.float64), 1, 2, 1)
    assert idx[0].tolist() == [2] or idx[0].tolist() == [3]


def test_plain_pieces():
    """The window counts the position itself; the temperature steps where (p + 1) reaches a multiple of the period; the convolution's last tap is
    the current token; sigmoid weights are not normalised."""
    T, H = 6, 1
    q = torch.zeros((T, H, 2), dtype=torch.float64)
    k = torch.zeros((T, H, 2), dtype=torch.float64)
    v = torch.arange(T, dtype=torch.float64).view(T, 1, 1).expand(T, H, 1).contiguous()
    o = P.windowed_softmax(q, k, v, 1.0, 2)
    assert torch.allclose(o[:, 0, 0], torch.tensor([0.0, 0.5, 1.5, 2.5, 3.5, 4.5], dtype=torch.float64))
    assert torch.allclose(P.windowed_softmax(q, k, v, 1.0, 1)[:, 0, 0], torch.arange(T, dtype=torch.float64))
    temp = P.query_temperature(7, {"coef": 1.0, "every": 3})
    assert torch.allclose(temp, 1.0 + torch.log(torch.tensor([1, 1, 2, 2, 2, 3, 3], dtype=torch.float64)))
    u = torch.arange(4, dtype=torch.float64).view(4, 1) + 1.0
    y = P.causal_conv(u, torch.tensor([[10.0, 1.0]]))
    assert y[:, 0].tolist() == [1.0, 12.0, 23.0, 34.0]
    o = P.sigmoid_weights(q, k, torch.ones((T, 1, 1), dtype=torch.float64), 1.0, None, None, None)
    assert torch.allclose(o[:, 0, 0], 0.5 * torch.arange(1, T + 1, dtype=torch.float64))
    o = P.sigmoid_weights(q, k, torch.ones((T, 1, 1), dtype=torch.float64), 1.0, torch.tensor([1.0]), torch.tensor([1.0]), torch.tensor([0.0]))
    want = torch.cumsum(torch.sigmoid(-torch.log1p(torch.arange(T, dtype=torch.float64))), 0)
    assert torch.allclose(o[:, 0, 0], want)


def test_plain_model_runs_and_prefix_property():
    """The plain model is causal: the logits at a position do not change when tokens are added behind it."""
    raw = td.CONFIGS["A"]["config"]
    w = td.tensors(raw, 5)
    toks = torch.randint(0, raw["vocab"], (30,), generator=torch.Generator().manual_seed(1)).tolist()
    a, b = P.logits(toks, raw, w), P.logits(toks[:19], raw, w)
    assert torch.allclose(a[:19], b, atol=1e-9) and torch.isfinite(a).all()
    assert len(P.greedy(toks[:5], 3, raw, w)) == 3
