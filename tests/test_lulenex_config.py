"""Lulenex without a device: the configuration's reader and its refusals, the plan (schedule, loop entries, caches per pass, tensor
names and shapes), and the plain implementation's own pieces on cases small enough to do by hand."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_lulenex as P
import tiny_lulenex as tl
from inference_bench_b200.config import ConfigError
from inference_bench_b200.config.lulenex import LulenexConfig
from inference_bench_b200.engine.model import plan_from_config
from inference_bench_b200.parts.base import FixedState, PagedKV, Several
from inference_bench_b200.parts.decoder import Decoder


@pytest.mark.parametrize("name", list(tl.CONFIGS))
def test_config_round_trip_and_plan(name):
    raw = tl.CONFIGS[name]["config"]
    cfg = LulenexConfig.from_dict(raw)
    assert LulenexConfig.from_dict(cfg.to_dict()) == cfg
    _, plan = plan_from_config(raw)
    runs = P.layer_runs(raw)
    assert [(e.layer, None if e.enter is None else e.enter[1]) for e in plan.schedule] == runs
    dec = Decoder(plan)
    specs = {s.name: tuple(s.shape) for s in dec.weight_specs()}
    made = tl.tensors(raw, 1)
    assert set(specs) == set(made) and all(tuple(made[n].shape) == specs[n] for n in made)
    needs = dec.cache_needs()
    assert len(needs) == len(runs)                       # every pass of a looped layer has a cache and state of its own
    for (layer, _), need in zip(runs, needs):
        assert isinstance(need, Several) and need.needs[-1] == FixedState((raw["width"],), torch.float32)     # the shift's last row
        m = raw["layers"][layer]["mixer"]
        if raw["layers"][layer]["type"] == "mamba1":
            assert need.needs[:2] == (FixedState((m["inner"], m["state"]), torch.float32), FixedState((max(m["conv"] - 1, 1), m["inner"]), torch.float32))
        else:
            a, r = m["left"], m["right"]
            assert need.needs[:2] == (PagedKV(a["kv_heads"], a["dim"], None), FixedState((r["heads"], r["dim"], r["vdim"]), torch.float32))


def test_a_model_without_a_loop_has_no_entry_tensors():
    raw = tl.CONFIGS["B"]["config"]
    _, plan = plan_from_config(raw)
    assert plan.stream_parts == () and all(e.enter is None for e in plan.schedule)
    assert not any(s.name.startswith("loop.") for s in Decoder(plan).weight_specs())
    no_key = {k: v for k, v in raw.items() if k != "loop"}
    assert LulenexConfig.from_dict(no_key).loop is None


@pytest.mark.parametrize("path,value,words", [
    (("layers", 0, "type"), "mamba2", "not supported"),
    (("layers", 1, "mixer", "left", "kv_heads"), 3, "multiple"),
    (("layers", 1, "mixer", "left", "vdim"), 8, "values are the keys"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 7, "even"),
    (("layers", 1, "mixer", "left", "rot", "dims"), 64, "at most dim"),
    (("layers", 1, "mixer", "left", "mask", "size"), 0, "positive"),
    (("layers", 1, "mixer", "right", "decay"), [0.5, 0.5], "decay"),
    (("layers", 1, "mixer", "right", "decay"), [0.5, 0.5, 1.5], "decay"),
    (("layers", 0, "mixer", "state"), 300, "at most 256"),
    (("layers", 0, "mlp", "kind"), "moe", "not supported"),
    (("loop", "stop"), 9, "not a loop"),
    (("loop", "times"), 0, "not a loop"),
    (("norm", "eps"), 0.0, "positive"),
])
def test_refusals(path, value, words):
    raw = copy.deepcopy(tl.CONFIGS["A"]["config"])
    at = raw
    for k in path[:-1]:
        at = at[k]
    at[path[-1]] = value
    with pytest.raises(ConfigError, match=words):
        LulenexConfig.from_dict(raw)


def test_missing_keys_are_named():
    raw = copy.deepcopy(tl.CONFIGS["A"]["config"])
    del raw["layers"][1]["mixer"]["left"]["scale"]
    with pytest.raises(ConfigError, match=r"layers\[1\].mixer.left.scale"):
        LulenexConfig.from_dict(raw)


# ------------------------------------------------------------------------------------------ the plain pieces by hand
def test_plain_token_shift_and_norm():
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, -2.0]], dtype=torch.float64)
    out = P.token_shift(h, torch.tensor([0.0, 0.5]))
    assert torch.allclose(out, torch.tensor([[1.0, 1.0], [3.0, 4.0], [5.0, 2.0]], dtype=torch.float64))
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    assert torch.allclose(P.scalar_norm(x, torch.tensor(2.0), 0.0), torch.tensor([[6.0, 8.0]], dtype=torch.float64) / 12.5 ** 0.5)


def test_plain_xielu_is_continuous_and_matches_its_two_sides():
    pq = torch.tensor([0.3, -0.2], dtype=torch.float64)
    z = torch.tensor([-3.0, -1e-9, 0.0, 1e-9, 2.0], dtype=torch.float64)
    y = P.xielu(z, pq)
    sp = lambda v: float(torch.log1p(torch.exp(torch.tensor(v, dtype=torch.float64))))
    assert abs(float(y[4]) - (sp(0.3) * 4.0 + 1.0)) < 1e-12
    assert abs(float(y[0]) - ((0.5 + sp(-0.2)) * (float(torch.exp(torch.tensor(-3.0, dtype=torch.float64))) - 1 + 3.0) - 1.5)) < 1e-12
    assert abs(float(y[1])) < 1e-8 and float(y[2]) == 0.0 and abs(float(y[3])) < 1e-8


def test_plain_blocks_of_positions_and_sink():
    """With one head, queries and keys that do not depend on the token and a block of 3: position 4 averages the values at 3 and 4 with
    the sink's share taken off; nothing of positions 0..2 enters."""
    W, D = 4, 2
    w = {"p.q": torch.zeros((D, W)), "p.q.b": torch.tensor([1.0, 0.0]), "p.k": torch.zeros((D, W)), "p.k.b": torch.tensor([1.0, 0.0]),
         "p.g": torch.zeros((1, W)), "p.sink": torch.tensor([0.0]), "p.o": torch.eye(W)[:, :D].contiguous(), "p.o.b": torch.zeros(W)}
    w["p.k"][1, 0] = 1.0          # the second key (and value) entry is the token's first input
    h = torch.zeros((6, W), dtype=torch.float64)
    h[:, 0] = torch.tensor([100.0, 200.0, 300.0, 1.0, 2.0, 3.0])
    m = {"heads": 1, "kv_heads": 1, "dim": D, "mask": {"size": 3}, "rot": {"base": 10.0, "dims": 0}, "scale": 0.0}
    out = P.chunked_attention(h, w, "p", m, 0.0)
    # scale 0: every seen key and the sink weigh the same; the gate is sigmoid(0) = 1/2
    assert torch.allclose(out[4, 1], torch.tensor((1.0 + 2.0) / 3 / 2, dtype=torch.float64))
    assert torch.allclose(out[3, 1], torch.tensor(1.0 / 2 / 2, dtype=torch.float64))
    assert torch.allclose(out[2, 1], torch.tensor(600.0 / 4 / 2, dtype=torch.float64))


def test_plain_decay_and_scan_recurrences():
    W = 2
    w = {"p.q": torch.eye(W), "p.k": torch.eye(W), "p.v": torch.eye(W), "p.g": torch.zeros((W, W)), "p.norm": torch.ones(W), "p.o": torch.eye(W)}
    h = torch.tensor([[2.0, 0.0], [2.0, 0.0]], dtype=torch.float64)
    m = {"heads": 1, "dim": W, "vdim": W, "decay": [0.5]}
    s = float(P.silu(torch.tensor(2.0, dtype=torch.float64)))
    out = P.decayed_linear_attention(h, w, "p", m, 0.0)
    # o_0 = s^3 e_0, o_1 = (0.5 + 1) s^3 e_0; after the norm over both entries both are sqrt(2) e_0; the gate halves them
    assert torch.allclose(out, torch.tensor([[2 ** 0.5 / 2, 0.0]] * 2, dtype=torch.float64))
    assert s > 0
