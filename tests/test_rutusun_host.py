"""Host-side pieces of the Rutusun family (no GPU): configuration reading, the order of layer runs and pass starts, the
registry, and checks of the float64 oracle against a second formulation of the same mechanism."""
import math

import pytest
import torch

import rutusun_oracle as O
from torchao_fork_b200._models import registry
from torchao_fork_b200._models.rutusun import Rutusun, RutusunArgs, rutusun_configs

F64 = torch.float64


def _cfg(loop=None):
    return O.model_config([O.mamba2_layer(mlp=O.dense()), O.attention_layer(mlp=O.mixture()), O.lightning_layer(mlp=None),
                           O.attention_layer(coef=None, mlp=O.dense(24))], loop=loop)


def test_configuration_round_trip_and_defaults():
    cfg = _cfg((1, 3, 3))
    a = RutusunArgs.from_dict(cfg)
    assert RutusunArgs.from_dict(a.to_dict()) == a
    assert a.layers[3].mixer.temp_coef == 0.0 and a.layers[2].mlp is None
    f = a.layers[1].mlp
    assert (f.experts, f.top, f.n_groups, f.keep, f.shared_ff) == (8, 2, 4, 2, 24)
    assert a.layers[0].mixer.conv_channels == 4 * 6 + 2 * 2 * 10
    one = _cfg()
    one["layers"][2]["mixer"]["decay"] = 0.875
    assert RutusunArgs.from_dict(one).layers[2].mixer.decay == [0.875] * 3
    for name, make in rutusun_configs.items():
        b = make()
        assert RutusunArgs.from_dict(b.to_dict()) == b, name


@pytest.mark.parametrize("loop,runs,enters", [(None, [0, 1, 2, 3], 0), ((1, 3, 3), [0, 1, 2, 1, 2, 1, 2, 3], 3),
                                               ((0, 4, 2), [0, 1, 2, 3, 0, 1, 2, 3], 2), ((2, 2, 2), [0, 1, 2, 3], 2),
                                               ((3, 4, 1), [0, 1, 2, 3], 1)])
def test_order_of_layer_runs_and_pass_starts(loop, runs, enters):
    a = RutusunArgs.from_dict(_cfg(loop))
    assert a.runs == runs
    sched = a.schedule
    assert [t for kind, t in sched if kind == "enter"] == list(range(enters))
    if loop:   # every pass start stands right in front of the span's first layer (or where the empty span would be)
        at = [k for k, (kind, _) in enumerate(sched) if kind == "enter"]
        for k in at:
            nxt = sched[k + 1] if k + 1 < len(sched) else None
            assert loop[0] == loop[1] or nxt == ("layer", loop[0])


def test_bad_configurations_are_refused():
    cfg = _cfg()
    cfg["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(AssertionError):
        RutusunArgs.from_dict(cfg)
    cfg = _cfg()
    cfg["layers"][1]["mlp"]["router"]["top"] = 5        # more than the kept groups hold
    with pytest.raises(AssertionError):
        RutusunArgs.from_dict(cfg)
    cfg = _cfg()
    cfg["layers"][0]["type"] = "unknown"
    with pytest.raises(NotImplementedError):
        RutusunArgs.from_dict(cfg)


def test_weights_are_checked_against_the_configuration():
    cfg = _cfg((1, 3, 2))
    w = O.random_weights(cfg, 0)
    m = Rutusun(RutusunArgs.from_dict(cfg), w, "cpu", torch.float32)
    assert m.layers[1].wgu.shape == (8, 32, 32) and m.layers[1].wd.shape == (8, 32, 16) and m.loop_step.shape == (2, 32)
    with pytest.warns(UserWarning):
        Rutusun(RutusunArgs.from_dict(cfg), dict(w, extra=torch.zeros(1)), "cpu", torch.float32)
    bad = dict(w)
    bad["l1.mix.sink"] = torch.zeros(5)
    with pytest.raises(ValueError):
        Rutusun(RutusunArgs.from_dict(cfg), bad, "cpu", torch.float32)
    del bad["l1.mix.sink"]
    with pytest.raises(KeyError):
        Rutusun(RutusunArgs.from_dict(cfg), bad, "cpu", torch.float32)


def test_registry_knows_the_family():
    fams = registry.families()
    assert "rutusun" in fams and "Rutusun-test" in fams["rutusun"].names()


def test_product_random_weights_name_every_tensor_of_a_configuration():
    cfg = rutusun_configs["Rutusun-test"]()
    w = Rutusun.random_weights(cfg, "cpu", torch.float32)
    Rutusun(cfg, w, "cpu", torch.float32)       # raises on a missing or an unused tensor


# ------------------------------------------------------------------------------------------------ the oracle against itself
def test_oracle_recurrence_equals_its_attention_form():
    """S_t = a S_(t-1) + k v^T read by q is attention without softmax whose weight on key j is a^(t-j) q.k."""
    g = torch.Generator().manual_seed(0)
    T, H, d, dv = 20, 2, 5, 4
    q, k, v = [torch.randn(T, H, c, generator=g, dtype=F64) for c in (d, d, dv)]
    decay = torch.tensor([0.9, 0.5], dtype=F64)
    rec = O.decayed_outer_recurrence(q, k, v, decay.expand(T, H), torch.ones(T, H, dtype=F64))
    t = torch.arange(T)
    for h in range(H):
        wgt = (q[:, h] @ k[:, h].T) * decay[h] ** (t.view(T, 1) - t.view(1, T)).clamp_min(0) * (t.view(T, 1) >= t.view(1, T))
        assert torch.allclose(rec[:, h], wgt @ v[:, h], atol=1e-10)


def test_oracle_sink_takes_weight_and_router_keeps_groups():
    g = torch.Generator().manual_seed(1)
    q, k, v = [torch.randn(6, 1, 4, generator=g, dtype=F64) for _ in range(3)]
    no = O.sink_attention(q, k, v, torch.tensor([-1e9], dtype=F64), 0.5)
    yes = O.sink_attention(q, k, v, torch.tensor([0.0], dtype=F64), 0.5)
    assert torch.allclose(no[0, 0], v[0, 0]) and float(yes[0, 0].abs().sum()) < float(no[0, 0].abs().sum())
    z = torch.randn(50, 12, generator=g, dtype=F64)
    chosen, weight = O.route(z, torch.full((12,), -2.0, dtype=F64), 3, 1, 2, 2.0)
    assert bool(((chosen // 4)[:, 0] == (chosen // 4)[:, 1]).all())     # both from the one kept group
    assert torch.allclose(weight.sum(-1), torch.full((50,), 2.0, dtype=F64))
    assert abs(float(O.query_temperature(20, 0.8, 4)[3]) - (1 + 0.8 * math.log(2))) < 1e-12
    assert float(O.query_temperature(20, 0.8, 4)[2]) == 1.0
