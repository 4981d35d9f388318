"""Host-side pieces of the Fedipel family (no GPU): configuration reading, which layers read which key/value cache and how
the cache is sized for them, the registry, and checks of the float64 oracle against a second formulation of the same
mechanism."""
import math

import pytest
import torch

import fedipel_oracle as O
from torchao_fork_b200._models import registry
from torchao_fork_b200._models.fedipel import Fedipel, FedipelArgs, fedipel_configs
from torchao_fork_b200._models.fedipel.model import NO_WINDOW

F64 = torch.float64


def _cfg():
    return O.model_config([O.retention_layer(mlp=O.dense()), O.attention_layer(mlp=O.mixture()), O.wkv_layer(mlp=None),
                           O.attention_layer(kv_from=1, size=5, keep=3, mlp=O.mixture(experts=4, top=3, shared=0))])


def _args(cfg, w=None):
    return FedipelArgs.from_dict(O.config_json(cfg), None if w is None else {k: tuple(v.shape) for k, v in w.items()})


def test_configuration_round_trip_defaults_and_sizes_that_only_a_tensor_gives():
    cfg = _cfg()
    w = O.random_weights(cfg, 0)
    a = _args(cfg, w)
    assert FedipelArgs.from_dict(a.to_dict(), {k: tuple(v.shape) for k, v in w.items()}) == a
    assert a.to_dict() == O.config_json(cfg)
    assert a.layers[2].mixer.rank == 6 and a.layers[2].mlp is None
    f = a.layers[1].mlp
    assert (f.experts, f.top, f.ff, f.shared_ff) == (6, 2, 16, 24) and a.layers[3].mlp.shared_ff == 0
    assert (a.residual_mult, a.logit_softcap) == (0.6, 12.0)
    assert a.readers_of(1) == [1, 3] and a.readers_of(3) == [] and a.layers[3].mixer.kv_from == 1
    with pytest.raises(AssertionError):      # no tensor shapes: nothing says how wide the decay's inner projection is
        _args(cfg)
    bare = O.model_config([O.attention_layer(rot=0, mlp=None)], softcap=0)
    del bare["layers"][0]["mixer"]["mask"], bare["residual_mult"]
    b = _args(bare)
    assert (b.layers[0].mixer.window, b.layers[0].mixer.keep, b.layers[0].mixer.rot.dims) == (NO_WINDOW, 0, 0)
    assert (b.residual_mult, b.logit_softcap) == (1.0, 0.0)
    for name, make in fedipel_configs.items():
        c = make()
        assert FedipelArgs.from_dict(dict(c.to_dict()), {f"l{i}.mix.w1": (la.mixer.rank, c.width) for i, la in enumerate(c.layers)
                                                        if la.type == "wkv"}) == c, name


def test_bad_configurations_are_refused():
    cfg = _cfg()
    cfg["layers"][1]["mixer"]["kv_heads"] = 3
    with pytest.raises(AssertionError):
        _args(cfg, O.random_weights(_cfg(), 0))
    cfg = _cfg()
    cfg["layers"][3]["mixer"]["kv_from"] = 0            # not an attention layer
    with pytest.raises(AssertionError):
        _args(cfg, O.random_weights(_cfg(), 0))
    cfg = _cfg()
    cfg["layers"][1]["mlp"]["router"]["top"] = 7        # more than there are experts
    with pytest.raises(AssertionError):
        _args(cfg, O.random_weights(_cfg(), 0))
    cfg = _cfg()
    cfg["layers"][0]["mixer"]["decay"] = [0.5]          # one decay for three heads
    with pytest.raises(AssertionError):
        _args(cfg, O.random_weights(_cfg(), 0))
    cfg = _cfg()
    cfg["layers"][0]["type"] = "unknown"
    with pytest.raises(NotImplementedError):
        _args(cfg, O.random_weights(_cfg(), 0))


def test_weights_are_regrouped_and_checked_against_the_configuration():
    cfg = _cfg()
    w = O.random_weights(cfg, 0)
    m = Fedipel(_args(cfg, w), w, "cpu", torch.float32)
    assert m.layers[0].w_in.shape == (2 * 3 * 8 + 2 * 3 * 12, 32) and m.layers[0].inv_freq.shape == (4,)
    assert m.layers[1].w_in.shape == (4 * 2 * 8 + 2 * 2 * 8 + 2 * 12, 32) and m.layers[3].w_in.shape == (4 * 2 * 8, 32)
    assert m.layers[1].wu.shape == (6, 16, 32) and m.layers[1].wd.shape == (6, 32, 16)
    assert m.layers[1].router.shape == (7, 32) and m.layers[3].router.shape == (4, 32)     # the shared expert's gate rides along
    assert m.layers[2].w_rkvg.shape == (4, 32, 32) and m.layers[2].mu.shape == (5, 32)
    lam = math.exp(float((w["l1.mix.lq1"].double() * w["l1.mix.lk1"].double()).sum())) - \
        math.exp(float((w["l1.mix.lq2"].double() * w["l1.mix.lk2"].double()).sum())) + 0.3
    assert abs(m.layers[1].lam - lam) < 1e-12
    with pytest.warns(UserWarning):
        Fedipel(_args(cfg, w), dict(w, extra=torch.zeros(1)), "cpu", torch.float32)
    bad = dict(w)
    bad["l1.mix.q.b"] = torch.zeros(5)
    with pytest.raises(ValueError):
        Fedipel(_args(cfg, w), bad, "cpu", torch.float32)
    del bad["l1.mix.q.b"]
    with pytest.raises(KeyError):
        Fedipel(_args(cfg, w), bad, "cpu", torch.float32)


def test_cache_is_sized_for_the_widest_reader_and_bounded_only_when_a_window_is_cut():
    cfg = _cfg()                                         # owner: window 9, 2 kept; borrower: window 5, 3 kept
    w = O.random_weights(cfg, 0)
    m = Fedipel(_args(cfg, w), w, "cpu", torch.float32)
    m.setup_caches(3, 100)
    c = m.run_state[1].window
    assert (c.ring, c.first_rows) == (9, 3) and c.k.shape == (3, 9, 2 * 2 * 8) and c.v_first.shape == (3, 3, 2 * 12)
    assert m.run_state[3].window is None and m.run_state[0].mat.s.shape == (3, 3, 8, 12)
    assert m.run_state[2].mat.s.shape == (3, 2, 16, 16) and m.run_state[2].shift.prev.shape == (3, 32)
    assert m.states.max_seq_length == 1 << 30            # no window was cut: a sequence may go on
    m = Fedipel(_args(cfg, w), w, "cpu", torch.float32)
    m.setup_caches(1, 6)
    assert m.run_state[1].window.ring == 6 and m.states.max_seq_length == 6
    s = m.states.slot_of("a")
    m.states.extend(s, 6)
    with pytest.raises(RuntimeError):
        m.states.extend(s, 1)
    m.states.slot_of("b")                                # a second request doubles the slots of every state
    assert m.run_state[1].window.k.shape[0] == 2 and m.run_state[2].shift.prev.shape[0] == 2 and m.max_batch_size == 2


def test_registry_knows_the_family():
    fams = registry.families()
    assert "fedipel" in fams and "Fedipel-test" in fams["fedipel"].names()


def test_product_random_weights_name_every_tensor_of_a_configuration():
    cfg = fedipel_configs["Fedipel-test"]()
    w = Fedipel.random_weights(cfg, "cpu", torch.float32)
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        Fedipel(cfg, w, "cpu", torch.float32)       # raises on a missing or an unused tensor


# ------------------------------------------------------------------------------------------------ the oracle against itself
def test_oracle_retention_equals_its_attention_form():
    """S_t = a S_(t-1) + k v^T read by q is attention without softmax whose weight on key j is a^(t-j) q.k."""
    g = torch.Generator().manual_seed(0)
    T, H, d, dv = 20, 2, 5, 4
    q, k, v = [torch.randn(T, H, c, generator=g, dtype=F64) for c in (d, d, dv)]
    decay = [0.9, 0.5]
    rec = O.retention_recurrence(q, k, v, decay)
    t = torch.arange(T)
    for h in range(H):
        wgt = (q[:, h] @ k[:, h].T) * decay[h] ** (t.view(T, 1) - t.view(1, T)).clamp_min(0) * (t.view(T, 1) >= t.view(1, T))
        assert torch.allclose(rec[:, h], wgt @ v[:, h], atol=1e-10)


def test_oracle_time_mixing_equals_its_attention_form():
    """The weight of key j for query t is r_t . (prod of decays j+1 .. t-1) k_j for j < t and r_t . (u k_t) for j = t."""
    g = torch.Generator().manual_seed(1)
    T, H, d = 12, 1, 3
    r, k, v = [torch.randn(T, H, d, generator=g, dtype=F64) for _ in range(3)]
    dec, u = torch.rand(T, H, d, generator=g, dtype=F64), torch.randn(H, d, generator=g, dtype=F64)
    rec = O.wkv_recurrence(r, k, v, dec, u)
    for t in range(T):
        o = (r[t, 0] * u[0] * k[t, 0]).sum() * v[t, 0]
        for j in range(t):
            o = o + (r[t, 0] * dec[j + 1:t, 0].prod(0) * k[j, 0]).sum() * v[j, 0]
        assert torch.allclose(rec[t, 0], o, atol=1e-10)


def test_oracle_rotation_keeps_scores_a_function_of_distance_and_window_mask_counts():
    g = torch.Generator().manual_seed(2)
    x, y = torch.randn(1, 1, 8, generator=g, dtype=F64), torch.randn(1, 1, 8, generator=g, dtype=F64)
    for layout in ("half", "interleaved"):
        s = [float((O.rotate(x, torch.tensor([p + 5]), 6, 100.0, layout) * O.rotate(y, torch.tensor([p]), 6, 100.0, layout)).sum())
             for p in (0, 3, 40)]
        assert max(s) - min(s) < 1e-9
        assert torch.equal(O.rotate(x, torch.tensor([9]), 6, 100.0, layout)[..., 6:], x[..., 6:])      # the rest passes unchanged
    # uniform scores: every visible key gets the same weight, so the result is the mean of the visible values
    T, size, keep = 30, 4, 2
    q, k = torch.zeros(T, 1, 1, 2, dtype=F64), torch.zeros(T, 1, 1, 2, dtype=F64)
    v = torch.randn(T, 1, 3, generator=g, dtype=F64)
    out = O.window_diff_attention(q, k, v, 1.0, size, keep, 0.0, 0.0)
    for i in (0, 3, 4, 5, 29):
        seen = sorted(set(range(min(keep, i + 1))) | set(range(max(0, i - size + 1), i + 1)))
        m = v[seen, 0].mean(0)
        assert torch.allclose(out[i, 0], m / m.pow(2).mean().sqrt(), atol=1e-9)
