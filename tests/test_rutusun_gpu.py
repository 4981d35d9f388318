"""Rutusun on the GPU against the float64 oracle (tests/rutusun_oracle.py): every mechanism's kernel alone, then the model
through the framework's step function, state manager, decode engine and Generator.  Configurations and weights are
made here; float32 runs are held to a tight bound at every position (only summation order differs), bfloat16 runs to
the rounding noise of bf16 products (`_within` says what a close call between two experts may do to one position)."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import rutusun_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 1e-4
F64 = torch.float64


def _lm():
    from torchao_fork_b200 import _lib
    return _lib, _lib.lm()


def _st():
    return torch.cuda.current_stream().cuda_stream


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _err(got, ref):
    """Root mean square of the difference (mean over the vocabulary taken off), relative to the reference's spread."""
    got, ref = torch.as_tensor(got).double().cpu(), torch.as_tensor(ref).double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-30)).max())


def _within(got, ref, tol, exact=False):
    """Every position within tol.  A bfloat16 run may leave the bound at one position in fifty (at least one): where two
    experts' choice scores are closer than bfloat16 rounding, the run and the oracle may choose differently, which moves
    that position's logits by far more than rounding does; the positions after it must be back inside."""
    got, ref = torch.as_tensor(got).double().cpu(), torch.as_tensor(ref).double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    e = d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-30)
    over = int((e > tol).sum())
    return over == 0 if exact else over <= max(1, e.numel() // 50)


def _bf16_tol(cfg, w, toks):
    """A bfloat16 run may be 3 times as far from the exact logits as bfloat16 rounding alone moves them."""
    return 3.0 * O.rounding_noise(cfg, w, toks, _err)


def _model(cfg, w, dtype=torch.float32, slots=2, seq=256):
    from torchao_fork_b200._models.rutusun import Rutusun, RutusunArgs
    m = Rutusun(RutusunArgs.from_dict(cfg), w, "cuda", dtype).eval()
    m.setup_caches(slots, seq)
    return m


def _tokens(cfg, n, seed=0):
    return torch.randint(0, cfg["vocab"], (n,), generator=_gen(seed)).tolist()


def _rows(segs):
    """[(slot, first position, rows)] -> per-row slot, pos, back, ahead and the segments' (first row, rows) on the device."""
    slot, pos, back, ahead, first, count = [], [], [], [], [], []
    for s, p0, c in segs:
        first.append(len(slot))
        count.append(c)
        slot += [s] * c
        pos += list(range(p0, p0 + c))
        back += list(range(c))
        ahead += list(range(c - 1, -1, -1))
    return _i32(slot), _i32(pos), _i32(back), _i32(ahead), _i32(first), _i32(count)


def _close(got, ref, tol=2e-5):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("W", [33, 256, 2500])
@pytest.mark.parametrize("parts", ["all", "norm_only", "no_next", "vec_only"])
def test_post_norm_residual_with_pass_additions_and_next_norm(W, parts):
    lib, L = _lm()
    g, n, eps = _gen(W), 5, 1e-5
    x, y, rows = torch.randn(n, W, generator=g) * 3, torch.randn(n, W, generator=g) * 7, torch.randn(n, W, generator=g)
    pw, vec, nw = [(1 + 0.3 * torch.randn(W, generator=g)).to(torch.bfloat16) for _ in range(3)]
    use_y, use_rows, use_vec, use_next = {"all": (1, 1, 1, 1), "norm_only": (0, 0, 0, 1), "no_next": (1, 1, 0, 0), "vec_only": (0, 0, 1, 1)}[parts]
    ref = x.double()
    if use_y:
        ref = ref + O.rms_norm(y.double() + (torch.randn(W, generator=_gen(W + 1)).double() if W != 256 else 0.0), pw.double(), eps)
    if use_rows:
        ref = ref + rows.double()
    if use_vec:
        ref = ref + vec.double()
    xd, yd, rd, pd, vd, nd = x.cuda(), y.cuda(), rows.cuda(), pw.cuda(), vec.cuda(), nw.cuda()
    h = torch.zeros(n, W, device="cuda", dtype=torch.bfloat16)
    bias = torch.randn(W, generator=_gen(W + 1)) if use_y and W != 256 else None
    bd = bias.cuda() if bias is not None else None
    lib.lm_check(L.ao_lm_postnorm_residual(xd.data_ptr(), yd.data_ptr() if use_y else None, lib.DT_F32,
                                           bd.data_ptr() if bd is not None else None, pd.data_ptr() if use_y else None,
                                           rd.data_ptr() if use_rows else None, vd.data_ptr() if use_vec else None,
                                           nd.data_ptr() if use_next else None, lib.DT_BF16, eps, n, W, h.data_ptr(), _st()), "postnorm")
    assert _close(xd, ref)
    if use_next:
        assert _close(h, O.rms_norm(ref, nw.double(), eps), 1e-2)


@pytest.mark.parametrize("H,G,d,dv,every", [(4, 2, 8, 12, 16), (3, 3, 33, 5, 1), (2, 1, 64, 64, 7)])
def test_query_key_preparation_bias_weight_and_temperature_steps(H, G, d, dv, every):
    lib, L = _lm()
    g, eps, coef = _gen(d), 1e-5, 0.7
    pos = [0, 1, every - 2, every - 1, every, 2 * every - 2, 2 * every - 1, 3 * every, 1000 * every - 1, 70000]
    pos = [p for p in pos if p >= 0]
    n, ld = len(pos), H * d + G * d + G * dv + 3
    proj = torch.randn(n, ld, generator=g)
    qb, kb, vb = [(0.5 * torch.randn(k, generator=g)) for k in (H * d, G * d, G * dv)]
    qw, kw = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    q = (proj[:, :H * d] + qb).double().view(n, H, d)
    k = (proj[:, H * d:(H + G) * d] + kb).double().view(n, G, d)
    temp = 1.0 + coef * torch.log(torch.floor((torch.tensor(pos, dtype=F64) + 1) / every) + 1.0)
    q_ref = O.rms_norm(q, qw.double(), eps) * temp.view(n, 1, 1)
    k_ref = O.rms_norm(k, kw.double(), eps)
    v_ref = (proj[:, (H + G) * d:(H + G) * d + G * dv] + vb).double()
    pd, dev = proj.cuda(), [t.cuda() for t in (qb, kb, vb, qw, kw)]
    posd = _i32(pos)
    qn, kn, vn = torch.empty(n, H, d, device="cuda"), torch.empty(n, G, d, device="cuda"), torch.empty(n, G * dv, device="cuda")
    # positions 0 .. n-1 of slot 1 of a cache with n rows also receive the keys and values
    ring_k, ring_v = torch.zeros(2, n, G, d, device="cuda"), torch.zeros(2, n, G * dv, device="cuda")
    rpos, rslot = _i32(list(range(n))[::-1]), _i32([1] * n)
    lib.lm_check(L.ao_lm_qk_norm_prep(pd.data_ptr(), ld, 0, H * d, (H + G) * d, *[t.data_ptr() for t in dev], coef, every,
                                      posd.data_ptr(), None, None, None, 0, n, H, G, d, dv, eps, lib.DT_F32, qn.data_ptr(),
                                      kn.data_ptr(), vn.data_ptr(), _st()), "qk_norm_prep")
    assert _close(qn, q_ref) and _close(kn, k_ref) and _close(vn, v_ref)
    lib.lm_check(L.ao_lm_qk_norm_prep(pd.data_ptr(), ld, 0, H * d, (H + G) * d, *[t.data_ptr() for t in dev], 0.0, 0,
                                      rpos.data_ptr(), rslot.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), n, n, H, G, d, dv, eps,
                                      lib.DT_F32, qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), _st()), "qk_norm_prep")
    assert _close(ring_k[1].flip(0), k_ref) and _close(ring_v[1].flip(0), v_ref) and float(ring_k[0].abs().max()) == 0.0
    # no temperature, no weights, no biases: plain unit-RMS rows
    lib.lm_check(L.ao_lm_qk_norm_prep(pd.data_ptr(), ld, 0, H * d, (H + G) * d, None, None, None, None, None, 0.0, 0, None, None, None,
                                      None, 0, n, H, G, d, dv, eps, lib.DT_F32, qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), _st()),
                 "qk_norm_prep")
    assert _close(qn, O.unit_rms(proj[:, :H * d].double().view(n, H, d), eps))


def _attend(q, k, v, sink, scale, cuts, dtype, tensor, slot=1, slots=3, ring=None, n_split=1):
    """q [T][H][d] fp32, k / v [T][G][.]: the attention kernel over the sequence in portions `cuts`, through the ring."""
    from torchao_fork_b200._models.segment_step import chunk_tiles
    import ctypes
    lib, L = _lm()
    dt = lib.DT_F32 if dtype == torch.float32 else lib.DT_BF16
    T, H, d = q.shape
    G, dv = k.shape[1], v.shape[2]
    S = ring or T
    rk = torch.full((slots, S, G, d), 7.0, device="cuda", dtype=dtype)      # what a freed slot may hold: never read
    rv = torch.full((slots, S, G, dv), -9.0, device="cuda", dtype=dtype)
    tr = ctypes.c_int()
    plan = L.ao_lm_chunk_attention_prompt_plan if tensor else L.ao_lm_chunk_attention_plan
    lib.lm_check(plan(dt, H, G, d, dv, ctypes.byref(tr)), "plan")
    assert tr.value > 0
    sk = sink.float().cuda()
    outs, at = [], 0
    for c in cuts:
        sl, ps, bk, ah, _, _ = _rows([(slot, at, c)])
        tf, tc = chunk_tiles(np.array([0]), np.array([c]), np.arange(at, at + c), tr.value, S)
        tfd, tcd = _i32(tf.tolist()), _i32(tc.tolist())
        qd = q[at:at + c].float().cuda().contiguous()
        kd, vd = k[at:at + c].to(dtype).cuda().contiguous(), v[at:at + c].to(dtype).cuda().contiguous()
        o = torch.empty(c, H * dv, device="cuda", dtype=dtype)
        common = (qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), rk.data_ptr(), rv.data_ptr(), dt, None, 0, None, 0, sk.data_ptr(),
                  sl.data_ptr(), ps.data_ptr(), bk.data_ptr(), tfd.data_ptr(), tcd.data_ptr(), len(tf), H, G, d, dv, S, scale, 0.0, 1.0)
        if tensor:
            lib.lm_check(L.ao_lm_sink_attention_prompt(*common, o.data_ptr(), H * dv, _st()), "sink_attention_prompt")
        else:
            ws = torch.empty(max(16, int(L.ao_lm_chunk_attention_workspace_bytes(len(tf), G, dv, n_split))), dtype=torch.uint8, device="cuda")
            lib.lm_check(L.ao_lm_sink_attention(*common, n_split, ws.data_ptr(), ws.numel(), o.data_ptr(), H * dv, _st()), "sink_attention")
        lib.lm_check(L.ao_lm_ring_append(kd.data_ptr(), vd.data_ptr(), c, G * d, G * dv, S, dt, sl.data_ptr(), ps.data_ptr(), ah.data_ptr(),
                                         rk.data_ptr(), rv.data_ptr(), _st()), "ring_append")
        outs.append(o.float().cpu().view(c, H, dv))
        at += c
    return torch.cat(outs)


ATTN = [(4, 2, 8, 12, False), (3, 1, 24, 40, False), (2, 2, 33, 7, False), (4, 2, 32, 48, True), (2, 1, 96, 96, True), (8, 8, 16, 128, True)]


@pytest.mark.parametrize("shape", range(len(ATTN)))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sink_attention_whole_portions_and_decoding(shape, dtype):
    H, G, d, dv, tensor = ATTN[shape]
    if tensor and dtype == torch.float32:
        pytest.skip("the tensor-core form reads bf16 keys and values")
    g, T = _gen(shape), 150
    q, k, v = torch.randn(T, H, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, G, dv, generator=g)
    sink = torch.randn(H, generator=g) + 1.0
    k16, v16 = k.to(dtype), v.to(dtype)
    ref = O.sink_attention((q.bfloat16() if tensor else q).double(), k16.double(), v16.double(), sink.double(), 0.3)
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    for cuts in ([T], [70, 2, 3, 64, 1, 1, 9], [1] * 20 + [130]):
        got = _attend(q, k, v, sink, 0.3, cuts, dtype, tensor)
        assert _close(got, ref, tol), cuts
    if not tensor:
        got = _attend(q, k, v, sink, 0.3, [140] + [1] * 10, dtype, False, n_split=5, ring=160)
        assert _close(got, ref, tol)


@pytest.mark.parametrize("tensor", [False, True])
@pytest.mark.parametrize("key,query", [(0, 149), (3, 64), (63, 64), (64, 64), (64, 127), (65, 64), (100, 99), (128, 149)])
def test_sink_attention_one_dominant_key_near_far_and_in_the_future(tensor, key, query):
    """One key stands out for one query: the output is that key's value when the key is not in the future — wherever it
    lies (the first token, a tile's edge, the query itself) — and the ordinary mixture otherwise; a dominant sink takes
    the weight away from every key."""
    H, G, d, dv, T = 2, 1, 32, 32, 150
    dtype = torch.bfloat16 if tensor else torch.float32
    g = _gen(key * 151 + query)
    q, k, v = torch.randn(T, H, d, generator=g) * 0.1, torch.randn(T, G, d, generator=g) * 0.1, torch.randn(T, G, dv, generator=g)
    q[query, :, 0], k[key, :, 0] = 40.0, 40.0
    sink = torch.tensor([0.0, -30.0])
    for cuts in ([T], [query, 1, T - query - 1] if 0 < query < T - 1 else [T]):
        got = _attend(q, k, v, sink, 1.0, cuts, dtype, tensor)
        ref = O.sink_attention(q.to(dtype).double() if tensor else q.double(), k.to(dtype).double(), v.to(dtype).double(), sink.double(), 1.0)
        assert _close(got, ref, 1e-5 if not tensor else 1.5e-2)
        if key <= query:
            assert _close(got[query, 0], v[key, 0].to(dtype), 2e-2)
    big = _attend(q, k, v, torch.tensor([2000.0, 2000.0]), 1.0, [T], dtype, tensor)
    assert float(big.abs().max()) < 1e-6


def _recurrence(q, k, v, a, b, a_head, skip, act, cuts, G, slots=3, slot=2, tile=0):
    """The kernel over one sequence in portions; q / k [T][G][d], v [T][H][dv], a / b [T][H] or None.  tile > 0: portions
    longer than that run in the tiled form."""
    from torchao_fork_b200._models.segment_step import scan_tiles
    lib, L = _lm()
    T, H, dv = v.shape
    d = q.shape[2]
    state = torch.full((slots, H, d, dv), 123.0, device="cuda")       # a freed slot's leftovers: not read at position 0
    ahd = a_head.float().cuda() if a_head is not None else None        # held: a pointer outlives no temporary
    skd = skip.float().cuda() if skip is not None else None
    outs, at = [], 0
    for c in cuts:
        sl, ps, bk, ah, sf, sc = _rows([(slot, at, c)])
        qd, kd, vd = [t[at:at + c].reshape(c, -1).float().cuda().contiguous() for t in (q, k, v)]
        ad = a[at:at + c].float().cuda().contiguous() if a is not None else None
        bd = b[at:at + c].float().cuda().contiguous() if b is not None else None
        o = torch.empty(c, H * dv, device="cuda")
        n_seg, s0, sn, n_whole, ws = 1, None, None, 0, None
        if tile and c > tile:
            tf, tc, t0, tn = scan_tiles(np.array([0]), np.array([c]), tile)
            sf, sc, s0, sn, n_seg, n_whole = _i32(tf.tolist()), _i32(tc.tolist()), _i32(t0.tolist()), _i32(tn.tolist()), len(tf), 1
            ws = torch.empty(int(L.ao_lm_outer_recurrence_workspace_bytes(n_seg, c, H, d, dv)) // 4, device="cuda")
        lib.lm_check(L.ao_lm_outer_recurrence(qd.data_ptr(), G * d, kd.data_ptr(), G * d, vd.data_ptr(), H * dv, act,
                                              ad.data_ptr() if a is not None else None, bd.data_ptr() if b is not None else None, H,
                                              ahd.data_ptr() if ahd is not None else None,
                                              skd.data_ptr() if skd is not None else None, H, G, d, dv,
                                              state.data_ptr(), sl.data_ptr(), ps.data_ptr(), sf.data_ptr(), sc.data_ptr(), n_seg,
                                              s0.data_ptr() if s0 is not None else None, sn.data_ptr() if sn is not None else None,
                                              n_whole, c, ws.data_ptr() if ws is not None else None, o.data_ptr(), H * dv, _st()),
                     "outer_recurrence")
        outs.append(o.cpu().view(c, H, dv))
        at += c
    return torch.cat(outs)


@pytest.mark.parametrize("H,G,d,dv", [(3, 3, 8, 12), (4, 2, 5, 33), (2, 1, 48, 48), (6, 6, 32, 32), (2, 2, 130, 70), (1, 1, 300, 40)])
def test_matrix_state_recurrence_both_forms_in_portions(H, G, d, dv):
    g, T = _gen(d), 70
    q, k, v = torch.randn(T, G, d, generator=g), torch.randn(T, G, d, generator=g), torch.randn(T, H, dv, generator=g)
    grp = torch.arange(H) // (H // G)
    # state-space form: decays and input scales per (row, head), groups of heads share q and k, a skip term
    a, b, skip = torch.rand(T, H, generator=g) * 0.5 + 0.5, torch.rand(T, H, generator=g) * 2, torch.randn(H, generator=g)
    ref = O.decayed_outer_recurrence(q.double()[:, grp], k.double()[:, grp], v.double(), a.double(), b.double()) \
        + skip.double().view(1, H, 1) * v.double()
    for cuts in ([T], [1] * T, [2, 3, 16, 1, 17, 15, 16]):
        assert _close(_recurrence(q, k, v, a, b, None, skip, 0, cuts, G), ref, 3e-5), cuts
    for tile, cuts in ((16, [T]), (5, [3, 40, 27]), (64, [1, 69]), (3, [35, 35])):      # the tiled form, tiles cut anywhere
        assert _close(_recurrence(q, k, v, a, b, None, skip, 0, cuts, G, tile=tile), ref, 3e-5), (tile, cuts)
    if H == G:
        # linear-attention form: a fixed decay per head, SiLU on load
        decay = torch.rand(H, generator=g) * 0.4 + 0.6
        ref = O.decayed_outer_recurrence(O.silu(q.double()), O.silu(k.double()), O.silu(v.double()), decay.double().expand(T, H),
                                         torch.ones(T, H, dtype=F64))
        for cuts in ([T], [33, 1, 1, 35]):
            assert _close(_recurrence(q, k, v, None, None, decay, None, 1, cuts, G), ref, 3e-5), cuts
            assert _close(_recurrence(q, k, v, None, None, decay, None, 1, cuts, G, tile=7), ref, 3e-5), cuts


def test_matrix_state_recurrence_remembers_the_first_token_and_batches_segments():
    lib, L = _lm()
    H, d, dv, g = 2, 16, 16, _gen(5)
    lens = [40, 1, 7]
    q, k, v = [[torch.randn(n, H, c, generator=g) for n in lens] for c in (d, d, dv)]
    decay = torch.tensor([1.0, 0.5])
    refs = [O.decayed_outer_recurrence(q[i].double(), k[i].double(), v[i].double(), decay.double().expand(n, H), torch.ones(n, H, dtype=F64))
            for i, n in enumerate(lens)]
    # with decay 1 the first token's outer product is still in the state at the end
    q0 = q[0].clone()
    only_first = O.decayed_outer_recurrence(q0.double()[-1:], k[0].double()[:1], v[0].double()[:1], torch.ones(1, H, dtype=F64), torch.ones(1, H, dtype=F64))
    assert float(only_first[0, 0].abs().max()) > 1e-3
    # all three sequences in one launch, slots out of order
    sl, ps, bk, ah, sf, sc = _rows([(2, 0, 40), (0, 0, 1), (1, 0, 7)])
    cat = lambda ts: torch.cat([t.reshape(t.shape[0], -1) for t in ts]).float().cuda().contiguous()
    qd, kd, vd = cat(q), cat(k), cat(v)
    state = torch.zeros(3, H, d, dv, device="cuda")
    ddec0 = decay.cuda()
    o = torch.empty(48, H * dv, device="cuda")
    lib.lm_check(L.ao_lm_outer_recurrence(qd.data_ptr(), H * d, kd.data_ptr(), H * d, vd.data_ptr(), H * dv, 0, None, None, 0,
                                          ddec0.data_ptr(), None, H, H, d, dv, state.data_ptr(), sl.data_ptr(), ps.data_ptr(),
                                          sf.data_ptr(), sc.data_ptr(), 3, None, None, 0, 48, None, o.data_ptr(), H * dv, _st()),
                 "outer_recurrence")
    assert _close(o.cpu().view(48, H, dv), torch.cat(refs), 3e-5)
    # the same three in the tiled form: 6-row tiles, segments of 7, 1 and 2 tiles; slot 1 continues a state, the others start
    from torchao_fork_b200._models.segment_step import scan_tiles
    tf, tc, s0, sn = scan_tiles(np.array([0, 40, 41]), np.array([40, 1, 7]), 6)
    dtf, dtc, ds0, dsn, ddec = _i32(tf.tolist()), _i32(tc.tolist()), _i32(s0.tolist()), _i32(sn.tolist()), decay.cuda()
    state2 = torch.full((3, H, d, dv), 9.0, device="cuda")
    ws = torch.empty(int(L.ao_lm_outer_recurrence_workspace_bytes(len(tf), 48, H, d, dv)) // 4, device="cuda")
    o2 = torch.empty(48, H * dv, device="cuda")
    lib.lm_check(L.ao_lm_outer_recurrence(qd.data_ptr(), H * d, kd.data_ptr(), H * d, vd.data_ptr(), H * dv, 0, None, None, 0,
                                          ddec.data_ptr(), None, H, H, d, dv, state2.data_ptr(), sl.data_ptr(), ps.data_ptr(),
                                          dtf.data_ptr(), dtc.data_ptr(), len(tf), ds0.data_ptr(), dsn.data_ptr(), 3, 48, ws.data_ptr(),
                                          o2.data_ptr(), H * dv, _st()),
                 "outer_recurrence")
    assert _close(o2.cpu().view(48, H, dv), torch.cat(refs), 3e-5)
    assert _close(state2, state, 3e-5)


@pytest.mark.parametrize("taps", [4, 1, 2, 7])
def test_state_space_inputs_convolution_memory_across_portions(taps):
    lib, L = _lm()
    g, T, C, H, eps = _gen(taps), 40, 19, 3, 1e-5
    ld = 5 + C + H
    proj = torch.randn(T, ld, generator=g) * 2
    proj[7, 5 + C] = 60.0           # a step size far in the linear part of softplus
    proj[8, 5 + C] = -60.0          # and one far in its exponential part
    cw, cb = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    dtb, alog = torch.randn(H, generator=g), torch.randn(H, generator=g) * 0.5
    ref_conv = O.silu(O.causal_conv(proj[:, 5:5 + C].double(), cw.double(), cb.double()))
    step = torch.nn.functional.softplus(proj[:, 5 + C:].double() + dtb.double(), threshold=1e9)
    ref_a = torch.exp(-torch.exp(alog.double()) * step)
    dev = [t.cuda() for t in (cw, cb, dtb, alog)]
    for cuts in ([T], [1] * T, [2, 1, 3, 5, 2, 27], [3, 37]):
        state = torch.full((2, max(1, taps - 1), C), 55.0, device="cuda")     # a freed slot's leftovers
        conv, a, b, at = [], [], [], 0
        for c in cuts:
            sl, ps, bk, ah, _, _ = _rows([(1, at, c)])
            pd = proj[at:at + c].cuda().contiguous()
            co, ao, bo = torch.empty(c, C, device="cuda"), torch.empty(c, H, device="cuda"), torch.empty(c, H, device="cuda")
            lib.lm_check(L.ao_lm_ssd_prep(pd.data_ptr(), ld, 5, 5 + C, c, C, taps, dev[0].data_ptr(), dev[1].data_ptr(), lib.DT_F32,
                                          state.data_ptr(), sl.data_ptr(), ps.data_ptr(), bk.data_ptr(), H, dev[2].data_ptr(),
                                          dev[3].data_ptr(), co.data_ptr(), ao.data_ptr(), bo.data_ptr(), _st()), "ssd_prep")
            lib.lm_check(L.ao_lm_conv_state_save(pd.data_ptr() + 4 * 5, ld, c, C, taps, sl.data_ptr(), ps.data_ptr(), bk.data_ptr(),
                                                 ah.data_ptr(), state.data_ptr(), _st()), "conv_state_save")
            conv.append(co.cpu()), a.append(ao.cpu()), b.append(bo.cpu())
            at += c
        assert _close(torch.cat(conv), ref_conv), cuts
        assert _close(torch.cat(a), ref_a) and _close(torch.cat(b), step, 1e-6), cuts


@pytest.mark.parametrize("width,groups", [(24, 1), (24, 3), (288, 2), (5, 5), (1030, 1)])
def test_gated_group_norm_gate_behind_and_in_front(width, groups):
    lib, L = _lm()
    g, n, eps = _gen(width), 4, 1e-5
    y, z = torch.randn(n, width + 3, generator=g) * 4, torch.randn(n, width + 5, generator=g) * 2
    wt = 1 + 0.3 * torch.randn(width, generator=g)
    yd, zd, wd = y.cuda(), z.cuda(), wt.cuda()
    out = torch.empty(n, width, device="cuda")
    for mode in (0, 1):
        lib.lm_check(L.ao_lm_gated_group_norm(yd.data_ptr(), width + 3, zd.data_ptr(), width + 5, mode, n, width, groups, wd.data_ptr(),
                                              lib.DT_F32, eps, out.data_ptr(), _st()), "gated_group_norm")
        yy, zz = y[:, :width].double(), z[:, :width].double()
        if mode == 0:
            ref = O.grouped_unit_rms(yy, groups, eps) * wt.double() * torch.sigmoid(zz)
        else:
            ref = O.grouped_unit_rms(yy * O.silu(zz), groups, eps) * wt.double()
        assert _close(out, ref), mode


@pytest.mark.parametrize("E,groups,keep,top", [(15, 3, 2, 4), (8, 4, 2, 2), (8, 8, 3, 3), (6, 1, 1, 6), (64, 8, 4, 8), (5, 5, 5, 1), (16, 2, 1, 8)])
def test_router_group_limited_choice_with_negative_scores(E, groups, keep, top):
    lib, L = _lm()
    g, n = _gen(E * 7 + top), 300
    z = torch.randn(n, E, generator=g) * 2
    corr = torch.randn(E, generator=g) * 0.5 - 1.5        # choice scores below zero: a closed group must not win as "0"
    chosen, weight = O.route(z.double(), corr.double(), groups, keep, top, 1.75)
    zd, cd = z.cuda(), corr.cuda()
    idx, wt = torch.empty(n, top, dtype=torch.int32, device="cuda"), torch.empty(n, top, device="cuda")
    lib.lm_check(L.ao_lm_router_group_topk_logits(zd.data_ptr(), n, E, top, cd.data_ptr(), groups, keep, 1.75, idx.data_ptr(),
                                                  wt.data_ptr(), _st()), "router")
    assert torch.equal(idx.cpu().long(), chosen)
    assert _close(wt, weight, 1e-6)
    assert _close(wt.sum(-1), torch.full((n,), 1.75, dtype=F64), 1e-5)


def test_silu_gated_unit_activation():
    lib, L = _lm()
    g = _gen(3)
    for ff in (40, 37):
        gu = (torch.randn(11, 2 * ff, generator=g) * 3).to(torch.bfloat16)
        gud, y = gu.cuda(), torch.empty(11, ff, device="cuda", dtype=torch.bfloat16)
        lib.lm_check(L.ao_lm_glu_act_shift(gud.data_ptr(), lib.DT_BF16, 11, ff, float("inf"), 1.0, 0.0, y.data_ptr(), _st()), "glu_act")
        ref = O.silu(gu[:, :ff].double()) * gu[:, ff:].double()
        assert _close(y, ref, 1e-2)


# ------------------------------------------------------------------------------------------------ the model
def _mixed():     # every mixer and both feed-forwards, a looped span in the middle, a layer without feed-forward
    return O.model_config([O.mamba2_layer(mlp=O.dense()), O.attention_layer(mlp=O.mixture()), O.lightning_layer(mlp=None),
                           O.attention_layer(heads=2, kv_heads=1, dim=16, vdim=8, coef=None, mlp=O.dense(24))], loop=(1, 3, 3))


def _plain():     # no loop at all; groups that hold one expert; no shared expert
    return O.model_config([O.lightning_layer(mlp=O.mixture(experts=4, top=2, groups=4, keep=3, shared=0)),
                           O.attention_layer(mlp=O.dense())], width=24, vocab=50)


def _ones():      # sizes that are 1 or equal: one head everywhere, one group, one expert chosen, a loop that runs once
    return O.model_config([O.attention_layer(heads=1, kv_heads=1, dim=16, vdim=16, every=1, mlp=O.mixture(experts=2, top=1, groups=1, keep=1, ff=16, shared=16)),
                           O.lightning_layer(heads=1, dim=16, vdim=16, decay=[1.0], mlp=O.dense(16)),
                           O.mamba2_layer(heads=1, vdim=16, state=16, groups=1, conv=1, norm_groups=1, mlp=O.dense(16))],
                          width=16, vocab=16, loop=(0, 3, 1))


def _tensor():    # head sizes that the tensor-core attention form covers; the loop from the first layer on
    return O.model_config([O.attention_layer(heads=4, kv_heads=2, dim=32, vdim=48, scale=0.2, mlp=O.dense(64)),
                           O.mamba2_layer(heads=4, vdim=16, state=32, groups=4, conv=3, norm_groups=4, mlp=O.mixture(experts=6, top=3, groups=3, keep=2)),
                           O.lightning_layer(heads=2, dim=32, vdim=32, mlp=O.dense(64))], width=64, vocab=97, loop=(0, 2, 2))


def _odd():       # odd sizes everywhere
    return O.model_config([O.lightning_layer(heads=3, dim=5, vdim=7, mlp=O.mixture(experts=9, top=2, groups=3, keep=1, ff=11, shared=13)),
                           O.mamba2_layer(heads=3, vdim=7, state=5, groups=1, conv=5, norm_groups=3, mlp=O.dense(29)),
                           O.attention_layer(heads=3, kv_heads=1, dim=11, vdim=5, every=3, mlp=None)], width=27, vocab=31, loop=(2, 3, 2))


CONFIGS = {"mixed": _mixed, "plain": _plain, "ones": _ones, "tensor": _tensor, "odd": _odd}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_and_every_layer_run_against_oracle(name, dtype):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 21)
    toks = _tokens(cfg, 45, 1)
    layers = []
    ref = O.forward(cfg, w, toks, layers)
    m = _model(cfg, w, dtype)
    logits, sums = m.step_engine.layer_sums(m.states.slot_of("a"), toks)
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    assert _within(logits, ref, tol, dtype == torch.float32)
    if dtype == torch.float32:
        assert sums.shape[0] == len(layers)
        for r in range(sums.shape[0]):
            assert _close(sums[r], layers[r], 1e-4), r


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_prefill_equals_token_by_token_and_portions(dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 22)
    toks = _tokens(cfg, 60, 2)
    ref = O.forward(cfg, w, toks)
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    m = _model(cfg, w, dtype)
    eng, st = m.step_engine, m.states
    for cuts in ([60], [1] * 60, [2, 2, 3, 2, 7, 1, 1, 17, 2, 23], [31, 1, 1, 1, 26]):
        got, at = [], 0
        for c in cuts:
            got.append(eng.step([(st.slot_of("r"), toks[at:at + c])], "all"))
            at += c
        st.release("r")
        assert _within(torch.cat(got), ref, tol, dtype == torch.float32), cuts


@pytest.mark.parametrize("min_rows", [1, 10 ** 9])
def test_either_attention_form_for_every_portion_and_batch(monkeypatch, min_rows):
    """The switch between the two forms of the attention kernel is a matter of speed: with the tensor-core form forced
    for every step (single decoded tokens included), and with it switched off, the logits stay the oracle's."""
    from torchao_fork_b200._models import segment_step as S
    monkeypatch.setattr(S, "PROMPT_MIN_ROWS", min_rows)
    cfg = _tensor()
    w = O.random_weights(cfg, 29)
    ta, tb = _tokens(cfg, 75, 9), _tokens(cfg, 40, 10)
    ra, rb = O.forward(cfg, w, ta), O.forward(cfg, w, tb)
    tol = max(_bf16_tol(cfg, w, ta), _bf16_tol(cfg, w, tb))
    m = _model(cfg, w, torch.bfloat16)
    eng, st = m.step_engine, m.states
    ga = [eng.step([(st.slot_of("a"), ta[:33])], "all")]
    both = eng.step([(st.slot_of("a"), ta[33:70]), (st.slot_of("b"), tb[:38])], "all")
    ga.append(both[:37])
    gb = [both[37:]]
    for i in range(2):
        both = eng.step([(st.slot_of("b"), tb[38 + i:39 + i]), (st.slot_of("a"), ta[70 + i:71 + i])], "all")
        gb.append(both[:1])
        ga.append(both[1:])
    ga.append(eng.step([(st.slot_of("a"), ta[72:])], "all"))
    assert _within(torch.cat(ga), ra, tol) and _within(torch.cat(gb), rb, tol)


def test_pieces_cut_inside_a_step_and_both_expert_paths(monkeypatch):
    from torchao_fork_b200._models import segment_step as S
    from torchao_fork_b200._models.rutusun import step as R
    cfg = _mixed()
    w = O.random_weights(cfg, 23)
    toks = _tokens(cfg, 70, 3)
    ref = O.forward(cfg, w, toks)
    m = _model(cfg, w)
    monkeypatch.setattr(S, "MAX_STEP_TOKENS", 13)   # the step itself in pieces of 13 rows
    got = m.step_engine.step([(m.states.slot_of("b"), toks)], "all")
    assert _err(got, ref) <= F32_TOL
    both = m.step_engine.step([(m.states.slot_of("c"), toks[:40]), (m.states.slot_of("d"), toks[:9])], [[39, 3], [8]])
    assert _err(both, ref[[39, 3, 8]]) <= F32_TOL
    monkeypatch.setattr(S, "MAX_STEP_TOKENS", 4096)
    monkeypatch.setattr(S, "REC_TILE", 4)           # the matrix-state recurrences in their tiled form, 4-row tiles
    both = m.step_engine.step([(m.states.slot_of("t1"), toks[:40]), (m.states.slot_of("t2"), toks[:3])], "all")
    both2 = m.step_engine.step([(m.states.slot_of("t2"), toks[3:41]), (m.states.slot_of("t1"), toks[40:41])], "all")
    assert _err(torch.cat([both[:40], both2[38:]]), ref[:41]) <= F32_TOL and _err(torch.cat([both[40:], both2[:38]]), ref[:41]) <= F32_TOL
    monkeypatch.setattr(S, "REC_TILE", 64)
    for limit in (0, 10 ** 9):                      # experts as sorted rows around GEMMs for every step / as matrix-vector kernels
        monkeypatch.setattr(R, "MOE_GEMV_TOKENS", limit)
        got = m.step_engine.step([(m.states.slot_of(("e", limit)), toks)], "all")
        assert _err(got, ref) <= F32_TOL


@pytest.mark.parametrize("name", ["mixed", "plain", "tensor"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batches_of_unequal_requests_equal_each_alone_and_slots_are_reused(dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 24)
    reqs = {k: _tokens(cfg, n, 10 + i) for i, (k, n) in enumerate([("a", 37), ("b", 9), ("c", 21), ("d", 30), ("e", 5)])}
    ref = {k: O.forward(cfg, w, t) for k, t in reqs.items()}
    tol = F32_TOL if dtype == torch.float32 else max(_bf16_tol(cfg, w, t) for t in reqs.values())
    m = _model(cfg, w, dtype, slots=2)      # three live requests force the state to grow
    eng, st = m.step_engine, m.states
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    # every step: (request, tokens) pairs; requests end, their slots go to the next ones
    plan = [[("a", 11), ("b", 2)], [("a", 1), ("b", 7), ("c", 6)], [("c", 15), ("a", 1)], [("d", 30), ("a", 24)], [("e", 3)], [("e", 1)], [("e", 1)]]
    for step in plan:
        segs, names = [], []
        for k, c in step:
            segs.append((st.slot_of(k), reqs[k][at[k]:at[k] + c]))
            names.append((k, c))
            at[k] += c
        out = eng.step(segs, "all")
        r = 0
        for k, c in names:
            got[k].append(out[r:r + c])
            r += c
            if at[k] == len(reqs[k]):
                st.release(k)
    assert m.max_batch_size >= 3 and st.alloc.in_use == 0
    for k in reqs:
        assert at[k] == len(reqs[k])
        assert _within(torch.cat(got[k]), ref[k], tol, dtype == torch.float32), k


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_remembers_far_tokens_and_the_cache_has_an_end(dtype):
    cfg = _mixed()
    w = O.random_weights(cfg, 25)
    toks = _tokens(cfg, 150, 4)
    ref = O.forward(cfg, w, toks)
    # the first token reaches the end: another first token moves the last logits
    other = O.forward(cfg, w, [(toks[0] + 1) % cfg["vocab"]] + toks[1:])
    assert _err(other[-1:], ref[-1:]) > 1e-3
    m = _model(cfg, w, dtype, seq=150)
    eng, st = m.step_engine, m.states
    got = [eng.step([(st.slot_of("r"), toks[:20])], "all")] + [eng.step([(st.slot_of("r"), [t])], "all") for t in toks[20:]]
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    assert _within(torch.cat(got), ref, tol, dtype == torch.float32)
    with pytest.raises(RuntimeError):
        eng.step([(st.slot_of("r"), [1])], "all")     # position 150 of a cache with 150 rows


@pytest.mark.parametrize("batch", [1, 2])
def test_greedy_generation_through_generator_and_graph(batch):
    from torchao_fork_b200._models.llama.generate import Generator
    cfg = _mixed()
    w = O.random_weights(cfg, 26)
    prompt = _tokens(cfg, 13, 5)
    want = O.greedy(cfg, w, prompt, 12)
    for use_graph in (False, True):
        m = _model(cfg, w, torch.float32, slots=batch)
        gen = Generator(m, batch, 64, temperature=0.0, top_k=None, use_graph=use_graph)
        for _ in range(2):      # the second call restarts the slots at position 0
            seq = gen.generate(torch.tensor(prompt), 12)
            assert seq.shape == (batch, 25)
            for b in range(batch):
                assert seq[b, 13:].tolist() == want, (use_graph, b)


def test_sampling_with_temperature_runs_through_the_framework_sampler():
    from torchao_fork_b200._models.llama.generate import Generator
    cfg = _plain()
    m = _model(cfg, O.random_weights(cfg, 27), torch.bfloat16, slots=1)
    gen = Generator(m, 1, 40, temperature=0.8, top_k=5, use_graph=True)
    seq = gen.generate(torch.tensor(_tokens(cfg, 6, 6)), 10)
    assert seq.shape == (1, 16) and int(seq.min()) >= 0 and int(seq.max()) < cfg["vocab"]


def test_command_line_generates_from_a_checkpoint_folder_and_a_named_configuration(tmp_path):
    import importlib
    G = importlib.import_module("torchao_fork_b200._models.llama.generate")
    cfg = _mixed()
    folder = str(tmp_path / "ckpt")
    O.write_checkpoint(folder, cfg, O.random_weights(cfg, 30))
    # the calls themselves are the check: folder or name -> registry -> prefill -> graph decode -> sampling
    G.main(checkpoint_path=folder, num_samples=1, max_new_tokens=9, prompt="1,2,3,4,5", temperature=0.0, precision=torch.float32)
    G.main(random_init="Rutusun-test", num_samples=1, max_new_tokens=6, prompt="7,8,9")


def test_named_configuration_through_the_registry():
    from torchao_fork_b200._models import registry
    m = registry.random_init("Rutusun-test", "cuda", torch.bfloat16)
    m.setup_caches(1, 64)
    out = m(torch.randint(0, 512, (1, 20), device="cuda"))
    assert out.shape == (1, 1, 512) and bool(torch.isfinite(out).all())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_runner_on_a_checkpoint_folder(tmp_path, dtype):
    cfg = _mixed()
    w = O.random_weights(cfg, 28)
    folder, out = str(tmp_path / "model"), str(tmp_path / "out")
    O.write_checkpoint(folder, cfg, w)
    a, b = _tokens(cfg, 29, 7), _tokens(cfg, 12, 8)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:17], "want": [0, 16]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[17:19], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": a[19:], "want": [9]}], "end": ["a"]},
             {"step": 3, "entries": [{"id": "b", "tokens": b[:11], "want": [10]}], "end": []},
             {"step": 4, "entries": [{"id": "b", "tokens": b[11:], "want": [0]}], "end": ["b"]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                        "--max-tokens", "64", "--slots", "1"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(5)]
    assert not os.path.exists(os.path.join(out, "1.f32"))
    ra, rb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    tol = F32_TOL if dtype == "float32" else max(_bf16_tol(cfg, w, a), _bf16_tol(cfg, w, b))
    V = cfg["vocab"]
    rd = lambda i: torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, V).copy())
    got_a, got_b = torch.cat([rd(0), rd(2)]), torch.cat([rd(3), rd(4)])
    assert _within(got_a, ra[[0, 16, 28]], tol, dtype == "float32") and _within(got_b, rb[[10, 11]], tol, dtype == "float32")
