"""Fedipel on the GPU against the float64 oracle (tests/fedipel_oracle.py): every mechanism's kernel alone, then the model
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

import fedipel_oracle as O

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 1e-4
F64 = torch.float64
BF16, F32 = 0, 1      # storage types of the library (AO_LM_BF16, AO_LM_F32)


def _lm():
    from torchao_fork_b200 import _lib
    return _lib, _lib.lm()


def _st():
    return torch.cuda.current_stream().cuda_stream


def _i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def _p(t):
    return None if t is None else t.data_ptr()


def _errs(got, ref):
    """Per position: root mean square of the difference (mean over the vocabulary taken off), relative to the reference's spread."""
    got, ref = torch.as_tensor(got).double().cpu(), torch.as_tensor(ref).double().cpu()
    d = got - ref
    d = d - d.mean(-1, keepdim=True)
    r = ref - ref.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / r.pow(2).mean(-1).sqrt().clamp_min(1e-30)


def _err(got, ref):
    return float(_errs(got, ref).max())


def _within(got, ref, tol, exact=False):
    """Every position within tol.  A bfloat16 run may leave the bound at one position in fifty (at least one): where two
    experts' logits are closer than bfloat16 rounding, the run and the oracle may choose differently, which moves that
    position's logits by far more than rounding does; the positions after it must be back inside."""
    e = _errs(got, ref)
    over = int((e > tol).sum())
    return over == 0 if exact else over <= max(1, e.numel() // 50)


def _bf16_tol(cfg, w, toks):
    """A bfloat16 run may be 3 times as far from the exact logits as bfloat16 rounding alone moves them."""
    return 3.0 * O.rounding_noise(cfg, w, toks, _err)


def _model(cfg, w, dtype=torch.float32, slots=2, seq=256):
    from torchao_fork_b200._models.fedipel import Fedipel, FedipelArgs
    args = FedipelArgs.from_dict(O.config_json(cfg), {k: tuple(v.shape) for k, v in w.items()})
    m = Fedipel(args, w, "cuda", dtype).eval()
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


def _tiles(segs, tile):
    """Tiles of <= tile rows inside the segments -> (first rows, counts, per segment first tile, tile count)."""
    tf, tc, s0, sn, at = [], [], [], [], 0
    for _, _, c in segs:
        s0.append(len(tf))
        k = 0
        for r in range(0, c, tile):
            tf.append(at + r)
            tc.append(min(tile, c - r))
            k += 1
        sn.append(k)
        at += c
    return _i32(tf), _i32(tc), _i32(s0), _i32(sn)


def _close(got, ref, tol=2e-5):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max()))


def _cuts(total, sizes):
    """Portions of the given sizes, repeated, until `total` rows are covered -> [(first, rows)]."""
    out, at, i = [], 0, 0
    while at < total:
        c = min(sizes[i % len(sizes)], total - at)
        out.append((at, c))
        at, i = at + c, i + 1
    return out


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("W", [33, 256, 2500])
@pytest.mark.parametrize("parts", ["add_norm", "norm_rows", "add_only", "in_place", "both_outputs"])
def test_layer_norm_with_weighted_residual_add(W, parts):
    lib, L = _lm()
    n, eps, mult = 7, 1e-5, 0.7
    g = _gen(W)
    x, y = torch.randn(n, W, generator=g) * 3 + 0.5, torch.randn(n, W, generator=g)
    wt, b = (1 + 0.2 * torch.randn(W, generator=g)).bfloat16().float(), (0.3 * torch.randn(W, generator=g)).bfloat16().float()
    xd, yd, wd, bd = x.cuda(), y.cuda(), wt.cuda(), b.cuda()
    out = torch.zeros(n, W, device="cuda")
    wb, bb = wd.bfloat16(), bd.bfloat16()      # (every device tensor keeps a name until its kernel has run)
    if parts == "add_norm":
        lib.lm_check(L.ao_lm_add_layer_norm(_p(xd), _p(yd), mult, None, n, W, _p(wd), _p(bd), F32, eps, None, _p(out), _st()), "ln")
        xs = x.double() + mult * y.double()
        assert _close(xd, xs, 1e-6) and _close(out, O.layer_norm(xs, wt.double(), b.double(), eps))
    elif parts == "norm_rows":
        rows = [5, 0, 3]
        rd = _i32(rows)
        ob = torch.zeros(3, W, device="cuda", dtype=torch.bfloat16)
        lib.lm_check(L.ao_lm_add_layer_norm(_p(xd), None, 0.0, _p(rd), 3, W, _p(wb), _p(bb), BF16, eps, None, _p(ob), _st()), "ln")
        assert torch.equal(xd.cpu(), x) and _close(ob.float(), O.layer_norm(x.double()[rows], wt.double(), b.double(), eps), 1e-2)
    elif parts == "add_only":
        lib.lm_check(L.ao_lm_add_layer_norm(_p(xd), _p(yd), mult, None, n, W, None, None, F32, eps, None, None, _st()), "ln")
        assert _close(xd, x.double() + mult * y.double(), 1e-6)
    elif parts == "in_place":
        lib.lm_check(L.ao_lm_add_layer_norm(_p(xd), None, 0.0, None, n, W, _p(wd), _p(bd), F32, eps, _p(xd), None, _st()), "ln")
        assert _close(xd, O.layer_norm(x.double(), wt.double(), b.double(), eps))
    else:
        ob = torch.zeros(n, W, device="cuda", dtype=torch.bfloat16)
        lib.lm_check(L.ao_lm_add_layer_norm(_p(xd), _p(yd), mult, None, n, W, _p(wb), _p(bb), BF16, eps, _p(out), _p(ob), _st()), "ln")
        ref = O.layer_norm(x.double() + mult * y.double(), wt.double(), b.double(), eps)
        assert _close(out, ref) and _close(ob.float(), ref, 1e-2)


@pytest.mark.parametrize("layout,pairing", [("interleaved", 0), ("half", 1)])
@pytest.mark.parametrize("d,dims", [(8, 8), (12, 4), (16, 0), (7, 6)])
def test_rotation_of_a_projection_row_both_pairings_partial_and_none(layout, pairing, d, dims):
    lib, L = _lm()
    n, Ha, Hb, base = 9, 3, 2, 700.0
    g = _gen(d * 10 + dims)
    ld = (Ha + Hb) * d + 5
    proj = torch.randn(n, ld, generator=g)
    pos = [0, 1, 2, 40, 41, 1000, 1001, 7, 8]
    inv = (base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / max(dims, 1))).float().cuda() if dims else None
    pd, posd = proj.cuda(), _i32(pos)
    lib.lm_check(L.ao_lm_rotary_rows(_p(pd), ld, n, _p(posd), _p(inv), dims, pairing, d, 2, Ha, 1.0, 2 + Ha * d, Hb, 0.25, _st()), "rot")
    a = O.rotate(proj[:, 2:2 + Ha * d].double().view(n, Ha, d), torch.tensor(pos), dims, base, layout)
    b = O.rotate(proj[:, 2 + Ha * d:2 + (Ha + Hb) * d].double().view(n, Hb, d), torch.tensor(pos), dims, base, layout) * 0.25
    assert _close(pd[:, 2:2 + Ha * d].view(n, Ha, d), a, 1e-4) and _close(pd[:, 2 + Ha * d:2 + (Ha + Hb) * d].view(n, Hb, d), b, 1e-4)
    assert torch.equal(pd[:, :2].cpu(), proj[:, :2]) and torch.equal(pd[:, 2 + (Ha + Hb) * d:].cpu(), proj[:, 2 + (Ha + Hb) * d:])


def _time_mix(r, k, v, z, w0, u, h, cuts, tile, slots=3, slot=2, dt=F32):
    """channel_recurrence over one sequence cut into portions (each its own launch) -> ([T][H][dv], saved shift row).
    tile > 0: portions longer than a tile run in the tiled form."""
    lib, L = _lm()
    T, H, d = r.shape
    dv = v.shape[-1]
    state = torch.full((slots, H, d, dv), 7.0, device="cuda")          # a reused slot holds rubbish: position 0 must not read it
    shift = torch.full((slots, h.shape[1]), 5.0, device="cuda")
    cast = (lambda t: t.cuda().bfloat16()) if dt == BF16 else (lambda t: t.cuda().float())
    w0d, ud = cast(w0), cast(u)
    outs = []
    for a, c in cuts:
        sl = slice(a, a + c)
        rd, kd, vd, zd, hd = (t[sl].float().cuda().contiguous() for t in (r, k, v, z, h))
        seg = [(slot, a, c)]
        sd, pd, _, _, sf, sc = _rows(seg)
        out = torch.zeros(c, H * dv, device="cuda")
        if tile and c > tile:
            tf, tc, s0, sn = _tiles(seg, tile)
            ws = torch.zeros(int(L.ao_lm_channel_recurrence_workspace_bytes(len(tf), c, H, d, dv)) // 4, device="cuda")
            args = (_p(tf), _p(tc), len(tf), _p(s0), _p(sn), 1, c, _p(ws))
        else:
            args = (_p(sf), _p(sc), 1, None, None, 0, c, None)
        lib.lm_check(L.ao_lm_channel_recurrence(_p(rd), H * d, _p(kd), H * d, _p(vd), H * dv, _p(zd), H * d, _p(w0d), _p(ud), dt, H, d, dv,
                                                _p(state), _p(sd), _p(pd), *args, _p(hd), _p(shift), h.shape[1], _p(out), H * dv, _st()),
                     "channel_recurrence")
        outs.append(out)
    assert float(state[:slot].min()) == 7.0 and float(shift[:slot].min()) == 5.0      # other slots untouched
    return torch.cat(outs).view(T, H, dv), shift[slot]


@pytest.mark.parametrize("H,d,dv", [(2, 16, 16), (3, 5, 7), (1, 64, 64), (2, 128, 32), (1, 40, 70)])
def test_time_mixing_recurrence_both_forms_in_portions(H, d, dv):
    T, Wh = 75, 11
    g = _gen(H * 100 + d)
    r, k = torch.randn(T, H, d, generator=g, dtype=F64), torch.randn(T, H, d, generator=g, dtype=F64) / math.sqrt(d)
    v = torch.randn(T, H, dv, generator=g, dtype=F64)
    z = torch.randn(T, H, d, generator=g, dtype=F64)
    w0 = (torch.randn(H * d, generator=g) - 1.5).bfloat16().double()
    u = (0.3 + 0.4 * torch.randn(H, d, generator=g)).bfloat16().double()
    h = torch.randn(T, Wh, generator=g, dtype=F64)
    dec = torch.exp(-torch.exp(z.float().double() + w0.view(H, d)))
    ref = O.wkv_recurrence(r.float().double(), k.float().double(), v.float().double(), dec, u)
    for cuts, tile in ([(0, T)], 0), ([(0, T)], 16), (_cuts(T, [1]), 0), (_cuts(T, [2, 17, 1, 33]), 16), (_cuts(T, [40, 3]), 7):
        got, saved = _time_mix(r, k, v, z.view(T, H * d), w0, u, h, cuts, tile)
        assert _close(got, ref, 2e-5), (cuts[:3], tile)
        assert torch.equal(saved.cpu(), h[-1].float())
    got, _ = _time_mix(r, k, v, z.view(T, H * d), w0, u, h, _cuts(T, [9, 30]), 16, dt=BF16)   # bf16 only stores w0 and the bonus
    assert _close(got, ref, 2e-5)


def test_time_mixing_keeps_a_slow_channel_and_forgets_a_fast_one():
    """One key channel barely decays, another is gone after a token: after 300 tokens the first token's value is still read
    through the slow channel and nothing of it through the fast one; the bonus reaches the current token only."""
    T, H, d = 300, 1, 4
    r, k, v, z = torch.zeros(T, H, d, dtype=F64), torch.zeros(T, H, d, dtype=F64), torch.zeros(T, H, d, dtype=F64), torch.zeros(T, H * d, dtype=F64)
    z[:, 0], z[:, 1] = -12.0, 3.0              # decays exp(-exp(-12)) ~ 1 and exp(-exp(3)) ~ 2e-9
    k[0, 0, :2], v[0, 0] = 1.0, torch.tensor([1.0, 2.0, 3.0, 4.0])
    r[:, 0, 0], r[2, 0, 1], r[0, 0, 1] = 1.0, 1.0, 1.0
    u = torch.zeros(H, d, dtype=F64)
    u[0, 1] = 0.5
    for cuts, tile in ([(0, T)], 64), (_cuts(T, [1]), 0), (_cuts(T, [63, 2]), 16):
        got, _ = _time_mix(r, k, v, z, torch.zeros(H * d, dtype=F64), u, torch.zeros(T, 3, dtype=F64), cuts, tile)
        assert _close(got[0, 0], v[0, 0] * 0.5, 1e-6)                        # only the bonus: the state was empty
        assert _close(got[1, 0], v[0, 0], 1e-6)                              # the state before any decay, read through the slow channel
        assert _close(got[2, 0], v[0, 0] * (math.exp(-math.exp(-12.0)) + math.exp(-math.exp(3.0))), 1e-5)   # fast channel gone
        assert _close(got[T - 1, 0], v[0, 0] * math.exp(-math.exp(-12.0) * (T - 2)), 1e-5)


@pytest.mark.parametrize("W", [24, 130])
def test_token_shift_blends_with_the_row_in_front_across_portions_and_slots(W):
    lib, L = _lm()
    g = _gen(W)
    n_mix = 5
    mu = torch.rand(n_mix, W, generator=g).bfloat16()
    a, b = torch.randn(9, W, generator=g), torch.randn(4, W, generator=g)
    state = torch.full((3, W), 9.0, device="cuda")

    def run(segs, h):
        sd, pd, bd, _, _, _ = _rows(segs)
        n = h.shape[0]
        out = torch.zeros(n_mix, n, W, device="cuda")
        hd, mud = h.cuda(), mu.float().cuda()
        lib.lm_check(L.ao_lm_token_shift_mix(_p(hd), _p(mud), n_mix, F32, _p(state), _p(sd), _p(pd), _p(bd), n, W, _p(out),
                                             _st()), "token_shift_mix")
        return out.cpu().double()

    def ref(h):
        prev = torch.cat([torch.zeros(1, W), h[:-1]], 0).double()
        return torch.stack([h.double() + (prev - h.double()) * mu[s].double() for s in range(n_mix)], 0)

    # two sequences in one step, both from position 0 (their slots hold rubbish that must not be read)
    got = run([(1, 0, 5), (2, 0, 4)], torch.cat([a[:5], b]))
    assert _close(got[:, :5], ref(a)[:, :5], 1e-6) and _close(got[:, 5:], ref(b), 1e-6)
    # sequence a continues from the row that the layer's recurrence saved for its slot
    state[1] = a[4].cuda()
    got = run([(1, 5, 4)], a[5:])
    assert _close(got, ref(a)[:, 5:], 1e-6)


@pytest.mark.parametrize("H,d,dv,dims", [(2, 16, 16, 16), (3, 8, 12, 4), (1, 32, 8, 0)])
def test_retention_rotation_recurrence_and_unit_rms_gate_in_portions(H, d, dv, dims):
    """The retention mixer between its two projections: rotate -> recurrence with a fixed decay per head -> unit RMS per head
    times SiLU of the gate, over a sequence cut into portions on a reused slot."""
    lib, L = _lm()
    T, base, eps = 70, 200.0, 1e-5
    g = _gen(H + d + dims)
    ld = 2 * H * d + 2 * H * dv
    proj = torch.randn(T, ld, generator=g)
    decay = [1.0 - 2.0 ** -(2 + 3 * hh) for hh in range(H)]
    pos = torch.arange(T)
    q = O.rotate(proj[:, :H * d].double().view(T, H, d), pos, dims, base, "half")
    k = O.rotate(proj[:, H * d:2 * H * d].double().view(T, H, d), pos, dims, base, "half") * d ** -0.5
    v, gate = proj[:, 2 * H * d:2 * H * d + H * dv].double().view(T, H, dv), proj[:, 2 * H * d + H * dv:].double()
    ref = O.unit_rms(O.retention_recurrence(q, k, v, decay), eps).reshape(T, H * dv) * O.silu(gate)
    inv = (base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / max(dims, 1))).float().cuda() if dims else None
    dec = torch.tensor(decay, device="cuda")
    for cuts, tile in ([(0, T)], 0), ([(0, T)], 16), (_cuts(T, [1, 2, 31]), 16):
        state = torch.full((2, H, d, dv), 3.0, device="cuda")
        outs = []
        for a, c in cuts:
            pd_ = proj[a:a + c].cuda().contiguous()
            seg = [(1, a, c)]
            sd, pd, _, _, sf, sc = _rows(seg)
            lib.lm_check(L.ao_lm_rotary_rows(_p(pd_), ld, c, _p(pd), _p(inv), dims, 1, d, 0, H, 1.0, H * d, H, d ** -0.5, _st()), "rot")
            rec = torch.zeros(c, H * dv, device="cuda")
            base_ptr = pd_.data_ptr()
            if tile and c > tile:
                tf, tc, s0, sn = _tiles(seg, tile)
                ws = torch.zeros(int(L.ao_lm_outer_recurrence_workspace_bytes(len(tf), c, H, d, dv)) // 4, device="cuda")
                args = (_p(tf), _p(tc), len(tf), _p(s0), _p(sn), 1, c, _p(ws))
            else:
                args = (_p(sf), _p(sc), 1, None, None, 0, c, None)
            lib.lm_check(L.ao_lm_outer_recurrence(base_ptr, ld, base_ptr + 4 * H * d, ld, base_ptr + 8 * H * d, ld, 0, None, None, H, _p(dec),
                                                  None, H, H, d, dv, _p(state), _p(sd), _p(pd), *args, _p(rec), H * dv, _st()), "rec")
            o = torch.zeros(c, H * dv, device="cuda")
            lib.lm_check(L.ao_lm_gated_group_norm(_p(rec), H * dv, base_ptr + 4 * (2 * H * d + H * dv), ld, 2, c, H * dv, H, None, F32, eps,
                                                  _p(o), _st()), "ggn")
            outs.append(o)
        assert _close(torch.cat(outs), ref, 1e-4), (cuts[:3], tile)


def _window_run(q, k, v, cuts, window, keep, scale, lam, ring, first_rows, dtype, slot=1, slots=3, eps=1e-5, out_scale=1.0, unit=1, n_split=1,
                tensor=False):
    """window_attention over one sequence cut into portions: prep-less (q, k, v are given rotated), every portion attends
    over the slot's ring / first-token store and its own rows, then its rows are appended.  -> [T][H][dv] fp32.
    tensor: the tensor-core form for prompt portions (bf16)."""
    lib, L = _lm()
    T, H, M, d = q.shape
    G, dv = k.shape[1], v.shape[-1]
    tdt, dt = (torch.bfloat16, BF16) if dtype == torch.bfloat16 else (torch.float32, F32)
    tr = __import__("ctypes").c_int()
    plan = L.ao_lm_window_attention_prompt_plan if tensor else L.ao_lm_window_attention_plan
    lib.lm_check(plan(dt, M, H, G, d, dv, __import__("ctypes").byref(tr)), "plan")
    assert tr.value > 0
    rk = torch.full((slots, ring, G * M * d), 50.0, device="cuda", dtype=tdt)       # rubbish that a fresh sequence must not see
    rv = torch.full((slots, ring, G * dv), 50.0, device="cuda", dtype=tdt)
    fk = torch.full((slots, max(1, first_rows), G * M * d), 50.0, device="cuda", dtype=tdt)
    fv = torch.full((slots, max(1, first_rows), G * dv), 50.0, device="cuda", dtype=tdt)
    outs = []
    for a, c in cuts:
        seg = [(slot, a, c)]
        sd, pd, bd, ad, _, _ = _rows(seg)
        tf, tc, _, _ = _tiles(seg, tr.value)
        qd = q[a:a + c].float().cuda().contiguous()
        kd, vd = k[a:a + c].cuda().to(tdt).contiguous(), v[a:a + c].cuda().to(tdt).contiguous()
        o = torch.zeros(c, H * dv, device="cuda", dtype=tdt)
        ws = torch.zeros(max(16, int(L.ao_lm_window_attention_workspace_bytes(len(tf), M, H, G, dv, n_split))), device="cuda", dtype=torch.uint8)
        common = (_p(qd), _p(kd), _p(vd), _p(rk), _p(rv), _p(fk), _p(fv), ring, first_rows, dt, _p(sd), _p(pd), _p(bd), _p(tf), _p(tc), len(tf),
                  M, H, G, d, dv, window, keep, scale, lam, unit, eps, out_scale)
        if tensor:
            lib.lm_check(L.ao_lm_window_attention_prompt(*common, _p(o), H * dv, _st()), "window_attention_prompt")
        else:
            lib.lm_check(L.ao_lm_window_attention(*common, n_split, _p(ws), ws.numel(), _p(o), H * dv, _st()), "window_attention")
        lib.lm_check(L.ao_lm_window_append(_p(kd), _p(vd), c, G * M * d, G * dv, ring, first_rows, dt, _p(sd), _p(pd), _p(ad), _p(rk), _p(rv),
                                           _p(fk), _p(fv), _st()), "window_append")
        outs.append(o.float())
    assert float(rk[:slot].float().min()) == 50.0 and float(fv[slot + 1:].float().min()) == 50.0
    return torch.cat(outs).view(T, H, dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,M,d,dv,window,keep", [(4, 2, 2, 8, 12, 9, 2), (3, 1, 2, 5, 7, 4, 0), (2, 2, 1, 16, 40, 13, 5), (6, 2, 2, 24, 33, 1, 1),
                                                    (1, 1, 2, 64, 128, 20, 30), (16, 1, 2, 8, 8, 6, 1), (40, 2, 2, 8, 8, 7, 2)])
def test_window_attention_whole_portions_and_decoding(dtype, H, G, M, d, dv, window, keep):
    T, scale, lam = 61, 0.4, 0.6
    g = _gen(H * 31 + d)
    rnd = lambda *s: torch.randn(*s, generator=g).to(dtype).double()       # values that the storage type holds exactly
    q, k, v = torch.randn(T, H, M, d, generator=g).double(), rnd(T, G, M, d), rnd(T, G, dv)
    q = q.float().double()
    ref = O.window_diff_attention(q, k, v, scale, window, keep, lam, 1e-5) * 0.7
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for cuts, ring, ns in (([(0, T)], window, 1), (_cuts(T, [1]), window, 1), (_cuts(T, [2, 7, 1, 19]), window + 3, 1),
                           (_cuts(T, [25, 1, 1]), max(window, keep) + 40, 1), (_cuts(T, [1]), window + 2, 2), (_cuts(T, [9, 1, 3]), window, 5),
                           ([(0, T)], window, 64)):      # key splits: some shares see no key at all
        got = _window_run(q, k, v, cuts, window, keep, scale, lam, ring, keep + (ring % 3), dtype, out_scale=0.7, n_split=ns)
        assert _close(got, ref, tol), (cuts[:3], ring, ns)


@pytest.mark.parametrize("H,G,M,d,dv,window,keep", [(4, 2, 2, 16, 32, 9, 2), (2, 1, 2, 64, 128, 70, 5), (3, 3, 1, 32, 16, 150, 0), (2, 2, 2, 48, 96, 1, 1),
                                                    (2, 1, 2, 16, 48, 64, 64)])
def test_window_attention_tensor_core_form_for_prompt_portions(H, G, M, d, dv, window, keep):
    T, scale, lam = 200, 0.3, 0.6
    g = _gen(H * 7 + d)
    rnd = lambda *s: torch.randn(*s, generator=g).bfloat16().double()
    q, k, v = rnd(T, H, M, d), rnd(T, G, M, d), rnd(T, G, dv)      # bf16 values: the operands of the tensor-core products are exact
    ref = O.window_diff_attention(q, k, v, scale, window, keep, lam, 1e-5) * 0.7
    for cuts, ring in ([(0, T)], window), (_cuts(T, [64, 1, 70, 17]), window + 5), (_cuts(T, [130, 3]), max(window, keep) + 100):
        got = _window_run(q, k, v, cuts, window, keep, scale, lam, ring, keep + 1, torch.bfloat16, out_scale=0.7, tensor=True)
        assert _close(got, ref, 1e-2), (cuts[:3], ring)     # what is left is the bf16 rounding of the result


@pytest.mark.parametrize("how", ["whole", "portions", "decoded", "tensor"])
@pytest.mark.parametrize("key,query,seen", [(0, 99, True), (2, 99, True), (3, 99, False), (60, 99, True), (59, 99, False), (99, 99, True),
                                            (100, 99, False), (3, 42, True), (40, 79, True), (39, 79, False), (2, 150, True), (111, 150, True),
                                            (110, 150, False)])
def test_window_attention_one_dominant_key_inside_and_outside_the_window_and_the_kept_tokens(how, key, query, seen):
    """Window 40, first 3 tokens kept.  One key matches one query so strongly that, when the mask lets the query see it, map 1
    returns that key's value; map 2 is uniform.  A key one step outside the window, the first token that is not kept, or a
    key in the future must leave no trace."""
    T, H, G, d, dv, window, keep = 151, 2, 1, 16, 16, 40, 3
    g = _gen(5)
    q, k = torch.zeros(T, H, 2, d, dtype=F64), torch.zeros(T, G, 2, d, dtype=F64)
    v = torch.randn(T, G, dv, generator=g, dtype=F64).float().double()
    mark = torch.zeros(d, dtype=F64)
    mark[3] = 1.0
    q[query, :, 0], k[key, 0, 0] = 30.0 * mark, 30.0 * mark
    cuts = {"whole": [(0, T)], "portions": _cuts(T, [37, 2, 5]), "decoded": [(0, 38)] + [(i, 1) for i in range(38, T)],
            "tensor": _cuts(T, [70, 17])}[how]
    if how == "tensor":
        v = v.bfloat16().double()
        got = _window_run(q, k, v, cuts, window, keep, 1.0, 0.0, 45, 4, torch.bfloat16, unit=0, tensor=True)[query, 0]
        lo = max(0, query - window + 1)
        visible = sorted(set(range(min(keep, query + 1))) | set(range(lo, query + 1)))
        assert _close(got, v[key, 0] if seen else v[visible, 0].mean(0), 1e-2), (key, query)
        return
    got = _window_run(q, k, v, cuts, window, keep, 1.0, 0.0, 45, 4, torch.float32, unit=0, n_split=3 if how == "decoded" else 1)[query, 0]
    lo = max(0, query - window + 1)
    visible = sorted(set(range(min(keep, query + 1))) | set(range(lo, query + 1)))
    mean = v[visible, 0].mean(0)
    if seen:
        assert _close(got, v[key, 0], 1e-4), (key, query)
    else:
        assert _close(got, mean, 1e-4), (key, query)


@pytest.mark.parametrize("H,G,d,dv,dims,own", [(4, 2, 8, 12, 4, True), (3, 1, 6, 5, 6, True), (2, 2, 16, 8, 0, True), (4, 2, 8, 12, 8, False)])
def test_query_key_value_preparation_biases_and_rotation_of_both_maps(H, G, d, dv, dims, own):
    lib, L = _lm()
    n, base = 6, 900.0
    g = _gen(H + d + dims)
    ld = 2 * H * d + (2 * G * d + G * dv if own else 0) + 3
    proj = torch.randn(n, ld, generator=g)
    qb, kb, vb = (torch.randn(s, generator=g).bfloat16() for s in (2 * H * d, 2 * G * d, G * dv))
    pos = [0, 1, 5, 300, 301, 17]
    inv = (base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / max(dims, 1))).float().cuda() if dims else None
    qn = torch.zeros(n, 2 * H, d, device="cuda")
    kn, vn = torch.zeros(n, 2 * G, d, device="cuda", dtype=torch.bfloat16), torch.zeros(n, G * dv, device="cuda", dtype=torch.bfloat16)
    ko, vo = 1 + 2 * H * d, 1 + 2 * H * d + 2 * G * d
    pd, qbd, kbd, vbd, posd = proj.cuda(), qb.cuda(), kb.cuda(), vb.cuda(), _i32(pos)
    lib.lm_check(L.ao_lm_qkv_rotary_prep(_p(pd), ld, 1, ko, vo, _p(qbd), _p(kbd) if own else None,
                                         _p(vbd) if own else None, _p(posd), _p(inv), dims, 0, n, 2 * H, 2 * G if own else 0, d,
                                         G * dv, BF16, _p(qn), _p(kn) if own else None, _p(vn) if own else None, _st()), "prep")
    p = torch.tensor(pos)
    rq = O.rotate((proj[:, 1:ko].double() + qb.double()).view(n, 2 * H, d), p, dims, base, "interleaved")
    assert _close(qn, rq, 1e-4)
    if own:
        rk = O.rotate((proj[:, ko:vo].double() + kb.double()).view(n, 2 * G, d), p, dims, base, "interleaved")
        assert _close(kn.float(), rk, 1e-2) and _close(vn.float(), proj[:, vo:vo + G * dv].double() + vb.double(), 1e-2)


@pytest.mark.parametrize("E,top,extra", [(8, 4, True), (5, 5, False), (1, 1, True), (70, 3, True)])
def test_router_softmax_over_the_chosen_logits_only_with_bias_and_gate(E, top, extra):
    lib, L = _lm()
    n = 19
    g = _gen(E)
    ld = E + (1 if extra else 0) + 2
    z = torch.randn(n, ld, generator=g) * 2
    bias = torch.randn(E, generator=g)
    idx, wt = torch.zeros(n, top, dtype=torch.int32, device="cuda"), torch.zeros(n, top, device="cuda")
    gate = torch.zeros(n, device="cuda")
    zd, bd = z.cuda(), bias.cuda()
    lib.lm_check(L.ao_lm_router_topk_renorm_logits(_p(zd), ld, _p(bd), n, E, top, E if extra else -1, _p(idx), _p(wt),
                                                   _p(gate) if extra else None, _st()), "router")
    zz = z[:, :E].double() + bias.double()
    val, ref_idx = torch.topk(zz, top, dim=-1)
    assert torch.equal(idx.cpu().long(), ref_idx) and _close(wt, torch.softmax(val, -1), 1e-6)
    assert abs(float(wt.sum(-1).min()) - 1.0) < 1e-5
    if extra:
        assert _close(gate, torch.sigmoid(z[:, E].double()), 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_squared_relu_units_tanh_and_soft_cap(dtype):
    lib, L = _lm()
    from torchao_fork_b200._models.experts import act_unit, chosen_experts
    dt = BF16 if dtype == torch.bfloat16 else F32
    n, W, ff, E, top = 5, 24, 40, 6, 2
    g = _gen(3)
    h = torch.randn(n, W, generator=g).to(dtype)
    wu, wd = (torch.randn(E, ff, W, generator=g) / 4).to(dtype), (torch.randn(E, W, ff, generator=g) / 6).to(dtype)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).int()
    wt, scale = torch.rand(n, top, generator=g), torch.rand(n, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    ref = torch.zeros(n, W, dtype=F64)
    for t in range(n):
        for c in range(top):
            e = int(idx[t, c])
            ref[t] += wt[t, c].double() * O.relu2_unit(h[t:t + 1].double(), wu[e].double(), wd[e].double())[0]
    shared = O.relu2_unit(h.double(), wu[0].double(), wd[0].double()) * scale.double()[:, None]
    for gemv in (True, False):
        out, _ = act_unit(L, dt, h.cuda(), wu[0].cuda(), wd[0].cuda(), scale.cuda(), _st())
        assert out.dtype == torch.float32 and _close(out, shared, tol)
        chosen_experts(L, dt, h.cuda(), idx.cuda(), wt.cuda(), wu.cuda(), wd.cuda(), out, float("inf"), 1.0, 0.0, gemv, True, _st(), gated=False)
        assert _close(out, shared + ref, tol), gemv
        out2 = torch.full((n, W), 9.0, device="cuda")
        chosen_experts(L, dt, h.cuda(), idx.cuda(), wt.cuda(), wu.cuda(), wd.cuda(), out2, float("inf"), 1.0, 0.0, gemv, False, _st(), gated=False)
        assert _close(out2, ref, tol), gemv
    z = (torch.randn(n, 50, generator=g) * 20).cuda()
    t = torch.zeros(n, 50, device="cuda", dtype=dtype)
    lib.lm_check(L.ao_lm_unary_rows(_p(z), F32, n, 50, 1, 0.0, None, 0, _p(t), dt, _st()), "tanh")
    assert _close(t.float(), torch.tanh(z.double()), 1e-6 if dtype == torch.float32 else 1e-2)
    lib.lm_check(L.ao_lm_unary_rows(_p(z), F32, n, 50, 2, 12.5, None, 0, _p(z), F32, _st()), "softcap")       # in place
    assert float(z.abs().max()) <= 12.5


def test_soft_cap_values():
    lib, L = _lm()
    z = torch.linspace(-80, 80, 331).view(1, -1)
    zd = z.cuda()
    lib.lm_check(L.ao_lm_unary_rows(_p(zd), F32, 1, z.shape[1], 2, 12.5, None, 0, _p(zd), F32, _st()), "softcap")
    assert _close(zd, 12.5 * torch.tanh(z.double() / 12.5), 1e-6)


@pytest.mark.parametrize("weight", [False, True])
def test_unit_rms_per_head_times_silu_gate(weight):
    lib, L = _lm()
    n, H, dv, eps = 6, 3, 10, 1e-5
    g = _gen(1)
    y, gate = torch.randn(n, H * dv, generator=g) * 4, torch.randn(n, H * dv, generator=g)
    wt = (1 + 0.3 * torch.randn(H * dv, generator=g)).bfloat16() if weight else None
    out = torch.zeros(n, H * dv, device="cuda", dtype=torch.bfloat16)
    yd, gd, wd = y.cuda(), gate.cuda(), wt.cuda() if weight else None
    lib.lm_check(L.ao_lm_gated_group_norm(_p(yd), H * dv, _p(gd), H * dv, 2, n, H * dv, H, _p(wd),
                                          BF16, eps, _p(out), _st()), "ggn")
    ref = O.unit_rms(y.double().view(n, H, dv), eps).reshape(n, H * dv) * (wt.double() if weight else 1.0) * O.silu(gate.double())
    assert _close(out.float(), ref, 1e-2)


# ------------------------------------------------------------------------------------------------ the model
def _mixed():     # every mixer and both feed-forwards; a layer without feed-forward; a layer that borrows keys and values under a mask of its own
    return O.model_config([O.retention_layer(mlp=O.dense()), O.attention_layer(mlp=O.mixture()), O.wkv_layer(mlp=None),
                           O.attention_layer(kv_from=1, size=5, keep=3, scale=0.3, diff=0.6, mlp=O.mixture(experts=4, top=3, shared=0)),
                           O.retention_layer(heads=2, dim=12, vdim=6, rot=4, mlp=O.dense(24))])


def _time_first():    # time mixing first and last; attention without rotation or kept tokens; no soft cap, residual weight 1
    return O.model_config([O.wkv_layer(heads=3, dim=8, rank=3, mlp=O.mixture(experts=5, top=1, ff=8, shared=8)),
                           O.attention_layer(heads=2, kv_heads=2, dim=6, vdim=10, size=7, keep=0, rot=0, mlp=None),
                           O.retention_layer(heads=1, dim=16, vdim=16, rot=0, decay=[1.0], mlp=O.dense(16)),
                           O.wkv_layer(heads=1, dim=24, rank=24, mlp=O.dense(48))], width=24, vocab=50, mult=1.0, softcap=0)


def _ones():      # sizes that are 1 or equal: one head everywhere, one expert, a window of one token
    return O.model_config([O.attention_layer(heads=1, kv_heads=1, dim=16, vdim=16, size=1, keep=1, rot=16, mlp=O.mixture(experts=1, top=1, ff=16, shared=16)),
                           O.retention_layer(heads=1, dim=16, vdim=16, rot=16, mlp=O.dense(16)),
                           O.wkv_layer(heads=1, dim=16, rank=1, mlp=O.dense(16)),
                           O.attention_layer(heads=1, kv_heads=1, dim=16, vdim=16, size=16, keep=16, rot=16, kv_from=0, mlp=None)], width=16, vocab=16)


def _odd():       # odd sizes everywhere; the borrower's window and kept tokens exceed the owner's
    return O.model_config([O.attention_layer(heads=3, kv_heads=1, dim=5, vdim=7, size=3, keep=1, rot=2, mlp=O.mixture(experts=7, top=3, ff=11, shared=13)),
                           O.wkv_layer(heads=3, dim=7, rank=5, mlp=O.dense(29)),
                           O.attention_layer(heads=3, kv_heads=1, dim=5, vdim=7, size=11, keep=4, rot=2, kv_from=0, mlp=O.dense(9)),
                           O.retention_layer(heads=3, dim=5, vdim=9, rot=2, mlp=None)], width=27, vocab=31, eps=1e-3, mult=1.3, softcap=4.0)


def _wide():      # a window that no test sequence outgrows, many kept tokens, head shapes of a real layer
    return O.model_config([O.attention_layer(heads=4, kv_heads=1, dim=32, vdim=64, size=1000, keep=40, rot=32, scale=0.2, mlp=O.dense(64)),
                           O.wkv_layer(heads=1, dim=64, rank=8, mlp=O.mixture(experts=8, top=8, ff=24, shared=24))], width=64, vocab=97)


CONFIGS = {"mixed": _mixed, "time_first": _time_first, "ones": _ones, "odd": _odd, "wide": _wide}


@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_prompt_and_every_layer_against_oracle(name, dtype):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 21)
    toks = _tokens(cfg, 45, 1)
    layers = []
    ref = O.forward(cfg, w, toks, layers_out=layers)
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
    whole = eng.step([(st.slot_of("w"), toks)], "all")
    assert _within(whole, ref, tol, dtype == torch.float32)
    one = torch.cat([eng.step([(st.slot_of("o"), [t])], "all") for t in toks])
    assert _within(one, ref, tol, dtype == torch.float32)
    st.release("w")
    for sizes in ([2], [7, 1, 2, 23], [33, 2]):
        got = torch.cat([eng.step([(st.slot_of("p"), toks[a:a + c])], "all") for a, c in _cuts(len(toks), sizes)])
        assert _within(got, ref, tol, dtype == torch.float32), sizes
        if dtype == torch.float32:
            assert _err(got, whole) < 5e-5      # the same sums, in another order at most
        st.release("p")


@pytest.mark.parametrize("min_rows", [1, 1000])
def test_either_attention_form_for_every_portion_and_batch(monkeypatch, min_rows):
    """bf16 with head sizes that both attention kernels cover: every step attends with the tensor-core form (min_rows 1, also
    single decoded tokens) or with the fp32 form (min_rows 1000, also long portions)."""
    import torchao_fork_b200._models.segment_step as S
    monkeypatch.setattr(S, "PROMPT_MIN_ROWS", min_rows)
    cfg = _wide()
    cfg["layers"][0]["mixer"]["mask"] = {"size": 50, "keep_first": 3}
    w = O.random_weights(cfg, 29)
    a, b = _tokens(cfg, 140, 3), _tokens(cfg, 30, 4)
    ra, rb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    tol = max(_bf16_tol(cfg, w, a), _bf16_tol(cfg, w, b))
    m = _model(cfg, w, torch.bfloat16, slots=2)
    eng, st = m.step_engine, m.states
    g1 = eng.step([(st.slot_of("a"), a[:100]), (st.slot_of("b"), b[:5])], "all")
    g2 = eng.step([(st.slot_of("b"), b[5:6]), (st.slot_of("a"), a[100:101])], "all")
    g3 = eng.step([(st.slot_of("a"), a[101:]), (st.slot_of("b"), b[6:])], "all")
    assert _within(torch.cat([g1[:100], g2[1:], g3[:39]]), ra, tol) and _within(torch.cat([g1[100:], g2[:1], g3[39:]]), rb, tol)


def test_pieces_cut_inside_a_step_both_recurrence_forms_and_both_expert_paths(monkeypatch):
    import torchao_fork_b200._models.segment_step as S
    import torchao_fork_b200._models.fedipel.step as FS
    cfg = _mixed()
    w = O.random_weights(cfg, 23)
    toks = _tokens(cfg, 150, 3)
    ref = O.forward(cfg, w, toks)
    for max_step, rec_tile, gemv in ((4096, 64, 16), (37, 64, 16), (4096, 8, 1000), (50, 1000, 0)):
        monkeypatch.setattr(S, "MAX_STEP_TOKENS", max_step)
        monkeypatch.setattr(S, "REC_TILE", rec_tile)
        monkeypatch.setattr(FS, "MOE_GEMV_TOKENS", gemv)
        for dtype in (torch.float32, torch.bfloat16):
            m = _model(cfg, w, dtype)
            got = m.step_engine.step([(m.states.slot_of("a"), toks)], "all")
            tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
            assert _within(got, ref, tol, dtype == torch.float32), (max_step, rec_tile, gemv, dtype)


@pytest.mark.parametrize("name", ["mixed", "odd"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_batches_of_unequal_requests_equal_each_alone_and_slots_are_reused(dtype, name):
    cfg = CONFIGS[name]()
    w = O.random_weights(cfg, 24)
    a, b, c = _tokens(cfg, 50, 4), _tokens(cfg, 21, 5), _tokens(cfg, 33, 6)
    ra, rb, rc = O.forward(cfg, w, a), O.forward(cfg, w, b), O.forward(cfg, w, c)
    tol = F32_TOL if dtype == torch.float32 else max(_bf16_tol(cfg, w, a), _bf16_tol(cfg, w, c))
    exact = dtype == torch.float32
    m = _model(cfg, w, dtype, slots=2)
    eng, st = m.step_engine, m.states
    # a prompt portion of one request beside single decoded tokens of another, request b finishes and c takes its slot
    g1 = eng.step([(st.slot_of("a"), a[:30]), (st.slot_of("b"), b[:20])], "all")
    assert _within(g1[:30], ra[:30], tol, exact) and _within(g1[30:], rb[:20], tol, exact)
    g2 = eng.step([(st.slot_of("b"), b[20:]), (st.slot_of("a"), a[30:33])], "all")
    assert _within(g2[:1], rb[20:], tol, exact) and _within(g2[1:], ra[30:33], tol, exact)
    slot_b = st.slot_of("b")
    st.release("b")
    assert st.slot_of("c") == slot_b                       # the freed slot, with b's state still in it
    g3 = eng.step([(st.slot_of("a"), a[33:34]), (st.slot_of("c"), c[:31])], "all")
    assert _within(g3[:1], ra[33:34], tol, exact) and _within(g3[1:], rc[:31], tol, exact)
    g4 = eng.step([(st.slot_of("c"), c[31:]), (st.slot_of("a"), a[34:])], "all")
    assert _within(g4[:2], rc[31:], tol, exact) and _within(g4[2:], ra[34:], tol, exact)
    # a third live request makes the state manager double its slots; the old ones keep their state
    d = _tokens(cfg, 9, 7)
    g5 = eng.step([(st.slot_of("d"), d)], "all")
    assert m.max_batch_size == 4 and _within(g5, O.forward(cfg, w, d), tol, exact)


def test_retention_remembers_the_first_token_after_hundreds():
    """A head whose decay is 1 - 2^-12 still reads most of the first token's value after 400 tokens, a head whose decay is
    0.5 nothing; decoded one by one, in portions and in the tiled form."""
    lib, L = _lm()
    T, H, d, dv = 400, 2, 4, 4
    q, k, v = torch.zeros(T, H, d), torch.zeros(T, H, d), torch.zeros(T, H, dv)
    k[0, :, 1], q[T - 1, :, 1] = 1.0, 1.0
    v[0, 0], v[0, 1] = torch.tensor([1.0, 2.0, 3.0, 4.0]), torch.tensor([5.0, 6.0, 7.0, 8.0])
    decay = [1.0 - 2.0 ** -12, 0.5]
    dec = torch.tensor(decay, device="cuda")
    for cuts, tile in ([(0, T)], 64), (_cuts(T, [1]), 0), (_cuts(T, [129, 2, 70]), 32):
        state = torch.full((1, H, d, dv), 3.0, device="cuda")
        for a, c in cuts:
            seg = [(0, a, c)]
            sd, pd, _, _, sf, sc = _rows(seg)
            qd, kd, vd = (t[a:a + c].cuda().contiguous() for t in (q, k, v))
            rec = torch.zeros(c, H * dv, device="cuda")
            if tile and c > tile:
                tf, tc, s0, sn = _tiles(seg, tile)
                ws = torch.zeros(int(L.ao_lm_outer_recurrence_workspace_bytes(len(tf), c, H, d, dv)) // 4, device="cuda")
                args = (_p(tf), _p(tc), len(tf), _p(s0), _p(sn), 1, c, _p(ws))
            else:
                args = (_p(sf), _p(sc), 1, None, None, 0, c, None)
            lib.lm_check(L.ao_lm_outer_recurrence(_p(qd), H * d, _p(kd), H * d, _p(vd), H * dv, 0, None, None, H, _p(dec), None, H, H, d, dv,
                                                  _p(state), _p(sd), _p(pd), *args, _p(rec), H * dv, _st()), "rec")
        last = rec[-1].view(H, dv).cpu().double()
        assert _close(last[0], v[0, 0].double() * decay[0] ** (T - 1), 1e-5) and float(last[1].abs().max()) < 1e-30


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_decoding_past_the_ring_and_sequences_longer_than_the_cache_was_asked_for(dtype):
    cfg = _mixed()
    w = O.random_weights(cfg, 25)
    toks = _tokens(cfg, 150, 9)
    ref = O.forward(cfg, w, toks)
    m = _model(cfg, w, dtype, slots=1, seq=64)        # every window fits 64 positions: the sequence may outgrow them
    eng, st = m.step_engine, m.states
    assert m.run_state[1].window.ring == 9 and m.run_state[1].window.first_rows == 3
    got = [eng.step([(st.slot_of("r"), toks[:20])], "all")] + [eng.step([(st.slot_of("r"), [t])], "all") for t in toks[20:]]
    tol = F32_TOL if dtype == torch.float32 else _bf16_tol(cfg, w, toks)
    assert _within(torch.cat(got), ref, tol, dtype == torch.float32)
    wide = _wide()
    m = _model(wide, O.random_weights(wide, 25), dtype, slots=1, seq=50)      # the window was cut to the cache: it has an end
    m.step_engine.step([(m.states.slot_of("r"), _tokens(wide, 50, 1))], "last")
    with pytest.raises(RuntimeError):
        m.step_engine.step([(m.states.slot_of("r"), [1])], "all")


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
    cfg = _time_first()
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
    G.main(random_init="Fedipel-test", num_samples=1, max_new_tokens=6, prompt="7,8,9")


def test_named_configuration_through_the_registry():
    from torchao_fork_b200._models import registry
    m = registry.random_init("Fedipel-test", "cuda", torch.bfloat16)
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
