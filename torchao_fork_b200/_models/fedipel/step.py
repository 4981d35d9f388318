"""The step function of Fedipel: runs the tokens a step brings — any mix of prompt portions and single decoded tokens of
several sequences — through the model's layers on the state that earlier steps left, as launches of libao_b200_lm
kernels (include/ao_b200_lm.h) and library GEMMs for the dense projections.

The residual x is fp32.  Every sublayer ends in ONE row kernel (`add_layer_norm`): x += m * result, and the next
sublayer's layer norm is taken while the row is still on chip.
  retention: ONE GEMM [q | k | v | gate] (fp32 result) -> `rotary_rows` (queries and keys in place, the keys' scale) ->
      `outer_recurrence` (a fixed decay per head, matrix state per slot; tiled for long portions) -> `gated_group_norm`
      (unit RMS per head, times SiLU of the gate) -> GEMM W_o.
  wkv: `token_shift_mix` (five blends of each row with the row in front of it, the slot's saved row at a portion's start)
      -> ONE batched GEMM for r, k, v, gate + GEMM w1 -> tanh -> GEMM w2 -> `channel_recurrence` (decay
      exp(-exp(. + w0)) made on load, bonus for the current token; saves the portion's last input row) ->
      `gated_group_norm` (unit RMS per head, weight, SiLU gate) -> GEMM W_o.
  attention: ONE GEMM [q | k | v] (or queries only, for a layer that borrows keys and values) -> `qkv_rotary_prep`
      (biases, rotation of both maps) -> `window_attention` over the owner's ring / first-token store and the step's own
      rows (both maps, their difference, unit RMS) -> GEMM W_o; `window_append` stores the step's keys and values once the
      last layer that reads them has run.
  feed-forward: GEMM [gate | up] -> `glu_act` -> GEMM down; or ONE GEMM [router | shared gate] (fp32) ->
      `router_topk_renorm_logits` -> shared expert (its squared-ReLU kernel also applies the sigmoid gate) + chosen experts
      (matrix-vector kernels for a few tokens, rows sorted by expert around grouped GEMMs for many).
Norms, rotations, router logits, attention scores and weights, decays, gates of the recurrences and every recurrent
state are fp32 in both storage types.

`StepEngine.step` is what prefill, the trace runner and tests call; `GraphDecodeEngine` wraps the same layer loop for
one token per sequence with all metadata in device memory, captured into a CUDA graph.
"""
import ctypes

import torch

from ... import _lib
from ..experts import ACT_SOFTCAP, ACT_TANH, act_unit, chosen_experts, glu_unit
from ..segment_step import GraphDecodeEngine, SegmentStepEngine, StepMeta, _p  # noqa: F401
from .model import Fedipel

# up to this many tokens the chosen experts run as index-driven matrix-vector kernels, beyond it as GEMMs over sorted rows
MOE_GEMV_TOKENS = 16
_INF = float("inf")
PAIR_INTERLEAVED, PAIR_HALVES = 0, 1      # rotation couples (2i, 2i + 1) / (i, i + dims / 2)
GATE_SILU_AFTER_NORM = 2                  # mode of gated_group_norm


class StepEngine(SegmentStepEngine):
    matrix_recurrences = True       # the step's metadata carries tiles for the tiled form of the matrix-state recurrences

    def __init__(self, model: Fedipel):
        super().__init__(model)
        cfg = self.cfg
        # attention layer -> the layer that owns the cache it reads; owner -> the last layer that reads it
        self.owner = {i: (i if la.mixer.kv_from is None else la.mixer.kv_from) for i, la in enumerate(cfg.layers) if la.type == "attention"}
        self.last_reader = {o: max(cfg.readers_of(o)) for o in set(self.owner.values())}

    def _attention_shapes(self):
        return sorted({("window", 2, la.mixer.heads, la.mixer.kv_heads, la.mixer.dim, la.mixer.vdim)
                       for la in self.cfg.layers if la.type == "attention"})

    def _attention_plan(self, shape):
        _, maps, H, G, d, dv = shape
        tr, pr = ctypes.c_int(), ctypes.c_int()
        _lib.lm_check(self.L.ao_lm_window_attention_plan(self.dt, maps, H, G, d, dv, ctypes.byref(tr)), "window_attention_plan")
        _lib.lm_check(self.L.ao_lm_window_attention_prompt_plan(self.dt, maps, H, G, d, dv, ctypes.byref(pr)), "window_attention_prompt_plan")
        return tr.value, 1 << 30, pr.value      # tiles may cross any position

    # ------------------------------------------------------------------------------------------------ layers
    def _norm(self, x, y, w, b, st, want_f32=False):
        """x += m * y (y None: nothing added); -> layer norm of x with (w, b) in the model's dtype, or as fp32 when a
        token-shift layer reads it (w None: only the add, -> None).  One launch."""
        cfg, dev = self.cfg, self.dev
        n, W = x.shape
        h = h32 = None
        if w is not None:
            if want_f32 and self.m.dtype != torch.float32:
                h32 = torch.empty(n, W, dtype=torch.float32, device=dev)
            else:
                h = torch.empty(n, W, dtype=self.m.dtype, device=dev)
        _lib.lm_check(self.L.ao_lm_add_layer_norm(_p(x), _p(y), cfg.residual_mult, None, n, W, _p(w), _p(b), self.dt, cfg.norm_eps,
                                                  _p(h32), _p(h), st), "add_layer_norm")
        return h if h32 is None else h32

    def _layers(self, d_tok: torch.Tensor, meta: StepMeta, after_run=None) -> torch.Tensor:
        m, cfg, L, dt, dev = self.m, self.cfg, self.L, self.dt, self.dev
        n, W = meta.n, cfg.width
        st = torch.cuda.current_stream(dev).cuda_stream
        x = torch.empty(n, W, dtype=torch.float32, device=dev)
        _lib.lm_check(L.ao_lm_embed(_p(m.embed), dt, _p(d_tok), n, W, _p(x), st), "embed")
        # the embedding's own norm, in place on the residual
        _lib.lm_check(L.ao_lm_add_layer_norm(_p(x), None, 0.0, None, n, W, _p(m.embed_norm), _p(m.embed_norm_b), dt, cfg.norm_eps,
                                             _p(x), None, st), "add_layer_norm")
        launches = 2
        layers = m.layers
        if not layers:
            return x
        h = self._norm(x, None, layers[0].norm1, layers[0].norm1_b, st, layers[0].args.type == "wkv")
        launches += 1
        step_kv = {}                    # owner layer -> the step's rotated keys and values
        for i, lay in enumerate(layers):
            la, ls = lay.args, m.run_state[i]
            if la.type == "retention":
                y, c = self._retention(lay, la.mixer, ls, h, meta, st)
            elif la.type == "wkv":
                y, c = self._wkv(lay, la.mixer, ls, h, meta, st)
            else:
                y, c = self._attention(i, lay, la.mixer, h, meta, step_kv, st)
            launches += c
            nxt = layers[i + 1] if i + 1 < len(layers) else None
            if la.mlp is not None:
                h = self._norm(x, y, lay.norm2, lay.norm2_b, st)
                y, c = self._feed_forward(lay, la.mlp, h, n, st)
                launches += c + 1
            nw, nb, n32 = (nxt.norm1, nxt.norm1_b, nxt.args.type == "wkv") if nxt is not None else (None, None, False)
            if after_run is not None:       # the residual as the layer leaves it
                self._norm(x, y, None, None, st)
                after_run(i, x)
                h = self._norm(x, None, nw, nb, st, n32) if nxt is not None else None
                launches += 2
            else:
                h = self._norm(x, y, nw, nb, st, n32)
                launches += 1
        self.launches = launches
        return x

    def _recurrence_tiles(self, meta: StepMeta):
        """(first rows, row counts, n, owner tables or None ...) of the recurrence launch: whole segments, or tiles."""
        if meta.rec is None:
            sf, sc, ns = meta.seg
            return sf, sc, ns, None, None, 0
        return meta.rec

    def _retention(self, lay, a, ls, h, meta: StepMeta, st):
        """Linear attention with a fixed decay per head over rotated queries and keys -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, d, dv, n = a.heads, a.dim, a.vdim, meta.n
        proj = self._mm_f32(h, lay.w_in)
        base, ld = proj.data_ptr(), lay.ld
        _lib.lm_check(L.ao_lm_rotary_rows(base, ld, n, _p(meta.pos), _p(lay.inv_freq), a.rot.dims, PAIR_HALVES, d, lay.q_off, H, 1.0,
                                          lay.k_off, H, d ** -0.5, st), "rotary_rows")
        rec = torch.empty(n, H * dv, dtype=torch.float32, device=dev)
        tf, tc, nt, s0, sn, nseg = self._recurrence_tiles(meta)
        ws, c = None, 1
        if s0 is not None:
            ws = torch.empty(int(L.ao_lm_outer_recurrence_workspace_bytes(nt, n, H, d, dv)) // 4, dtype=torch.float32, device=dev)
            c = 3
        _lib.lm_check(L.ao_lm_outer_recurrence(base + 4 * lay.q_off, ld, base + 4 * lay.k_off, ld, base + 4 * lay.v_off, ld, 0, None,
                                               None, H, _p(lay.decay), None, H, H, d, dv, _p(ls.mat.s), _p(meta.slot), _p(meta.pos),
                                               _p(tf), _p(tc), nt, _p(s0), _p(sn), nseg, n, _p(ws), _p(rec), H * dv, st),
                      "outer_recurrence")
        o = torch.empty(n, H * dv, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_gated_group_norm(_p(rec), H * dv, base + 4 * lay.g_off, ld, GATE_SILU_AFTER_NORM, n, H * dv, H, None, dt,
                                               self.cfg.norm_eps, _p(o), st), "gated_group_norm")
        return self._mm_f32(o, lay.w_out), 4 + c

    def _bmm_f32(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """[b][n][K] x [b][M][K]^T -> fp32 [b][n][M]: several projections of one shape, each with an input of its own."""
        if a.dtype == torch.bfloat16:
            return torch.bmm(a, w.transpose(1, 2), out_dtype=torch.float32)
        return torch.bmm(a, w.transpose(1, 2))

    def _wkv(self, lay, a, ls, h, meta: StepMeta, st):
        """Time mixing with a decay per token and key channel; h is the fp32 norm output -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, d, n, W = a.heads, a.dim, meta.n, self.cfg.width
        mixes = torch.empty(5, n, W, dtype=tdt, device=dev)                    # inputs of r, k, v, gate, decay
        _lib.lm_check(L.ao_lm_token_shift_mix(_p(h), _p(lay.mu), 5, dt, _p(ls.shift.prev), _p(meta.slot), _p(meta.pos), _p(meta.back),
                                              n, W, _p(mixes), st), "token_shift_mix")
        rkvg = self._bmm_f32(mixes[:4], lay.w_rkvg)                            # fp32 [4][n][H d]
        z1 = self._mm_f32(mixes[4], lay.w1)
        t1 = torch.empty(n, a.rank, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_unary_rows(_p(z1), _lib.DT_F32, n, a.rank, ACT_TANH, 0.0, None, 0, _p(t1), dt, st), "unary_rows")
        zw = self._mm_f32(t1, lay.w2)                                          # the decay's pre-activation, without w0
        rec = torch.empty(n, H * d, dtype=torch.float32, device=dev)
        tf, tc, nt, s0, sn, nseg = self._recurrence_tiles(meta)
        ws, c = None, 1
        if s0 is not None:
            ws = torch.empty(int(L.ao_lm_channel_recurrence_workspace_bytes(nt, n, H, d, d)) // 4, dtype=torch.float32, device=dev)
            c = 3
        hd = H * d
        _lib.lm_check(L.ao_lm_channel_recurrence(_p(rkvg[0]), hd, _p(rkvg[1]), hd, _p(rkvg[2]), hd, _p(zw), hd, _p(lay.w0), _p(lay.bonus),
                                                 dt, H, d, d, _p(ls.mat.s), _p(meta.slot), _p(meta.pos), _p(tf), _p(tc), nt, _p(s0),
                                                 _p(sn), nseg, n, _p(ws), _p(h), _p(ls.shift.prev), W, _p(rec), hd, st),
                      "channel_recurrence")
        o = torch.empty(n, hd, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_gated_group_norm(_p(rec), hd, _p(rkvg[3]), hd, GATE_SILU_AFTER_NORM, n, hd, H, _p(lay.mix_norm), dt,
                                               self.cfg.norm_eps, _p(o), st), "gated_group_norm")
        return self._mm_f32(o, lay.w_out), 7 + c

    def _attention(self, i, lay, a, h, meta: StepMeta, step_kv, st):
        """Differential attention under a window that keeps the first tokens -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, G, d, dv, n = a.heads, a.kv_heads, a.dim, a.vdim, meta.n
        owner = self.owner[i]
        cache = self.m.run_state[owner].window
        proj = self._mm_f32(h, lay.w_in)
        qn = torch.empty(n, H, 2, d, dtype=torch.float32, device=dev)
        own = owner == i
        if own:
            kn = torch.empty(n, G, 2, d, dtype=tdt, device=dev)
            vn = torch.empty(n, G, dv, dtype=tdt, device=dev)
            step_kv[i] = (kn, vn)
        kn, vn = step_kv[owner]
        _lib.lm_check(L.ao_lm_qkv_rotary_prep(_p(proj), lay.ld, lay.q_off, lay.k_off, lay.v_off, _p(lay.q_b), _p(lay.k_b), _p(lay.v_b),
                                              _p(meta.pos), _p(lay.inv_freq), a.rot.dims, PAIR_INTERLEAVED, n, 2 * H, 2 * G if own else 0,
                                              d, G * dv, dt, _p(qn), _p(kn) if own else None, _p(vn) if own else None, st),
                      "qkv_rotary_prep")
        tf, tc, nt, tensor = meta.attn[("window", 2, H, G, d, dv)]
        o = torch.empty(n, H * dv, dtype=tdt, device=dev)
        window, keep = min(a.window, cache.ring), min(a.keep, cache.first_rows)
        common = (_p(qn), _p(kn), _p(vn), _p(cache.k), _p(cache.v), _p(cache.k_first), _p(cache.v_first), cache.ring, cache.first_rows,
                  dt, _p(meta.slot), _p(meta.pos), _p(meta.back), _p(tf), _p(tc), nt, 2, H, G, d, dv, window, keep, a.scale, lay.lam, 1,
                  self.cfg.norm_eps, 1.0 - a.diff)
        c = 4
        if tensor:      # prompt portions: the tensor-core form
            _lib.lm_check(L.ao_lm_window_attention_prompt(*common, _p(o), H * dv, st), "window_attention_prompt")
        else:
            ns = self._splits(nt * G, window + keep)    # few rows over a long window: the keys are shared out over more CTAs
            ws = torch.empty(max(16, int(L.ao_lm_window_attention_workspace_bytes(nt, 2, H, G, dv, ns))), dtype=torch.uint8, device=dev)
            _lib.lm_check(L.ao_lm_window_attention(*common, ns, _p(ws), ws.numel(), _p(o), H * dv, st), "window_attention")
            c += 1 if ns > 1 else 0
        if self.last_reader[owner] == i:        # nobody reads the old rows any more: the step's rows enter the cache
            _lib.lm_check(L.ao_lm_window_append(_p(kn), _p(vn), n, G * 2 * d, G * dv, cache.ring, cache.first_rows, dt, _p(meta.slot),
                                                _p(meta.pos), _p(meta.ahead), _p(cache.k), _p(cache.v), _p(cache.k_first),
                                                _p(cache.v_first), st), "window_append")
            del step_kv[owner]
            c += 1
        return self._mm_f32(o, lay.w_out), c

    def _feed_forward(self, lay, f, h, n, st):
        """-> (fp32 [n][W], launches)"""
        L, dt, dev = self.L, self.dt, self.dev
        if f.kind == "dense":
            return glu_unit(L, dt, h, lay.w_gu, lay.w_down, _INF, 1.0, 0.0, st)
        E = f.experts
        z = self._mm_f32(h, lay.router)                                        # [n][E (+ 1: the shared expert's gate)]
        ridx = torch.empty(n, f.top, dtype=torch.int32, device=dev)
        rwt = torch.empty(n, f.top, dtype=torch.float32, device=dev)
        sgate = torch.empty(n, dtype=torch.float32, device=dev) if f.shared_ff else None
        _lib.lm_check(L.ao_lm_router_topk_renorm_logits(_p(z), z.shape[1], _p(lay.router_b), n, E, f.top, E if f.shared_ff else -1,
                                                        _p(ridx), _p(rwt), _p(sgate), st), "router_topk_renorm_logits")
        launches = 2
        if f.shared_ff:
            out, c = act_unit(L, dt, h, lay.su, lay.sd, sgate, st)
            launches += c
        else:
            out = torch.empty(n, self.cfg.width, dtype=torch.float32, device=dev)
        launches += chosen_experts(L, dt, h, ridx, rwt, lay.wu, lay.wd, out, _INF, 1.0, 0.0, n <= MOE_GEMV_TOKENS,
                                   bool(f.shared_ff), st, gated=False)
        return out, launches

    def _logits_dev(self, x, d_rows, k, out=None):
        m, cfg, dev = self.m, self.cfg, self.dev
        st = torch.cuda.current_stream(dev).cuda_stream
        xn = torch.empty(k, cfg.width, dtype=m.dtype, device=dev)
        _lib.lm_check(self.L.ao_lm_add_layer_norm(_p(x), None, 0.0, _p(d_rows), k, cfg.width, _p(m.final_norm), _p(m.final_norm_b),
                                                  self.dt, cfg.norm_eps, None, _p(xn), st), "add_layer_norm")
        lg = self._mm_f32(xn, m.head)
        if cfg.logit_softcap:
            _lib.lm_check(self.L.ao_lm_unary_rows(_p(lg), _lib.DT_F32, k, cfg.vocab_size, ACT_SOFTCAP, cfg.logit_softcap, None, 0,
                                                  _p(lg), _lib.DT_F32, st), "unary_rows")
        if out is not None:
            out.copy_(lg)
            return out
        return lg
