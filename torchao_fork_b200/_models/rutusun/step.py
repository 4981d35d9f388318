"""The step function of Rutusun: runs the tokens a step brings — any mix of prompt portions and single decoded tokens of
several sequences — through the model's layer runs on the state that earlier steps left, as launches of libao_b200_lm
kernels (include/ao_b200_lm.h) and library GEMMs for the dense projections.

The residual x is fp32.  Every sublayer ends in ONE row kernel (`postnorm_residual`): the sublayer's result enters x
through its own RMS norm, what a pass over the looped span adds in front of its first layer (the embedding output, the
pass's learned vector) is added, and the next sublayer's input norm is taken while the row is still in registers.
  attention: ONE GEMM [q | k | v] (fp32 result) -> `qk_norm_prep` (biases, weighted unit-RMS queries and keys, query
      temperature; also stores the keys and values in the slot's cache) -> `sink_attention` over the slot's cached keys /
      values and the step's own rows (tensor-core form for prompt portions in bf16, fp32 form with key splits otherwise)
      -> GEMM W_o (its bias joins the result in the sublayer's closing kernel).
  lightning: ONE GEMM [q | k | v | gate] (fp32) -> `outer_recurrence` (SiLU on load, fixed decay per head, matrix state
      per slot) -> `gated_group_norm` (norm, then sigmoid gate) -> GEMM W_o.
  mamba2: GEMM W_in (fp32) -> `ssd_prep` (convolution + SiLU over [x | B | C], softplus step sizes, decays) ->
      `conv_state_save` -> `outer_recurrence` (k = B, q = C per group, skip term) -> `gated_group_norm` (SiLU gate, then
      grouped norm) -> GEMM W_o.
  feed-forward: GEMM [gate | up] -> `glu_act` -> GEMM down; or router logits (GEMM, fp32) -> `router_group_topk` ->
      shared expert + chosen experts (matrix-vector kernels for a few tokens, rows sorted by expert around grouped GEMMs
      for many).
Norms, router scores, attention scores and weights, decays, step sizes, gates and every recurrent state are fp32 in both
storage types.

`StepEngine.step` is what prefill, the trace runner and tests call; `GraphDecodeEngine` wraps the same layer loop for
one token per sequence with all metadata in device memory, captured into a CUDA graph.
"""
import torch

from ... import _lib
from ..experts import chosen_experts, glu_unit
from ..segment_step import GraphDecodeEngine, SegmentStepEngine, StepMeta, _p  # noqa: F401
from .model import Rutusun

# up to this many tokens the chosen experts run as index-driven matrix-vector kernels, beyond it as GEMMs over sorted rows
MOE_GEMV_TOKENS = 16
_INF = float("inf")


class StepEngine(SegmentStepEngine):
    matrix_recurrences = True       # the step's metadata carries tiles for the tiled form of `outer_recurrence`

    def __init__(self, model: Rutusun):
        super().__init__(model)
        # the work in order, with what stands between two sublayers resolved once: (layer run, pass vectors in front of it)
        self.plan = []
        pending, r = [], 0
        for kind, i in self.cfg.schedule:
            if kind == "enter":
                pending.append(i)
            else:
                self.plan.append((r, i, pending))
                pending, r = [], r + 1
        self.tail_enters = pending      # passes over an empty span at the very end

    def _attention_shapes(self):
        S = self.m.max_seq_length
        return [(la.mixer.heads, la.mixer.kv_heads, la.mixer.dim, la.mixer.vdim, S) for la in self.cfg.layers if la.type == "attention"]

    # ------------------------------------------------------------------------------------------------ layers
    def _post(self, x, y, post_w, enters, emb, next_w, h, st, y_bias=None):
        """x += norm(y) * post_w; the pass vectors of `enters` (and the embedding output for every pass but the first);
        h = norm(x) * next_w.  One launch unless several passes start at once."""
        m, cfg, L, dt = self.m, self.cfg, self.L, self.dt
        n, W = x.shape
        k = 0
        steps = list(enters)
        while True:
            t = steps.pop(0) if steps else None
            last = not steps
            _lib.lm_check(L.ao_lm_postnorm_residual(
                _p(x), _p(y), _lib.DT_F32, _p(y_bias), _p(post_w), _p(emb) if t is not None and t > 0 else None,
                m.loop_step[t].data_ptr() if t is not None else None, _p(next_w) if last else None, dt, cfg.norm_eps, n, W,
                _p(h) if last and next_w is not None else None, st), "postnorm_residual")
            k += 1
            y = post_w = y_bias = None
            if last:
                return k

    def _layers(self, d_tok: torch.Tensor, meta: StepMeta, after_run=None) -> torch.Tensor:
        m, cfg, L, dt, dev = self.m, self.cfg, self.L, self.dt, self.dev
        n, W = meta.n, cfg.width
        st = torch.cuda.current_stream(dev).cuda_stream
        x = torch.empty(n, W, dtype=torch.float32, device=dev)
        h = torch.empty(n, W, dtype=m.dtype, device=dev)
        _lib.lm_check(L.ao_lm_embed(_p(m.embed), dt, _p(d_tok), n, W, _p(x), st), "embed")
        launches = 1
        emb = None
        if cfg.loop and cfg.loop[2] > 1:
            emb = x.clone()
            launches += 1
        plan = self.plan
        if not plan:
            self._post(x, None, None, self.tail_enters, emb, None, None, st)
            return x
        launches += self._post(x, None, None, plan[0][2], emb, m.layers[plan[0][1]].norm1, h, st)
        for k, (r, li, _) in enumerate(plan):
            lay, rs = m.layers[li], m.run_state[r]
            la = lay.args
            y_bias = lay.o_b if la.type == "attention" else None     # the output projection's bias joins the result in `_post`
            if la.type == "attention":
                y, c = self._attention(lay, la.mixer, rs, h, meta, st)
            elif la.type == "lightning":
                y, c = self._lightning(lay, la.mixer, rs, h, meta, st)
            else:
                y, c = self._mamba2(lay, la.mixer, rs, h, meta, st)
            launches += c
            if k + 1 < len(plan):
                nxt_enters, nxt_norm = plan[k + 1][2], m.layers[plan[k + 1][1]].norm1
            else:
                nxt_enters, nxt_norm = self.tail_enters, None
            if la.mlp is not None:
                launches += self._post(x, y, lay.norm1b, [], emb, lay.norm2, h, st, y_bias)
                y, c = self._feed_forward(lay, la.mlp, h, n, st)
                launches += c
                post_w, y_bias = lay.norm2b, None
            else:
                post_w = lay.norm1b
            if after_run is not None:       # the residual as the layer leaves it, before the next pass's additions
                launches += self._post(x, y, post_w, [], emb, None, None, st, y_bias)
                after_run(r, x)
                if nxt_enters or nxt_norm is not None:
                    launches += self._post(x, None, None, nxt_enters, emb, nxt_norm, h, st)
            else:
                launches += self._post(x, y, post_w, nxt_enters, emb, nxt_norm, h, st, y_bias)
        self.launches = launches
        return x

    def _recurrence(self, q, ldq, k, ldk, v, ldv, act, a, b, a_head, skip, H, G, d, dv, rs, meta: StepMeta, rec, st) -> int:
        """`outer_recurrence` over the step: whole segments in one launch, or — when a segment is longer than a tile — the
        tiled form in three.  q, k, v, a, b: device addresses."""
        L = self.L
        if meta.rec is None:
            sf, sc, ns = meta.seg
            _lib.lm_check(L.ao_lm_outer_recurrence(q, ldq, k, ldk, v, ldv, act, a, b, H, a_head, skip, H, G, d, dv, _p(rs.mat.s),
                                                   _p(meta.slot), _p(meta.pos), _p(sf), _p(sc), ns, None, None, 0, meta.n, None,
                                                   _p(rec), H * dv, st), "outer_recurrence")
            return 1
        tf, tc, nt, s0, sn, nseg = meta.rec
        ws = torch.empty(int(L.ao_lm_outer_recurrence_workspace_bytes(nt, meta.n, H, d, dv)) // 4, dtype=torch.float32, device=self.dev)
        _lib.lm_check(L.ao_lm_outer_recurrence(q, ldq, k, ldk, v, ldv, act, a, b, H, a_head, skip, H, G, d, dv, _p(rs.mat.s),
                                               _p(meta.slot), _p(meta.pos), _p(tf), _p(tc), nt, _p(s0), _p(sn), nseg, meta.n, _p(ws),
                                               _p(rec), H * dv, st), "outer_recurrence")
        return 3

    def _attention(self, lay, a, rs, h, meta: StepMeta, st):
        """Causal attention with a sink over the slot's cache and the step's rows -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, G, d, dv, n = a.heads, a.kv_heads, a.dim, a.vdim, meta.n
        S = rs.ring.ring
        proj = self._mm_f32(h, lay.w_in)
        qn = torch.empty(n, H, d, dtype=torch.float32, device=dev)
        kn = torch.empty(n, G, d, dtype=tdt, device=dev)
        vn = torch.empty(n, G, dv, dtype=tdt, device=dev)
        o = torch.empty(n, H * dv, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_qk_norm_prep(_p(proj), lay.ld, lay.q_off, lay.k_off, lay.v_off, _p(lay.q_b), _p(lay.k_b), _p(lay.v_b),
                                           _p(lay.q_norm), _p(lay.k_norm), a.temp_coef, a.temp_every, _p(meta.pos), _p(meta.slot),
                                           _p(rs.ring.k), _p(rs.ring.v), S, n, H, G, d, dv, self.cfg.norm_eps, dt, _p(qn), _p(kn),
                                           _p(vn), st), "qk_norm_prep")
        tf, tc, nt, tensor = meta.attn[(H, G, d, dv, S)]
        common = (_p(qn), _p(kn), _p(vn), _p(rs.ring.k), _p(rs.ring.v), dt, None, 0, None, 0, _p(lay.sink), _p(meta.slot),
                  _p(meta.pos), _p(meta.back), _p(tf), _p(tc), nt, H, G, d, dv, S, a.scale, 0.0, 1.0)
        split = 0
        if tensor:
            _lib.lm_check(L.ao_lm_sink_attention_prompt(*common, _p(o), o.shape[1], st), "sink_attention_prompt")
        else:
            ns = self._splits(nt * G, S)
            nbytes = int(L.ao_lm_chunk_attention_workspace_bytes(nt, G, dv, ns))
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
            _lib.lm_check(L.ao_lm_sink_attention(*common, ns, _p(ws), ws.numel(), _p(o), o.shape[1], st), "sink_attention")
            split = 1 if ns > 1 else 0
        return self._mm_f32(o, lay.w_out), 4 + split

    def _lightning(self, lay, a, rs, h, meta: StepMeta, st):
        """Linear attention with a fixed decay per head -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, d, dv, n = a.heads, a.dim, a.vdim, meta.n
        proj = self._mm_f32(h, lay.w_in)
        base, ld = proj.data_ptr(), lay.ld
        rec = torch.empty(n, H * dv, dtype=torch.float32, device=dev)
        c = self._recurrence(base + 4 * lay.q_off, ld, base + 4 * lay.k_off, ld, base + 4 * lay.v_off, ld, 1, None, None,
                             _p(lay.decay), None, H, H, d, dv, rs, meta, rec, st)
        o = torch.empty(n, H * dv, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_gated_group_norm(_p(rec), H * dv, base + 4 * lay.g_off, ld, 0, n, H * dv, 1, _p(lay.mix_norm), dt,
                                               self.cfg.norm_eps, _p(o), st), "gated_group_norm")
        return self._mm_f32(o, lay.w_out), 3 + c

    def _mamba2(self, lay, a, rs, h, meta: StepMeta, st):
        """Selective state space in its matrix-state form -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, dv, N, G, n = a.heads, a.vdim, a.state, a.groups, meta.n
        inner, ch = a.inner, a.conv_channels
        proj = self._mm_f32(h, lay.w_in)                                   # [n][z | x | B | C | step] fp32
        base, ld = proj.data_ptr(), lay.ld
        xbc = torch.empty(n, ch, dtype=torch.float32, device=dev)
        ab = torch.empty(2, n, H, dtype=torch.float32, device=dev)
        _lib.lm_check(L.ao_lm_ssd_prep(base, ld, inner, inner + ch, n, ch, a.conv, _p(lay.conv_w), _p(lay.conv_b), dt, _p(rs.conv.x),
                                       _p(meta.slot), _p(meta.pos), _p(meta.back), H, _p(lay.dt_bias), _p(lay.a_log), _p(xbc),
                                       _p(ab[0]), _p(ab[1]), st), "ssd_prep")
        _lib.lm_check(L.ao_lm_conv_state_save(base + 4 * inner, ld, n, ch, a.conv, _p(meta.slot), _p(meta.pos), _p(meta.back),
                                              _p(meta.ahead), _p(rs.conv.x), st), "conv_state_save")
        xb = xbc.data_ptr()
        rec = torch.empty(n, inner, dtype=torch.float32, device=dev)
        c = self._recurrence(xb + 4 * (inner + G * N), ch, xb + 4 * inner, ch, xb, ch, 0, _p(ab[0]), _p(ab[1]), None, _p(lay.skip),
                             H, G, N, dv, rs, meta, rec, st)
        o = torch.empty(n, inner, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_gated_group_norm(_p(rec), inner, base, ld, 1, n, inner, a.norm_groups, _p(lay.mix_norm), dt,
                                               self.cfg.norm_eps, _p(o), st), "gated_group_norm")
        return self._mm_f32(o, lay.w_out), 5 + c

    def _feed_forward(self, lay, f, h, n, st):
        """-> (fp32 [n][W], launches)"""
        L, dt, dev = self.L, self.dt, self.dev
        if f.kind == "dense":
            return glu_unit(L, dt, h, lay.w_gu, lay.w_down, _INF, 1.0, 0.0, st)
        z = self._mm_f32(h, lay.router)
        ridx = torch.empty(n, f.top, dtype=torch.int32, device=dev)
        rwt = torch.empty(n, f.top, dtype=torch.float32, device=dev)
        _lib.lm_check(L.ao_lm_router_group_topk_logits(_p(z), n, f.experts, f.top, _p(lay.correction), f.n_groups, f.keep, f.scale,
                                                       _p(ridx), _p(rwt), st), "router_group_topk_logits")
        launches = 2
        if f.shared_ff:
            out, c = glu_unit(L, dt, h, lay.sgu, lay.sd, _INF, 1.0, 0.0, st)
            launches += c
        else:
            out = torch.empty(n, self.cfg.width, dtype=torch.float32, device=dev)
        launches += chosen_experts(L, dt, h, ridx, rwt, lay.wgu, lay.wd, out, _INF, 1.0, 0.0, n <= MOE_GEMV_TOKENS,
                                   bool(f.shared_ff), st)
        return out, launches

    def _logits_dev(self, x, d_rows, k, out=None):
        m, cfg, dev = self.m, self.cfg, self.dev
        st = torch.cuda.current_stream(dev).cuda_stream
        xn = torch.empty(k, cfg.width, dtype=m.dtype, device=dev)
        _lib.lm_check(self.L.ao_lm_streams_norm(_p(x), _p(d_rows), k, 1, cfg.width, None, _p(m.final_norm), self.dt, 0.0,
                                                cfg.norm_eps, None, _p(xn), st), "streams_norm")
        lg = self._mm_f32(xn, m.head)
        if out is not None:
            out.copy_(lg)
            return out
        return lg
