"""The step function of Tadolix: runs the tokens a step brings — any mix of prompt portions and single decoded tokens of
several sequences — through the model's layer runs on the state that earlier steps left, as launches of libao_b200_lm
kernels (include/ao_b200_lm.h) and library GEMMs for the dense projections.

Per sublayer: read-out of the streams + norm (`streams_norm`) -> [mixer only: causal convolution added to the input] ->
the sublayer -> write-back into the streams (`streams_update`, which also saves the convolution's memory).
  parallel mixer: ONE GEMM for [q | k | v | gate | z | x | gate of the recurrence] with an fp32 result -> `qk_prep` (unit-RMS
      queries and keys) -> `chunk_attention` over the ring cache and the step's own rows -> `ring_append` -> `mingru_scan`
      -> ONE GEMM over [attention result | recurrence result] with [W_o left | W_o right]: the two branch scales are
      applied by the kernels that write the operands, so the sum of the branches is the GEMM's own accumulation.
  rglru mixer: GEMM [y | x] (fp32) -> `causal_conv` -> batched GEMM of the block-diagonal gates -> `rglru_scan` (saves the
      convolution's memory too) -> GEMM W_o.
  feed-forward: GEMM [gate | up] -> `gelu_glu` -> GEMM down.
The streams, norms, gates, recurrences, attention scores and weights are fp32 in both storage types.

`StepEngine.step` is what prefill, the trace runner and tests call; `GraphDecodeEngine` wraps the same layer loop for
one token per sequence with all metadata in device memory, captured into a CUDA graph (the Llama DecodeEngine's role).
"""
from typing import Optional

import torch

from ... import _lib
from ..segment_step import (MAX_STEP_TOKENS, PROMPT_MIN_ROWS, SCAN_TILE, GraphDecodeEngine, SegmentStepEngine, StepMeta, _p,  # noqa: F401
                            chunk_tiles, scan_tiles, segments_of)
from .model import RGLRU_DECAY, Tadolix


class StepEngine(SegmentStepEngine):
    def __init__(self, model: Tadolix):
        super().__init__(model)

    def _attention_shapes(self):
        out = []
        for la in self.cfg.layers:
            if la.type == "parallel":
                a = la.mixer.left
                out.append((a.heads, a.kv_heads, a.dim, a.vdim, a.chunk))
        return out

    def _layers(self, d_tok: torch.Tensor, meta: StepMeta, after_run=None) -> torch.Tensor:
        m, cfg, L, dt, dev = self.m, self.cfg, self.L, self.dt, self.dev
        n, W, S = meta.n, cfg.width, max(1, cfg.streams)
        st = torch.cuda.current_stream(dev).cuda_stream
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=m.dtype, device=dev)
        x = torch.empty(n, S, W, **f32)
        hn = torch.empty(n, W, **f32)
        h = torch.empty(n, W, **act)
        _lib.lm_check(L.ao_lm_embed_sinusoid(_p(m.embed), dt, _p(d_tok), _p(meta.pos), n, W, cfg.embedding_scale, _p(m.pos_freq),
                                             S, _p(x), st), "embed_sinusoid")
        launches = 1
        taps = cfg.canon_taps
        for r, li in enumerate(cfg.runs):
            lay, rs = m.layers[li], m.run_state[r]
            la = lay.args
            hc = lay.hc[0]
            # ---- mixer sublayer
            if taps:
                _lib.lm_check(L.ao_lm_streams_norm(_p(x), None, n, S, W, _p(hc[0]) if hc else None, _p(lay.norm[0]), dt, 1.0,
                                                   cfg.norm_eps, _p(hn), None, st), "streams_norm")
                _lib.lm_check(L.ao_lm_causal_conv(_p(hn), W, None, n, W, taps, _p(lay.canon), None, dt, 1, _p(rs.canon.x),
                                                  _p(meta.slot), _p(meta.pos), _p(meta.back), None, _p(h), st), "causal_conv")
                launches += 2
            else:
                _lib.lm_check(L.ao_lm_streams_norm(_p(x), None, n, S, W, _p(hc[0]) if hc else None, _p(lay.norm[0]), dt, 1.0,
                                                   cfg.norm_eps, None, _p(h), st), "streams_norm")
                launches += 1
            if la.type == "parallel":
                y, k = self._parallel(lay, la.mixer, rs, h, meta, st)
            else:
                y, k = self._rglru(lay, la.mixer, rs, h, meta, st)
            launches += k + 1
            _lib.lm_check(L.ao_lm_streams_update(
                _p(x), _p(y), _lib.DT_F32, n, S, W, _p(hc[2]) if hc else None, _p(hc[1]) if hc else None, dt,
                _p(hn) if taps > 1 else None, _p(rs.canon.x) if taps > 1 else None, taps, _p(meta.slot), _p(meta.back),
                _p(meta.ahead), st), "streams_update")
            # ---- feed-forward sublayer
            if la.ff:
                hc = lay.hc[1]
                _lib.lm_check(L.ao_lm_streams_norm(_p(x), None, n, S, W, _p(hc[0]) if hc else None, _p(lay.norm[1]), dt, 1.0,
                                                   cfg.norm_eps, None, _p(h), st), "streams_norm")
                gu = torch.mm(h, lay.w_gu.t())
                ya = torch.empty(n, la.ff, **act)
                _lib.lm_check(L.ao_lm_gelu_glu(_p(gu), dt, n, la.ff, _p(ya), st), "gelu_glu")
                y = self._mm_f32(ya, lay.w_down)
                _lib.lm_check(L.ao_lm_streams_update(_p(x), _p(y), _lib.DT_F32, n, S, W, _p(hc[2]) if hc else None,
                                                     _p(hc[1]) if hc else None, dt, None, None, 0, None, None, None, st),
                              "streams_update")
                launches += 5
            if after_run is not None:
                after_run(r, x)
        self.launches = launches
        return x

    def _parallel(self, lay, mx, rs, h, meta: StepMeta, st):
        """Attention over the chunk + minimal GRU, both from one projection -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        a, Rw, n = mx.left, mx.right_width, meta.n
        H, G, d, dv = a.heads, a.kv_heads, a.dim, a.vdim
        proj = self._mm_f32(h, lay.w_in)                                   # [n][ld] fp32
        qn = torch.empty(n, H, d, dtype=torch.float32, device=dev)
        kn = torch.empty(n, G, d, dtype=tdt, device=dev)
        vn = torch.empty(n, G, dv, dtype=tdt, device=dev)
        both = torch.empty(n, H * dv + Rw, dtype=tdt, device=dev)          # [attention result | recurrence result]
        _lib.lm_check(L.ao_lm_qk_prep(_p(proj), lay.ld, lay.q_off, lay.k_off, lay.v_off, n, H, G, d, dv, self.cfg.norm_eps, dt,
                                      _p(qn), _p(kn), _p(vn), st), "qk_prep")
        tf, tc, nt, tensor = meta.attn[(H, G, d, dv, a.chunk)]
        common = (_p(qn), _p(kn), _p(vn), _p(rs.ring.k), _p(rs.ring.v), dt, proj.data_ptr() + 4 * lay.g_off, lay.ld,
                  _p(lay.dist_bias), lay.dist_bias.shape[1], _p(meta.slot), _p(meta.pos), _p(meta.back), _p(tf), _p(tc), nt, H, G, d,
                  dv, a.chunk, a.scale, a.softcap, mx.left_scale)
        split = 0
        if tensor:
            _lib.lm_check(L.ao_lm_chunk_attention_prompt(*common, _p(both), both.shape[1], st), "chunk_attention_prompt")
        else:
            ns = self._splits(nt * G, a.chunk)
            nbytes = int(L.ao_lm_chunk_attention_workspace_bytes(nt, G, dv, ns))
            ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
            _lib.lm_check(L.ao_lm_chunk_attention(*common, ns, _p(ws), ws.numel(), _p(both), both.shape[1], st), "chunk_attention")
            split = 1 if ns > 1 else 0
        _lib.lm_check(L.ao_lm_ring_append(_p(kn), _p(vn), n, G * d, G * dv, a.chunk, dt, _p(meta.slot), _p(meta.pos),
                                          _p(meta.ahead), _p(rs.ring.k), _p(rs.ring.v), st), "ring_append")
        sf, sc, snt, seg0, segn, ns = meta.scan
        ws = self._scan_ws(meta, Rw)
        _lib.lm_check(L.ao_lm_mingru_scan(
            _p(proj), lay.ld, lay.z_off, lay.x_off, lay.gr_off, _p(lay.z_b), _p(lay.x_b), dt, Rw, _p(rs.rec.s), _p(meta.slot),
            _p(meta.pos), _p(meta.back), _p(sf), _p(sc), snt, _p(seg0), _p(segn), ns, _p(ws), mx.right_scale,
            both.data_ptr() + H * dv * both.element_size(), both.shape[1], st), "mingru_scan")
        y = self._mm_f32(both, lay.w_out)
        return y, 6 + split + (2 if seg0 is not None else 0)

    def _rglru(self, lay, mx, rs, h, meta: StepMeta, st):
        """gelu branch x real-gated linear recurrence over a short convolution -> (fp32 [n][W], launches)."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        Rw, nb, n = mx.width, mx.blocks, meta.n
        bw = Rw // nb
        proj = self._mm_f32(h, lay.w_in)                                   # [n][y | x] fp32
        u = torch.empty(n, Rw, dtype=torch.float32, device=dev)
        ub = torch.empty(n, Rw, dtype=tdt, device=dev) if tdt != torch.float32 else u
        _lib.lm_check(L.ao_lm_causal_conv(proj.data_ptr() + 4 * Rw, 2 * Rw, _p(lay.x_b), n, Rw, mx.conv, _p(lay.conv_w),
                                          _p(lay.conv_b), dt, 0, _p(rs.conv.x), _p(meta.slot), _p(meta.pos), _p(meta.back),
                                          _p(u), _p(ub) if ub is not u else None, st), "causal_conv")
        ublk = ub.view(n, nb, bw).transpose(0, 1)                          # [blocks][n][bw]
        gates = torch.bmm(ublk, lay.w_gates, out_dtype=torch.float32) if tdt == torch.bfloat16 else torch.bmm(ublk, lay.w_gates)
        out = torch.empty(n, Rw, dtype=tdt, device=dev)
        sf, sc, snt, seg0, segn, ns = meta.scan
        ws = self._scan_ws(meta, Rw)
        _lib.lm_check(L.ao_lm_rglru_scan(
            _p(gates), n, bw, _p(lay.ra_b), _p(lay.ri_b), _p(lay.lam), RGLRU_DECAY, _p(u), _p(proj), 2 * Rw, _p(lay.y_b), dt, Rw,
            _p(rs.rec.s), proj.data_ptr() + 4 * Rw, 2 * Rw, _p(lay.x_b), _p(rs.conv.x) if mx.conv > 1 else None, mx.conv,
            _p(meta.slot), _p(meta.pos),
            _p(meta.back), _p(sf), _p(sc), snt, _p(seg0), _p(segn), ns, _p(ws), _p(out), st), "rglru_scan")
        y = self._mm_f32(out, lay.w_out)
        return y, 5 + (2 if seg0 is not None else 0)

    def _logits_dev(self, x, d_rows, k, out=None):
        m, cfg, dev = self.m, self.cfg, self.dev
        st = torch.cuda.current_stream(dev).cuda_stream
        xn = torch.empty(k, cfg.width, dtype=m.dtype, device=dev)
        _lib.lm_check(self.L.ao_lm_streams_norm(_p(x), _p(d_rows), k, max(1, cfg.streams), cfg.width, None, _p(m.final_norm),
                                                self.dt, 1.0, cfg.norm_eps, None, _p(xn), st), "streams_norm")
        lg = self._mm_f32(xn, m.head)
        if out is not None:
            out.copy_(lg)
            return out
        return lg
