"""The step function of Bitipel: runs the tokens a step brings — any mix of prompt portions and single decoded tokens of
several sequences — through the model's layers on the state that earlier steps left, as launches of libao_b200_lm
kernels (include/ao_b200_lm.h) and library GEMMs for the dense projections.

Per layer: token shift -> ONE GEMM for [queries | latent down-projection | gate logits] -> split / latent norm / rotary /
cache append -> key up-projection folded into the queries (batched GEMM, fp32 result) -> latent attention kernel over
the cached rows (fp32 scores and weights, sink, gate) -> value up-projection (batched GEMM) -> output GEMM -> residual
add with the scalar RMS norm (saves the token-shift memory, writes the experts' input) -> router kernel -> experts
(matrix-vector kernels for a few tokens, rows sorted by expert around library GEMMs for many) -> residual add with
norm + depth-weighted average of all layer results.  The residual stream and every statistic are fp32.

`StepEngine.step` is what prefill, the trace runner and tests call; `GraphDecodeEngine` wraps the same layer loop for
one token per sequence with all metadata in device memory, captured into a CUDA graph (the Llama DecodeEngine's role).
"""
from typing import List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from ... import _lib
from ..experts import chosen_experts
from .model import GLU_ALPHA, Bitipel

# a portion longer than this is cut into pieces (bounds the workspace: the layer results of a step are all kept)
MAX_STEP_TOKENS = 2048
# up to this many tokens the experts run as index-driven matrix-vector kernels, beyond it as GEMMs over sorted rows
MOE_GEMV_TOKENS = 16
# prompt portions of at least this many tokens per sequence (on average over the step) attend in the expanded form:
# the sequence's cached latents are up-projected into per-head keys and values once per layer and step
EXPAND_MIN_TOKENS = 32
# ... unless the expanded keys and values of all sequences of the step would take more than this
EXPAND_MAX_BYTES = 4 << 30


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class StepEngine:
    def __init__(self, model: Bitipel):
        assert model.device.type == "cuda", "Bitipel runs on CUDA only: there is no CPU path"
        self.m, self.cfg = model, model.config
        self.dev = model.device
        self.dt = _lib.DT_BF16 if model.dtype == torch.bfloat16 else _lib.DT_F32
        self.L = _lib.lm()
        if model.dtype == torch.float32:
            # true fp32 products: no TF32 / reduced-precision accumulation in the library GEMMs
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        self.sm_count = torch.cuda.get_device_properties(self.dev).multi_processor_count
        self.launches = 0
        # rows of one sequence that an attention CTA shares its key tiles for, per attention shape of the model
        import ctypes
        self.tile_tokens = {}
        for la in self.cfg.layers:
            a = la.mixer
            tt = ctypes.c_int()
            _lib.lm_check(self.L.ao_lm_latent_attention_plan(self.dt, a.heads, a.kv_rank, a.rot_dim, ctypes.byref(tt)), "latent_attention_plan")
            self.tile_tokens[(a.heads, a.kv_rank, a.rot_dim)] = tt.value
        # attention shapes that the expanded (prompt) kernel covers, and its tile
        self.expand_ok, self.expand_tile = {}, 0
        for la in self.cfg.layers:
            a = la.mixer
            tt = ctypes.c_int()
            _lib.lm_check(self.L.ao_lm_latent_attention_expanded_plan(self.dt, a.dim, a.rot_dim, a.vdim, ctypes.byref(tt)),
                          "latent_attention_expanded_plan")
            self.expand_ok[(a.dim, a.rot_dim, a.vdim)] = tt.value > 0
            self.expand_tile = max(self.expand_tile, tt.value)

    # ------------------------------------------------------------------------------------------------ public
    @torch.no_grad()
    def step(self, segments: Sequence[Tuple[int, Union[torch.Tensor, Sequence[int]]]],
             want: Union[str, Sequence[Sequence[int]]] = "last") -> torch.Tensor:
        """segments: [(slot, tokens)] — the next tokens of the sequences in those slots (each slot at most once).
        want: "last" (the last token of every segment), "all", or per segment the indices among ITS tokens.
        Returns fp32 logits [wanted][vocab] in segment order.  Positions continue from the state manager's lengths."""
        st = self.m.states
        toks, slots, poss, rows, bounds = [], [], [], [], []
        at = 0
        for k, (slot, t) in enumerate(segments):
            t = torch.as_tensor(t).reshape(-1).to(torch.int64).cpu().numpy() if not isinstance(t, np.ndarray) else t.astype(np.int64)
            n = len(t)
            assert n > 0
            p0 = st.extend(slot, n)
            toks.append(t)
            slots.append(np.full(n, slot, np.int32))
            poss.append(np.arange(p0, p0 + n, dtype=np.int32))
            sel = [n - 1] if want == "last" else list(range(n)) if want == "all" else list(want[k])
            rows += [at + int(i) for i in sel]
            bounds.append((at, at + n))
            at += n
        tok, slot, pos = np.concatenate(toks), np.concatenate(slots), np.concatenate(poss)
        if (tok < 0).any() or (tok >= self.cfg.vocab_size).any():
            raise ValueError("token id outside the vocabulary")
        total = at
        if total <= MAX_STEP_TOKENS:
            x = self._run(tok, slot, pos)
            return self._logits(x, rows)
        # long portions: pieces of at most MAX_STEP_TOKENS tokens, in order (a piece may end inside a segment)
        rows_np = np.asarray(rows, np.int64)
        result = torch.empty(len(rows), self.cfg.vocab_size, dtype=torch.float32, device=self.dev)
        for lo in range(0, total, MAX_STEP_TOKENS):
            hi = min(total, lo + MAX_STEP_TOKENS)
            x = self._run(tok[lo:hi], slot[lo:hi], pos[lo:hi])
            where = np.flatnonzero((rows_np >= lo) & (rows_np < hi))     # wanted rows keep the order they were asked in
            if len(where):
                result[torch.from_numpy(where).to(self.dev)] = self._logits(x, (rows_np[where] - lo).tolist())
        return result

    # ------------------------------------------------------------------------------------------------ pieces
    def _tiles(self, slot: np.ndarray, pos: np.ndarray, tile_tokens: int):
        """Runs of <= tile_tokens consecutive rows of one sequence (what one attention CTA shares its key tiles for)."""
        n = len(slot)
        brk = np.flatnonzero((slot[1:] != slot[:-1]) | (pos[1:] != pos[:-1] + 1)) + 1
        starts = np.concatenate([[0], brk])
        ends = np.concatenate([brk, [n]])
        first, count = [], []
        for s, e in zip(starts, ends):
            f = np.arange(s, e, tile_tokens)
            first.append(f)
            count.append(np.minimum(tile_tokens, e - f))
        return np.concatenate(first).astype(np.int32), np.concatenate(count).astype(np.int32)

    def _run(self, tok: np.ndarray, slot: np.ndarray, pos: np.ndarray) -> torch.Tensor:
        """One piece through all layers -> the stream that goes to the output norm, fp32 [n][W]."""
        n = len(tok)
        metas = {}
        for key, tile_tokens in self.tile_tokens.items():
            metas[key] = self._tiles(slot, pos, tile_tokens)
        expand = self._expand_plan(slot, pos)
        # one host->device copy for all metadata
        parts = [tok.view(np.int32), slot, pos]
        for key in sorted(metas):
            parts += list(metas[key])
        if expand is not None:
            parts += list(expand[0])
        packed = torch.from_numpy(np.concatenate(parts)).to(self.dev, non_blocking=True)
        o = 0
        d_tok = packed[o:o + 2 * n].view(torch.int64); o += 2 * n
        d_slot = packed[o:o + n]; o += n
        d_pos = packed[o:o + n]; o += n
        tiles = {}
        for key in sorted(metas):
            k = len(metas[key][0])
            tiles[key] = (packed[o:o + k], packed[o + k:o + 2 * k], k)
            o += 2 * k
        if expand is not None:
            k = len(expand[0][0])
            tiles["expanded"] = (packed[o:o + k], packed[o + k:o + 2 * k], packed[o + 2 * k:o + 3 * k], k, expand[1], expand[2])
        return self._layers(n, d_tok, d_slot, d_pos, tiles, int(pos.max()), None, n <= MOE_GEMV_TOKENS)

    def _expand_plan(self, slot: np.ndarray, pos: np.ndarray):
        """When the step's sequences bring enough tokens each: ((tile_first, tile_count, tile_kv_row), [(slot, keys, row)],
        rows) — tiles of the expanded attention kernel, and where each sequence's keys 0 .. its last position go in the
        step's expanded key / value buffers.  None: the folded (decode) form serves the step."""
        if not self.expand_tile:
            return None
        n = len(slot)
        brk = np.flatnonzero((slot[1:] != slot[:-1]) | (pos[1:] != pos[:-1] + 1)) + 1
        starts, ends = np.concatenate([[0], brk]), np.concatenate([brk, [n]])
        if n < EXPAND_MIN_TOKENS * len(starts):
            return None
        first, count, kvrow, hist, rows, seen = [], [], [], [], 0, {}
        for s, e in zip(starts, ends):
            sl, keys = int(slot[s]), int(pos[e - 1]) + 1
            if sl in seen:          # a sequence in two runs of one step: not a case worth a second copy of its keys
                return None
            seen[sl] = rows
            f = np.arange(s, e, self.expand_tile)
            first.append(f)
            count.append(np.minimum(self.expand_tile, e - f))
            kvrow.append(np.full(len(f), rows))
            hist.append((sl, keys, rows))
            rows += keys
        per_row = max(la.mixer.heads * (la.mixer.dim + la.mixer.vdim) for la in self.cfg.layers) * 2
        if rows * per_row > EXPAND_MAX_BYTES:
            return None
        return ((np.concatenate(first).astype(np.int32), np.concatenate(count).astype(np.int32),
                 np.concatenate(kvrow).astype(np.int32)), hist, rows)

    def _splits(self, n_tiles: int, H: int, max_pos: int) -> int:
        """Key splits of the attention launch: enough CTAs to fill the GPU when few tokens attend over many keys."""
        groups = -(-((H + 3) // 4) // 8)
        ctas = n_tiles * groups
        key_tiles = max_pos // 32 + 1
        if ctas >= self.sm_count or key_tiles <= 2:
            return 1
        return max(1, min(key_tiles, -(-2 * self.sm_count // ctas), 64))

    def _layers(self, n, d_tok, d_slot, d_pos, tiles, max_pos, n_split, gemv_experts) -> torch.Tensor:
        m, cfg, L, dt, dev = self.m, self.cfg, self.L, self.dt, self.dev
        W, nl = cfg.width, cfg.n_layer
        tdt = m.dtype
        st = torch.cuda.current_stream(dev).cuda_stream
        f32 = dict(dtype=torch.float32, device=dev)
        act = dict(dtype=tdt, device=dev)
        streams = torch.empty(nl + 1, n, W, **f32)      # the embedding output and every layer's result
        avg = [torch.empty(n, W, **f32), torch.empty(n, W, **f32)]
        xmid = torch.empty(n, W, **f32)
        h = torch.empty(n, W, **act)
        xc = torch.empty(n, W, **act)
        ffo = torch.empty(n, W, **f32)
        _lib.lm_check(L.ao_lm_embed(_p(m.embed), dt, _p(d_tok), n, W, _p(streams), st), "embed")
        x = streams[0]
        launches = 1
        for i, lay in enumerate(m.layers):
            a, f = lay.args.mixer, lay.args.mlp
            H, dn, dr, dv, R = a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank
            _lib.lm_check(L.ao_lm_token_shift(_p(x), _p(lay.shift), dt, _p(lay.shift_state.prev), _p(d_slot), _p(d_pos), n, W,
                                              _p(h), st), "token_shift")
            proj = torch.mm(h, lay.w_in.t())
            src = m.layers[a.kv_from] if a.kv_from is not None else lay
            cache = src.kv_cache
            S = cache.c.shape[1]
            qn = torch.empty(H, n, dn, **act)
            qr = torch.empty(n, H, dr, **f32)
            gate = torch.empty(n, H, **f32)
            own = a.kv_from is None
            _lib.lm_check(L.ao_lm_latent_prep(
                _p(proj), dt, proj.shape[1], n, H, dn, dr, R, lay.q_off, lay.kv_off, lay.g_off, _p(lay.c_norm), cfg.norm_eps,
                a.rot_dims, _p(lay.inv_freq), _p(d_slot), _p(d_pos), _p(cache.c) if own else None,
                _p(cache.kr) if own else None, S, _p(qn), _p(qr), _p(gate), st), "latent_prep")
            xp = tiles.get("expanded") if self.expand_ok[(dn, dr, dv)] else None
            if xp is not None:
                y = self._attend_expanded(lay, a, cache, xp, qn, qr, gate, d_slot, d_pos, n, st)
                launches += 2 + 2 * len(xp[4])
            else:
                y = self._attend_folded(lay, a, cache, tiles, qn, qr, gate, d_slot, d_pos, n, max_pos, n_split, st)
                launches += 4 + (1 if self._last_splits > 1 else 0)
            nxt = avg[i & 1]
            launches += 4   # token shift, input projection, split / cache append, residual add with norm
            if f is None:
                _lib.lm_check(L.ao_lm_residual_norm(
                    _p(x), _p(y), dt, _p(lay.norm1), dt, cfg.residual_mult, cfg.norm_eps, n, W, _p(streams[i + 1]),
                    _p(lay.shift_state.prev), _p(d_slot), _p(streams), i + 1, n * W, _p(lay.dwa), _p(nxt), None, st),
                    "residual_norm")
                x = nxt
                continue
            _lib.lm_check(L.ao_lm_residual_norm(
                _p(x), _p(y), dt, _p(lay.norm1), dt, cfg.residual_mult, cfg.norm_eps, n, W, _p(xmid),
                _p(lay.shift_state.prev), _p(d_slot), None, 0, 0, None, None, _p(xc), st), "residual_norm")
            launches += self._experts(lay, f, xc, ffo, n, gemv_experts, st)
            _lib.lm_check(L.ao_lm_residual_norm(
                _p(xmid), _p(ffo), _lib.DT_F32, _p(lay.norm2), dt, cfg.residual_mult, cfg.norm_eps, n, W, _p(streams[i + 1]),
                None, None, _p(streams), i + 1, n * W, _p(lay.dwa), _p(nxt), None, st), "residual_norm")
            launches += 1
            x = nxt
        self.launches = launches
        return x

    def _attend_folded(self, lay, a, cache, tiles, qn, qr, gate, d_slot, d_pos, n, max_pos, n_split, st) -> torch.Tensor:
        """Attention over the cached latents themselves: the key up-projection is folded into the query and the value
        up-projection follows the weighted sum of latents (what a decoded token costs least with) -> [n][W]."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, dr, dv, R = a.heads, a.rot_dim, a.vdim, a.kv_rank
        S = cache.c.shape[1]
        # q_abs[h] = q_n[h] @ uk[h]  (fp32 result)
        qa = torch.bmm(qn, lay.uk, out_dtype=torch.float32) if tdt == torch.bfloat16 else torch.bmm(qn, lay.uk)
        tf, tc, nt = tiles[(H, R, dr)]
        ns = n_split if n_split is not None else self._splits(nt, H, max_pos)
        self._last_splits = ns
        ws_bytes = int(L.ao_lm_latent_attention_workspace_bytes(n, H, R, ns))
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        olat = torch.empty(n, H, R, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_latent_attention(
            _p(qa), _p(qr), _p(cache.c), _p(cache.kr), dt, S, _p(d_slot), _p(d_pos), _p(tf), _p(tc), nt, n, H, R, dr,
            a.scale, _p(lay.sink), _p(gate), max_pos, ns, _p(ws), ws.numel(), _p(olat), st), "latent_attention")
        ov = torch.bmm(olat.transpose(0, 1), lay.uvT)                          # [H][n][dv]
        return torch.mm(ov.transpose(0, 1).reshape(n, H * dv), lay.o.t())      # [n][W]

    def _attend_expanded(self, lay, a, cache, xp, qn, qr, gate, d_slot, d_pos, n, st) -> torch.Tensor:
        """Attention of prompt portions over per-head keys and values: every sequence's cached latents 0 .. its last
        position are up-projected by two GEMMs, then one kernel runs all (token tile, head) pairs -> [n][W]."""
        L, dt, dev, tdt = self.L, self.dt, self.dev, self.m.dtype
        H, dn, dr, dv = a.heads, a.dim, a.rot_dim, a.vdim
        tf, tc, trow, nt, hist, rows = xp
        kx = torch.empty(rows, H * dn, dtype=tdt, device=dev)
        vx = torch.empty(rows, H * dv, dtype=tdt, device=dev)
        for sl, keys, r0 in hist:
            c = cache.c[sl, :keys]
            torch.mm(c, lay.ukx.t(), out=kx[r0:r0 + keys])
            torch.mm(c, lay.uvx, out=vx[r0:r0 + keys])
        oh = torch.empty(n, H * dv, dtype=tdt, device=dev)
        _lib.lm_check(L.ao_lm_latent_attention_expanded(
            _p(qn), _p(qr), _p(kx), _p(vx), _p(cache.kr), dt, cache.c.shape[1], _p(d_slot), _p(d_pos), _p(tf), _p(tc), _p(trow),
            nt, n, H, dn, dr, dv, a.scale, _p(lay.sink), _p(gate), _p(oh), st), "latent_attention_expanded")
        return torch.mm(oh, lay.o.t())

    def _experts(self, lay, f, xc, ffo, n, gemv, st) -> int:
        """ffo (fp32 [n][W]) = shared expert + sum of the chosen experts weighted by their router scores."""
        L, dt, dev, W = self.L, self.dt, self.dev, self.cfg.width
        tdt = self.m.dtype
        ridx = torch.empty(n, f.top, dtype=torch.int32, device=dev)
        rwt = torch.empty(n, f.top, dtype=torch.float32, device=dev)
        if gemv or f.experts > 1024:
            _lib.lm_check(L.ao_lm_router_topk(_p(xc), _p(lay.router), dt, n, W, f.experts, f.top, _p(ridx), _p(rwt), st), "router_topk")
        else:   # many tokens: the logits as one GEMM with an fp32 result, then softmax and choice per token
            z = torch.mm(xc, lay.router.t(), out_dtype=torch.float32) if tdt == torch.bfloat16 else torch.mm(xc, lay.router.t())
            _lib.lm_check(L.ao_lm_router_topk_logits(_p(z), n, f.experts, f.top, _p(ridx), _p(rwt), st), "router_topk_logits")
        esz = lay.wgu.element_size()
        if gemv:
            if f.shared_ff:
                sa = torch.empty(n, f.shared_ff, dtype=tdt, device=dev)
                _lib.lm_check(L.ao_lm_expert_gate_up(_p(xc), _p(lay.sgu), _p(lay.sgu) + f.shared_ff * W * esz, dt, None, n, 1, W,
                                                     f.shared_ff, 0, f.shared_limit, GLU_ALPHA, _p(sa), st), "expert_gate_up")
                _lib.lm_check(L.ao_lm_expert_down(_p(sa), _p(lay.sd), dt, None, None, n, 1, W, f.shared_ff, 0, _p(ffo), st),
                              "expert_down")
            return (3 if f.shared_ff else 1) + chosen_experts(L, dt, xc, ridx, rwt, lay.wgu, lay.wd, ffo, f.limit, GLU_ALPHA, 1.0,
                                                             True, bool(f.shared_ff), st)
        launches = 1
        if f.shared_ff:
            sgu = torch.mm(xc, lay.sgu.t())
            sa = torch.empty(n, f.shared_ff, dtype=tdt, device=dev)
            _lib.lm_check(L.ao_lm_glu_act(_p(sgu), dt, n, f.shared_ff, f.shared_limit, GLU_ALPHA, _p(sa), st), "glu_act")
            sd = torch.mm(sa, lay.sd.t())
            ffo.zero_()
            _lib.lm_check(L.ao_lm_add_cast(_p(sd), dt, n * W, _p(ffo), st), "add_cast")
            launches += 5
        # rows sorted by expert around grouped GEMMs (bf16) or one exact GEMM pair per expert that has rows (fp32)
        return launches + chosen_experts(L, dt, xc, ridx, rwt, lay.wgu, lay.wd, ffo, f.limit, GLU_ALPHA, 1.0, False,
                                         bool(f.shared_ff), st)

    def _logits(self, x: torch.Tensor, rows: List[int]) -> torch.Tensor:
        """fp32 logits of the given rows: output norm (one number as weight) then the head product with an fp32 result."""
        m, dev = self.m, self.dev
        k = len(rows)
        if k == 0:
            return torch.empty(0, self.cfg.vocab_size, dtype=torch.float32, device=dev)
        d_rows = torch.tensor(rows, dtype=torch.int32).to(dev, non_blocking=True)
        return self._logits_dev(x, d_rows, k)

    def _logits_dev(self, x, d_rows, k, out=None):
        m, dev = self.m, self.dev
        st = torch.cuda.current_stream(dev).cuda_stream
        xn = torch.empty(k, self.cfg.width, dtype=m.dtype, device=dev)
        _lib.lm_check(self.L.ao_lm_scalar_norm_rows(_p(x), _p(d_rows), k, self.cfg.width, _p(m.final_norm), self.dt,
                                                    self.cfg.norm_eps, _p(xn), st), "scalar_norm_rows")
        if m.dtype == torch.bfloat16:
            lg = torch.mm(xn, m.head.t(), out_dtype=torch.float32)
        else:
            lg = torch.mm(xn, m.head.t())
        if out is not None:
            out.copy_(lg)
            return out
        return lg


class GraphDecodeEngine:
    """One decoded token per sequence and step for a fixed batch (slots 0 .. B-1, all at the same position), with the
    tokens, positions and every launch parameter in device memory: the step is captured into a CUDA graph once and
    replayed per token.  Same surface as the Llama DecodeEngine (set_state / step / capture / tok / next_tok / logits)."""

    def __init__(self, model: Bitipel, batch_size: int = 1, temperature: float = 0.8, top_k: Optional[int] = 200):
        assert model.states is not None and model.max_batch_size >= batch_size, "call model.setup_caches first"
        self.model, self.cfg, self.B = model, model.config, batch_size
        self.eng = model.step_engine
        self.device = dev = model.device
        self.temperature, self.top_k = temperature, top_k
        self.S = model.max_seq_length
        B = batch_size
        self.tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.next_tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.pos = torch.zeros(B, dtype=torch.int32, device=dev)
        self.slot = torch.arange(B, dtype=torch.int32, device=dev)
        self.rows = torch.arange(B, dtype=torch.int32, device=dev)
        self.tile_first = torch.arange(B, dtype=torch.int32, device=dev)
        self.tile_count = torch.ones(B, dtype=torch.int32, device=dev)
        self.logits = torch.zeros(B, self.cfg.vocab_size, dtype=torch.float32, device=dev)
        self.tiles = {key: (self.tile_first, self.tile_count, B) for key in self.eng.tile_tokens}
        # a fixed number of key splits over the whole cache: CTAs past a sequence's length leave at once
        ctas = B * max(-(-H // 16) for H, _, _ in self.eng.tile_tokens)
        self.n_split = max(1, min(-(-self.S // 32), -(-2 * self.eng.sm_count // ctas), 64))
        self.graph = None
        self.graph_stream = None
        self._noise = None
        self._host_pos = 0
        self.launches_per_step = 0
        self.mega = False
        self.tp = None

    def _launch_step(self):
        eng = self.eng
        x = eng._layers(self.B, self.tok, self.slot, self.pos, self.tiles, self.S - 1, self.n_split, True)
        eng._logits_dev(x, self.rows, self.B, out=self.logits)
        self._sample(self.logits)
        self.tok.copy_(self.next_tok)
        self.pos.add_(1)
        self.launches_per_step = eng.launches + 5

    def _sample(self, logits):
        """Greedy: argmax over the fp32 logits.  Otherwise the framework's sampling kernel (temperature, exact top-k,
        exponential-noise argmax), which reads bf16 logits."""
        st = torch.cuda.current_stream(self.device).cuda_stream
        if self.temperature == 0.0:
            _lib.lm_check(self.eng.L.ao_lm_argmax(logits.data_ptr(), logits.stride(0), self.B, logits.shape[1],
                                                  self.next_tok.data_ptr(), st), "argmax")
            return
        if self._noise is None:
            self._noise = torch.empty(logits.shape, dtype=torch.float32, device=self.device)
        noise = self._noise.exponential_(1)
        lb = logits.to(torch.bfloat16)
        _lib.check(_lib.lib().ao_b200_sample(lb.data_ptr(), lb.stride(0), self.B, lb.shape[1], float(self.temperature),
                                             0 if self.top_k is None else int(self.top_k), noise.data_ptr(), noise.stride(0),
                                             self.next_tok.data_ptr(), st), "sample")

    def capture(self):
        tok0, pos0 = self.tok.clone(), self.pos.clone()
        saved = [(l.shift_state.prev.clone()) for l in self.model.layers]
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):   # warm-up outside the capture (library handles, attribute calls)
                self._launch_step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._launch_step()
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        for l, s in zip(self.model.layers, saved):   # the trial steps wrote token-shift memory (cache rows at pos0.. are rewritten anyway)
            l.shift_state.prev.copy_(s)
        torch.cuda.synchronize(self.device)
        return self

    def capture_streaming(self, h_tok, h_out):
        assert h_tok.is_pinned() and h_out.is_pinned() and self.graph is not None
        tok0, pos0 = self.tok.clone(), self.pos.clone()
        saved = [(l.shift_state.prev.clone()) for l in self.model.layers]
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.tok.copy_(h_tok, non_blocking=True)
            self._launch_step()
            h_out.copy_(self.next_tok, non_blocking=True)
        self.graph_stream = g
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        for l, s in zip(self.model.layers, saved):
            l.shift_state.prev.copy_(s)
        torch.cuda.synchronize(self.device)
        return self

    def set_state(self, tokens: torch.Tensor, pos: int):
        """tokens [B] = the token every sequence feeds next, pos = its position (the prompt's length)."""
        if not 0 <= pos < self.S:
            raise ValueError(f"position {pos} outside the cache (max_seq_length {self.S})")
        self.tok.copy_(tokens.reshape(-1).to(torch.int64))
        self.pos.fill_(pos)
        self._host_pos = pos

    def step(self) -> torch.Tensor:
        if self._host_pos >= self.S:
            raise RuntimeError(f"decode step at position {self._host_pos} would run past the cache (max_seq_length {self.S})")
        self._host_pos += 1
        st = self.model.states
        for b in range(self.B):
            if b in st.length:
                st.length[b] = self._host_pos
        if self.graph is not None:
            self.graph.replay()
        else:
            self._launch_step()
        return self.next_tok

    def check_status(self):
        return None
