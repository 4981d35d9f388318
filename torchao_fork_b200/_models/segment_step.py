"""What the step functions of the slotted sequence models share: a step is a list of segments (the next tokens of some
sequences: prompt portions and single decoded tokens in any mix); its rows get device-side metadata (slot, position, rows
of the same segment in front and behind, tiles for recurrences and for every attention shape, the segments themselves)
in one host-to-device copy; long steps are cut into pieces; wanted rows go through the output norm and the head product.
A model family derives its StepEngine from SegmentStepEngine and supplies `_attention_shapes`, `_layers` and
`_logits_dev`.  GraphDecodeEngine wraps a family's layer loop for one token per sequence with all metadata in device
memory, captured into a CUDA graph (the Llama DecodeEngine's role).
"""
import ctypes
from typing import Dict, List, Optional, Sequence, Tuple, Union

import numpy as np
import torch

from .. import _lib

# a portion longer than this is cut into pieces (bounds the workspace)
MAX_STEP_TOKENS = 4096
# rows of a recurrence tile; a step whose segments all fit one tile scans in one launch
SCAN_TILE = 32
# steps that bring at least this many rows per sequence (on average) attend with the tensor-core kernel (bf16 models,
# head sizes it covers); decoded tokens and short portions use the fp32 kernel, which shares a key block between the
# few rows of a tile and all query heads of a key/value head
PROMPT_MIN_ROWS = 16
# rows of a tile of a matrix-state recurrence: a step with a longer segment runs the recurrence in its tiled form
REC_TILE = 64


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


class StepMeta:
    """Device-side description of a step's rows: per row slot / position / rows of its segment in front (back) and
    behind (ahead); tiles of the recurrences; tiles of every attention shape."""
    n: int
    slot: torch.Tensor
    pos: torch.Tensor
    back: torch.Tensor
    ahead: torch.Tensor
    scan: tuple          # (tile_first, tile_count, n_tiles, seg_tile0 | None, seg_tiles | None, n_segments)
    attn: Dict[tuple, tuple]   # attention shape -> (tile_first, tile_count, n_tiles, tensor-core form?)
    seg: tuple           # (first row, rows, n) of the step's segments, whole
    rec: Optional[tuple] = None   # tiles of the matrix-state recurrences (as `scan`), when some segment is longer than one tile


def segments_of(slot: np.ndarray, pos: np.ndarray):
    """(first row, rows) of every run of consecutive positions of one sequence."""
    n = len(slot)
    brk = np.flatnonzero((slot[1:] != slot[:-1]) | (pos[1:] != pos[:-1] + 1)) + 1
    starts = np.concatenate([[0], brk]).astype(np.int64)
    ends = np.concatenate([brk, [n]]).astype(np.int64)
    return starts, ends - starts


def scan_tiles(starts: np.ndarray, counts: np.ndarray, tile: int):
    """Tiles of <= `tile` rows inside the segments, and per segment its first tile and tile count (None, None when
    every segment is one tile)."""
    first, count, seg0, segn = [], [], [], []
    for s, c in zip(starts, counts):
        f = np.arange(s, s + c, tile)
        seg0.append(len(first))
        segn.append(len(f))
        first += f.tolist()
        count += np.minimum(tile, s + c - f).tolist()
    first, count = np.asarray(first, np.int32), np.asarray(count, np.int32)
    if max(segn) == 1:
        return first, count, None, None
    return first, count, np.asarray(seg0, np.int32), np.asarray(segn, np.int32)


def chunk_tiles(starts: np.ndarray, counts: np.ndarray, pos: np.ndarray, tile_rows: int, chunk: int):
    """Runs of <= tile_rows rows of one segment that lie inside ONE chunk of the sequence's positions."""
    first, count = [], []
    for s, c in zip(starts, counts):
        r, end = int(s), int(s + c)
        while r < end:
            room = chunk - int(pos[r]) % chunk          # rows up to the chunk's end
            k = min(tile_rows, room, end - r)
            first.append(r)
            count.append(k)
            r += k
    return np.asarray(first, np.int32), np.asarray(count, np.int32)


class SegmentStepEngine:
    def __init__(self, model):
        assert model.device.type == "cuda", f"{type(model).__name__} runs on CUDA only: there is no CPU path"
        self.m, self.cfg = model, model.config
        self.dev = model.device
        self.dt = _lib.DT_BF16 if model.dtype == torch.bfloat16 else _lib.DT_F32
        self.L = _lib.lm()
        if model.dtype == torch.float32:
            # true fp32 products: no TF32 / reduced-precision accumulation in the library GEMMs
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        self.launches = 0
        self.sm_count = torch.cuda.get_device_properties(self.dev).multi_processor_count
        # rows of one sequence that an attention CTA takes, per attention shape (H, G, d, dv, chunk) of the model
        self.attn_keys, self.prompt_keys = {}, {}
        for shape in self._attention_shapes():
            rows, chunk, prompt_rows = self._attention_plan(shape)
            if rows <= 0:
                raise NotImplementedError(f"attention shape not covered by the kernels: {shape}")
            self.attn_keys[shape] = (rows, chunk, False)
            if prompt_rows > 0:
                self.prompt_keys[shape] = (prompt_rows, chunk, True)

    def _attention_shapes(self):
        """One hashable shape per kind of attention layer of the model; (H, G, d, dv, chunk) for the chunk kernels."""
        return []

    def _attention_plan(self, shape):
        """-> (rows of one sequence that an attention CTA takes, span of positions that a tile must not leave, rows per
        CTA of the tensor-core form for prompt portions or 0).  A family whose attention is another kernel overrides it."""
        H, G, d, dv, chunk = shape
        tr, pr = ctypes.c_int(), ctypes.c_int()
        _lib.lm_check(self.L.ao_lm_chunk_attention_plan(self.dt, H, G, d, dv, ctypes.byref(tr)), "chunk_attention_plan")
        _lib.lm_check(self.L.ao_lm_chunk_attention_prompt_plan(self.dt, H, G, d, dv, ctypes.byref(pr)), "chunk_attention_prompt_plan")
        return tr.value, chunk, pr.value

    # ------------------------------------------------------------------------------------------------ public
    @torch.no_grad()
    def step(self, segments: Sequence[Tuple[int, Union[torch.Tensor, Sequence[int]]]],
             want: Union[str, Sequence[Sequence[int]]] = "last") -> torch.Tensor:
        """segments: [(slot, tokens)] — the next tokens of the sequences in those slots (each slot at most once).
        want: "last" (the last token of every segment), "all", or per segment the indices among ITS tokens.
        Returns fp32 logits [wanted][vocab] in segment order.  Positions continue from the state manager's lengths."""
        st = self.m.states
        toks, slots, poss, rows = [], [], [], []
        at = 0
        seen = set()
        for k, (slot, t) in enumerate(segments):
            t = torch.as_tensor(t).reshape(-1).to(torch.int64).cpu().numpy() if not isinstance(t, np.ndarray) else t.astype(np.int64)
            n = len(t)
            assert n > 0 and slot not in seen, "every slot at most once per step, with at least one token"
            seen.add(slot)
            p0 = st.extend(slot, n)
            toks.append(t)
            slots.append(np.full(n, slot, np.int32))
            poss.append(np.arange(p0, p0 + n, dtype=np.int32))
            sel = [n - 1] if want == "last" else list(range(n)) if want == "all" else list(want[k])
            rows += [at + int(i) for i in sel]
            at += n
        tok, slot, pos = np.concatenate(toks), np.concatenate(slots), np.concatenate(poss)
        if (tok < 0).any() or (tok >= self.cfg.vocab_size).any():
            raise ValueError("token id outside the vocabulary")
        total = at
        if total <= MAX_STEP_TOKENS:
            x = self._run(tok, slot, pos)
            return self._logits(x, rows)
        # long portions: pieces of at most MAX_STEP_TOKENS tokens, in order (a piece may end inside a segment; the state
        # that a piece leaves is what the next one starts from, exactly as between steps)
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
    def _meta(self, slot: np.ndarray, pos: np.ndarray, tok: np.ndarray):
        """All of a piece's metadata in ONE host-to-device copy -> (device tokens, StepMeta)."""
        n = len(slot)
        starts, counts = segments_of(slot, pos)
        back, ahead = np.empty(n, np.int32), np.empty(n, np.int32)
        for s, c in zip(starts, counts):
            back[s:s + c] = np.arange(c)
            ahead[s:s + c] = np.arange(c - 1, -1, -1)
        sf, sc, seg0, segn = scan_tiles(starts, counts, SCAN_TILE)
        parts = [tok.view(np.int32), slot, pos, back, ahead, sf, sc, starts.astype(np.int32), counts.astype(np.int32)]
        if seg0 is not None:
            parts += [seg0, segn]
        attn_np = {}
        prompt = n >= PROMPT_MIN_ROWS * len(starts)
        meta_shapes = {shape: (self.prompt_keys[shape] if prompt and shape in self.prompt_keys else key)
                       for shape, key in self.attn_keys.items()}
        for key in sorted(set(meta_shapes.values())):
            attn_np[key] = chunk_tiles(starts, counts, pos, key[0], key[1])
            parts += list(attn_np[key])
        rec = scan_tiles(starts, counts, REC_TILE) if getattr(self, "matrix_recurrences", False) else None
        if rec is not None and rec[2] is not None:
            parts += list(rec)
        packed = torch.from_numpy(np.concatenate(parts)).to(self.dev, non_blocking=True)
        o = [0]

        def take(k):
            v = packed[o[0]:o[0] + k]
            o[0] += k
            return v

        d_tok = take(2 * n).view(torch.int64)
        meta = StepMeta()
        meta.n = n
        meta.slot, meta.pos, meta.back, meta.ahead = take(n), take(n), take(n), take(n)
        nt = len(sf)
        tf, tc = take(nt), take(nt)
        meta.seg = (take(len(starts)), take(len(starts)), len(starts))
        if seg0 is not None:
            meta.scan = (tf, tc, nt, take(len(seg0)), take(len(seg0)), len(seg0))
        else:
            meta.scan = (tf, tc, nt, None, None, 0)
        tables = {}
        for key in sorted(attn_np):
            k = len(attn_np[key][0])
            tables[key] = (take(k), take(k), k, key[2])
        meta.attn = {shape: tables[key] for shape, key in meta_shapes.items()}
        if rec is not None and rec[2] is not None:
            meta.rec = (take(len(rec[0])), take(len(rec[0])), len(rec[0]), take(len(rec[2])), take(len(rec[2])), len(rec[2]))
        return d_tok, meta

    def _run(self, tok: np.ndarray, slot: np.ndarray, pos: np.ndarray) -> torch.Tensor:
        """One piece through all layer runs -> the streams [n][S][W], fp32."""
        d_tok, meta = self._meta(slot, pos, tok)
        return self._layers(d_tok, meta)

    def _mm_f32(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """a @ w^T with an fp32 result (what fp32 kernels read next)."""
        if a.dtype == torch.bfloat16:
            return torch.mm(a, w.t(), out_dtype=torch.float32)
        return torch.mm(a, w.t())

    def _splits(self, ctas: int, chunk: int) -> int:
        """Key splits of the fp32 attention kernel: enough CTAs to fill the GPU when few rows attend over a long chunk
        (a decoded token late in its chunk).  It depends on sizes only, so a captured graph keeps it."""
        key_blocks = -(-chunk // 32)
        if ctas >= self.sm_count or key_blocks <= 2:
            return 1
        return max(1, min(key_blocks, -(-4 * self.sm_count // ctas), 64))

    def _scan_ws(self, meta: StepMeta, channels: int):
        tf, tc, nt, seg0, segn, ns = meta.scan
        if seg0 is None:
            return None
        nbytes = int(self.L.ao_lm_scan_workspace_bytes(nt, channels))
        return torch.empty(nbytes // 4, dtype=torch.float32, device=self.dev)

    def _logits(self, x: torch.Tensor, rows: List[int]) -> torch.Tensor:
        """fp32 logits of the given rows: sum of the streams, output norm, head product with an fp32 result."""
        k = len(rows)
        if k == 0:
            return torch.empty(0, self.cfg.vocab_size, dtype=torch.float32, device=self.dev)
        d_rows = torch.tensor(rows, dtype=torch.int32).to(self.dev, non_blocking=True)
        return self._logits_dev(x, d_rows, k)

    @torch.no_grad()
    def layer_sums(self, slot: int, tokens) -> Tuple[torch.Tensor, torch.Tensor]:
        """Debugging aid: runs `tokens` as the next tokens of `slot` and returns (logits of all rows, the sum of the
        streams (of the residual, where there is one stream) after every layer run [runs][n][W])."""
        st = self.m.states
        t = np.asarray(tokens, np.int64)
        p0 = st.extend(slot, len(t))
        d_tok, meta = self._meta(np.full(len(t), slot, np.int32), np.arange(p0, p0 + len(t), dtype=np.int32), t)
        sums = []
        x = self._layers(d_tok, meta, after_run=lambda r, x: sums.append(x.sum(1) if x.dim() == 3 else x.clone()))
        return self._logits(x, list(range(len(t)))), torch.stack(sums)


class GraphDecodeEngine:
    """One decoded token per sequence and step for a fixed batch (slots 0 .. B-1, all at the same position), with the
    tokens, positions and every launch parameter in device memory: the step is captured into a CUDA graph once and
    replayed per token.  Same surface as the Llama DecodeEngine (set_state / step / capture / tok / next_tok / logits)."""

    def __init__(self, model, batch_size: int = 1, temperature: float = 0.8, top_k: Optional[int] = 200):
        assert model.states is not None and model.max_batch_size >= batch_size, "call model.setup_caches first"
        self.model, self.cfg, self.B = model, model.config, batch_size
        self.eng = model.step_engine
        self.device = dev = model.device
        self.temperature, self.top_k = temperature, top_k
        self.S = model.max_seq_length
        B = batch_size
        self.tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.next_tok = torch.zeros(B, dtype=torch.int64, device=dev)
        self.logits = torch.zeros(B, self.cfg.vocab_size, dtype=torch.float32, device=dev)
        ar = torch.arange(B, dtype=torch.int32, device=dev)
        ones, zeros = torch.ones(B, dtype=torch.int32, device=dev), torch.zeros(B, dtype=torch.int32, device=dev)
        meta = StepMeta()
        meta.n = B
        meta.slot, meta.pos, meta.back, meta.ahead = ar, torch.zeros(B, dtype=torch.int32, device=dev), zeros, zeros
        meta.scan = (ar, ones, B, None, None, 0)       # one row per sequence: every tile is a whole segment
        meta.attn = {shape: (ar, ones, B, False) for shape in self.eng.attn_keys}
        meta.seg = (ar, ones, B)
        self.meta, self.pos, self.rows = meta, meta.pos, ar
        self.graph = None
        self.graph_stream = None
        self._noise = None
        self._host_pos = 0
        self.launches_per_step = 0
        self.mega = False
        self.tp = None

    def _launch_step(self):
        eng = self.eng
        x = eng._layers(self.tok, self.meta)
        eng._logits_dev(x, self.rows, self.B, out=self.logits)
        self._sample(self.logits)
        self.tok.copy_(self.next_tok)
        self.pos.add_(1)
        self.launches_per_step = eng.launches + 6

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

    def _state_tensors(self):
        return [t for rs in self.model.run_state for part in rs.parts() for t in part.buffers()]

    def _with_saved_state(self, fn):
        """Runs fn (trial steps / a capture, which execute the step) and puts tokens, positions and every recurrent
        state of the batch's slots back as they were."""
        tok0, pos0 = self.tok.clone(), self.pos.clone()
        saved = [t[: self.B].clone() for t in self._state_tensors()]
        fn()
        torch.cuda.synchronize(self.device)
        self.tok.copy_(tok0)
        self.pos.copy_(pos0)
        for t, s in zip(self._state_tensors(), saved):
            t[: self.B].copy_(s)
        torch.cuda.synchronize(self.device)

    def capture(self):
        def trial():
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                for _ in range(2):   # warm-up outside the capture (library handles, attribute calls)
                    self._launch_step()
            torch.cuda.current_stream(self.device).wait_stream(side)
        self._with_saved_state(trial)

        def cap():
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._launch_step()
        self._with_saved_state(cap)
        return self

    def capture_streaming(self, h_tok, h_out):
        assert h_tok.is_pinned() and h_out.is_pinned() and self.graph is not None

        def cap():
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.tok.copy_(h_tok, non_blocking=True)
                self._launch_step()
                h_out.copy_(self.next_tok, non_blocking=True)
            self.graph_stream = g
        self._with_saved_state(cap)
        return self

    def set_state(self, tokens: torch.Tensor, pos: int):
        """tokens [B] = the token every sequence feeds next, pos = its position (the prompt's length)."""
        if not 0 <= pos < self.S:
            raise ValueError(f"position {pos} outside what setup_caches allowed (max_seq_length {self.S})")
        self.tok.copy_(tokens.reshape(-1).to(torch.int64))
        self.pos.fill_(pos)
        self._host_pos = pos

    def step(self) -> torch.Tensor:
        if self._host_pos >= self.S:
            raise RuntimeError(f"decode step at position {self._host_pos} is past max_seq_length {self.S}")
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
