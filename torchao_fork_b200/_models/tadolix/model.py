"""Tadolix: a decoder-only language model built from
  * a residual kept as several fp32 streams (hyper-connections): a sublayer reads a learned combination of the streams
    through an RMS norm whose weight is stored as the deviation from one, and its result is written back through a
    learned mixing matrix; the model's output reads the plain sum of the streams,
  * a short causal convolution over time in front of every mixer, added to the mixer's input,
  * two kinds of mixer: "parallel" = attention over chunks of the sequence (grouped heads, unit-RMS queries and keys,
    soft-capped scores, a learned bias per distance bucket, a sigmoid gate on the output) side by side with a minimal
    GRU whose gates read only the current token; "rglru" = a gelu branch times a real-gated linear recurrence over a
    short convolution, gates from block-diagonal matrices,
  * a dense tanh-GELU gated feed-forward (a layer may have none),
  * a span of layers that runs several times in a row with the same weights and separate state per pass,
  * token embeddings times a constant plus sinusoidal positions.

This module holds the configuration (every size and constant is read from a checkpoint's config.json), the weights in
the layout the kernels want, and the per-sequence state (cache.py).  The compute is step.py.
Checkpoint tensor names: embed, head, final.norm, l<i>.{norm1,norm2,canon1,hc<q>.{in,out,mix}},
l<i>.mix.left.{q,k,v,rel,g,o}, l<i>.mix.right.{z,z.b,x,x.b,g,o}, l<i>.mix.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o},
l<i>.mlp.{gate,up,down}; linear weights are [out][in].
"""
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..cache import ConvState, RecurrentState, RingKVCache, SequenceStates
from ..checkpoint import read_config, read_safetensors

# fixed by the design
SINUSOID_BASE = 10000.0
RGLRU_DECAY = 8.0
MAX_STREAMS = 8     # what the stream kernels hold in registers
MAX_TAPS = 8


@dataclass
class ChunkAttentionArgs:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    chunk: int          # positions per chunk of the mask
    bias_max: int       # distance at which the bias buckets end
    scale: float
    softcap: float      # 0: scores are not capped


@dataclass
class ParallelArgs:
    left: ChunkAttentionArgs
    right_width: int
    left_scale: float
    right_scale: float


@dataclass
class RgLruArgs:
    width: int
    blocks: int
    conv: int           # taps of the convolution in front of the recurrence


@dataclass
class LayerArgs:
    type: str                   # "parallel" | "rglru"
    mixer: object
    ff: int = 0                 # 0: no feed-forward


@dataclass
class TadolixArgs:
    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    streams: int = 0            # 0: one stream with a plain residual sum (no read-out / write-back weights)
    canon_taps: int = 0         # 0: no convolution in front of the mixers
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times)
    layers: List[LayerArgs] = field(default_factory=list)
    block_size: int = 1 << 30   # no built-in context limit: every state has a fixed size

    @property
    def n_layer(self):
        return len(self.layers)

    @property
    def runs(self) -> List[int]:
        """Layer index of every layer run, in order (a looped layer appears once per pass)."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    @classmethod
    def from_dict(cls, cfg: dict) -> "TadolixArgs":
        layers = []
        for i, lay in enumerate(cfg["layers"]):
            m, kind = lay["mixer"], lay["type"]
            if kind == "parallel":
                a = m["left"]
                left = ChunkAttentionArgs(heads=int(a["heads"]), kv_heads=int(a["kv_heads"]), dim=int(a["dim"]), vdim=int(a["vdim"]),
                                          chunk=int(a["mask"]["size"]), bias_max=int(a["bias_max"]), scale=float(a["scale"]),
                                          softcap=float(a.get("softcap") or 0.0))
                assert left.heads % left.kv_heads == 0, f"layer {i}: {left.heads} heads over {left.kv_heads} key/value heads"
                mixer = ParallelArgs(left, int(m["right"]["width"]), float(m["left_scale"]), float(m["right_scale"]))
            elif kind == "rglru":
                mixer = RgLruArgs(int(m["width"]), int(m["blocks"]), int(m["conv"]))
                assert mixer.width % mixer.blocks == 0 and 1 <= mixer.conv <= MAX_TAPS, f"layer {i}: {mixer}"
            else:
                raise NotImplementedError(f"layer {i}: mixer type {kind!r}")
            f = lay.get("mlp")
            if f and f.get("kind", "dense") != "dense":
                raise NotImplementedError(f"layer {i}: feed-forward kind {f.get('kind')!r}")
            layers.append(LayerArgs(kind, mixer, int(f["ff"]) if f else 0))
        loop = cfg.get("loop")
        if loop:
            loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
            assert 0 <= loop[0] <= loop[1] <= len(layers) and loop[2] >= 1, f"loop {loop}"
        streams = int(cfg.get("streams") or 0)
        taps = int((cfg.get("canon") or {}).get("taps") or 0)
        assert streams <= MAX_STREAMS and taps <= MAX_TAPS
        return cls(vocab_size=int(cfg["vocab"]), width=int(cfg["width"]), norm_eps=float(cfg["norm"]["eps"]),
                   embedding_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), streams=streams, canon_taps=taps,
                   loop=loop, layers=layers)

    def to_dict(self) -> dict:
        out = []
        for lay in self.layers:
            m = lay.mixer
            if lay.type == "parallel":
                a = m.left
                mx = {"left": {"bias_max": a.bias_max, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads,
                               "mask": {"size": a.chunk}, "scale": a.scale, "softcap": a.softcap, "vdim": a.vdim},
                      "left_scale": m.left_scale, "right": {"width": m.right_width}, "right_scale": m.right_scale}
            else:
                mx = {"blocks": m.blocks, "conv": m.conv, "width": m.width}
            out.append({"mixer": mx, "mlp": {"ff": lay.ff, "kind": "dense"} if lay.ff else None, "type": lay.type})
        cfg = {"architecture": "Tadolix", "embedding": {"scale": self.embedding_scale}, "layers": out,
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.width}
        if self.streams:
            cfg["streams"] = self.streams
        if self.canon_taps:
            cfg["canon"] = {"taps": self.canon_taps}
        if self.loop:
            cfg["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return cfg


def distance_bias_table(rel: torch.Tensor, bias_max: int, n_dist: int) -> torch.Tensor:
    """rel [B][H] (one row per bucket) -> fp32 [H][n_dist], column n = the bias at distance n: one bucket per distance
    below B // 2, then (B - B // 2) logarithmic steps up to bias_max, everything farther in the last bucket."""
    B = rel.shape[0]
    half = B // 2
    rows = []
    for n in range(n_dist):
        if n < half:
            rows.append(n)
        elif half == 0 or bias_max <= half:
            rows.append(B - 1)
        else:
            rows.append(min(B - 1, half + int(math.floor(math.log(n / half) / math.log(bias_max / half) * (B - half)))))
    return rel.to(torch.float32)[torch.tensor(rows, dtype=torch.long, device=rel.device)].t().contiguous()


def _pattern(n_layer, width, heads, kv_heads, dim, chunk, ff, vocab, streams=4, taps=4, blocks=None):
    """n_layer layers, every third a parallel layer with a feed-forward, the others recurrent without."""
    layers = []
    for i in range(n_layer):
        if i % 3 == 0:
            a = ChunkAttentionArgs(heads, kv_heads, dim, dim, chunk, 2 * chunk, 1.0 / math.sqrt(dim) * 4.0, 30.0)
            layers.append(LayerArgs("parallel", ParallelArgs(a, width, 0.7, 1.1), ff))
        else:
            layers.append(LayerArgs("rglru", RgLruArgs(width, blocks or max(1, width // 256), 4), ff))
    return TadolixArgs(vocab, width, 1e-6, 8.0, streams, taps, None, layers)


# named random-init configurations (benchmarks and examples; checkpoints carry their own config.json)
tadolix_configs = {
    "Tadolix-test": lambda: _pattern(3, 128, 4, 2, 32, 16, 192, 512, streams=2, taps=3, blocks=4),
    # layers of the size of a 1-2 B parameter model / of a 7-8 B parameter model (a layer benchmark)
    "Tadolix-2k": lambda: _pattern(3, 2048, 16, 4, 128, 1024, 6144, 32000),
    "Tadolix-4k": lambda: _pattern(3, 4096, 32, 8, 128, 1024, 12288, 128256),
}


class _Layer:
    """One layer's tensors as the kernels read them (plain attributes; the module registers them as buffers)."""


class _RunState:
    """Per-sequence state of ONE layer run (a looped layer has one per pass)."""
    canon: Optional[ConvState] = None
    ring: Optional[RingKVCache] = None
    rec: Optional[RecurrentState] = None
    conv: Optional[ConvState] = None

    def parts(self):
        return [p for p in (self.canon, self.ring, self.rec, self.conv) if p is not None]


class Tadolix(nn.Module):
    def __init__(self, config: TadolixArgs, weights: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32), "Tadolix runs in bfloat16 or float32"
        self.config, self.dtype = config, dtype
        self.device = torch.device(device)
        self.max_batch_size = -1
        self.max_seq_length = -1
        self.states: Optional[SequenceStates] = None
        self.run_state: List[_RunState] = []
        self._step = None
        self._take(weights)

    # ------------------------------------------------------------------------------------------------ weights
    def _take(self, w: Dict[str, torch.Tensor]):
        cfg, dev, dt = self.config, self.device, self.dtype
        used = set()

        def get(name, shape=None):
            if name not in w:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            t = w[name]
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)}, the configuration asks for {tuple(shape)}")
            return t.to(device=dev, dtype=dt)

        def buf(name, t):
            self.register_buffer(name.replace(".", "__"), t.contiguous(), persistent=False)
            return getattr(self, name.replace(".", "__"))

        W, V, S = cfg.width, cfg.vocab_size, cfg.streams
        self.embed = buf("embed", get("embed", (V, W)))
        self.head = buf("head", get("head", (V, W)))
        self.final_norm = buf("final.norm", get("final.norm", (W,)))
        i2 = torch.arange((W + 1) // 2, dtype=torch.float64)
        self.pos_freq = buf("pos_freq", (SINUSOID_BASE ** (-2.0 * i2 / W)).to(dev))     # float64: the angle is formed in double
        self.layers: List[_Layer] = []
        for i, la in enumerate(cfg.layers):
            p, L = f"l{i}.", _Layer()
            L.args = la
            L.norm = [buf(p + "norm1", get(p + "norm1", (W,))), None]
            L.canon = buf(p + "canon1", get(p + "canon1", (W, cfg.canon_taps))) if cfg.canon_taps else None
            L.hc = [None, None]
            for q in (1, 2):
                if S and (q == 1 or la.ff):
                    L.hc[q - 1] = (buf(f"{p}hc{q}.in", get(f"{p}hc{q}.in", (S,))), buf(f"{p}hc{q}.out", get(f"{p}hc{q}.out", (S,))),
                                   buf(f"{p}hc{q}.mix", get(f"{p}hc{q}.mix", (S, S))))
            if la.type == "parallel":
                m = la.mixer
                a, Rw, q = m.left, m.right_width, p + "mix."
                H, G, d, dv = a.heads, a.kv_heads, a.dim, a.vdim
                parts = [get(q + "left.q", (H * d, W)), get(q + "left.k", (G * d, W)), get(q + "left.v", (G * dv, W)),
                         get(q + "left.g", (H * dv, W)), get(q + "right.z", (Rw, W)), get(q + "right.x", (Rw, W)),
                         get(q + "right.g", (Rw, W))]
                offs = [0]
                for t in parts:
                    offs.append(offs[-1] + t.shape[0])
                L.q_off, L.k_off, L.v_off, L.g_off, L.z_off, L.x_off, L.gr_off, L.ld = offs
                L.w_in = buf(q + "in", torch.cat(parts, 0))        # [q | k | v | gate | z | x | gate of the recurrence][W]: one GEMM
                L.w_out = buf(q + "out", torch.cat([get(q + "left.o", (W, H * dv)), get(q + "right.o", (W, Rw))], 1))
                L.z_b, L.x_b = buf(q + "right.z.b", get(q + "right.z.b", (Rw,))), buf(q + "right.x.b", get(q + "right.x.b", (Rw,)))
                rel = get(q + "left.rel")
                if rel.dim() != 2 or rel.shape[1] != H or rel.shape[0] < 1:
                    raise ValueError(f"{q}left.rel: shape {tuple(rel.shape)}, expected [buckets][{H}]")
                L.dist_bias = buf(q + "left.dist_bias", distance_bias_table(w[q + "left.rel"].to(dev), a.bias_max, a.chunk))
            else:
                m, q = la.mixer, p + "mix."
                Rw, nb = m.width, m.blocks
                bw = Rw // nb
                L.w_in = buf(q + "in", torch.cat([get(q + "y", (Rw, W)), get(q + "x", (Rw, W))], 0))    # [y | x][W]
                L.y_b, L.x_b = buf(q + "y.b", get(q + "y.b", (Rw,))), buf(q + "x.b", get(q + "x.b", (Rw,)))
                L.conv_w, L.conv_b = buf(q + "conv", get(q + "conv", (Rw, m.conv))), buf(q + "conv.b", get(q + "conv.b", (Rw,)))
                # both gates of a block from one batched product: [blocks][in][r out | i out]
                L.w_gates = buf(q + "gates", torch.cat([get(q + "ra", (nb, bw, bw)).transpose(1, 2),
                                                        get(q + "ri", (nb, bw, bw)).transpose(1, 2)], 2))
                L.ra_b, L.ri_b = buf(q + "ra.b", get(q + "ra.b", (nb, bw)).reshape(Rw)), buf(q + "ri.b", get(q + "ri.b", (nb, bw)).reshape(Rw))
                L.lam = buf(q + "lam", get(q + "lam", (Rw,)))
                L.w_out = buf(q + "o", get(q + "o", (W, Rw)))
            if la.ff:
                L.norm[1] = buf(p + "norm2", get(p + "norm2", (W,)))
                L.w_gu = buf(p + "mlp.gu", torch.cat([get(p + "mlp.gate", (la.ff, W)), get(p + "mlp.up", (la.ff, W))], 0))
                L.w_down = buf(p + "mlp.down", get(p + "mlp.down", (W, la.ff)))
            self.layers.append(L)
        extra = sorted(set(w) - used)
        if extra:
            raise ValueError(f"checkpoint tensors the configuration does not use: {extra[:8]}{' ...' if len(extra) > 8 else ''}")

    @classmethod
    def from_checkpoint(cls, folder, device="cuda", dtype=torch.bfloat16):
        cfg = TadolixArgs.from_dict(read_config(folder))
        return cls(cfg, read_safetensors(os.path.join(str(folder), "model.safetensors")), device, dtype).eval()

    @classmethod
    def from_name(cls, name, device="cuda", dtype=torch.bfloat16):
        return cls.random_init(tadolix_configs[name](), device, dtype)

    @classmethod
    def random_init(cls, cfg: TadolixArgs, device="cuda", dtype=torch.bfloat16, seed=1234):
        """Seeded random weights of every tensor the configuration names (no checkpoints exist offline), drawn on `device`."""
        g = torch.Generator(device=device).manual_seed(seed)
        W, S = cfg.width, cfg.streams

        def mat(o, i, s=1.0):
            return (torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * (s / math.sqrt(i))).to(dtype)

        def vec(n, mean=0.0, s=1.0):
            n = n if isinstance(n, tuple) else (n,)
            return (mean + s * torch.randn(*n, generator=g, device=device, dtype=torch.float32)).to(dtype)

        w = {"embed": vec((cfg.vocab_size, W), 0.0, 0.1), "head": mat(cfg.vocab_size, W), "final.norm": vec(W, 0.0, 0.1)}
        for i, la in enumerate(cfg.layers):
            p, m = f"l{i}.", la.mixer
            w[p + "norm1"] = vec(W, 0.0, 0.1)
            if cfg.canon_taps:
                w[p + "canon1"] = vec((W, cfg.canon_taps), 0.0, 0.3)
            for q in ((1, 2) if la.ff else (1,)):
                if S:
                    w[f"{p}hc{q}.in"], w[f"{p}hc{q}.out"] = vec(S, 1.0 / S, 0.1), vec(S, 0.5, 0.2)
                    w[f"{p}hc{q}.mix"] = (torch.eye(S, device=device) * 0.9 + 0.05 * torch.randn(S, S, generator=g, device=device)).to(dtype)
            if la.type == "parallel":
                a, Rw, q = m.left, m.right_width, p + "mix."
                H, G, d, dv = a.heads, a.kv_heads, a.dim, a.vdim
                w[q + "left.q"], w[q + "left.k"], w[q + "left.v"] = mat(H * d, W), mat(G * d, W), mat(G * dv, W)
                w[q + "left.g"], w[q + "left.o"], w[q + "left.rel"] = mat(H * dv, W), mat(W, H * dv), vec((32, H), 0.0, 0.5)
                w[q + "right.z"], w[q + "right.x"], w[q + "right.g"], w[q + "right.o"] = mat(Rw, W), mat(Rw, W), mat(Rw, W), mat(W, Rw)
                w[q + "right.z.b"], w[q + "right.x.b"] = vec(Rw, -1.0, 1.0), vec(Rw, 0.0, 0.3)
            else:
                Rw, nb, q = m.width, m.blocks, p + "mix."
                bw = Rw // nb
                w[q + "y"], w[q + "x"], w[q + "o"] = mat(Rw, W), mat(Rw, W), mat(W, Rw)
                w[q + "y.b"], w[q + "x.b"], w[q + "conv.b"] = vec(Rw, 0.0, 0.1), vec(Rw, 0.0, 0.1), vec(Rw, 0.0, 0.1)
                w[q + "conv"] = vec((Rw, m.conv), 0.3, 0.3)
                w[q + "ra"] = (torch.randn(nb, bw, bw, generator=g, device=device) / math.sqrt(bw)).to(dtype)
                w[q + "ri"] = (torch.randn(nb, bw, bw, generator=g, device=device) / math.sqrt(bw)).to(dtype)
                w[q + "ra.b"], w[q + "ri.b"], w[q + "lam"] = vec((nb, bw), 0.0, 1.0), vec((nb, bw), 0.0, 1.0), vec(Rw, -3.0, 1.0)
            if la.ff:
                w[p + "norm2"] = vec(W, 0.0, 0.1)
                w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"] = mat(la.ff, W), mat(la.ff, W), mat(W, la.ff)
        return cls(cfg, w, device, dtype).eval()

    def weight_bytes(self, ignore_embeddings=False) -> int:
        skip = {"embed"} if ignore_embeddings else set()
        return sum(b.numel() * b.element_size() for n, b in self.named_buffers() if n not in skip)

    # ------------------------------------------------------------------------------------------------ state
    def setup_caches(self, max_batch_size, max_seq_length, dtype=None, device=None, kv_cache_quantization=False):
        """Per-sequence state for `max_batch_size` slots, one set per layer run: the mixer convolution's memory, and a
        ring of keys / values + a recurrence state (parallel layers) or a recurrence state + its convolution's memory
        (recurrent layers).  None of it grows with the sequence, so max_seq_length only bounds what generation may ask
        for.  Same call as the Llama's setup_caches."""
        if kv_cache_quantization:
            raise NotImplementedError("Tadolix keeps its ring of keys and values in the model's dtype")
        if self.states is not None and self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size:
            return
        cfg, dev, n = self.config, self.device, max_batch_size
        self.max_batch_size, self.max_seq_length = max_batch_size, max_seq_length
        self.states = SequenceStates(n, 1 << 30)
        self.run_state = []
        for li in cfg.runs:
            la, rs = cfg.layers[li], _RunState()
            if cfg.canon_taps:
                rs.canon = ConvState(n, cfg.canon_taps, cfg.width, dev)
            if la.type == "parallel":
                a = la.mixer.left
                rs.ring = RingKVCache(n, a.chunk, a.kv_heads, a.dim, a.vdim, self.dtype, dev)
                rs.rec = RecurrentState(n, la.mixer.right_width, dev)
            else:
                rs.rec = RecurrentState(n, la.mixer.width, dev)
                rs.conv = ConvState(n, la.mixer.conv, la.mixer.width, dev)
            for part in (rs.canon, rs.ring, rs.rec, rs.conv):
                if part is not None:
                    self.states.on_grow.append(part.grow)
            self.run_state.append(rs)
        self.states.on_grow.append(lambda k: setattr(self, "max_batch_size", k))
        self._step = None

    def state_bytes_per_sequence(self) -> int:
        total = 0
        for rs in self.run_state:
            for part in (rs.canon, rs.ring, rs.rec, rs.conv):
                if part is not None:
                    total += sum(b.numel() * b.element_size() for b in part.buffers()) // self.max_batch_size
        return total

    @property
    def step_engine(self):
        """The step function over this model's weights and state (step.py), made on first use."""
        if self._step is None:
            from .step import StepEngine
            assert self.states is not None, "call setup_caches first"
            self._step = StepEngine(self)
        return self._step

    def make_decode_engine(self, batch_size, temperature=0.8, top_k=200, **unused):
        from .step import GraphDecodeEngine
        return GraphDecodeEngine(self, batch_size, temperature, top_k)

    @torch.no_grad()
    def forward(self, idx: torch.Tensor, input_pos: Optional[torch.Tensor] = None) -> torch.Tensor:
        """idx [B][T] at positions input_pos [T] (default 0 .. T-1) of the sequences in slots 0 .. B-1 -> logits of the
        LAST position [B][1][vocab] in fp32 (what generation samples from).  The Llama's forward call shape.  The state
        is recurrent: positions must continue where the slots stand (or restart at 0)."""
        assert self.states is not None, "Caches must be initialized first"
        B, T = idx.shape
        start = 0 if input_pos is None else int(input_pos[0])
        st = self.states
        segs = []
        for b in range(B):
            slot = st.slot_of(("batch", b))
            assert slot == b, "generation batches own slots 0 .. B-1: release other requests first"
            assert start == 0 or st.length[slot] == start, "a recurrent state cannot jump to another position"
            st.length[slot] = start
            segs.append((slot, idx[b]))
        logits = self.step_engine.step(segs, want="last")
        return logits.view(B, 1, -1)
