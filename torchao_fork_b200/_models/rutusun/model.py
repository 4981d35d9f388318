"""Rutusun: a decoder-only language model whose layers each pick one of three mixers and one of two feed-forwards:
  * "attention": causal softmax attention over grouped heads with projection biases, a learned per-coordinate weight on
    unit-RMS queries and keys, no rotation (positions enter through a query temperature that grows with the logarithm of
    the position, and through the causal mask), and a learned sink per head in the softmax denominator;
  * "lightning": linear attention with a fixed decay per head over SiLU queries, keys and values, an RMS norm over the
    concatenated heads and a sigmoid gate;
  * "mamba2": a selective state space in its dual (matrix-state) form: a short causal convolution + SiLU over [x | B | C],
    softplus step sizes, one decay per head and step, a skip term, a SiLU gate in front of a grouped RMS norm;
  * feed-forward: a dense SiLU-gated unit, or a mixture of such units with a sigmoid router (selection correction,
    group-limited choice, renormalised weights times a constant) plus a shared expert; a layer may have none;
  * every sublayer is normed on the way in and on the way out: x += norm_b(f(norm(x)));
  * a span of layers may run several times in a row with the same weights and separate state per pass; every pass starts
    by adding a learned vector, and every pass but the first also the embedding output.

This module holds the configuration (every size and constant is read from a checkpoint's config.json), the weights in
the layout the kernels want, and the per-sequence state (cache.py).  The compute is step.py.
Checkpoint tensor names: embed, head, final.norm, loop.step, l<i>.{norm1,norm1b,norm2,norm2b},
l<i>.mix.{q,q.b,k,k.b,v,v.b,q.norm,k.norm,sink,o,o.b} | l<i>.mix.{q,k,v,g,norm,o} |
l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}, l<i>.mlp.{gate,up,down} |
l<i>.mlp.{router,correction,e<j>.{gate,up,down},shared.{gate,up,down}}; linear weights are [out][in].
"""
import math
import os
import warnings
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..cache import ConvState, MatrixState, RingKVCache, SequenceStates
from ..checkpoint import read_config, read_safetensors

MAX_TAPS = 64


@dataclass
class SinkAttentionArgs:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float = 0.0      # 0: no query temperature
    temp_every: int = 1


@dataclass
class LightningArgs:
    heads: int
    dim: int
    vdim: int
    decay: List[float] = field(default_factory=list)


@dataclass
class Mamba2Args:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @property
    def inner(self):
        return self.heads * self.vdim

    @property
    def conv_channels(self):
        return self.inner + 2 * self.groups * self.state


@dataclass
class MlpArgs:
    kind: str                   # "dense" | "moe"
    ff: int                     # of the dense unit or of one expert
    experts: int = 0
    top: int = 0
    n_groups: int = 1
    keep: int = 1
    scale: float = 1.0
    shared_ff: int = 0          # 0: no shared expert


@dataclass
class LayerArgs:
    type: str                   # "attention" | "lightning" | "mamba2"
    mixer: object
    mlp: Optional[MlpArgs] = None


@dataclass
class RutusunArgs:
    vocab_size: int
    width: int
    norm_eps: float
    loop: Optional[Tuple[int, int, int]] = None     # (start, stop, times)
    layers: List[LayerArgs] = field(default_factory=list)
    block_size: int = 1 << 30

    @property
    def n_layer(self):
        return len(self.layers)

    @property
    def schedule(self) -> List[tuple]:
        """The order of work: ("enter", pass number) in front of every pass over the looped span, ("layer", index)."""
        n = len(self.layers)
        if not self.loop:
            return [("layer", i) for i in range(n)]
        a, b, times = self.loop
        out = [("layer", i) for i in range(a)]
        for t in range(times):
            out.append(("enter", t))
            out += [("layer", i) for i in range(a, b)]
        return out + [("layer", i) for i in range(b, n)]

    @property
    def runs(self) -> List[int]:
        """Layer index of every layer run, in order (a looped layer appears once per pass)."""
        return [i for kind, i in self.schedule if kind == "layer"]

    @property
    def has_attention(self):
        return any(la.type == "attention" for la in self.layers)

    @classmethod
    def from_dict(cls, cfg: dict) -> "RutusunArgs":
        layers = []
        for i, lay in enumerate(cfg["layers"]):
            m, kind = lay["mixer"], lay["type"]
            if kind == "attention":
                qt = m.get("q_temp") or {}
                mixer = SinkAttentionArgs(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                          float(qt.get("coef", 0.0)), int(qt.get("every", 1)))
                assert mixer.heads % mixer.kv_heads == 0, f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key/value heads"
                assert mixer.temp_coef == 0.0 or mixer.temp_every >= 1, f"layer {i}: {mixer}"
            elif kind == "lightning":
                dec = m["decay"]
                dec = [float(v) for v in dec] if isinstance(dec, (list, tuple)) else [float(dec)] * int(m["heads"])   # one number: every head
                mixer = LightningArgs(int(m["heads"]), int(m["dim"]), int(m["vdim"]), dec)
                assert len(mixer.decay) == mixer.heads, f"layer {i}: {len(mixer.decay)} decays for {mixer.heads} heads"
            elif kind == "mamba2":
                mixer = Mamba2Args(int(m["heads"]), int(m["vdim"]), int(m["state"]), int(m["groups"]), int(m["conv"]),
                                   int(m.get("norm_groups", 1)))
                assert mixer.heads % mixer.groups == 0 and mixer.inner % mixer.norm_groups == 0 and 1 <= mixer.conv <= MAX_TAPS, \
                    f"layer {i}: {mixer}"
            else:
                raise NotImplementedError(f"layer {i}: mixer type {kind!r}")
            f, mlp = lay.get("mlp"), None
            if f:
                fk = f.get("kind", "dense")
                if fk == "dense":
                    mlp = MlpArgs("dense", int(f["ff"]))
                elif fk == "moe":
                    r = f["router"]
                    g = r.get("groups") or {}
                    sh = f.get("shared")
                    mlp = MlpArgs("moe", int(f["expert"]["ff"]), int(r["experts"]), int(r["top"]), int(g.get("count", 1)),
                                  int(g.get("keep", g.get("count", 1))), float(r.get("scale", 1.0)), int(sh["ff"]) if sh else 0)
                    per = mlp.experts // max(1, mlp.n_groups)
                    assert mlp.n_groups >= 1 and mlp.experts % mlp.n_groups == 0 and 1 <= mlp.keep <= mlp.n_groups and \
                        1 <= mlp.top <= mlp.keep * per, f"layer {i}: {mlp}"
                else:
                    raise NotImplementedError(f"layer {i}: feed-forward kind {fk!r}")
            layers.append(LayerArgs(kind, mixer, mlp))
        loop = cfg.get("loop")
        if loop:
            loop = (int(loop["start"]), int(loop["stop"]), int(loop["times"]))
            assert 0 <= loop[0] <= loop[1] <= len(layers) and loop[2] >= 1, f"loop {loop}"
        return cls(vocab_size=int(cfg["vocab"]), width=int(cfg["width"]), norm_eps=float(cfg["norm"]["eps"]), loop=loop,
                   layers=layers)

    def to_dict(self) -> dict:
        out = []
        for lay in self.layers:
            m, f = lay.mixer, lay.mlp
            if lay.type == "attention":
                mx = {"dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "scale": m.scale, "vdim": m.vdim}
                if m.temp_coef != 0.0:
                    mx["q_temp"] = {"coef": m.temp_coef, "every": m.temp_every}
            elif lay.type == "lightning":
                mx = {"decay": list(m.decay), "dim": m.dim, "heads": m.heads, "vdim": m.vdim}
            else:
                mx = {"conv": m.conv, "groups": m.groups, "heads": m.heads, "norm_groups": m.norm_groups, "state": m.state,
                      "vdim": m.vdim}
            if f is None:
                fd = None
            elif f.kind == "dense":
                fd = {"ff": f.ff, "kind": "dense"}
            else:
                fd = {"expert": {"ff": f.ff}, "kind": "moe",
                      "router": {"experts": f.experts, "groups": {"count": f.n_groups, "keep": f.keep}, "scale": f.scale, "top": f.top}}
                if f.shared_ff:
                    fd["shared"] = {"ff": f.shared_ff}
            out.append({"mixer": mx, "mlp": fd, "type": lay.type})
        cfg = {"architecture": "Rutusun", "layers": out, "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size,
               "width": self.width}
        if self.loop:
            cfg["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return cfg


def _decays(heads):
    """Per-head decays spread between a short and a long memory."""
    return [1.0 - 2.0 ** -(2.0 + 6.0 * h / max(1, heads - 1)) for h in range(heads)]


def _pattern(n_layer, width, heads, kv_heads, dim, ff, vocab, experts=0, top=0, expert_ff=0, state=128, loop=None, kinds=None):
    """Layers cycling attention -> lightning -> mamba2, feed-forwards alternating dense / mixture (when experts > 0)."""
    kinds = kinds or ("attention", "lightning", "mamba2")
    layers = []
    for i in range(n_layer):
        kind = kinds[i % len(kinds)]
        if kind == "attention":
            mixer = SinkAttentionArgs(heads, kv_heads, dim, dim, 1.0 / math.sqrt(dim), 0.3, 512)
        elif kind == "lightning":
            mixer = LightningArgs(heads, dim, dim, _decays(heads))
        else:
            mixer = Mamba2Args(heads, dim, state, max(1, kv_heads // 2), 4, 2)
        if experts and i % 2 == 1:
            mlp = MlpArgs("moe", expert_ff, experts, top, 4, 2, 2.0, expert_ff)
        else:
            mlp = MlpArgs("dense", ff)
        layers.append(LayerArgs(kind, mixer, mlp))
    return RutusunArgs(vocab, width, 1e-5, loop, layers)


# named random-init configurations (benchmarks and examples; checkpoints carry their own config.json)
rutusun_configs = {
    "Rutusun-test": lambda: _pattern(3, 128, 4, 2, 32, 192, 512, experts=8, top=2, expert_ff=64, state=16, loop=(0, 2, 2)),
    # layers of the size of a 1-2 B parameter model / of a 7-8 B parameter model (a layer benchmark)
    "Rutusun-2k": lambda: _pattern(3, 2048, 16, 4, 128, 6144, 32000),
    "Rutusun-4k": lambda: _pattern(3, 4096, 32, 8, 128, 12288, 128256),
    "Rutusun-2k-moe": lambda: _pattern(4, 2048, 16, 4, 128, 6144, 32000, experts=32, top=4, expert_ff=1024),
}


class _Layer:
    """One layer's tensors as the kernels read them (plain attributes; the module registers them as buffers)."""


class _RunState:
    """Per-sequence state of ONE layer run (a looped layer has one per pass)."""
    ring: Optional[RingKVCache] = None
    mat: Optional[MatrixState] = None
    conv: Optional[ConvState] = None

    def parts(self):
        return [p for p in (self.ring, self.mat, self.conv) if p is not None]


class Rutusun(nn.Module):
    def __init__(self, config: RutusunArgs, weights: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32), "Rutusun runs in bfloat16 or float32"
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

        def get(name, shape=None, dtype=dt):
            if name not in w:
                raise KeyError(f"checkpoint has no tensor {name!r}")
            used.add(name)
            t = w[name]
            if shape is not None and tuple(t.shape) != tuple(shape):
                raise ValueError(f"{name}: shape {tuple(t.shape)}, the configuration asks for {tuple(shape)}")
            return t.to(device=dev, dtype=dtype)

        def buf(name, t):
            self.register_buffer(name.replace(".", "__"), t.contiguous(), persistent=False)
            return getattr(self, name.replace(".", "__"))

        def glu(prefix, ff):
            """[gate | up][W] for one GEMM, and the down projection."""
            return (torch.cat([get(prefix + "gate", (ff, W)), get(prefix + "up", (ff, W))], 0), get(prefix + "down", (W, ff)))

        W, V = cfg.width, cfg.vocab_size
        f32 = torch.float32
        self.embed = buf("embed", get("embed", (V, W)))
        self.head = buf("head", get("head", (V, W)))
        self.final_norm = buf("final.norm", get("final.norm", (W,)))
        self.loop_step = buf("loop.step", get("loop.step", (cfg.loop[2], W))) if cfg.loop else None
        self.layers: List[_Layer] = []
        for i, la in enumerate(cfg.layers):
            p, q, L, m = f"l{i}.", f"l{i}.mix.", _Layer(), la.mixer
            L.args = la
            L.norm1, L.norm1b = buf(p + "norm1", get(p + "norm1", (W,))), buf(p + "norm1b", get(p + "norm1b", (W,)))
            if la.type == "attention":
                H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
                L.w_in = buf(q + "in", torch.cat([get(q + "q", (H * d, W)), get(q + "k", (G * d, W)), get(q + "v", (G * dv, W))], 0))
                L.q_off, L.k_off, L.v_off, L.ld = 0, H * d, (H + G) * d, (H + G) * d + G * dv
                L.q_b, L.k_b, L.v_b = buf(q + "q.b", get(q + "q.b", (H * d,))), buf(q + "k.b", get(q + "k.b", (G * d,))), \
                    buf(q + "v.b", get(q + "v.b", (G * dv,)))
                L.q_norm, L.k_norm = buf(q + "q.norm", get(q + "q.norm", (d,))), buf(q + "k.norm", get(q + "k.norm", (d,)))
                L.sink = buf(q + "sink", get(q + "sink", (H,), f32))
                L.w_out = buf(q + "o", get(q + "o", (W, H * dv)))
                L.o_b = buf(q + "o.b", get(q + "o.b", (W,), f32))          # added to the fp32 product
            elif la.type == "lightning":
                H, d, dv = m.heads, m.dim, m.vdim
                L.w_in = buf(q + "in", torch.cat([get(q + "q", (H * d, W)), get(q + "k", (H * d, W)), get(q + "v", (H * dv, W)),
                                                  get(q + "g", (H * dv, W))], 0))
                L.q_off, L.k_off, L.v_off, L.g_off, L.ld = 0, H * d, 2 * H * d, 2 * H * d + H * dv, 2 * H * (d + dv)
                L.decay = buf(q + "decay", torch.tensor(m.decay, dtype=f32, device=dev))
                L.mix_norm = buf(q + "norm", get(q + "norm", (H * dv,)))
                L.w_out = buf(q + "o", get(q + "o", (W, H * dv)))
            else:
                H, ch, inner = m.heads, m.conv_channels, m.inner
                L.ld = 2 * inner + 2 * m.groups * m.state + H
                L.w_in = buf(q + "in", get(q + "in", (L.ld, W)))           # [z | x | B | C | step][W]
                L.conv_w, L.conv_b = buf(q + "conv", get(q + "conv", (ch, m.conv))), buf(q + "conv.b", get(q + "conv.b", (ch,)))
                L.dt_bias, L.a_log = buf(q + "dt_bias", get(q + "dt_bias", (H,))), buf(q + "A_log", get(q + "A_log", (H,)))
                L.skip = buf(q + "D", get(q + "D", (H,), f32))
                L.mix_norm = buf(q + "norm", get(q + "norm", (inner,)))
                L.w_out = buf(q + "o", get(q + "o", (W, inner)))
            f = la.mlp
            if f is not None:
                L.norm2, L.norm2b = buf(p + "norm2", get(p + "norm2", (W,))), buf(p + "norm2b", get(p + "norm2b", (W,)))
                r = p + "mlp."
                if f.kind == "dense":
                    gu, dn = glu(r, f.ff)
                    L.w_gu, L.w_down = buf(r + "gu", gu), buf(r + "down", dn)
                else:
                    pairs = [glu(f"{r}e{e}.", f.ff) for e in range(f.experts)]
                    L.wgu = buf(r + "experts.gu", torch.stack([a for a, _ in pairs], 0))      # [E][2 ff][W]
                    L.wd = buf(r + "experts.down", torch.stack([b for _, b in pairs], 0))     # [E][W][ff]
                    L.router = buf(r + "router", get(r + "router", (f.experts, W)))
                    L.correction = buf(r + "correction", get(r + "correction", (f.experts,), f32)) if r + "correction" in w else None
                    if f.shared_ff:
                        gu, dn = glu(r + "shared.", f.shared_ff)
                        L.sgu, L.sd = buf(r + "shared.gu", gu), buf(r + "shared.down", dn)
            self.layers.append(L)
        extra = sorted(set(w) - used)
        if extra:   # e.g. the feed-forward norms of a layer that has no feed-forward: nothing reads them
            warnings.warn(f"checkpoint tensors the configuration does not use: {extra[:8]}{' ...' if len(extra) > 8 else ''}")

    @classmethod
    def from_checkpoint(cls, folder, device="cuda", dtype=torch.bfloat16):
        cfg = RutusunArgs.from_dict(read_config(folder))
        return cls(cfg, read_safetensors(os.path.join(str(folder), "model.safetensors")), device, dtype).eval()

    @classmethod
    def from_name(cls, name, device="cuda", dtype=torch.bfloat16):
        return cls.random_init(rutusun_configs[name](), device, dtype)

    @staticmethod
    def random_weights(cfg: RutusunArgs, device="cpu", dtype=torch.bfloat16, seed=1234) -> Dict[str, torch.Tensor]:
        """Seeded random weights of every tensor the configuration names (no checkpoints exist offline)."""
        g = torch.Generator(device=device).manual_seed(seed)
        W = cfg.width

        def mat(o, i, s=1.0):
            return (torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * (s / math.sqrt(i))).to(dtype)

        def vec(n, mean=0.0, s=1.0):
            n = n if isinstance(n, tuple) else (n,)
            return (mean + s * torch.randn(*n, generator=g, device=device, dtype=torch.float32)).to(dtype)

        def glu(prefix, ff):
            w[prefix + "gate"], w[prefix + "up"], w[prefix + "down"] = mat(ff, W), mat(ff, W), mat(W, ff)

        w = {"embed": vec((cfg.vocab_size, W), 0.0, 1.0), "head": mat(cfg.vocab_size, W), "final.norm": vec(W, 1.0, 0.1)}
        if cfg.loop:
            w["loop.step"] = vec((cfg.loop[2], W), 0.0, 0.3)
        for i, la in enumerate(cfg.layers):
            p, q, m = f"l{i}.", f"l{i}.mix.", la.mixer
            w[p + "norm1"], w[p + "norm1b"] = vec(W, 1.0, 0.1), vec(W, 1.0, 0.1)
            if la.type == "attention":
                H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
                w[q + "q"], w[q + "k"], w[q + "v"], w[q + "o"] = mat(H * d, W), mat(G * d, W), mat(G * dv, W), mat(W, H * dv)
                w[q + "q.b"], w[q + "k.b"], w[q + "v.b"], w[q + "o.b"] = vec(H * d, 0.0, 0.2), vec(G * d, 0.0, 0.2), vec(G * dv, 0.0, 0.2), vec(W, 0.0, 0.2)
                w[q + "q.norm"], w[q + "k.norm"], w[q + "sink"] = vec(d, 1.0, 0.2), vec(d, 1.0, 0.2), vec(H, 0.0, 1.0)
            elif la.type == "lightning":
                H, d, dv = m.heads, m.dim, m.vdim
                w[q + "q"], w[q + "k"], w[q + "v"], w[q + "g"] = mat(H * d, W), mat(H * d, W), mat(H * dv, W), mat(H * dv, W)
                w[q + "norm"], w[q + "o"] = vec(H * dv, 1.0, 0.1), mat(W, H * dv)
            else:
                H, ch, inner = m.heads, m.conv_channels, m.inner
                w[q + "in"] = mat(2 * inner + 2 * m.groups * m.state + H, W)
                w[q + "conv"], w[q + "conv.b"] = vec((ch, m.conv), 0.2, 0.4), vec(ch, 0.0, 0.2)
                w[q + "dt_bias"], w[q + "A_log"], w[q + "D"] = vec(H, -1.0, 1.0), vec(H, -0.5, 0.7), vec(H, 1.0, 0.3)
                w[q + "norm"], w[q + "o"] = vec(inner, 1.0, 0.1), mat(W, inner)
            f = la.mlp
            if f is None:
                continue
            w[p + "norm2"], w[p + "norm2b"] = vec(W, 1.0, 0.1), vec(W, 1.0, 0.1)
            if f.kind == "dense":
                glu(p + "mlp.", f.ff)
            else:
                for e in range(f.experts):
                    glu(f"{p}mlp.e{e}.", f.ff)
                w[p + "mlp.router"], w[p + "mlp.correction"] = mat(f.experts, W, 2.0), vec(f.experts, 0.0, 0.2)
                if f.shared_ff:
                    glu(p + "mlp.shared.", f.shared_ff)
        return w

    @classmethod
    def random_init(cls, cfg: RutusunArgs, device="cuda", dtype=torch.bfloat16, seed=1234):
        return cls(cfg, cls.random_weights(cfg, device, dtype, seed), device, dtype).eval()

    def weight_bytes(self, ignore_embeddings=False) -> int:
        skip = {"embed"} if ignore_embeddings else set()
        return sum(b.numel() * b.element_size() for n, b in self.named_buffers() if n not in skip)

    # ------------------------------------------------------------------------------------------------ state
    def setup_caches(self, max_batch_size, max_seq_length, dtype=None, device=None, kv_cache_quantization=False):
        """Per-sequence state for `max_batch_size` slots, one set per layer run: keys and values of up to max_seq_length
        positions (attention; the ring cache with as many rows as the longest sequence), a matrix state per head (lightning,
        mamba2) and the convolution's memory (mamba2).  Same call as the Llama's setup_caches."""
        if kv_cache_quantization:
            raise NotImplementedError("Rutusun keeps its keys and values in the model's dtype")
        if self.states is not None and self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size:
            return
        cfg, dev, n = self.config, self.device, max_batch_size
        self.max_batch_size, self.max_seq_length = max_batch_size, max_seq_length
        self.states = SequenceStates(n, max_seq_length if cfg.has_attention else 1 << 30)
        self.run_state = []
        for li in cfg.runs:
            la, rs = cfg.layers[li], _RunState()
            m = la.mixer
            if la.type == "attention":
                rs.ring = RingKVCache(n, max_seq_length, m.kv_heads, m.dim, m.vdim, self.dtype, dev)
            elif la.type == "lightning":
                rs.mat = MatrixState(n, m.heads, m.dim, m.vdim, dev)
            else:
                rs.mat = MatrixState(n, m.heads, m.state, m.vdim, dev)
                rs.conv = ConvState(n, m.conv, m.conv_channels, dev)
            for part in rs.parts():
                self.states.on_grow.append(part.grow)
            self.run_state.append(rs)
        self.states.on_grow.append(lambda k: setattr(self, "max_batch_size", k))
        self._step = None

    def state_bytes_per_sequence(self) -> int:
        return sum(b.numel() * b.element_size() for rs in self.run_state for part in rs.parts() for b in part.buffers()) \
            // self.max_batch_size

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
