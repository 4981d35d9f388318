"""Fedipel: a decoder-only language model on a pre-norm residual, x += m * f(layer_norm(x)) with one constant m for every
sublayer.  Each layer picks one of three mixers and one of two feed-forwards:
  * "retention": linear attention with a fixed decay per head and neither softmax nor denominator; queries and keys are
    rotated by position (pairs (i, i + dims/2)), keys scaled by dim^-1/2; every head's read-out is brought to unit RMS and
    gated by SiLU of a projection of its own;
  * "wkv": time mixing over a matrix state whose decay is made per token and key channel by a small two-step projection,
    with a bonus for the current token; every projection reads its own blend of the row and the row in front of it;
  * "attention": differential attention (two softmax maps per head over the same values, a_1 - lambda * a_2, unit RMS)
    under a sliding window that also keeps the first tokens of the sequence, grouped heads, projection biases, rotation
    of the first coordinates of every map (pairs (2i, 2i + 1)); a layer may borrow the rotated keys and the values of an
    earlier layer's cache and project queries only;
  * feed-forward: a dense SiLU-gated unit, or a mixture of ungated squared-ReLU experts (the weights are a softmax over the
    chosen logits only) plus a shared expert behind a sigmoid gate of one number per token; a layer may have none.
The embedding output goes through a layer norm of its own; the logits are soft-capped.

This module holds the configuration (every size and constant is read from a checkpoint's config.json or from a tensor's
shape), the weights in the layout the kernels want, and the per-sequence state (cache.py).  The compute is step.py.
Checkpoint tensor names: embed, embed.norm[.b], final.norm[.b], head, l<i>.norm{1,2}[.b],
l<i>.mix.{q,k,v,g,o} | l<i>.mix.{mu.{r,k,v,g,w},r,k,v,g,w1,w2,w0,u,norm,o} | l<i>.mix.{q,k,v}[.b], l<i>.mix.{lq1,lk1,lq2,lk2,o},
l<i>.mlp.{gate,up,down} | l<i>.mlp.{router,router.b,e<j>.{up,down},shared.{up,down,sg}}; linear weights are [out][in].
"""
import math
import os
import warnings
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from ..cache import MatrixState, SequenceStates, TokenShiftState, WindowKVCache
from ..checkpoint import read_config, read_safetensors

NO_WINDOW = 1 << 30     # a mask without a window size: plain causal attention


@dataclass
class RotaryArgs:
    dims: int = 0               # 0: no rotation
    base: float = 10000.0

    def inv_freq(self, device) -> Optional[torch.Tensor]:
        """base^(-2i/dims), i < dims/2, rounded once to fp32."""
        if self.dims == 0:
            return None
        i = torch.arange(self.dims // 2, dtype=torch.float64)
        return torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * i / self.dims).to(torch.float32).to(device)


@dataclass
class RetentionArgs:
    heads: int
    dim: int
    vdim: int
    decay: List[float] = field(default_factory=list)
    rot: RotaryArgs = field(default_factory=RotaryArgs)


@dataclass
class WkvArgs:
    heads: int
    dim: int
    rank: int = 0               # inner size of the decay's two-step projection (a checkpoint gives it by a tensor's shape)


@dataclass
class DiffAttentionArgs:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: int = NO_WINDOW
    keep: int = 0
    rot: RotaryArgs = field(default_factory=RotaryArgs)
    kv_from: Optional[int] = None


@dataclass
class MlpArgs:
    kind: str                   # "dense" | "moe"
    ff: int                     # of the dense unit or of one expert
    experts: int = 0
    top: int = 0
    shared_ff: int = 0          # 0: no shared expert


@dataclass
class LayerArgs:
    type: str                   # "retention" | "wkv" | "attention"
    mixer: object
    mlp: Optional[MlpArgs] = None


def _rot(m) -> RotaryArgs:
    r = m.get("rot")
    if not r:
        return RotaryArgs()
    return RotaryArgs(int(r["dims"]), float(r["base"]))


@dataclass
class FedipelArgs:
    vocab_size: int
    width: int
    norm_eps: float
    residual_mult: float = 1.0
    logit_softcap: float = 0.0      # 0: none
    layers: List[LayerArgs] = field(default_factory=list)
    block_size: int = 1 << 30

    @property
    def n_layer(self):
        return len(self.layers)

    @property
    def has_attention(self):
        return any(la.type == "attention" for la in self.layers)

    def readers_of(self, i: int) -> List[int]:
        """The attention layers that read layer i's keys and values: itself and the layers that borrow them."""
        return [j for j, la in enumerate(self.layers)
                if la.type == "attention" and (j == i if la.mixer.kv_from is None else la.mixer.kv_from == i)]

    @classmethod
    def from_dict(cls, cfg: dict, shapes: Optional[Dict[str, tuple]] = None) -> "FedipelArgs":
        """cfg: a checkpoint's config.json.  shapes: the checkpoint's tensor shapes, for sizes that only they give."""
        layers = []
        for i, lay in enumerate(cfg["layers"]):
            m, kind = lay["mixer"], lay["type"]
            if kind == "retention":
                mixer = RetentionArgs(int(m["heads"]), int(m["dim"]), int(m["vdim"]), [float(v) for v in m["decay"]], _rot(m))
                assert len(mixer.decay) == mixer.heads, f"layer {i}: {len(mixer.decay)} decays for {mixer.heads} heads"
            elif kind == "wkv":
                rank = int(m["rank"]) if "rank" in m else int(shapes[f"l{i}.mix.w1"][0]) if shapes else 0
                mixer = WkvArgs(int(m["heads"]), int(m["dim"]), rank)
                assert mixer.rank > 0, f"layer {i}: the decay projection's inner size is in neither the configuration nor a tensor"
                assert mixer.dim <= 128, f"layer {i}: the time-mixing kernel keeps at most 128 key channels per head"
            elif kind == "attention":
                mask = m.get("mask") or {}
                src = m.get("kv_from")
                mixer = DiffAttentionArgs(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                          float(m["diff"]), int(mask.get("size", NO_WINDOW)), int(mask.get("keep_first", 0)),
                                          _rot(m), None if src is None else int(src))
                assert mixer.heads % mixer.kv_heads == 0, f"layer {i}: {mixer.heads} heads over {mixer.kv_heads} key/value heads"
                assert mixer.window >= 1 and mixer.keep >= 0, f"layer {i}: {mixer}"
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    assert 0 <= j < i and layers[j].type == "attention" and layers[j].mixer.kv_from is None, \
                        f"layer {i} borrows keys and values of layer {j}, which has none of its own in front of it"
                    s = layers[j].mixer
                    assert (s.kv_heads, s.dim, s.vdim) == (mixer.kv_heads, mixer.dim, mixer.vdim), f"layer {i}: head shapes differ from layer {j}'s"
            else:
                raise NotImplementedError(f"layer {i}: mixer type {kind!r}")
            if kind != "wkv":
                assert mixer.rot.dims % 2 == 0 and 0 <= mixer.rot.dims <= mixer.dim, f"layer {i}: rotation over {mixer.rot.dims} of {mixer.dim}"
            f, mlp = lay.get("mlp"), None
            if f:
                fk = f.get("kind", "dense")
                if fk == "dense":
                    mlp = MlpArgs("dense", int(f["ff"]))
                elif fk == "moe":
                    r, sh = f["router"], f.get("shared")
                    mlp = MlpArgs("moe", int(f["expert"]["ff"]), int(r["experts"]), int(r["top"]), int(sh["ff"]) if sh else 0)
                    assert 1 <= mlp.top <= mlp.experts, f"layer {i}: {mlp}"
                else:
                    raise NotImplementedError(f"layer {i}: feed-forward kind {fk!r}")
            layers.append(LayerArgs(kind, mixer, mlp))
        return cls(vocab_size=int(cfg["vocab"]), width=int(cfg["width"]), norm_eps=float(cfg["norm"]["eps"]),
                   residual_mult=float(cfg.get("residual_mult", 1.0)), logit_softcap=float(cfg.get("logit_softcap") or 0.0),
                   layers=layers)

    def to_dict(self) -> dict:
        out = []
        for lay in self.layers:
            m, f = lay.mixer, lay.mlp
            rot = {"base": m.rot.base, "dims": m.rot.dims} if lay.type != "wkv" and m.rot.dims else None
            if lay.type == "retention":
                mx = {"decay": list(m.decay), "dim": m.dim, "heads": m.heads, "vdim": m.vdim}
            elif lay.type == "wkv":
                mx = {"dim": m.dim, "heads": m.heads}
            else:
                mx = {"diff": m.diff, "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "scale": m.scale, "vdim": m.vdim}
                mask = {"keep_first": m.keep}
                if m.window != NO_WINDOW:
                    mask["size"] = m.window
                mx["mask"] = mask
                if m.kv_from is not None:
                    mx["kv_from"] = m.kv_from
            if rot:
                mx["rot"] = rot
            if f is None:
                fd = None
            elif f.kind == "dense":
                fd = {"ff": f.ff, "kind": "dense"}
            else:
                fd = {"expert": {"ff": f.ff}, "kind": "moe", "router": {"experts": f.experts, "top": f.top}}
                if f.shared_ff:
                    fd["shared"] = {"ff": f.shared_ff}
            out.append({"mixer": mx, "mlp": fd, "type": lay.type})
        cfg = {"architecture": "Fedipel", "layers": out, "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "vocab": self.vocab_size, "width": self.width}
        if self.logit_softcap:
            cfg["logit_softcap"] = self.logit_softcap
        return cfg


def _decays(heads):
    """Per-head decays spread between a short and a long memory."""
    return [1.0 - 2.0 ** -(3.0 + 6.0 * h / max(1, heads - 1)) for h in range(heads)]


def _pattern(n_layer, width, heads, kv_heads, dim, ff, vocab, window=4096, keep=8, experts=0, top=0, expert_ff=0, kinds=None, rank=64):
    """Layers cycling retention -> attention -> wkv; a second attention layer borrows the first one's keys and values;
    feed-forwards alternate dense / mixture (when experts > 0)."""
    kinds = kinds or ("retention", "attention", "wkv")
    layers, first_attn = [], None
    for i in range(n_layer):
        kind = kinds[i % len(kinds)]
        if kind == "retention":
            mixer = RetentionArgs(heads, dim, dim, _decays(heads), RotaryArgs(dim, 5e5))
        elif kind == "attention":
            # two maps of dim / 2 per head: the same query / key width per head as one map of `dim`
            mixer = DiffAttentionArgs(heads, kv_heads, dim // 2, dim, 1.0 / math.sqrt(dim // 2), 0.6, window, keep,
                                      RotaryArgs(dim // 4, 1e4), first_attn)
            first_attn = i if first_attn is None else first_attn
        else:
            mixer = WkvArgs(width // 64, 64, rank)
        if experts and i % 2 == 1:
            mlp = MlpArgs("moe", expert_ff, experts, top, expert_ff)
        else:
            mlp = MlpArgs("dense", ff)
        layers.append(LayerArgs(kind, mixer, mlp))
    return FedipelArgs(vocab, width, 1e-5, 0.8, 30.0, layers)


# named random-init configurations (benchmarks and examples; checkpoints carry their own config.json)
fedipel_configs = {
    "Fedipel-test": lambda: _pattern(5, 128, 4, 2, 32, 192, 512, window=24, keep=2, experts=6, top=2, expert_ff=64,
                                     kinds=("retention", "attention", "wkv", "attention", "retention"), rank=8),
    # layers of the size of a 1-2 B parameter model / of a 7-8 B parameter model (a layer benchmark)
    "Fedipel-2k": lambda: _pattern(3, 2048, 16, 4, 128, 6144, 32000),
    "Fedipel-4k": lambda: _pattern(3, 4096, 32, 8, 128, 12288, 128256),
    "Fedipel-2k-moe": lambda: _pattern(4, 2048, 16, 4, 128, 6144, 32000, experts=32, top=4, expert_ff=1024),
}


class _Layer:
    """One layer's tensors as the kernels read them (plain attributes; the module registers them as buffers)."""


class _LayerState:
    """Per-sequence state of one layer."""
    window: Optional[WindowKVCache] = None     # of an attention layer with projections of its own
    mat: Optional[MatrixState] = None
    shift: Optional[TokenShiftState] = None

    def parts(self):
        return [p for p in (self.window, self.mat, self.shift) if p is not None]


class Fedipel(nn.Module):
    def __init__(self, config: FedipelArgs, weights: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16):
        super().__init__()
        assert dtype in (torch.bfloat16, torch.float32), "Fedipel runs in bfloat16 or float32"
        self.config, self.dtype = config, dtype
        self.device = torch.device(device)
        self.max_batch_size = -1
        self.max_seq_length = -1
        self.states: Optional[SequenceStates] = None
        self.run_state: List[_LayerState] = []
        self._step = None
        self._take(weights)

    # ------------------------------------------------------------------------------------------------ weights
    def _take(self, w: Dict[str, torch.Tensor]):
        cfg, dev, dt = self.config, self.device, self.dtype
        used = set()
        f32 = torch.float32

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

        def norm(name):
            return buf(name, get(name, (W,))), buf(name + ".b", get(name + ".b", (W,)))

        W, V = cfg.width, cfg.vocab_size
        self.embed = buf("embed", get("embed", (V, W)))
        self.embed_norm, self.embed_norm_b = norm("embed.norm")
        self.final_norm, self.final_norm_b = norm("final.norm")
        self.head = buf("head", get("head", (V, W)))
        self.layers: List[_Layer] = []
        for i, la in enumerate(cfg.layers):
            p, q, L, m = f"l{i}.", f"l{i}.mix.", _Layer(), la.mixer
            L.args = la
            L.norm1, L.norm1_b = norm(p + "norm1")
            if la.type == "retention":
                H, d, dv = m.heads, m.dim, m.vdim
                L.w_in = buf(q + "in", torch.cat([get(q + "q", (H * d, W)), get(q + "k", (H * d, W)), get(q + "v", (H * dv, W)),
                                                  get(q + "g", (H * dv, W))], 0))
                L.q_off, L.k_off, L.v_off, L.g_off, L.ld = 0, H * d, 2 * H * d, 2 * H * d + H * dv, 2 * H * (d + dv)
                L.decay = buf(q + "decay", torch.tensor(m.decay, dtype=f32, device=dev))
                L.inv_freq = buf(q + "inv_freq", m.rot.inv_freq(dev)) if m.rot.dims else None
                L.w_out = buf(q + "o", get(q + "o", (W, H * dv)))
            elif la.type == "wkv":
                H, d, R = m.heads, m.dim, m.rank
                L.mu = buf(q + "mu", torch.stack([get(q + "mu." + s, (W,)) for s in "rkvgw"], 0))              # [5][W]
                L.w_rkvg = buf(q + "rkvg", torch.stack([get(q + s, (H * d, W)) for s in "rkvg"], 0))             # [4][H d][W]
                L.w1, L.w2 = buf(q + "w1", get(q + "w1", (R, W))), buf(q + "w2", get(q + "w2", (H * d, R)))
                L.w0, L.bonus = buf(q + "w0", get(q + "w0", (H * d,))), buf(q + "u", get(q + "u", (H, d)))
                L.mix_norm = buf(q + "norm", get(q + "norm", (H * d,)))
                L.w_out = buf(q + "o", get(q + "o", (W, H * d)))
            else:
                H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
                parts = [get(q + "q", (H * 2 * d, W))]
                L.q_b = buf(q + "q.b", get(q + "q.b", (H * 2 * d,)))
                L.k_b = L.v_b = None
                if m.kv_from is None:
                    parts += [get(q + "k", (G * 2 * d, W)), get(q + "v", (G * dv, W))]
                    L.k_b, L.v_b = buf(q + "k.b", get(q + "k.b", (G * 2 * d,))), buf(q + "v.b", get(q + "v.b", (G * dv,)))
                L.w_in = buf(q + "in", torch.cat(parts, 0))
                L.q_off, L.k_off, L.v_off, L.ld = 0, H * 2 * d, (H + G) * 2 * d, L.w_in.shape[0]
                lam = [get(q + s, (d,), torch.float64).cpu() for s in ("lq1", "lk1", "lq2", "lk2")]
                L.lam = float(torch.exp((lam[0] * lam[1]).sum()) - torch.exp((lam[2] * lam[3]).sum()) + m.diff)
                L.inv_freq = buf(q + "inv_freq", m.rot.inv_freq(dev)) if m.rot.dims else None
                L.w_out = buf(q + "o", get(q + "o", (W, H * dv)))
            f = la.mlp
            if f is not None:
                L.norm2, L.norm2_b = norm(p + "norm2")
                r = p + "mlp."
                if f.kind == "dense":
                    L.w_gu = buf(r + "gu", torch.cat([get(r + "gate", (f.ff, W)), get(r + "up", (f.ff, W))], 0))
                    L.w_down = buf(r + "down", get(r + "down", (W, f.ff)))
                else:
                    L.wu = buf(r + "experts.up", torch.stack([get(f"{r}e{e}.up", (f.ff, W)) for e in range(f.experts)], 0))      # [E][ff][W]
                    L.wd = buf(r + "experts.down", torch.stack([get(f"{r}e{e}.down", (W, f.ff)) for e in range(f.experts)], 0))  # [E][W][ff]
                    rows = [get(r + "router", (f.experts, W))]
                    if f.shared_ff:     # the shared expert's gate logit rides along in the router's product
                        rows.append(get(r + "shared.sg", (1, W)))
                        L.su, L.sd = buf(r + "shared.up", get(r + "shared.up", (f.shared_ff, W))), \
                            buf(r + "shared.down", get(r + "shared.down", (W, f.shared_ff)))
                    L.router = buf(r + "router", torch.cat(rows, 0))
                    L.router_b = buf(r + "router.b", get(r + "router.b", (f.experts,), f32))
            self.layers.append(L)
        extra = sorted(set(w) - used)
        if extra:   # e.g. the feed-forward norms of a layer that has no feed-forward: nothing reads them
            warnings.warn(f"checkpoint tensors the configuration does not use: {extra[:8]}{' ...' if len(extra) > 8 else ''}")

    @classmethod
    def from_checkpoint(cls, folder, device="cuda", dtype=torch.bfloat16):
        w = read_safetensors(os.path.join(str(folder), "model.safetensors"))
        cfg = FedipelArgs.from_dict(read_config(folder), {k: tuple(v.shape) for k, v in w.items()})
        return cls(cfg, w, device, dtype).eval()

    @classmethod
    def from_name(cls, name, device="cuda", dtype=torch.bfloat16):
        return cls.random_init(fedipel_configs[name](), device, dtype)

    @staticmethod
    def random_weights(cfg: FedipelArgs, device="cpu", dtype=torch.bfloat16, seed=1234) -> Dict[str, torch.Tensor]:
        """Seeded random weights of every tensor the configuration names (no checkpoints exist offline)."""
        g = torch.Generator(device=device).manual_seed(seed)
        W = cfg.width

        def mat(o, i, s=1.0):
            return (torch.randn(o, i, generator=g, device=device, dtype=torch.float32) * (s / math.sqrt(i))).to(dtype)

        def vec(n, mean=0.0, s=1.0):
            n = n if isinstance(n, tuple) else (n,)
            return (mean + s * torch.randn(*n, generator=g, device=device, dtype=torch.float32)).to(dtype)

        def norm(name):
            w[name], w[name + ".b"] = vec(W, 1.0, 0.1), vec(W, 0.0, 0.1)

        w = {"embed": vec((cfg.vocab_size, W), 0.0, 1.0), "head": mat(cfg.vocab_size, W)}
        norm("embed.norm")
        norm("final.norm")
        for i, la in enumerate(cfg.layers):
            p, q, m = f"l{i}.", f"l{i}.mix.", la.mixer
            norm(p + "norm1")
            if la.type == "retention":
                H, d, dv = m.heads, m.dim, m.vdim
                w[q + "q"], w[q + "k"], w[q + "v"], w[q + "g"] = mat(H * d, W), mat(H * d, W), mat(H * dv, W), mat(H * dv, W)
                w[q + "o"] = mat(W, H * dv)
            elif la.type == "wkv":
                H, d, R = m.heads, m.dim, m.rank
                for s in "rkvgw":
                    w[q + "mu." + s] = vec(W, 0.5, 0.2)
                for s in "rkvg":
                    w[q + s] = mat(H * d, W)
                w[q + "w1"], w[q + "w2"], w[q + "w0"] = mat(R, W), mat(H * d, R), vec(H * d, -1.5, 0.7)
                w[q + "u"], w[q + "norm"], w[q + "o"] = vec((H, d), 0.3, 0.3), vec(H * d, 1.0, 0.1), mat(W, H * d)
            else:
                H, G, d, dv = m.heads, m.kv_heads, m.dim, m.vdim
                w[q + "q"], w[q + "q.b"] = mat(H * 2 * d, W), vec(H * 2 * d, 0.0, 0.2)
                if m.kv_from is None:
                    w[q + "k"], w[q + "v"] = mat(G * 2 * d, W), mat(G * dv, W)
                    w[q + "k.b"], w[q + "v.b"] = vec(G * 2 * d, 0.0, 0.2), vec(G * dv, 0.0, 0.2)
                for s in ("lq1", "lk1", "lq2", "lk2"):
                    w[q + s] = vec(d, 0.0, 0.3 / math.sqrt(d))
                w[q + "o"] = mat(W, H * dv)
            f = la.mlp
            if f is None:
                continue
            norm(p + "norm2")
            r = p + "mlp."
            if f.kind == "dense":
                w[r + "gate"], w[r + "up"], w[r + "down"] = mat(f.ff, W), mat(f.ff, W), mat(W, f.ff)
            else:
                for e in range(f.experts):
                    w[f"{r}e{e}.up"], w[f"{r}e{e}.down"] = mat(f.ff, W), mat(W, f.ff)
                w[r + "router"], w[r + "router.b"] = mat(f.experts, W, 2.0), vec(f.experts, 0.0, 0.2)
                if f.shared_ff:
                    w[r + "shared.up"], w[r + "shared.down"], w[r + "shared.sg"] = mat(f.shared_ff, W), mat(W, f.shared_ff), mat(1, W)
        return w

    @classmethod
    def random_init(cls, cfg: FedipelArgs, device="cuda", dtype=torch.bfloat16, seed=1234):
        return cls(cfg, cls.random_weights(cfg, device, dtype, seed), device, dtype).eval()

    def weight_bytes(self, ignore_embeddings=False) -> int:
        skip = {"embed"} if ignore_embeddings else set()
        return sum(b.numel() * b.element_size() for n, b in self.named_buffers() if n not in skip)

    # ------------------------------------------------------------------------------------------------ state
    def setup_caches(self, max_batch_size, max_seq_length, dtype=None, device=None, kv_cache_quantization=False):
        """Per-sequence state for `max_batch_size` slots: a ring of keys and values as long as the widest window that
        reads it (never longer than max_seq_length) with the kept first positions beside it (attention layers with
        projections of their own), a matrix state per head (retention, wkv) and the last input row (wkv).  A sequence may
        grow past max_seq_length when no window had to be cut to it.  Same call as the Llama's setup_caches."""
        if kv_cache_quantization:
            raise NotImplementedError("Fedipel keeps its keys and values in the model's dtype")
        if self.states is not None and self.max_seq_length >= max_seq_length and self.max_batch_size >= max_batch_size:
            return
        cfg, dev, n = self.config, self.device, max_batch_size
        self.max_batch_size, self.max_seq_length = max_batch_size, max_seq_length
        self.run_state = []
        bounded = False
        for i, la in enumerate(cfg.layers):
            m, ls = la.mixer, _LayerState()
            if la.type == "attention":
                if m.kv_from is None:
                    readers = [cfg.layers[j].mixer for j in cfg.readers_of(i)]
                    widest = max(r.window for r in readers)
                    bounded |= widest > max_seq_length
                    ring = min(widest, max_seq_length)
                    first = min(max(r.keep for r in readers), max_seq_length)
                    ls.window = WindowKVCache(n, ring, first, m.kv_heads * 2 * m.dim, m.kv_heads * m.vdim, self.dtype, dev)
            elif la.type == "retention":
                ls.mat = MatrixState(n, m.heads, m.dim, m.vdim, dev)
            else:
                ls.mat = MatrixState(n, m.heads, m.dim, m.dim, dev)
                ls.shift = TokenShiftState(n, cfg.width, dev)
            self.run_state.append(ls)
        self.states = SequenceStates(n, max_seq_length if bounded else 1 << 30)
        for ls in self.run_state:
            for part in ls.parts():
                self.states.on_grow.append(part.grow)
        self.states.on_grow.append(lambda k: setattr(self, "max_batch_size", k))
        self._step = None

    def state_bytes_per_sequence(self) -> int:
        return sum(b.numel() * b.element_size() for ls in self.run_state for part in ls.parts() for b in part.buffers()) \
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
