"""Plain, slow restatement of the Rutusun decoder in float64 torch on the CPU: one function per mechanism, written from
the equations alone.  It shares no code with the package: tests compare the framework's kernels, state manager and
scheduler against it.  Weights are a dict {tensor name: tensor} with the checkpoint's names, the configuration is the
dict that config.json holds.  Every function takes a WHOLE sequence from position 0: nothing is cached here.

Notation: W = model width, T = tokens, H / G = query / key-value heads (or heads / groups of a state-space mixer),
d / dv = key / value size per head, N = state size.  A linear weight is stored [out][in]: y = M @ x.
"""
import math

import torch

F64 = torch.float64
# When set, what a bfloat16 implementation stores in bfloat16 (inputs and results of matrix products, activations,
# cached keys and values) is rounded to bfloat16 here as well; the distance between that run and the exact one is the
# size of rounding noise for a given model and input.
ROUND_BF16 = False


def _r(x):
    return x.to(torch.bfloat16).to(F64) if ROUND_BF16 else x


def _w(w, name):
    return w[name].to(F64)


def linear(x, w, name, bias=None):
    y = _r(x) @ _w(w, name).T
    if bias is not None:
        y = y + _w(w, bias)
    return _r(y)


def silu(z):
    return z * torch.sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return unit_rms(x, eps) * weight


# ---------------------------------------------------------------------------------------------------- mixers
def sink_attention(q, k, v, sink, scale):
    """q [T][H][d], k [T][G][d], v [T][G][dv], sink [H]: causal softmax whose denominator also holds exp(sink_h) (no key,
    no value, unscaled) -> [T][H][dv]."""
    T, H, d = q.shape
    G = k.shape[1]
    rep = H // G
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // rep
        s = (q[:, h] @ k[:, g].T) * scale                                  # [T][T]
        s = s.masked_fill(torch.ones(T, T, dtype=torch.bool).triu(1), -math.inf)
        m = torch.maximum(s.max(-1, keepdim=True).values, sink[h].reshape(1, 1))
        p = torch.exp(s - m)
        den = p.sum(-1, keepdim=True) + torch.exp(sink[h] - m)
        out[:, h] = (p / den) @ v[:, g]
    return out


def query_temperature(T, coef, every):
    """[T]: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T, dtype=F64)
    return 1.0 + coef * torch.log(torch.floor((p + 1.0) / every) + 1.0)


def attention_mixer(cfg, m, w, p, h):
    eps = cfg["norm"]["eps"]
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w, p + "q", p + "q.b").view(T, H, d)
    k = linear(h, w, p + "k", p + "k.b").view(T, G, d)
    v = linear(h, w, p + "v", p + "v.b").view(T, G, dv)
    q = rms_norm(q, _w(w, p + "q.norm"), eps)
    k = _r(rms_norm(k, _w(w, p + "k.norm"), eps))
    if m.get("q_temp"):
        q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"]).view(T, 1, 1)
    o = sink_attention(q, k, v, _w(w, p + "sink"), m["scale"])
    return linear(o.reshape(T, H * dv), w, p + "o", p + "o.b")


def decayed_outer_recurrence(q, k, v, a, b):
    """S_t = a_t S_(t-1) + b_t k_t v_t^T from S = 0, o_t = S_t^T q_t.  q, k [T][H][d], v [T][H][dv], a, b [T][H]."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=F64)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for t in range(T):
        S = a[t].view(H, 1, 1) * S + b[t].view(H, 1, 1) * k[t].unsqueeze(2) * v[t].unsqueeze(1)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def lightning_mixer(cfg, m, w, p, h):
    eps = cfg["norm"]["eps"]
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(linear(h, w, p + "q")).view(T, H, d)
    k = silu(linear(h, w, p + "k")).view(T, H, d)
    v = silu(linear(h, w, p + "v")).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=F64).view(1, H).expand(T, H)
    o = decayed_outer_recurrence(_r(q), _r(k), _r(v), decay, torch.ones(T, H, dtype=F64)).reshape(T, H * dv)
    o = rms_norm(o, _w(w, p + "norm"), eps) * torch.sigmoid(linear(h, w, p + "g"))
    return linear(o, w, p + "o")


def causal_conv(x, kernel, bias):
    """x [T][C], kernel [C][taps]: y_t = bias + sum_j kernel[:, j] x_(t - taps + 1 + j), zeros in front of row 0."""
    T, taps = x.shape[0], kernel.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=F64), x], 0)
    y = bias.expand(T, -1).clone()
    for j in range(taps):
        y = y + kernel[:, j] * pad[j:j + T]
    return y


def grouped_unit_rms(x, groups, eps):
    T, C = x.shape
    return unit_rms(x.view(T, groups, C // groups), eps).reshape(T, C)


def mamba2_mixer(cfg, m, w, p, h):
    eps = cfg["norm"]["eps"]
    T = h.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    proj = linear(h, w, p + "in")
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = _r(silu(_r(causal_conv(xbc, _w(w, p + "conv"), _w(w, p + "conv.b")))))
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt + _w(w, p + "dt_bias"), beta=1.0, threshold=1e9)
    a = torch.exp(-torch.exp(_w(w, p + "A_log")) * dt)                        # [T][H]
    grp = torch.arange(H) // (H // G)
    y = decayed_outer_recurrence(C[:, grp], B[:, grp], x, a, dt) + _w(w, p + "D").view(1, H, 1) * x
    y = y.reshape(T, inner) * silu(z)
    y = grouped_unit_rms(y, m["norm_groups"], eps) * _w(w, p + "norm")
    return linear(y, w, p + "o")


# ---------------------------------------------------------------------------------------------------- feed-forward
def glu_expert(h, w, p):
    return linear(silu(linear(h, w, p + "gate")) * linear(h, w, p + "up"), w, p + "down")


def route(z, correction, n_groups, keep, top, scale):
    """z [T][E] router logits -> (chosen [T][top] expert numbers, weights [T][top])."""
    T, E = z.shape
    s = torch.sigmoid(z)
    choice = s + correction
    per = E // n_groups
    grouped = choice.view(T, n_groups, per)
    gscore = grouped.topk(min(2, per), dim=-1).values.sum(-1)                 # [T][groups]
    kept = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    chosen = masked.topk(top, dim=-1).indices
    sw = s.gather(1, chosen)
    return chosen, sw / (sw.sum(-1, keepdim=True) + 1e-20) * scale


def moe(cfg, f, w, p, h):
    r = f["router"]
    E = r["experts"]
    z = _r(h) @ _w(w, p + "router").T
    chosen, weight = route(z, _w(w, p + "correction"), r["groups"]["count"], r["groups"]["keep"], r["top"], r["scale"])
    out = torch.zeros_like(h)
    for e in range(E):
        rows, col = (chosen == e).nonzero(as_tuple=True)
        if len(rows):
            out[rows] += weight[rows, col].unsqueeze(1) * glu_expert(h[rows], w, f"{p}e{e}.")
    if f.get("shared"):
        out = out + glu_expert(h, w, p + "shared.")
    return out


def feed_forward(cfg, f, w, p, h):
    if f["kind"] == "dense":
        return glu_expert(h, w, p)
    return moe(cfg, f, w, p, h)


# ---------------------------------------------------------------------------------------------------- the model
MIXERS = {"attention": attention_mixer, "lightning": lightning_mixer, "mamba2": mamba2_mixer}


def layer(cfg, i, w, x):
    lay, eps, p = cfg["layers"][i], cfg["norm"]["eps"], f"l{i}."
    y = MIXERS[lay["type"]](cfg, lay["mixer"], w, p + "mix.", rms_norm(x, _w(w, p + "norm1"), eps))
    x = x + rms_norm(y, _w(w, p + "norm1b"), eps)
    if lay.get("mlp"):
        y = feed_forward(cfg, lay["mlp"], w, p + "mlp.", rms_norm(x, _w(w, p + "norm2"), eps))
        x = x + rms_norm(y, _w(w, p + "norm2b"), eps)
    return x


def forward(cfg, w, tokens, layer_out=None):
    """Logits [T][vocab] of a whole sequence; layer_out (a list) receives the residual after every layer run."""
    x0 = _w(w, "embed")[torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    a, b, times = (loop["start"], loop["stop"], loop["times"]) if loop else (0, 0, 0)

    def run(i, x):
        x = layer(cfg, i, w, x)
        if layer_out is not None:
            layer_out.append(x)
        return x

    for i in range(a if loop else n):
        x = run(i, x)
    if loop:
        for t in range(times):
            if t > 0:
                x = x + x0
            x = x + _w(w, "loop.step")[t]
            for i in range(a, b):
                x = run(i, x)
        for i in range(b, n):
            x = run(i, x)
    x = rms_norm(x, _w(w, "final.norm"), cfg["norm"]["eps"])
    return _r(x) @ _w(w, "head").T


def rounding_noise(cfg, w, tokens, measure):
    """measure(exact logits, logits of the run that rounds to bfloat16 wherever a bfloat16 implementation does)."""
    global ROUND_BF16
    exact = forward(cfg, w, tokens)
    ROUND_BF16 = True
    try:
        rounded = forward(cfg, w, tokens)
    finally:
        ROUND_BF16 = False
    return measure(exact, rounded)


def greedy(cfg, w, prompt, n_new):
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks[len(prompt):]


# ------------------------------------------------------------------------------------------------ test models
def attention_layer(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.4, coef=0.7, every=16, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if coef is not None:
        m["q_temp"] = {"coef": coef, "every": every}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def lightning_layer(heads=3, dim=8, vdim=12, decay=None, mlp=None):
    decay = decay or [math.exp(-1.0 / (1.5 + 6.0 * h)) for h in range(heads)]
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}, "mlp": mlp}


def mamba2_layer(heads=4, vdim=6, state=10, groups=2, conv=4, norm_groups=2, mlp=None):
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def mixture(experts=8, top=2, ff=16, groups=4, keep=2, scale=2.5, shared=24):
    f = {"kind": "moe", "expert": {"ff": ff},
         "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def model_config(layers, width=32, vocab=61, loop=None, eps=1e-5):
    cfg = {"architecture": "Rutusun", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Every tensor the configuration names, seeded, sized so that each mechanism moves the logits."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=1.0):
        return torch.randn(o, i, generator=g, dtype=torch.float32) * (s / math.sqrt(i))

    def vec(n, mean=0.0, s=1.0):
        n = n if isinstance(n, tuple) else (n,)
        return mean + s * torch.randn(*n, generator=g, dtype=torch.float32)

    def unit(p, ff):
        w[p + "gate"], w[p + "up"], w[p + "down"] = mat(ff, W, 1.5), mat(ff, W, 1.5), mat(W, ff, 1.5)

    w = {"embed": vec((V, W), 0.0, 1.0), "head": mat(V, W, 2.0), "final.norm": vec(W, 1.0, 0.2)}
    if cfg.get("loop"):
        w["loop.step"] = vec((cfg["loop"]["times"], W), 0.0, 0.5)
    for i, lay in enumerate(cfg["layers"]):
        p, q, m = f"l{i}.", f"l{i}.mix.", lay["mixer"]
        w[p + "norm1"], w[p + "norm1b"] = vec(W, 1.0, 0.2), vec(W, 1.0, 0.2)
        if lay["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"], w[q + "o"] = mat(H * d, W, 2.0), mat(G * d, W, 2.0), mat(G * dv, W), mat(W, H * dv)
            w[q + "q.b"], w[q + "k.b"], w[q + "v.b"], w[q + "o.b"] = vec(H * d, 0.0, 0.3), vec(G * d, 0.0, 0.3), vec(G * dv, 0.0, 0.3), vec(W, 0.0, 0.3)
            w[q + "q.norm"], w[q + "k.norm"], w[q + "sink"] = vec(d, 1.0, 0.3), vec(d, 1.0, 0.3), vec(H, 0.5, 1.0)
        elif lay["type"] == "lightning":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"], w[q + "g"] = mat(H * d, W, 2.0), mat(H * d, W, 2.0), mat(H * dv, W, 2.0), mat(H * dv, W)
            w[q + "norm"], w[q + "o"] = vec(H * dv, 1.0, 0.2), mat(W, H * dv)
        else:
            H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, ch = H * dv, H * dv + 2 * G * N
            w[q + "in"] = mat(2 * inner + 2 * G * N + H, W, 1.5)
            w[q + "conv"], w[q + "conv.b"] = vec((ch, m["conv"]), 0.25, 0.4), vec(ch, 0.0, 0.2)
            w[q + "dt_bias"], w[q + "A_log"], w[q + "D"] = vec(H, -1.5, 1.0), vec(H, -1.0, 0.7), vec(H, 1.0, 0.3)
            w[q + "norm"], w[q + "o"] = vec(inner, 1.0, 0.2), mat(W, inner)
        f = lay.get("mlp")
        if not f:
            continue
        w[p + "norm2"], w[p + "norm2b"] = vec(W, 1.0, 0.2), vec(W, 1.0, 0.2)
        if f["kind"] == "dense":
            unit(p + "mlp.", f["ff"])
        else:
            E = f["router"]["experts"]
            for e in range(E):
                unit(f"{p}mlp.e{e}.", f["expert"]["ff"])
            w[p + "mlp.router"], w[p + "mlp.correction"] = mat(E, W, 3.0), vec(E, -0.3, 0.4)
            if f.get("shared"):
                unit(p + "mlp.shared.", f["shared"]["ff"])
    return {k: v.to(dtype) for k, v in w.items()}


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw data) in `folder`."""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = {torch.bfloat16: "BF16", torch.float32: "F32", torch.int32: "I32"}
    header, blobs, at = {}, [], 0
    for name, t in w.items():
        raw = t.contiguous().reshape(-1).view(torch.uint8).numpy().tobytes()
        header[name] = {"dtype": names[t.dtype], "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(os.path.join(folder, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
