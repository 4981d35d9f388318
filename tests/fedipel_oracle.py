"""A plain, slow statement of the Fedipel design, one function per mechanism, token by token where the design is a
recurrence.  It shares no code with the package: tests compare the package's kernels and step function against it.
Everything is computed in the dtype of the tensors it is given (float64 by default: the weights' own rounding is the only
one).  `w` maps checkpoint tensor names to tensors, `cfg` is the checkpoint's config.json as a dict.
"""
import math

import torch

ROUND_BF16 = False      # rounding_noise() sets it: activations are rounded to bfloat16 where a bfloat16 run stores them


def _r(x):
    return x.to(torch.bfloat16).to(x.dtype) if ROUND_BF16 else x


def layer_norm(x, weight, bias, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * weight + bias


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotate(x, positions, dims, base, layout):
    """x [T][heads][dim]; the first `dims` coordinates of every head turn by position * base^(-2i/dims); pairs are
    (i, i + dims/2) for layout "half", (2i, 2i + 1) for layout "interleaved"."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]            # [T][half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    if layout == "half":
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    else:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    return out


def retention(h, w, p, m, eps):
    """Decayed linear attention without a softmax; h [T][W] from position 0.  Returns [T][W]."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotate(q, pos, rot["dims"], rot["base"], "half")
    k = rotate(k, pos, rot["dims"], rot["base"], "half") * d ** -0.5
    o = retention_recurrence(q, k, v, m["decay"])
    o = unit_rms(o, eps).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return _r(_r(o) @ w[p + "o"].T)


def retention_recurrence(q, k, v, decay):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head; q, k [T][H][d], v [T][H][dv] -> [T][H][dv]."""
    T, H, d = q.shape
    dv = v.shape[-1]
    o = torch.zeros(T, H, dv, dtype=q.dtype)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=q.dtype)
        for t in range(T):
            S = decay[hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    return o


def wkv(h, w, p, m, eps):
    """Time mixing with a data-dependent decay per key channel and a bonus for the current token."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, W, dtype=h.dtype), h[:-1]], 0)
    mix = {s: _r(h + (prev - h) * w[p + "mu." + s]) for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(T, H, d)
    k = (mix["k"] @ w[p + "k"].T).view(T, H, d)
    v = (mix["v"] @ w[p + "v"].T).view(T, H, d)
    gate = silu(mix["g"] @ w[p + "g"].T)
    dec = torch.exp(-torch.exp(_r(torch.tanh(mix["w"] @ w[p + "w1"].T)) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    o = wkv_recurrence(r, k, v, dec, w[p + "u"].view(H, d))
    o = unit_rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return _r(_r(o) @ w[p + "o"].T)


def wkv_recurrence(r, k, v, dec, u):
    """o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t, then S_t = diag(dec_t) S_(t-1) + k_t v_t^T; all [T][H][d], u [H][d]."""
    T, H, d = r.shape
    dv = v.shape[-1]
    o = torch.zeros(T, H, dv, dtype=r.dtype)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=r.dtype)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S + u[hd][:, None] * kv).T @ r[t, hd]
            S = dec[t, hd][:, None] * S + kv
    return o


def attention_keys_values(h, w, p, m):
    """Rotated keys [T][G][2][d] and values [T][G][dv] of a layer that has projections of its own."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G * 2, d)
    k = rotate(k, torch.arange(T), rot["dims"], rot["base"], "interleaved").view(T, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    return _r(k), _r(v)


def diff_attention(h, w, p, m, eps, kv):
    """Differential attention under a sliding window that keeps the first tokens; kv = (keys, values) of this layer or of
    the layer it borrows them from."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H * 2, d)
    q = rotate(q, torch.arange(T), rot["dims"], rot["base"], "interleaved").view(T, H, 2, d)
    k, v = kv
    lam = torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum()) + m["diff"]
    out = window_diff_attention(_r(q), k, v, m["scale"], size, keep, lam, eps) * (1.0 - m["diff"])
    return _r(_r(out.reshape(T, H * dv)) @ w[p + "o"].T)


def window_diff_attention(q, k, v, scale, size, keep, lam, eps):
    """q [T][H][M][d], k [T][G][M][d], v [T][G][dv]: M softmax maps per head under the mask
    j <= i and (i - j < size or j < keep); two maps combine as a_1 - lam a_2; the result is brought to unit RMS per head."""
    T, H, M, d = q.shape
    G, dv = k.shape[1], v.shape[-1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & ((i - j < size) | (j < keep))
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for mp in range(M):
            s = (q[:, hd, mp] @ k[:, g, mp].T) * scale
            s = s.masked_fill(~seen, -math.inf)
            maps.append(torch.softmax(s, -1) @ v[:, g])
        out[:, hd] = unit_rms(maps[0] - lam * maps[1] if M == 2 else maps[0], eps)
    return out


def relu2_unit(h, up, down):
    return _r(torch.relu(_r(h @ up.T)) ** 2) @ down.T


def feed_forward(h, w, p, f):
    if f["kind"] == "dense":
        return _r(silu(_r(h @ w[p + "gate"].T)) * _r(h @ w[p + "up"].T)) @ w[p + "down"].T
    E, top = f["router"]["experts"], f["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    val, idx = torch.topk(z, top, dim=-1)
    wt = torch.softmax(val, -1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for c in range(top):
            e = int(idx[t, c])
            out[t] += wt[t, c] * relu2_unit(h[t:t + 1], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])[0]
    if f.get("shared"):
        out = out + relu2_unit(h, w[p + "shared.up"], w[p + "shared.down"]) * torch.sigmoid(h @ w[p + "shared.sg"].T)
    return out


def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None):
    """Logits [T][vocab] of a whole sequence from position 0.  layers_out (a list) receives the residual after every layer."""
    w = {k: v.to(dtype) if v.is_floating_point() else v for k, v in w.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = layer_norm(x, w["embed.norm"], w["embed.norm.b"], eps)
    kvs = {}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        h = _r(layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps))
        if lay["type"] == "retention":
            y = retention(h, w, p + "mix.", m, eps)
        elif lay["type"] == "wkv":
            y = wkv(h, w, p + "mix.", m, eps)
        else:
            src = m.get("kv_from")
            if src is None:
                kvs[i] = attention_keys_values(h, w, p + "mix.", m)
            y = diff_attention(h, w, p + "mix.", m, eps, kvs[i if src is None else src])
        x = x + mult * y
        if lay.get("mlp"):
            h = _r(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps))
            x = x + mult * feed_forward(h, w, p + "mlp.", lay["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    x = _r(layer_norm(x, w["final.norm"], w["final.norm.b"], eps))
    z = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z


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
def retention_layer(heads=3, dim=8, vdim=12, decay=None, rot=8, base=500.0, mlp=None):
    decay = decay or [math.exp(-1.0 / (1.5 + 9.0 * h)) for h in range(heads)]
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    return {"type": "retention", "mixer": m, "mlp": mlp}


def wkv_layer(heads=2, dim=16, rank=6, mlp=None):
    """rank is not part of the configuration (a tensor's shape gives it); random_weights reads it from `_rank`."""
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp, "_rank": rank}


def attention_layer(heads=4, kv_heads=2, dim=8, vdim=12, scale=0.5, diff=0.3, size=9, keep=2, rot=4, base=300.0, kv_from=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
         "mask": {"size": size, "keep_first": keep}}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff=40):
    return {"kind": "dense", "ff": ff}


def mixture(experts=6, top=2, ff=16, shared=24):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def model_config(layers, width=32, vocab=61, eps=1e-5, mult=0.6, softcap=12.0):
    cfg = {"architecture": "Fedipel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult, "layers": layers}
    if softcap:
        cfg["logit_softcap"] = softcap
    return cfg


def config_json(cfg):
    """The configuration as a checkpoint's config.json holds it (without the test builders' private keys)."""
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in lay.items() if not k.startswith("_")} for lay in cfg["layers"]]
    return out


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Every tensor the configuration names, seeded, sized so that each mechanism moves the logits."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]

    def mat(o, i, s=1.0):
        return torch.randn(o, i, generator=g, dtype=torch.float32) * (s / math.sqrt(i))

    def vec(n, mean=0.0, s=1.0):
        n = n if isinstance(n, tuple) else (n,)
        return mean + s * torch.randn(*n, generator=g, dtype=torch.float32)

    def norm(name):
        w[name], w[name + ".b"] = vec(W, 1.0, 0.2), vec(W, 0.0, 0.2)

    w = {"embed": vec((V, W), 0.0, 1.0), "head": mat(V, W, 2.0)}
    norm("embed.norm")
    norm("final.norm")
    for i, lay in enumerate(cfg["layers"]):
        p, q, m = f"l{i}.", f"l{i}.mix.", lay["mixer"]
        norm(p + "norm1")
        if lay["type"] == "retention":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"], w[q + "g"] = mat(H * d, W, 2.0), mat(H * d, W, 2.0), mat(H * dv, W, 2.0), mat(H * dv, W)
            w[q + "o"] = mat(W, H * dv)
        elif lay["type"] == "wkv":
            H, d, R = m["heads"], m["dim"], lay.get("_rank", 6)
            for s in "rkvgw":
                w[q + "mu." + s] = vec(W, 0.5, 0.3)
            for s in "rkvg":
                w[q + s] = mat(H * d, W, 1.5)
            w[q + "w1"], w[q + "w2"], w[q + "w0"] = mat(R, W, 1.5), mat(H * d, R, 1.5), vec(H * d, -1.5, 0.8)
            w[q + "u"], w[q + "norm"], w[q + "o"] = vec((H, d), 0.3, 0.4), vec(H * d, 1.0, 0.2), mat(W, H * d)
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "q.b"] = mat(H * 2 * d, W, 2.0), vec(H * 2 * d, 0.0, 0.3)
            if m.get("kv_from") is None:
                w[q + "k"], w[q + "v"] = mat(G * 2 * d, W, 2.0), mat(G * dv, W)
                w[q + "k.b"], w[q + "v.b"] = vec(G * 2 * d, 0.0, 0.3), vec(G * dv, 0.0, 0.3)
            for s in ("lq1", "lk1", "lq2", "lk2"):
                w[q + s] = vec(d, 0.0, 0.5 / math.sqrt(d))
            w[q + "o"] = mat(W, H * dv)
        f = lay.get("mlp")
        if not f:
            continue
        norm(p + "norm2")
        r = p + "mlp."
        if f["kind"] == "dense":
            w[r + "gate"], w[r + "up"], w[r + "down"] = mat(f["ff"], W, 1.5), mat(f["ff"], W, 1.5), mat(W, f["ff"], 1.5)
        else:
            E, ff = f["router"]["experts"], f["expert"]["ff"]
            for e in range(E):
                w[f"{r}e{e}.up"], w[f"{r}e{e}.down"] = mat(ff, W, 1.5), mat(W, ff, 1.5)
            w[r + "router"], w[r + "router.b"] = mat(E, W, 3.0), vec(E, 0.0, 0.4)
            if f.get("shared"):
                fs = f["shared"]["ff"]
                w[r + "shared.up"], w[r + "shared.down"], w[r + "shared.sg"] = mat(fs, W, 1.5), mat(W, fs, 1.5), mat(1, W, 2.0)
    return {k: v.to(dtype) for k, v in w.items()}


def write_checkpoint(folder, cfg, w):
    """config.json + model.safetensors (8-byte little-endian header length, JSON header, raw data) in `folder`."""
    import json
    import os
    import struct
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(config_json(cfg), f)
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
