"""A plain, slow statement of the Fedipel design, one function per mechanism, token by token where the design is a
recurrence.  It shares no code with the package: tests compare the package's kernels and step function against it.
Everything is computed in the dtype of the tensors it is given (float64 by default: the weights' own rounding is the only
one).  `w` maps checkpoint tensor names to tensors, `cfg` is the checkpoint's config.json as a dict.
"""
import math

import torch


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
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = m["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = unit_rms(o, eps).reshape(T, H * dv) * silu(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def wkv(h, w, p, m, eps):
    """Time mixing with a data-dependent decay per key channel and a bonus for the current token."""
    T, W = h.shape
    H, d = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros(1, W, dtype=h.dtype), h[:-1]], 0)
    mix = {s: h + (prev - h) * w[p + "mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w[p + "r"].T).view(T, H, d)
    k = (mix["k"] @ w[p + "k"].T).view(T, H, d)
    v = (mix["v"] @ w[p + "v"].T).view(T, H, d)
    gate = silu(mix["g"] @ w[p + "g"].T)
    dec = torch.exp(-torch.exp(torch.tanh(mix["w"] @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"])).view(T, H, d)
    u = w[p + "u"].view(H, d)
    o = torch.zeros(T, H, d, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, d, dtype=h.dtype)
        for t in range(T):
            kv = torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = (S + u[hd][:, None] * kv).T @ r[t, hd]
            S = dec[t, hd][:, None] * S + kv
    o = unit_rms(o, eps).reshape(T, H * d) * w[p + "norm"] * gate
    return o @ w[p + "o"].T


def attention_keys_values(h, w, p, m):
    """Rotated keys [T][G][2][d] and values [T][G][dv] of a layer that has projections of its own."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G * 2, d)
    k = rotate(k, torch.arange(T), rot["dims"], rot["base"], "interleaved").view(T, G, 2, d)
    v = (h @ w[p + "v"].T + w[p + "v.b"]).view(T, G, dv)
    return k, v


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
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = (j <= i) & ((i - j < size) | (j < keep))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for mp in range(2):
            s = (q[:, hd, mp] @ k[:, g, mp].T) * m["scale"]
            s = s.masked_fill(~seen, -math.inf)
            maps.append(torch.softmax(s, -1) @ v[:, g])
        out[:, hd] = unit_rms(maps[0] - lam * maps[1], eps) * (1.0 - m["diff"])
    return out.reshape(T, H * dv) @ w[p + "o"].T


def relu2_unit(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def feed_forward(h, w, p, f):
    if f["kind"] == "dense":
        return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T
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
        h = layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps)
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
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            x = x + mult * feed_forward(h, w, p + "mlp.", lay["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    x = layer_norm(x, w["final.norm"], w["final.norm.b"], eps)
    z = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
