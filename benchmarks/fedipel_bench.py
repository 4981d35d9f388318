"""Prefill and decode throughput of Fedipel layers at sizes of real models (random weights), beside the framework's
closest existing family — Rutusun, which also mixes softmax attention, decayed linear attention and a second matrix-state
mixer — at equal size in bf16 (the named configurations of the same width, layer count, vocabulary and feed-forward), and
the design's own kernels timed alone against their roofline, each beside the like kernel of that family.
`python bench.py --workload fedipel-layers` prints the result as one JSON line; this file is the measurement.

Timing: CUDA events on the launching stream after 3 warm-up runs; model inputs and weights exceed L2, the kernel-alone
timings write a 256 MB buffer between runs.  Rooflines: measured copy bandwidth and cuBLAS bf16 rate of
MEASURED_PEAKS.json ("of measured"), or 6.65 TB/s and 1590 TF/s ("of fallback"); the fp32 multiply-add rate that the
matrix-state recurrences are held to is 148 SMs x 128 lanes x 2 x 1.9 GHz = 72 TF/s (nominal).
"""
import ctypes
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from benchmarks.bitipel_bench import peaks, timed  # noqa: E402

FP32_TFLOPS = 148 * 128 * 2 * 1.9e9 / 1e12


def model_numbers(name, other, prompt_len, decode_ctx, decode_steps):
    """prefill tokens/s of a prompt and decode tokens/s (batch 1, CUDA graph) for Fedipel `name` and Rutusun `other`."""
    from torchao_fork_b200._models import registry
    from torchao_fork_b200._models.llama.generate import Generator, prefill
    dev = torch.device("cuda")
    out = {}
    for fam, nm in (("fedipel", name), ("rutusun", other)):
        model = registry.random_init(nm, dev, torch.bfloat16)
        S = max(prompt_len, decode_ctx + decode_steps + 8)
        gen = Generator(model, 1, S, temperature=0.0, top_k=None)
        prompt = torch.randint(0, model.config.vocab_size, (1, prompt_len), device=dev)
        pos = torch.arange(prompt_len, device=dev, dtype=torch.int32)
        with torch.no_grad():
            ms_prefill = timed(lambda: prefill(model, prompt, pos, temperature=0.0, top_k=None), iters=8, warmup=3)
            prefill(model, prompt[:, :decode_ctx], pos[:decode_ctx], temperature=0.0, top_k=None)

            def decode():
                gen.engine.set_state(torch.zeros(1, dtype=torch.int64, device=dev), decode_ctx)
                gen.decode_tokens(decode_steps)
            ms_decode = timed(decode, iters=3, warmup=2) / decode_steps
        wb = model.weight_bytes(True)
        out[fam] = {"configuration": nm, "prefill_tokens": prompt_len, "prefill_ms": round(ms_prefill, 3),
                    "prefill_tok_per_s": round(prompt_len / ms_prefill * 1e3, 1), "decode_context": decode_ctx,
                    "decode_ms_per_token": round(ms_decode, 4), "decode_tok_per_s": round(1e3 / ms_decode, 1),
                    "decode_weight_gbs": round(wb / ms_decode / 1e6, 1),
                    "launches_per_decode_step": int(getattr(gen.engine, "launches_per_step", 0)), "weight_gb": round(wb / 1e9, 3),
                    "state_bytes_per_sequence": model.state_bytes_per_sequence()}
        del gen, model
        torch.cuda.empty_cache()
    return out


def kernel_numbers(name, prompt_len, decode_ctx):
    """The design's kernels alone, at one layer's shapes, with the like kernel of the Rutusun family beside each."""
    from torchao_fork_b200 import _lib
    from torchao_fork_b200._models.fedipel import fedipel_configs
    from torchao_fork_b200._models.segment_step import REC_TILE, chunk_tiles, scan_tiles
    hbm, tf, src = peaks()
    L = _lib.lm()
    dev = torch.device("cuda")
    st = torch.cuda.current_stream().cuda_stream
    cfg = fedipel_configs[name]()
    att = next(la for la in cfg.layers if la.type == "attention").mixer
    ret = next(la for la in cfg.layers if la.type == "retention").mixer
    wkv = next(la for la in cfg.layers if la.type == "wkv").mixer
    W = cfg.width
    H, G, d, dv = att.heads, att.kv_heads, att.dim, att.vdim
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    res = {"roofline_source": src, "hbm_gbs": hbm, "bf16_tflops": tf, "fp32_fma_tflops_nominal": round(FP32_TFLOPS, 1)}
    bf = dict(dtype=torch.bfloat16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    i32 = lambda v: torch.as_tensor(np.asarray(v, np.int32)).to(dev)
    p = lambda t: None if t is None else t.data_ptr()
    n, C = prompt_len, max(prompt_len, decode_ctx + 1)
    pos_np = np.arange(n)
    slot, pos, back = i32(np.zeros(n)), i32(pos_np), i32(pos_np)

    def frac(byts, ms):
        return {"gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}

    # ---- window attention over a whole prompt that the window covers (tensor-core form, two maps of d with values of dv),
    # beside the sink attention of the Rutusun family (one map of 2 d) over the same pairs
    tr = ctypes.c_int()
    L.ao_lm_window_attention_prompt_plan(0, 2, H, G, d, dv, ctypes.byref(tr))
    qn = torch.randn(n, H, 2, d, **f32)
    kn, vn = torch.randn(n, G, 2, d, **bf), torch.randn(n, G, dv, **bf)
    ring_k, ring_v = torch.randn(1, C, G, 2 * d, **bf), torch.randn(1, C, G, dv, **bf)
    first_k, first_v = torch.randn(1, 8, G, 2 * d, **bf), torch.randn(1, 8, G, dv, **bf)
    out = torch.empty(n, H * dv, **bf)
    pairs = n * (n + 1) / 2
    f, c = chunk_tiles(np.array([0]), np.array([n]), pos_np, tr.value, 1 << 30)
    tf_, tc_ = i32(f), i32(c)

    def win_prompt():
        _lib.lm_check(L.ao_lm_window_attention_prompt(p(qn), p(kn), p(vn), p(ring_k), p(ring_v), p(first_k), p(first_v), C, 8, 0, p(slot),
                                                      p(pos), p(back), p(tf_), p(tc_), len(f), 2, H, G, d, dv, C, 4, att.scale, 0.7, 1,
                                                      1e-6, 0.5, p(out), H * dv, st), "window_attention_prompt")
    ms = timed(win_prompt, flush=flush)
    flops, issued = 2.0 * pairs * H * 2 * (d + dv), 2.0 * pairs * H * 2 * (d + 3 * dv)
    res["window_attention_prefill"] = {"tokens": n, "maps": 2, "d": d, "dv": dv, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                                       "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4), "issued_tflops": round(issued / ms / 1e9, 2),
                                       "frac_issued": round(issued / ms / 1e9 / tf, 4)}
    L.ao_lm_chunk_attention_prompt_plan(0, H, G, 2 * d, dv, ctypes.byref(tr))
    sq, sk = torch.randn(n, H, 2 * d, **f32), torch.randn(n, G, 2 * d, **bf)
    sink = torch.zeros(H, **f32)
    if tr.value:
        f2, c2 = chunk_tiles(np.array([0]), np.array([n]), pos_np, tr.value, C)
        tf2, tc2 = i32(f2), i32(c2)

        def sink_prompt():
            _lib.lm_check(L.ao_lm_sink_attention_prompt(p(sq), p(sk), p(vn), p(ring_k), p(ring_v), 0, None, H * dv, None, 64, p(sink),
                                                        p(slot), p(pos), p(back), p(tf2), p(tc2), len(f2), H, G, 2 * d, dv, C, att.scale,
                                                        0.0, 1.0, p(out), H * dv, st), "sink_attention_prompt")
        ms = timed(sink_prompt, flush=flush)
        flops, issued = 2.0 * pairs * H * (2 * d + dv), 2.0 * pairs * H * (2 * d + 3 * dv)
        res["rutusun_sink_attention_prefill_same_pairs"] = {"tokens": n, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                                                            "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4),
                                                            "issued_tflops": round(issued / ms / 1e9, 2),
                                                            "frac_issued": round(issued / ms / 1e9 / tf, 4)}

    # ---- attention of one decoded token over decode_ctx cached keys (fp32 form with key splits): the cache rows are read once
    one, last, zero, cnt = i32([0]), i32([decode_ctx]), i32([0]), i32([1])
    o1 = torch.empty(1, H * dv, **bf)
    ns = max(1, min(-(-(C + 4) // 32), -(-4 * 148 // G), 64))      # what the step function picks for one sequence
    aws = torch.empty(max(16, int(L.ao_lm_window_attention_workspace_bytes(1, 2, H, G, dv, ns))), dtype=torch.uint8, device=dev)

    def win_decode():
        _lib.lm_check(L.ao_lm_window_attention(p(qn), p(kn), p(vn), p(ring_k), p(ring_v), p(first_k), p(first_v), C, 8, 0, p(one), p(last),
                                               p(zero), p(zero), p(cnt), 1, 2, H, G, d, dv, C, 4, att.scale, 0.7, 1, 1e-6, 0.5, ns, p(aws),
                                               aws.numel(), p(o1), H * dv, st), "window_attention")
    ms = timed(win_decode, flush=flush)
    byts = decode_ctx * G * (2 * d + dv) * 2
    res["window_attention_decode"] = {"keys": decode_ctx, "splits": ns, "us": round(ms * 1e3, 2), "cache_bytes": byts, **frac(byts, ms)}
    ns2 = max(1, min(-(-C // 32), -(-4 * 148 // G), 64))
    aws2 = torch.empty(max(16, int(L.ao_lm_chunk_attention_workspace_bytes(1, G, dv, ns2))), dtype=torch.uint8, device=dev)

    def sink_decode():
        _lib.lm_check(L.ao_lm_sink_attention(p(sq), p(sk), p(vn), p(ring_k), p(ring_v), 0, None, 0, None, 0, p(sink), p(one), p(last),
                                             p(zero), p(zero), p(cnt), 1, H, G, 2 * d, dv, C, att.scale, 0.0, 1.0, ns2, p(aws2),
                                             aws2.numel(), p(o1), H * dv, st), "sink_attention")
    ms = timed(sink_decode, flush=flush)
    res["rutusun_sink_attention_decode"] = {"keys": decode_ctx, "splits": ns2, "us": round(ms * 1e3, 2), "cache_bytes": byts, **frac(byts, ms)}
    return res, dict(L=L, _lib=_lib, cfg=cfg, ret=ret, wkv=wkv, att=att, W=W, n=n, flush=flush, bf=bf, f32=f32, i32=i32, p=p, st=st,
                     slot=slot, pos=pos, back=back, last=last, cnt=cnt, frac=frac, hbm=hbm, REC_TILE=REC_TILE, scan_tiles=scan_tiles)


def recurrence_and_row_numbers(res, k):
    """Second half of the kernels alone: the two matrix-state recurrences and the row kernels."""
    L, _lib, cfg, ret, wkv, W, n = k["L"], k["_lib"], k["cfg"], k["ret"], k["wkv"], k["W"], k["n"]
    flush, bf, f32, i32, p, st, frac = k["flush"], k["bf"], k["f32"], k["i32"], k["p"], k["st"], k["frac"]
    slot, pos, back, last, cnt = k["slot"], k["pos"], k["back"], k["last"], k["cnt"]
    seg_f, seg_c = i32([0]), i32([n])
    rtf, rtc, rs0, rsn = [i32(t) for t in k["scan_tiles"](np.array([0]), np.array([n]), k["REC_TILE"])]

    # ---- time mixing (decay per token and key channel, bonus) beside the fixed-decay recurrence that retention shares with
    # the Rutusun family's lightning mixer, at the same heads and head sizes
    Hh, dd = wkv.heads, wkv.dim
    r_, k_, v_, z_ = (torch.randn(n, Hh * dd, **f32) for _ in range(4))
    w0, u = torch.randn(Hh * dd, **bf) - 1.5, torch.randn(Hh, dd, **bf)
    state, o = torch.zeros(1, Hh, dd, dd, **f32), torch.empty(n, Hh * dd, **f32)
    hsrc, shift = torch.randn(n, W, **f32), torch.zeros(1, W, **f32)
    cws = torch.empty(int(L.ao_lm_channel_recurrence_workspace_bytes(len(rtf), n, Hh, dd, dd)) // 4, **f32)
    ows = torch.empty(int(L.ao_lm_outer_recurrence_workspace_bytes(len(rtf), n, Hh, dd, dd)) // 4, **f32)
    a_head = torch.full((Hh,), 0.97, **f32)

    def chan(rows, sf_, sc, ps, tiled):
        _lib.lm_check(L.ao_lm_channel_recurrence(p(r_), Hh * dd, p(k_), Hh * dd, p(v_), Hh * dd, p(z_), Hh * dd, p(w0), p(u), 0, Hh, dd, dd,
                                                 p(state), p(slot), p(ps), p(sf_), p(sc), len(rtf) if tiled else 1, p(rs0) if tiled else None,
                                                 p(rsn) if tiled else None, 1 if tiled else 0, rows, p(cws) if tiled else None, p(hsrc),
                                                 p(shift), W, p(o), Hh * dd, st), "channel_recurrence")

    def outer(rows, sf_, sc, ps, tiled):
        _lib.lm_check(L.ao_lm_outer_recurrence(p(r_), Hh * dd, p(k_), Hh * dd, p(v_), Hh * dd, 0, None, None, Hh, p(a_head), None, Hh, Hh, dd,
                                               dd, p(state), p(slot), p(ps), p(sf_), p(sc), len(rtf) if tiled else 1, p(rs0) if tiled else None,
                                               p(rsn) if tiled else None, 1 if tiled else 0, rows, p(ows) if tiled else None, p(o), Hh * dd,
                                               st), "outer_recurrence")
    flops = 4.0 * n * Hh * dd * dd
    for key, fn, streams in (("time_mixing_recurrence", chan, 5), ("fixed_decay_recurrence_same_shape", outer, 4)):
        ms = timed(lambda: fn(n, rtf, rtc, pos, True), flush=flush)
        byts = n * Hh * dd * 4 * streams
        res[key + "_prefill"] = {"tokens": n, "heads": Hh, "d": dd, "dv": dd, "ms": round(ms, 4), "fp32_tflops": round(flops / ms / 1e9, 2),
                                 "frac_fp32_fma_nominal": round(flops / ms / 1e9 / FP32_TFLOPS, 4), **frac(byts, ms)}
        ms = timed(lambda: fn(1, seg_f, cnt, last, False), flush=flush)
        byts = 2 * Hh * dd * dd * 4      # the state is read and written once
        res[key + "_decode"] = {"us": round(ms * 1e3, 2), "state_bytes": byts // 2, **frac(byts, ms)}

    # ---- row kernels over a prompt: residual add + layer norm beside the Rutusun family's post-norm residual (the same
    # traffic: x read and written, y read, h written); token shift; rotations; the gated unit-RMS norm in both gate modes
    x, y, h = torch.randn(n, W, **f32), torch.randn(n, W, **f32), torch.empty(n, W, **bf)
    wa, wb_ = torch.ones(W, **bf), torch.zeros(W, **bf)

    def add_ln():
        _lib.lm_check(L.ao_lm_add_layer_norm(p(x), p(y), 0.01, None, n, W, p(wa), p(wb_), 0, 1e-6, None, p(h), st), "add_layer_norm")

    def post():
        _lib.lm_check(L.ao_lm_postnorm_residual(p(x), p(y), 1, None, p(wa), None, None, p(wa), 0, 1e-6, n, W, p(h), st), "postnorm_residual")
    byts = n * W * (4 + 4 + 4 + 2)
    res["add_layer_norm_prefill"] = {"ms": round(ms := timed(add_ln, flush=flush), 4), **frac(byts, ms)}
    res["rutusun_postnorm_residual_prefill"] = {"ms": round(ms := timed(post, flush=flush), 4), **frac(byts, ms)}
    mu, mixes = torch.rand(5, W, **bf), torch.empty(5, n, W, **bf)

    def shift_mix():
        _lib.lm_check(L.ao_lm_token_shift_mix(p(x), p(mu), 5, 0, p(shift), p(slot), p(pos), p(back), n, W, p(mixes), st), "token_shift_mix")
    res["token_shift_mix_prefill"] = {"ms": round(ms := timed(shift_mix, flush=flush), 4), **frac(n * W * (4 + 5 * 2), ms)}
    Hr, dr, dvr = ret.heads, ret.dim, ret.vdim
    ld = 2 * Hr * (dr + dvr)
    proj = torch.randn(n, ld, **f32)
    inv = ret.rot.inv_freq(proj.device)

    def rotary():
        _lib.lm_check(L.ao_lm_rotary_rows(p(proj), ld, n, p(pos), p(inv), ret.rot.dims, 1, dr, 0, Hr, 1.0, Hr * dr, Hr, 0.999, st), "rotary_rows")
    res["rotary_rows_prefill"] = {"ms": round(ms := timed(rotary, flush=flush), 4), **frac(n * 2 * Hr * dr * 8, ms)}
    a = k["att"]
    H, G, d, dv = a.heads, a.kv_heads, a.dim, a.vdim
    lda = 2 * H * d + 2 * G * d + G * dv
    pj = torch.randn(n, lda, **f32)
    qb, kb, vb = torch.zeros(2 * H * d, **bf), torch.zeros(2 * G * d, **bf), torch.zeros(G * dv, **bf)
    qn, kn, vn = torch.empty(n, 2 * H, d, **f32), torch.empty(n, 2 * G, d, **bf), torch.empty(n, G * dv, **bf)
    inv_a = a.rot.inv_freq(proj.device)

    def prep():
        _lib.lm_check(L.ao_lm_qkv_rotary_prep(p(pj), lda, 0, 2 * H * d, 2 * H * d + 2 * G * d, p(qb), p(kb), p(vb), p(pos), p(inv_a),
                                              a.rot.dims, 0, n, 2 * H, 2 * G, d, G * dv, 0, p(qn), p(kn), p(vn), st), "qkv_rotary_prep")
    res["qkv_rotary_prep_prefill"] = {"ms": round(ms := timed(prep, flush=flush), 4),
                                      **frac(n * (lda * 4 + 2 * H * d * 4 + (2 * G * d + G * dv) * 2), ms)}
    rec, gate, go = torch.randn(n, Hr * dvr, **f32), torch.randn(n, Hr * dvr, **f32), torch.empty(n, Hr * dvr, **bf)
    nw = torch.ones(Hr * dvr, **bf)
    for key, mode, wt in (("unit_rms_silu_gate_prefill", 2, None), ("rutusun_gated_norm_sigmoid_prefill", 0, nw)):
        def gnorm():
            _lib.lm_check(L.ao_lm_gated_group_norm(p(rec), Hr * dvr, p(gate), Hr * dvr, mode, n, Hr * dvr, Hr if mode == 2 else 1, p(wt), 0,
                                                   1e-6, p(go), st), "gated_group_norm")
        res[key] = {"ms": round(ms := timed(gnorm, flush=flush), 4), **frac(n * Hr * dvr * (4 + 4 + 2), ms)}
    return res


def run(sizes=(("Fedipel-2k", "Rutusun-2k"), ("Fedipel-4k", "Rutusun-4k")), expert_sizes=(("Fedipel-2k-moe", "Rutusun-2k-moe"),),
        prompt_len=2048, decode_ctx=1536, decode_steps=64):
    """`sizes`: whole models and the kernels alone; `expert_sizes`: whole models whose odd layers are mixtures of experts
    (the mixers are those of the first size of the same width, so their kernels are not timed again)."""
    out = {"metric": "fedipel_layers_prefill_decode", "dtype": "bf16", "data": "synthetic", "n_gpus": 1, "sizes": {}}
    for name, other in sizes:
        res, k = kernel_numbers(name, prompt_len, decode_ctx)
        out["sizes"][name] = {"models": model_numbers(name, other, prompt_len, decode_ctx, decode_steps),
                              "kernels": recurrence_and_row_numbers(res, k)}
    for name, other in expert_sizes:
        out["sizes"][name] = {"models": model_numbers(name, other, prompt_len, decode_ctx, decode_steps)}
    return out


if __name__ == "__main__":
    print(json.dumps(run()))
