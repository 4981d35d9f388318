"""Prefill and decode throughput of Rutusun layers at sizes of real models (random weights), beside the Llama family at
equal size in bf16 (same width, vocabulary and layer count, heads of 128 with 4:1 grouping, a feed-forward sized so that
the weights per layer match), and the design's own kernels timed alone against their roofline, each beside the like
kernel of the framework's other models.  `python bench.py --workload rutusun-layers` prints the result as one JSON line;
this file is the measurement.

Timing: CUDA events on the launching stream after 3 warm-up runs; model inputs and weights exceed L2, the kernel-alone
timings write a 256 MB buffer between runs.  Rooflines: measured copy bandwidth and cuBLAS bf16 rate of
MEASURED_PEAKS.json ("of measured"), or 6.65 TB/s and 1590 TF/s ("of fallback"); the fp32 multiply-add rate that the
matrix-state recurrence is held to is 148 SMs x 128 lanes x 2 x 1.9 GHz = 72 TF/s (nominal).
"""
import ctypes
import json
import math
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from benchmarks.bitipel_bench import peaks, timed  # noqa: E402
from benchmarks.tadolix_bench import llama_equal  # noqa: E402

FP32_TFLOPS = 148 * 128 * 2 * 1.9e9 / 1e12


def model_numbers(name, prompt_len, decode_ctx, decode_steps):
    """prefill tokens/s of a prompt and decode tokens/s (batch 1, CUDA graph) for Rutusun `name` and the Llama of equal size."""
    from torchao_fork_b200._models.llama.generate import Generator, prefill
    from torchao_fork_b200._models.rutusun import Rutusun, rutusun_configs
    dev = torch.device("cuda")
    out = {}
    cfg = rutusun_configs[name]()
    own_bytes = None
    for fam in ("rutusun", "llama"):
        model = Rutusun.from_name(name, dev) if fam == "rutusun" else llama_equal(cfg, own_bytes, dev)
        if fam == "rutusun":
            own_bytes = model.weight_bytes(True)
        S = max(prompt_len, decode_ctx + decode_steps + 8)
        gen = Generator(model, 1, S, temperature=0.0, top_k=None)
        prompt = torch.randint(0, cfg.vocab_size, (1, prompt_len), device=dev)
        pos = torch.arange(prompt_len, device=dev, dtype=torch.int32)
        with torch.no_grad():
            ms_prefill = timed(lambda: prefill(model, prompt, pos, temperature=0.0, top_k=None), iters=8, warmup=3)
            prefill(model, prompt[:, :decode_ctx], pos[:decode_ctx], temperature=0.0, top_k=None)

            def decode():
                gen.engine.set_state(torch.zeros(1, dtype=torch.int64, device=dev), decode_ctx)
                gen.decode_tokens(decode_steps)
            ms_decode = timed(decode, iters=3, warmup=2) / decode_steps
        wb = own_bytes if fam == "rutusun" else sum(p.numel() * p.element_size() for n, p in model.named_parameters()
                                                    if "tok_embeddings" not in n)
        out[fam] = {"prefill_tokens": prompt_len, "prefill_ms": round(ms_prefill, 3), "prefill_tok_per_s": round(prompt_len / ms_prefill * 1e3, 1),
                    "decode_context": decode_ctx, "decode_ms_per_token": round(ms_decode, 4), "decode_tok_per_s": round(1e3 / ms_decode, 1),
                    "decode_weight_gbs": round(wb / ms_decode / 1e6, 1),
                    "launches_per_decode_step": int(getattr(gen.engine, "launches_per_step", 0)), "weight_gb": round(wb / 1e9, 3)}
        if fam == "rutusun":
            out[fam]["state_bytes_per_sequence"] = model.state_bytes_per_sequence()
        del gen, model
        torch.cuda.empty_cache()
    return out


def kernel_numbers(name, prompt_len, decode_ctx):
    """The design's kernels alone, at one layer's shapes, with the like kernel of another family beside each."""
    from torchao_fork_b200 import _lib
    from torchao_fork_b200._models.rutusun import rutusun_configs
    from torchao_fork_b200._models.segment_step import REC_TILE, SCAN_TILE, chunk_tiles, scan_tiles
    hbm, tf, src = peaks()
    L = _lib.lm()
    dev = torch.device("cuda")
    st = torch.cuda.current_stream().cuda_stream
    cfg = rutusun_configs[name]()
    att = next(la for la in cfg.layers if la.type == "attention").mixer
    lin = next(la for la in cfg.layers if la.type == "lightning").mixer
    ssd = next(la for la in cfg.layers if la.type == "mamba2").mixer
    W = cfg.width
    H, G, d, dv = att.heads, att.kv_heads, att.dim, att.vdim
    flush = torch.zeros(64 << 20, dtype=torch.float32, device=dev)
    res = {"roofline_source": src, "hbm_gbs": hbm, "bf16_tflops": tf, "fp32_fma_tflops_nominal": round(FP32_TFLOPS, 1)}
    bf = dict(dtype=torch.bfloat16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    i32 = lambda v: torch.as_tensor(np.asarray(v, np.int32)).to(dev)
    n, C = prompt_len, max(prompt_len, decode_ctx + 1)

    # ---- causal attention with a sink over a whole prompt (tensor-core form), beside the chunked attention of the Tadolix
    # family at the same shape with one chunk as long as the prompt (gate and distance bias on), and the library attention
    pos_np = np.arange(n)
    slot, pos, back = i32(np.zeros(n)), i32(pos_np), i32(pos_np)
    tr = ctypes.c_int()
    L.ao_lm_chunk_attention_prompt_plan(0, H, G, d, dv, ctypes.byref(tr))
    qn = torch.randn(n, H, d, **f32)
    kn, vn = torch.randn(n, G, d, **bf), torch.randn(n, G, dv, **bf)
    ring_k, ring_v = torch.randn(1, C, G, d, **bf), torch.randn(1, C, G, dv, **bf)
    sink = torch.zeros(H, **f32)
    gate, bias = torch.randn(n, H * dv, **f32), torch.randn(H, 64, **f32)
    out = torch.empty(n, H * dv, **bf)
    pairs = n * (n + 1) / 2
    if tr.value:
        f, c = chunk_tiles(np.array([0]), np.array([n]), pos_np, tr.value, C)
        tf_, tc_ = i32(f), i32(c)

        def attend(g, b, s):
            _lib.lm_check(L.ao_lm_sink_attention_prompt(
                qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), 0, g, H * dv, b, 64, s,
                slot.data_ptr(), pos.data_ptr(), back.data_ptr(), tf_.data_ptr(), tc_.data_ptr(), len(f), H, G, d, dv, C, att.scale,
                0.0, 1.0, out.data_ptr(), H * dv, st), "sink_attention_prompt")
        flops, issued = 2.0 * pairs * H * (d + dv), 2.0 * pairs * H * (d + 3 * dv)
        for key, args in (("sink_attention_prefill", (None, None, sink.data_ptr())),
                          ("tadolix_chunk_attention_prefill_same_shape", (gate.data_ptr(), bias.data_ptr(), None))):
            ms = timed(lambda: attend(*args), flush=flush)
            res[key] = {"tokens": n, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                        "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4), "issued_tflops": round(issued / ms / 1e9, 2),
                        "frac_issued": round(issued / ms / 1e9 / tf, 4)}
    q = torch.randn(1, H, n, 128, **bf)
    ms = timed(lambda: torch.nn.functional.scaled_dot_product_attention(q, q, q, is_causal=True), flush=flush)
    flops = 2.0 * pairs * H * 256
    res["library_sdpa_same_pairs"] = {"tokens": n, "ms": round(ms, 3), "tflops": round(flops / ms / 1e9, 2),
                                      "frac_bf16_tensor_peak": round(flops / ms / 1e9 / tf, 4)}

    # ---- attention of one decoded token over decode_ctx cached keys: the cache rows are read once
    one, last, zero, cnt = i32([0]), i32([decode_ctx]), i32([0]), i32([1])
    o1 = torch.empty(1, H * dv, **bf)
    ns = max(1, min(-(-C // 32), -(-4 * 148 // G), 64))      # what the step function picks for one sequence
    aws = torch.empty(max(16, int(L.ao_lm_chunk_attention_workspace_bytes(1, G, dv, ns))), dtype=torch.uint8, device=dev)

    def attend_decode():
        _lib.lm_check(L.ao_lm_sink_attention(
            qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), ring_k.data_ptr(), ring_v.data_ptr(), 0, None, 0, None, 0, sink.data_ptr(),
            one.data_ptr(), last.data_ptr(), zero.data_ptr(), zero.data_ptr(), cnt.data_ptr(), 1, H, G, d, dv, C, att.scale, 0.0,
            1.0, ns, aws.data_ptr(), aws.numel(), o1.data_ptr(), H * dv, st), "sink_attention")
    ms = timed(attend_decode, flush=flush)
    byts = decode_ctx * G * (d + dv) * 2
    res["sink_attention_decode"] = {"keys": decode_ctx, "splits": ns, "us": round(ms * 1e3, 2), "cache_bytes": byts,
                                    "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    core = _lib.lib()
    q1 = torch.randn(1, H, 128, **bf)
    kc, vc = torch.randn(1, G, C, 128, **bf), torch.randn(1, G, C, 128, **bf)
    ipos = torch.full((1,), decode_ctx, dtype=torch.int32, device=dev)
    lo = torch.empty(1, H, 128, **bf)
    lns = max(1, min(64, -(-C // 32)))
    lws = torch.zeros(max(16, int(core.ao_b200_decode_attention_workspace_bytes(1, H, lns))), dtype=torch.uint8, device=dev)

    def llama_decode_attention():
        _lib.check(core.ao_b200_decode_attention(q1.data_ptr(), kc.data_ptr(), vc.data_ptr(), ipos.data_ptr(), lo.data_ptr(), 1, H, G,
                                                 128, C, 1.0 / math.sqrt(128), lns, lws.data_ptr(), lws.numel(), st), "decode_attention")
    ms = timed(llama_decode_attention, flush=flush)
    byts = 2 * G * decode_ctx * 128 * 2
    res["llama_attention_decode"] = {"keys": decode_ctx, "splits": lns, "us": round(ms * 1e3, 2), "cache_bytes": byts,
                                     "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}

    # ---- the matrix-state recurrence over a whole prompt and for one decoded token, in both forms
    seg_f, seg_c = i32([0]), i32([n])
    for key, mx in (("lightning", lin), ("mamba2", ssd)):
        if key == "lightning":
            Hh, Gg, dd, dvv = mx.heads, mx.heads, mx.dim, mx.vdim
        else:
            Hh, Gg, dd, dvv = mx.heads, mx.groups, mx.state, mx.vdim
        qq, kk, vv = torch.randn(n, Gg * dd, **f32), torch.randn(n, Gg * dd, **f32), torch.randn(n, Hh * dvv, **f32)
        a, b = torch.rand(n, Hh, **f32) * 0.1 + 0.9, torch.rand(n, Hh, **f32)
        a_head, skip = torch.full((Hh,), 0.95, **f32), torch.ones(Hh, **f32)
        state, o = torch.zeros(1, Hh, dd, dvv, **f32), torch.empty(n, Hh * dvv, **f32)
        lit = key == "lightning"

        rtf, rtc, rs0, rsn = [i32(t) for t in scan_tiles(np.array([0]), np.array([n]), REC_TILE)]
        rws = torch.empty(int(L.ao_lm_outer_recurrence_workspace_bytes(len(rtf), n, Hh, dd, dvv)) // 4, **f32)

        def rec(rows, sf_, sc, ps, tiled):
            _lib.lm_check(L.ao_lm_outer_recurrence(
                qq.data_ptr(), Gg * dd, kk.data_ptr(), Gg * dd, vv.data_ptr(), Hh * dvv, 1 if lit else 0, None if lit else a.data_ptr(),
                None if lit else b.data_ptr(), Hh, a_head.data_ptr() if lit else None, None if lit else skip.data_ptr(), Hh, Gg, dd,
                dvv, state.data_ptr(), slot.data_ptr(), ps.data_ptr(), sf_.data_ptr(), sc.data_ptr(), len(rtf) if tiled else 1,
                rs0.data_ptr() if tiled else None, rsn.data_ptr() if tiled else None, 1 if tiled else 0, rows,
                rws.data_ptr() if tiled else None, o.data_ptr(), Hh * dvv, st), "outer_recurrence")
        ms_seq = timed(lambda: rec(n, seg_f, seg_c, pos, False), flush=flush)
        ms = timed(lambda: rec(n, rtf, rtc, pos, True), flush=flush)
        flops = 4.0 * n * Hh * dd * dvv
        byts = n * (2 * Gg * dd + 2 * Hh * dvv) * 4
        res[key + "_recurrence_prefill"] = {"tokens": n, "heads": Hh, "d": dd, "dv": dvv, "ms": round(ms, 4), "ms_one_cta_per_segment": round(ms_seq, 4),
                                            "fp32_tflops": round(flops / ms / 1e9, 2), "frac_fp32_fma_nominal": round(flops / ms / 1e9 / FP32_TFLOPS, 4),
                                            "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
        ms = timed(lambda: rec(1, seg_f, cnt, last, False), flush=flush)
        byts = 2 * Hh * dd * dvv * 4      # the state is read and written once
        res[key + "_recurrence_decode"] = {"us": round(ms * 1e3, 2), "state_bytes": byts // 2, "gbs": round(byts / ms / 1e6, 1),
                                           "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    # the like kernel: the Tadolix family's gated per-channel recurrence over as many rows and W channels (three launches)
    sf, sc, seg0, segn = scan_tiles(np.array([0]), np.array([n]), SCAN_TILE)
    d_sf, d_sc, d_s0, d_sn = i32(sf), i32(sc), i32(seg0), i32(segn)
    proj = torch.randn(n, 3 * W, **f32)
    zb, xb = torch.zeros(W, **bf), torch.zeros(W, **bf)
    sstate, so = torch.zeros(1, W, **f32), torch.empty(n, W, **bf)
    ws = torch.empty(int(L.ao_lm_scan_workspace_bytes(len(sf), W)) // 4, **f32)

    def mingru():
        _lib.lm_check(L.ao_lm_mingru_scan(proj.data_ptr(), 3 * W, 0, W, 2 * W, zb.data_ptr(), xb.data_ptr(), 0, W, sstate.data_ptr(),
                                          slot.data_ptr(), pos.data_ptr(), back.data_ptr(), d_sf.data_ptr(), d_sc.data_ptr(), len(sf),
                                          d_s0.data_ptr(), d_sn.data_ptr(), 1, ws.data_ptr(), 1.0, so.data_ptr(), W, st), "mingru_scan")
    ms = timed(mingru, flush=flush)
    byts = n * W * (3 * 4 + 2)
    res["tadolix_mingru_scan_prefill"] = {"tokens": n, "channels": W, "ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1),
                                          "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}

    # ---- row kernels over a prompt: post-norm residual with the next norm (reads x fp32 and y fp32, writes x and h),
    # the state-space inputs, the gated group norm; beside the Tadolix family's read-out norm + write-back of one stream
    x, y, h = torch.randn(n, W, **f32), torch.randn(n, W, **f32), torch.empty(n, W, **bf)
    wa, wb_ = torch.ones(W, **bf), torch.ones(W, **bf)

    def post():
        _lib.lm_check(L.ao_lm_postnorm_residual(x.data_ptr(), y.data_ptr(), 1, None, wa.data_ptr(), None, None, wb_.data_ptr(), 0, 1e-6, n, W,
                                                h.data_ptr(), st), "postnorm_residual")
    ms = timed(post, flush=flush)
    byts = n * W * (4 + 4 + 4 + 2)
    res["postnorm_residual_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    xs = torch.randn(n, 1, W, **f32)

    def tadolix_pair():
        _lib.lm_check(L.ao_lm_streams_update(xs.data_ptr(), y.data_ptr(), 1, n, 1, W, None, None, 0, None, None, 0, None, None, None, st),
                      "streams_update")
        _lib.lm_check(L.ao_lm_streams_norm(xs.data_ptr(), None, n, 1, W, None, wa.data_ptr(), 0, 1.0, 1e-6, None, h.data_ptr(), st),
                      "streams_norm")
    ms = timed(tadolix_pair, flush=flush)
    byts = n * W * (4 + 4 + 4 + 4 + 2)
    res["tadolix_update_then_norm_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    inner, ch, Hs = ssd.inner, ssd.conv_channels, ssd.heads
    ld = 2 * inner + 2 * ssd.groups * ssd.state + Hs
    pj = torch.randn(n, ld, **f32)
    cw, cb = torch.randn(ch, ssd.conv, **bf), torch.zeros(ch, **bf)
    dtb, alog = torch.zeros(Hs, **bf), torch.zeros(Hs, **bf)
    cstate = torch.zeros(1, max(1, ssd.conv - 1), ch, **f32)
    co, ao, bo = torch.empty(n, ch, **f32), torch.empty(n, Hs, **f32), torch.empty(n, Hs, **f32)

    def prep():
        _lib.lm_check(L.ao_lm_ssd_prep(pj.data_ptr(), ld, inner, inner + ch, n, ch, ssd.conv, cw.data_ptr(), cb.data_ptr(), 0,
                                       cstate.data_ptr(), slot.data_ptr(), pos.data_ptr(), back.data_ptr(), Hs, dtb.data_ptr(),
                                       alog.data_ptr(), co.data_ptr(), ao.data_ptr(), bo.data_ptr(), st), "ssd_prep")
    ms = timed(prep, flush=flush)
    byts = n * ch * 8
    res["ssd_prep_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    go = torch.empty(n, inner, **bf)
    nw = torch.ones(inner, **bf)

    def gnorm():
        _lib.lm_check(L.ao_lm_gated_group_norm(co.data_ptr(), ch, pj.data_ptr(), ld, 1, n, inner, ssd.norm_groups, nw.data_ptr(), 0, 1e-6,
                                               go.data_ptr(), st), "gated_group_norm")
    ms = timed(gnorm, flush=flush)
    byts = n * inner * (4 + 4 + 2)
    res["gated_group_norm_prefill"] = {"ms": round(ms, 4), "gbs": round(byts / ms / 1e6, 1), "frac_hbm": round(byts / ms / 1e6 / hbm, 4)}
    return res


def run(sizes=("Rutusun-2k", "Rutusun-4k"), prompt_len=2048, decode_ctx=1536, decode_steps=64):
    out = {"metric": "rutusun_layers_prefill_decode", "dtype": "bf16", "data": "synthetic", "n_gpus": 1, "sizes": {}}
    for name in sizes:
        out["sizes"][name] = {"models": model_numbers(name, prompt_len, decode_ctx, decode_steps),
                              "kernels": kernel_numbers(name, prompt_len, decode_ctx)}
    return out


if __name__ == "__main__":
    print(json.dumps(run()))
