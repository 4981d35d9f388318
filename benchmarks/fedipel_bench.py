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
    aws = torch.empty(max(16, int(L.ao_lm_window_attention_workspace_bytes(1, 2, G, dv, ns))), dtype=torch.uint8, device=dev)

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
