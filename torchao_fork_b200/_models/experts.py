"""Mixtures of experts on chosen (token, expert) pairs, for any family whose experts are gated linear units,
y = W_down (g * sigmoid(alpha * g) * (u + shift)) with g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit), or
ungated units y = W_down act(W_up h) with act the square of ReLU (`chosen_experts(..., gated=False)`, `act_unit`):
a handful of tokens run as index-driven matrix-vector kernels (no host round trip: the step can be captured into a CUDA
graph), many tokens are sorted by expert around grouped library GEMMs.  The router that makes idx / weight is the
family's own."""
from typing import Optional

import torch

from .. import _lib


def _p(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def glu_unit(L, dt, x: torch.Tensor, w_gu: torch.Tensor, w_down: torch.Tensor, limit, alpha, shift, st, f32_out=True):
    """One dense unit over all rows: GEMM [gate | up] -> activation kernel -> GEMM down.  -> ([n][W], launches)."""
    n, ff = x.shape[0], w_down.shape[1]
    gu = torch.mm(x, w_gu.t())
    ya = torch.empty(n, ff, dtype=x.dtype, device=x.device)
    _lib.lm_check(L.ao_lm_glu_act_shift(_p(gu), dt, n, ff, limit, alpha, shift, _p(ya), st), "glu_act")
    if f32_out and x.dtype == torch.bfloat16:
        return torch.mm(ya, w_down.t(), out_dtype=torch.float32), 3
    return torch.mm(ya, w_down.t()), 3


ACT_RELU2, ACT_TANH, ACT_SOFTCAP = 0, 1, 2     # kinds of ao_lm_unary_rows


def act_unit(L, dt, x: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, row_scale: Optional[torch.Tensor], st, f32_out=True):
    """One ungated unit over all rows: GEMM up -> squared ReLU (times row_scale[t], fp32 [n], when given) -> GEMM down.
    -> ([n][W], launches)."""
    n, ff = x.shape[0], w_down.shape[1]
    u = torch.mm(x, w_up.t())
    ya = torch.empty(n, ff, dtype=x.dtype, device=x.device)
    _lib.lm_check(L.ao_lm_unary_rows(_p(u), dt, n, ff, ACT_RELU2, 0.0, _p(row_scale), 1, _p(ya), dt, st), "unary_rows")
    if f32_out and x.dtype == torch.bfloat16:
        return torch.mm(ya, w_down.t(), out_dtype=torch.float32), 3
    return torch.mm(ya, w_down.t()), 3


def chosen_experts(L, dt, xc: torch.Tensor, ridx: torch.Tensor, rwt: torch.Tensor, wgu: torch.Tensor, wd: torch.Tensor,
                   out: torch.Tensor, limit: float, alpha: float, shift: float, gemv: bool, accumulate: bool, st,
                   gated: bool = True) -> int:
    """out (fp32 [n][W]) = (accumulate ? out : 0) + sum_k rwt[t][k] * expert ridx[t][k] of xc[t].
    wgu [E][2 ff][W] (gate rows, then up rows; ungated experts: [E][ff][W], up rows only), wd [E][W][ff].
    Returns the launches made."""
    n, W = xc.shape
    E, top, ff = wgu.shape[0], ridx.shape[1], wd.shape[2]
    tdt, dev = xc.dtype, xc.device
    esz = wgu.element_size()

    def act(gu, rows, ya):
        if gated:
            _lib.lm_check(L.ao_lm_glu_act_shift(_p(gu), dt, rows, ff, limit, alpha, shift, _p(ya), st), "glu_act")
        else:
            _lib.lm_check(L.ao_lm_unary_rows(_p(gu), dt, rows, ff, ACT_RELU2, 0.0, None, 0, _p(ya), dt, st), "unary_rows")

    if gemv:
        ya = torch.empty(n * top, ff, dtype=tdt, device=dev)
        if gated:
            _lib.lm_check(L.ao_lm_expert_gate_up_shift(_p(xc), _p(wgu), _p(wgu) + ff * W * esz, dt, _p(ridx), n, top, W, ff, 2 * ff * W,
                                                       limit, alpha, shift, _p(ya), st), "expert_gate_up")
        else:
            _lib.lm_check(L.ao_lm_expert_up_act(_p(xc), _p(wgu), dt, _p(ridx), n, top, W, ff, ff * W, ACT_RELU2, _p(ya), st),
                          "expert_up_act")
        _lib.lm_check(L.ao_lm_expert_down(_p(ya), _p(wd), dt, _p(ridx), _p(rwt), n, top, W, ff, 1 if accumulate else 0, _p(out), st),
                      "expert_down")
        return 2
    launches = 0
    if not accumulate:
        out.zero_()
        launches += 1
    # rows sorted by expert: one grouped GEMM per projection (bf16), or one exact GEMM pair per expert that has rows (fp32)
    flat = ridx.view(-1)
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    mrows = n * top
    grouped = tdt == torch.bfloat16 and W % 8 == 0 and ff % 8 == 0 and hasattr(torch, "_grouped_mm")
    xs = torch.empty(mrows, W, dtype=tdt, device=dev)
    _lib.lm_check(L.ao_lm_gather_rows(_p(xc), dt, _p(order), top, mrows, W, _p(xs), st), "gather_rows")
    if grouped:
        offs = torch.cumsum(counts, 0).to(torch.int32)
        gu = torch._grouped_mm(xs, wgu.transpose(1, 2), offs=offs)
        ya = torch.empty(mrows, ff, dtype=tdt, device=dev)
        act(gu, mrows, ya)
        ys = torch._grouped_mm(ya, wd.transpose(1, 2), offs=offs)
        _lib.lm_check(L.ao_lm_scatter_add_rows(_p(ys), dt, _p(order), _p(rwt), top, mrows, W, _p(out), st), "scatter_add_rows")
        return launches + 9
    counts = counts.tolist()
    ys = torch.empty(mrows, W, dtype=tdt, device=dev)
    ya = torch.empty(max(counts), ff, dtype=tdt, device=dev)
    at = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        gu = torch.mm(xs[at:at + c], wgu[e].t())
        act(gu, c, ya)
        torch.mm(ya[:c], wd[e].t(), out=ys[at:at + c])
        at += c
        launches += 3
    _lib.lm_check(L.ao_lm_scatter_add_rows(_p(ys), dt, _p(order), _p(rwt), top, mrows, W, _p(out), st), "scatter_add_rows")
    return launches + 4
