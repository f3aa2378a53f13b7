"""Sparse mixture-of-experts feed-forward on the device (``csrc/moe_sparse.cu``): a router with softmax scores, an
additive correction that only steers the CHOICE, un-renormalised scaled weights and identity experts; expert GEMVs that
follow the expert index without a host round trip; a clamped gated activation; the weighted combination in fp32.

    s = softmax(Wr h + b);  chosen = top-k of (s + correction);  weight = s[chosen] * scale
    renormalised form:  chosen = top-k of the logits,  weight = softmax over the chosen logits only
    sigmoid form:       s = sigmoid(Wr h + b) per expert, then as the first form
    the weight multiplies the expert's output, or (``in_scale``) its input:  sum_j expert_j(w_j h)
    act(g, u) = g' * sigmoid(alpha * g') * (u' + shift),  g' = min(g, limit),  u' = clamp(u, -limit, limit)
    (limit = inf, alpha = 1, shift = 0 is the plain silu(g) * u)
    expert index >= E: identity expert (output = input)

Expert weights use the layout of the grouped expert layers (``modules/moe``): ``gate_up [E, W, 2F]``, ``down [E, F, W]``.
Every op has a PyTorch restatement for CPU.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch

from . import _lib

GROUP = "window_moe"
GLU_ALPHA = 1.702


def _code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and _lib.available(GROUP)


def clamped_glu_ref(gate: torch.Tensor, up: torch.Tensor, limit: float, alpha: float = GLU_ALPHA,
                    up_shift: float = 1.0, act: str = "sigmoid") -> torch.Tensor:
    g = gate.float().clamp(max=limit)
    u = up.float().clamp(-limit, limit)
    if act == "gelu_tanh":
        return (torch.nn.functional.gelu(g, approximate="tanh") * (u + up_shift)).to(gate.dtype)
    return (g * torch.sigmoid(alpha * g) * (u + up_shift)).to(gate.dtype)


def clamped_glu(gate_up: torch.Tensor, limit: float, alpha: float = GLU_ALPHA, up_shift: float = 1.0) -> torch.Tensor:
    """``gate_up [..., 2F]`` (gate | up) -> ``[..., F]``."""
    F = gate_up.shape[-1] // 2
    if _use_kernel(gate_up):
        gu = gate_up if gate_up.is_contiguous() else gate_up.contiguous()
        out = torch.empty(gu.shape[:-1] + (F,), dtype=gu.dtype, device=gu.device)
        L = _lib.lib(GROUP)
        rc = L.nxd_clamped_glu(_c.c_int(_code(gu.dtype)), _lib.ptr(gu), _lib.ptr(out), _c.c_longlong(gu.numel() // (2 * F)),
                               _c.c_int(F), _c.c_float(limit), _c.c_float(alpha), _c.c_float(up_shift), _lib.stream_ptr())
        _lib.check(rc, "nxd_clamped_glu", L)
        return out
    return clamped_glu_ref(gate_up[..., :F], gate_up[..., F:], limit, alpha, up_shift)


def glu_bias(src: torch.Tensor, gate_offset: int, up_offset: int, width: int, gate_bias: Optional[torch.Tensor] = None,
             up_bias: Optional[torch.Tensor] = None, limit: Optional[float] = None, alpha: float = GLU_ALPHA,
             up_shift: float = 1.0, act: str = "sigmoid") -> torch.Tensor:
    """Gated activation whose gate and up halves are column ranges of a wider projection output ``src [M, ld]``, each
    with an optional fp32 bias -> ``[M, width]``.  ``limit=None``: the plain ``silu(gate) * up``; ``act="gelu_tanh"``:
    the gate goes through the tanh form of gelu, ``0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3)))``."""
    if limit is None:
        limit, alpha, up_shift = float("inf"), 1.0, 0.0
    M = src.shape[0]
    if _use_kernel(src) and src.stride(1) == 1:
        out = torch.empty(M, width, dtype=src.dtype, device=src.device)
        gb = gate_bias.float().contiguous() if gate_bias is not None else None
        ub = up_bias.float().contiguous() if up_bias is not None else None
        L = _lib.lib(GROUP)
        rc = L.nxd_glu_bias(_c.c_int(_code(src.dtype)), _lib.ptr(src), _c.c_longlong(src.stride(0)), _c.c_int(gate_offset),
                            _c.c_int(up_offset), _lib.ptr(gb), _lib.ptr(ub), _lib.ptr(out), _c.c_longlong(M),
                            _c.c_int(width), _c.c_float(limit), _c.c_float(alpha), _c.c_float(up_shift),
                            _c.c_int(1 if act == "gelu_tanh" else 0), _lib.stream_ptr())
        _lib.check(rc, "nxd_glu_bias", L)
        return out
    g = src[:, gate_offset: gate_offset + width].float()
    u = src[:, up_offset: up_offset + width].float()
    if gate_bias is not None:
        g = g + gate_bias.float()
    if up_bias is not None:
        u = u + up_bias.float()
    return clamped_glu_ref(g, u, limit, alpha, up_shift, act).to(src.dtype)


def route(h: torch.Tensor, router_w: torch.Tensor, correction: Optional[torch.Tensor], top: int, scale: float,
          shared_gate_w: Optional[torch.Tensor] = None, logit_bias: Optional[torch.Tensor] = None,
          renormalize: bool = False, score: str = "softmax") -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]]:
    """``h [N, W]``, ``router_w [R, W]`` fp32 -> ``(index [N, top] int32, weight [N, top] fp32, shared gate [N] fp32)``.
    ``logit_bias [R]`` is added to the logits; ``renormalize``: the largest logits are chosen and weighted by the softmax
    over the chosen logits only (``correction`` does not apply); ``score="sigmoid"``: every expert's score is the sigmoid
    of its own logit instead of the softmax over all of them."""
    assert score in ("softmax", "sigmoid") and not (renormalize and score == "sigmoid")
    N, W = h.shape
    R = router_w.shape[0]
    if _use_kernel(h) and router_w.dtype == torch.float32:
        h = h if h.is_contiguous() else h.contiguous()
        idx = torch.empty(N, top, dtype=torch.int32, device=h.device)
        wts = torch.empty(N, top, dtype=torch.float32, device=h.device)
        sg = torch.empty(N, dtype=torch.float32, device=h.device) if shared_gate_w is not None else None
        corr = correction.float().contiguous() if correction is not None else None
        wsg = shared_gate_w.float().reshape(-1).contiguous() if shared_gate_w is not None else None
        zb = logit_bias.float().contiguous() if logit_bias is not None else None
        L = _lib.lib(GROUP)
        rc = L.nxd_moe_router(_c.c_int(_code(h.dtype)), _lib.ptr(h), _lib.ptr(router_w.contiguous()), _lib.ptr(corr),
                              _lib.ptr(wsg), _lib.ptr(idx), _lib.ptr(wts), _lib.ptr(sg), _c.c_longlong(N), _c.c_int(W),
                              _c.c_int(R), _c.c_int(top), _c.c_float(scale), _lib.ptr(zb),
                              _c.c_int(2 if score == "sigmoid" else int(renormalize)), _lib.stream_ptr())
        _lib.check(rc, "nxd_moe_router", L)
        return idx, wts, sg
    hf = h.float()
    z = hf @ router_w.float().t()
    if logit_bias is not None:
        z = z + logit_bias.float()
    sg = torch.sigmoid(hf @ shared_gate_w.float().reshape(-1)) if shared_gate_w is not None else None
    if renormalize:
        val, idx = torch.topk(z, top, dim=-1)
        return idx.to(torch.int32), torch.softmax(val, dim=-1) * scale, sg
    s = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, dim=-1)
    choice = s + correction.float() if correction is not None else s
    idx = torch.topk(choice, top, dim=-1).indices
    wts = s.gather(1, idx) * scale
    return idx.to(torch.int32), wts, sg


def gate_up_act(h: torch.Tensor, w_gate_up: torch.Tensor, idx: Optional[torch.Tensor], limit: float,
                alpha: float = GLU_ALPHA, up_shift: float = 1.0, in_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Activated intermediate of every (token, choice) pair: ``h [N, W]``, ``w_gate_up [E, W, 2F]``, ``idx [N, top]`` (or
    ``None``: one dense expert, ``top = 1``) -> ``[N * top, F]``.  Rows of identity experts are left untouched (zeros).
    ``in_scale [N, top]`` fp32: the pair's input row is multiplied by it (in fp32) before the products."""
    N, W = h.shape
    E, _, F2 = w_gate_up.shape
    F = F2 // 2
    top = idx.shape[1] if idx is not None else 1
    if _use_kernel(h) and w_gate_up.dtype == h.dtype:
        h = h if h.is_contiguous() else h.contiguous()
        act = torch.zeros(N * top, F, dtype=h.dtype, device=h.device)
        isc = in_scale.float().contiguous() if in_scale is not None else None
        L = _lib.lib(GROUP)
        rc = L.nxd_moe_gate_up_act(_c.c_int(_code(h.dtype)), _lib.ptr(h), _lib.ptr(w_gate_up), _lib.ptr(idx),
                                   _lib.ptr(act), _c.c_longlong(N * top), _c.c_int(top), _c.c_int(W), _c.c_int(F),
                                   _c.c_int(E), _c.c_float(limit), _c.c_float(alpha), _c.c_float(up_shift),
                                   _lib.ptr(isc), _lib.stream_ptr())
        _lib.check(rc, "nxd_moe_gate_up_act", L)
        return act
    act = torch.zeros(N * top, F, dtype=h.dtype, device=h.device)
    e_of = idx.reshape(-1).long() if idx is not None else torch.zeros(N, dtype=torch.long, device=h.device)
    tok = torch.arange(N, device=h.device).repeat_interleave(top)
    for e in range(E):
        rows = (e_of == e).nonzero().reshape(-1)
        if rows.numel():
            x = h[tok[rows]].float()
            if in_scale is not None:
                x = x * in_scale.reshape(-1)[rows].float().unsqueeze(1)
            gu = x @ w_gate_up[e].float()
            act[rows] = clamped_glu_ref(gu[:, :F], gu[:, F:], limit, alpha, up_shift).to(h.dtype)
    return act


def down_combine(act: torch.Tensor, w_down: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, h: torch.Tensor,
                 shared_act: Optional[torch.Tensor] = None, shared_down: Optional[torch.Tensor] = None,
                 shared_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``sum_j wts[t, j] * expert_j(act) (+ identity terms wts * h) (+ shared_gate * shared expert)`` -> fp32 ``[N, W]``.
    ``w_down [E, F, W]``, ``shared_down [Fs, W]``."""
    N, W = h.shape
    E, F, _ = w_down.shape
    top = idx.shape[1]
    if _use_kernel(h) and w_down.dtype == h.dtype:
        y = torch.empty(N, W, dtype=torch.float32, device=h.device)
        Fs = shared_act.shape[1] if shared_act is not None else 0
        L = _lib.lib(GROUP)
        rc = L.nxd_moe_down_combine(_c.c_int(_code(h.dtype)), _lib.ptr(act), _lib.ptr(w_down), _lib.ptr(idx),
                                    _lib.ptr(wts), _lib.ptr(h), _lib.ptr(shared_act), _lib.ptr(shared_down),
                                    _lib.ptr(shared_gate), _lib.ptr(y), _c.c_longlong(N), _c.c_int(top), _c.c_int(W),
                                    _c.c_int(F), _c.c_int(Fs), _c.c_int(E), _lib.stream_ptr())
        _lib.check(rc, "nxd_moe_down_combine", L)
        return y
    y = torch.zeros(N, W, dtype=torch.float32, device=h.device)
    il = idx.long()
    for j in range(top):
        e_of = il[:, j]
        ident = e_of >= E
        y[ident] += wts[ident, j:j + 1] * h[ident].float()
        for e in range(E):
            rows = (e_of == e).nonzero().reshape(-1)
            if rows.numel():
                y[rows] += wts[rows, j:j + 1] * (act[rows * top + j].float() @ w_down[e].float())
    if shared_act is not None:
        s = shared_act.float() @ shared_down.float()
        y += s * shared_gate.reshape(-1, 1) if shared_gate is not None else s
    return y


def gather_combine(ys: torch.Tensor, slot: torch.Tensor, idx: torch.Tensor, wts: torch.Tensor, h: torch.Tensor,
                   num_experts: int, shared_out: Optional[torch.Tensor] = None,
                   shared_gate: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Combination for the sorted (GEMM) path: ``ys [pairs, W]`` expert outputs in sorted order, ``slot [N, top]`` the row
    of every (token, choice) -> fp32 ``[N, W]``."""
    N, W = h.shape
    top = idx.shape[1]
    if _use_kernel(h) and ys.dtype == h.dtype:
        y = torch.empty(N, W, dtype=torch.float32, device=h.device)
        L = _lib.lib(GROUP)
        rc = L.nxd_moe_gather_combine(_c.c_int(_code(h.dtype)), _lib.ptr(ys), _lib.ptr(slot), _lib.ptr(idx), _lib.ptr(wts),
                                      _lib.ptr(h), _lib.ptr(shared_out), _lib.ptr(shared_gate), _lib.ptr(y),
                                      _c.c_longlong(N), _c.c_int(top), _c.c_int(W), _c.c_int(num_experts),
                                      _lib.stream_ptr())
        _lib.check(rc, "nxd_moe_gather_combine", L)
        return y
    ident = (idx >= num_experts).unsqueeze(-1)
    rows = torch.where(ident, h.float().unsqueeze(1), ys[slot.long().clamp(max=max(ys.shape[0] - 1, 0))].float()) \
        if ys.shape[0] else h.float().unsqueeze(1).expand(N, top, W)
    y = (rows * wts.unsqueeze(-1)).sum(1)
    if shared_out is not None:
        y = y + (shared_out.float() * shared_gate.reshape(-1, 1) if shared_gate is not None else shared_out.float())
    return y
