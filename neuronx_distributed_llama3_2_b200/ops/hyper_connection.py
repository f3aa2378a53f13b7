"""Hyper-connections (``csrc/hyper_connection.cu``): the residual stream of a token is ``S`` parallel fp32 streams.

    read    u = sum_s in[s] x_s;   h = rms_norm(u) * w                      (what the sublayer gets)
    write   x_t <- sum_s mix[s, t] x_s + out[t] * y     for all t at once    (``mix`` is indexed [from, to])

``y`` is the sublayer's output, or the mean of two branch outputs that are each RMS-normed over the width with a weight of
their own.  ``hc_step`` does the write of one sublayer and the read of the next in one pass over the streams; with
``S = 1`` and all weights 1 it is the plain pre-norm residual.  (Zhu et al., "Hyper-Connections".)
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch

from . import _lib

GROUP = "retention_serving"
MAX_STREAMS = 8


def _code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def _rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def hc_step(streams: torch.Tensor, y: Optional[torch.Tensor] = None, mix: Optional[torch.Tensor] = None,
            out_w: Optional[torch.Tensor] = None, in_w: Optional[torch.Tensor] = None,
            norm_w: Optional[torch.Tensor] = None, eps: float = 1e-6, out_dtype: torch.dtype = torch.bfloat16,
            y2: Optional[torch.Tensor] = None, branch_w: Optional[Tuple[torch.Tensor, torch.Tensor]] = None
            ) -> Optional[torch.Tensor]:
    """``streams [N, S, W]`` fp32, updated IN PLACE when ``y [N, W]`` is given (``mix [S, S]``, ``out_w [S]``; with
    ``y2`` and ``branch_w = (w, w2)`` the written value is ``0.5 * (rms_norm(y) * w + rms_norm(y2) * w2)``).  With
    ``in_w [S]`` and ``norm_w [W]`` the normed weighted sum of the (new) streams is returned as ``[N, W]`` in
    ``out_dtype``; else ``None``."""
    N, S, W = streams.shape
    assert streams.dtype == torch.float32 and streams.is_contiguous()
    assert (y2 is None) == (branch_w is None)
    if streams.is_cuda and _lib.available(GROUP) and (y is None or y.dtype in (torch.bfloat16, torch.float32)):
        if y is not None:
            y = y if y.is_contiguous() else y.contiguous()
            if y2 is not None:
                y2 = y2.to(y.dtype)
                y2 = y2 if y2.is_contiguous() else y2.contiguous()
            if y.dtype == torch.bfloat16 and out_dtype == torch.float32:
                y, y2 = y.float(), (y2.float() if y2 is not None else None)
        h = torch.empty(N, W, dtype=out_dtype, device=streams.device) if in_w is not None else None
        wa, wb = branch_w if branch_w is not None else (None, None)
        L = _lib.lib(GROUP)
        rc = L.nxd_hc_step(_c.c_int(_code(y.dtype) if y is not None else 1), _c.c_int(_code(out_dtype)),
                           _lib.ptr(streams), _lib.ptr(y), _lib.ptr(y2), _lib.ptr(wa), _lib.ptr(wb), _lib.ptr(mix),
                           _lib.ptr(out_w), _lib.ptr(in_w), _lib.ptr(norm_w), _lib.ptr(h), _c.c_longlong(N), _c.c_int(S),
                           _c.c_int(W), _c.c_float(eps), _lib.stream_ptr())
        _lib.check(rc, "nxd_hc_step", L)
        return h
    if y is not None:
        yf = y.float()
        if y2 is not None:
            yf = 0.5 * (_rms(yf, eps) * branch_w[0].float() + _rms(y2.float(), eps) * branch_w[1].float())
        new = torch.einsum("st,nsw->ntw", mix.float(), streams) + out_w.float().reshape(1, S, 1) * yf.unsqueeze(1)
        streams.copy_(new)
    if in_w is None:
        return None
    u = torch.einsum("s,nsw->nw", in_w.float(), streams)
    return (_rms(u, eps) * norm_w.float()).to(out_dtype)
