"""RMSNorm (optionally fused with the residual add) -- autograd wrapper."""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch

from . import _lib


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 and _lib.available()


def rms_norm_ref(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (y * w.float()).to(x.dtype)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, residual):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        res2 = res_out = None
        if residual is not None:
            res2 = residual.reshape(-1, H)
            if not res2.is_contiguous():
                res2 = res2.contiguous()
            res_out = torch.empty_like(x2)
        wc = w if w.dtype == torch.bfloat16 else w.to(torch.bfloat16)
        rc = _lib.lib().nxd_rmsnorm_fwd(_lib.ptr(x2), _lib.ptr(res2), _lib.ptr(wc), _lib.ptr(y), _lib.ptr(res_out),
                                        _lib.ptr(rstd), _c.c_int(rows), _c.c_int(H), _c.c_float(eps),
                                        _lib.stream_ptr())
        _lib.check(rc, "nxd_rmsnorm_fwd")
        normed_in = res_out if residual is not None else x2
        ctx.save_for_backward(normed_in, wc, rstd)
        ctx.has_residual = residual is not None
        ctx.w_dtype = w.dtype
        ctx.shape = x.shape
        if residual is not None:
            return y.reshape(x.shape), res_out.reshape(x.shape)
        return y.reshape(x.shape), None

    @staticmethod
    def backward(ctx, dy, dres_out):
        xin, wc, rstd = ctx.saved_tensors
        rows, H = xin.shape
        dy2 = dy.reshape(rows, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres2 = None
        if dres_out is not None:
            dres2 = dres_out.reshape(rows, H)
            if not dres2.is_contiguous():
                dres2 = dres2.contiguous()
        dx = torch.empty_like(xin)
        P = _lib.lib().nxd_rmsnorm_bwd_num_partials(_c.c_int(rows))
        scratch = torch.empty(P * H, dtype=torch.float32, device=xin.device)
        dw = torch.empty(H, dtype=torch.float32, device=xin.device)
        rc = _lib.lib().nxd_rmsnorm_bwd(_lib.ptr(dy2), _lib.ptr(xin), _lib.ptr(wc), _lib.ptr(rstd), _lib.ptr(dres2),
                                        _lib.ptr(dx), _lib.ptr(None), _lib.ptr(dw), _c.c_int(0), _lib.ptr(scratch),
                                        _c.c_int(rows), _c.c_int(H), _lib.stream_ptr())
        _lib.check(rc, "nxd_rmsnorm_bwd")
        dx = dx.reshape(ctx.shape)
        # d(x + r) flows equally to x and to the residual input
        return dx, dw.to(ctx.w_dtype), None, (dx if ctx.has_residual else None)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if _use_kernel(x):
        return _RMSNormFn.apply(x, w, eps, None)[0]
    return rms_norm_ref(x, w, eps)


def fused_add_rms_norm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor,
                       eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """``s = x + residual; return rmsnorm(s), s`` in one pass over HBM."""
    if _use_kernel(x):
        return _RMSNormFn.apply(x, w, eps, residual)
    s = x + residual
    return rms_norm_ref(s, w, eps), s


# ---- norm on a sublayer's OUTPUT, added to an fp32 residual stream (``csrc/post_norm.cu``) ---------------------------
_POST_GROUP = "window_moe"


def _post_code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def post_norm_residual_(x: torch.Tensor, y: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype = None,
                        offset: float = 1.0):
    """``x += y / sqrt(mean(y^2) + eps) * (offset + w)`` in place on the fp32 stream ``x``; returns ``(x, x.to(out_dtype))``
    (the rounded copy that the next sublayer's matrix products read; ``None`` without ``out_dtype``).  With
    ``offset = 1`` the weight is stored around zero."""
    assert x.dtype == torch.float32 and x.shape == y.shape
    W = x.shape[-1]
    if x.is_cuda and y.dtype in (torch.bfloat16, torch.float32) and _lib.available(_POST_GROUP):
        assert x.is_contiguous()
        y2 = y if y.is_contiguous() else y.contiguous()
        wc = w if w.dtype in (torch.bfloat16, torch.float32) else w.float()
        h = torch.empty(x.shape, dtype=out_dtype, device=x.device) if out_dtype is not None else None
        L = _lib.lib(_POST_GROUP)
        rc = L.nxd_post_norm_residual(_c.c_int(_post_code(y2.dtype)), _c.c_int(_post_code(wc.dtype)),
                                      _c.c_int(_post_code(out_dtype) if out_dtype is not None else 1), _lib.ptr(y2),
                                      _lib.ptr(wc), _lib.ptr(x), _lib.ptr(h), _c.c_longlong(x.numel() // W), _c.c_int(W),
                                      _c.c_float(eps), _c.c_float(offset), _lib.stream_ptr())
        _lib.check(rc, "nxd_post_norm_residual", L)
        return x, h
    yf = y.float()
    x.add_(yf / torch.sqrt(yf.pow(2).mean(-1, keepdim=True) + eps) * (offset + w.float()))
    return x, (x.to(out_dtype) if out_dtype is not None else None)


def rms_norm_offset(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype, offset: float = 1.0) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps) * (offset + w)`` with fp32 statistics, result in ``out_dtype``."""
    W = x.shape[-1]
    if x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and _lib.available(_POST_GROUP):
        x2 = x if x.is_contiguous() else x.contiguous()
        wc = w if w.dtype in (torch.bfloat16, torch.float32) else w.float()
        h = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        L = _lib.lib(_POST_GROUP)
        rc = L.nxd_post_norm_residual(_c.c_int(_post_code(x2.dtype)), _c.c_int(_post_code(wc.dtype)),
                                      _c.c_int(_post_code(out_dtype)), _lib.ptr(x2), _lib.ptr(wc), _lib.ptr(None),
                                      _lib.ptr(h), _c.c_longlong(x.numel() // W), _c.c_int(W), _c.c_float(eps),
                                      _c.c_float(offset), _lib.stream_ptr())
        _lib.check(rc, "nxd_post_norm_residual", L)
        return h
    xf = x.float()
    return (xf / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (offset + w.float())).to(out_dtype)


# ---- pre- and post-norm of a sublayer boundary in one pass over an fp32 stream (``csrc/post_norm.cu``) ---------------
def norm_ref(v: torch.Tensor, w: torch.Tensor, eps: float, center: bool) -> torch.Tensor:
    vf = v.float()
    if center:
        vf = vf - vf.mean(-1, keepdim=True)
    return vf / torch.sqrt(vf.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def norm_chain_(x: torch.Tensor, y: Optional[torch.Tensor], w_post: Optional[torch.Tensor],
                w_next: Optional[torch.Tensor], eps: float, out_dtype: Optional[torch.dtype] = None,
                center: bool = True):
    """``x += norm(y) * w_post`` in place on the fp32 stream ``x`` (skipped without ``y``), then
    ``h = (norm(x) * w_next).to(out_dtype)`` (skipped without ``w_next``); returns ``(x, h)``.  ``center``: layer norm
    without bias (mean removed, variance of the deviations); otherwise RMS norm.  Weights are plain (not one-plus)."""
    assert x.dtype == torch.float32 and (y is None or y.shape == x.shape)
    W = x.shape[-1]
    if x.is_cuda and (y is None or y.dtype in (torch.bfloat16, torch.float32)) and _lib.available("hybrid_serving"):
        assert x.is_contiguous()
        y2 = None if y is None else (y if y.is_contiguous() else y.contiguous())
        wp = None if w_post is None else w_post.float().contiguous()
        wn = None if w_next is None else w_next.float().contiguous()
        h = torch.empty(x.shape, dtype=out_dtype, device=x.device) if wn is not None else None
        L = _lib.lib("hybrid_serving")
        rc = L.nxd_norm_chain(_c.c_int(_post_code(y2.dtype) if y2 is not None else 1),
                              _c.c_int(_post_code(out_dtype) if h is not None else 1), _lib.ptr(y2), _lib.ptr(wp),
                              _lib.ptr(x), _lib.ptr(wn), _lib.ptr(h), _c.c_longlong(x.numel() // W), _c.c_int(W),
                              _c.c_float(eps), _c.c_int(int(center)), _lib.stream_ptr())
        _lib.check(rc, "nxd_norm_chain", L)
        return x, h
    if y is not None:
        x.add_(norm_ref(y, w_post, eps, center))
    return x, (norm_ref(x, w_next, eps, center).to(out_dtype) if w_next is not None else None)


# ---- parallel sublayers with layer scale and a gated residual, and the next norm, in one pass (``csrc/post_norm.cu``) ----
def gated_residual_norm_(x: torch.Tensor, y1: Optional[torch.Tensor], y2: Optional[torch.Tensor] = None,
                         y2_bias: Optional[torch.Tensor] = None, gate: Optional[torch.Tensor] = None,
                         gate_offsets=(0, 0), gate_bias1: Optional[torch.Tensor] = None,
                         gate_bias2: Optional[torch.Tensor] = None, scale1: Optional[torch.Tensor] = None,
                         scale2: Optional[torch.Tensor] = None, w_next: Optional[torch.Tensor] = None, eps: float = 1e-6,
                         out_dtype: Optional[torch.dtype] = None):
    """On the fp32 stream ``x [rows, W]``, in place:

        x += scale1 * sigmoid(gate[:, o1:o1+W] + gate_bias1) * y1 + scale2 * sigmoid(gate[:, o2:o2+W] + gate_bias2) * (y2 + y2_bias)

    then ``h = (x / sqrt(mean(x^2) + eps) * w_next).to(out_dtype)`` where ``w_next`` is ONE number (an RMS norm with a
    single weight for all coordinates).  ``y1 = None``: no update (the plain norm of the stream); ``y2``, ``gate``,
    scales, biases and ``w_next`` are optional.  ``gate [rows, ld]`` may be a wider projection output whose columns
    ``o1 ...`` / ``o2 ...`` are the two gates' pre-activations.  Returns ``(x, h)``."""
    assert x.dtype == torch.float32 and x.dim() == 2
    rows, W = x.shape
    ok = lambda t: t is None or (t.dtype in (torch.bfloat16, torch.float32) and t.stride(-1) == 1)     # noqa: E731
    if x.is_cuda and ok(y1) and ok(y2) and ok(gate) and _lib.available("delta_serving"):
        assert x.is_contiguous()
        y1c = None if y1 is None else (y1 if y1.is_contiguous() else y1.contiguous())
        y2c = None if y2 is None else (y2 if y2.is_contiguous() else y2.contiguous())
        f32 = lambda t: None if t is None else t.float().contiguous()                                    # noqa: E731
        wn, b2, g1, g2, s1, s2 = f32(w_next), f32(y2_bias), f32(gate_bias1), f32(gate_bias2), f32(scale1), f32(scale2)
        h = torch.empty(rows, W, dtype=out_dtype, device=x.device) if wn is not None else None
        code = lambda t: 1 if (t is None or t.dtype == torch.float32) else 0                            # noqa: E731
        L = _lib.lib("delta_serving")
        rc = L.nxd_gated_residual_norm(_lib.ptr(x), _lib.ptr(y1c), _c.c_int(code(y1c)), _lib.ptr(y2c), _c.c_int(code(y2c)),
                                       _lib.ptr(b2), _lib.ptr(gate), _c.c_int(code(gate)),
                                       _c.c_longlong(gate.stride(0) if gate is not None else 0),
                                       _c.c_int(gate_offsets[0]), _c.c_int(gate_offsets[1]), _lib.ptr(g1), _lib.ptr(g2),
                                       _lib.ptr(s1), _lib.ptr(s2), _lib.ptr(wn), _lib.ptr(h),
                                       _c.c_int(_post_code(out_dtype) if h is not None else 1), _c.c_longlong(rows),
                                       _c.c_int(W), _c.c_float(eps), _lib.stream_ptr())
        _lib.check(rc, "nxd_gated_residual_norm", L)
        return x, h

    def term(y, bias, off, gbias, scale):
        v = y.float()
        if bias is not None:
            v = v + bias.float()
        if scale is not None:
            v = v * scale.float()
        if gate is not None:
            z = gate[:, off: off + W].float()
            v = v * torch.sigmoid(z + gbias.float() if gbias is not None else z)
        return v

    if y1 is not None:
        upd = term(y1, None, gate_offsets[0], gate_bias1, scale1)
        if y2 is not None:
            upd = upd + term(y2, y2_bias, gate_offsets[1], gate_bias2, scale2)
        x.add_(upd)
    if w_next is None:
        return x, None
    return x, (x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w_next.float().reshape(())).to(out_dtype)
