"""Gated delta rule ops over a per-line fp32 state (``csrc/delta_rule.cu``): a recurrent mixer whose matrix memory is
decayed, corrected by the error of its own prediction, and read out, per head and token:

    S <- g_t * S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t          S [dim, vdim]

(the delta rule with a decay gate; Yang, Kautz, Hatamizadeh, "Gated Delta Networks: Improving Mamba2 with Delta Rule").
``g_t = exp(-exp(A) softplus(a_t + dt_bias))`` is one number per head, or one per head and key channel (it then scales
the rows of ``S``); ``beta_t = sigmoid(b_t)``.  Queries, keys and values pass a short causal convolution over time (per
channel, no bias, zeros before the start) and silu; queries and keys are then unit vectors per head,
``x / sqrt(sum x^2 + unit_eps)``, the queries times ``qscale``.

State per cache line: ``S [heads, dim, vdim]`` and the last ``taps - 1`` raw projections ``[taps - 1, channels]``, both
fp32.  A row whose first position is 0 starts from zeros; any other row continues from what its line holds, so a prompt
may arrive in portions and a line that is handed to a new request needs no clearing.  Decays, beta, the unit norms and
the state are fp32 whatever the activation dtype.  Every op has a PyTorch restatement for CPU.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

GROUP = "delta_serving"


def _code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and _lib.available(GROUP)


def _i32(t):
    if t is None:
        return None
    return t if (t.dtype == torch.int32 and t.is_contiguous()) else t.to(torch.int32).contiguous()


def _rows(x: torch.Tensor) -> Tuple[torch.Tensor, int]:
    """``x [B, T, n]`` as rows of a (possibly wider) buffer: the tensor and the distance between rows in elements."""
    B, T, _ = x.shape
    if x.stride(2) == 1 and (B == 1 or x.stride(0) == T * x.stride(1)):
        return x, x.stride(1)
    x = x.contiguous()
    return x, x.stride(1)


def delta_prep(proj: torch.Tensor, offsets: Tuple[int, int, int], conv_w: torch.Tensor, conv_state: torch.Tensor,
               q_start: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, qscale: float,
               unit_eps: float = 1e-6, n_new: Optional[torch.Tensor] = None,
               seq_ids: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``proj [B, T, ld]`` holds the raw projections at columns ``offsets = (q, k, v)`` (``kv_heads * dim``,
    ``kv_heads * dim``, ``heads * vdim`` channels); ``conv_w [channels, taps]`` fp32 in q | k | v order (last column = the
    current token); ``conv_state [lines, taps - 1, channels]`` fp32, moved to the end of the step in place.
    Returns fp32 ``(q [B, T, kv_heads, dim], k [B, T, kv_heads, dim], v [B, T, heads, vdim])``."""
    B, T, _ = proj.shape
    G, H, D, Dv = kv_heads, heads, dim, vdim
    C, taps = conv_w.shape
    K = taps - 1
    assert C == 2 * G * D + H * Dv and conv_state.shape[1:] == (K, C), (conv_w.shape, conv_state.shape)
    if _use_kernel(proj):
        proj, ld = _rows(proj)
        dev = proj.device
        qn = torch.empty(B, T, G, D, dtype=torch.float32, device=dev)
        kn = torch.empty(B, T, G, D, dtype=torch.float32, device=dev)
        vn = torch.empty(B, T, H, Dv, dtype=torch.float32, device=dev)
        qs, nn_, sid = _i32(q_start), _i32(n_new), _i32(seq_ids)
        L = _lib.lib(GROUP)
        common = (_c.c_int(_code(proj.dtype)), _lib.ptr(proj), _c.c_longlong(ld), _c.c_int(offsets[0]),
                  _c.c_int(offsets[1]), _c.c_int(offsets[2]))
        rc = L.nxd_delta_prep(*common, _lib.ptr(conv_w), _lib.ptr(conv_state), _lib.ptr(qn), _lib.ptr(kn), _lib.ptr(vn),
                              _lib.ptr(qs), _lib.ptr(nn_), _lib.ptr(sid), _c.c_int(B), _c.c_int(T), _c.c_int(H),
                              _c.c_int(G), _c.c_int(D), _c.c_int(Dv), _c.c_int(taps), _c.c_float(qscale),
                              _c.c_float(unit_eps), _lib.stream_ptr())
        _lib.check(rc, "nxd_delta_prep", L)
        rc = L.nxd_delta_conv_state(*common, _lib.ptr(conv_state), _lib.ptr(qs), _lib.ptr(nn_), _lib.ptr(sid),
                                    _c.c_int(B), _c.c_int(T), _c.c_int(H), _c.c_int(G), _c.c_int(D), _c.c_int(Dv),
                                    _c.c_int(taps), _lib.stream_ptr())
        _lib.check(rc, "nxd_delta_conv_state", L)
        return qn, kn, vn
    raw = torch.cat([proj[..., offsets[0]: offsets[0] + G * D], proj[..., offsets[1]: offsets[1] + G * D],
                     proj[..., offsets[2]: offsets[2] + H * Dv]], dim=-1).float()                  # [B, T, C]
    out = torch.zeros(B, T, C, dtype=torch.float32, device=proj.device)
    w = conv_w.float()
    for b in range(B):
        n = T if n_new is None else min(int(n_new[b]), T)
        if n <= 0:
            continue
        line = b if seq_ids is None else int(seq_ids[b])
        p0 = int(q_start[b])
        past = conv_state[line].clone()
        if p0 < K:                                         # positions before the start of the sequence are zeros
            past[: K - p0] = 0.0
        seq = torch.cat([past, raw[b, :n]], dim=0)         # [K + n, C]: position p0 - K + i
        acc = torch.zeros(n, C, dtype=torch.float32, device=proj.device)
        for j in range(taps):
            acc += w[:, j] * seq[j: j + n]
        out[b, :n] = F.silu(acc)
        conv_state[line] = seq[n: n + K]
    q = out[..., : G * D].reshape(B, T, G, D)
    k = out[..., G * D: 2 * G * D].reshape(B, T, G, D)
    v = out[..., 2 * G * D:].reshape(B, T, H, Dv)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + unit_eps) * qscale
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + unit_eps)
    return q.contiguous(), k.contiguous(), v.contiguous()


def delta_scan(qn: torch.Tensor, kn: torch.Tensor, vn: torch.Tensor, a_pre: torch.Tensor, a_offset: int,
               b_pre: torch.Tensor, b_offset: int, a_log: torch.Tensor, dt_bias: torch.Tensor, S: torch.Tensor,
               q_start: torch.Tensor, per_channel: bool, n_new: Optional[torch.Tensor] = None,
               seq_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``qn, kn [B, T, G, dim]``, ``vn [B, T, H, vdim]`` fp32 (``delta_prep``); ``a_pre [B * T, lda]`` fp32 holds the decay
    pre-activations at column ``a_offset + h`` (or ``a_offset + h * dim + i`` with ``per_channel``), ``b_pre [B * T, ldb]``
    fp32 the beta pre-activations at ``b_offset + h``; ``a_log [H]``, ``dt_bias [H]`` or ``[H * dim]`` fp32;
    ``S [lines, H, dim, vdim]`` fp32, updated in place for line ``seq_ids[b]`` (default ``b``).  Tokens ``t >= n_new[b]``
    are padding: they leave the state alone and come out as zeros.  On the GPU ``a_pre`` and ``b_pre`` are overwritten
    with the decay factors and beta.  Returns fp32 ``o [B, T, H, vdim]``."""
    B, T, G, D = qn.shape
    H, Dv = vn.shape[2], vn.shape[3]
    if qn.is_cuda and _lib.available(GROUP):
        assert qn.is_contiguous() and kn.is_contiguous() and vn.is_contiguous() and S.is_contiguous()
        assert a_pre.dtype == torch.float32 and b_pre.dtype == torch.float32 and a_pre.stride(1) == 1 and b_pre.stride(1) == 1
        out = torch.empty(B, T, H, Dv, dtype=torch.float32, device=qn.device)
        qs, nn_, sid = _i32(q_start), _i32(n_new), _i32(seq_ids)
        L = _lib.lib(GROUP)
        rc = L.nxd_delta_scan(_lib.ptr(qn), _lib.ptr(kn), _lib.ptr(vn), _lib.ptr(a_pre), _c.c_longlong(a_pre.stride(0)),
                              _c.c_int(a_offset), _lib.ptr(b_pre), _c.c_longlong(b_pre.stride(0)), _c.c_int(b_offset),
                              _lib.ptr(a_log), _lib.ptr(dt_bias), _lib.ptr(S), _lib.ptr(out), _lib.ptr(qs), _lib.ptr(nn_),
                              _lib.ptr(sid), _c.c_int(B), _c.c_int(T), _c.c_int(H), _c.c_int(G), _c.c_int(D), _c.c_int(Dv),
                              _c.c_int(int(per_channel)), _lib.stream_ptr())
        _lib.check(rc, "nxd_delta_scan", L)
        return out
    out = torch.zeros(B, T, H, Dv, dtype=torch.float32, device=qn.device)
    na = H * D if per_channel else H
    a = a_pre.reshape(B, T, -1)[..., a_offset: a_offset + na].float() + dt_bias.float()
    g = torch.exp(-torch.exp(a_log.float()).reshape(H, 1) * F.softplus(a).reshape(B, T, H, -1))   # [B, T, H, D or 1]
    beta = torch.sigmoid(b_pre.reshape(B, T, -1)[..., b_offset: b_offset + H].float())
    rep = H // G
    for b in range(B):
        n = T if n_new is None else min(int(n_new[b]), T)
        if n <= 0:
            continue
        line = b if seq_ids is None else int(seq_ids[b])
        Sb = torch.zeros_like(S[line]) if int(q_start[b]) == 0 else S[line].clone()        # [H, D, Dv]
        for t in range(n):
            k = kn[b, t].repeat_interleave(rep, dim=0)                                      # [H, D]
            q = qn[b, t].repeat_interleave(rep, dim=0)
            Sb = Sb * g[b, t].reshape(H, -1, 1)
            u = beta[b, t].reshape(H, 1) * (vn[b, t] - torch.einsum("hdv,hd->hv", Sb, k))
            Sb = Sb + k.unsqueeze(-1) * u.unsqueeze(1)
            out[b, t] = torch.einsum("hdv,hd->hv", Sb, q)
        S[line] = Sb
    return out
