"""Matrix-memory recurrent mixer (mLSTM) ops over a per-line fp32 state (``csrc/mlstm.cu``), and the gated head output
that follows it.

Per head, with log-space input / forget gates ``i_t`` / ``f_t`` and a running maximum ``m`` (``m_0 = 0``, zero state):

    m_t = max(f_t + m_{t-1}, i_t)
    S_t = exp(f_t + m_{t-1} - m_t) S_{t-1} + exp(i_t - m_t) k_t v_t^T
    n_t = exp(f_t + m_{t-1} - m_t) n_{t-1} + exp(i_t - m_t) k_t
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)

Gates, state and the division are fp32 whatever the activation dtype.  A row whose first position is 0 starts from the
zero state; any other row continues from the state its cache line holds, so a prompt may arrive in portions and a line
that is handed to a new request needs no clearing.  Every op has a PyTorch restatement for CPU.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

GROUP = "hybrid_serving"
DENOMINATOR_FLOOR = 1e-6


def _code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and _lib.available(GROUP)


def _i32(t):
    if t is None:
        return None
    return t if (t.dtype == torch.int32 and t.is_contiguous()) else t.to(torch.int32).contiguous()


def soft_cap(x: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(x / cap) if cap and cap > 0 else x


def mlstm_gates(h: torch.Tensor, w: torch.Tensor, bias: torch.Tensor, heads: int, cap: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``h [N, W]``, ``w [2 * heads, W]`` (input-gate rows, then forget-gate rows), ``bias [2 * heads]`` fp32 ->
    fp32 ``(i, f) [N, heads]``: ``i = cap tanh(x_i / cap)``, ``f = logsigmoid(cap tanh(x_f / cap))``.  The dot
    products accumulate in fp32 and are never rounded to the activation dtype."""
    N, W = h.shape
    if _use_kernel(h) and w.dtype == h.dtype:
        h2 = h if h.is_contiguous() else h.contiguous()
        gi = torch.empty(N, heads, dtype=torch.float32, device=h.device)
        gf = torch.empty(N, heads, dtype=torch.float32, device=h.device)
        L = _lib.lib(GROUP)
        rc = L.nxd_mlstm_gates(_c.c_int(_code(h.dtype)), _lib.ptr(h2), _lib.ptr(w), _lib.ptr(bias), _lib.ptr(gi),
                               _lib.ptr(gf), _c.c_longlong(N), _c.c_int(W), _c.c_int(heads), _c.c_float(cap),
                               _lib.stream_ptr())
        _lib.check(rc, "nxd_mlstm_gates", L)
        return gi, gf
    pre = h.float() @ w.float().t() + bias.float()
    return soft_cap(pre[:, :heads], cap), F.logsigmoid(soft_cap(pre[:, heads:], cap))


def mlstm_scan(proj: torch.Tensor, offsets: Tuple[int, int, int], gi: torch.Tensor, gf: torch.Tensor,
               state: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], q_start: torch.Tensor, heads: int, dim: int,
               vdim: int, qscale: float, n_new: Optional[torch.Tensor] = None,
               seq_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``proj [B, T, ld]`` holds the step's queries / keys / values head-major at column ``offsets = (q, k, v)``;
    ``gi / gf [B * T, heads]`` fp32; ``state = (S [lines, heads, dim, vdim], n [lines, heads, dim], m [lines, heads])``
    fp32, updated in place for line ``seq_ids[b]`` (default ``b``).  Tokens ``t >= n_new[b]`` are padding: they leave
    the state alone and come out as zeros.  Returns fp32 ``o [B, T, heads, vdim]``."""
    B, T, ld = proj.shape
    S, n, m = state
    if _use_kernel(proj):
        assert proj.is_contiguous() and S.is_contiguous() and n.is_contiguous() and m.is_contiguous()
        out = torch.empty(B, T, heads, vdim, dtype=torch.float32, device=proj.device)
        nxn = torch.empty(B, heads, dim, dtype=torch.float32, device=proj.device)
        nxm = torch.empty(B, heads, dtype=torch.float32, device=proj.device)
        qs, nn_, sid = _i32(q_start), _i32(n_new), _i32(seq_ids)      # converted copies stay alive across the launch
        L = _lib.lib(GROUP)
        rc = L.nxd_mlstm_scan(_c.c_int(_code(proj.dtype)), _lib.ptr(proj), _c.c_longlong(ld), _c.c_int(offsets[0]),
                              _c.c_int(offsets[1]), _c.c_int(offsets[2]), _lib.ptr(gi), _lib.ptr(gf), _lib.ptr(S),
                              _lib.ptr(n), _lib.ptr(m), _lib.ptr(nxn), _lib.ptr(nxm), _lib.ptr(out), _lib.ptr(qs),
                              _lib.ptr(nn_), _lib.ptr(sid), _c.c_int(B), _c.c_int(T), _c.c_int(heads),
                              _c.c_int(dim), _c.c_int(vdim), _c.c_float(qscale), _lib.stream_ptr())
        _lib.check(rc, "nxd_mlstm_scan", L)
        return out
    out = torch.zeros(B, T, heads, vdim, dtype=torch.float32, device=proj.device)
    q = proj[..., offsets[0]: offsets[0] + heads * dim].float().reshape(B, T, heads, dim) * qscale
    k = proj[..., offsets[1]: offsets[1] + heads * dim].float().reshape(B, T, heads, dim)
    v = proj[..., offsets[2]: offsets[2] + heads * vdim].float().reshape(B, T, heads, vdim)
    gi, gf = gi.reshape(B, T, heads), gf.reshape(B, T, heads)
    for b in range(B):
        cnt = T if n_new is None else min(int(n_new[b]), T)
        if cnt <= 0:
            continue
        line = b if seq_ids is None else int(seq_ids[b])
        if int(q_start[b]) == 0:
            Sb, nb, mb = torch.zeros_like(S[line]), torch.zeros_like(n[line]), torch.zeros_like(m[line])
        else:
            Sb, nb, mb = S[line].clone(), n[line].clone(), m[line].clone()
        for t in range(cnt):
            mn = torch.maximum(gf[b, t] + mb, gi[b, t])
            a, w = torch.exp(gf[b, t] + mb - mn), torch.exp(gi[b, t] - mn)
            Sb = a[:, None, None] * Sb + (w[:, None] * k[b, t])[:, :, None] * v[b, t][:, None, :]
            nb = a[:, None] * nb + w[:, None] * k[b, t]
            mb = mn
            den = torch.maximum((nb * q[b, t]).sum(-1).abs(), torch.exp(-mb)) + DENOMINATOR_FLOOR
            out[b, t] = torch.einsum("hdv,hd->hv", Sb, q[b, t]) / den[:, None]
        S[line], n[line], m[line] = Sb, nb, mb
    return out


def _chunk_states(u, ftot, mloc, s0, m0, want_m: bool):
    """The pass that is sequential over chunks (``csrc/mlstm.cu: mlstm_chunk_states_kernel``): ``u [BH, NC, E]`` becomes
    the state at every chunk's start; returns ``(state after the last chunk [BH, E], m at chunk starts, m after)``."""
    BH, NC, E = u.shape
    s_out = torch.empty(BH, E, dtype=torch.float32, device=u.device)
    m_start = torch.empty(BH, NC, dtype=torch.float32, device=u.device) if want_m else None
    m_out = torch.empty(BH, dtype=torch.float32, device=u.device) if want_m else None
    if u.is_cuda and _lib.available(GROUP):
        L = _lib.lib(GROUP)
        rc = L.nxd_mlstm_chunk_states(_lib.ptr(u), _lib.ptr(ftot), _lib.ptr(mloc), _lib.ptr(s0), _lib.ptr(m0),
                                      _lib.ptr(s_out), _lib.ptr(m_start), _lib.ptr(m_out), _c.c_longlong(BH), _c.c_int(NC),
                                      _c.c_longlong(E), _lib.stream_ptr())
        _lib.check(rc, "nxd_mlstm_chunk_states", L)
        return s_out, m_start, m_out
    s, m = s0.clone(), m0.clone()
    for c in range(NC):
        mn = torch.maximum(ftot[:, c] + m, mloc[:, c])
        a, b = torch.exp(ftot[:, c] + m - mn), torch.exp(mloc[:, c] - mn)
        uc = u[:, c].clone()
        u[:, c] = s
        if want_m:
            m_start[:, c] = m
        s = a[:, None] * s + b[:, None] * uc
        m = mn
    s_out.copy_(s)
    if want_m:
        m_out.copy_(m)
    return s_out, m_start, m_out


NO_INPUT = -1e30         # log input gate of a padding token: it adds nothing and (with log forget gate 0) decays nothing


def mlstm_chunkwise(proj: torch.Tensor, offsets: Tuple[int, int, int], gi: torch.Tensor, gf: torch.Tensor,
                    state: Tuple[torch.Tensor, torch.Tensor, torch.Tensor], q_start: torch.Tensor, heads: int, dim: int,
                    vdim: int, qscale: float, n_new: Optional[torch.Tensor] = None,
                    seq_ids: Optional[torch.Tensor] = None, chunk: int = 64) -> torch.Tensor:
    """``mlstm_scan`` for long steps, in chunk-wise form: same arguments, same result up to fp32 rounding.

    With ``F_t`` the running sum of the log forget gates inside a chunk and ``(S_c, n_c, m_c)`` the state at its start,
    ``m_t = F_t + max(m_c, max_{s<=t}(i_s - F_s))`` is exactly the running maximum of the token-by-token form, and

        S_t^T q_t = exp(F_t + m_c - m_t) S_c^T q_t + sum_{s<=t} exp(F_t - F_s + i_s - m_t) (k_s . q_t) v_s

    (``n_t . q_t`` likewise), so a chunk's outputs are four matrix products (q k^T, (q k^T * decay) v, q S_c, and
    (k * w)^T v for the state) and every exponent is <= 0.  Only the walk over chunk states is sequential (one small
    kernel).  Everything runs in fp32: the matrix products are fp32 library products, gates and state never leave fp32."""
    B, T, _ = proj.shape
    H, D, Dv, L = heads, dim, vdim, chunk
    dev, f32 = proj.device, torch.float32
    S, n, m = state
    NC = (T + L - 1) // L
    Tp = NC * L
    cnt = n_new.long() if n_new is not None else torch.full((B,), T, device=dev, dtype=torch.long)
    real = torch.arange(Tp, device=dev).reshape(1, Tp) < cnt.clamp(max=T).reshape(B, 1)            # [B, Tp]

    def heads_of(off, width):                                      # -> [B, H, NC, L, width] fp32, padding rows zero
        x = proj[..., off: off + H * width].to(f32).reshape(B, T, H, width)
        if Tp != T:
            x = torch.cat([x, x.new_zeros(B, Tp - T, H, width)], dim=1)
        x = x * real.reshape(B, Tp, 1, 1)
        return x.reshape(B, NC, L, H, width).permute(0, 3, 1, 2, 4)

    q, k, v = heads_of(offsets[0], D) * qscale, heads_of(offsets[1], D), heads_of(offsets[2], Dv)

    def gates_of(g, fill):                                         # [B*T, H] -> [B, H, NC, L]
        g = g.reshape(B, T, H)
        if Tp != T:
            g = torch.cat([g, g.new_zeros(B, Tp - T, H)], dim=1)
        g = torch.where(real.reshape(B, Tp, 1), g, torch.full_like(g, fill))
        return g.reshape(B, NC, L, H).permute(0, 3, 1, 2)

    fg, ig = gates_of(gf, 0.0), gates_of(gi, NO_INPUT)
    F = torch.cumsum(fg, dim=-1)                                   # inclusive, inside the chunk
    ftot = F[..., -1]                                              # [B, H, NC]
    g = ig - F
    gmax = g.max(dim=-1).values
    mloc = ftot + gmax
    # the chunk's own contribution to the state, relative to its local maximum
    w = torch.exp(g - gmax.unsqueeze(-1))                          # [B, H, NC, L], <= 1
    kw = k * w.unsqueeze(-1)
    u = torch.matmul(kw.transpose(-1, -2), v).reshape(B * H, NC, D * Dv)
    un = kw.sum(dim=-2).reshape(B * H, NC, D)
    # state before the step: zero for rows that start a sequence, else what the line holds
    lines = seq_ids.long() if seq_ids is not None else torch.arange(B, device=dev)
    cont = (q_start.reshape(B) != 0).to(f32)
    s0 = (S[lines] * cont.reshape(B, 1, 1, 1)).reshape(B * H, D * Dv)
    n0 = (n[lines] * cont.reshape(B, 1, 1)).reshape(B * H, D)
    m0 = (m[lines] * cont.reshape(B, 1)).reshape(B * H)
    ft2, ml2 = ftot.reshape(B * H, NC).contiguous(), mloc.reshape(B * H, NC).contiguous()
    s_end, m_start, m_end = _chunk_states(u, ft2, ml2, s0.contiguous(), m0.contiguous(), True)
    n_end, _, _ = _chunk_states(un, ft2, ml2, n0.contiguous(), m0.contiguous(), False)
    Sc, nc_, mc = u.reshape(B, H, NC, D, Dv), un.reshape(B, H, NC, D), m_start.reshape(B, H, NC)
    # outputs of every chunk
    m_t = F + torch.maximum(mc.unsqueeze(-1), torch.cummax(g, dim=-1).values)                      # [B, H, NC, L]
    causal = torch.ones(L, L, dtype=torch.bool, device=dev).tril()
    expo = (F - m_t).unsqueeze(-1) + g.unsqueeze(-2)                                               # [.., t, s]
    decay = torch.exp(expo.masked_fill(~causal, float("-inf")))
    P = torch.matmul(q, k.transpose(-1, -2)) * decay
    inter = torch.exp(F + mc.unsqueeze(-1) - m_t)                                                  # [B, H, NC, L]
    num = torch.matmul(P, v) + inter.unsqueeze(-1) * torch.matmul(q, Sc)
    nq = P.sum(dim=-1) + inter * (q * nc_.unsqueeze(-2)).sum(dim=-1)
    den = torch.maximum(nq.abs(), torch.exp(-m_t)) + DENOMINATOR_FLOOR
    out = (num / den.unsqueeze(-1)).permute(0, 2, 3, 1, 4).reshape(B, Tp, H, Dv)[:, :T]
    out = out * real[:, :T].reshape(B, T, 1, 1)
    # rows with no real token keep their state (blended by the row mask on the device: no host read)
    kf = (cnt > 0).to(f32)
    S[lines] = s_end.reshape(B, H, D, Dv) * kf.reshape(B, 1, 1, 1) + S[lines] * (1 - kf).reshape(B, 1, 1, 1)
    n[lines] = n_end.reshape(B, H, D) * kf.reshape(B, 1, 1) + n[lines] * (1 - kf).reshape(B, 1, 1)
    m[lines] = m_end.reshape(B, H) * kf.reshape(B, 1) + m[lines] * (1 - kf).reshape(B, 1)
    return out.contiguous()


def head_norm_gate(o: torch.Tensor, gate_src: torch.Tensor, gate_offset: int, heads: int, vdim: int,
                   weight: Optional[torch.Tensor], eps: float, normalize: bool, out_dtype: torch.dtype,
                   gate_act: str = "sigmoid") -> torch.Tensor:
    """``o [N, heads, vdim]`` -> ``[N, heads * vdim]`` in ``out_dtype``: every head divided by its root mean square
    (``normalize``; fp32, ``eps`` inside the root), times ``weight [heads * vdim]`` (optional), times
    ``sigmoid(gate)`` (or ``silu(gate)`` with ``gate_act="silu"``) where the gate pre-activations are columns
    ``gate_offset ...`` of ``gate_src [N, ld]`` (rows ``gate_src.stride(0)`` apart)."""
    N = o.shape[0]
    gate_src = gate_src.reshape(N, -1) if gate_src.is_contiguous() else gate_src
    ld = gate_src.stride(0) if gate_src.dim() == 2 else gate_src.shape[-1]
    if (_use_kernel(gate_src) and gate_src.dtype == out_dtype and gate_src.dim() == 2 and gate_src.stride(1) == 1
            and o.is_contiguous() and (o.dtype == torch.float32 or o.dtype == out_dtype)):
        out = torch.empty(N, heads * vdim, dtype=out_dtype, device=o.device)
        wf = weight.float().contiguous() if weight is not None else None
        L = _lib.lib(GROUP)
        rc = L.nxd_head_norm_gate(_c.c_int(_code(o.dtype)), _c.c_int(_code(out_dtype)), _lib.ptr(o), _lib.ptr(gate_src),
                                  _c.c_longlong(ld), _c.c_int(gate_offset), _lib.ptr(wf), _lib.ptr(out), _c.c_longlong(N),
                                  _c.c_int(heads), _c.c_int(vdim), _c.c_int(int(normalize)), _c.c_float(eps),
                                  _c.c_int(1 if gate_act == "silu" else 0), _lib.stream_ptr())
        _lib.check(rc, "nxd_head_norm_gate", L)
        return out
    of = o.float().reshape(N, heads, vdim)
    if normalize:
        of = of / torch.sqrt(of.pow(2).mean(-1, keepdim=True) + eps)
    of = of.reshape(N, heads * vdim)
    if weight is not None:
        of = of * weight.float()
    g = gate_src.reshape(N, -1)[:, gate_offset: gate_offset + heads * vdim].float()
    return (of * (F.silu(g) if gate_act == "silu" else torch.sigmoid(g))).to(out_dtype)
