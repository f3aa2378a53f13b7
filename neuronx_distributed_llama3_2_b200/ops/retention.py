"""Retention: linear attention with a fixed decay per head and no softmax or denominator (``csrc/retention.cu``), on a
per-line fp32 state of the cache / state manager.

    S_t = decay_h S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t           S: [dim, vdim] per head

Queries and keys are rotated inside the kernel (``rope = (cos, sin)`` tables ``[positions, rot/2]``, pair ``i`` =
dimensions ``(i, i + rot/2)`` with ``rope_layout="halves"`` or ``(2i, 2i + 1)`` with ``"pairs"``); the keys are multiplied
by ``kscale`` after the rotation.  Rotation, products, decay and state are fp32 whatever the activation dtype.

``retention_scan`` walks the step's tokens one by one (token generation, short steps); ``retention_chunkwise`` is the same
step in chunks of 64 tokens (matrix-shaped work inside a chunk, one sequential pass over the chunk states).  Both have
a plain PyTorch restatement used on CPU.
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional, Tuple

import torch

from . import _lib

GROUP = "retention_serving"
CHUNK = 64
_SMEM_LIMIT = 220 * 1024


def _code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and _lib.available(GROUP)


def _i32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t if (t.dtype == torch.int32 and t.is_contiguous()) else t.to(torch.int32).contiguous()


def chunkwise_applies(dim: int, vdim: int) -> bool:
    """The chunk-wise kernels keep a chunk's q, k, scores and a tile of at most 128 value columns (and that tile of a
    head's state) in shared memory."""
    vt = min(128, (vdim + 3) // 4 * 4)
    local = (2 * CHUNK * (dim + 1) + CHUNK * (CHUNK + 1) + CHUNK * vt) * 4
    cross = (dim * vt + CHUNK * dim) * 4
    return max(local, cross) <= _SMEM_LIMIT


def _rotate_ref(x: torch.Tensor, pos: torch.Tensor, rope, layout: str) -> torch.Tensor:
    if rope is None:
        return x
    from .rope import rope_halves_ref, rope_interleaved_ref

    return (rope_halves_ref if layout == "halves" else rope_interleaved_ref)(x, pos, rope[0], rope[1])


def retention_ref(proj: torch.Tensor, offsets: Tuple[int, int, int], decay: torch.Tensor, state: torch.Tensor,
                  q_start: torch.Tensor, heads: int, dim: int, vdim: int, kscale: float, rope, rope_layout: str,
                  n_new: Optional[torch.Tensor], seq_ids: Optional[torch.Tensor]) -> torch.Tensor:
    B, T, _ = proj.shape
    out = torch.zeros(B, T, heads, vdim, dtype=torch.float32, device=proj.device)
    pos = q_start.long().reshape(B, 1) + torch.arange(T, device=proj.device).reshape(1, T)
    q = _rotate_ref(proj[..., offsets[0]: offsets[0] + heads * dim].float().reshape(B, T, heads, dim), pos, rope, rope_layout)
    k = _rotate_ref(proj[..., offsets[1]: offsets[1] + heads * dim].float().reshape(B, T, heads, dim), pos, rope,
                    rope_layout) * kscale
    v = proj[..., offsets[2]: offsets[2] + heads * vdim].float().reshape(B, T, heads, vdim)
    a = decay.float().reshape(heads, 1, 1)
    for b in range(B):
        cnt = T if n_new is None else min(int(n_new[b]), T)
        if cnt <= 0:
            continue
        line = b if seq_ids is None else int(seq_ids[b])
        S = torch.zeros_like(state[line]) if int(q_start[b]) == 0 else state[line].clone()
        for t in range(cnt):
            S = a * S + k[b, t].unsqueeze(-1) * v[b, t].unsqueeze(-2)
            out[b, t] = torch.einsum("hdv,hd->hv", S, q[b, t])
        state[line] = S
    return out


def _launch(chunkwise: bool, proj, offsets, decay, state, q_start, heads, dim, vdim, kscale, rope, rope_layout, n_new,
            seq_ids) -> torch.Tensor:
    B, T, ld = proj.shape
    assert proj.is_contiguous() and state.is_contiguous() and state.dtype == torch.float32
    assert decay.dtype == torch.float32 and decay.numel() == heads
    out = torch.empty(B, T, heads, vdim, dtype=torch.float32, device=proj.device)
    qs, nn_, sid = _i32(q_start), _i32(n_new), _i32(seq_ids)          # converted copies stay alive across the launch
    cos, sin = rope if rope is not None else (None, None)
    rot = 2 * cos.shape[1] if cos is not None else 0
    tail = (_c.c_int(B), _c.c_int(T), _c.c_int(heads), _c.c_int(dim), _c.c_int(vdim), _c.c_float(kscale), _lib.ptr(cos),
            _lib.ptr(sin), _c.c_int(rot), _c.c_int(int(rope_layout == "halves")),
            _c.c_int(cos.shape[0] if cos is not None else 0), _lib.stream_ptr())
    head = (_c.c_int(_code(proj.dtype)), _lib.ptr(proj), _c.c_longlong(ld), _c.c_int(offsets[0]), _c.c_int(offsets[1]),
            _c.c_int(offsets[2]), _lib.ptr(decay), _lib.ptr(state), _lib.ptr(out))
    L = _lib.lib(GROUP)
    if chunkwise:
        nc = (T + CHUNK - 1) // CHUNK
        u = torch.empty(B, heads, nc, dim, vdim, dtype=torch.float32, device=proj.device)
        qrot = torch.empty(B * T, heads, dim, dtype=torch.float32, device=proj.device)
        rc = L.nxd_retention_chunkwise(*head, _lib.ptr(u), _lib.ptr(qrot), _lib.ptr(qs), _lib.ptr(nn_), _lib.ptr(sid), *tail)
        _lib.check(rc, "nxd_retention_chunkwise", L)
    else:
        rc = L.nxd_retention_scan(*head, _lib.ptr(qs), _lib.ptr(nn_), _lib.ptr(sid), *tail)
        _lib.check(rc, "nxd_retention_scan", L)
    return out


def retention_scan(proj: torch.Tensor, offsets: Tuple[int, int, int], decay: torch.Tensor, state: torch.Tensor,
                   q_start: torch.Tensor, heads: int, dim: int, vdim: int, kscale: float = 1.0,
                   rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, rope_layout: str = "halves",
                   n_new: Optional[torch.Tensor] = None, seq_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``proj [B, T, ld]`` holds the step's queries / keys / values head-major at column ``offsets = (q, k, v)``;
    ``decay [heads]`` fp32; ``state [lines, heads, dim, vdim]`` fp32, updated in place for line ``seq_ids[b]`` (default
    ``b``); a row with ``q_start[b] == 0`` starts from the zero state.  Tokens ``t >= n_new[b]`` are padding: they leave
    the state alone and come out as zeros.  Returns fp32 ``o [B, T, heads, vdim]``."""
    if _use_kernel(proj):
        return _launch(False, proj, offsets, decay, state, q_start, heads, dim, vdim, kscale, rope, rope_layout, n_new,
                       seq_ids)
    return retention_ref(proj, offsets, decay, state, q_start, heads, dim, vdim, kscale, rope, rope_layout, n_new, seq_ids)


def retention_chunkwise(proj: torch.Tensor, offsets: Tuple[int, int, int], decay: torch.Tensor, state: torch.Tensor,
                        q_start: torch.Tensor, heads: int, dim: int, vdim: int, kscale: float = 1.0,
                        rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, rope_layout: str = "halves",
                        n_new: Optional[torch.Tensor] = None, seq_ids: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``retention_scan`` for long steps, in chunk-wise form: same arguments, same result up to fp32 rounding.  With
    ``S_c`` the state at a chunk's start and ``t`` counted inside the chunk,

        o_t = decay^(t+1) S_c^T q_t + sum_{s <= t} decay^(t-s) (q_t . k_s) v_s,    S_(c+1) = decay^L S_c + sum_s decay^(L-1-s) k_s v_s^T
    """
    if _use_kernel(proj) and chunkwise_applies(dim, vdim):
        return _launch(True, proj, offsets, decay, state, q_start, heads, dim, vdim, kscale, rope, rope_layout, n_new,
                       seq_ids)
    return retention_scan(proj, offsets, decay, state, q_start, heads, dim, vdim, kscale, rope, rope_layout, n_new, seq_ids)
