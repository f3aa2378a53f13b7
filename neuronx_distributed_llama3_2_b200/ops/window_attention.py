"""Attention over the KV cache with a sliding window, kept first tokens and a linear distance bias
(``csrc/window_attention.cu``), next to the plain causal ops of ``ops/attention.py``.

    visible(i, j) = j <= i and (window is None or i - j < window or j < keep_first)
                    and (chunk is None or i // chunk == j // chunk)        chunk boundaries at absolute multiples of the size
    score(i, j)   = scale * <q_i, k_j> - slope_h * (i - j)
    p(i, j)       = exp(score(i, j)) / (sum over visible j' of exp(score(i, j')) [+ exp(sink_h)])

``sinks``: a learned per-head logit that is attached to no position and only takes probability mass.  The value rows may be
a column range of the key rows (``cache_v`` a view of ``cache_k``): the cache of a compressed key/value projection.

Head sizes are free (query/key size ``D`` and value size ``Dv`` may differ); activations and cache are bf16 or fp32, the
softmax and the unit-RMS normalisation of queries and keys run in fp32.  The prefill op reads keys and values from the
cache, so a step may start at any position of a sequence (``q_start``), and the same entry points serve a contiguous
cache ``[lines, G, S, D]`` and a paged one ``[pages, G, page, D]`` + block table.

Every op has a plain PyTorch restatement used on CPU (and as the oracle of the kernel tests).
"""
from __future__ import annotations

import ctypes as _c
from typing import Optional

import torch

from . import _lib

GROUP = "window_moe"


def _code(dtype: torch.dtype) -> int:
    return {torch.bfloat16: 0, torch.float32: 1}[dtype]


def _use_kernel(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and _lib.available(GROUP)


def _i32(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t if (t.dtype == torch.int32 and t.is_contiguous()) else t.to(torch.int32).contiguous()


def distance_slopes(n_heads: int, exponent: float = 8.0, device=None) -> torch.Tensor:
    """Geometric per-head slopes ``2 ** (-exponent * (h + 1) / n_heads)`` of the linear distance bias, fp32 ``[H]``."""
    h = torch.arange(1, n_heads + 1, dtype=torch.float64)
    return torch.pow(2.0, -exponent * h / n_heads).to(torch.float32).to(device)


def _cache_rows(cache: torch.Tensor, line: int, n: int, block_table, page_size: int) -> torch.Tensor:
    """Rows ``[0, n)`` of a cache line as ``[G, n, D]``."""
    if block_table is None:
        return cache[line, :, :n]
    pages = block_table[line, : (n + page_size - 1) // page_size].long()
    return cache[pages].permute(1, 0, 2, 3).reshape(cache.shape[1], -1, cache.shape[3])[:, :n]


def _cache_args(cache_k, cache_v, block_table, page_size, rows: bool = False):
    """Strides (in elements) of the cache tensors; with ``rows`` also the pitch between consecutive cache rows, which
    lets ``cache_v`` be a column range of ``cache_k``."""
    bt = _i32(block_table)
    assert cache_k.stride(3) == 1 and cache_v.stride(3) == 1
    k = (_c.c_longlong(cache_k.stride(0)), _c.c_longlong(cache_k.stride(1)))
    v = (_c.c_longlong(cache_v.stride(0)), _c.c_longlong(cache_v.stride(1)))
    if rows:
        k, v = k + (_c.c_longlong(cache_k.stride(2)),), v + (_c.c_longlong(cache_v.stride(2)),)
    else:
        assert cache_k.stride(2) == cache_k.shape[3] and cache_v.stride(2) == cache_v.shape[3]
    return k + v + (_lib.ptr(bt), _c.c_int(page_size if bt is not None else 0),
                    _c.c_int(bt.shape[1] if bt is not None else 0)), bt


def qk_norm_cache_write(qkv: torch.Tensor, cache_k: Optional[torch.Tensor], cache_v: Optional[torch.Tensor],
                        q_start: torch.Tensor, heads: int, kv_heads: int, dim: int, vdim: int, eps: float,
                        n_new: Optional[torch.Tensor] = None, seq_ids: Optional[torch.Tensor] = None,
                        normalize: bool = True, block_table: Optional[torch.Tensor] = None,
                        page_size: int = 0, writeback: bool = False, q_weight: Optional[torch.Tensor] = None,
                        k_weight: Optional[torch.Tensor] = None, rope: Optional[tuple] = None,
                        value_from_key: bool = False, value_heads: Optional[int] = None, rope_layout: str = "pairs",
                        whole_norm: bool = False) -> torch.Tensor:
    """``q_weight / k_weight [dim]``: weight of the per-head norm (after the division).  ``rope = (cos, sin)`` tables
    ``[positions, rot/2]`` (``ops.rope.build_interleaved_rope_cache``): queries and keys turn pairwise on their first
    ``rot`` dimensions, after the norm; pair ``i`` is the dimensions ``(2i, 2i + 1)`` (``rope_layout="pairs"``) or
    ``(i, i + rot/2)`` (``"halves"``).  ``value_from_key``: the projection has no value columns, the cached value is
    the raw key projection (taken ahead of the norm and the rotation).  ``whole_norm``: the root mean square is taken
    over ALL query heads of a row at once (and over all its key heads), and ``q_weight [heads * dim]`` /
    ``k_weight [kv_heads * dim]`` cover the whole projection.

    ``qkv [B, T, heads*dim (+ kv_heads*dim + kv_heads*vdim)]`` -> ``q [B, T, heads, dim]``; with a cache given the
    key and value heads of the real rows (``t < n_new[b]``) are written at position ``q_start[b] + t`` of cache line
    ``seq_ids[b]``.  ``normalize``: queries and keys are divided by their root mean square over ``dim`` (fp32, ``eps``
    inside the root) before they are written.  ``writeback``: the normalised keys of the real rows also replace the
    raw ones inside ``qkv`` (for a kernel that reads q / k / v as strided views of the projection output).
    ``value_heads``: the row holds that many value heads instead of ``kv_heads`` (value head ``g`` then serves the key
    heads ``g, g + value_heads, ...``: several attention maps over the same values).  ``qkv`` may be a column range of
    a wider projection output (rows ``stride(1)`` apart)."""
    B, T, n_out = qkv.shape
    has_kv = cache_k is not None
    gv = kv_heads if value_heads is None else int(value_heads)
    n_v = 0 if value_from_key else gv * vdim
    assert n_out == heads * dim + ((kv_heads * dim + n_v) if has_kv else 0), (n_out, heads, kv_heads, dim, vdim)
    assert not value_from_key or (vdim == dim and gv == kv_heads)
    if _use_kernel(qkv):
        rows_ok = qkv.stride(2) == 1 and (B == 1 or qkv.stride(0) == T * qkv.stride(1)) and qkv.stride(1) >= n_out
        assert rows_ok or not writeback
        qkv = qkv if rows_ok else qkv.contiguous()
        ld = qkv.stride(1)
        q = torch.empty(B, T, heads, dim, dtype=qkv.dtype, device=qkv.device)
        qs, nn_, sid = _i32(q_start), _i32(n_new), _i32(seq_ids)
        ck = cache_k if has_kv else q
        cv = cache_v if has_kv else q
        cargs, bt = _cache_args(ck, cv, block_table if has_kv else None, page_size)
        max_pos = (bt.shape[1] * page_size if bt is not None else ck.shape[2]) if has_kv else 0
        L = _lib.lib(GROUP)
        qw = q_weight.float().contiguous() if q_weight is not None else None
        kw = k_weight.float().contiguous() if k_weight is not None else None
        cos, sin = rope if rope is not None else (None, None)
        # scratch of the whole-projection statistics (1 / rms of all query heads, of all key heads, per row)
        stat = torch.empty(B * T, 2, dtype=torch.float32, device=qkv.device) if (whole_norm and normalize) else None
        rc = L.nxd_qk_prep_cache_write(_c.c_int(_code(qkv.dtype)), _lib.ptr(qkv), _c.c_longlong(ld), _lib.ptr(q),
                                       _lib.ptr(ck), _lib.ptr(cv), *cargs, _lib.ptr(qs), _lib.ptr(nn_), _lib.ptr(sid),
                                       _c.c_int(B), _c.c_int(T), _c.c_int(heads), _c.c_int(kv_heads), _c.c_int(dim),
                                       _c.c_int(vdim), _c.c_int(int(has_kv)), _c.c_int(int(normalize)), _c.c_float(eps),
                                       _c.c_int(max_pos), _c.c_int(int(writeback and has_kv)), _lib.ptr(qw), _lib.ptr(kw),
                                       _lib.ptr(cos), _lib.ptr(sin), _c.c_int(2 * cos.shape[1] if cos is not None else 0),
                                       _c.c_int(int(value_from_key)), _c.c_int(gv),
                                       _c.c_int(int(rope_layout == "halves")), _c.c_int(int(whole_norm)),
                                       _lib.ptr(stat), _lib.stream_ptr())
        _lib.check(rc, "nxd_qk_prep_cache_write", L)
        return q

    pos_bt = q_start.long().reshape(B, 1) + torch.arange(T, device=qkv.device).reshape(1, T)

    def unit(x, w):
        xf = x.float()
        if normalize and whole_norm:
            xf = xf / torch.sqrt(xf.pow(2).mean((-2, -1), keepdim=True) + eps)
        elif normalize:
            xf = xf / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        if w is not None:
            xf = xf * (w.float().reshape(xf.shape[-2:]) if whole_norm else w.float())
        if rope is not None:
            from .rope import rope_halves_ref, rope_interleaved_ref

            xf = (rope_halves_ref if rope_layout == "halves" else rope_interleaved_ref)(xf, pos_bt, rope[0], rope[1])
        return xf.to(x.dtype)

    q = unit(qkv[..., : heads * dim].reshape(B, T, heads, dim), q_weight)
    if has_kv:
        k_raw = qkv[..., heads * dim: (heads + kv_heads) * dim].reshape(B, T, kv_heads, dim)
        k = unit(k_raw, k_weight)
        v = k_raw if value_from_key else qkv[..., (heads + kv_heads) * dim:].reshape(B, T, gv, vdim)
        for b in range(B):
            n = T if n_new is None else int(n_new[b])
            line = b if seq_ids is None else int(seq_ids[b])
            p0 = int(q_start[b])
            if writeback:
                qkv[b, :n, heads * dim: (heads + kv_heads) * dim] = k[b, :n].reshape(n, kv_heads * dim)
            for t in range(n):
                pos = p0 + t
                if block_table is not None:
                    page, off = int(block_table[line, pos // page_size]), pos % page_size
                    cache_k[page, :, off] = k[b, t]
                    cache_v[page, :, off] = v[b, t]
                else:
                    cache_k[line, :, pos] = k[b, t]
                    cache_v[line, :, pos] = v[b, t]
    return q.contiguous()


def window_attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_pos: torch.Tensor, scale: float,
                         window: Optional[int], keep_first: int, slopes: Optional[torch.Tensor],
                         chunk: Optional[int] = None, sinks: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One sequence in fp32: ``q [Tq, H, D]`` at positions ``q_pos [Tq]`` over keys ``k [G, Tk, D]`` / ``v [Gv, Tk, Dv]``
    at positions ``0 .. Tk - 1``; with fewer value heads than key heads, key head ``g`` reads value head ``g % Gv``."""
    H, G = q.shape[1], k.shape[0]
    kf = k.float().repeat_interleave(H // G, dim=0)
    if v.shape[0] != G:
        v = v[torch.arange(G, device=v.device) % v.shape[0]]
    vf = v.float().repeat_interleave(H // G, dim=0)
    s = torch.einsum("qhd,hkd->hqk", q.float(), kf) * scale
    j = torch.arange(k.shape[1], device=q.device)
    dist = (q_pos.reshape(-1, 1) - j.reshape(1, -1))                      # [Tq, Tk]
    vis = dist >= 0
    if window is not None and window > 0:
        vis = vis & ((dist < window) | (j.reshape(1, -1) < keep_first))
    if chunk:
        vis = vis & (torch.div(q_pos.reshape(-1, 1), chunk, rounding_mode="floor")
                     == torch.div(j.reshape(1, -1), chunk, rounding_mode="floor"))
    if slopes is not None:
        s = s - slopes.float().reshape(H, 1, 1) * dist.float()
    s = s.masked_fill(~vis, float("-inf"))
    if sinks is not None:
        s = torch.cat([s, sinks.float().reshape(H, 1, 1).expand(H, s.shape[1], 1)], dim=-1)
    p = torch.softmax(s, dim=-1)
    if sinks is not None:
        p = p[..., :-1]
    p = torch.nan_to_num(p, nan=0.0)                                      # a row that sees nothing
    return torch.einsum("hqk,hkd->qhd", p, vf)


def window_attention_prefill(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, q_start: torch.Tensor,
                             scale: float, window: Optional[int] = None, keep_first: int = 0,
                             slopes: Optional[torch.Tensor] = None, n_new: Optional[torch.Tensor] = None,
                             seq_ids: Optional[torch.Tensor] = None, block_table: Optional[torch.Tensor] = None,
                             page_size: int = 0, impl: str = "auto", chunk: Optional[int] = None,
                             sinks: Optional[torch.Tensor] = None, value_heads: Optional[int] = None) -> torch.Tensor:
    """``impl``: ``auto`` | ``generic`` (fp32-math tile kernel, any sizes) | ``mma`` (bf16 tensor-core kernel, an error
    where it does not apply) -- for tests and measurements.

    ``q [B, T, H, D]``: new tokens of every row at positions ``q_start[b] + t`` (their keys / values already in the
    cache) -> ``[B, T, H, Dv]``.  Rows ``t >= n_new[b]`` are padding and come out as zeros."""
    B, T, H, D = q.shape
    G, Dv = cache_k.shape[1], cache_v.shape[3]
    w = int(window) if window else 0
    if _use_kernel(q):
        q = q if q.is_contiguous() else q.contiguous()
        out = torch.empty(B, T, H, Dv, dtype=q.dtype, device=q.device)
        qs, nn_, sid = _i32(q_start), _i32(n_new), _i32(seq_ids)
        cargs, bt = _cache_args(cache_k, cache_v, block_table, page_size, rows=True)
        sk = sinks.float().contiguous() if sinks is not None else None
        L = _lib.lib(GROUP)
        rc = L.nxd_masked_attn_prefill(_c.c_int(_code(q.dtype)), _lib.ptr(q), _lib.ptr(cache_k), _lib.ptr(cache_v),
                                       *cargs, _lib.ptr(out), _lib.ptr(qs), _lib.ptr(nn_), _lib.ptr(sid),
                                       _lib.ptr(slopes), _lib.ptr(sk), _c.c_int(B), _c.c_int(T), _c.c_int(H), _c.c_int(G),
                                       _c.c_int(D), _c.c_int(Dv), _c.c_float(scale), _c.c_int(w), _c.c_int(keep_first),
                                       _c.c_int(int(chunk) if chunk else 0),
                                       _c.c_int({"auto": 0, "generic": 1, "mma": 2}[impl]),
                                       _c.c_int(int(value_heads) if value_heads else 0), _lib.stream_ptr())
        _lib.check(rc, "nxd_masked_attn_prefill", L)
        return out
    out = torch.zeros(B, T, H, Dv, dtype=q.dtype, device=q.device)
    for b in range(B):
        n = T if n_new is None else int(n_new[b])
        if n == 0:
            continue
        line = b if seq_ids is None else int(seq_ids[b])
        p0 = int(q_start[b])
        kk = _cache_rows(cache_k, line, p0 + n, block_table, page_size)
        vv = _cache_rows(cache_v, line, p0 + n, block_table, page_size)
        pos = torch.arange(p0, p0 + n, device=q.device)
        out[b, :n] = window_attention_ref(q[b, :n], kk, vv, pos, scale, w, keep_first, slopes, chunk, sinks).to(q.dtype)
    return out


def window_attention_decode(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, positions: torch.Tensor,
                            scale: float, window: Optional[int] = None, keep_first: int = 0,
                            slopes: Optional[torch.Tensor] = None, seq_ids: Optional[torch.Tensor] = None,
                            block_table: Optional[torch.Tensor] = None, page_size: int = 0,
                            impl: str = "auto", chunk: Optional[int] = None,
                            sinks: Optional[torch.Tensor] = None, value_heads: Optional[int] = None) -> torch.Tensor:
    """One new token per row: ``q [B, H, D]`` at ``positions[b]`` -> ``[B, H, Dv]``; only the kept first rows and the
    window's rows of the cache line are read."""
    B, H, D = q.shape
    G, Dv = cache_k.shape[1], cache_v.shape[3]
    w = int(window) if window else 0
    if _use_kernel(q):
        q = q if q.is_contiguous() else q.contiguous()
        out = torch.empty(B, H, Dv, dtype=q.dtype, device=q.device)
        pos, sid = _i32(positions), _i32(seq_ids)
        cargs, bt = _cache_args(cache_k, cache_v, block_table, page_size, rows=True)
        sk = sinks.float().contiguous() if sinks is not None else None
        if (impl == "auto" and q.dtype == torch.bfloat16 and G == 1 and not w and not chunk and slopes is None
                and cache_v.data_ptr() == cache_k.data_ptr() and cache_v.stride(2) == cache_k.stride(2)
                and cache_v.stride(0) == cache_k.stride(0)):
            # latent rows (one key/value head, values = the first columns of the key rows): the kernel that streams the
            # rows once per 16 query heads, with the context split over CTAs when the batch alone does not fill the GPU
            from . import latent_attention as la

            if la.latent_decode(q, cache_k, Dv, out, pos, sid, sk, scale, bt, page_size):
                return out
        L = _lib.lib(GROUP)
        rc = L.nxd_masked_attn_decode(_c.c_int(_code(q.dtype)), _lib.ptr(q), _lib.ptr(cache_k), _lib.ptr(cache_v), *cargs,
                                      _lib.ptr(out), _lib.ptr(pos), _lib.ptr(sid), _lib.ptr(slopes), _lib.ptr(sk),
                                      _c.c_int(B), _c.c_int(H), _c.c_int(G), _c.c_int(D), _c.c_int(Dv), _c.c_float(scale),
                                      _c.c_int(w), _c.c_int(keep_first), _c.c_int(int(chunk) if chunk else 0),
                                      _c.c_int({"auto": 0, "generic": 1, "mma": 2}[impl]),
                                      _c.c_int(int(value_heads) if value_heads else 0), _lib.stream_ptr())
        _lib.check(rc, "nxd_masked_attn_decode", L)
        return out
    out = torch.empty(B, H, Dv, dtype=q.dtype, device=q.device)
    for b in range(B):
        line = b if seq_ids is None else int(seq_ids[b])
        p = int(positions[b])
        kk = _cache_rows(cache_k, line, p + 1, block_table, page_size)
        vv = _cache_rows(cache_v, line, p + 1, block_table, page_size)
        out[b] = window_attention_ref(q[b:b + 1], kk, vv, torch.tensor([p], device=q.device), scale, w, keep_first,
                                      slopes, chunk, sinks)[0].to(q.dtype)
    return out


def diff_attention_combine(maps: torch.Tensor, lq1: torch.Tensor, lk1: torch.Tensor, lq2: torch.Tensor,
                           lk2: torch.Tensor, diff: float, eps: float) -> torch.Tensor:
    """Differential attention: ``maps [N, 2 * H, Dv]`` holds two softmax attention maps over the same values (heads
    ``0 .. H-1``: map 1, ``H .. 2H-1``: map 2) -> ``[N, H * Dv]``: ``o = a1 - lambda a2`` with
    ``lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff`` (one number, fp32), every head divided by its root mean square
    (``eps`` inside the root), times ``1 - diff``."""
    N, H2, Dv = maps.shape
    H = H2 // 2
    if _use_kernel(maps):
        maps = maps if maps.is_contiguous() else maps.contiguous()
        out = torch.empty(N, H * Dv, dtype=maps.dtype, device=maps.device)
        L = _lib.lib(GROUP)
        rc = L.nxd_diff_attn_combine(_c.c_int(_code(maps.dtype)), _lib.ptr(maps), _lib.ptr(out), _lib.ptr(lq1),
                                     _lib.ptr(lk1), _lib.ptr(lq2), _lib.ptr(lk2), _c.c_longlong(N), _c.c_int(H),
                                     _c.c_int(Dv), _c.c_int(lq1.numel()), _c.c_float(diff), _c.c_float(eps),
                                     _lib.stream_ptr())
        _lib.check(rc, "nxd_diff_attn_combine", L)
        return out
    lam = torch.exp((lq1.float() * lk1.float()).sum()) - torch.exp((lq2.float() * lk2.float()).sum()) + diff
    o = maps[:, :H].float() - lam * maps[:, H:].float()
    o = o / torch.sqrt(o.pow(2).mean(-1, keepdim=True) + eps) * (1.0 - diff)
    return o.reshape(N, H * Dv).to(maps.dtype)


def tc_prefill_applies(q: torch.Tensor, dim: int, vdim: int, n_out: int) -> bool:
    """The tcgen05 windowed prefill kernel serves bf16 on the GPU, equal key and value size of 64 or 128, and projection
    rows whose pitch keeps every head 16-byte aligned."""
    from . import backend

    return (q.is_cuda and q.dtype == torch.bfloat16 and dim == vdim and dim in (64, 128) and n_out % 8 == 0
            and backend.attn_backend() == "nxd" and _lib.available())


def window_attention_tc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int] = None,
                        keep_first: int = 0, slopes: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Prefill from position 0 on the tcgen05 flash-attention kernel (``csrc/flash_attn_tc.cu``, windowed
    instantiation): ``q [B, H, T, D]``, ``k / v [B, G, T, D]`` as (strided) views with unit stride on ``D`` ->
    ``[B, H, T, D]`` stored as ``[B, T, H, D]``.  All rows are taken as ``T`` tokens long (right padding only ever
    sits behind the real tokens of a causal row)."""
    from .flash_attn import _fix, _strides

    q, k, v = _fix(q), _fix(k), _fix(v)
    B, H, T, D = q.shape
    G = k.shape[1]
    o = torch.empty(B, T, H, D, dtype=q.dtype, device=q.device).permute(0, 2, 1, 3)
    L = _lib.lib()
    rc = L.nxd_flash_attn_fwd_tc_window(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _strides(q, k, v, o),
                                        _c.c_int(B), _c.c_int(H), _c.c_int(G), _c.c_int(T), _c.c_int(T), _c.c_int(D),
                                        _c.c_float(scale), _c.c_int(int(window) if window else 0), _c.c_int(keep_first),
                                        _lib.ptr(slopes), _lib.stream_ptr())
    _lib.check(rc, "nxd_flash_attn_fwd_tc_window")
    return o
