"""Rotary position embedding, incl. Llama-3 frequency scaling.

Reference: HF ``apply_rotary_pos_emb`` used at
``examples/training/llama/modeling_llama_nxd.py:398-399``; Llama-3 scaling
``examples/inference/llama3/neuron_modeling_llama.py:234-298``.
"""
from __future__ import annotations

import ctypes as _c
import math
from typing import Optional, Tuple

import torch

from . import _lib


def llama3_scale_inv_freq(inv_freq: torch.Tensor, factor: float = 32.0, low_freq_factor: float = 1.0,
                          high_freq_factor: float = 4.0, original_max_position: int = 8192) -> torch.Tensor:
    """Llama-3.x "llama3" rope scaling: long wavelengths are slowed by ``factor``, short ones
    kept, the band between interpolated smoothly."""
    low_wavelen = original_max_position / low_freq_factor
    high_wavelen = original_max_position / high_freq_factor
    wavelen = 2 * math.pi / inv_freq
    scaled = torch.where(wavelen > low_wavelen, inv_freq / factor, inv_freq)
    smooth = (original_max_position / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    smoothed = (1 - smooth) * inv_freq / factor + smooth * inv_freq
    mid = (wavelen <= low_wavelen) & (wavelen >= high_wavelen)
    return torch.where(mid, smoothed, scaled)


def build_rope_cache(max_pos: int, head_dim: int, theta: float = 500000.0, rope_scaling: Optional[dict] = None,
                     device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos``/``sin`` tables of shape ``[max_pos, head_dim/2]``."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    if rope_scaling and rope_scaling.get("rope_type", rope_scaling.get("type")) == "llama3":
        inv_freq = llama3_scale_inv_freq(
            inv_freq, rope_scaling.get("factor", 32.0), rope_scaling.get("low_freq_factor", 1.0),
            rope_scaling.get("high_freq_factor", 4.0), rope_scaling.get("original_max_position_embeddings", 8192))
    t = torch.arange(max_pos, dtype=torch.float32, device=device)
    freqs = torch.outer(t, inv_freq)
    return freqs.cos().contiguous(), freqs.sin().contiguous()


def wavelength_scaled_frequencies(freq: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """The Llama-3.1 slowdown of long waves (``llama3_scale_inv_freq`` above, in the dtype of ``freq``): with wavelength
    ``l = 2 pi / f``, ``f`` stays where ``l < original / high``, becomes ``f / factor`` where ``l > original / low``, and
    in between ``(1 - s) f / factor + s f`` with ``s = (original / l - low) / (high - low)``."""
    wave = 2.0 * math.pi / freq
    s = (original / wave - low) / (high - low)
    mid = (1.0 - s) * freq / factor + s * freq
    return torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, mid))


def build_interleaved_rope_cache(max_pos: int, dims: int, base: float, device=None,
                                 scaling: Optional[Tuple[float, float, float, float]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 ``cos`` / ``sin`` tables ``[max_pos, dims/2]`` of the angles ``p * base ** (-2 i / dims)``, evaluated in
    float64 (a position of a few thousand times a frequency loses digits of the angle in fp32).  ``scaling = (factor, low,
    high, original)``: the frequencies first go through ``wavelength_scaled_frequencies``."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims)
    if scaling is not None:
        freq = wavelength_scaled_frequencies(freq, *[float(x) for x in scaling])
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float64), freq)
    return ang.cos().float().contiguous().to(device), ang.sin().float().contiguous().to(device)


def rope_interleaved_ref(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x [..., heads, D]`` with ``positions [...]``: the pairs ``(2i, 2i + 1)`` of the first ``2 * cos.shape[1]``
    dimensions turn by the angle of (position, i): ``(u, v) -> (u cos - v sin, v cos + u sin)``; the rest pass."""
    rot = 2 * cos.shape[1]
    c = cos[positions.long()].unsqueeze(-2).to(x.dtype)
    s = sin[positions.long()].unsqueeze(-2).to(x.dtype)
    u, v = x[..., 0:rot:2], x[..., 1:rot:2]
    out = x.clone()
    out[..., 0:rot:2] = u * c - v * s
    out[..., 1:rot:2] = v * c + u * s
    return out


def rope_halves_ref(x: torch.Tensor, positions: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """As ``rope_interleaved_ref`` with the pairs ``(i, i + rot/2)`` ("rotate half" layout) of the first ``rot =
    2 * cos.shape[1]`` dimensions."""
    half = cos.shape[1]
    c = cos[positions.long()].unsqueeze(-2).to(x.dtype)
    s = sin[positions.long()].unsqueeze(-2).to(x.dtype)
    u, v = x[..., :half], x[..., half: 2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], dim=-1)


def _positions(T: int, pos_div: int, pos_mod: int, positions, device):
    if positions is not None:
        return positions.reshape(-1).long()
    return (torch.arange(T, device=device) // pos_div) % pos_mod


def rope_ref(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int, pos_div: int, pos_mod: int,
             positions=None, inverse: bool = False) -> torch.Tensor:
    """x: [T, heads, D]; rotate the first ``n_rot_heads`` heads (rotate-half convention)."""
    T, Hh, D = x.shape
    pos = _positions(T, pos_div, pos_mod, positions, x.device)
    c = cos[pos].unsqueeze(1).float()
    s = sin[pos].unsqueeze(1).float()
    if inverse:
        s = -s
    xr = x[:, :n_rot_heads].float()
    x1, x2 = xr[..., : D // 2], xr[..., D // 2:]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)
    return torch.cat([out, x[:, n_rot_heads:]], dim=1)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, n_rot_heads, pos_div, pos_mod, positions):
        ctx.args = (n_rot_heads, pos_div, pos_mod)
        ctx.save_for_backward(cos, sin, positions if positions is not None else torch.empty(0))
        ctx.has_pos = positions is not None
        out = x.contiguous().clone()
        _launch(out, cos, sin, n_rot_heads, pos_div, pos_mod, positions, False)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin, positions = ctx.saved_tensors
        n_rot_heads, pos_div, pos_mod = ctx.args
        dx = dy.contiguous().clone()
        _launch(dx, cos, sin, n_rot_heads, pos_div, pos_mod, positions if ctx.has_pos else None, True)
        return dx, None, None, None, None, None, None


def _launch(x, cos, sin, n_rot_heads, pos_div, pos_mod, positions, inverse):
    T, Hh, D = x.shape
    pos_t = None
    if positions is not None:
        pos_t = positions.reshape(-1).to(torch.int32).contiguous()
    rc = _lib.lib().nxd_rope_inplace(_lib.ptr(x), _lib.ptr(cos), _lib.ptr(sin), _lib.ptr(pos_t), _c.c_longlong(T),
                                     _c.c_int(Hh), _c.c_int(n_rot_heads), _c.c_int(D), _c.c_int(pos_div),
                                     _c.c_int(pos_mod), _c.c_int(1 if inverse else 0), _lib.stream_ptr())
    _lib.check(rc, "nxd_rope_inplace")


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, n_rot_heads: int, pos_div: int = 1,
               pos_mod: int = 1 << 30, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rotate heads ``[0, n_rot_heads)`` of ``x [T, heads, D]``.  Token ``t`` sits at position
    ``positions[t]`` or ``(t // pos_div) % pos_mod`` ([S,B] layout: div=B, mod=S; [B,S]: div=1, mod=S)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 16 == 0 and _lib.available():
        return _RopeFn.apply(x, cos, sin, n_rot_heads, pos_div, pos_mod, positions)
    return rope_ref(x, cos, sin, n_rot_heads, pos_div, pos_mod, positions)


def rope_inplace_(x: torch.Tensor, cos, sin, n_rot_heads: int, pos_div: int = 1, pos_mod: int = 1 << 30,
                  positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Inference variant: rotate in place (no autograd)."""
    if x.is_cuda and x.dtype == torch.bfloat16 and _lib.available():
        assert x.is_contiguous()
        _launch(x, cos, sin, n_rot_heads, pos_div, pos_mod, positions, False)
        return x
    x.copy_(rope_ref(x, cos, sin, n_rot_heads, pos_div, pos_mod, positions))
    return x
