"""Gogalix: a decoder-only hybrid family whose layers are listed in the configuration, one by one.

  * the residual stream ``x`` is fp32.  A layer is PARALLEL: one RMS norm (its weight is a single number) feeds the
    mixer and the feed-forward alike, and both results are added at once, each times a per-coordinate layer scale and
    a sigmoid gate computed from the same normed input:
    ``h = norm1(x);  x += ls1 * sigmoid(rg1 h + b1) * mixer(h) + ls2 * sigmoid(rg2 h + b2) * ff(h)``;
  * ``delta`` / ``channel_delta``: the gated delta rule (``ops/delta_rule.py``) behind short convolutions, with one
    decay per head, or one per head and key channel computed through a low-rank pair; per-head unit-RMS output norm with a
    weight shared by the heads, and an output gate (``silu`` of a full projection, or ``sigmoid`` of a low-rank one);
  * ``attention``: differential attention -- two softmax maps per head over the same values, combined as
    ``a1 - lambda a2`` (Ye et al., "Differential Transformer"), no rotation, a configured score scale and a sliding
    window; a layer with ``kv_from: j`` has no key / value projections and reads layer ``j``'s cache;
  * feed-forward: dense ``down(silu(gate h + b) * (up h + b)) + b``, or a mixture of bias-free experts of the same shape
    whose router (with a bias) picks the ``top`` largest logits and weights them by the softmax over the chosen logits;
  * the embedding is multiplied by ``embedding.scale``.

Parameter modules only; the forward over the KV cache and the recurrent state lives in
``inference/hybrid.py: GogalixInferenceModel``.  Everything that multiplies the normed input of a layer (mixer
projections, output-gate projection, the two residual gates, the dense gate / up) is ONE fused matrix ``in_proj``;
``columns`` says where each part starts.  Tensor parallelism is not wired for this family.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..modules.moe.sparse import SparseMoE
from ..parallel.layers import ColumnParallelLinear, ParallelEmbedding, RowParallelLinear

UNIT_NORM_EPS = 1e-6            # inside the root of the unit-vector normalisation of delta-rule queries and keys
COLUMN_ALIGN = 8                # parts of the fused projection start on 16-byte boundaries (bf16)


@dataclass
class DeltaMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int                          # taps of the short convolution
    per_channel: bool = False          # one decay per head and key channel (through a low-rank pair)
    rank: int = 0                      # inner size of the low-rank pairs (read from the checkpoint's shapes)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], per_channel: bool) -> "DeltaMixerConfig":
        c = cls(heads=int(d["heads"]), kv_heads=int(d.get("kv_heads", d["heads"])), dim=int(d["dim"]),
                vdim=int(d["vdim"]), conv=int(d["conv"]), per_channel=per_channel, rank=int(d.get("rank", 0)))
        if c.heads % c.kv_heads:
            raise ValueError(f"delta mixer: {c.heads} heads over {c.kv_heads} query/key heads")
        if c.conv < 1:
            raise ValueError(f"delta mixer: convolution of {c.conv} taps")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "conv": self.conv}
        if self.per_channel and self.rank:
            d["rank"] = self.rank
        return d

    @property
    def channels(self) -> int:
        return 2 * self.kv_heads * self.dim + self.heads * self.vdim


@dataclass
class DiffAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float                        # the constant of lambda, and (1 - diff) after the head norm
    window: Optional[int]              # mask.size; None = plain causal
    kv_from: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "DiffAttentionConfig":
        mask = d.get("mask") or {}
        c = cls(heads=int(d["heads"]), kv_heads=int(d.get("kv_heads", d["heads"])), dim=int(d["dim"]),
                vdim=int(d.get("vdim", d["dim"])), scale=float(d["scale"]), diff=float(d["diff"]),
                window=int(mask["size"]) if mask.get("size") else None,
                kv_from=int(d["kv_from"]) if d.get("kv_from") is not None else None)
        if c.heads % c.kv_heads:
            raise ValueError(f"attention: {c.heads} query heads over {c.kv_heads} key/value heads")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale, "diff": self.diff}
        if self.window:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass
class FeedForwardConfig:
    kind: str                          # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FeedForwardConfig":
        kind = d.get("kind", "dense")
        if kind == "dense":
            return cls(kind="dense", ff=int(d["ff"]))
        if kind == "moe":
            c = cls(kind="moe", ff=int(d["expert"]["ff"]), experts=int(d["router"]["experts"]), top=int(d["router"]["top"]))
            if not 1 <= c.top <= c.experts:
                raise ValueError(f"mixture of experts: top {c.top} of {c.experts}")
            return c
        raise ValueError(f"unknown feed-forward kind {kind!r}")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


MIXER_CONFIGS: Dict[str, Callable[[Dict[str, Any]], Any]] = {
    "delta": lambda d: DeltaMixerConfig.from_dict(d, per_channel=False),
    "channel_delta": lambda d: DeltaMixerConfig.from_dict(d, per_channel=True),
    "attention": DiffAttentionConfig.from_dict,
}


@dataclass
class GogalixLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[FeedForwardConfig]


@dataclass
class GogalixConfig:
    vocab_size: int
    hidden_size: int
    embedding_scale: float = 1.0
    layers: List[GogalixLayerConfig] = field(default_factory=list)
    rms_norm_eps: float = 1e-6
    torch_dtype: torch.dtype = torch.bfloat16
    model_type: str = "gogalix"
    # read by shared inference code
    sequence_parallel_enabled: bool = False
    activation_checkpointing: bool = False
    initializer_range: float = 0.02

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @classmethod
    def from_dict(cls, d: Dict[str, Any], torch_dtype: torch.dtype = torch.bfloat16) -> "GogalixConfig":
        layers: List[GogalixLayerConfig] = []
        for i, L in enumerate(d["layers"]):
            if L["type"] not in MIXER_CONFIGS:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r} (known: {sorted(MIXER_CONFIGS)})")
            m = MIXER_CONFIGS[L["type"]](L["mixer"])
            if L["type"] == "attention" and m.kv_from is not None:
                j = m.kv_from
                src = layers[j].mixer if 0 <= j < i and layers[j].type == "attention" else None
                if src is None or src.kv_from is not None or (src.kv_heads, src.dim, src.vdim) != (m.kv_heads, m.dim, m.vdim):
                    raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with projections of its "
                                     f"own and the same key/value shapes")
            layers.append(GogalixLayerConfig(L["type"], m, FeedForwardConfig.from_dict(L["mlp"]) if L.get("mlp") else None))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), layers=layers,
                   rms_norm_eps=float(d["norm"]["eps"]), torch_dtype=torch_dtype)

    @classmethod
    def from_json(cls, path: str, torch_dtype: torch.dtype = torch.bfloat16) -> "GogalixConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f), torch_dtype)

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": "Gogalix", "vocab": self.vocab_size, "width": self.hidden_size,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.rms_norm_eps},
                "layers": [{"type": L.type, "mixer": L.mixer.to_dict(), "mlp": L.mlp.to_dict() if L.mlp else None}
                           for L in self.layers]}

    def with_checkpoint_shapes(self, sd: Dict[str, torch.Tensor]) -> "GogalixConfig":
        """Sizes that only the checkpoint tells: the inner size of the low-rank pairs of ``channel_delta`` layers."""
        for i, L in enumerate(self.layers):
            if L.type == "channel_delta":
                L.mixer.rank = int(sd[f"l{i}.mix.a1"].shape[0])
        return self


def _init(std: float) -> Callable:
    return lambda w: nn.init.normal_(w, mean=0.0, std=std)


def _up8(n: int) -> int:
    return (n + COLUMN_ALIGN - 1) // COLUMN_ALIGN * COLUMN_ALIGN


def in_proj_columns(config: GogalixConfig, layer: GogalixLayerConfig) -> Tuple[Dict[str, Tuple[int, int]], int]:
    """``{part: (first column, columns)}`` of a layer's fused input projection, and its total width.  Every part starts
    on a multiple of ``COLUMN_ALIGN`` columns (rows of zeros fill the gaps)."""
    W, m = config.hidden_size, layer.mixer
    parts: List[Tuple[str, int]] = []
    if layer.type == "attention":                   # queries (map-major), then keys (map-major) and values of its own
        own = 2 * m.kv_heads * m.dim + m.kv_heads * m.vdim if m.kv_from is None else 0
        parts.append(("qkv", 2 * m.heads * m.dim + own))
    else:
        parts.append(("qkv", m.channels))                                             # q | k | v, convolved together
        if m.per_channel:
            parts += [("a1", m.rank), ("g1", m.rank)]
        else:
            parts.append(("g", m.heads * m.vdim))
    parts.append(("rg1", W))
    if layer.mlp is not None:
        parts.append(("rg2", W))
        if layer.mlp.kind == "dense":
            parts += [("gate", layer.mlp.ff), ("up", layer.mlp.ff)]
    cols, at = {}, 0
    for name, n in parts:
        cols[name] = (at, n)
        at = _up8(at + n)
    return cols, at


class DeltaMixer(nn.Module):
    """Convolution weights ``[channels, taps]`` (q | k | v), the fp32-output projection of the recurrence's gates
    (``gate_proj``: beta rows, then -- with one decay per head -- the decay rows, padded to a multiple of 8 rows), decay
    constants, the output norm weight tiled over the heads, the second halves of the low-rank pairs, output projection."""

    def __init__(self, config: GogalixConfig, m: DeltaMixerConfig, device=None):
        super().__init__()
        self.cfg = m
        dt, std, W = config.torch_dtype, config.initializer_range, config.hidden_size
        f32 = dict(dtype=torch.float32, device=device)
        self.conv_weight = nn.Parameter(torch.empty(m.channels, m.conv, **f32).normal_(0.0, 0.3))
        n_gate = m.heads if m.per_channel else 2 * m.heads
        self.gate_proj = nn.Parameter(torch.zeros(_up8(n_gate), W, dtype=dt, device=device))
        self.a_log = nn.Parameter(torch.zeros(m.heads, **f32))
        self.dt_bias = nn.Parameter(torch.zeros(m.heads * m.dim if m.per_channel else m.heads, **f32))
        self.out_norm = nn.Parameter(torch.ones(m.heads * m.vdim, **f32))
        if m.per_channel:
            rk = _up8(m.rank)           # inner size padded with zero columns: the GEMM kernels want multiples of 8
            self.a2 = nn.Parameter(torch.zeros(m.heads * m.dim, rk, dtype=dt, device=device))
            self.g2 = nn.Parameter(torch.zeros(m.heads * m.vdim, rk, dtype=dt, device=device))
        self.o_proj = RowParallelLinear(m.heads * m.vdim, W, bias=False, input_is_parallel=True, dtype=dt, device=device,
                                        init_method=_init(std))


class DiffAttentionMixer(nn.Module):
    """The four vectors of lambda and the output projection (the query / key / value rows are part of the layer's fused
    input projection, queries and keys MAP-MAJOR: all heads of map 1, then all heads of map 2)."""

    def __init__(self, config: GogalixConfig, m: DiffAttentionConfig, device=None):
        super().__init__()
        self.cfg = m
        f32 = dict(dtype=torch.float32, device=device)
        self.lq1, self.lk1 = nn.Parameter(torch.zeros(m.dim, **f32)), nn.Parameter(torch.zeros(m.dim, **f32))
        self.lq2, self.lk2 = nn.Parameter(torch.zeros(m.dim, **f32)), nn.Parameter(torch.zeros(m.dim, **f32))
        self.o_proj = RowParallelLinear(m.heads * m.vdim, config.hidden_size, bias=False, input_is_parallel=True,
                                        dtype=config.torch_dtype, device=device, init_method=_init(config.initializer_range))


MIXERS: Dict[str, Callable[..., nn.Module]] = {"delta": DeltaMixer, "channel_delta": DeltaMixer,
                                               "attention": DiffAttentionMixer}


class DenseGatedMlp(nn.Module):
    """Biases of the gate and up rows (the rows themselves are part of the layer's fused input projection) and the biased
    down projection."""

    def __init__(self, config: GogalixConfig, m: FeedForwardConfig, device=None):
        super().__init__()
        f32 = dict(dtype=torch.float32, device=device)
        self.gate_bias = nn.Parameter(torch.zeros(m.ff, **f32))
        self.up_bias = nn.Parameter(torch.zeros(m.ff, **f32))
        self.down_proj = RowParallelLinear(m.ff, config.hidden_size, bias=False, input_is_parallel=True,
                                           dtype=config.torch_dtype, device=device, init_method=_init(config.initializer_range))
        self.down_bias = nn.Parameter(torch.zeros(config.hidden_size, **f32))


class GogalixDecoderLayer(nn.Module):
    def __init__(self, config: GogalixConfig, layer: GogalixLayerConfig, device=None):
        super().__init__()
        W = config.hidden_size
        f32 = dict(dtype=torch.float32, device=device)
        self.type = layer.type
        self.columns, n_out = in_proj_columns(config, layer)
        self.norm1 = nn.Parameter(torch.ones(1, **f32))                 # the norm's weight: one number
        self.in_proj = ColumnParallelLinear(W, n_out, bias=False, gather_output=False, dtype=config.torch_dtype,
                                            device=device, init_method=_init(config.initializer_range))
        self.mixer = MIXERS[layer.type](config, layer.mixer, device=device)
        self.ls1 = nn.Parameter(torch.ones(W, **f32))
        self.rg1_bias = nn.Parameter(torch.zeros(W, **f32))
        self.mlp = None
        self.mlp_kind = layer.mlp.kind if layer.mlp is not None else None
        if layer.mlp is not None:
            self.ls2 = nn.Parameter(torch.ones(W, **f32))
            self.rg2_bias = nn.Parameter(torch.zeros(W, **f32))
            if layer.mlp.kind == "dense":
                self.mlp = DenseGatedMlp(config, layer.mlp, device=device)
            else:
                self.mlp = SparseMoE(W, layer.mlp.experts, layer.mlp.top, layer.mlp.ff, None, dtype=config.torch_dtype,
                                     device=device, router_bias=True, renormalize=True)


class GogalixForCausalLM(nn.Module):
    def __init__(self, config: GogalixConfig, device=None):
        super().__init__()
        self.config = config
        dt = config.torch_dtype
        self.embed_tokens = ParallelEmbedding(config.vocab_size, config.hidden_size, dtype=dt, device=device,
                                              init_method=_init(config.initializer_range))
        self.layers = nn.ModuleList([GogalixDecoderLayer(config, L, device=device) for L in config.layers])
        self.norm = nn.Parameter(torch.ones(1, dtype=torch.float32, device=device))
        self.lm_head = ColumnParallelLinear(config.hidden_size, config.vocab_size, bias=False, gather_output=False,
                                            dtype=dt, device=device, init_method=_init(config.initializer_range))


def _map_major(w: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
    """Rows ``[heads, 2 maps, dim]`` -> ``[2 maps, heads, dim]``: the two attention maps of a head become two separate
    heads, all heads of map 1 first."""
    return w.reshape(heads, 2, dim, -1).transpose(0, 1).reshape(2 * heads * dim, -1)


def _head_major(w: torch.Tensor, heads: int, dim: int) -> torch.Tensor:
    return w.reshape(2, heads, dim, -1).transpose(0, 1).reshape(2 * heads * dim, -1)


def _pad_rows(w: torch.Tensor, rows: int) -> torch.Tensor:
    return w if w.shape[0] == rows else torch.cat([w, w.new_zeros(rows - w.shape[0], w.shape[1])], dim=0)


def convert_gogalix_state_dict(sd: Dict[str, torch.Tensor], config: GogalixConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names (``embed``, ``l<i>.norm1``, ``l<i>.mix.<name>``, ``l<i>.mlp.<name>``, ``l<i>.ls1 / rg1 / rg1.b``
    ..., ``final.norm``, ``head``; linear weights ``[out, in]``) -> this module's state dict."""
    config.with_checkpoint_shapes(sd)
    W = config.hidden_size
    out: Dict[str, torch.Tensor] = {"embed_tokens.weight": sd["embed"], "lm_head.weight": sd["head"],
                                    "norm": sd["final.norm"].float().reshape(1)}
    for i, L in enumerate(config.layers):
        src, dst, m = f"l{i}.", f"layers.{i}.", L.mixer
        mix = lambda n: sd[src + "mix." + n]                                          # noqa: E731
        cols, n_out = in_proj_columns(config, L)
        parts: Dict[str, torch.Tensor] = {"rg1": sd[src + "rg1"]}
        out[dst + "norm1"] = sd[src + "norm1"].float().reshape(1)
        out[dst + "ls1"], out[dst + "rg1_bias"] = sd[src + "ls1"].float(), sd[src + "rg1.b"].float()
        if L.type == "attention":
            rows = [_map_major(mix("q"), m.heads, m.dim)]
            if m.kv_from is None:
                rows += [_map_major(mix("k"), m.kv_heads, m.dim), mix("v")]
            parts["qkv"] = torch.cat(rows, dim=0)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[dst + "mixer." + n] = mix(n).float()
        else:
            parts["qkv"] = torch.cat([mix("q"), mix("k"), mix("v")], dim=0)
            out[dst + "mixer.conv_weight"] = torch.cat([mix("q.conv"), mix("k.conv"), mix("v.conv")], dim=0).float()
            out[dst + "mixer.a_log"] = mix("A_log").float()
            out[dst + "mixer.dt_bias"] = mix("dt_bias").float()
            out[dst + "mixer.out_norm"] = mix("norm").float().repeat(m.heads)
            if m.per_channel:
                parts["a1"], parts["g1"] = mix("a1"), mix("g1")
                gate_rows = mix("b")
                rk = _up8(m.rank)
                out[dst + "mixer.a2"] = _pad_rows(mix("a2").t(), rk).t()
                out[dst + "mixer.g2"] = _pad_rows(mix("g2").t(), rk).t()
            else:
                parts["g"] = mix("g")
                gate_rows = torch.cat([mix("b"), mix("a")], dim=0)
            out[dst + "mixer.gate_proj"] = _pad_rows(gate_rows, _up8(gate_rows.shape[0]))
        out[dst + "mixer.o_proj.weight"] = mix("o")
        if L.mlp is not None:
            parts["rg2"] = sd[src + "rg2"]
            out[dst + "ls2"], out[dst + "rg2_bias"] = sd[src + "ls2"].float(), sd[src + "rg2.b"].float()
            if L.mlp.kind == "dense":
                parts["gate"], parts["up"] = sd[src + "mlp.gate"], sd[src + "mlp.up"]
                out[dst + "mlp.gate_bias"], out[dst + "mlp.up_bias"] = sd[src + "mlp.gate.b"].float(), sd[src + "mlp.up.b"].float()
                out[dst + "mlp.down_proj.weight"], out[dst + "mlp.down_bias"] = sd[src + "mlp.down"], sd[src + "mlp.down.b"].float()
            else:
                E = L.mlp.experts
                out[dst + "mlp.router.linear_router.weight"] = sd[src + "mlp.router"].float()
                out[dst + "mlp.router.logit_bias"] = sd[src + "mlp.router.b"].float()
                out[dst + "mlp.router.correction"] = torch.zeros(E)
                out[dst + "mlp.experts.gate_up_proj.weight"] = torch.stack(
                    [torch.cat([sd[f"{src}mlp.e{e}.gate"].t(), sd[f"{src}mlp.e{e}.up"].t()], dim=1) for e in range(E)])
                out[dst + "mlp.experts.down_proj.weight"] = torch.stack([sd[f"{src}mlp.e{e}.down"].t() for e in range(E)])
        fused = parts["rg1"].new_zeros(n_out, W)
        for name, (at, n) in cols.items():
            assert parts[name].shape == (n, W), (i, name, parts[name].shape, n)
            fused[at: at + n] = parts[name]
        out[dst + "in_proj.weight"] = fused
    return {k: v.contiguous() for k, v in out.items()}


def export_gogalix_state_dict(model: GogalixForCausalLM) -> Dict[str, torch.Tensor]:
    """The inverse of ``convert_gogalix_state_dict``: this module's parameters under the checkpoint names."""
    cfg, sd = model.config, model.state_dict()
    out: Dict[str, torch.Tensor] = {"embed": sd["embed_tokens.weight"], "head": sd["lm_head.weight"],
                                    "final.norm": sd["norm"].reshape(())}
    for i, L in enumerate(cfg.layers):
        src, dst, m = f"layers.{i}.", f"l{i}.", L.mixer
        cols, _ = in_proj_columns(cfg, L)
        fused = sd[src + "in_proj.weight"]
        part = lambda n: fused[cols[n][0]: cols[n][0] + cols[n][1]]                    # noqa: E731
        out[dst + "norm1"] = sd[src + "norm1"].reshape(())
        out[dst + "ls1"], out[dst + "rg1"], out[dst + "rg1.b"] = sd[src + "ls1"], part("rg1"), sd[src + "rg1_bias"]
        if L.type == "attention":
            nq, nk = 2 * m.heads * m.dim, 2 * m.kv_heads * m.dim
            out[dst + "mix.q"] = _head_major(part("qkv")[:nq], m.heads, m.dim)
            if m.kv_from is None:
                out[dst + "mix.k"] = _head_major(part("qkv")[nq: nq + nk], m.kv_heads, m.dim)
                out[dst + "mix.v"] = part("qkv")[nq + nk:]
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[dst + "mix." + n] = sd[src + "mixer." + n]
        else:
            a, c = m.kv_heads * m.dim, m.heads * m.vdim
            qkv, cw, gp = part("qkv"), sd[src + "mixer.conv_weight"], sd[src + "mixer.gate_proj"]
            out[dst + "mix.q"], out[dst + "mix.k"], out[dst + "mix.v"] = qkv[:a], qkv[a:2 * a], qkv[2 * a:]
            out[dst + "mix.q.conv"], out[dst + "mix.k.conv"], out[dst + "mix.v.conv"] = cw[:a], cw[a:2 * a], cw[2 * a:]
            out[dst + "mix.A_log"], out[dst + "mix.dt_bias"] = sd[src + "mixer.a_log"], sd[src + "mixer.dt_bias"]
            out[dst + "mix.norm"] = sd[src + "mixer.out_norm"][: m.vdim]
            out[dst + "mix.b"] = gp[: m.heads]
            if m.per_channel:
                out[dst + "mix.a1"], out[dst + "mix.g1"] = part("a1"), part("g1")
                out[dst + "mix.a2"], out[dst + "mix.g2"] = sd[src + "mixer.a2"][:, : m.rank], sd[src + "mixer.g2"][:, : m.rank]
            else:
                out[dst + "mix.a"], out[dst + "mix.g"] = gp[m.heads: 2 * m.heads], part("g")
        out[dst + "mix.o"] = sd[src + "mixer.o_proj.weight"]
        if L.mlp is not None:
            out[dst + "ls2"], out[dst + "rg2"], out[dst + "rg2.b"] = sd[src + "ls2"], part("rg2"), sd[src + "rg2_bias"]
            if L.mlp.kind == "dense":
                out[dst + "mlp.gate"], out[dst + "mlp.up"] = part("gate"), part("up")
                out[dst + "mlp.gate.b"], out[dst + "mlp.up.b"] = sd[src + "mlp.gate_bias"], sd[src + "mlp.up_bias"]
                out[dst + "mlp.down"], out[dst + "mlp.down.b"] = sd[src + "mlp.down_proj.weight"], sd[src + "mlp.down_bias"]
            else:
                F = L.mlp.ff
                gu, dn = sd[src + "mlp.experts.gate_up_proj.weight"], sd[src + "mlp.experts.down_proj.weight"]
                out[dst + "mlp.router"], out[dst + "mlp.router.b"] = sd[src + "mlp.router.linear_router.weight"], sd[src + "mlp.router.logit_bias"]
                for e in range(L.mlp.experts):
                    out[f"{dst}mlp.e{e}.gate"], out[f"{dst}mlp.e{e}.up"] = gu[e, :, :F].t(), gu[e, :, F:].t()
                    out[f"{dst}mlp.e{e}.down"] = dn[e].t()
    return {k: v.detach().clone().contiguous() for k, v in out.items()}


def tiny_gogalix(torch_dtype: torch.dtype = torch.float32, **kw) -> GogalixConfig:
    """A small configuration for tests and smoke runs: one layer of every mixer kind, grouped heads, a window of 9, a
    layer that reads another layer's keys and values, a dense and a sparse feed-forward and a layer without one."""
    att = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "diff": 0.4, "mask": {"size": 9}}
    d = {"architecture": "Gogalix", "vocab": 112, "width": 40, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
         "layers": [{"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3},
                     "mlp": {"kind": "dense", "ff": 56}},
                    {"type": "attention", "mixer": att,
                     "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}}},
                    {"type": "channel_delta", "mixer": {"heads": 2, "kv_heads": 2, "dim": 12, "vdim": 8, "conv": 4, "rank": 6},
                     "mlp": None},
                    {"type": "attention", "mixer": dict(att, kv_from=1, mask={"size": 5}), "mlp": {"kind": "dense", "ff": 32}}]}
    d.update(kw)
    return GogalixConfig.from_dict(d, torch_dtype=torch_dtype)
