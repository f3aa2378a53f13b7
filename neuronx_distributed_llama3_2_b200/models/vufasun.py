"""Vufasun: a decoder-only hybrid family whose layers are listed in the configuration, one by one.

  * the residual stream is ``streams`` parallel fp32 streams per token (hyper-connections, ``ops/hyper_connection.py``):
    a sublayer reads the RMS norm of a learned weighted sum of the streams, and its output is written into every stream
    with a weight of its own, next to a learned ``streams x streams`` mixing of the streams.  All streams start as the
    embedding; the model's final norm reads their plain sum.  One stream with unit weights is the pre-norm residual;
  * ``attention``: softmax attention of grouped heads over the KV cache, partial "rotate half" rotation, a configured score
    scale, and a learned per-head sink logit in the softmax denominator;
  * ``parallel``: two mixers side by side on the same normed input, each output RMS-normed over the width with a weight
    of its own, the result is half their sum.  Left: softmax attention whose queries and keys are RMS-normed over the
    WHOLE projection (all heads at once) before the rotation, whose frequencies may be slowed at long wavelengths.
    Right: retention (``ops/retention.py``) -- rotated queries and keys, keys scaled by ``dim ** -0.5``, a fixed decay
    per head, per-head unit RMS, an output gate ``silu(W_g h)``;
  * feed-forward: dense ``down(gelu_tanh(gate h) * (up h))``, or a mixture of ``silu`` experts whose router scores are
    sigmoids, not renormalised, and multiply the chosen experts' INPUT, plus an always-on shared expert;
  * ``loop``: a range of layers runs several times in a row with the same weights; every pass has cache and state of its
    own (``layer_runs()`` is the order, one cache index per run);
  * the output head is the embedding table.

Parameter modules only; the forward over the KV cache and the recurrent state lives in
``inference/hybrid.py: VufasunInferenceModel``.  Everything that multiplies the mixer's normed input is ONE fused matrix
``in_proj`` (``columns`` says where each part starts).  Tensor parallelism is not wired for this family.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from ..modules.moe.sparse import SparseMoE
from ..ops.linear import gemm_nt
from ..parallel.layers import ColumnParallelLinear, ParallelEmbedding, RowParallelLinear

COLUMN_ALIGN = 8                # parts of the fused projection start on 16-byte boundaries (bf16)


@dataclass
class RotaryConfig:
    dims: int
    base: float
    scaling: Optional[Tuple[float, float, float, float]] = None      # (factor, low, high, original)

    @classmethod
    def from_dict(cls, d: Optional[Dict[str, Any]]) -> Optional["RotaryConfig"]:
        if not d or not d.get("dims"):
            return None
        sc = d.get("scaling")
        scaling = (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])) if sc else None
        c = cls(dims=int(d["dims"]), base=float(d["base"]), scaling=scaling)
        if c.dims % 2:
            raise ValueError(f"rotation over an odd number of dimensions ({c.dims})")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"dims": self.dims, "base": self.base}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return d


@dataclass
class SoftmaxAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotaryConfig]
    sink: bool = False                 # a learned per-head logit in the softmax denominator
    whole_norm: bool = False           # RMS norm of q and of k over the whole projection, ahead of the rotation

    @classmethod
    def from_dict(cls, d: Dict[str, Any], sink: bool, whole_norm: bool) -> "SoftmaxAttentionConfig":
        c = cls(heads=int(d["heads"]), kv_heads=int(d.get("kv_heads", d["heads"])), dim=int(d["dim"]),
                vdim=int(d.get("vdim", d["dim"])), scale=float(d["scale"]), rot=RotaryConfig.from_dict(d.get("rot")),
                sink=sink, whole_norm=whole_norm)
        if c.heads % c.kv_heads:
            raise ValueError(f"attention: {c.heads} query heads over {c.kv_heads} key/value heads")
        if c.rot is not None and c.rot.dims > c.dim:
            raise ValueError(f"attention: rotation over {c.rot.dims} of {c.dim} dimensions")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                             "scale": self.scale}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d

    @property
    def columns(self) -> int:
        return self.heads * self.dim + self.kv_heads * (self.dim + self.vdim)


@dataclass
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: List[float]
    rot: Optional[RotaryConfig]

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "RetentionConfig":
        c = cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d.get("vdim", d["dim"])),
                decay=[float(x) for x in d["decay"]], rot=RotaryConfig.from_dict(d.get("rot")))
        if len(c.decay) != c.heads:
            raise ValueError(f"retention: {len(c.decay)} decays for {c.heads} heads")
        if c.rot is not None and c.rot.dims > c.dim:
            raise ValueError(f"retention: rotation over {c.rot.dims} of {c.dim} dimensions")
        return c

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d

    @property
    def columns(self) -> int:                       # q | k | v | g
        return 2 * self.heads * self.dim + 2 * self.heads * self.vdim


@dataclass
class ParallelMixerConfig:
    left: SoftmaxAttentionConfig
    right: RetentionConfig

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ParallelMixerConfig":
        return cls(left=SoftmaxAttentionConfig.from_dict(d["left"], sink=False, whole_norm=True),
                   right=RetentionConfig.from_dict(d["right"]))

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass
class FeedForwardConfig:
    kind: str                          # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0
    shared_ff: int = 0

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "FeedForwardConfig":
        kind = d.get("kind", "dense")
        if kind == "dense":
            return cls(kind="dense", ff=int(d["ff"]))
        if kind == "moe":
            c = cls(kind="moe", ff=int(d["expert"]["ff"]), experts=int(d["router"]["experts"]), top=int(d["router"]["top"]),
                    shared_ff=int((d.get("shared") or {}).get("ff", 0)))
            if not 1 <= c.top <= c.experts:
                raise ValueError(f"mixture of experts: top {c.top} of {c.experts}")
            return c
        raise ValueError(f"unknown feed-forward kind {kind!r}")

    def to_dict(self) -> Dict[str, Any]:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d: Dict[str, Any] = {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


MIXER_CONFIGS: Dict[str, Callable[[Dict[str, Any]], Any]] = {
    "attention": lambda d: SoftmaxAttentionConfig.from_dict(d, sink=True, whole_norm=False),
    "parallel": ParallelMixerConfig.from_dict,
}


@dataclass
class VufasunLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[FeedForwardConfig]


@dataclass
class VufasunConfig:
    vocab_size: int
    hidden_size: int
    streams: int = 1
    layers: List[VufasunLayerConfig] = field(default_factory=list)
    loop: Optional[Tuple[int, int, int]] = None          # (start, stop, times): layers start .. stop-1 run `times` times
    rms_norm_eps: float = 1e-6
    torch_dtype: torch.dtype = torch.bfloat16
    model_type: str = "vufasun"
    # read by shared inference code
    sequence_parallel_enabled: bool = False
    activation_checkpointing: bool = False
    initializer_range: float = 0.02

    @property
    def num_hidden_layers(self) -> int:
        """Layer RUNS: what the cache / state manager holds an entry for."""
        return len(self.layer_runs())

    def layer_runs(self) -> List[int]:
        """The layer index of every run, in order: the looped range ``times`` times in a row, then the rest."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    @classmethod
    def from_dict(cls, d: Dict[str, Any], torch_dtype: torch.dtype = torch.bfloat16) -> "VufasunConfig":
        layers: List[VufasunLayerConfig] = []
        for i, L in enumerate(d["layers"]):
            if L["type"] not in MIXER_CONFIGS:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r} (known: {sorted(MIXER_CONFIGS)})")
            layers.append(VufasunLayerConfig(L["type"], MIXER_CONFIGS[L["type"]](L["mixer"]),
                                             FeedForwardConfig.from_dict(L["mlp"]) if L.get("mlp") else None))
        loop = None
        lp = d.get("loop")
        if lp and int(lp.get("times", 1)) != 1 and int(lp["stop"]) > int(lp["start"]):
            loop = (int(lp["start"]), int(lp["stop"]), int(lp["times"]))
            if not (0 <= loop[0] < loop[1] <= len(layers)) or loop[2] < 1:
                raise ValueError(f"loop {loop} over {len(layers)} layers")
        streams = int(d.get("streams") or 1)
        if streams < 1:
            raise ValueError(f"{streams} streams")
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), streams=streams, layers=layers, loop=loop,
                   rms_norm_eps=float(d["norm"]["eps"]), torch_dtype=torch_dtype)

    def with_checkpoint_shapes(self, sd: Dict[str, torch.Tensor]) -> "VufasunConfig":
        """What only the checkpoint tells: an attention mixer has a sink term exactly when its ``sink`` tensor exists, and
        whole-projection query / key norms exactly when their weights do."""
        for i, L in enumerate(self.layers):
            prefix = f"l{i}.mix." + ("" if L.type == "attention" else "left.")
            a = L.mixer if L.type == "attention" else L.mixer.left
            a.sink = prefix + "sink" in sd
            a.whole_norm = prefix + "q.norm" in sd
        return self

    @classmethod
    def from_json(cls, path: str, torch_dtype: torch.dtype = torch.bfloat16) -> "VufasunConfig":
        if os.path.isdir(path):
            path = os.path.join(path, "config.json")
        with open(path) as f:
            return cls.from_dict(json.load(f), torch_dtype)

    def to_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": "Vufasun", "vocab": self.vocab_size, "width": self.hidden_size,
                             "streams": self.streams, "norm": {"eps": self.rms_norm_eps},
                             "layers": [{"type": L.type, "mixer": L.mixer.to_dict(),
                                         "mlp": L.mlp.to_dict() if L.mlp else None} for L in self.layers]}
        if self.loop is not None:
            d["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        return d


def _init(std: float) -> Callable:
    return lambda w: nn.init.normal_(w, mean=0.0, std=std)


def _up8(n: int) -> int:
    return (n + COLUMN_ALIGN - 1) // COLUMN_ALIGN * COLUMN_ALIGN


def in_proj_columns(layer: VufasunLayerConfig) -> Tuple[Dict[str, Tuple[int, int]], int]:
    """``{part: (first column, columns)}`` of a layer's fused mixer projection, and its total width.  ``attention``: one
    part ``qkv``; ``parallel``: ``left`` (q | k | v) and ``right`` (q | k | v | g).  Every part starts on a multiple of
    ``COLUMN_ALIGN`` columns (rows of zeros fill the gaps)."""
    if layer.type == "attention":
        parts = [("qkv", layer.mixer.columns)]
    else:
        parts = [("left", layer.mixer.left.columns), ("right", layer.mixer.right.columns)]
    cols, at = {}, 0
    for name, n in parts:
        cols[name] = (at, n)
        at = _up8(at + n)
    return cols, at


def _linear_out(config: VufasunConfig, n_in: int, device) -> RowParallelLinear:
    return RowParallelLinear(n_in, config.hidden_size, bias=False, input_is_parallel=True, dtype=config.torch_dtype,
                             device=device, init_method=_init(config.initializer_range))


class SoftmaxAttentionMixer(nn.Module):
    """Output projection, the optional sink logits ``[heads]`` and the optional whole-projection norm weights (the query /
    key / value rows are part of the layer's fused input projection)."""

    def __init__(self, config: VufasunConfig, m: SoftmaxAttentionConfig, device=None):
        super().__init__()
        self.cfg = m
        f32 = dict(dtype=torch.float32, device=device)
        self.sink = nn.Parameter(torch.zeros(m.heads, **f32)) if m.sink else None
        self.q_norm = nn.Parameter(torch.ones(m.heads * m.dim, **f32)) if m.whole_norm else None
        self.k_norm = nn.Parameter(torch.ones(m.kv_heads * m.dim, **f32)) if m.whole_norm else None
        self.o_proj = _linear_out(config, m.heads * m.vdim, device)


class RetentionMixer(nn.Module):
    """Output projection and the per-head decays (constants of the configuration, kept as an fp32 buffer)."""

    def __init__(self, config: VufasunConfig, m: RetentionConfig, device=None):
        super().__init__()
        self.cfg = m
        self.register_buffer("decay", torch.tensor(m.decay, dtype=torch.float32, device=device), persistent=False)
        self.o_proj = _linear_out(config, m.heads * m.vdim, device)


class ParallelMixer(nn.Module):
    def __init__(self, config: VufasunConfig, m: ParallelMixerConfig, device=None):
        super().__init__()
        self.cfg = m
        f32 = dict(dtype=torch.float32, device=device)
        self.left = SoftmaxAttentionMixer(config, m.left, device=device)
        self.right = RetentionMixer(config, m.right, device=device)
        self.left_out = nn.Parameter(torch.ones(config.hidden_size, **f32))
        self.right_out = nn.Parameter(torch.ones(config.hidden_size, **f32))


MIXERS: Dict[str, Callable[..., nn.Module]] = {"attention": SoftmaxAttentionMixer, "parallel": ParallelMixer}


class DenseGatedMlp(nn.Module):
    """``down(gelu_tanh(gate h) * (up h))``; gate | up rows fused."""

    def __init__(self, config: VufasunConfig, m: FeedForwardConfig, device=None):
        super().__init__()
        self.ff = m.ff
        self.ff_pad = _up8(m.ff)              # the up rows start on a 16-byte boundary of the fused output
        self.gate_up_proj = ColumnParallelLinear(config.hidden_size, 2 * self.ff_pad, bias=False, gather_output=False,
                                                 dtype=config.torch_dtype, device=device,
                                                 init_method=_init(config.initializer_range))
        self.down_proj = _linear_out(config, m.ff, device)


class VufasunDecoderLayer(nn.Module):
    def __init__(self, config: VufasunConfig, layer: VufasunLayerConfig, device=None):
        super().__init__()
        W, S = config.hidden_size, config.streams
        f32 = dict(dtype=torch.float32, device=device)
        self.type = layer.type
        self.columns, n_out = in_proj_columns(layer)
        self.norm1 = nn.Parameter(torch.ones(W, **f32))
        self.hc1_in, self.hc1_out = nn.Parameter(torch.ones(S, **f32)), nn.Parameter(torch.ones(S, **f32))
        self.hc1_mix = nn.Parameter(torch.eye(S, **f32))
        self.in_proj = ColumnParallelLinear(W, n_out, bias=False, gather_output=False, dtype=config.torch_dtype,
                                            device=device, init_method=_init(config.initializer_range))
        self.mixer = MIXERS[layer.type](config, layer.mixer, device=device)
        self.mlp = None
        self.mlp_kind = layer.mlp.kind if layer.mlp is not None else None
        if layer.mlp is not None:
            self.norm2 = nn.Parameter(torch.ones(W, **f32))
            self.hc2_in, self.hc2_out = nn.Parameter(torch.ones(S, **f32)), nn.Parameter(torch.ones(S, **f32))
            self.hc2_mix = nn.Parameter(torch.eye(S, **f32))
            if layer.mlp.kind == "dense":
                self.mlp = DenseGatedMlp(config, layer.mlp, device=device)
            else:
                self.mlp = SparseMoE(W, layer.mlp.experts, layer.mlp.top, layer.mlp.ff, None,
                                     shared_intermediate_size=layer.mlp.shared_ff, dtype=config.torch_dtype, device=device,
                                     score="sigmoid", weight_on_input=True, shared_gated=False)


class TiedHead(nn.Module):
    """The output head is the embedding table: ``logits = x E^T`` in fp32."""

    def __init__(self, embedding: nn.Module):
        super().__init__()
        self._embedding = [embedding]            # not a submodule: the table is registered once, as the embedding

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self._embedding[0].weight
        return gemm_nt(x.reshape(-1, x.shape[-1]).to(w.dtype), w, out_dtype=torch.float32).reshape(x.shape[:-1] + (w.shape[0],))


class VufasunForCausalLM(nn.Module):
    """``layers`` holds one module per configured layer; ``layer_sequence()`` is the list the model runs, in which a looped
    layer appears once per pass (same module, another cache / state index)."""

    def __init__(self, config: VufasunConfig, device=None):
        super().__init__()
        self.config = config
        dt = config.torch_dtype
        self.embed_tokens = ParallelEmbedding(config.vocab_size, config.hidden_size, dtype=dt, device=device,
                                              init_method=_init(config.initializer_range))
        self.layers = nn.ModuleList([VufasunDecoderLayer(config, L, device=device) for L in config.layers])
        self.norm = nn.Parameter(torch.ones(config.hidden_size, dtype=torch.float32, device=device))
        self.lm_head = TiedHead(self.embed_tokens)

    def layer_sequence(self) -> List[VufasunDecoderLayer]:
        return [self.layers[i] for i in self.config.layer_runs()]


def _fused_rows(parts: Dict[str, torch.Tensor], cols: Dict[str, Tuple[int, int]], n_out: int, W: int) -> torch.Tensor:
    first = next(iter(parts.values()))
    fused = first.new_zeros(n_out, W)
    for name, (at, n) in cols.items():
        assert parts[name].shape == (n, W), (name, tuple(parts[name].shape), n)
        fused[at: at + n] = parts[name]
    return fused


def _gated_rows(w: Dict[str, torch.Tensor]) -> torch.Tensor:
    """``gate`` / ``up`` ``[F, W]`` -> the grouped-expert layout ``[W, 2F]`` (gate | up on the output dim)."""
    return torch.cat([w["gate"].t(), w["up"].t()], dim=1)


def convert_vufasun_state_dict(sd: Dict[str, torch.Tensor], config: VufasunConfig) -> Dict[str, torch.Tensor]:
    """Checkpoint names (``embed``, ``final.norm``, ``l<i>.norm1 / norm2``, ``l<i>.hc1.in / out / mix`` ...,
    ``l<i>.mix.<name>``, ``l<i>.mlp.<name>``; linear weights ``[out, in]``) -> this module's state dict."""
    W, S = config.hidden_size, config.streams
    out: Dict[str, torch.Tensor] = {"embed_tokens.weight": sd["embed"], "norm": sd["final.norm"].float()}

    def streams_of(src: str, dst: str) -> None:
        if src + "in" in sd:
            out[dst + "_in"], out[dst + "_out"] = sd[src + "in"].float(), sd[src + "out"].float()
            out[dst + "_mix"] = sd[src + "mix"].float()
        elif S == 1:                                  # no stream weights: the plain residual sum
            out[dst + "_in"], out[dst + "_out"], out[dst + "_mix"] = torch.ones(1), torch.ones(1), torch.ones(1, 1)
        else:
            raise KeyError(f"{src}in: {S} streams need their weights")

    for i, L in enumerate(config.layers):
        src, dst, m = f"l{i}.", f"layers.{i}.", L.mixer
        mix = lambda n: sd[src + "mix." + n]                                          # noqa: E731
        cols, n_out = in_proj_columns(L)
        out[dst + "norm1"] = sd[src + "norm1"].float()
        streams_of(src + "hc1.", dst + "hc1")

        def attention_extras(a, name: str, to: str) -> None:
            if a.sink:
                out[to + "sink"] = mix(name + "sink").float()
            if a.whole_norm:
                out[to + "q_norm"], out[to + "k_norm"] = mix(name + "q.norm").float(), mix(name + "k.norm").float()

        if L.type == "attention":
            parts = {"qkv": torch.cat([mix("q"), mix("k"), mix("v")], dim=0)}
            attention_extras(m, "", dst + "mixer.")
            out[dst + "mixer.o_proj.weight"] = mix("o")
        else:
            parts = {"left": torch.cat([mix("left.q"), mix("left.k"), mix("left.v")], dim=0),
                     "right": torch.cat([mix("right.q"), mix("right.k"), mix("right.v"), mix("right.g")], dim=0)}
            attention_extras(m.left, "left.", dst + "mixer.left.")
            out[dst + "mixer.left.o_proj.weight"], out[dst + "mixer.right.o_proj.weight"] = mix("left.o"), mix("right.o")
            out[dst + "mixer.left_out"], out[dst + "mixer.right_out"] = mix("left.out").float(), mix("right.out").float()
        out[dst + "in_proj.weight"] = _fused_rows(parts, cols, n_out, W)
        if L.mlp is None:
            continue
        out[dst + "norm2"] = sd[src + "norm2"].float()
        streams_of(src + "hc2.", dst + "hc2")
        ml = lambda n: sd[src + "mlp." + n]                                           # noqa: E731
        if L.mlp.kind == "dense":
            F, Fp = L.mlp.ff, _up8(L.mlp.ff)
            gu = ml("gate").new_zeros(2 * Fp, W)
            gu[:F], gu[Fp: Fp + F] = ml("gate"), ml("up")
            out[dst + "mlp.gate_up_proj.weight"], out[dst + "mlp.down_proj.weight"] = gu, ml("down")
        else:
            E = L.mlp.experts
            out[dst + "mlp.router.linear_router.weight"] = ml("router").float()
            out[dst + "mlp.router.correction"] = torch.zeros(E)
            out[dst + "mlp.experts.gate_up_proj.weight"] = torch.stack(
                [_gated_rows({"gate": ml(f"e{e}.gate"), "up": ml(f"e{e}.up")}) for e in range(E)])
            out[dst + "mlp.experts.down_proj.weight"] = torch.stack([ml(f"e{e}.down").t() for e in range(E)])
            if L.mlp.shared_ff:
                out[dst + "mlp.shared.gate_up_proj.weight"] = _gated_rows({"gate": ml("shared.gate"),
                                                                           "up": ml("shared.up")}).unsqueeze(0)
                out[dst + "mlp.shared.down_proj.weight"] = ml("shared.down").t().unsqueeze(0)
    return {k: v.contiguous() for k, v in out.items()}


def export_vufasun_state_dict(model: VufasunForCausalLM) -> Dict[str, torch.Tensor]:
    """The inverse of ``convert_vufasun_state_dict``: this module's parameters under the checkpoint names."""
    cfg, sd = model.config, model.state_dict()
    out: Dict[str, torch.Tensor] = {"embed": sd["embed_tokens.weight"], "final.norm": sd["norm"]}
    for i, L in enumerate(cfg.layers):
        src, dst, m = f"layers.{i}.", f"l{i}.", L.mixer
        cols, _ = in_proj_columns(L)
        fused = sd[src + "in_proj.weight"]
        part = lambda n: fused[cols[n][0]: cols[n][0] + cols[n][1]]                    # noqa: E731
        out[dst + "norm1"] = sd[src + "norm1"]
        for q in ("hc1", "hc2") if L.mlp is not None else ("hc1",):
            for n in ("in", "out", "mix"):
                out[f"{dst}{q}.{n}"] = sd[f"{src}{q}_{n}"]

        def split_attention(rows, a, prefix):
            nq, nk = a.heads * a.dim, a.kv_heads * a.dim
            out[prefix + "q"], out[prefix + "k"], out[prefix + "v"] = rows[:nq], rows[nq: nq + nk], rows[nq + nk:]

        def attention_extras(a, frm: str, to: str) -> None:
            if a.sink:
                out[to + "sink"] = sd[frm + "sink"]
            if a.whole_norm:
                out[to + "q.norm"], out[to + "k.norm"] = sd[frm + "q_norm"], sd[frm + "k_norm"]

        if L.type == "attention":
            split_attention(part("qkv"), m, dst + "mix.")
            attention_extras(m, src + "mixer.", dst + "mix.")
            out[dst + "mix.o"] = sd[src + "mixer.o_proj.weight"]
        else:
            split_attention(part("left"), m.left, dst + "mix.left.")
            r, rows = m.right, part("right")
            a, c = r.heads * r.dim, r.heads * r.vdim
            out[dst + "mix.right.q"], out[dst + "mix.right.k"] = rows[:a], rows[a: 2 * a]
            out[dst + "mix.right.v"], out[dst + "mix.right.g"] = rows[2 * a: 2 * a + c], rows[2 * a + c:]
            attention_extras(m.left, src + "mixer.left.", dst + "mix.left.")
            out[dst + "mix.left.o"], out[dst + "mix.right.o"] = sd[src + "mixer.left.o_proj.weight"], sd[src + "mixer.right.o_proj.weight"]
            out[dst + "mix.left.out"], out[dst + "mix.right.out"] = sd[src + "mixer.left_out"], sd[src + "mixer.right_out"]
        if L.mlp is None:
            continue
        out[dst + "norm2"] = sd[src + "norm2"]
        if L.mlp.kind == "dense":
            F, Fp = L.mlp.ff, _up8(L.mlp.ff)
            gu = sd[src + "mlp.gate_up_proj.weight"]
            out[dst + "mlp.gate"], out[dst + "mlp.up"], out[dst + "mlp.down"] = gu[:F], gu[Fp: Fp + F], sd[src + "mlp.down_proj.weight"]
        else:
            F = L.mlp.ff
            gu, dn = sd[src + "mlp.experts.gate_up_proj.weight"], sd[src + "mlp.experts.down_proj.weight"]
            out[dst + "mlp.router"] = sd[src + "mlp.router.linear_router.weight"]
            for e in range(L.mlp.experts):
                out[f"{dst}mlp.e{e}.gate"], out[f"{dst}mlp.e{e}.up"] = gu[e, :, :F].t(), gu[e, :, F:].t()
                out[f"{dst}mlp.e{e}.down"] = dn[e].t()
            if L.mlp.shared_ff:
                Fs = L.mlp.shared_ff
                sgu = sd[src + "mlp.shared.gate_up_proj.weight"][0]
                out[dst + "mlp.shared.gate"], out[dst + "mlp.shared.up"] = sgu[:, :Fs].t(), sgu[:, Fs:].t()
                out[dst + "mlp.shared.down"] = sd[src + "mlp.shared.down_proj.weight"][0].t()
    return {k: v.detach().clone().contiguous() for k, v in out.items()}


def tiny_vufasun(torch_dtype: torch.dtype = torch.float32, **kw) -> VufasunConfig:
    """A small configuration for tests and smoke runs: three streams, a sink-attention layer without a feed-forward, a
    parallel layer with a sparse feed-forward of two chosen experts, a sink-attention layer with a dense one; the first
    two layers run twice."""
    att = {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.3, "rot": {"base": 10000.0, "dims": 8}}
    par = {"left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.2,
                    "rot": {"base": 5000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 32}}},
           "right": {"heads": 3, "dim": 8, "vdim": 16, "decay": [0.9, 0.97, 0.995], "rot": {"base": 100.0, "dims": 4}}}
    d = {"architecture": "Vufasun", "vocab": 96, "width": 40, "streams": 3, "norm": {"eps": 1e-5},
         "loop": {"start": 0, "stop": 2, "times": 2},
         "layers": [{"type": "attention", "mixer": att, "mlp": None},
                    {"type": "parallel", "mixer": par,
                     "mlp": {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 5, "top": 2}, "shared": {"ff": 16}}},
                    {"type": "attention", "mixer": dict(att, heads=2, kv_heads=2), "mlp": {"kind": "dense", "ff": 52}}]}
    d.update(kw)
    return VufasunConfig.from_dict(d, torch_dtype=torch_dtype)
