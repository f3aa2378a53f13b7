"""Hybrid families (recurrent mixers next to attention over the cache) over the framework's step function: Rasodra and,
further down, Gogalix and Vufasun.

Rasodra over the framework's step function: chunked attention, latent attention and the recurrent matrix memory on
one KV cache / state manager.

The step function (``forward_infer``: padding, cache lines through ``seq_ids``, indexed logits, sampler, ``generate``),
the schedulers and the runners are the mixin's; this class says what a layer does with the stream:

  * ``hidden`` is the fp32 residual stream ``x``, ``residual`` carries ``norm1(x)`` of the layer about to run, in the
    activation dtype: the norm after a sublayer, the residual add and the norm before the next sublayer are one kernel
    (``ops.norm.norm_chain_``);
  * ``attention``: q | k projection -> per-head norm + rotation + cache write (K = normalised rotated key, V = the key as
    projected) -> attention over the cache with the chunk mask -> output projection;
  * ``latent_attention``: q | latent | gate projection -> latent norm, rotations and the cache row ``[c | k_rot]`` ->
    absorbed queries (one batched product with ``uk``) -> attention over the latent rows with the sink in the
    denominator (one key/value "head", value = the ``c`` columns of the same tensor) -> per-head ``uv`` product ->
    sigmoid gate -> output projection;
  * ``mlstm``: q | k | v | gate projection, fp32 gate dot products -> scan over the step's tokens on the line's fp32 state
    -> unit-RMS per head, weight, sigmoid gate -> output projection;
  * a layer with ``weights_of`` runs its owner's modules on cache tensors / state of its own (the cache and the state are
    indexed by the position in the layer list, the modules by the owner).
A step may start at any position: attention reads earlier keys from the cache, the scan continues from the line's state.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..models.gogalix import UNIT_NORM_EPS, GogalixConfig, GogalixForCausalLM
from ..models.rasodra import RasodraConfig, RasodraForCausalLM
from ..models.vufasun import VufasunConfig, VufasunForCausalLM
from ..ops import activation as act_ops
from ..ops import attention as attn_ops
from ..ops import delta_rule as delta_ops
from ..ops import hyper_connection as hc_ops
from ..ops import latent_attention as la_ops
from ..ops import mlstm as mlstm_ops
from ..ops import moe_sparse as moe_ops
from ..ops import norm as norm_ops
from ..ops import retention as ret_ops
from ..ops import rope as rope_ops
from ..ops import window_attention as wa_ops
from ..ops.linear import gemm_nt
from .config import InferenceConfig
from .kv_cache import KVCache
from .model import KVCacheInferenceMixin


class RasodraInferenceModel(KVCacheInferenceMixin, RasodraForCausalLM):
    supports_prefill_at_offset = True

    def __init__(self, config: RasodraConfig, inference_config: Optional[InferenceConfig] = None, device=None):
        RasodraForCausalLM.__init__(self, config, device=device)
        self._init_inference(inference_config)
        self._sequence = self.layer_sequence()
        self._rope_cache: Dict[Tuple[int, float], Tuple[torch.Tensor, torch.Tensor]] = {}
        self.layer_probe = None            # callable(i, x) after every layer run (debugging / layer-by-layer checks)

    # -- where the pieces are ---------------------------------------------------------------------------------------
    def _decoder_layers(self):
        return self._sequence

    def _embedding(self):
        return self.embed_tokens

    def _final_norm(self):
        return self.norm

    def init_kv_cache(self, device=None, dtype=None) -> KVCache:
        ic, cfg = self.inference_config, self.config
        device = device or next(self.parameters()).device
        specs, states = [], {}
        for i, L in enumerate(cfg.layers):
            m = L.mixer
            if L.type == "attention":
                specs.append((m.kv_heads, m.dim, m.vdim))
            elif L.type == "latent_attention":
                specs.append((1, m.kv_rank + m.rot_dim, m.kv_rank, "columns"))
            else:
                specs.append(None)
                states[i] = {"S": (m.heads, m.dim, m.vdim), "n": (m.heads, m.dim), "m": (m.heads,)}
        self.kv_cache = KVCache(len(cfg.layers), ic.max_batch_size, 0, ic.seq_len, 0, dtype=dtype or cfg.torch_dtype,
                                device=device, paged=ic.paged_kv, page_size=ic.page_size,
                                num_pages=ic.num_kv_pages if ic.paged_kv else None, layer_specs=specs, state_specs=states)
        return self.kv_cache

    def _rotary_tables(self, rot, device) -> Tuple[torch.Tensor, torch.Tensor]:
        key = (rot.dims, rot.base)
        t = self._rope_cache.get(key)
        if t is None or t[0].device != device or t[0].shape[0] < self.kv_cache.seq_len:
            t = rope_ops.build_interleaved_rope_cache(self.kv_cache.seq_len, rot.dims, rot.base, device=device)
            self._rope_cache[key] = t
        return t

    def _embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        return super()._embed(input_ids).float()           # the stream is fp32 from the first layer on

    def _add_norm(self, norm, hidden: torch.Tensor, residual: Optional[torch.Tensor]):
        """Only the model's final norm comes through here: plain norm of the fp32 stream."""
        return norm(hidden, out_dtype=self.config.torch_dtype), None

    @staticmethod
    def _proj(linear, x: torch.Tensor) -> torch.Tensor:
        """``x W^T (+ b)`` of a linear layer through the framework's GEMM dispatch directly (tensor-parallel size 1, no
        gradients: the layer's autograd and collective wrappers would only cost host time per step)."""
        y = gemm_nt(x.reshape(-1, x.shape[-1]), linear.weight)
        if getattr(linear, "bias", None) is not None:
            y = y.add_(linear.bias)
        return y.reshape(x.shape[:-1] + (linear.weight.shape[0],))

    # -- mixers: h [B, T, W] in the activation dtype -> [B, T, W] ---------------------------------------------------------
    def _paged(self) -> dict:
        kc = self.kv_cache
        return dict(block_table=kc.block_table, page_size=kc.page_size) if kc.paged else {}

    TC_PREFILL_MIN_TOKENS = 128          # shorter steps stay on the cache-reading kernels

    def _chunks_as_batch(self, qk, m, T: int) -> bool:
        return (T >= self.TC_PREFILL_MIN_TOKENS and not self._step_past_context and not self.kv_cache.paged
                and (not m.chunk or T <= m.chunk or T % m.chunk == 0)
                and wa_ops.tc_prefill_applies(qk, m.dim, m.vdim, qk.shape[-1]))

    def _mix_attention(self, i, mixer, h, q_start, n_new, seq_ids):
        m, cfg = mixer.cfg, self.config
        B, T, _ = h.shape
        ck, cv = self.kv_cache.layer(i)
        paged = self._paged()
        qk = self._proj(mixer.qk_proj, h)
        rope = self._rotary_tables(m.rot, h.device) if m.rot is not None else None
        q = wa_ops.qk_norm_cache_write(qk, ck, cv, q_start, m.heads, m.kv_heads, m.dim, m.vdim, cfg.rms_norm_eps,
                                       n_new=n_new, seq_ids=seq_ids, q_weight=mixer.q_norm, k_weight=mixer.k_norm,
                                       rope=rope, value_from_key=True, **paged)
        if T == 1:
            o = wa_ops.window_attention_decode(q[:, 0], ck, cv, q_start, m.scale, seq_ids=seq_ids, chunk=m.chunk, **paged)
        elif self._chunks_as_batch(qk, m, T):
            # prompts from position 0 whose length is a whole number of chunks (or one partial chunk): every chunk is an
            # independent causal sequence, so the step runs on the tcgen05 flash-attention kernel with the chunks as
            # batch rows; K comes back from the cache rows just written, V is the key columns of the projection output
            size = m.chunk if (m.chunk and T > m.chunk) else T
            lines = seq_ids.long() if seq_ids is not None else torch.arange(B, device=h.device)
            kx = ck[lines, :, :T].transpose(1, 2).contiguous().reshape(B * (T // size), size, m.kv_heads, m.dim)
            vx = qk[..., m.heads * m.dim:].reshape(B * (T // size), size, m.kv_heads, m.dim)
            qx = q.reshape(B * (T // size), size, m.heads, m.dim)
            o = attn_ops.flash_attn_func(qx.permute(0, 2, 1, 3), kx.permute(0, 2, 1, 3), vx.permute(0, 2, 1, 3),
                                         softmax_scale=m.scale, causal=True).permute(0, 2, 1, 3)
        else:
            o = wa_ops.window_attention_prefill(q, ck, cv, q_start, m.scale, n_new=n_new, seq_ids=seq_ids, chunk=m.chunk,
                                                **paged)
        return self._proj(mixer.o_proj, o.reshape(B, T, m.heads * m.vdim))

    def _latent_rows(self, ck, lines, n_ctx: int) -> torch.Tensor:
        """Rows ``[0, n_ctx)`` of the given cache lines of a latent cache tensor, ``[len(lines), n_ctx, rank + rot]``."""
        kc = self.kv_cache
        if not kc.paged:
            return ck[lines.long(), 0, :n_ctx]
        n_pages = (n_ctx + kc.page_size - 1) // kc.page_size
        pages = kc.block_table[lines.long(), :n_pages].long()                      # [B, n_pages]
        return ck[pages][:, :, 0].reshape(pages.shape[0], n_pages * kc.page_size, ck.shape[-1])[:, :n_ctx]

    def _step_context_len(self, q_start, n_new, T: int) -> int:
        """Positions that the step's rows reach at most.  A step that starts every row at position 0 needs no look at the
        device (T, which keeps the step capturable in a CUDA graph); a step of portions reads it back once."""
        if not self._step_past_context:
            return T
        if "n_ctx" not in self._step_kv:
            self._step_kv["n_ctx"] = int((q_start + (n_new if n_new is not None else T)).max())
        return self._step_kv["n_ctx"]

    def _mix_latent(self, i, mixer, h, q_start, n_new, seq_ids):
        m, cfg, dt = mixer.cfg, self.config, self.config.torch_dtype
        B, T, _ = h.shape
        N, H, R = B * T, m.heads, m.kv_rank
        ck, cv = self.kv_cache.layer(i)                    # cv: the first kv_rank columns of ck's rows
        paged = self._paged()
        proj = self._proj(mixer.in_proj, h)
        rope = self._rotary_tables(m.rot, h.device)
        if T == 1:
            # token generation: absorbed queries over the latent rows, value projection after the attention
            q_abs = torch.empty(N, H, R + m.rot_dim, dtype=dt, device=h.device)
            q_nope = la_ops.latent_prep(proj, 0, mixer.q_cols, q_abs, ck, mixer.kv_norm, rope, q_start, H, m.dim,
                                        m.rot_dim, R, cfg.rms_norm_eps, n_new=n_new, seq_ids=seq_ids, **paged)
            q_abs[..., :R] = torch.bmm(q_nope.transpose(0, 1), mixer.uk).transpose(0, 1)
            o_lat = wa_ops.window_attention_decode(q_abs, ck, cv, q_start, m.scale, seq_ids=seq_ids, sinks=mixer.sink,
                                                   **paged)
            o = torch.bmm(o_lat.transpose(0, 1), mixer.uv.transpose(1, 2)).transpose(0, 1).contiguous()   # [N, H, vdim]
        else:
            # prompt steps: per-head keys and values expanded from the latent rows of every line of the step (all
            # positions up to the step's end: a portion at an offset sees the earlier rows too), then attention with
            # head size dim + rot; the expansion is two matrix products over the rows
            q = la_ops.latent_prep(proj, 0, mixer.q_cols, None, ck, mixer.kv_norm, rope, q_start, H, m.dim, m.rot_dim, R,
                                   cfg.rms_norm_eps, n_new=n_new, seq_ids=seq_ids, **paged)
            n_ctx = self._step_context_len(q_start, n_new, T)
            lines = seq_ids if seq_ids is not None else torch.arange(B, device=h.device)
            rows = self._latent_rows(ck, lines, n_ctx)                               # [B, n_ctx, R + rot]
            c = rows[..., :R].reshape(B * n_ctx, R)
            keys = torch.empty(B, n_ctx, H, m.dim + m.rot_dim, dtype=dt, device=h.device)
            keys[..., :m.dim] = gemm_nt(c.contiguous(), mixer.uk.reshape(H * m.dim, R)).reshape(B, n_ctx, H, m.dim)
            keys[..., m.dim:] = rows[..., R:].unsqueeze(2)
            vals = gemm_nt(c.contiguous(), mixer.uv.reshape(H * m.vdim, R)).reshape(B, n_ctx, H, m.vdim)
            o = wa_ops.window_attention_prefill(q.reshape(B, T, H, m.dim + m.rot_dim), keys.permute(0, 2, 1, 3),
                                                vals.permute(0, 2, 1, 3), q_start, m.scale, n_new=n_new,
                                                sinks=mixer.sink).reshape(N, H, m.vdim)
        y = mlstm_ops.head_norm_gate(o, proj.reshape(N, -1), mixer.q_cols + mixer.kv_cols, H, m.vdim, None,
                                     cfg.rms_norm_eps, False, dt)
        return self._proj(mixer.o_proj, y.reshape(B, T, H * m.vdim))

    CHUNKWISE_MIN_TOKENS = 64
    CHUNKWISE_FP32 = False               # fp32 serving keeps the token-by-token scan (tests switch this on)

    def _mix_mlstm(self, i, mixer, h, q_start, n_new, seq_ids):
        m, cfg, dt = mixer.cfg, self.config, self.config.torch_dtype
        B, T, W = h.shape
        N, H = B * T, m.heads
        st = self.kv_cache.state(i)
        proj = self._proj(mixer.in_proj, h)
        gi, gf = mlstm_ops.mlstm_gates(h.reshape(N, W), mixer.gate_weight, mixer.gate_bias, H, m.gate_cap)
        # long bf16 steps take the chunk-wise form (matrix products); token generation, short steps and fp32 serving the
        # token-by-token scan
        chunkwise = T >= self.CHUNKWISE_MIN_TOKENS and (dt != torch.float32 or self.CHUNKWISE_FP32)
        run = mlstm_ops.mlstm_chunkwise if chunkwise else mlstm_ops.mlstm_scan
        o = run(proj, (0, H * m.dim, 2 * H * m.dim), gi, gf, (st["S"], st["n"], st["m"]), q_start, H, m.dim, m.vdim,
                m.dim ** -0.5, n_new=n_new, seq_ids=seq_ids)
        y = mlstm_ops.head_norm_gate(o.reshape(N, H, m.vdim), proj.reshape(N, -1), 2 * H * m.dim + H * m.vdim, H, m.vdim,
                                     mixer.out_norm, cfg.rms_norm_eps, True, dt)
        return self._proj(mixer.o_proj, y.reshape(B, T, H * m.vdim))

    _MIX = {"attention": _mix_attention, "latent_attention": _mix_latent, "mlstm": _mix_mlstm}

    # -- one layer --------------------------------------------------------------------------------------------------
    def _layer(self, i: int, layer, hidden, residual, positions, seq_ids, lengths, prefill):
        dt = self.config.torch_dtype
        x = hidden if hidden.is_contiguous() else hidden.contiguous()
        h = residual if residual is not None else layer.norm1(x, out_dtype=dt)
        if "q_start" not in self._step_kv:      # one int32 copy of the rows' first positions per step, not per kernel
            self._step_kv["q_start"] = positions[:, 0].to(torch.int32).contiguous()
        q_start = self._step_kv["q_start"]
        n_new = self._step_new_tokens if prefill else None
        y = self._MIX[layer.type](self, i, layer.mixer, h, q_start, n_new, seq_ids)
        nxt = self._sequence[i + 1].norm1 if i + 1 < len(self._sequence) else None
        if layer.mlp is None:
            x, h = layer.norm1b.add_to(x, y, nxt, dt)
        else:
            x, h = layer.norm1b.add_to(x, y, layer.norm2, dt)
            y = self._proj(layer.mlp.down_proj, act_ops.relu_squared(self._proj(layer.mlp.up_proj, h)))
            x, h = layer.norm2b.add_to(x, y, nxt, dt)
        if self.layer_probe is not None:
            self.layer_probe(i, x)
        return x, h

    def forward_speculation(self, *a, **kw):
        raise NotImplementedError("the speculation verify graph is not wired for this family")


class GogalixInferenceModel(KVCacheInferenceMixin, GogalixForCausalLM):
    """Gogalix over the KV cache / state manager.  The step function (padding, cache lines through ``seq_ids``, indexed
    logits, sampler, ``generate``), the schedulers and the runners are the mixin's; this class says what a layer does:

      * ``hidden`` is the fp32 stream ``x``, ``residual`` carries ``norm1(x)`` of the layer about to run in the
        activation dtype (the residual update of a layer and the next layer's norm are one kernel);
      * ONE matrix product of the normed input gives the mixer's projections, its output gate, both residual gates and
        the dense gate / up (``layer.in_proj``, parts at ``layer.columns``); the kernels read their part in place;
      * ``attention``: the two maps of every head are separate heads of the windowed attention over the cache (queries
        and keys map-major, the value heads shared by the two maps), then ``a1 - lambda a2`` + head norm;
      * ``delta`` / ``channel_delta``: short convolution + silu + unit norm from the line's convolution state, the
        gated-delta recurrence on the line's fp32 state, head norm * weight * output gate;
      * ``x += ls1 * sigmoid(rg1) * mixer + ls2 * sigmoid(rg2) * ff`` and the next norm in one pass.
    A step may start at any position: attention reads earlier keys from the cache, the recurrence continues from the
    line's state."""

    supports_prefill_at_offset = True

    def __init__(self, config: GogalixConfig, inference_config: Optional[InferenceConfig] = None, device=None):
        GogalixForCausalLM.__init__(self, config, device=device)
        self._init_inference(inference_config)
        self.layer_probe = None            # callable(i, x) after every layer run (debugging / layer-by-layer checks)

    def _decoder_layers(self):
        return self.layers

    def _embedding(self):
        return self.embed_tokens

    def _final_norm(self):
        return self.norm

    def init_kv_cache(self, device=None, dtype=None) -> KVCache:
        ic, cfg = self.inference_config, self.config
        device = device or next(self.parameters()).device
        specs, states, share = [], {}, {}
        for i, L in enumerate(cfg.layers):
            m = L.mixer
            if L.type == "attention":
                # the two maps' keys are 2 * kv_heads key heads (map-major); both maps read the same kv_heads value heads
                specs.append((2 * m.kv_heads, m.dim, m.vdim, "heads", m.kv_heads))
                if m.kv_from is not None:
                    share[i] = m.kv_from
            else:
                specs.append(None)
                states[i] = {"S": (m.heads, m.dim, m.vdim), "conv": (m.conv - 1, m.channels)}
        self.kv_cache = KVCache(len(cfg.layers), ic.max_batch_size, 0, ic.seq_len, 0, dtype=dtype or cfg.torch_dtype,
                                device=device, paged=ic.paged_kv, page_size=ic.page_size,
                                num_pages=ic.num_kv_pages if ic.paged_kv else None, layer_specs=specs, share_from=share,
                                state_specs=states)
        return self.kv_cache

    def _embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        return super()._embed(input_ids).float().mul_(self.config.embedding_scale)       # the stream is fp32

    def _add_norm(self, norm, hidden: torch.Tensor, residual: Optional[torch.Tensor]):
        """Only the model's final norm comes through here: plain one-weight RMS norm of the fp32 stream."""
        W = hidden.shape[-1]
        h = norm_ops.gated_residual_norm_(hidden.reshape(-1, W), None, w_next=norm, eps=self.config.rms_norm_eps,
                                          out_dtype=self.config.torch_dtype)[1]
        return h.reshape(hidden.shape), None

    def _paged(self) -> dict:
        kc = self.kv_cache
        return dict(block_table=kc.block_table, page_size=kc.page_size) if kc.paged else {}

    # -- mixers: big [N, n_out] = the fused projection of the normed input -> [N, W] in the activation dtype -------------
    def _mix_attention(self, i, layer, h2, big, B, T, q_start, n_new, seq_ids):
        mixer, m, cfg = layer.mixer, layer.mixer.cfg, self.config
        H, G, D, Dv = m.heads, m.kv_heads, m.dim, m.vdim
        kc = self.kv_cache
        ck, cv = kc.layer(i)
        owns = kc.owns(i)
        paged = self._paged()
        at, n = layer.columns["qkv"]
        qkv = big.view(B, T, -1)[..., at: at + n]
        q = wa_ops.qk_norm_cache_write(qkv, ck if owns else None, cv if owns else None, q_start, 2 * H, 2 * G, D, Dv,
                                       cfg.rms_norm_eps, n_new=n_new, seq_ids=seq_ids, normalize=False, value_heads=G,
                                       **paged)
        if T == 1:
            maps = wa_ops.window_attention_decode(q[:, 0], ck, cv, q_start, m.scale, m.window, seq_ids=seq_ids,
                                                  value_heads=G, **paged)
        else:
            maps = wa_ops.window_attention_prefill(q, ck, cv, q_start, m.scale, m.window, n_new=n_new, seq_ids=seq_ids,
                                                   value_heads=G, **paged)
        o = wa_ops.diff_attention_combine(maps.reshape(B * T, 2 * H, Dv), mixer.lq1, mixer.lk1, mixer.lq2, mixer.lk2,
                                          m.diff, cfg.rms_norm_eps)
        return gemm_nt(o, mixer.o_proj.weight)

    def _mix_delta(self, i, layer, h2, big, B, T, q_start, n_new, seq_ids):
        mixer, m, cfg, dt = layer.mixer, layer.mixer.cfg, self.config, self.config.torch_dtype
        H, G, D, Dv, N = m.heads, m.kv_heads, m.dim, m.vdim, B * T
        st = self.kv_cache.state(i)
        at = layer.columns["qkv"][0]
        qn, kn, vn = delta_ops.delta_prep(big.view(B, T, -1), (at, at + G * D, at + 2 * G * D), mixer.conv_weight,
                                          st["conv"], q_start, H, G, D, Dv, D ** -0.5, UNIT_NORM_EPS, n_new=n_new,
                                          seq_ids=seq_ids)
        # pre-activations of the recurrence's gates stay fp32: beta rows, then (one decay per head) the decay rows
        gates = gemm_nt(h2, mixer.gate_proj, out_dtype=torch.float32)
        if m.per_channel:
            rk = mixer.a2.shape[1]              # the low-rank inner size, padded; the padding columns of `big` are zeros
            a_pre = gemm_nt(big[:, layer.columns["a1"][0]:][:, :rk].contiguous(), mixer.a2, out_dtype=torch.float32)
            a_off = 0
            gate_src = gemm_nt(big[:, layer.columns["g1"][0]:][:, :rk].contiguous(), mixer.g2)
            gate_off, gate_act = 0, "sigmoid"
        else:
            a_pre, a_off = gates, H
            gate_src, gate_off, gate_act = big, layer.columns["g"][0], "silu"
        o = delta_ops.delta_scan(qn, kn, vn, a_pre, a_off, gates, 0, mixer.a_log, mixer.dt_bias, st["S"], q_start,
                                 m.per_channel, n_new=n_new, seq_ids=seq_ids)
        y = mlstm_ops.head_norm_gate(o.reshape(N, H, Dv), gate_src, gate_off, H, Dv, mixer.out_norm, cfg.rms_norm_eps,
                                     True, dt, gate_act=gate_act)
        return gemm_nt(y, mixer.o_proj.weight)

    _MIX = {"attention": _mix_attention, "delta": _mix_delta, "channel_delta": _mix_delta}

    # -- one layer --------------------------------------------------------------------------------------------------
    def _layer(self, i: int, layer, hidden, residual, positions, seq_ids, lengths, prefill):
        cfg, dt = self.config, self.config.torch_dtype
        B, T, W = hidden.shape
        N = B * T
        x = (hidden if hidden.is_contiguous() else hidden.contiguous()).view(N, W)
        h2 = (residual.reshape(N, W) if residual is not None else
              norm_ops.gated_residual_norm_(x, None, w_next=layer.norm1, eps=cfg.rms_norm_eps, out_dtype=dt)[1])
        if "q_start" not in self._step_kv:      # one int32 copy of the rows' first positions per step, not per kernel
            self._step_kv["q_start"] = positions[:, 0].to(torch.int32).contiguous()
        q_start = self._step_kv["q_start"]
        n_new = self._step_new_tokens if prefill else None
        big = gemm_nt(h2, layer.in_proj.weight)
        cols = layer.columns
        y1 = self._MIX[layer.type](self, i, layer, h2, big, B, T, q_start, n_new, seq_ids)
        y2 = y2_bias = None
        if layer.mlp_kind == "dense":
            ff = layer.mlp.gate_bias.shape[0]
            act = moe_ops.glu_bias(big, cols["gate"][0], cols["up"][0], ff, layer.mlp.gate_bias, layer.mlp.up_bias)
            y2, y2_bias = gemm_nt(act, layer.mlp.down_proj.weight), layer.mlp.down_bias
        elif layer.mlp_kind == "moe":
            y2 = layer.mlp(h2)                                       # fp32 [N, W]
        nxt = self.layers[i + 1].norm1 if i + 1 < len(self.layers) else None
        has_ff = layer.mlp_kind is not None
        x, h_next = norm_ops.gated_residual_norm_(
            x, y1, y2, y2_bias, gate=big, gate_offsets=(cols["rg1"][0], cols["rg2"][0] if has_ff else 0),
            gate_bias1=layer.rg1_bias, gate_bias2=layer.rg2_bias if has_ff else None, scale1=layer.ls1,
            scale2=layer.ls2 if has_ff else None, w_next=nxt, eps=cfg.rms_norm_eps, out_dtype=dt)
        if self.layer_probe is not None:
            self.layer_probe(i, x.view(B, T, W))
        return x.view(B, T, W), (h_next.view(B, T, W) if h_next is not None else None)

    def forward_speculation(self, *a, **kw):
        raise NotImplementedError("the speculation verify graph is not wired for this family")


class VufasunInferenceModel(KVCacheInferenceMixin, VufasunForCausalLM):
    """Vufasun over the KV cache / state manager.  The step function (padding, cache lines through ``seq_ids``, indexed
    logits, sampler, ``generate``), the schedulers and the runners are the mixin's; this class says what a layer does:

      * ``hidden`` is the fp32 streams ``[B, T, streams * W]`` (stream-major per token), ``residual`` carries the normed
        weighted sum that the sublayer about to run reads, in the activation dtype: the write of a sublayer's output into
        the streams and the read of the next sublayer are one kernel (``ops.hyper_connection.hc_step``);
      * ONE matrix product of the mixer's input gives all its projections (``layer.in_proj``, parts at
        ``layer.columns``); the kernels read their part in place;
      * softmax attention: whole-projection norm (left branch of a parallel layer) + "rotate half" rotation + cache write
        in one kernel, then attention over the cache with the sink logit in the denominator (``attention`` layers); a
        bf16 prompt from position 0 without a sink term and with equal key / value sizes of 64 or 128 runs on the tcgen05
        flash-attention kernel instead;
      * retention: rotation, key scale and the recurrence on the line's fp32 state in one kernel (token by token, or in
        chunks of 64 tokens for long steps), then unit RMS per head * ``silu`` gate;
      * a parallel layer hands both branch outputs to the stream kernel, which norms and averages them;
      * a looped layer appears once per pass in the run list: same modules, cache / state of the run's own index.
    A step may start at any position: attention reads earlier keys from the cache, the recurrence continues from the
    line's state."""

    supports_prefill_at_offset = True
    CHUNKWISE_MIN_TOKENS = 64            # shorter steps walk the recurrence token by token
    TC_PREFILL_MIN_TOKENS = 128          # shorter steps stay on the cache-reading attention kernels

    def __init__(self, config: VufasunConfig, inference_config: Optional[InferenceConfig] = None, device=None):
        VufasunForCausalLM.__init__(self, config, device=device)
        self._init_inference(inference_config)
        self._sequence = self.layer_sequence()
        self._rope_cache: Dict[tuple, Tuple[torch.Tensor, torch.Tensor]] = {}
        self._unit_in: Optional[torch.Tensor] = None
        self.layer_probe = None            # callable(i, x) after every layer run (debugging / layer-by-layer checks)

    def _decoder_layers(self):
        return self._sequence

    def _embedding(self):
        return self.embed_tokens

    def _final_norm(self):
        return self.norm

    def init_kv_cache(self, device=None, dtype=None) -> KVCache:
        ic, cfg = self.inference_config, self.config
        device = device or next(self.parameters()).device
        specs, states = [], {}
        for run, li in enumerate(cfg.layer_runs()):           # one cache / state entry per layer RUN
            L = cfg.layers[li]
            a = L.mixer if L.type == "attention" else L.mixer.left
            specs.append((a.kv_heads, a.dim, a.vdim))
            if L.type == "parallel":
                r = L.mixer.right
                states[run] = {"S": (r.heads, r.dim, r.vdim)}
        self.kv_cache = KVCache(len(specs), ic.max_batch_size, 0, ic.seq_len, 0, dtype=dtype or cfg.torch_dtype,
                                device=device, paged=ic.paged_kv, page_size=ic.page_size,
                                num_pages=ic.num_kv_pages if ic.paged_kv else None, layer_specs=specs, state_specs=states)
        return self.kv_cache

    def _rotary_tables(self, rot, device) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        if rot is None:
            return None
        key = (rot.dims, rot.base, rot.scaling)
        t = self._rope_cache.get(key)
        if t is None or t[0].device != device or t[0].shape[0] < self.kv_cache.seq_len:
            t = rope_ops.build_interleaved_rope_cache(self.kv_cache.seq_len, rot.dims, rot.base, device=device,
                                                      scaling=rot.scaling)
            self._rope_cache[key] = t
        return t

    def _embed(self, input_ids: torch.Tensor) -> torch.Tensor:
        x = super()._embed(input_ids).float()                 # every stream starts as the embedding, in fp32
        B, T, W = x.shape
        S = self.config.streams
        return x.unsqueeze(2).expand(B, T, S, W).reshape(B, T, S * W)

    def _add_norm(self, norm, hidden: torch.Tensor, residual: Optional[torch.Tensor]):
        """Only the model's final norm comes through here: RMS norm of the plain sum of the streams."""
        S, W = self.config.streams, self.config.hidden_size
        if self._unit_in is None or self._unit_in.device != hidden.device:
            self._unit_in = torch.ones(S, dtype=torch.float32, device=hidden.device)
        x = hidden.reshape(-1, S, W)
        h = hc_ops.hc_step(x if x.is_contiguous() else x.contiguous(), in_w=self._unit_in, norm_w=norm,
                           eps=self.config.rms_norm_eps, out_dtype=self.config.torch_dtype)
        return h.reshape(hidden.shape[:-1] + (W,)), None

    def _paged(self) -> dict:
        kc = self.kv_cache
        return dict(block_table=kc.block_table, page_size=kc.page_size) if kc.paged else {}

    # -- mixers: columns of big [B, T, n_out] = the fused projection of the normed input -> [N, W] ------------------------
    def _softmax_attention(self, run, mixer, big, at, B, T, q_start, n_new, seq_ids):
        m, cfg = mixer.cfg, self.config
        ck, cv = self.kv_cache.layer(run)
        paged = self._paged()
        qkv = big[..., at: at + m.columns]
        q = wa_ops.qk_norm_cache_write(qkv, ck, cv, q_start, m.heads, m.kv_heads, m.dim, m.vdim, cfg.rms_norm_eps,
                                       n_new=n_new, seq_ids=seq_ids, normalize=m.whole_norm, q_weight=mixer.q_norm,
                                       k_weight=mixer.k_norm, rope=self._rotary_tables(m.rot, big.device),
                                       rope_layout="halves", whole_norm=m.whole_norm, **paged)
        if T == 1:
            o = wa_ops.window_attention_decode(q[:, 0], ck, cv, q_start, m.scale, seq_ids=seq_ids, sinks=mixer.sink,
                                               **paged)
        elif (mixer.sink is None and T >= self.TC_PREFILL_MIN_TOKENS and not self._step_past_context
              and not self.kv_cache.paged and wa_ops.tc_prefill_applies(qkv, m.dim, m.vdim, big.shape[-1])):
            # prompts from position 0 without a sink term on the tcgen05 flash-attention kernel: K comes back from the cache
            # rows just written (normed and rotated), V is the value columns of the projection output, read in place
            lines = seq_ids.long() if seq_ids is not None else torch.arange(B, device=big.device)
            vx = qkv[..., (m.heads + m.kv_heads) * m.dim:].reshape(B, T, m.kv_heads, m.vdim)
            o = attn_ops.flash_attn_func(q.permute(0, 2, 1, 3), ck[lines, :, :T], vx.permute(0, 2, 1, 3),
                                         softmax_scale=m.scale, causal=True).permute(0, 2, 1, 3)
        else:
            o = wa_ops.window_attention_prefill(q, ck, cv, q_start, m.scale, n_new=n_new, seq_ids=seq_ids,
                                                sinks=mixer.sink, **paged)
        return gemm_nt(o.reshape(B * T, m.heads * m.vdim), mixer.o_proj.weight)

    def _retention(self, run, mixer, big, at, B, T, q_start, n_new, seq_ids):
        m, cfg, dt = mixer.cfg, self.config, self.config.torch_dtype
        H, D, Dv, N = m.heads, m.dim, m.vdim, B * T
        state = self.kv_cache.state(run)["S"]
        offsets = (at, at + H * D, at + 2 * H * D)
        step = ret_ops.retention_chunkwise if T >= self.CHUNKWISE_MIN_TOKENS else ret_ops.retention_scan
        o = step(big, offsets, mixer.decay, state, q_start, H, D, Dv, D ** -0.5,
                 rope=self._rotary_tables(m.rot, big.device), rope_layout="halves", n_new=n_new, seq_ids=seq_ids)
        y = mlstm_ops.head_norm_gate(o.reshape(N, H, Dv), big.view(N, -1), at + 2 * H * D + H * Dv, H, Dv, None,
                                     cfg.rms_norm_eps, True, dt, gate_act="silu")
        return gemm_nt(y, mixer.o_proj.weight)

    def _feed_forward(self, layer, h2: torch.Tensor) -> torch.Tensor:
        if layer.mlp_kind == "moe":
            return layer.mlp(h2)                                       # fp32 [N, W]
        mlp = layer.mlp
        gu = gemm_nt(h2, mlp.gate_up_proj.weight)
        act = moe_ops.glu_bias(gu, 0, mlp.ff_pad, mlp.ff, act="gelu_tanh")
        return gemm_nt(act, mlp.down_proj.weight)

    # -- one layer run ------------------------------------------------------------------------------------------------
    def _layer(self, i: int, layer, hidden, residual, positions, seq_ids, lengths, prefill):
        cfg, dt, eps = self.config, self.config.torch_dtype, self.config.rms_norm_eps
        B, T, SW = hidden.shape
        S, W, N = cfg.streams, cfg.hidden_size, B * T
        x = (hidden if hidden.is_contiguous() else hidden.contiguous()).view(N, S, W)
        h = (residual.reshape(N, W) if residual is not None else
             hc_ops.hc_step(x, in_w=layer.hc1_in, norm_w=layer.norm1, eps=eps, out_dtype=dt))
        if "q_start" not in self._step_kv:      # one int32 copy of the rows' first positions per step, not per kernel
            self._step_kv["q_start"] = positions[:, 0].to(torch.int32).contiguous()
        q_start = self._step_kv["q_start"]
        n_new = self._step_new_tokens if prefill else None
        big = gemm_nt(h, layer.in_proj.weight).view(B, T, -1)
        y2 = branch_w = None
        if layer.type == "attention":
            y = self._softmax_attention(i, layer.mixer, big, layer.columns["qkv"][0], B, T, q_start, n_new, seq_ids)
        else:
            y = self._softmax_attention(i, layer.mixer.left, big, layer.columns["left"][0], B, T, q_start, n_new, seq_ids)
            y2 = self._retention(i, layer.mixer.right, big, layer.columns["right"][0], B, T, q_start, n_new, seq_ids)
            branch_w = (layer.mixer.left_out, layer.mixer.right_out)
        nxt = self._sequence[i + 1] if i + 1 < len(self._sequence) else None
        in_next, norm_next = (nxt.hc1_in, nxt.norm1) if nxt is not None else (None, None)
        if layer.mlp is None:
            h_next = hc_ops.hc_step(x, y, layer.hc1_mix, layer.hc1_out, in_next, norm_next, eps, dt, y2=y2,
                                    branch_w=branch_w)
        else:
            h2 = hc_ops.hc_step(x, y, layer.hc1_mix, layer.hc1_out, layer.hc2_in, layer.norm2, eps, dt, y2=y2,
                                branch_w=branch_w)
            h_next = hc_ops.hc_step(x, self._feed_forward(layer, h2), layer.hc2_mix, layer.hc2_out, in_next, norm_next,
                                    eps, dt)
        if self.layer_probe is not None:
            self.layer_probe(i, x.sum(dim=1).view(B, T, W))
        return x.view(B, T, SW), (h_next.view(B, T, W) if h_next is not None else None)

    def forward_speculation(self, *a, **kw):
        raise NotImplementedError("the speculation verify graph is not wired for this family")
