"""``SparseMoE``: dropless inference feed-forward built from the MoE pieces of this package -- a ``RouterBiasedTopK``,
the grouped ``Experts`` (clamped gated activation, or the plain ``silu(gate) * up`` with ``limit=None``), optional
identity experts and an optional gated shared expert.  ``router_bias``: the router has a bias on its logits;
``renormalize``: the experts with the largest logits are chosen and weighted by the softmax over the chosen logits only.
``score="sigmoid"``: every expert's score is the sigmoid of its own logit.  ``weight_on_input``: the routing weight
multiplies the chosen expert's input instead of its output, ``sum_j expert_j(w_j h)``.  ``shared_gated=False``: the
shared expert is added as it is, without a sigmoid gate of its own.

Two execution paths over the same parameters:
  * pairs   every (token, choice) pair runs a GEMV against the chosen expert's weights, picked by the index ON THE
            DEVICE (``ops.moe_sparse``): no host round trip, CUDA-graph capturable; the path of token generation,
            where the reference's ``forward_selective_loading`` loops over tokens on the host
            (``modules/moe/expert_mlps.py:267-296``);
  * sorted  tokens are sorted by expert and every expert multiplies its own segment with a GEMM (the dropless
            ``forward_all_experts`` scheme of ``ExpertMLPs``), then one gather-combine kernel.
The combination (chosen experts, identity experts, shared expert times its sigmoid gate) is summed in fp32.
"""
from __future__ import annotations

from typing import Optional

import torch

from ...ops import moe_sparse
from .experts import Experts
from .moe_parallel_layers import LinearRouter
from .routing import RouterBiasedTopK

# pairs per expert above which the sorted GEMM path takes over from the per-pair GEMVs
SORTED_PATH_MIN_PAIRS_PER_EXPERT = 16.0


class SparseMoE(torch.nn.Module):
    def __init__(self, hidden_size: int, num_experts: int, top_k: int, intermediate_size: int, limit: float,
                 num_identity_experts: int = 0, affinity_scale: float = 1.0, shared_intermediate_size: int = 0,
                 shared_limit: Optional[float] = None, alpha: float = moe_sparse.GLU_ALPHA,
                 dtype: torch.dtype = torch.float32, device=None, router_bias: bool = False, renormalize: bool = False,
                 score: str = "softmax", weight_on_input: bool = False, shared_gated: bool = True):
        super().__init__()
        self.weight_on_input = weight_on_input
        dev = device if device is not None else torch.device("cpu")
        self.hidden_size, self.num_experts, self.top_k = hidden_size, num_experts, top_k
        if limit is None:            # plain silu(gate) * up: no clamp, unit slope, no shift of the linear half
            limit, alpha, self.up_shift = float("inf"), 1.0, 0.0
        else:
            self.up_shift = 1.0
        shift = self.up_shift
        self.limit, self.alpha = limit, alpha
        self.router = RouterBiasedTopK(num_experts, top_k, hidden_size, num_identity_experts, affinity_scale, device=dev,
                                       bias=router_bias, renormalize=renormalize, score=score)
        self.experts = Experts(num_experts, hidden_size, intermediate_size, True, None, dtype=dtype, device=dev,
                               glu_fn=lambda gu: moe_sparse.clamped_glu(gu, limit, alpha, shift))
        self.shared = None
        if shared_intermediate_size > 0:
            sl = shared_limit if shared_limit is not None else limit
            self.shared_limit = sl
            self.shared = Experts(1, hidden_size, shared_intermediate_size, True, None, dtype=dtype, device=dev,
                                  glu_fn=lambda gu: moe_sparse.clamped_glu(gu, sl, alpha, shift))
            self.shared_gate = LinearRouter(hidden_size, 1, dtype=torch.float32, device=dev) if shared_gated else None

    def _use_sorted(self, n_tokens: int) -> bool:
        # the sorted path reads the per-expert counts on the host: not while a CUDA graph is being captured
        if torch.cuda.is_available() and torch.cuda.is_current_stream_capturing():
            return False
        return n_tokens * self.top_k / max(self.num_experts, 1) >= SORTED_PATH_MIN_PAIRS_PER_EXPERT

    def forward(self, h: torch.Tensor, path: Optional[str] = None) -> torch.Tensor:
        """``h [N, W]`` (activation dtype) -> combined output ``[N, W]`` in fp32."""
        gated = self.shared is not None and self.shared_gate is not None
        idx, wts, sg = self.router.select(h, self.shared_gate.weight if gated else None)
        sorted_path = self._use_sorted(h.shape[0]) if path is None else path == "sorted"
        if sorted_path:
            return self._forward_sorted(h, idx, wts, sg)
        w_gu, w_d = self.experts.gate_up_proj.weight, self.experts.down_proj.weight
        in_scale = None
        if self.weight_on_input:            # the weight goes into the expert; the outputs are summed as they are
            in_scale, wts = wts, self._ones_like(wts)
        act = moe_sparse.gate_up_act(h, w_gu, idx, self.limit, self.alpha, self.up_shift, in_scale=in_scale)
        s_act = s_down = None
        if self.shared is not None:
            s_act = moe_sparse.gate_up_act(h, self.shared.gate_up_proj.weight, None, self.shared_limit, self.alpha,
                                           self.up_shift)
            s_down = self.shared.down_proj.weight[0]
        return moe_sparse.down_combine(act, w_d, idx, wts, h, s_act, s_down, sg)

    def _ones_like(self, wts: torch.Tensor) -> torch.Tensor:
        ones = getattr(self, "_ones", None)
        if ones is None or ones.shape != wts.shape or ones.device != wts.device:
            ones = self._ones = torch.ones_like(wts)
        return ones

    def _forward_sorted(self, h, idx, wts, sg):
        N, E, k = h.shape[0], self.num_experts, self.top_k
        flat = idx.reshape(-1).long()
        order = torch.argsort(flat, stable=True)                      # identity experts (index >= E) sort to the end
        counts = torch.bincount(flat.clamp(max=E), minlength=E + 1)[:E].tolist()    # the one host read of the layer
        n_real = sum(counts)
        token_of = order[:n_real] // k
        slot = torch.empty(N * k, dtype=torch.int32, device=h.device)
        slot[order] = torch.arange(N * k, dtype=torch.int32, device=h.device)
        xs = h[token_of]
        if self.weight_on_input:
            xs = (xs.float() * wts.reshape(-1)[order[:n_real]].unsqueeze(1)).to(h.dtype)
            wts = self._ones_like(wts)
        ys = torch.empty(n_real, h.shape[1], dtype=h.dtype, device=h.device)
        start = 0
        for e, n in enumerate(counts):
            if n:
                seg = xs[start:start + n].unsqueeze(0)
                ys[start:start + n] = self.experts(seg, expert_indices=torch.tensor([e], device=h.device))[0]
                start += n
        shared_out = self.shared(h.unsqueeze(0))[0] if self.shared is not None else None
        return moe_sparse.gather_combine(ys, slot.reshape(N, k), idx, wts, h, E, shared_out, sg)
