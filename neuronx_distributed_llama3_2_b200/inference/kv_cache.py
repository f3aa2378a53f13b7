"""KV cache state for the inference graphs (reference keeps the cache as aliased parameters of the compiled
graph and re-emits the whole cache every step, ``examples/inference/modules/model_base.py:114-125,388-422``).

Here the cache is a plain device allocation per layer that the kernels update IN PLACE:
  contiguous  ``[lines, kv_heads_local, seq_len, head_dim]``
  paged       ``[pages, kv_heads_local, page_size, head_dim]`` + a block table ``[lines, max_pages]``

Paged mode has two flavours: the static identity mapping (every line owns ``max_pages`` pages up front) and, with
``num_pages``, a POOL smaller than ``lines * max_pages`` managed by the native page allocator
(``runtime.native.PagedKVPool``): lines get pages as they grow (``reserve``), give them back (``free``), can be forked
copy-on-write (``fork``) and rolled back (``truncate``).  The block table is a device tensor updated in place, so CUDA
graphs that captured it see the new mapping.

Layers need not be alike: ``layer_specs[i] = (kv_heads, key_dim, value_dim)`` gives layer ``i`` its own shapes (key and
value sizes may differ), and ``share_from[i] = j`` makes layer ``i`` read layer ``j``'s keys and values instead of
holding its own (cross-layer KV sharing: ``layer(i)`` returns ``j``'s tensors, nothing is allocated for ``i``).
A spec ``(kv_heads, key_dim, value_dim, "columns")`` keeps ONE tensor per layer whose value is the first ``value_dim``
columns of the key rows (the latent cache of a compressed key/value projection); a spec ``None`` is a layer without
keys and values; a spec ``(kv_heads, key_dim, value_dim, "heads", value_heads)`` gives the value tensor its own number
of heads (several attention maps -- key heads -- over the same values).

Recurrent layers keep a STATE per cache line instead: ``state_specs[i] = {name: shape}`` allocates fp32 tensors
``[lines, *shape]`` (``state(i)``).  State is per line, not per page: ``fork`` copies it, and a layer that starts a
sequence at position 0 starts from zero by itself, so a line that is handed out again needs no clearing.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional, Tuple

import torch


class KVCache:
    def __init__(self, num_layers: int, lines: int, kv_heads: int, seq_len: int, head_dim: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, paged: bool = False, page_size: int = 128,
                 num_pages: Optional[int] = None, layer_specs: Optional[List[Optional[Tuple[int, int, int]]]] = None,
                 share_from: Optional[Dict[int, int]] = None,
                 state_specs: Optional[Dict[int, Dict[str, Tuple[int, ...]]]] = None):
        self.num_layers, self.lines, self.kv_heads, self.seq_len, self.head_dim = num_layers, lines, kv_heads, seq_len, head_dim
        self.share_from = dict(share_from or {})
        for i, j in self.share_from.items():
            if j in self.share_from or not (0 <= j < num_layers) or j == i:
                raise ValueError(f"layer {i} cannot share the keys/values of layer {j}")
        specs = layer_specs if layer_specs is not None else [(kv_heads, head_dim, head_dim)] * num_layers
        self.paged, self.page_size = paged, page_size
        self.pool = None
        if paged:
            self.max_pages = (seq_len + page_size - 1) // page_size
            if num_pages is None:
                n_pages = lines * self.max_pages
                # static identity mapping: every line owns its pages up front
                self.block_table = torch.arange(n_pages, dtype=torch.int32, device=device).reshape(lines, self.max_pages)
            else:
                from ..runtime.native import PagedKVPool

                n_pages = num_pages
                self.pool = PagedKVPool(n_pages, page_size, lines, self.max_pages)
                self.block_table = torch.zeros(lines, self.max_pages, dtype=torch.int32, device=device)
            lead, rows = n_pages, page_size
        else:
            lead, rows = lines, seq_len
            self.block_table = None
        self.k: List[Optional[torch.Tensor]] = []
        self.v: List[Optional[torch.Tensor]] = []
        for i in range(num_layers):
            if i in self.share_from:
                self.k.append(None)
                self.v.append(None)
                continue
            if specs[i] is None:                       # a layer without keys and values (recurrent state only)
                self.k.append(None)
                self.v.append(None)
                continue
            g, dk, dv = specs[i][:3]
            self.k.append(torch.zeros((lead, g, rows, dk), dtype=dtype, device=device))
            if len(specs[i]) > 3 and specs[i][3] == "columns":
                self.v.append(self.k[-1][..., :dv])    # the values are columns of the key rows: one tensor
            elif len(specs[i]) > 4 and specs[i][3] == "heads":
                self.v.append(torch.zeros((lead, int(specs[i][4]), rows, dv), dtype=dtype, device=device))
            else:
                self.v.append(torch.zeros((lead, g, rows, dv), dtype=dtype, device=device))
        self.states: Dict[int, Dict[str, torch.Tensor]] = {
            i: {name: torch.zeros((lines,) + tuple(shape), dtype=torch.float32, device=device)
                for name, shape in spec.items()} for i, spec in (state_specs or {}).items()}

    def owns(self, i: int) -> bool:
        """False for a layer that reads another layer's keys and values."""
        return i not in self.share_from

    def layer(self, i: int) -> Tuple[torch.Tensor, torch.Tensor]:
        i = self.share_from.get(i, i)
        return self.k[i], self.v[i]

    def state(self, i: int) -> Dict[str, torch.Tensor]:
        """The recurrent state tensors ``[lines, ...]`` (fp32) of layer ``i``."""
        return self.states[i]

    def _tensors(self) -> List[torch.Tensor]:
        """Every allocation once (a value tensor that is a column range of its key tensor is not one)."""
        out = []
        for t in self.k + self.v:
            if t is not None and t._base is None:
                out.append(t)
        return out

    def _state_tensors(self) -> List[torch.Tensor]:
        return [t for d in self.states.values() for t in d.values()]

    def reset(self) -> None:
        for t in self._tensors() + self._state_tensors():
            t.zero_()
        if self.pool is not None:
            for line in range(self.lines):
                self.pool.free_line(line)
            self.block_table.zero_()

    # -- dynamic page pool (no-ops for the contiguous cache and the static mapping) ---------------------------------------
    def sync_lines(self, lines: Iterable[int]) -> None:
        """Copy the allocator's page lists of ``lines`` into the device block table."""
        if self.pool is None:
            return
        rows = list(lines)
        if not rows:
            return
        host = torch.tensor([self.pool.block_row(r)[0] for r in rows], dtype=torch.int32)
        self.block_table[torch.tensor(rows, dtype=torch.long, device=self.block_table.device)] = host.to(
            self.block_table.device, non_blocking=True)

    def reserve(self, line: int, n_tokens: int) -> None:
        """Room for ``n_tokens`` tokens in total on ``line`` (``MemoryError`` when the pool is exhausted)."""
        if self.pool is not None and self.pool.reserve(line, n_tokens) > 0:
            self.sync_lines([line])

    def free(self, line: int) -> None:
        if self.pool is not None:
            self.pool.free_line(line)

    def truncate(self, line: int, n_tokens: int) -> None:
        if self.pool is not None and self.pool.truncate(line, n_tokens) > 0:
            self.sync_lines([line])

    def _copy_page(self, src: int, dst: int) -> None:
        for t in self._tensors():
            t[dst].copy_(t[src])

    def fork(self, src: int, dst: int) -> None:
        """``dst`` continues from ``src``'s content: full pages shared, the partial last page copied."""
        assert self.pool is not None, "fork needs the dynamic page pool (num_pages=...)"
        copy = self.pool.fork(src, dst)
        if copy is not None:
            self._copy_page(*copy)
        for t in self._state_tensors():
            t[dst].copy_(t[src])
        self.sync_lines([dst])

    def prepare_write(self, line: int, pos: int) -> None:
        """Before writing position ``pos`` of ``line``: give the line a private copy of that page if it is shared."""
        if self.pool is None:
            return
        copy = self.pool.unshare(line, pos)
        if copy is not None:
            self._copy_page(*copy)
            self.sync_lines([line])

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self._tensors() + self._state_tensors())
