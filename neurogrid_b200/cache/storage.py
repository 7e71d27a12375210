"""Device memory behind the cache manager's bookkeeping.

Layers with the same need share a group.  A paged group holds, for each of its layers,
keys and values as ``[pages, n_kv_heads, page_size, head_dim]`` in the compute dtype; one
page id is valid in every layer of its group.  Pages of a need without values have no value half.  A slot group holds ``[layers, slots, *shape]``
in the element type its need names, set to the need's initial value when a request starts.  The reference keeps one pool per attention layer in fp16
(gpu/cuda/paged_attention.cu:34-67) and conv states on the host between steps.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .manager import PagedNeed, SlotNeed


_SLOT_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16, "int32": torch.int32}


@dataclass
class LayerCache:
    kind: str                 # "paged" | "slot" | "none"
    group: int = -1           # index among groups of its kind
    index: int = -1           # layer's index inside the group


class CacheStorage:
    def __init__(self, needs: Sequence[object], *, pages_per_group, page_size: int, max_requests: int,
                 dtype: torch.dtype, device):
        """``needs`` maps a cache id to its PagedNeed / SlotNeed / None.  ``pages_per_group`` is
        an int (every paged group gets that many pages) or a callable ``need -> pages``."""
        self.page_size, self.dtype, self.device = page_size, dtype, device
        self.paged_needs: List[PagedNeed] = []
        self.slot_needs: List[SlotNeed] = []
        self.layers: Dict[int, LayerCache] = {}
        counts_p: List[int] = []
        counts_s: List[int] = []
        def place(need) -> LayerCache:
            if need is None:
                return LayerCache("none")
            if isinstance(need, PagedNeed):
                if need not in self.paged_needs:
                    self.paged_needs.append(need)
                    counts_p.append(0)
                g = self.paged_needs.index(need)
                counts_p[g] += 1
                return LayerCache("paged", g, counts_p[g] - 1)
            if isinstance(need, SlotNeed):
                if need not in self.slot_needs:
                    self.slot_needs.append(need)
                    counts_s.append(0)
                g = self.slot_needs.index(need)
                counts_s[g] += 1
                return LayerCache("slot", g, counts_s[g] - 1)
            raise TypeError(f"a layer declared an unknown cache need: {need!r}")

        # a layer that keeps several things declares a tuple of needs and is handed a tuple of views
        for cid in sorted(needs):
            need = needs[cid]
            self.layers[cid] = tuple(place(n) for n in need) if isinstance(need, tuple) else place(need)
        self.pages_per_group = [pages_per_group(n) if callable(pages_per_group) else int(pages_per_group)
                                for n in self.paged_needs]
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        for need, n_layers, pages in zip(self.paged_needs, counts_p, self.pages_per_group):
            shape = (n_layers, pages, need.n_kv_heads, page_size, need.head_dim)
            vh, vd = need.value_shape()
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros((n_layers, pages, vh, page_size, vd), dtype=dtype, device=device)
                          if need.values else None)
        for need in self.slot_needs:
            if need.dtype not in _SLOT_DTYPES:
                raise TypeError(f"a layer asks for state of dtype {need.dtype!r}; one of {sorted(_SLOT_DTYPES)}")
        self.state: List[torch.Tensor] = [
            torch.full((n_layers, max_requests) + tuple(need.shape), need.init, dtype=_SLOT_DTYPES[need.dtype],
                       device=device)
            for need, n_layers in zip(self.slot_needs, counts_s)]

    def reset_slot(self, slot: int) -> None:
        """Every layer's state of the slot back to its need's initial value (a request starts)."""
        for s, need in zip(self.state, self.slot_needs):
            s[:, slot].fill_(need.init)

    def bytes_per_token(self) -> int:
        esz = torch.empty((), dtype=self.dtype).element_size()
        return sum(k.shape[0] * n.elements_per_token() * esz for k, n in zip(self.k, self.paged_needs))

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v + self.state if t is not None)
