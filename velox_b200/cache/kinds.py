"""Kinds of cache: how what a mixer asks for (its `cache_spec()`) is stored.

The cache manager knows pages, block tables and slots; it does not know what lies
in a page.  For every kind of need, a `CacheKind` says
  * whether it is kept in pages (one entry per position, found through the
    request's block table) or in a slot (fixed size per request),
  * for pages: the window (0: every position stays), the bytes of one page of one
    layer, how the storage of a group of layers is allocated, and what a layer's
    mixer is handed (`LayerCache`),
  * for slots: the tensor [slots, ...] of one layer and how a slot is cleared.
A kind is registered for the class of its spec (`register_cache_kind`), from
anywhere: a test registers a cache of one latent vector per position without
touching this package.  Keys and values in pages (`PagedKV`), one latent row per
position in pages (`PagedLatent`) and fixed-size state (`FixedState`) are registered here.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

from ..parts.base import CacheParts, FixedState, PagedKV, PagedLatent  # noqa: F401  (CacheParts: part of this module's interface)


@dataclass
class LayerCache:
    """What a layer's mixer gets: its group (index into the step context's
    groups, -1 for none), whether it writes, and its storage: `k_pool`/`v_pool`
    for keys and values, `state` for a slot kind, `pages` for a paged kind with a
    layout of its own.  A mixer made of several (its need was a `CacheParts`) gets
    its members' caches in `parts`."""
    group: int = -1
    writes: bool = True
    k_pool: Optional[torch.Tensor] = None
    v_pool: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    pages: Optional[torch.Tensor] = None
    parts: Optional[list] = None


class CacheKind:
    paged = True

    # -- kinds kept in pages ---------------------------------------------------
    def window(self, spec) -> int:
        """Positions a query still reads (0: all).  Pages behind it are given back."""
        return 0

    def keep_first(self, spec) -> int:
        """With a window: the first positions that stay readable all the same."""
        return 0

    def page_bytes(self, spec, page_size: int, element_bytes: int) -> int:
        """Bytes of one page of one layer."""
        raise NotImplementedError

    def allocate(self, spec, layers: int, num_pages: int, page_size: int, dtype, device) -> torch.Tensor:
        """Storage of a group of `layers` layers; its first dimension is the layer."""
        raise NotImplementedError

    def layer_cache(self, storage: Optional[torch.Tensor], index: int, group: int) -> LayerCache:
        """What layer `index` of the group's storage hands its mixer."""
        raise NotImplementedError

    def layer_cache_of(self, spec, storage: Optional[torch.Tensor], index: int, group: int,
                       page_size: int) -> LayerCache:
        """The same for kinds whose layout depends on the spec (the manager calls this one)."""
        return self.layer_cache(storage, index, group)

    # -- kinds kept in slots ---------------------------------------------------
    def allocate_state(self, spec, slots: int, device) -> torch.Tensor:
        raise NotImplementedError

    def clear_slot(self, state: torch.Tensor, slot: int) -> None:
        state[slot].zero_()


class PagedKVKind(CacheKind):
    """Keys and values of every position: [layer, K|V, page, kv head, offset in page,
    head_dim] (the reference keeps a K and a V pool [page, kv head, offset, head_dim]
    per layer, src/paged/pages.rs:62-74, 101-109).  Where a value has another size
    than a key, a layer's storage is flat: its K pool [page, kv head, offset, head_dim]
    followed by its V pool [page, kv head, offset, v_head_dim]."""

    def window(self, spec: PagedKV) -> int:
        return spec.window

    def keep_first(self, spec: PagedKV) -> int:
        return spec.keep_first if spec.window > 0 else 0

    def page_bytes(self, spec: PagedKV, page_size, element_bytes):
        return (spec.num_kv_heads * spec.head_dim + spec.value_heads * spec.value_dim) * page_size * element_bytes

    def allocate(self, spec: PagedKV, layers, num_pages, page_size, dtype, device):
        if spec.value_dim == spec.head_dim and spec.value_heads == spec.num_kv_heads:
            return torch.empty((layers, 2, num_pages, spec.num_kv_heads, page_size, spec.head_dim), dtype=dtype, device=device)
        cells = num_pages * page_size
        return torch.empty((layers, cells * (spec.num_kv_heads * spec.head_dim + spec.value_heads * spec.value_dim)),
                           dtype=dtype, device=device)

    def layer_cache(self, storage, index, group):
        if storage is None:
            return LayerCache(group, True)
        return LayerCache(group, True, storage[index, 0], storage[index, 1], None, storage[index])

    def layer_cache_of(self, spec: PagedKV, storage, index, group, page_size):
        if storage is None or storage.dim() != 2:
            return self.layer_cache(storage, index, group)
        k_row, v_row = spec.num_kv_heads * spec.head_dim, spec.value_heads * spec.value_dim
        cells = storage.shape[1] // (k_row + v_row)   # pages * page size
        flat = storage[index]
        k = flat[:cells * k_row].view(-1, spec.num_kv_heads, page_size, spec.head_dim)
        v = flat[cells * k_row:].view(-1, spec.value_heads, page_size, spec.value_dim)
        return LayerCache(group, True, k, v, None, flat)


class PagedLatentKind(CacheKind):
    """One row per position: [layer, page, 1, offset in page, width].  The mixer is handed the same tensor as
    `k_pool` and `v_pool` (and `pages`): an attention kernel reads it as one key/value head whose value is
    the first part of the key's row."""

    def window(self, spec: PagedLatent) -> int:
        return spec.window

    def page_bytes(self, spec: PagedLatent, page_size, element_bytes):
        return spec.width * page_size * element_bytes

    def allocate(self, spec: PagedLatent, layers, num_pages, page_size, dtype, device):
        return torch.empty((layers, num_pages, 1, page_size, spec.width), dtype=dtype, device=device)

    def layer_cache(self, storage, index, group):
        if storage is None:
            return LayerCache(group, True)
        return LayerCache(group, True, storage[index], storage[index], None, storage[index])


class FixedStateKind(CacheKind):
    paged = False

    def allocate_state(self, spec: FixedState, slots, device):
        return torch.zeros((slots,) + tuple(spec.shape), dtype=getattr(torch, spec.dtype), device=device)


_KINDS: Dict[type, CacheKind] = {}


def register_cache_kind(spec_class: type, kind: CacheKind) -> CacheKind:
    _KINDS[spec_class] = kind
    return kind


def unregister_cache_kind(spec_class: type) -> None:
    _KINDS.pop(spec_class, None)


def cache_kind(spec) -> CacheKind:
    for cls in type(spec).__mro__:
        if cls in _KINDS:
            return _KINDS[cls]
    raise TypeError("a layer asks for a cache of unknown kind %r; registered kinds: %s"
                    % (spec, sorted(c.__name__ for c in _KINDS)))


register_cache_kind(PagedKV, PagedKVKind())
register_cache_kind(PagedLatent, PagedLatentKind())
register_cache_kind(FixedState, FixedStateKind())
