"""The device side of the cache: one tensor per cache id.

A paged cache whose keys and values have one width is ``[num_pages, 2 (keys, values), kv_heads,
page_size, head_dim]`` in the model's type: the rows of one page and head lie together
(``page_size * head_dim`` contiguous elements), so a kernel fetches a page's keys for one head as
one contiguous run.  With different widths a page holds its keys ``[kv_heads, page_size, key_dim]``
and behind them its values ``[kv_heads, page_size, value_dim]``; ``CacheStorage[c]`` is then the
flat ``[num_pages, elements per page]`` tensor and ``keys(c)`` / ``values(c)`` are views of the two
halves (for equal widths they are ``[c][:, 0]`` and ``[c][:, 1]``).  The attention kernels of this
package take equal widths only.  Caches of one group are indexed by the same page ids.  Inside a
row (the ``head_dim`` values of one position and head) the 16-byte chunks are permuted by the position (``kv_swizzle`` in csrc/common.cuh, mirrored by
``kernels.ops.kv_swizzle``): a page copied into shared memory as it is, by one bulk copy, can then be
read by the tensor-core loads without bank conflicts.  Only the kernels (and tests that fill a cache
by hand) know of the permutation.  A state cache is ``[num_slots, *shape]``.

The reference keeps two tensors per layer, keys packed ``[blocks, kvh, hd/x, bs, x]`` and values
``[blocks, kvh, hd, bs]`` (src/kv_cache/cache_engine.cpp:66-102), a layout made for scalar loads.
"""

from __future__ import annotations

import torch

from .manager import CacheManager, PagedCacheSpec, StateCacheSpec


def paged_cache_bytes_per_page(spec: PagedCacheSpec, page_size: int, dtype: torch.dtype) -> int:
    return (spec.num_kv_heads * page_size * (spec.key_dim + spec.value_dim)
            * torch.empty((), dtype=dtype).element_size())


def bytes_per_page(cache_specs, page_size: int, dtype: torch.dtype) -> int:
    """Bytes one page id costs over all paged caches (every group gets the same number of pages)."""
    return sum(paged_cache_bytes_per_page(s, page_size, dtype) for s in cache_specs if isinstance(s, PagedCacheSpec))


class CacheStorage:
    def __init__(self, manager: CacheManager, dtype: torch.dtype, device: torch.device | str):
        self.tensors: list[torch.Tensor | None] = []
        self.specs = list(manager.cache_specs)
        self.page_size = manager.page_size
        for cache_id, spec in enumerate(manager.cache_specs):
            if isinstance(spec, PagedCacheSpec):
                pages = manager.groups[manager.group_of_cache[cache_id]].pool.num_pages
                # Zeros, not empty: the null page is read by nothing, but a debugger should see zeros there.
                if spec.key_dim == spec.value_dim:
                    shape = (pages, 2, spec.num_kv_heads, manager.page_size, spec.key_dim)
                else:
                    shape = (pages, spec.num_kv_heads * manager.page_size * (spec.key_dim + spec.value_dim))
                self.tensors.append(torch.zeros(shape, dtype=dtype, device=device))
            elif isinstance(spec, StateCacheSpec):
                self.tensors.append(torch.zeros((manager.max_requests, *spec.shape),
                                                dtype=getattr(torch, spec.dtype), device=device))
            else:
                self.tensors.append(None)

    def __getitem__(self, cache_id: int) -> torch.Tensor | None:
        return self.tensors[cache_id]

    def keys(self, cache_id: int) -> torch.Tensor:
        """[num_pages, kv_heads, page_size, key_dim]: a view of the pages' key halves."""
        spec, tensor = self.specs[cache_id], self.tensors[cache_id]
        if spec.key_dim == spec.value_dim:
            return tensor[:, 0]
        split = spec.num_kv_heads * self.page_size * spec.key_dim
        return tensor[:, :split].view(tensor.shape[0], spec.num_kv_heads, self.page_size, spec.key_dim)

    def values(self, cache_id: int) -> torch.Tensor:
        """[num_pages, kv_heads, page_size, value_dim]: a view of the pages' value halves."""
        spec, tensor = self.specs[cache_id], self.tensors[cache_id]
        if spec.key_dim == spec.value_dim:
            return tensor[:, 1]
        split = spec.num_kv_heads * self.page_size * spec.key_dim
        return tensor[:, split:].view(tensor.shape[0], spec.num_kv_heads, self.page_size, spec.value_dim)

    def reset_state_slot(self, manager: CacheManager, slot: int) -> None:
        """A slot that a new request takes starts from zero."""
        for cache_id in manager.state_cache_ids:
            self.tensors[cache_id][slot].zero_()

    def poison_pages(self, manager: CacheManager, group: int, pages: list[int]) -> None:
        """Fill given-back pages with NaN (tests: a kernel that reads a page it should not shows up)."""
        live = [p for p in pages if p != 0]
        if not live:
            return
        index = torch.tensor(live, dtype=torch.long, device=self.tensors[manager.groups[group].cache_ids[0]].device)
        for cache_id in manager.groups[group].cache_ids:
            self.tensors[cache_id].index_fill_(0, index, float("nan"))
