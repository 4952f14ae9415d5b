"""Pre-allocated paged KV cache + block allocator.

Replaces the reference's per-step ``torch.cat`` cache growth (a full O(T) copy
and a fresh allocation per layer per token; gptj_modeling.py:229-233,
gpt_bigcode_modeling.py:288-289).  Layout per layer: ``[num_blocks, kv_heads_per_rank,
block_size, head_dim]`` for K and for V, sized once for the 180 GB of HBM3e.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List

import torch


class KVCache:
    def __init__(self, num_layers: int, num_blocks: int, block_size: int, kv_heads: int, head_dim: int, dtype, device):
        self.num_layers, self.num_blocks, self.block_size = num_layers, num_blocks, block_size
        self.kv_heads, self.head_dim = kv_heads, head_dim
        self.data = torch.zeros(num_layers, 2, num_blocks, kv_heads, block_size, head_dim, dtype=dtype, device=device)

    def k(self, layer: int) -> torch.Tensor:
        return self.data[layer, 0]

    def v(self, layer: int) -> torch.Tensor:
        return self.data[layer, 1]

    @staticmethod
    def bytes_per_block(num_layers, block_size, kv_heads, head_dim, dtype) -> int:
        return num_layers * 2 * block_size * kv_heads * head_dim * torch.empty((), dtype=dtype).element_size()

    def copy_blocks_from(self, old: "KVCache", src: int, dst: int, n: int):
        self.data[:, :, dst:dst + n] = old.data[:, :, src:src + n]


class LatentCache:
    """Paged cache of latent-attention layers: ONE vector per token and layer run (the RMS-normed down-projection
    from which keys and values of every head are re-derived), instead of a key and a value per head.

    ``ranks[i]`` is the latent width of layer run i -- a layer that is run several times (weight-shared loop) owns
    one plane per pass, since each pass sees different activations.  Plane layout ``[num_blocks, block_size, rank]``
    equals the multi-head layout ``[num_blocks, kv_heads = 1, block_size, head_dim = rank]``, so the same block
    tables, slot mapping and allocator serve it, and the multi-query tcgen05 kernels can read it."""

    def __init__(self, ranks, num_blocks: int, block_size: int, dtype, device):
        self.ranks, self.num_blocks, self.block_size = list(ranks), num_blocks, block_size
        self.num_layers = len(self.ranks)
        self.planes = [torch.zeros(num_blocks, block_size, r, dtype=dtype, device=device) for r in self.ranks]

    def latent(self, run: int) -> torch.Tensor:
        return self.planes[run]

    @staticmethod
    def bytes_per_block(ranks, block_size, dtype) -> int:
        return sum(ranks) * block_size * torch.empty((), dtype=dtype).element_size()

    def copy_blocks_from(self, old: "LatentCache", src: int, dst: int, n: int):
        for mine, theirs in zip(self.planes, old.planes):
            mine[dst:dst + n] = theirs[src:src + n]


class BlockAllocator:
    """Reference-counted free-list allocator over cache blocks (block 0 is reserved as the padding target).

    A block is held by every sequence whose block table names it (`share` adds a holder, `release` removes one).  A
    block whose last holder leaves returns to the free list -- unless it is *pinned as cached* (`keep`: a full prompt
    block registered in the prefix index), in which case it waits in an LRU of evictable blocks and is only reclaimed,
    oldest first, when the free list is empty (`on_evict(block)` tells the index)."""

    def __init__(self, num_blocks: int, reserve_first: bool = True):
        self.num_blocks = num_blocks
        first = 1 if reserve_first else 0
        self.free: List[int] = list(range(num_blocks - 1, first - 1, -1))
        self.ref = [0] * num_blocks
        self.kept = set()                         # blocks registered in a prefix index
        self.evictable: "OrderedDict[int, None]" = OrderedDict()   # kept blocks nobody holds, least recently used first
        self.on_evict = None

    @property
    def num_free(self) -> int:
        return len(self.free) + len(self.evictable)

    def alloc(self, n: int) -> List[int]:
        if n > self.num_free:
            raise MemoryError(f"KV cache exhausted: want {n} blocks, {self.num_free} free")
        out = []
        for _ in range(n):
            if self.free:
                b = self.free.pop()
            else:
                b, _ = self.evictable.popitem(last=False)
                self.kept.discard(b)
                if self.on_evict is not None:
                    self.on_evict(b)
            self.ref[b] = 1
            out.append(b)
        return out

    def share(self, block: int):
        """One more holder of a cached block (a sequence re-using a prompt prefix)."""
        self.ref[block] += 1
        self.evictable.pop(block, None)

    def keep(self, block: int):
        self.kept.add(block)

    def release(self, blocks: List[int]):
        for b in reversed(blocks):
            self.ref[b] -= 1
            assert self.ref[b] >= 0, f"block {b} released more often than held"
            if self.ref[b] == 0:
                if b in self.kept:
                    self.evictable[b] = None      # most recently used end
                else:
                    self.free.append(b)


class HybridCache:
    """Cache of models that mix attention layers with recurrent ones.

    Two kinds of storage behind one object: *pages* for the keys and values of attention layers -- planes
    ``[num_blocks, kv_heads, block_size, dk]`` and ``[num_blocks, kv_heads, block_size, dv]`` (key and value sizes may
    differ), addressed through the same block tables, slot mapping and ``BlockAllocator`` as ``KVCache`` -- and *state
    slots* for everything a sequence carries from token to token in constant size: recurrent states, the tails of short
    convolutions, the previous token or activation.  Every state tensor is ``[num_slots, *shape]``; a sequence owns row
    ``slot`` of all of them from its first token to its release (``SlotAllocator``).  States are not cleared when a slot
    changes hands: the kernels start from zeros whenever a sequence's first row is its position 0.

    A third kind of page serves latent-attention layers: one row ``[num_blocks, block_size, width]`` per token (the layout
    of ``LatentCache``), through the same block tables.

    ``kv_layers``: {layer key: (kv_heads, dk, dv)}; ``states``: {(layer key, name): (shape, dtype)}; ``latents``:
    {layer key: row width}."""

    def __init__(self, kv_layers, states, num_blocks: int, block_size: int, num_slots: int, dtype, device, latents=None):
        self.num_blocks, self.block_size, self.num_slots = num_blocks, block_size, num_slots
        self.kv_layers = dict(kv_layers)
        self.latent_layers = dict(latents or {})
        self.num_layers = len(self.kv_layers) + len(self.latent_layers)
        self.lplanes = {key: torch.zeros(num_blocks, block_size, w, dtype=dtype, device=device)
                        for key, w in self.latent_layers.items()}
        self.kplanes = {key: torch.zeros(num_blocks, h, block_size, dk, dtype=dtype, device=device)
                        for key, (h, dk, dv) in self.kv_layers.items()}
        self.vplanes = {key: torch.zeros(num_blocks, h, block_size, dv, dtype=dtype, device=device)
                        for key, (h, dk, dv) in self.kv_layers.items()}
        self.states = {key: torch.zeros(num_slots, *shape, dtype=dt, device=device) for key, (shape, dt) in states.items()}

    def k(self, layer) -> torch.Tensor:
        return self.kplanes[layer]

    def v(self, layer) -> torch.Tensor:
        return self.vplanes[layer]

    def latent(self, layer) -> torch.Tensor:
        return self.lplanes[layer]

    def state(self, layer, name: str) -> torch.Tensor:
        return self.states[(layer, name)]

    @staticmethod
    def bytes_per_block(kv_layers, block_size, dtype, latents=None) -> int:
        per_token = sum(h * (dk + dv) for h, dk, dv in kv_layers.values()) + sum((latents or {}).values())
        return per_token * block_size * torch.empty((), dtype=dtype).element_size()

    def state_bytes_per_slot(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.states.values())

    def copy_blocks_from(self, old: "HybridCache", src: int, dst: int, n: int):
        """Pages src..src+n of ``old`` become pages dst.. here; the state slots (same numbering) come along."""
        for key in self.kplanes:
            self.kplanes[key][dst:dst + n] = old.kplanes[key][src:src + n]
            self.vplanes[key][dst:dst + n] = old.vplanes[key][src:src + n]
        for key in self.lplanes:
            self.lplanes[key][dst:dst + n] = old.lplanes[key][src:src + n]
        for key, t in self.states.items():
            t.copy_(old.states[key])


class SlotAllocator:
    """Free list over the state slots of a HybridCache: one slot per live sequence."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self.free: List[int] = list(range(num_slots - 1, -1, -1))

    @property
    def num_free(self) -> int:
        return len(self.free)

    def alloc(self) -> int:
        if not self.free:
            raise MemoryError(f"no free state slot: all {self.num_slots} are held by live sequences")
        return self.free.pop()

    def release(self, slot: int):
        assert 0 <= slot < self.num_slots and slot not in self.free, f"state slot {slot} released twice"
        self.free.append(slot)
