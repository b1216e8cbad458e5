"""Generation with a persistent compressed KV cache, shared by the family adapters that support it."""

from __future__ import annotations


class CompressedCacheMixin:
    """Adds `_attend_cached` to an adapter: `apply_turboquant(..., kv_cache_capacity=n)` sets
    `kv_cache_capacity`, and the adapter's `forward` calls `_attend_cached` instead of compressing and attending
    over the new tokens alone when HF hands it a cache object."""
    SUPPORTS_KV_CACHE = True
    kv_cache_capacity: int | None = None  # set by apply_turboquant(..., kv_cache_capacity=n)

    def _attend_cached(self, q, k, v, past_key_values, attention_mask):
        """Generation with a persistent compressed cache (no counterpart in the reference, whose adapters run
        with `use_cache = False`).  The HF cache object only keeps count of the positions (it is fed one channel
        of each key and value, so that `cache_position` and the rotary or learned positions advance as usual)
        and tells one generation from the next: a cache object this layer has not seen starts a new sequence."""
        import weakref

        from ..kv_cache import CompressedKVCache
        B, Hkv, T, D = k.shape
        owner = getattr(self, "_tq_owner", None)
        cache = getattr(self, "_tq_cache", None)
        seen = int(past_key_values.get_seq_length(self.layer_idx))
        if owner is None or owner() is not past_key_values:
            # A cache object this layer has not met starts a new sequence -- but only an EMPTY one can: the
            # compressed tokens of a pre-filled HF cache (a resumed generation, a second generation interleaved
            # with the first, assisted decoding) live nowhere, and attending over the new tokens alone would be
            # silently wrong.
            if seen != 0:
                raise RuntimeError(
                    f"layer {self.layer_idx}: the HF cache handed over already holds {seen} positions that this "
                    "layer's compressed cache never saw (the compressed cache follows one generation at a time; "
                    "start each generation from an empty cache object and do not interleave generations)")
            if cache is None or (cache.batch, cache.kv_heads) != (B, Hkv) or cache.key_indices.device != k.device:
                cache = CompressedKVCache(self.key_compressor, self.val_compressor, B, Hkv, self.kv_cache_capacity,
                                          device=k.device)
                self._tq_cache = cache
            cache.reset()
            self._tq_owner = weakref.ref(past_key_values)
        elif seen != cache.length:
            raise RuntimeError(f"layer {self.layer_idx}: the HF cache holds {seen} positions but the compressed cache "
                               f"{cache.length}; cache reordering or cropping (beam search, rollback) is not supported")
        cache.append(k, v)
        past_key_values.update(k[..., :1], v[..., :1], self.layer_idx)
        return cache.attend(q, causal=True, attention_mask=attention_mask)
