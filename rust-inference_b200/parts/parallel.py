"""Two mixers side by side: both read the same input, and the result is left_scale * left + right_scale * right.

The sum is not taken here: the part returns a :class:`~.base.WeightedSum`, and the connection to the residual
(``parts/link.py``) adds the two terms with their factors in float32 while the next norm reads the stream, so neither
output is rounded a second time.  The children's tensors carry the prefixes "left." and "right."; what they ask of the
cache is put together into one request (keys and values of the one, state of the other, in this order), and each child
is handed its own share.
"""
from __future__ import annotations

from dataclasses import replace

from .base import CacheRequest, Mixer, WeightedSum
from .registry import build_part, part_class, register_mixer

_SIDES = ("left", "right")


@register_mixer("parallel")
class ParallelMixer(Mixer):

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.left = build_part("mixer", spec.left, env)
        self.right = build_part("mixer", spec.right, env)
        self._requests = [self.left.cache_request(), self.right.cache_request()]
        if sum(1 for r in self._requests if r is not None and r.kv_heads > 0) > 1:
            raise ValueError("two mixers side by side that both keep keys and values are not built")

    @property
    def graph_safe(self):
        return self.left.graph_safe and self.right.graph_safe

    @property
    def position(self):
        return getattr(self.left, "position", None) or getattr(self.right, "position", None)

    @classmethod
    def param_infos(cls, spec):
        infos = {}
        for side in _SIDES:
            record = getattr(spec, side)
            for local, info in part_class("mixer", record).param_infos(record).items():
                infos[f"{side}.{local}"] = info
        return infos

    def load(self, tensors):
        for side in _SIDES:
            pre = side + "."
            getattr(self, side).load({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})

    def weight_bytes(self):
        return self.left.weight_bytes() + self.right.weight_bytes()

    def reads_first(self):
        return self.left.reads_first()

    def prepare(self, max_positions):
        self.left.prepare(max_positions)
        self.right.prepare(max_positions)

    @staticmethod
    def _states(r):
        if r is None:
            return []
        own = [(tuple(r.state_shape), r.state_dtype)] if r.state_shape else []
        return own + [(tuple(s), d) for s, d in r.more_state]

    def cache_request(self):
        kv = next((r for r in self._requests if r is not None and r.kv_heads > 0), None)
        states = self._states(self._requests[0]) + self._states(self._requests[1])
        if kv is None and not states:
            return None
        first = states[0] if states else ((), None)
        return CacheRequest(kv_heads=kv.kv_heads if kv else 0, head_dim=kv.head_dim if kv else 0,
                            window=kv.window if kv else 0, chunk=kv.chunk if kv else 0,
                            shared_kv=kv.shared_kv if kv else False, state_shape=first[0],
                            state_dtype=first[1] if states else CacheRequest().state_dtype, more_state=tuple(states[1:]))

    def _share(self, cache, which):
        """The part of the layer's cache entry that child ``which`` asked for."""
        r = self._requests[which]
        tensors = ([cache.state] if cache.state is not None else []) + list(cache.more_state)
        start = len(self._states(self._requests[0])) if which == 1 else 0
        mine = tensors[start:start + len(self._states(r))]
        has_kv = r is not None and r.kv_heads > 0
        return replace(cache, k_pool=cache.k_pool if has_kv else None, v_pool=cache.v_pool if has_kv else None,
                       page_table=cache.page_table if has_kv else None, state=mine[0] if mine else None,
                       more_state=tuple(mine[1:]))

    def __call__(self, x, ctx, cache):
        left = self.left(x, ctx, self._share(cache, 0))
        right = self.right(x, ctx, self._share(cache, 1))
        return WeightedSum(((left, float(self.spec.left_scale)), (right, float(self.spec.right_scale))))
