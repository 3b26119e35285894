"""Two mixers side by side on the same input: ``left_scale * left(h) + right_scale * right(h)``.

Any two registered mixers can be paired.  At most one of them may keep pages (the plan gives every
entry one cache group); their state tensors are simply listed one after the other, the left one's
first.
"""

from __future__ import annotations

from gllm_b200 import ops
from gllm_b200.parts.base import MIXERS, Mixer, MixerCache, build_part, register_mixer


@register_mixer("parallel")
class ParallelMixer(Mixer):
    def __init__(self, names, left, right, left_scale: float = 1.0, right_scale: float = 1.0):
        super().__init__(names)
        self.left: Mixer = build_part(MIXERS, left)
        self.right: Mixer = build_part(MIXERS, right)
        self.left_scale, self.right_scale = float(left_scale), float(right_scale)
        if self.left.kv_requirement() is not None and self.right.kv_requirement() is not None:
            raise ValueError("only one of two parallel mixers may keep cache pages")

    @property
    def graph_safe_portions(self):
        return self.left.graph_safe_portions and self.right.graph_safe_portions

    def _states_of(self, mixer):
        need = mixer.state_requirement()
        return () if need is None else (tuple(need) if isinstance(need, (tuple, list)) else (need,))

    def kernel_needs(self):
        needs: dict = {}
        for part in (self.left, self.right):
            for key, values in part.kernel_needs().items():
                needs.setdefault(key, set()).update(values)
        return needs

    def kv_requirement(self):
        return self.left.kv_requirement() or self.right.kv_requirement()

    def state_requirement(self):
        return (self._states_of(self.left) + self._states_of(self.right)) or None

    def expected_tensors(self):
        return {**self.left.expected_tensors(), **self.right.expected_tensors()}

    def load(self, get, dtype, device):
        self.left.load(get, dtype, device)
        self.right.load(get, dtype, device)

    def _cache_of(self, mixer, cache: MixerCache, first: int) -> MixerCache:
        count = len(self._states_of(mixer))
        states = tuple(cache.states[first:first + count])
        keeps_pages = mixer.kv_requirement() is not None
        return MixerCache(group=cache.group if keeps_pages else None, pages=cache.pages if keeps_pages else None,
                          writes=cache.writes, state=states[0] if states else None, states=states,
                          requirement=cache.requirement if keeps_pages else None, block_size=cache.block_size)

    def forward(self, x, ctx, cache):
        sink, ctx.residual_sink = getattr(ctx, "residual_sink", None), None     # the branches are scaled first
        left = ops.as_tensor(self.left.forward(x, ctx, self._cache_of(self.left, cache, 0)))
        right = ops.as_tensor(self.right.forward(x, ctx, self._cache_of(self.right, cache, len(self._states_of(self.left)))))
        ctx.residual_sink = sink
        return ops.scaled_sum(left, right, self.left_scale, self.right_scale)
