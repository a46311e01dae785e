"""Feed-forward parts.  ``swiglu``: andre-fu/prism's dense MLP
(engine/executor.py:125-127): fused gate/up projection, ``silu(gate) * up``,
down projection; no biases (engine/weight_pool.py:194-199).  ``mlp``: up
projection, an elementwise activation, down projection."""

from __future__ import annotations

from .base import DetachedProjection, FeedForward, ParamSpec, WeightSource, register_part
from .. import ops


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """``names``: the gate, up and down tensors' names in the model file."""

    def __init__(self, hidden_size: int, intermediate_size: int,
                 names=("gate_proj.weight", "up_proj.weight", "down_proj.weight")):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.names = tuple(names)

    def params(self):
        H, I = self.hidden_size, self.intermediate_size
        return [
            ParamSpec("gate_up_w", (WeightSource(self.names[0], (I, H)),
                                    WeightSource(self.names[1], (I, H)))),
            ParamSpec("down_w", (WeightSource(self.names[2], (H, I)),)),
        ]

    def forward(self, ctx, x):
        return ops.feed_forward_swiglu(ctx, x, self.w["gate_up_w"], self.w["down_w"])


@register_part("feed_forward", "mlp")
class ActMLP(FeedForward):
    """``down(act(up(x)))`` without gate.  ``activation``: one of ``ops.ACTIVATIONS`` (``relu2``: the square of
    relu; ``gelu_tanh``; ``silu``; ``relu``).  ``names``: the up and down tensors' names in the model file."""

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "relu2",
                 names=("up_proj.weight", "down_proj.weight")):
        if activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {activation!r}: one of {sorted(ops.ACTIVATIONS)}")
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        self.activation = activation
        self.names = tuple(names)
        self._own_up = self._own_down = True

    detachable_out = detachable_in = True

    def _sources(self):
        H, I = self.hidden_size, self.intermediate_size
        return WeightSource(self.names[0], (I, H)), WeightSource(self.names[1], (H, I))

    def params(self):
        up, down = self._sources()
        return ([ParamSpec("up_w", (up,))] if self._own_up else []) + ([ParamSpec("down_w", (down,))] if self._own_down else [])

    def detach_out_projection(self):
        self._own_down = False
        return DetachedProjection(self.handed_over(self._sources()[1]), (), self.intermediate_size)

    def detach_in_projection(self):
        self._own_up = False
        return DetachedProjection(self.handed_over(self._sources()[0]), (), self.intermediate_size)

    def forward_inner(self, ctx, x, out, proj=None):
        ops.feed_forward_hidden(ctx, x, self.w.get("up_w"), self.activation, out, hidden=proj)

    def forward(self, ctx, x):
        return ops.feed_forward_act(ctx, x, self.w["up_w"], self.w["down_w"], self.activation)
