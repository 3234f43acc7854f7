"""Feed-forward parts.  ``MLP``: ``down(act(up(x)))`` with biases, the dense
two-matrix form of mlx_lm/models/gpt2.py:71-80 with the inner width and the
activation as parameters; the activation runs in the first product's
epilogue and the residual add in the second's."""

from __future__ import annotations

from .base import FeedForward, Init, register_part
from .linear import ACTIVATIONS, Linear


class MLP(FeedForward):
    replayable = True
    def __init__(self, name: str, width: int, inner: int, activation: str = "gelu_new", bias: bool = True,
                 stored: str = "out_in", up_name: str = "c_fc", down_name: str = "c_proj", init: Init = Init(),
                 bias_init: Init = Init()):
        if activation not in ACTIVATIONS:
            raise ValueError(f"{name}: activation {activation!r} is not one of {sorted(a for a in ACTIVATIONS if a)}")
        self.name, self.width, self.inner, self.activation = name, width, inner, activation
        self.up = Linear(f"{name}.{up_name}", width, inner, bias, stored, init=init, bias_init=bias_init)
        self.down = Linear(f"{name}.{down_name}", inner, width, bias, stored, init=init, bias_init=bias_init)

    def children(self):
        return (self.up, self.down)

    def fold_input_norm(self, norm) -> bool:
        return self.up.fold_norm(norm)

    def forward(self, ctx, x, residual):
        h = self.up.forward(ctx, x, ctx.ws.get("ffn_hidden", x.shape[0], self.inner, x.dtype),
                            activation=self.activation)
        return self.down.forward(ctx, h, residual, residual=residual)


register_part("feed_forward", "mlp", MLP)
