"""Dense gated feed-forward: down(act(gate(x)) * up(x)), no biases; act is SiLU (SwiGLU) or the
tanh form of GELU.

gate and up are one packed projection [gate | up]
(tinyvllm/models/qwen3.py:316-346; activation tinyvllm/kernels/pointwise.cu:274-285).

A block that computes the input projections of all its parts as one product, and their output
projections as one product too, builds the part with ``hosted=True``: the part then declares no
matrices of its own, tells the block which checkpoint tensors make up its share
(``input_rows``, ``output_cols``) and only turns its columns of the common projection into
its columns of the common input of the output product (``between``).
"""

from __future__ import annotations

from ..ops import kernels, linear, linear_into_stream, linear_norm, linear_silu
from .base import BuildContext, ParamSpec, Part
from .registry import register_part


class SwiGLU(Part):
    def __init__(self, ctx: BuildContext, *, hidden_size: int, intermediate_size: int,
                 names: dict | None = None, activation: str = "silu", hosted: bool = False) -> None:
        if activation not in kernels.ACTIVATIONS:
            raise ValueError(f"activation is one of {', '.join(kernels.ACTIVATIONS)}, not {activation!r}")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation = activation
        self.hosted = hosted
        n = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight",
             **(names or {})}
        self.names = {key: f"{ctx.prefix}.{value}" for key, value in n.items()}
        self.gate_up_weight = self.down_weight = None

    def param_specs(self):
        if self.hosted:
            return []
        return [
            ParamSpec.packed("gate_up_weight", [(self.names["gate"], self.intermediate_size),
                                                (self.names["up"], self.intermediate_size)],
                             self.hidden_size),
            ParamSpec.single("down_weight", self.names["down"],
                             (self.hidden_size, self.intermediate_size)),
        ]

    def streamed_weights(self):
        return [] if self.hosted else [self.gate_up_weight, self.down_weight]

    # ------------------------------------------------- as a guest of a block
    def input_rows(self):
        """(checkpoint tensor, rows) of the input projections, in the order of their columns."""
        return [(self.names["gate"], self.intermediate_size), (self.names["up"], self.intermediate_size)]

    def output_cols(self):
        """(checkpoint tensor, columns) of the output projection."""
        return (self.names["down"], self.intermediate_size)

    def between(self, projected, at: int, ctx, out) -> None:
        """act(gate) * up from the columns ``at ...`` of the common projection into ``out``."""
        kernels.gated_act(projected, at, at + self.intermediate_size, self.intermediate_size,
                          self.activation, out=out)

    # ------------------------------------------------------------ on its own
    def _activated(self, x):
        if self.activation == "silu":
            return linear_silu(x, self.gate_up_weight)
        return kernels.gated_act(linear(x, self.gate_up_weight), 0, self.intermediate_size,
                                 self.intermediate_size, self.activation)

    def forward(self, x, ctx):
        return linear(self._activated(x), self.down_weight)

    def forward_normed(self, hidden, residual, norm, ctx):
        """forward(norm(hidden + residual)) and the new residual stream; the output is None when
        the down projection has added it to the stream itself."""
        if self.activation != "silu":
            if hidden is None:
                x = norm.forward(residual)
            elif residual is None:
                x, residual = norm.forward(hidden), hidden
            else:
                x, residual = norm.add(hidden, residual)
            return self.forward(x, ctx), residual
        activated, residual = linear_norm(hidden, residual, norm, self.gate_up_weight, silu=True)
        return linear_into_stream(activated, self.down_weight, residual)


register_part("feed_forward", "swiglu", SwiGLU)
register_part("feed_forward", "gated_mlp", SwiGLU)
