"""Gated feed-forward: down(act(gate(x)) * up(x)) with one fused [gate; up] matrix
(mstar/model/components/distributed/mlp.py:78-81; gate is shard 0, up shard 1); act is the
SiLU or the tanh form of gelu.  With ``bias`` the three products add one: the first product
is then taken in float, bias, activation and multiplication are one kernel, and the down
product's bias travels with the output (``OutputWithBias``) to whatever adds it to the
residual."""
from __future__ import annotations

import torch

from .. import ops
from ..weights.names import ParamSpec
from .base import Runtime
from .registry import register_part


class OutputWithBias:
    """A sublayer's output ``y + bias`` with the bias not added yet: a block whose kernel adds
    the output to the residual takes the bias along; ``materialize()`` adds it here."""

    def __init__(self, y: torch.Tensor, bias: torch.Tensor):
        self.y, self.bias = y, bias
        self.shape, self.dtype = y.shape, y.dtype

    def materialize(self) -> torch.Tensor:
        return self.y + self.bias.to(self.y.dtype)


class GatedMLP:
    graph_safe = True       # nothing per-step is read from the host

    @classmethod
    def param_specs(cls, spec) -> dict:
        out = {
            "gate_up.weight": ParamSpec((2 * spec.intermediate_size, spec.hidden_size)),
            "down.weight": ParamSpec((spec.hidden_size, spec.intermediate_size)),
        }
        if getattr(spec, "bias", False):
            out["gate_up.bias"] = ParamSpec((2 * spec.intermediate_size,), role="vector",
                                            init="zeros")
            out["down.bias"] = ParamSpec((spec.hidden_size,), role="vector", init="zeros")
        return out

    def __init__(self, spec, params: dict, runtime: Runtime):
        self.gate_up_bias = self.down_bias = None
        if getattr(spec, "bias", False):
            self.gate_up_bias = params["gate_up.bias"].contiguous()
            self.down_bias = params["down.bias"].contiguous()
        if spec.activation not in ops.GATE_ACTIVATIONS:
            raise ValueError(f"gated_mlp activation {spec.activation!r} has no kernel "
                             f"({sorted(ops.GATE_ACTIVATIONS)} have)")
        self.spec = spec
        self.runtime = runtime
        self.gate_up = params["gate_up.weight"]
        self.down = params["down.weight"]

    def forward(self, x, ctx):
        if self.gate_up_bias is not None:
            gu = ops.linear(x, self.gate_up, out_dtype=torch.float32, static_weights=True)
            h = ops.bias_act_mul(gu, self.gate_up_bias, self.runtime.dtype, self.spec.activation)
            return OutputWithBias(ops.linear(h, self.down, static_weights=True), self.down_bias)
        return ops.linear(ops.gated_up(x, self.gate_up, static_weights=True,
                                       kind=self.spec.activation), self.down, static_weights=True)


class MLP:
    """down(act(up(x))) without a gate; the activation (relu squared, tanh gelu or silu) is
    a kernel of its own between the two products, or, for a few rows and relu squared, the
    epilogue of the first."""

    graph_safe = True

    @classmethod
    def param_specs(cls, spec) -> dict:
        return {
            "up.weight": ParamSpec((spec.intermediate_size, spec.hidden_size)),
            "down.weight": ParamSpec((spec.hidden_size, spec.intermediate_size)),
        }

    def __init__(self, spec, params: dict, runtime: Runtime):
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"mlp activation {spec.activation!r} has no kernel "
                             f"({sorted(ops.ACTIVATIONS)} have)")
        self.spec = spec
        self.runtime = runtime
        self.up = params["up.weight"]
        self.down = params["down.weight"]

    def forward(self, x, ctx):
        h = ops.linear_act(x, self.up, self.spec.activation, static_weights=True)
        return ops.linear(h, self.down, static_weights=True)


register_part("ffn", "gated_mlp", GatedMLP)
register_part("ffn", "mlp", MLP)
