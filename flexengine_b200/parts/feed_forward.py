"""Feed-forwards: the dense gated one, down( act(gate(h)) * up(h) ), act = silu (SwiGLU) or the tanh form of GELU; the dense
one without a gate, down( act(up(h)) ), act = xIELU or the square of relu; and the routed one (a mixture of experts of either form).

Formula: tests/unit/test_synthetic_qwen.py:30-36 of the reference (its product code
calls the module opaquely, src/flexengine/inference/models/qwen2.py:130).  gate and up
are held as one [2I, H] matrix so that one product feeds the activation kernel.
"""
from __future__ import annotations

from .base import FeedForward, register_feed_forward


class SwiGLU(FeedForward):
    takes_prenormed = True

    ACTIVATIONS = ("silu", "gelu_tanh")

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "silu", bias: bool = False):
        self.hidden_size = int(hidden_size)
        self.intermediate_size = int(intermediate_size)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"unknown gate activation {activation!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.activation = activation
        self.has_bias = bool(bias)
        self.gate_up_weight = None
        self.down_weight = None
        self.gate_up_bias = self.down_bias = None
        if self.has_bias:
            self.takes_prenormed = False

    def parameter_shapes(self) -> dict:
        h, i = self.hidden_size, self.intermediate_size
        shapes = {"gate_up.weight": ((2 * i, h), "matrix"), "down.weight": ((h, i), "matrix")}
        if self.has_bias:
            shapes.update({"gate_up.bias": ((2 * i,), "vector"), "down.bias": ((h,), "vector")})
        return shapes

    def reads_first(self):
        return self.gate_up_weight

    def forward(self, ctx, h, follow=None, upcoming=None, defer_bias=False):
        """``defer_bias``: the caller adds the last product's bias itself (a norm's kernel that reads the output next);
        (rows in float32, bias) come back."""
        if self.has_bias:
            ops = ctx.ops
            # the products stay float32 until their biases are in: one rounding each
            gate_up = ops.linear(h, self.gate_up_weight, None, out_float32=True)
            act = ops.gated_activation(gate_up, self.intermediate_size, self.activation, bias=self.gate_up_bias, out_dtype=ctx.dtype)
            if defer_bias:
                return ops.linear(act, self.down_weight, None, out_float32=True), self.down_bias
            return ops.linear(act, self.down_weight, self.down_bias)
        if self.activation != "silu":
            act = ctx.ops.linear_gated(h, self.gate_up_weight, self.intermediate_size, self.activation)
            return ctx.ops.linear(act, self.down_weight)
        if follow is None and upcoming is None:
            return ctx.ops.linear(ctx.ops.linear_swiglu(h, self.gate_up_weight, self.intermediate_size), self.down_weight)
        # a decode step on kernels that take the hints: each product is told which matrix is streamed after it
        act = ctx.ops.linear_swiglu(h, self.gate_up_weight, self.intermediate_size, upcoming=self.down_weight)
        return ctx.ops.linear(act, self.down_weight, follow=follow, upcoming=upcoming)


class ActivatedMlp(FeedForward):
    """down( act(up(h)) ), one matrix up, one down, no gate.  ``activation``:
    "xielu": two-sided, with two learned numbers p, q (``act``): z > 0: softplus(p) z^2 + z/2;
             z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2;
    "relu2": the square of relu(z)."""

    ACTIVATIONS = ("xielu", "relu2")
    takes_prenormed = False

    def __init__(self, hidden_size: int, intermediate_size: int, activation: str = "xielu"):
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        if activation not in self.ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r}; known: {', '.join(self.ACTIVATIONS)}")
        self.activation = activation
        self.up_weight = self.down_weight = self.act = None

    def parameter_shapes(self) -> dict:
        h, i = self.hidden_size, self.intermediate_size
        shapes = {"up.weight": ((i, h), "matrix"), "down.weight": ((h, i), "matrix")}
        if self.activation == "xielu":
            shapes["act"] = ((2,), "vector")
        return shapes

    def reads_first(self):
        return self.up_weight

    def forward(self, ctx, h):
        ops = ctx.ops
        if self.activation == "xielu":
            return ops.linear(ops.activation(ops.linear(h, self.up_weight), "xielu", self.act), self.down_weight)
        # the product's epilogue squares where a kernel of this package takes the product; else product, then activation
        return ops.linear(ops.linear_activated(h, self.up_weight, self.activation), self.down_weight)


class RoutedExperts(FeedForward):
    """A mixture of small gated feed-forward layers: every token runs its ``top`` best experts of ``experts``.

    Router logits z = W_router h and s = softmax(z) over all experts in float32; the ``top`` largest s are
    chosen and used as weights, times ``scale``, not renormalised; the output is the weighted sum of the chosen
    experts' down( silu(gate h) * up h ), plus a shared expert of the same form (size ``shared_size``, 0 for
    none) that every token runs.  Tokens are sorted by expert on the device and each expert multiplies its own
    rows (``ops.routed_experts``): no count ever comes back to the host, so the step can be a CUDA graph."""

    ROUTERS = ("softmax_all", "softmax_chosen")
    ACTIVATIONS = ("silu", "clamped", "relu2")

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, scale: float = 1.0, shared_size: int = 0,
                 router: str = "softmax_all", activation: str = "silu", limit: float = 0.0, identity: int = 0,
                 correction: bool = False, groups: int = 1, keep: int = 1):
        """``router`` "softmax_all": as above; "softmax_chosen": the ``top`` largest logits are chosen and the weights are
        the softmax over the chosen logits only.  ``activation`` "silu": as above; "clamped": with g = min(gate h, limit)
        and u = clamp(up h, -limit, limit) an expert is down( g * sigmoid(1.702 g) * (u + 1) ); "relu2": an expert has no
        gate and is down( relu(up h)^2 ).
        ``identity``: the router has that many further outputs, after the experts', that stand for experts which return
        their input (times the weight); they have no tensors.  ``correction``: a learned number per router output is added
        to the scores for the choice only; the weights are the uncorrected scores.  ``groups``, ``keep``: the router's
        outputs form ``groups`` equal groups of neighbours, a group's score is its largest (corrected) score, and only
        outputs of the ``keep`` best groups can be chosen."""
        self.hidden_size, self.experts, self.top = int(hidden_size), int(experts), int(top)
        self.expert_size, self.scale, self.shared_size = int(expert_size), float(scale), int(shared_size)
        if router not in self.ROUTERS or activation not in self.ACTIVATIONS:
            raise ValueError(f"router {router!r} / activation {activation!r}: known are {self.ROUTERS} and {self.ACTIVATIONS}")
        if activation == "clamped" and not limit > 0.0:
            raise ValueError("the clamped activation needs a positive limit")
        self.router, self.activation, self.limit = router, activation, float(limit)
        self.identity, self.correction, self.groups, self.keep = int(identity), bool(correction), int(groups), int(keep)
        outputs = self.experts + self.identity
        if self.identity < 0 or self.groups < 1 or outputs % self.groups or not (1 <= self.keep <= self.groups):
            raise ValueError("the groups must share the router's outputs out equally, and 1 <= keep <= groups")
        if (self.correction or self.groups > 1) and router != "softmax_all":
            raise ValueError("a correction and groups go with the softmax over all router outputs")
        if self.shared_size and activation == "relu2":
            raise ValueError("the shared expert is a gated one")
        self.router_weight = self.router_correction = self.experts_gate_up_weight = self.experts_up_weight = self.experts_down_weight = None
        self.shared_gate_up_weight = self.shared_down_weight = None

    def parameter_shapes(self) -> dict:
        h, e, f = self.hidden_size, self.experts, self.expert_size
        shapes = {"router.weight": ((e + self.identity, h), "float32"), "experts.down.weight": ((e * h, f), "matrix")}
        if self.activation == "relu2":
            shapes["experts.up.weight"] = ((e * f, h), "matrix")
        else:
            shapes["experts.gate_up.weight"] = ((e * 2 * f, h), "matrix")
        if self.correction:
            shapes["router.correction"] = ((e + self.identity,), "vector")
        if self.shared_size:
            shapes["shared.gate_up.weight"] = ((2 * self.shared_size, h), "matrix")
            shapes["shared.down.weight"] = ((h, self.shared_size), "matrix")
        return shapes

    def reads_first(self):
        return self.router_weight

    def forward(self, ctx, h):
        ops = ctx.ops
        e, f, d = self.experts, self.expert_size, self.hidden_size
        logits = ops.linear(h, self.router_weight, None, out_float32=True)
        shared = None
        if self.shared_size:
            shared = ops.linear(ops.linear_swiglu(h, self.shared_gate_up_weight, self.shared_size), self.shared_down_weight)
        down = self.experts_down_weight.view(e, d, f)
        if self.activation == "relu2" or self.identity or self.correction or self.groups > 1:
            chosen, weights = ops.route_top(logits, self.top, self.scale, over_chosen=self.router == "softmax_chosen",
                                            correction=self.router_correction, groups=(self.groups, self.keep))
            first = self.experts_up_weight.view(e, f, d) if self.activation == "relu2" else self.experts_gate_up_weight.view(e, 2 * f, d)
            return ops.routed_experts(h, chosen, weights, first, down, shared, activation=self.activation, limit=self.limit,
                                      identity=self.identity)
        gate_up = self.experts_gate_up_weight.view(e, 2 * f, d)
        if self.router == "softmax_all" and self.activation == "silu":
            chosen, weights = ops.route_top(logits, self.top, self.scale)
            return ops.routed_experts(h, chosen, weights, gate_up, down, shared)
        chosen, weights = ops.route_top(logits, self.top, self.scale, over_chosen=self.router == "softmax_chosen")
        return ops.routed_experts(h, chosen, weights, gate_up, down, shared, activation=self.activation, limit=self.limit)


register_feed_forward("swiglu", SwiGLU)
register_feed_forward("gated_mlp", SwiGLU)
register_feed_forward("xielu_mlp", ActivatedMlp)
register_feed_forward("mlp", ActivatedMlp)
register_feed_forward("routed_experts", RoutedExperts)
