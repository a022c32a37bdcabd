"""Routed feed-forward (mixture of experts): ``num_experts`` small feed-forwards without biases, of which every
token uses ``top``.

    z = W_r h (+ b with ``router_bias``)                 router, computed in float32
    s = sigmoid(z), or softmax(z) over all router outputs (``router_score``); "softmax_chosen": s = z chooses, and the
        weights are the softmax over the chosen z alone
    c = s + correction                                   the choice scores (``correction``: a learned vector; else c = s)
    ``groups`` = (count, keep): the router outputs form ``count`` equal groups of neighbours, a group's score is its
        largest c, and only members of the ``keep`` best groups can be chosen
    chosen = the ``top`` outputs of largest c (the lower index wins a tie)
    w_e = s_e, or s_e / sum over the chosen when ``renormalize``
    weight_on "input":   out = sum_e f_e(w_e h)          weight_on "output":  out = sum_e w_e f_e(h)
    f_e(x) = down_e( act(gate_e(x)) * up_e(x) )          ``gated`` (activation "silu" or "gelu_tanh")
    f_e(x) = down_e( act(up_e(x)) )                      not gated (activation "relu2", the square of relu)

The last ``identity_experts`` router outputs have no tensors: f_e(x) = x.  ``shared_intermediate`` > 0 adds one more
expert of the same form that every token uses with weight 1 (tensors under ``names["shared"]``).

The experts' tensors are ``<prefix>.e<i>.{gate,up,down}`` and the router ``<prefix>.router`` unless ``names`` says
otherwise; they are stacked into [E, 2 ff, hidden] (gate and up; [E, ff, hidden] when not gated) and [E, hidden, ff]
when loaded, and the tokens of a step are sorted by expert on the device (kernels/library.py ``routed_mlp``): nothing of
it waits for the host."""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import FeedForward, WeightSpec, MATRIX, VECTOR


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    ACTIVATIONS = ("silu", "gelu_tanh")
    PLAIN_ACTIVATIONS = ("relu2",)

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, activation: str = "silu",
                 renormalize: bool = False, weight_on: str = "output", gated: bool = True, router_score: str = "sigmoid",
                 correction: bool = False, groups=None, identity_experts: int = 0, shared_intermediate: int = 0,
                 router_bias: bool = False, names=None, prefix: str = ""):
        super().__init__(prefix)
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.num_experts, self.top = int(num_experts), int(top)
        self.identity_experts = int(identity_experts)
        self.outputs = self.num_experts + self.identity_experts          # what the router scores
        if self.num_experts <= 0 or self.identity_experts < 0:
            raise ValueError("num_experts must be positive and identity_experts not negative")
        if not 0 < self.top <= self.outputs:
            raise ValueError(f"top ({self.top}) must lie in 1 .. experts + identity experts ({self.outputs})")
        self.gated = bool(gated)
        allowed = self.ACTIVATIONS if self.gated else self.PLAIN_ACTIVATIONS
        if activation not in allowed:
            raise ValueError(f"activation of {'gated' if self.gated else 'plain'} experts must be one of {allowed}, got '{activation}'")
        if weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be 'input' or 'output', got '{weight_on}'")
        if router_score not in ("sigmoid", "softmax", "softmax_chosen"):
            raise ValueError(f"router_score must be 'sigmoid', 'softmax' or 'softmax_chosen', got '{router_score}'")
        self.router_bias = bool(router_bias)
        self.activation, self.renormalize, self.weight_on = activation, bool(renormalize), weight_on
        self.router_score, self.correction = router_score, bool(correction)
        count, keep = (int(v) for v in groups) if groups is not None else (1, 1)
        if count < 1 or not 1 <= keep <= count or self.outputs % count or self.top > keep * (self.outputs // count):
            raise ValueError(f"groups ({count}, keep {keep}) must divide the {self.outputs} router outputs evenly and "
                             f"leave at least top ({self.top}) of them")
        self.groups = (count, keep)
        self.shared_intermediate = int(shared_intermediate)
        self.names = {"router": "router", "router_bias": "router.b", "expert": "e{}", "gate": "gate", "up": "up", "down": "down",
                      "correction": "correction", "shared": "shared"}
        self.names.update(names or {})
        self.w_router = self.w_gate_up = self.w_down = self.correction_w = self.router_bias_w = None
        self.shared_up = self.shared_down = None
        self.gate_up_layout = "blocked"

    def _expert(self, e: int, which: str) -> str:
        return f"{self.names['expert'].format(e)}.{self.names[which]}"

    def _shared(self, which: str) -> str:
        return f"{self.names['shared']}.{self.names[which]}"

    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = {self.names["router"]: WeightSpec((self.outputs, self.hidden_size), MATRIX)}
        if self.correction:
            s[self.names["correction"]] = WeightSpec((self.outputs,), VECTOR, init="normal", init_scale=0.05)
        if self.router_bias:
            s[self.names["router_bias"]] = WeightSpec((self.outputs,), VECTOR, init="normal", init_scale=0.5)
        for e in range(self.num_experts):
            if self.gated:
                s[self._expert(e, "gate")] = WeightSpec((self.intermediate_size, self.hidden_size), MATRIX)
            s[self._expert(e, "up")] = WeightSpec((self.intermediate_size, self.hidden_size), MATRIX)
            s[self._expert(e, "down")] = WeightSpec((self.hidden_size, self.intermediate_size), MATRIX)
        if self.shared_intermediate > 0:
            if self.gated:
                s[self._shared("gate")] = WeightSpec((self.shared_intermediate, self.hidden_size), MATRIX)
            s[self._shared("up")] = WeightSpec((self.shared_intermediate, self.hidden_size), MATRIX)
            s[self._shared("down")] = WeightSpec((self.hidden_size, self.shared_intermediate), MATRIX)
        return s

    def load(self, tensors, ops, act_dtype) -> None:
        def all_of(*which):
            ts = [[tensors[self._expert(e, w)] for e in range(self.num_experts)] for w in which]
            same = all(t.dtype == ts[0][0].dtype for l in ts for t in l)
            return [[t if same else t.to(torch.float32) for t in l] for l in ts]
        self.w_router = tensors[self.names["router"]]
        if self.correction:
            self.correction_w = tensors[self.names["correction"]].to(torch.float32).contiguous()
        if self.router_bias:
            self.router_bias_w = tensors[self.names["router_bias"]].to(torch.float32).contiguous()
        if self.gated:
            gates, ups = all_of("gate", "up")
            # one tensor for gate and up of all experts; the kernel library chooses how their rows are laid out
            self.w_gate_up, self.gate_up_layout = ops.stack_gate_up(gates, ups)
        else:
            self.w_gate_up, self.gate_up_layout = torch.stack(all_of("up")[0], dim=0).contiguous(), "plain"
        self.w_down = torch.stack(all_of("down")[0], dim=0).contiguous()
        if self.shared_intermediate > 0:
            if self.gated:
                g, u = tensors[self._shared("gate")], tensors[self._shared("up")]
                dt = g.dtype if g.dtype == u.dtype else torch.float32
                self.shared_up = ops.merge_gate_up(g.to(dt), u.to(dt))
            else:
                self.shared_up = tensors[self._shared("up")]
            self.shared_down = tensors[self._shared("down")]

    def _router(self):
        if (self.router_score, self.correction_w, self.groups, self.identity_experts, self.router_bias_w) == \
                ("sigmoid", None, (1, 1), 0, None):
            return None
        return dict(score=self.router_score, correction=self.correction_w, groups=self.groups,
                    identity=self.identity_experts, bias=self.router_bias_w)

    def forward(self, h, ctx, residual):
        ops = ctx.ops
        target = residual
        if target is None:
            target = torch.empty((h.shape[0], self.hidden_size), dtype=torch.float32, device=h.device)
        ops.routed_mlp(h, self.w_router, self.w_gate_up, self.gate_up_layout, self.w_down, residual, self.top,
                       self.renormalize, self.weight_on, self.activation, out=None if residual is not None else target,
                       router=self._router())
        if self.shared_intermediate > 0:              # one more expert that every token uses, added to the sum
            if self.gated:
                ops.gated_mlp(h, self.shared_up, self.shared_down, target, self.shared_intermediate,
                              activation=self.activation)
            else:
                ops.plain_mlp(h, self.shared_up, self.shared_down, target, self.activation)
        return target
