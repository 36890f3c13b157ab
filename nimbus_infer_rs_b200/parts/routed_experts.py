"""A feed-forward of routed experts."""
from __future__ import annotations

import torch

from ..csrc.ops import GATE_ACTIVATIONS, GLU_ACTIVATIONS, PARAM_ACTIVATIONS
from .base import MATRIX, VECTOR, FeedForward, ParamSpec, register_part
from .feed_forward import GatedMLP
from .linear import Linear


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    """``residual += sum_{e in chosen} s_e * down_e(act(gate_e h) * (up_e h))``, or, with
    ``gated=False``, ``s_e * down_e(act(up_e h))`` (experts of two matrices).

    ``s = softmax(router h)`` over all ``n_experts`` in fp32; the ``top`` experts with the
    largest scores are chosen per token (of equal scores the lower index); their weights are
    their own scores, divided by the chosen scores' sum only if ``renormalize``.  Experts have
    no biases; ``activation`` is the gate's (``silu``, ``gelu_tanh``, ``gelu_erf``, ``none``).

    ``scores="sigmoid"`` is another way to choose: ``s = sigmoid(router h)``; the choice score of
    an expert is ``s_e + correction_e`` (a learned number per expert, if ``correction``); with
    ``groups`` > 1 the experts form that many equal groups of neighbours, a group's score is the
    sum of its ``group_top`` largest choice scores, and only experts of the ``keep_groups`` best
    groups can be chosen (of equal scores the lower group); the ``top`` largest choice scores
    win; the weights are the winners' ``s`` (without the correction), with ``renormalize``
    divided by ``sum + norm_eps``, times ``route_scale``.  Gated experts may combine their halves
    by ``swish_clamp`` with the bound ``limit`` (``parts/feed_forward.py``).  With ``shared`` (a
    mapping with ``hidden``, ``activation``, ``limit``) one more gated feed-forward of that size
    runs for every token and is added; the router's weight rows then ride on that expert's first
    product (the rows under its gate and up halves), and this part has no router product.

    The router's logits are a product of the same rows as the mixer's projections in a block
    whose sublayers share one norm; ``router_from_mixer`` then reads them from the columns the
    mixer's fused projection appended for it (``ctx.shared_projection``) and this part has no
    router product of its own, only the router's weight rows inside that projection.

    The step's (token, choice) pairs are grouped by expert on the device; a tiled product per
    group runs the gated first half, another the second half, and the weighted results are added
    into the stream in the order of the choices.  Nothing comes back to the host.
    """
    graph_safe = True

    def __init__(self, width: int, n_experts: int, top: int, hidden: int, activation: str = "silu",
                 renormalize: bool = False, router_from_mixer: bool = False, gated: bool = True,
                 scores: str = "softmax", correction: bool = False, groups: int = 1,
                 keep_groups: int = 1, group_top: int = 2, route_scale: float = 1.0,
                 norm_eps: float = 0.0, limit: float | None = None, shared: dict | None = None):
        known = GLU_ACTIVATIONS if gated else GATE_ACTIVATIONS
        if activation not in known:
            raise ValueError(f"unknown activation {activation!r} (have {sorted(known)})")
        if (limit is not None) != (activation in PARAM_ACTIVATIONS):
            raise ValueError(f"activation {activation!r} and limit={limit!r} do not go together")
        if scores not in ("softmax", "sigmoid"):
            raise ValueError(f"scores={scores!r}: softmax or sigmoid")
        if scores == "softmax" and (correction or groups > 1 or route_scale != 1.0):
            raise ValueError("a choice bias, groups and a scale belong to sigmoid scores")
        self.scores, self.has_correction = scores, bool(correction)
        self.groups, self.keep_groups, self.group_top = int(groups), int(keep_groups), int(group_top)
        if self.groups > 1 and (int(n_experts) % self.groups or not 1 <= self.keep_groups <= self.groups
                                or self.keep_groups * (int(n_experts) // self.groups) < int(top)):
            raise ValueError(f"{groups} groups (keep {keep_groups}) do not fit {n_experts} experts, top={top}")
        self.route_scale, self.norm_eps = float(route_scale), float(norm_eps)
        self.act_param = float(limit) if limit is not None else 0.0
        # the shared expert's first product also gives the router's logits (one read of the rows)
        self.router_from_shared = bool(shared) and not router_from_mixer
        self.shared = None if not shared else GatedMLP(
            int(width), int(shared["hidden"]), shared.get("activation", activation),
            shared.get("limit"), extra_outputs=int(n_experts) if self.router_from_shared else 0)
        self.width, self.n_experts, self.top, self.hidden = int(width), int(n_experts), int(top), int(hidden)
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"top={top} of {n_experts} experts")
        self.activation = activation
        self.act_code = GLU_ACTIVATIONS[activation]
        self.renormalize = bool(renormalize)
        self.router_from_mixer = bool(router_from_mixer)
        self.gated = bool(gated)
        self.router = None if (self.router_from_mixer or self.router_from_shared) \
            else Linear(self.width, self.n_experts, bias=False)
        self.gate = self.up = self.down = self.correction = None

    def children(self):
        out = {} if self.router is None else {"router": self.router}
        if self.shared is not None:
            out["shared"] = self.shared
        return out

    def param_specs(self):
        e, f, d = self.n_experts, self.hidden, self.width
        specs = {"up": ParamSpec((e, f, d), MATRIX), "down": ParamSpec((e, d, f), MATRIX)}
        if self.gated:
            specs["gate"] = ParamSpec((e, f, d), MATRIX)
        if self.has_correction:
            specs["correction"] = ParamSpec((e,), VECTOR)
        return specs

    can_overwrite = True

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        if self.shared is not None:
            # the shared expert first: it can write over the buffer, the chosen ones add to it
            self.shared.forward(ctx, h, residual, accumulate=accumulate)
        elif not accumulate:
            residual.zero_()
        lay, ops, dev = ctx.layout, ctx.ops, h.device
        n, top = lay.n_rows, self.top
        if self.router_from_mixer or self.router_from_shared:
            logits, col = ctx.shared_projection
        else:
            logits, col = self.router(ctx, h, out_dtype=torch.float32), 0
        idx = torch.empty((n, top), device=dev, dtype=torch.int32)
        weight = torch.empty((n, top), device=dev, dtype=torch.float32)
        if self.scores == "sigmoid":
            ops.moe_route_sigmoid(logits, col, self.correction, self.n_experts, top, self.groups,
                                  self.keep_groups, self.group_top, self.renormalize, self.norm_eps,
                                  self.route_scale, lay, idx, weight)
        else:
            ops.moe_route(logits, col, self.n_experts, top, self.renormalize, lay, idx, weight)
        offsets = torch.empty(self.n_experts + 1, device=dev, dtype=torch.int32)
        order = torch.empty(n * top, device=dev, dtype=torch.int32)
        place = torch.empty(n * top, device=dev, dtype=torch.int32)
        ops.moe_group(idx, self.n_experts, offsets, order, place)
        mid = torch.empty((n * top, self.hidden), device=dev, dtype=ctx.rt.act_dtype)
        if self.gated:
            ops.moe_linear(h, order, top, offsets, self.gate, self.up, mid, self.act_code,
                           self.act_param)
        else:
            ops.moe_linear(h, order, top, offsets, self.up, None, mid, self.act_code)
        y = torch.empty((n * top, self.width), device=dev, dtype=torch.float32)
        ops.moe_linear(mid, None, 1, offsets, self.down, None, y)
        ops.moe_combine(y, place, weight, residual)
