"""A feed-forward of routed experts beside a shared expert.

``num_experts`` gated feed-forwards (W_down (silu(W_gate x) * (W_up x)), no biases), of which each
token uses ``top``.  Router: z = W_router x in float32, scores s = sigmoid(z) or (``score``
"softmax") softmax(z) over all experts.  The choice is made on s + correction (a stored vector),
the weights use s without it.  The experts form ``group_count`` equal groups of neighbours; a
group's score is the sum of its ``group_top`` largest choice scores (2, or 1: its largest), and only
experts of the ``group_keep`` best groups can be chosen (the others count as minus infinity).  The
``top`` largest choice scores win; their weights are their scores s over the sum of those
(+ ``weight_eps``), times ``route_scale``, or (``normalize`` off) s times ``route_scale``.  The
output is the weighted sum of the chosen experts' outputs plus, when there is a shared expert, its
output, times sigmoid(W_sg x) (one number per token) when ``shared_gate`` is on.
"""

from __future__ import annotations

from typing import Optional

import torch

from ..kernels import ops
from .base import FeedForward
from .registry import register_feed_forward
from .spec import TensorSpec


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, ctx, prefix: str, hidden_size: int, intermediate_size: int, num_experts: int, top: int,
                 route_scale: float, group_count: int = 1, group_keep: int = 1,
                 shared_intermediate_size: Optional[int] = None, weight_eps: float = 1e-20,
                 names: Optional[dict] = None, score: str = "sigmoid", group_top: int = 2, normalize: bool = True,
                 shared_gate: bool = True):
        if score not in ops.ROUTER_SCORES or int(group_top) not in (1, 2):
            raise ValueError(f"routed_experts: score {score!r} ({sorted(ops.ROUTER_SCORES)}) or group_top "
                             f"{group_top!r} (1, 2) is not known")
        if num_experts % group_count or group_keep > group_count or top > group_keep * (num_experts // group_count):
            raise ValueError(f"routed_experts: {num_experts} experts in {group_count} groups, {group_keep} kept, "
                             f"{top} chosen do not fit")
        self.prefix = prefix
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.num_experts, self.top = int(num_experts), int(top)
        self.route_scale, self.weight_eps = float(route_scale), float(weight_eps)
        self.group_count, self.group_keep = int(group_count), int(group_keep)
        self.shared_size = None if shared_intermediate_size is None else int(shared_intermediate_size)
        self.score, self.group_top, self.normalize = score, int(group_top), bool(normalize)
        self.shared_gate = bool(shared_gate) and self.shared_size is not None
        self.names = dict(expert="e{}.", gate="gate", up="up", down="down", router="router",
                          correction="correction", shared="shared.", shared_gate="shared.sg")
        self.names.update(names or {})
        self.out_dtype = ctx.dtype
        self.w_router = self.correction = self.w_gate_up = self.w_down = None
        self.shared_gate_up = self.shared_down = None

    def tensor_specs(self):
        p, n, w, f = self.prefix, self.names, self.hidden_size, self.intermediate_size
        specs = []
        for e in range(self.num_experts):
            q = p + n["expert"].format(e)
            specs += [TensorSpec(q + n["gate"], (f, w)), TensorSpec(q + n["up"], (f, w)),
                      TensorSpec(q + n["down"], (w, f))]
        specs += [TensorSpec(p + n["router"], (self.num_experts, w)),
                  TensorSpec(p + n["correction"], (self.num_experts,), role="vector", init="normal")]
        if self.shared_size is not None:
            q, s = p + n["shared"], self.shared_size
            specs += [TensorSpec(q + n["gate"], (s, w)), TensorSpec(q + n["up"], (s, w)),
                      TensorSpec(q + n["down"], (w, s))]
            if self.shared_gate:
                specs.append(TensorSpec(p + n["shared_gate"], (1, w)))
        return specs

    def load(self, tensors):
        p, n = self.prefix, self.names
        names = [p + n["expert"].format(e) for e in range(self.num_experts)]
        # [experts, 2F, W]: an expert's gate rows, then its up rows; [experts, W, F]
        self.w_gate_up = torch.stack([torch.cat([tensors[q + n["gate"]], tensors[q + n["up"]]], dim=0)
                                      for q in names]).contiguous()
        self.w_down = torch.stack([tensors[q + n["down"]] for q in names]).contiguous()
        # one product gives the router's logits and, behind them, the shared expert's gate; its rows are
        # filled up to a multiple of 8 with zeros
        rows = [tensors[p + n["router"]]]
        if self.shared_size is not None:
            q = p + n["shared"]
            if self.shared_gate:
                rows.append(tensors[p + n["shared_gate"]])
            self.shared_gate_up = torch.cat([tensors[q + n["gate"]], tensors[q + n["up"]]], dim=0).contiguous()
            self.shared_down = tensors[q + n["down"]]
        have = sum(r.shape[0] for r in rows)
        if have % 8:
            rows.append(torch.zeros(8 - have % 8, self.hidden_size, dtype=rows[0].dtype, device=rows[0].device))
        self.w_router = torch.cat(rows, dim=0).contiguous()
        self.correction = tensors[p + n["correction"]]

    def forward(self, x):
        logits = ops.linear(x, self.w_router, out_dtype=torch.float32 if x.dtype != torch.float32 else None)
        ids, weights = ops.route_experts(logits, self.correction, self.num_experts, self.top, self.group_count,
                                         self.group_keep, self.route_scale, self.weight_eps, score=self.score,
                                         group_top=self.group_top, normalize=self.normalize)
        shared = None
        if self.shared_size is not None:
            shared = ops.linear(ops.gated_linear(x, self.shared_gate_up), self.shared_down)
        return ops.routed_experts(x, ids, weights, self.w_gate_up, self.w_down, shared, logits,
                                  self.num_experts if self.shared_gate else -1, self.out_dtype)
