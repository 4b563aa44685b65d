"""Feed-forwards: dense gated (SwiGLU), dense squared-ReLU, and table-routed mixture of experts (the latter two at the
end of the file).

SwiGLU:

gate = Wg x, up = Wu x, z = up * gate / (1 + exp(-gate)) with the activation and the
product in 32-bit and one rounding, y = Wd z; no bias.  Reference:
src/transformer.cpp:597-617 (order), src/decode.cu:746-764 (activation).  Gate and
up rows are kept in one matrix, row 2i the gate's and row 2i+1 the up's i-th, so that one
product makes both and the activation can run in that product's epilogue.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels as K
from .base import BuildContext, FeedForward, ParamSpec, register_part


class SwiGLU(FeedForward):
    def __init__(self, ctx: BuildContext, prefix: str, intermediate_size: int,
                 names: Optional[Dict[str, str]] = None):
        self.hidden = ctx.hidden_size
        self.inter = int(intermediate_size)
        n = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            self.names["gate"]: ParamSpec((self.inter, self.hidden)),
            self.names["up"]: ParamSpec((self.inter, self.hidden)),
            self.names["down"]: ParamSpec((self.hidden, self.inter)),
        }

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g = tensors.pop(self.names["gate"])
        u = tensors.pop(self.names["up"])
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden).contiguous()
        del g, u
        self.w_down = tensors.pop(self.names["down"]).contiguous()

    takes_pending_norm = True       # x goes into K.linear_swiglu, and nowhere else
    captures_start = True

    def forward(self, x, batch) -> torch.Tensor:
        z = K.linear_swiglu(x, self.w_gate_up)    # [M, inter]
        return K.linear(z, self.w_down)


register_part("feed_forward", "swiglu", SwiGLU)


class GatedDense(FeedForward):
    """y = Wdown (act(Wgate x) * (Wup x)) with ``act`` "gelu_tanh" or "silu"; or, with ``act`` "clamped_swish" and its
    ``limit``, y = Wdown (g sigmoid(1.702 g) (u + 1)) with g = min(Wgate x, limit) and u = clamp(Wup x, -limit, limit);
    no bias.  Gate and up rows are one matrix with row 2i the gate's and row 2i + 1 the up's i-th, so one product makes
    both and the activation runs in that product's epilogue on the tensor-core kernels (kernels.linear_swiglu), in
    32-bit with one rounding."""

    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, intermediate_size: int, act: str = "gelu_tanh", limit: float = 0.0,
                 names: Optional[Dict[str, str]] = None):
        self.hidden = ctx.hidden_size
        self.inter = int(intermediate_size)
        if act not in K.GATE_ACTS:
            raise ValueError(f"feed-forward at {prefix!r}: unknown activation {act!r}; known: {sorted(K.GATE_ACTS)}")
        if act == "clamped_swish" and not float(limit) > 0:
            raise ValueError(f"feed-forward at {prefix!r}: the clamped activation needs a positive limit, got {limit}")
        self.act, self.limit = act, float(limit)
        n = {"gate": "gate", "up": "up", "down": "down"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.w_gate_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.names["gate"]: ParamSpec((self.inter, self.hidden), std=0.05),
                self.names["up"]: ParamSpec((self.inter, self.hidden), std=0.05),
                self.names["down"]: ParamSpec((self.hidden, self.inter), std=0.05)}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        g, u = tensors.pop(self.names["gate"]), tensors.pop(self.names["up"])
        self.w_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.inter, self.hidden).contiguous()
        self.w_down = tensors.pop(self.names["down"]).contiguous()

    def forward(self, x, batch) -> torch.Tensor:
        return K.linear(K.linear_swiglu(x, self.w_gate_up, self.act, self.limit), self.w_down)


class SquaredReLU(FeedForward):
    """y = Wdown relu(Wup x)^2; no gate, no bias."""

    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, intermediate_size: int, names: Optional[Dict[str, str]] = None):
        self.hidden = ctx.hidden_size
        self.inter = int(intermediate_size)
        n = {"up": "up", "down": "down"}
        n.update(names or {})
        self.names = {k: prefix + v for k, v in n.items()}
        self.w_up = self.w_down = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.names["up"]: ParamSpec((self.inter, self.hidden)),
                self.names["down"]: ParamSpec((self.hidden, self.inter))}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_up = tensors.pop(self.names["up"]).contiguous()
        self.w_down = tensors.pop(self.names["down"]).contiguous()

    def forward(self, x, batch) -> torch.Tensor:
        from ..kernels import moe as KM
        return K.linear(KM.relu2(K.linear(x, self.w_up)), self.w_down)


class TableMoE(FeedForward):
    """Mixture of experts whose router is a table: token id t uses the experts table[t, 0..top-1] (all different),
    each with weight 1/top.  An expert: g = min(Wgate x, limit), u = clamp(Wup x, -limit, limit),
    y = Wdown (g * sigmoid(alpha * g) * (u + 1)); no biases.  The step's tokens are grouped by expert on the
    device and every product runs once over all groups (kernels/moe.py)."""

    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_experts: int, top: int, intermediate_size: int, limit: float,
                 vocab_size: int, alpha: float = 1.702, names: Optional[Dict[str, str]] = None):
        self.hidden = ctx.hidden_size
        self.n_experts, self.top, self.inter = int(n_experts), int(top), int(intermediate_size)
        self.limit, self.alpha, self.vocab = float(limit), float(alpha), int(vocab_size)
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"moe at {prefix!r}: {self.top} of {self.n_experts} experts per token")
        n = {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "table": "table"}
        n.update(names or {})
        self.prefix, self.n = prefix, n
        self.w_gate_up = self.w_down = self.table = None

    def _name(self, e: int, which: str) -> str:
        return self.prefix + self.n["expert"].format(e) + self.n[which]

    def param_specs(self) -> Dict[str, ParamSpec]:
        s: Dict[str, ParamSpec] = {}
        for e in range(self.n_experts):
            s[self._name(e, "gate")] = ParamSpec((self.inter, self.hidden), std=0.05)
            s[self._name(e, "up")] = ParamSpec((self.inter, self.hidden), std=0.05)
            s[self._name(e, "down")] = ParamSpec((self.hidden, self.inter))
        s[self.prefix + self.n["table"]] = ParamSpec((self.vocab, self.top), role="int_table", init="distinct_below",
                                                     high=self.n_experts)
        return s

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        E = range(self.n_experts)
        # an expert's gate rows, then its up rows: one product makes both
        self.w_gate_up = torch.stack([torch.cat([tensors.pop(self._name(e, "gate")), tensors.pop(self._name(e, "up"))], dim=0)
                                      for e in E]).contiguous()
        self.w_down = torch.stack([tensors.pop(self._name(e, "down")) for e in E]).contiguous()
        self.table = tensors.pop(self.prefix + self.n["table"]).to(torch.int32).contiguous()

    def forward(self, x, batch) -> torch.Tensor:
        from ..kernels import moe as KM
        if batch is None:
            raise RuntimeError("a table-routed feed-forward needs the step's token ids")
        ids = batch.token_ids[: x.shape[0]]
        perm, off = KM.route_by_table(ids, self.table, self.n_experts)
        return KM.experts_ffn(x, perm, off, self.w_gate_up, self.w_down, self.top, self.limit, self.alpha, 1.0 / self.top)


register_part("feed_forward", "gated_dense", GatedDense)
register_part("feed_forward", "relu2", SquaredReLU)
register_part("feed_forward", "table_moe", TableMoE)


class ScoredMoE(FeedForward):
    """Mixture of experts with independent scores: z = Wr x (float32), s = sigmoid(z); the ``top`` experts with the largest
    scores run, each on the token's row times its score (not renormalised): y = sum_e Wdown_e relu(Wup_e (s_e x))^2.  A shared
    expert of the same form (its own width) may run for every token, times sigmoid(wg . x).  No biases.

    Since s > 0 the scaled input is the same as s^2 on the expert's output: the products run on x, grouped by expert on
    the device (kernels/moe.py), and the sum at the end applies the squares.  The router's matrix and the shared gate's
    row are one product with a float32 result."""

    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_experts: int, top: int, intermediate_size: int,
                 shared_size: int = 0, names: Optional[Dict[str, str]] = None):
        self.hidden = ctx.hidden_size
        self.n_experts, self.top, self.inter, self.shared = int(n_experts), int(top), int(intermediate_size), int(shared_size)
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"moe at {prefix!r}: {self.top} of {self.n_experts} experts per token")
        n = {"expert": "e{}.", "up": "up", "down": "down", "router": "router", "shared": "shared.", "shared_gate": "shared.sg"}
        n.update(names or {})
        self.prefix, self.n = prefix, n
        self.w_up = self.w_down = self.w_router = self.ws_up = self.ws_down = None

    def _name(self, e: int, which: str) -> str:
        return self.prefix + self.n["expert"].format(e) + self.n[which]

    def param_specs(self) -> Dict[str, ParamSpec]:
        s: Dict[str, ParamSpec] = {}
        for e in range(self.n_experts):
            s[self._name(e, "up")] = ParamSpec((self.inter, self.hidden), std=0.05)
            s[self._name(e, "down")] = ParamSpec((self.hidden, self.inter), std=0.05)
        s[self.prefix + self.n["router"]] = ParamSpec((self.n_experts, self.hidden), std=0.3)
        if self.shared:
            p = self.prefix + self.n["shared"]
            s[p + self.n["up"]] = ParamSpec((self.shared, self.hidden), std=0.05)
            s[p + self.n["down"]] = ParamSpec((self.hidden, self.shared), std=0.05)
            s[self.prefix + self.n["shared_gate"]] = ParamSpec((1, self.hidden), std=0.1)
        return s

    def check_kernels(self, dtype) -> None:
        if self.top > 16:
            raise K.KernelError(f"moe: {self.top} experts per token are not supported (up to 16)")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        E = range(self.n_experts)
        self.w_up = torch.stack([tensors.pop(self._name(e, "up")) for e in E]).contiguous()
        self.w_down = torch.stack([tensors.pop(self._name(e, "down")) for e in E]).contiguous()
        rows = [tensors.pop(self.prefix + self.n["router"])]
        if self.shared:
            p = self.prefix + self.n["shared"]
            self.ws_up = tensors.pop(p + self.n["up"]).contiguous()
            self.ws_down = tensors.pop(p + self.n["down"]).contiguous()
            rows.append(tensors.pop(self.prefix + self.n["shared_gate"]).reshape(1, self.hidden))
        self.w_router = torch.cat(rows, dim=0).contiguous()

    def forward(self, x, batch) -> torch.Tensor:
        from ..kernels import moe as KM
        M = x.shape[0]
        z = K.linear(x, self.w_router, out_dtype=torch.float32)            # [M, experts (+ 1)]
        perm, off, _, score2 = KM.route_topk(z, self.n_experts, self.top)
        y, place = KM.experts_relu2(x, perm, off, self.w_up, self.w_down, self.top)
        shared = gate = None
        if self.shared:
            shared = K.linear(KM.relu2(K.linear(x, self.ws_up)), self.ws_down)
            gate = z[:, self.n_experts]
        return KM.combine_gated(y, place, score2, shared, gate, M, self.top)


register_part("feed_forward", "scored_moe", ScoredMoE)


class SoftmaxMoE(FeedForward):
    """Mixture of silu-gated experts under a softmax router with a choice correction and expert groups: z = Wr x (float32),
    s = softmax(z) over all experts; experts are CHOSEN by s + correction (a stored value per expert), only among the
    experts of the ``keep`` best of ``n_groups`` equal runs of neighbouring experts (a run's score is its largest choice
    score); the ``top`` chosen experts' outputs are weighted by their s, divided by the sum of the chosen s, times
    ``scale``.  An expert: Wdown (silu(Wgate x) * (Wup x)); a shared expert of the same form (its own width) may run for
    every token and is added as it is.  No biases.  The step's (token, choice) pairs are grouped by expert on the device
    and every product runs once over all groups (kernels/moe.py)."""

    captures_start = True

    def __init__(self, ctx: BuildContext, prefix: str, n_experts: int, top: int, intermediate_size: int, n_groups: int = 0,
                 keep: int = 0, scale: float = 1.0, correction: bool = True, shared_size: int = 0,
                 names: Optional[Dict[str, str]] = None):
        self.hidden = ctx.hidden_size
        self.n_experts, self.top, self.inter, self.shared = int(n_experts), int(top), int(intermediate_size), int(shared_size)
        self.n_groups, self.keep, self.scale, self.corrected = int(n_groups), int(keep), float(scale), bool(correction)
        if not (1 <= self.top <= self.n_experts):
            raise ValueError(f"moe at {prefix!r}: {self.top} of {self.n_experts} experts per token")
        if self.n_groups > 1 and (self.n_experts % self.n_groups or not 1 <= self.keep <= self.n_groups
                                  or self.keep * (self.n_experts // self.n_groups) < self.top):
            raise ValueError(f"moe at {prefix!r}: {self.n_experts} experts in {self.n_groups} groups of which {self.keep} stay, "
                             f"{self.top} per token")
        n = {"expert": "e{}.", "gate": "gate", "up": "up", "down": "down", "router": "router", "correction": "correction",
             "shared": "shared."}
        n.update(names or {})
        self.prefix, self.n = prefix, n
        self.w_gate_up = self.w_down = self.w_router = self.correction = self.ws_gate_up = self.ws_down = None

    def _name(self, e: int, which: str) -> str:
        return self.prefix + self.n["expert"].format(e) + self.n[which]

    def param_specs(self) -> Dict[str, ParamSpec]:
        s: Dict[str, ParamSpec] = {}
        for e in range(self.n_experts):
            s[self._name(e, "gate")] = ParamSpec((self.inter, self.hidden), std=0.05)
            s[self._name(e, "up")] = ParamSpec((self.inter, self.hidden), std=0.05)
            s[self._name(e, "down")] = ParamSpec((self.hidden, self.inter), std=0.05)
        s[self.prefix + self.n["router"]] = ParamSpec((self.n_experts, self.hidden), std=0.3)
        if self.corrected:
            s[self.prefix + self.n["correction"]] = ParamSpec((self.n_experts,), role="norm", init="normal", std=0.05)
        if self.shared:
            p = self.prefix + self.n["shared"]
            s[p + self.n["gate"]] = ParamSpec((self.shared, self.hidden), std=0.05)
            s[p + self.n["up"]] = ParamSpec((self.shared, self.hidden), std=0.05)
            s[p + self.n["down"]] = ParamSpec((self.hidden, self.shared), std=0.05)
        return s

    def check_kernels(self, dtype) -> None:
        if self.top > 16:
            raise K.KernelError(f"moe: {self.top} experts per token are not supported (up to 16)")
        if self.n_groups > 64:
            raise K.KernelError(f"moe: {self.n_groups} expert groups are not supported (up to 64)")

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        E = range(self.n_experts)
        # an expert's gate rows, then its up rows: one product makes both
        self.w_gate_up = torch.stack([torch.cat([tensors.pop(self._name(e, "gate")), tensors.pop(self._name(e, "up"))], dim=0)
                                      for e in E]).contiguous()
        self.w_down = torch.stack([tensors.pop(self._name(e, "down")) for e in E]).contiguous()
        self.w_router = tensors.pop(self.prefix + self.n["router"]).contiguous()
        if self.corrected:
            self.correction = tensors.pop(self.prefix + self.n["correction"]).to(torch.float32).contiguous()
        if self.shared:
            p = self.prefix + self.n["shared"]
            g, u = tensors.pop(p + self.n["gate"]), tensors.pop(p + self.n["up"])
            self.ws_gate_up = torch.stack([g, u], dim=1).reshape(2 * self.shared, self.hidden).contiguous()
            self.ws_down = tensors.pop(p + self.n["down"]).contiguous()

    def forward(self, x, batch) -> torch.Tensor:
        from ..kernels import moe as KM
        M = x.shape[0]
        z = K.linear(x, self.w_router, out_dtype=torch.float32)
        perm, off, weight = KM.route_softmax(z, self.correction, self.n_experts, self.top, self.n_groups, self.keep, self.scale)
        y, place, _ = KM.expert_pairs(x, perm, off, self.w_gate_up, self.w_down, self.top, float("inf"), 1.0, 0.0)
        shared = K.linear(K.linear_swiglu(x, self.ws_gate_up, "silu"), self.ws_down) if self.shared else None
        return KM.combine_gated(y, place, weight, shared, None, M, self.top)


register_part("feed_forward", "softmax_moe", SoftmaxMoE)
