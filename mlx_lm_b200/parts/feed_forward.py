"""Feed-forward parts.  ``MLP``: ``down(act(up(x)))`` with biases, the dense
two-matrix form of mlx_lm/models/gpt2.py:71-80 with the inner width and the
activation as parameters; the activation runs in the first product's
epilogue and the residual add in the second's."""

from __future__ import annotations

from .base import VECTOR, FeedForward, Init, ParamSpec, register_part
import torch

from .. import ops
from .linear import ACTIVATIONS, FusedLinear, Linear


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


class GatedMLP(FeedForward):
    """``down(silu(gate(x)) * up(x))`` without biases.  ``gate`` and ``up`` run as one product whose two halves
    a small kernel multiplies; the residual stream (float32) is added in the last product's epilogue.
    ``unit="bounded"``: the gated unit is ``g' sigmoid(1.702 g') (u' + 1)`` with ``g' = min(gate(x), limit)`` and
    ``u' = clamp(up(x), -limit, limit)`` instead."""
    replayable = True
    kernel_libs = ("elementwise",)

    def __init__(self, name: str, width: int, inner: int, gate_name: str = "gate", up_name: str = "up",
                 down_name: str = "down", init: Init = Init(), unit: str = "silu", limit: float = 0.0):
        if unit not in ops.GATED_UNITS:
            raise ValueError(f"{name}: gated unit {unit!r} is not one of {sorted(ops.GATED_UNITS)}")
        self.name, self.width, self.inner = name, width, inner
        self.unit, self.limit = unit, float(limit)
        self.gate_up = FusedLinear(f"{name}.gate_up", width, [(f"{name}.{gate_name}", inner), (f"{name}.{up_name}", inner)],
                                   init=init)
        self.down = Linear(f"{name}.{down_name}", inner, width, bias=False, weight_suffix="", init=init)

    def children(self):
        return (self.gate_up, self.down)

    def forward(self, ctx, x, residual):
        T = x.shape[0]
        both = ctx.ws.get("ffn_gate_up", T, 2 * self.inner, x.dtype)
        self.gate_up.forward(ctx, x, both)
        h = ctx.ws.get("ffn_hidden", T, self.inner, x.dtype)
        ops.label(self.name + ".act", 4.0 * T * self.inner, 3.0 * x.element_size() * T * self.inner)
        ops.gated_unit(both, h, ctx.stream, unit=self.unit, limit=self.limit)
        return self.down.forward(ctx, h, residual, residual=residual)

    def branch(self, ctx, x):
        """The result alone, float32 ``[T, width]``, for a block that adds it to the stream itself: ``(rows, 1)``."""
        T = x.shape[0]
        both = ctx.ws.get("ffn_gate_up", T, 2 * self.inner, x.dtype)
        self.gate_up.forward(ctx, x, both)
        h = ctx.ws.get("ffn_hidden", T, self.inner, x.dtype)
        ops.label(self.name + ".act", 4.0 * T * self.inner, 3.0 * x.element_size() * T * self.inner)
        ops.gated_unit(both, h, ctx.stream, unit=self.unit, limit=self.limit)
        return self.down.forward(ctx, h, ctx.ws.get("ffn_out", T, self.width, torch.float32)), 1


register_part("feed_forward", "gated_mlp", GatedMLP)


class ExpertsMLP(FeedForward):
    """A mixture of experts: ``n_experts`` small gated feed-forwards ``down(silu(gate(z)) * up(z))`` without biases
    (``<name>.e<i>.gate|up|down``), of which every token uses the ``top`` with the largest router scores.

    The router (``<name>.router`` ``[n_experts, width]``) gives float32 logits; ``score``: ``sigmoid`` of each, or the
    ``softmax`` over the experts; the chosen experts' scores are the weights, divided by their sum only with
    ``renormalize``.  ``scale_input``: the weight multiplies the expert's INPUT, ``sum_c expert_c(w_c x)``; else its
    output, ``sum_c w_c expert_c(x)``.  (With the input scaled, ``w`` is applied to the float32 sums of the gate and up
    products, which are linear in the input.)

    Options of the router: ``correction`` (a tensor ``<name>.correction``, one number per router output, added to the
    scores for the choice only: the weights are the scores without it); ``groups = (count, keep)``: the router outputs
    form ``count`` equal groups of neighbours, a group's score is its largest choice score, and only outputs of the
    ``keep`` best groups can be chosen; ``identity``: the router has that many more outputs than there are experts with
    tensors, and a token that chooses one of them gets its own input back (times the weight); ``renormalize_eps`` is
    added to the sum the weights are divided by; ``weight_scale`` multiplies every weight.  ``unit="bounded"`` with
    ``limit``: the experts' gated unit is ``g' sigmoid(1.702 g') (u' + 1)``, ``g' = min(g, limit)``, ``u' = clamp(u,
    -limit, limit)``, and the weight multiplies the unit's OUTPUT (``scale_input=False``).  ``shared``: a feed-forward
    that runs for every token beside the experts and is added.

    The experts' weights are stacked at bind time (``[E, 2 inner, width]`` gate rows then up rows, ``[E, width,
    inner]``); a step routes (``ops.moe_route``), sorts its (token, choice) slots by expert into tiles
    (``ops.moe_plan``) and runs two products over the tiles, the gated unit in the first one's epilogue: ``ops.moe_gemm``
    for the few slots of decoding steps, ``ops.moe_gather`` and ``ops.moe_gemm_tc05`` (tcgen05, TMA) for many.  ``branch`` returns one float32 row per slot, ``top`` rows a token, which the caller sums in the order
    of the choices; ``forward`` adds them to a float32 stream."""
    replayable = True
    kernel_libs = ("moe", "moe_tcgen05", "dyt")
    MANY_SLOTS = 512     # (token, choice) slots of a step from which the 128-row tiles pay
    FEW_SLOTS_AN_EXPERT = 8   # up to so many slots an expert on average, the weights are streamed by a warp per column

    def __init__(self, name: str, width: int, inner: int, n_experts: int, top: int, score: str = "sigmoid",
                 renormalize: bool = False, scale_input: bool = True, router_name: str = "router",
                 expert_prefix: str = "e", gate_name: str = "gate", up_name: str = "up", down_name: str = "down",
                 init: Init = Init(), router_init: Init = Init(), correction: bool = False, groups=None, identity: int = 0,
                 renormalize_eps: float = 0.0, weight_scale: float = 1.0, unit: str = "silu", limit: float = 0.0,
                 shared: FeedForward = None, correction_name: str = "correction"):
        n_outputs = n_experts + int(identity)
        if n_experts < 0 or identity < 0 or not 1 <= top <= n_outputs:
            raise ValueError(f"{name}: {top} of {n_experts} experts and {identity} identity experts")
        if score not in ops.MOE_SCORES:
            raise ValueError(f"{name}: router score {score!r} is not one of {sorted(ops.MOE_SCORES)}")
        if unit not in ops.GATED_UNITS:
            raise ValueError(f"{name}: gated unit {unit!r} is not one of {sorted(ops.GATED_UNITS)}")
        if scale_input != (unit == "silu"):
            raise ValueError(f"{name}: the routing weight goes on the input of the silu unit and on the output of the "
                             f"bounded one; other pairings are not built")
        count, keep = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        if count < 1 or n_outputs % count or not 1 <= keep <= count or top > keep * (n_outputs // count):
            raise ValueError(f"{name}: {n_outputs} router outputs in {count} groups of which {keep} stay, {top} chosen")
        self.name, self.width, self.inner, self.n_experts, self.top = name, width, inner, n_experts, top
        self.score, self.renormalize, self.scale_input = score, renormalize, scale_input
        self.identity, self.n_outputs, self.groups, self.keep_groups = int(identity), n_outputs, count, keep
        self.renormalize_eps, self.weight_scale, self.unit, self.limit = float(renormalize_eps), float(weight_scale), unit, float(limit)
        self.shared = shared
        self.correction_name = f"{name}.{correction_name}" if correction else None
        self.correction = None
        self.router = Linear(f"{name}.{router_name}", width, n_outputs, bias=False, weight_suffix="", init=router_init)
        self.names = [(f"{name}.{expert_prefix}{e}.{gate_name}", f"{name}.{expert_prefix}{e}.{up_name}",
                       f"{name}.{expert_prefix}{e}.{down_name}") for e in range(n_experts)]
        self.init = init
        self.w_in = self.w_out = None

    def children(self):
        return (self.router,) + ((self.shared,) if self.shared is not None else ())

    def param_specs(self):
        from .base import MATRIX
        specs = []
        if self.correction_name:
            specs.append(ParamSpec(self.correction_name, (self.n_outputs,), VECTOR, Init(0.0, 0.02)))
        for g, u, d in self.names:
            specs += [ParamSpec(g, (self.inner, self.width), MATRIX, self.init),
                      ParamSpec(u, (self.inner, self.width), MATRIX, self.init),
                      ParamSpec(d, (self.width, self.inner), MATRIX, Init(0.0, self.inner ** -0.5))]
        return specs

    def bind(self, tensors, dtype, device) -> None:
        self.correction = tensors[self.correction_name].contiguous() if self.correction_name else None
        if not self.names:        # identity experts only
            return
        self.w_in = torch.stack([torch.cat([tensors[g], tensors[u]], dim=0) for g, u, _ in self.names]).contiguous()
        self.w_out = torch.stack([tensors[d] for _, _, d in self.names]).contiguous()

    def branch(self, ctx, x):
        if self.identity or self.shared is not None:
            raise ops.KernelError(f"{self.name}: identity experts and a shared expert add to the stream themselves (forward)")
        y, _, _ = self._experts(ctx, x)
        return y, self.top

    def _experts(self, ctx, x):
        """The chosen experts' rows, float32 ``[T * top, width]`` (rows of identity experts are not written), with the
        choices ``sel_expert`` and their weights."""
        T, E, top, F_, D = x.shape[0], self.n_experts, self.top, self.inner, self.width
        S, EO = T * top, self.n_outputs
        logits = self.router.forward(ctx, x, ctx.ws.get("moe_logits", T, (EO + 7) // 8 * 8, torch.float32)[:, :EO])
        sel_e = ctx.ws.flat("moe_sel_expert", S, torch.int32)
        sel_w = ctx.ws.flat("moe_sel_weight", S, torch.float32)
        ops.label(self.name + ".route", 8.0 * T * EO, 4.0 * T * EO + 8.0 * S)
        ops.moe_route(logits, ctx.token_req, top, sel_e, sel_w, ctx.stream, score=self.score, renormalize=self.renormalize,
                      correction=self.correction, groups=self.groups, keep_groups=self.keep_groups, identity=self.identity,
                      renormalize_eps=self.renormalize_eps, weight_scale=self.weight_scale)
        y = ctx.ws.get("moe_out", S, D, torch.float32)
        if E == 0:
            return y, sel_e, sel_w
        unit = dict(unit=self.unit, limit=self.limit)
        tc = x.dtype == torch.bfloat16 and D % 8 == 0 and F_ % 8 == 0 and x.stride(0) % 8 == 0
        # many slots: tiles of 128 rows of one expert on the 5th-generation tensor cores, the rows gathered in the
        # plan's order first; few slots an expert (decoding): tiles of 4, a warp per output column; between them tiles
        # of 64 on mma.sync through the sorted list; float32 and odd sizes: the CUDA cores
        many = tc and S >= self.MANY_SLOTS
        few = tc and not many and S <= self.FEW_SLOTS_AN_EXPERT * E and max(D, F_) <= ops.MOE_FEW_MAX_INNER
        rows = ops.moe_tc05_tile_rows() if many else ops.moe_few_rows() if few else ops.moe_tile_rows(tc)
        max_tiles = ops.moe_max_tiles(S, E, rows)
        order = ctx.ws.flat("moe_sorted", S, torch.int32)
        tiles = ctx.ws.flat("moe_tiles", 3 * max_tiles + 1, torch.int32)
        n_tiles = tiles[3 * max_tiles:]
        ops.moe_plan(sel_e, S, E, rows, order, tiles, n_tiles, ctx.stream)
        h = ctx.ws.get("moe_hidden", S, F_, x.dtype)
        es = x.element_size()
        if many:
            xs = ctx.ws.get("moe_rows", S, D, x.dtype)
            ops.label(self.name + ".gather", 0.0, es * (T + S) * D)
            ops.moe_gather(x, top, order, tiles, n_tiles, max_tiles, xs, ctx.stream)
            ops.label(self.name + ".experts.in", 4.0 * S * D * F_, es * (min(E, S) * 2 * F_ * D + S * D + S * F_))
            ops.moe_gemm_tc05(xs, self.w_in, F_, order, tiles, n_tiles, max_tiles, h, ctx.status, ctx.stream,
                              sel_weight=sel_w, gated=True, **unit)
            ops.label(self.name + ".experts.out", 2.0 * S * D * F_, es * (min(E, S) * F_ * D + S * F_) + 4.0 * S * D)
            ops.moe_gemm_tc05(h, self.w_out, D, order, tiles, n_tiles, max_tiles, y, ctx.status, ctx.stream)
            return y, sel_e, sel_w
        ops.label(self.name + ".experts.in", 4.0 * S * D * F_, es * (min(E, S) * 2 * F_ * D + T * D + S * F_))
        ops.moe_gemm(x, top, self.w_in, F_, order, tiles, n_tiles, max_tiles, rows, h, ctx.stream, sel_weight=sel_w, gated=True,
                     **unit)
        ops.label(self.name + ".experts.out", 2.0 * S * D * F_, es * (min(E, S) * F_ * D + S * F_) + 4.0 * S * D)
        ops.moe_gemm(h, 1, self.w_out, D, order, tiles, n_tiles, max_tiles, rows, y, ctx.stream)
        return y, sel_e, sel_w

    def forward(self, ctx, x, residual):
        y, sel_e, sel_w = self._experts(ctx, x)
        terms = self.top
        ops.label(self.name + ".sum", terms * x.shape[0] * self.width, 4.0 * (terms + 2) * x.shape[0] * self.width)
        if self.identity:
            ops.moe_combine(residual, y, sel_e, sel_w, x, terms, ctx.stream, token_req=ctx.token_req)
        else:
            ops.dyt_residual(residual, y, ctx.stream, terms=terms, token_req=ctx.token_req)
        if self.shared is not None:
            residual = self.shared.forward(ctx, x, residual)
        return residual


register_part("feed_forward", "experts_mlp", ExpertsMLP)


class LearnedActMLP(FeedForward):
    """``down(act(up(x)))`` without biases, where ``act`` has numbers of its own that the layer learns (a tensor
    ``<name>.act``).  ``xielu``: two numbers ``(a, b)``; ``z > 0: softplus(a) z^2 + z/2``,
    ``z <= 0: (1/2 + softplus(b)) (exp(z) - 1 - z) + z/2``.  The activation is a kernel of its own between the two
    products (float32 arithmetic, in place); the residual stream (float32) is added in the second product's epilogue."""
    replayable = True
    kernel_libs = ("elementwise",)
    ACTS = {"xielu": 2}      # name -> how many numbers

    def __init__(self, name: str, width: int, inner: int, activation: str = "xielu", up_name: str = "up",
                 down_name: str = "down", act_name: str = "act", init: Init = Init()):
        if activation not in self.ACTS:
            raise ValueError(f"{name}: activation {activation!r} is not one of {sorted(self.ACTS)}")
        self.name, self.width, self.inner, self.activation = name, width, inner, activation
        self.act_name = f"{name}.{act_name}"
        self.up = Linear(f"{name}.{up_name}", width, inner, bias=False, weight_suffix="", init=init)
        self.down = Linear(f"{name}.{down_name}", inner, width, bias=False, weight_suffix="", init=Init(0.0, inner ** -0.5))
        self.act = None

    def children(self):
        return (self.up, self.down)

    def param_specs(self):
        return [ParamSpec(self.act_name, (self.ACTS[self.activation],), VECTOR, Init(0.0, 0.5))]

    def bind(self, tensors, dtype, device) -> None:
        self.act = tensors[self.act_name].contiguous()

    def forward(self, ctx, x, residual):
        T = x.shape[0]
        h = self.up.forward(ctx, x, ctx.ws.get("ffn_hidden", T, self.inner, x.dtype))
        ops.label(self.name + ".act", 8.0 * T * self.inner, 2.0 * x.element_size() * T * self.inner)
        ops.xielu(h, h, self.act, ctx.stream)
        return self.down.forward(ctx, h, residual, residual=residual)


register_part("feed_forward", "learned_act_mlp", LearnedActMLP)
