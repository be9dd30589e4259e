"""A routed feed-forward (mixture of experts) of gated units, clamped or plain.

Router: z = W_router x in float32, scores sigmoid(z) (``score`` "sigmoid") or softmax(z) ("softmax");
every token uses the ``top_k`` experts with the largest scores (the lower index wins a tie); the
weights are those scores, divided by their sum if ``renormalize``.  Expert e: g = min(W_gate,e h, limit),
u = clamp(W_up,e h, -limit, limit), y = g sigmoid(alpha g) (u + 1), output W_down,e y, no biases.  The
weight multiplies the expert's INPUT (``weight_on`` "input": out = sum_j expert_j(w_j x)) or its output
("output": out = sum_j w_j expert_j(x)).  ``limit`` None: the expert is the plain gated unit
W_down,e (silu(W_gate,e h) * W_up,e h).  ``groups`` > 1 with ``keep`` < groups: the experts form ``groups``
equal groups of neighbours, a group's score is its largest member's, and only experts of the ``keep`` best groups
can be chosen.  With ``renormalize`` the chosen scores are divided by their sum + ``renorm_eps``.
``correction``: a tensor of one number an expert is added to the scores for the CHOICE only (the weights stay the
scores).  ``weight_scale`` multiplies the weights.  ``identity`` = n: the router has n more outputs than there are
experts; the last n are identity experts without tensors, whose output is their input (times the weight).
``shared``: a feed-forward part (with its prefix ``shared_prefix`` below this one's) that runs for every token beside
the routed experts and adds its own output.

Routing, the expert-sorted order and the products are planned and run on the device (csrc/moe.cu):
nothing is read back, so steps of single tokens are captured like any other part's.  In bfloat16 the
two products run on the tcgen05 tensor cores as grouped products over 128-row tiles that each belong
to one expert (the persistent kernel of csrc/gemm_tc.cu with a plan), the first with the gated
activation in its epilogue over gate and up rows interleaved by 16; in float32, and at sizes that
kernel does not take, on CUDA cores in tiles of 64 rows.

Parameters: ``hidden_size``, ``intermediate_size``, ``limit``, ``alpha``, ``num_experts``, ``top_k``,
``score``, ``renormalize``, ``renorm_eps``, ``weight_on``, ``groups``, ``keep``, ``correction``, ``weight_scale``,
``identity``, ``shared``, ``shared_prefix``.  Tensors below the prefix: router [E + identity, hidden];
e<j>.gate, e<j>.up [ff, hidden]; e<j>.down [hidden, ff]; correction [E + identity].
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import FEED_FORWARDS, FeedForward, TensorSpec, build_part


@FEED_FORWARDS.register("routed_clamped_glu")
class RoutedClampedGLU(FeedForward):
    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        self.limit = float(p["limit"]) if p.get("limit") is not None else 0.0  # 0: no clamp, silu(gate) * up
        if p.get("limit") is not None and not self.limit > 0:
            raise ValueError("limit must be positive (or None for the plain gated unit)")
        self.alpha = float(p.get("alpha", 1.702))
        self.num_experts = int(p["num_experts"])
        self.top_k = int(p["top_k"])
        self.score = p.get("score", "sigmoid")
        self.renormalize = bool(p.get("renormalize", False))
        self.weight_on = p.get("weight_on", "output")
        self.renorm_eps = float(p.get("renorm_eps", 0.0))
        self.groups = int(p.get("groups", 1))
        self.keep = int(p.get("keep", self.groups))
        if self.groups < 1 or self.num_experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.num_experts} experts cannot form {self.groups} equal groups of which {self.keep} are kept")
        if self.top_k > self.keep * ((self.num_experts + int(p.get("identity", 0) or 0)) // self.groups):
            raise ValueError(f"top_k {self.top_k} exceeds the {self.keep} kept groups' experts")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {self.score!r} (known: sigmoid, softmax)")
        if self.weight_on not in ("input", "output"):
            raise ValueError(f"weight_on must be 'input' or 'output', got {self.weight_on!r}")
        if not 0 < self.top_k <= self.num_experts + int(p.get("identity", 0) or 0):
            raise ValueError(f"top_k {self.top_k} does not fit {self.num_experts} experts")
        self.identity = int(p.get("identity", 0) or 0)
        self.router_outputs = self.num_experts + self.identity
        self.has_correction = bool(p.get("correction", False))
        self.weight_scale = float(p.get("weight_scale", 1.0))
        if self.router_outputs > 256:
            raise ValueError("the router kernel takes up to 256 experts")
        if self.identity and (self.weight_on != "output" or self.groups != 1):
            raise ValueError("identity experts are built with the weight on the output and without groups")
        if self.top_k > self.router_outputs:
            raise ValueError(f"top_k {self.top_k} does not fit {self.router_outputs} router outputs")
        self.shared = build_part(FEED_FORWARDS, p["shared"]) if p.get("shared") is not None else None
        self.shared_prefix = str(p.get("shared_prefix", "shared."))
        self.correction = None
        self.router = self.gate_up = self.down = None
        self.tensor_cores = False

    @classmethod
    def expected_tensors(cls, spec: PartSpec, prefix: str) -> list[TensorSpec]:
        p = spec.params
        hidden, inter, experts = int(p["hidden_size"]), int(p["intermediate_size"]), int(p["num_experts"])
        out = []
        for e in range(experts):
            out += [TensorSpec(f"{prefix}e{e}.gate", (inter, hidden)), TensorSpec(f"{prefix}e{e}.up", (inter, hidden)),
                    TensorSpec(f"{prefix}e{e}.down", (hidden, inter))]
        outputs = experts + int(p.get("identity", 0) or 0)
        out.append(TensorSpec(prefix + "router", (outputs, hidden)))
        if p.get("correction", False):
            out.append(TensorSpec(prefix + "correction", (outputs,), init="zeros"))
        if p.get("shared") is not None:
            out += FEED_FORWARDS.get(p["shared"].kind).expected_tensors(p["shared"], prefix + str(p.get("shared_prefix", "shared.")))
        return out

    def load(self, tensors: dict, prefix: str, device, dtype) -> None:
        E = self.num_experts
        self.router = tensors[prefix + "router"].to(device=device, dtype=torch.float32).contiguous()
        if self.has_correction:
            self.correction = tensors[prefix + "correction"].to(device=device, dtype=torch.float32).contiguous()
        if self.shared is not None:
            self.shared.load(tensors, prefix + self.shared_prefix, device, dtype)
        from . import swiglu_bf16

        # per expert [gate; up] stacked, [E, 2 ff, hidden], and [E, hidden, ff]; for the tensor-core product the
        # gate and up rows of an expert are interleaved by 16 instead, as the gated epilogue reads them
        self.tensor_cores = (dtype == torch.bfloat16 and swiglu_bf16.usable(self.hidden_size, self.intermediate_size)
                             and self.intermediate_size % 8 == 0)
        join = swiglu_bf16.interleave if self.tensor_cores else (lambda gate, up: torch.cat([gate, up], dim=0))
        self.gate_up = torch.stack([join(tensors[f"{prefix}e{e}.gate"], tensors[f"{prefix}e{e}.up"])
                                    for e in range(E)]).to(device=device, dtype=dtype).contiguous()
        self.down = torch.stack([tensors[f"{prefix}e{e}.down"] for e in range(E)]).to(device=device, dtype=dtype).contiguous()

    def _rows(self, tokens: int, tile: int) -> tuple:
        """(row tiles, rows) the expert-sorted order of ``tokens`` tokens can take at most: every
        expert's rows are padded to whole tiles."""
        entries = tokens * self.top_k
        tiles = entries // tile + min(self.num_experts, entries)
        return tiles, tiles * tile

    def forward(self, ctx, x, acc) -> None:
        tokens, top, E = x.shape[0], self.top_k, self.num_experts
        # tiles of 128 sorted rows on the tensor cores, of 16 where an expert gets 16 rows or fewer on average
        # (steps of single tokens: the products then stream the chosen experts' weights); 64 on CUDA cores
        if not self.tensor_cores:
            tile = ops.moe_tile_rows()
        elif tokens * top <= ops.GROUPED_TILE_ROWS_FEW * E:
            tile = ops.GROUPED_TILE_ROWS_FEW
        else:
            tile = ops.GROUPED_TILE_ROWS
        tiles, rows = self._rows(tokens, tile)
        # scratch sized once for the largest step (and the tile size that takes most), so that its addresses never change
        capacity = max(ctx.token_capacity, tokens)
        few = self._rows(min(capacity, ops.GROUPED_TILE_ROWS_FEW * E // top), ops.GROUPED_TILE_ROWS_FEW)
        most = self._rows(capacity, tile if not self.tensor_cores else ops.GROUPED_TILE_ROWS)
        most_tiles, most_rows = max(few[0], most[0]), max(few[1], most[1])
        choice = ctx.buffer("moe.choice", (tokens, top), torch.int32)
        weight = ctx.buffer("moe.weight", (tokens, top), torch.float32)
        position = ctx.buffer("moe.position", (tokens, top), torch.int32)
        plan = ctx.buffer("moe.plan", (most_tiles + 1,), torch.int32)[:tiles + 1]
        sorted_x = ctx.buffer("moe.sorted", (most_rows, self.hidden_size), ctx.dtype)[:rows]
        act = ctx.buffer("moe.act", (most_rows, self.intermediate_size), ctx.dtype)[:rows]
        y = ctx.buffer("moe.y", (most_rows, self.hidden_size), torch.float32)[:rows]
        on_input = self.weight_on == "input"
        # a shared part with a gate of one number a token: the router's kernel has the token's row at hand and takes it along
        gate_w = getattr(self.shared, "token_gate_weight", None)
        shared_gate = ctx.buffer("moe.shared_gate", (tokens,), torch.float32) if gate_w is not None else None
        ops.moe_route(x, self.router, choice, weight, self.score == "softmax", self.renormalize, self.groups, self.keep,
                      self.renorm_eps, correction=self.correction, scale=self.weight_scale,
                      token_gate=(gate_w, shared_gate) if gate_w is not None else None)
        ops.moe_plan(choice, position, plan, E, tile)
        ops.moe_scatter(x, position, weight, sorted_x, top, weighted=on_input)
        if self.tensor_cores:
            ops.gemm_tc_grouped(sorted_x, self.gate_up, act, plan, glu=True, limit=self.limit, alpha=self.alpha,
                                tile_rows=tile)
            ops.gemm_tc_grouped(act, self.down, y, plan, tile_rows=tile)
        else:
            ops.moe_gemm_simt(sorted_x, self.gate_up, act, plan, glu=True, limit=self.limit, alpha=self.alpha)
            ops.moe_gemm_simt(act, self.down, y, plan)
        ops.moe_combine(y, position, weight, acc, top, weighted=not on_input, x=x if self.identity else None)
        if self.shared is not None and shared_gate is not None:
            self.shared.forward(ctx, x, acc, row_scale=shared_gate)
        elif self.shared is not None:
            self.shared.forward(ctx, x, acc)
