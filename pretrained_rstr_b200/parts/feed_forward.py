"""Feed-forwards.  ``dense_mlp``: up -> activation -> down, added to the residual stream
(``dev/examples/gpt2.clj:160-166``).  Width, inner size (not tied to 4*width as in
``gpt2.clj:150``), activation and biases are parameters."""
from __future__ import annotations

from ..csrc import ops
from .interfaces import FeedForward
from .linear import Linear
from .registry import register_part


class DenseMLP(FeedForward):
    graph_safe = True
    accepts_lazy_norm = True      # the first matrix product may compute the norm itself
    def __init__(self, up: Linear, down: Linear, width: int, inner: int, activation: str, runtime):
        if activation not in ops.ACT_CODES:
            raise ValueError(f"dense_mlp: unknown activation {activation!r}")
        if (up.n_in, up.n_out) != (width, inner) or (down.n_in, down.n_out) != (inner, width):
            raise ValueError("dense_mlp: matrices have the wrong shape")
        self.up, self.down = up, down
        self.width, self.inner, self.activation = width, inner, activation
        self.runtime = runtime

    def forward(self, ctx, h, x) -> None:
        t = x.shape[0]
        u = ctx.scratch("mlp_inner", (ctx.token_capacity, self.inner), self.runtime.dtype)[:t]
        self.up.forward(ctx, h, u, act=self.activation)
        self.down.forward(ctx, u, x, resid=x)


def _dense_mlp(p, store, rt) -> DenseMLP:
    layout = p.get("weight_layout", "out_in")
    up = Linear.from_store(store, p["weights"]["up"], layout, p["width"], p["inner"],
                           p.get("bias", False), rt)
    down = Linear.from_store(store, p["weights"]["down"], layout, p["inner"], p["width"],
                             p.get("bias", False), rt)
    return DenseMLP(up, down, p["width"], p["inner"], p["activation"], rt)


register_part("feed_forward", "dense_mlp", _dense_mlp)
