"""Gated linear attention: a recurrent mixer with a matrix-valued state per head.

With h the mixer's input, per token t and head:
    q = Wq h / sqrt(dim),  k = Wk h  (dim each),  v = Wv h  (vdim)
    a = sigmoid(Wa2 (Wa1 h) + b)^(1/tau)            a decay per key channel, in float32
    S_t = diag(a) S_(t-1) + k v^T                   the state [dim, vdim], float32, zero at a sequence's start
    o   = S_t^T q
    out = Wo concat_heads( rmsnorm(o) * gain * silu(Wg h) )      the norm over vdim, one gain for all heads
The state lives in the cache's per-sequence state ([slots, H, dim, vdim]); a step walks its new tokens in
order from the state the steps before left, so a prompt, its pieces and single tokens give the same result.

Order of work: q, k, v and the gate are one product with the stacked matrix; the decay's two small products; the
recurrence (``ops.gla_recurrent``, which also turns the decay's projection into the decay); norm and gate in one
kernel; the output projection.
"""
from __future__ import annotations

import torch

from .. import ops
from ..profiler import section
from .base import CacheRequest, Mixer
from .registry import ParamInfo, register_mixer


@register_mixer("gla")
class GatedLinearAttention(Mixer):
    graph_safe = True

    @classmethod
    def param_infos(cls, spec):
        D, H, r = spec.hidden_size, spec.num_heads, spec.decay_rank
        return {"q": ParamInfo((H * spec.dim, D)), "k": ParamInfo((H * spec.dim, D)), "v": ParamInfo((H * spec.vdim, D)),
                "g": ParamInfo((H * spec.vdim, D)), "o": ParamInfo((D, H * spec.vdim)), "norm": ParamInfo((spec.vdim,), "gain"),
                "a1": ParamInfo((r, D)), "a2": ParamInfo((H * spec.dim, r)), "a2.b": ParamInfo((H * spec.dim,), "gain")}

    def load(self, tensors):
        s = self.spec
        self.proj = torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0).contiguous()
        self.q_col, self.k_col = 0, s.num_heads * s.dim
        self.v_col = 2 * s.num_heads * s.dim
        self.g_col = self.v_col + s.num_heads * s.vdim
        self.a1, self.a2, self.bias = tensors["a1"].contiguous(), tensors["a2"].contiguous(), tensors["a2.b"]
        self.gain, self.o = tensors["norm"], tensors["o"].contiguous()

    def weight_bytes(self):
        return (self.proj.numel() + self.a1.numel() + self.a2.numel() + self.o.numel()) * self.proj.element_size()

    def reads_first(self):
        return self.proj

    def cache_request(self):
        s = self.spec
        return CacheRequest(state_shape=(s.num_heads, s.dim, s.vdim), state_dtype=torch.float32)

    def __call__(self, x, ctx, cache):
        s = self.spec
        H = s.num_heads
        with section("gla q/k/v/gate proj"):
            proj = ops.linear(x, self.proj)
        with section("gla decay proj"):
            z = ops.linear(ops.linear(x, self.a1), self.a2)
        with section("gla recurrence"):
            o = ops.gla_recurrent(proj, self.q_col, self.k_col, self.v_col, z, self.bias, s.tau, s.dim ** -0.5, cache.state,
                                  ctx.seq_slot, ctx.seq_start, H, s.dim, s.vdim, single=ctx.decode_only)
        with section("gla norm/gate"):
            y = ops.head_norm_gate(o, self.gain, s.eps, proj[:, self.g_col:self.g_col + H * s.vdim], self.env.dtype, "silu")
        with section("gla o proj"):
            return ops.linear(y, self.o)
