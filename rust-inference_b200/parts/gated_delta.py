"""The gated delta rule: a recurrent mixer with a matrix-valued state per head.

With h the mixer's input, per token and value head (query/key head = head // (heads // qk_heads)):
    q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))     a short causal convolution per channel
    q <- q / sqrt(sum q^2 + 1e-6) / sqrt(dim),   k <- k / sqrt(sum k^2 + 1e-6)
    beta = sigmoid(Wb h)                                               one per head
    g = exp(-exp(A_log) * softplus(Wa2 (Wa1 h) + dt_bias))             one decay per head and key channel
    S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q       S [dim, vdim], float32
    out = Wo concat_heads( o / rms(o) * gain * sigmoid(Wg2 (Wg1 h)) )          the norm over vdim, one gain for all heads
Everything after the projections' and the convolution's rounding is float32.  Per sequence the cache keeps the state S
([slots, H, dim, vdim]) and the convolution's last taps-1 inputs ([slots, taps-1, channels]); a step walks its new
tokens in order from what the steps before left, so a prompt, its pieces and single tokens give the same result.

Order of work: q, k, v, beta and the inner parts of the two low-rank projections are one product with the stacked
matrix; the two small outer products; convolution and silu (``ops.short_conv``); the recurrence
(``ops.delta_rule_recurrent``: unit vectors, decays, beta and the state); norm and gate in one kernel; the output
projection.
"""
from __future__ import annotations

import torch

from .. import ops
from ..profiler import section
from .base import CacheRequest, Mixer
from .registry import ParamInfo, register_mixer


@register_mixer("gated_delta")
class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.num_heads % spec.num_qk_heads:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_qk_heads} query/key heads")
        if spec.conv < 1:
            raise ValueError("the convolution has at least one tap")

    @classmethod
    def param_infos(cls, spec):
        D, H, G, dim, vdim = spec.hidden_size, spec.num_heads, spec.num_qk_heads, spec.dim, spec.vdim
        return {"q": ParamInfo((G * dim, D)), "k": ParamInfo((G * dim, D)), "v": ParamInfo((H * vdim, D)),
                "q.conv": ParamInfo((G * dim, spec.conv), "vector"), "k.conv": ParamInfo((G * dim, spec.conv), "vector"),
                "v.conv": ParamInfo((H * vdim, spec.conv), "vector"), "b": ParamInfo((H, D)),
                "A_log": ParamInfo((H,), "vector"), "norm": ParamInfo((vdim,), "gain"),
                "a1": ParamInfo((spec.decay_rank, D)), "a2": ParamInfo((H * dim, spec.decay_rank)),
                "dt_bias": ParamInfo((H * dim,), "vector"), "g1": ParamInfo((spec.gate_rank, D)),
                "g2": ParamInfo((H * vdim, spec.gate_rank)), "o": ParamInfo((D, H * vdim))}

    def load(self, tensors):
        s = self.spec
        qk, vw = s.num_qk_heads * s.dim, s.num_heads * s.vdim

        def rows8(t):            # zero rows up to a multiple of 8: every block of columns of the product starts on 16 bytes
            pad = -t.shape[0] % 8
            return t if not pad else torch.cat([t, t.new_zeros((pad, t.shape[1]))], dim=0)

        def cols8(t):            # ... and the matrices that read the padded blocks get zero columns
            pad = -t.shape[1] % 8
            return t if not pad else torch.cat([t, t.new_zeros((t.shape[0], pad))], dim=1)

        blocks = [rows8(torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0)), rows8(tensors["b"]),
                  rows8(tensors["a1"]), rows8(tensors["g1"])]
        self.proj = torch.cat(blocks, dim=0).contiguous()
        self.channels = 2 * qk + vw
        self.q_col, self.k_col, self.v_col = 0, qk, 2 * qk
        self.b_col = blocks[0].shape[0]
        self.a_col = self.b_col + blocks[1].shape[0]
        self.g_col = self.a_col + blocks[2].shape[0]
        self.a_rank, self.g_rank = blocks[2].shape[0], blocks[3].shape[0]
        self.conv = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).contiguous()
        self.conv_t = self.conv.t().contiguous()            # [taps, channels]: what the kernel of eight channels per thread reads
        self.a2, self.g2 = cols8(tensors["a2"]).contiguous(), cols8(tensors["g2"]).contiguous()
        self.dt_bias, self.a_log, self.gain = tensors["dt_bias"], tensors["A_log"], tensors["norm"]
        self.o = tensors["o"].contiguous()

    def weight_bytes(self):
        return (self.proj.numel() + self.a2.numel() + self.g2.numel() + self.o.numel()) * self.proj.element_size()

    def reads_first(self):
        return self.proj

    def cache_request(self):
        s = self.spec
        return CacheRequest(state_shape=(s.num_heads, s.dim, s.vdim), state_dtype=torch.float32,
                            more_state=(((s.conv - 1, 2 * s.num_qk_heads * s.dim + s.num_heads * s.vdim), torch.float32),))

    def heads_out(self, x, ctx, cache):
        """Everything but the output projection: [tokens, H * vdim] in the compute dtype."""
        s = self.spec
        H = s.num_heads
        single = ctx.decode_only
        with section("delta q/k/v/beta/low-rank proj"):
            proj = ops.linear(x, self.proj)
        with section("delta decay and gate proj"):
            za = ops.linear(proj[:, self.a_col:self.a_col + self.a_rank].contiguous(), self.a2)
            zg = ops.linear(proj[:, self.g_col:self.g_col + self.g_rank].contiguous(), self.g2)
        with section("delta conv"):
            qkv = ops.short_conv(proj, 0, self.conv, cache.more_state[0], ctx.tok_seq, ctx.seq_slot, ctx.seq_start, single=single,
                                 weight_t=self.conv_t)
        with section("delta recurrence"):
            o = ops.delta_rule_recurrent(qkv, self.q_col, self.k_col, self.v_col, proj, self.b_col, za, self.dt_bias, self.a_log,
                                         s.dim ** -0.5, cache.state, ctx.seq_slot, ctx.seq_start, H, s.num_qk_heads, s.dim,
                                         s.vdim, single=single)
        with section("delta norm/gate"):
            return ops.head_norm_gate(o, self.gain, s.eps, zg, self.env.dtype, "sigmoid")

    def __call__(self, x, ctx, cache):
        y = self.heads_out(x, ctx, cache)
        with section("delta o proj"):
            return ops.linear(y, self.o)
