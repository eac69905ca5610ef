"""Latent attention: keys and values of all heads are expanded from one cached latent per token.

With h the mixer's input, per token:
    q      = Wq h                       per head [dim plain, rot_dim to rotate]
    down   = Wdkv h                     [kv_rank + rot_dim]
    c      = rmsnorm(down[:kv_rank])    the latent (gain ``dkv.norm``)
    r      = rotate(down[kv_rank:])     one rotated key part for all heads
    k_h    = [Wuk_h c, r],  v_h = Wuv_h c
    score  = (q_plain . Wuk_h c + rotate(q_rot) . r) * scale,  causal, the last ``window`` keys
    softmax, with exp(sink_h) in the denominator if the record says so
    out    = Wo concat_h(gate_h * sum_j p_j v_hj),  gate = sigmoid(Wg h) per head or per element
Only [c, r] is cached: one row of kv_rank + rot_dim per token.

Order of work here: the three projections of h are one product with the stacked matrix; the key up-projection
is folded into the query (qa_h = Wuk_h^T q_plain: a product per head), so that the score against a cached row is
qa_h . c + rotate(q_rot) . r and attention runs as H query heads over ONE key head of kv_rank + rot_dim elements
whose values are the keys themselves (the cache keeps one pool; the attention kernels get it as both).  The
first kv_rank elements of the result are the weighted sum of latents, to which the value up-projection is
applied per head; then the gate and the output projection.  Prompts, pieces of prompts and single tokens take the
same path.
"""
from __future__ import annotations

import torch

from .. import ops
from ..profiler import section
from .base import CacheRequest, Mixer
from .registry import ParamInfo, build_part, register_mixer

GATES = ("", "head", "element")


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.gate not in GATES:
            raise ValueError(f"gate {spec.gate!r} is not built (known: head, element, none)")
        if spec.rot_dim % 2:
            raise ValueError(f"rot_dim {spec.rot_dim} must be even")
        self.position = build_part("position", spec.position, env)
        if spec.rot_dim and not getattr(self.position, "pairs", False):
            raise ValueError(f"latent attention turns neighbouring pairs; position kind {spec.position.kind!r} does not")
        self.sink = None

    @classmethod
    def gate_rows(cls, spec) -> int:
        return {"": 0, "head": spec.num_heads, "element": spec.num_heads * spec.vdim}[spec.gate]

    @classmethod
    def param_infos(cls, spec):
        D, H = spec.hidden_size, spec.num_heads
        infos = {"q": ParamInfo((H * (spec.dim + spec.rot_dim), D)), "dkv": ParamInfo((spec.kv_rank + spec.rot_dim, D)),
                 "dkv.norm": ParamInfo((spec.kv_rank,), "gain"), "uk": ParamInfo((H * spec.dim, spec.kv_rank)),
                 "uv": ParamInfo((H * spec.vdim, spec.kv_rank)), "o": ParamInfo((D, H * spec.vdim))}
        if spec.sink:
            infos["sink"] = ParamInfo((H,), "gain")
        if spec.gate:
            infos["g"] = ParamInfo((cls.gate_rows(spec), D))
        return infos

    def load(self, tensors):
        s = self.spec
        H = s.num_heads
        stack = [tensors["q"], tensors["dkv"]] + ([tensors["g"]] if s.gate else [])
        self.proj = torch.cat(stack, dim=0).contiguous()
        self.q_col, self.dkv_col = 0, H * (s.dim + s.rot_dim)
        self.g_col = self.dkv_col + s.kv_rank + s.rot_dim
        self.latent_gain = tensors["dkv.norm"]
        # [H, kv_rank, dim]: qa_h = Wuk_h^T q_plain_h as a product per head
        self.uk_t = tensors["uk"].view(H, s.dim, s.kv_rank).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].view(H, s.vdim, s.kv_rank).contiguous()
        self.o = tensors["o"].contiguous()
        self.sink = tensors["sink"] if s.sink else None

    def weight_bytes(self):
        return (self.proj.numel() + self.uk_t.numel() + self.uv.numel() + self.o.numel()) * self.proj.element_size()

    def reads_first(self):
        return self.proj

    def cache_request(self):
        s = self.spec
        return CacheRequest(kv_heads=1, head_dim=s.kv_rank + s.rot_dim, window=s.window, shared_kv=True)

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    def __call__(self, x, ctx, cache):
        s = self.spec
        T, H, Dk = x.shape[0], s.num_heads, s.kv_rank + s.rot_dim
        with section("latent q/dkv/gate proj"):
            proj = ops.linear(x, self.proj)
        with section("latent key fold"):
            q = proj[:, :self.dkv_col].view(T, H, s.dim + s.rot_dim)
            qa = ops.linear_heads(q[:, :, :s.dim], self.uk_t)
        with section("latent norm/rope/append"):
            qf = ops.latent_prep(proj, self.q_col, self.dkv_col, qa, H, s.dim, s.rot_dim, s.kv_rank, self.latent_gain, s.eps,
                                 self.position.fused_table(), cache.k_pool, cache.page_table, ctx.tok_seq, ctx.tok_pos,
                                 ctx.seq_slot, write=cache.writes)
        pool = cache.k_pool
        fast = ops.fast_attention_supported(qf.dtype, Dk, cache.page_size)
        with section("attention"):
            if fast and ctx.decode_only:
                lat = ops.attention_decode(qf, pool, pool, cache.page_table, ctx.seq_slot, ctx.seq_len, s.scale, s.window,
                                           ctx.len_bucket, sink=self.sink)
            elif fast:
                lat = ops.attention_prefill(qf, pool, pool, cache.page_table, ctx.seq_slot, ctx.seq_start, ctx.seq_len,
                                            ctx.max_new, s.scale, s.window, sink=self.sink, v_dims=s.kv_rank)
            else:
                lat = ops.attention(qf, pool, pool, cache.page_table, ctx.seq_slot, ctx.seq_start, ctx.seq_len, ctx.max_new,
                                    s.scale, s.window, sink=self.sink)
        with section("latent value unfold"):
            heads = ops.linear_heads(lat[:, :, :s.kv_rank], self.uv)
        if s.gate:
            with section("latent gate"):
                ops.gate_heads(heads, proj[:, self.g_col:self.g_col + self.gate_rows(s)], "sigmoid")
        with section("attn o proj"):
            return ops.linear(heads.view(T, H * s.vdim), self.o)
