"""Causal grouped-query attention over the paged cache.

Order of work, as in thanhauco/rust-inference src/models/qwen3.rs:71-100:
q/k/v projections (one product with the stacked matrix), per-head RMSNorm of q
and k, position encoding, append k and v to the cache, attention over the
cache, output projection.  Norm, rotation and append are one kernel.

Sizes, the window (or the chunked mask), the scale, the per-head norm, the sink term and the
position encoding all come from the spec; the part does not know which model it is in.

Values of another size than the keys (``v_head_dim``): the kernels work with one head size, so the
part runs them at Dp = the larger of the two rounded up to 16 and pads at load: the query, key and
value matrices get zero rows (a zero query element times a zero key element adds exactly 0 to a
score), the output matrix zero columns.  Nothing of the padding reaches a result.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..profiler import section
from .base import CacheRequest, Mixer, PositionEncoding
from .registry import ParamInfo, build_part, register_mixer


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_kv_heads} kv heads")
        if spec.qk_norm is not None and getattr(spec.qk_norm, "kind", None) != "rmsnorm":
            raise ValueError(f"the attention part norms its heads with RMSNorm inside its kernel; a per-head norm of kind "
                             f"{getattr(spec.qk_norm, 'kind', None)!r} is not built")
        self.position = build_part("position", spec.position, env)
        self.scale = spec.scale or 1.0 / math.sqrt(spec.head_dim)
        self.q_gain = self.k_gain = self.sink = None
        self.Dk, self.Dv = spec.head_dim, (spec.v_head_dim or spec.head_dim)
        self.Dp = self.Dk if self.Dk == self.Dv else -(-max(self.Dk, self.Dv) // 16) * 16
        if self.Dp != self.Dk and spec.qk_norm is not None:
            raise ValueError("a per-head norm of queries and keys with values of another size is not built")
        if spec.window and spec.chunk:
            raise ValueError("an attention layer has a window or a chunked mask, not both")
        self.rot = getattr(spec.position, "rot", None) or getattr(spec.position, "rotary_dim", 0)
        if self.rot > self.Dk:
            raise ValueError(f"{self.rot} rotated elements in heads of {self.Dk}")

    @classmethod
    def param_infos(cls, spec):
        D, H, KV, Dh = spec.hidden_size, spec.num_heads, spec.num_kv_heads, spec.head_dim
        Dv = spec.v_head_dim or Dh
        q, k, v, o, sink = spec.names
        infos = {q: ParamInfo((H * Dh, D)), k: ParamInfo((KV * Dh, D)), v: ParamInfo((KV * Dv, D)), o: ParamInfo((D, H * Dv))}
        if spec.qk_norm is not None:
            infos["q_norm.weight"] = ParamInfo((Dh,), "gain")
            infos["k_norm.weight"] = ParamInfo((Dh,), "gain")
        if spec.sink:
            infos[sink] = ParamInfo((H,), "vector")
        return infos

    def load(self, tensors):
        s = self.spec
        q, k, v, o, sink = s.names
        D, Dp = s.hidden_size, self.Dp

        def rows(t, heads, size):          # [heads * size, D] -> [heads * Dp, D] with zero rows after each head's own
            if size == Dp:
                return t
            out = t.new_zeros((heads, Dp, D))
            out[:, :size] = t.view(heads, size, D)
            return out.view(heads * Dp, D)

        self.qkv = torch.cat([rows(tensors[q], s.num_heads, self.Dk), rows(tensors[k], s.num_kv_heads, self.Dk),
                              rows(tensors[v], s.num_kv_heads, self.Dv)], dim=0).contiguous()
        wo = tensors[o]
        if self.Dv != Dp:
            padded = wo.new_zeros((D, s.num_heads, Dp))
            padded[:, :, :self.Dv] = wo.view(D, s.num_heads, self.Dv)
            wo = padded.view(D, s.num_heads * Dp)
        self.o = wo.contiguous()
        if s.qk_norm is not None:
            self.q_gain, self.k_gain = tensors["q_norm.weight"], tensors["k_norm.weight"]
        if s.sink:
            self.sink = tensors[sink]

    def weight_bytes(self):
        return (self.qkv.numel() + self.o.numel()) * self.qkv.element_size()

    def reads_first(self):
        return self.qkv

    def cache_request(self):
        s = self.spec
        return CacheRequest(kv_heads=s.num_kv_heads, head_dim=self.Dp, window=s.window, chunk=s.chunk)

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    def __call__(self, x, ctx, cache):
        s = self.spec
        with section("attn q/k/v proj"):
            qkv = ops.linear(x, self.qkv)
        table = self.position.fused_table()
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        meta = (ctx.tok_seq, ctx.tok_pos, ctx.seq_slot)
        with section("attn norm/rope/append"):
            if table is not None or type(self.position).apply is PositionEncoding.apply:
                # norm, rotation (by table, or none) and append in one kernel
                rot = self.rot if table is not None else 0
                q = ops.qk_norm_rope_append(qkv, s.num_heads, s.num_kv_heads, self.Dp, self.q_gain, self.k_gain, eps,
                                            table, rot, cache.k_pool, cache.v_pool, cache.page_table, *meta,
                                            write_kv=cache.writes, pairs=getattr(self.position, "pairs", False))
            else:
                # a position encoding with a rule of its own: norm q and k, let it work on them, append
                T, H, KV, Dh = x.shape[0], s.num_heads, s.num_kv_heads, self.Dp
                qw, kw = H * Dh, KV * Dh
                q = ops.qk_norm_rope_append(qkv[:, :qw].contiguous(), H, 0, Dh, self.q_gain, None, eps, None, 0,
                                            None, None, None, *meta, write_kv=False)
                k = ops.qk_norm_rope_append(qkv[:, qw:qw + kw].contiguous(), KV, 0, Dh, self.k_gain, None, eps, None, 0,
                                            None, None, None, *meta, write_kv=False)
                q, k = self.position.apply(q, k, ctx)
                if cache.writes:
                    kv = torch.cat([k.reshape(T, kw), qkv[:, qw + kw:]], dim=1).contiguous()
                    ops.qk_norm_rope_append(kv, 0, KV, Dh, None, None, eps, None, 0, cache.k_pool, cache.v_pool,
                                            cache.page_table, *meta, write_kv=True)
                q = q.contiguous()
        fast = ops.fast_attention_supported(q.dtype, self.Dp, cache.page_size)
        with section("attention"):
            if fast and ctx.decode_only:
                out = ops.attention_decode(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_len,
                                           self.scale, s.window, ctx.len_bucket, sink=self.sink, chunk=s.chunk)
            elif fast:
                out = ops.attention_prefill(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot,
                                            ctx.seq_start, ctx.seq_len, ctx.max_new, self.scale, s.window, sink=self.sink,
                                            chunk=s.chunk)
            else:
                out = ops.attention(q, cache.k_pool, cache.v_pool, cache.page_table, ctx.seq_slot, ctx.seq_start,
                                    ctx.seq_len, ctx.max_new, self.scale, s.window, sink=self.sink, chunk=s.chunk)
        with section("attn o proj"):
            return ops.linear(out.view(x.shape[0], s.num_heads * self.Dp), self.o)
