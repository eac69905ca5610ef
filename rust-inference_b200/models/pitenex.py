"""Pitenex: a decoder whose layers run a mixer and a feed-forward side by side behind one layer norm (with bias),
x <- x + residual_mult * (mixer(h) + ff(h)).  The mixer is itself two mixers side by side, a weighted sum of
grouped-query attention (keys and values of different sizes, rotation of neighbouring pairs, a mask of chunks counted
from the sequence's start, a sink term in the softmax) and the gated delta rule (short convolutions, unit-norm queries
and keys, a decay per key channel).  Feed-forwards are dense (gelu-gated) or routed (clamped swish experts, identity
experts, a shared expert).  The embedding adds a hashed table of (previous token, token) pairs; the output matrix is
the embedding table, and the logits are multiplied by a constant.

config.json keys (every size and every constant that may differ between models comes from here)::

    architecture              "Pitenex"
    vocab, width              sizes of the embedding table
    embedding.bigram          {buckets, mul_prev, mul_cur}: row (prev * mul_prev + token * mul_cur) mod buckets of the
                              tensor ``bigram`` [buckets + 1, width]; a sequence's first token takes row ``buckets``
    norm.eps                  eps of every norm (layer norms and the RMS norm over the delta rule's heads)
    residual_mult             factor on what a layer adds to the residual
    logit_scale               factor on the logits
    layers[i]                 {type "parallel", mixer, mlp}
      mixer.left              heads, kv_heads, dim (queries and keys), vdim (values), scale, rot {base, dims},
                              mask {size} (absent: every earlier key)
      mixer.right             heads, kv_heads (query/key heads), dim, vdim, conv (taps); the inner sizes of its two
                              low-rank projections are ``decay_rank`` and ``gate_rank`` if the record has them, else
                              they are read from the shapes of ``a1`` and ``g1`` when a checkpoint is loaded
      mixer.left_scale, mixer.right_scale
      mlp                     null, {kind "dense", ff} or {kind "moe", router {experts, identity, top},
                              expert {ff, limit}, shared {ff, limit} (optional)}

Tensor names: ``embed``, ``bigram``, ``final.norm`` (+ ``.b``), and per layer i ``l<i>.norm1`` (+ ``.b``),
``l<i>.mix.left.q|k|v|o|sink``, ``l<i>.mix.right.q|k|v`` (+ ``.conv``) ``|b|A_log|norm|a1|a2|dt_bias|g1|g2|o``,
``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router|correction|e<j>.gate|up|down|shared.gate|up|down``.
The model itself is not written here: ``to_spec`` names the parts and the generic model runs them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, GatedDeltaSpec, GatedFFSpec, HeadSpec, HyperConnectionSpec, LayerNormSpec,
                            ModelSpec, MoESpec, NoPositionSpec, PairHashEmbeddingSpec, ParallelLayerSpec, ParallelMixerSpec,
                            RopePairsSpec, ScheduleEntry)
from .ranudra import MAX_POSITIONS, _checkpoint_shapes, _freeze, _get, _pos_int, _thaw

SWISH_ALPHA = 1.702          # the experts' gate: g sigmoid(1.702 g)
LAYER_TYPES = ("parallel",)


@register_architecture("Pitenex", "pitenex")
@dataclass(frozen=True)
class PitenexConfig:
    vocab: int
    width: int
    buckets: int
    mul_prev: int
    mul_cur: int
    eps: float
    residual_mult: float
    logit_scale: float
    layers: Tuple[tuple, ...]                    # frozen layer records of config.json
    eos_token_ids: Tuple[int, ...] = ()

    # ---- config.json <-> object -------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "PitenexConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        big = (d.get("embedding") or {}).get("bigram")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                   buckets=_pos_int(big, "buckets", "embedding.bigram"), mul_prev=_get(big, "mul_prev", "embedding.bigram", int),
                   mul_cur=_get(big, "mul_cur", "embedding.bigram", int), eps=float(_get(d.get("norm"), "eps", "norm")),
                   residual_mult=float(_get(d, "residual_mult", "config")), logit_scale=float(_get(d, "logit_scale", "config")),
                   layers=tuple(_freeze(l) for l in layers), eos_token_ids=eos_ids)

    def layer_records(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self) -> dict:
        d = {"architecture": "Pitenex", "vocab": self.vocab, "width": self.width,
             "embedding": {"bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
             "norm": {"eps": self.eps}, "residual_mult": self.residual_mult, "logit_scale": self.logit_scale,
             "layers": self.layer_records()}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- checks ------------------------------------------------------------------
    def validate(self) -> None:
        if not (self.eps > 0):
            raise ConfigError("norm.eps must be positive")
        if self.mul_prev < 0 or self.mul_cur < 0:
            raise ConfigError("embedding.bigram: the multipliers must not be negative")
        for i, layer in enumerate(self.layer_records()):
            what = f"layers[{i}]"
            if layer.get("type") not in LAYER_TYPES:
                raise ConfigError(f"config.json: {what}.type {layer.get('type')!r} is not built (known: {', '.join(LAYER_TYPES)})")
            m = layer.get("mixer")
            left, right = (m or {}).get("left"), (m or {}).get("right")
            for key in ("left_scale", "right_scale"):
                _get(m, key, what + ".mixer")
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _pos_int(left, key, what + ".mixer.left")
                _pos_int(right, key, what + ".mixer.right")
            for side, rec in (("left", left), ("right", right)):
                if rec["heads"] % rec["kv_heads"]:
                    raise ConfigError(f"config.json: {what}.mixer.{side}: {rec['heads']} heads over {rec['kv_heads']} kv_heads")
            _get(left, "scale", what + ".mixer.left")
            rot = left.get("rot")
            if rot is not None and rot.get("dims", 0):
                dims = _pos_int(rot, "dims", what + ".mixer.left.rot")
                if dims % 2 or dims > left["dim"]:
                    raise ConfigError(f"config.json: {what}.mixer.left.rot.dims {dims} must be even and at most dim {left['dim']}")
                if not float(_get(rot, "base", what + ".mixer.left.rot")) > 0:
                    raise ConfigError(f"config.json: {what}.mixer.left.rot.base must be positive")
            if left.get("mask") is not None:
                _pos_int(left["mask"], "size", what + ".mixer.left.mask")
            _pos_int(right, "conv", what + ".mixer.right")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            kind = mlp.get("kind")
            if kind == "dense":
                _pos_int(mlp, "ff", what + ".mlp")
            elif kind == "moe":
                r = mlp.get("router")
                E, top = _pos_int(r, "experts", what + ".mlp.router"), _pos_int(r, "top", what + ".mlp.router")
                ident = int((r or {}).get("identity", 0) or 0)
                if ident < 0 or top > E + ident:
                    raise ConfigError(f"config.json: {what}.mlp.router: top {top} of {E} + {ident} experts")
                for part in ("expert", "shared"):
                    rec = mlp.get(part)
                    if rec is None and part == "shared":
                        continue
                    _pos_int(rec, "ff", f"{what}.mlp.{part}")
                    _get(rec, "limit", f"{what}.mlp.{part}")
            else:
                raise ConfigError(f"config.json: {what}.mlp.kind {kind!r} is not built (known: dense, moe)")

    # ---- the model as parts --------------------------------------------------------
    def _mixer(self, m):
        D = self.width
        left, right = m["left"], m["right"]
        rot = left.get("rot") or {}
        position = NoPositionSpec()
        if rot.get("dims", 0):
            position = RopePairsSpec(rotary_dim=int(rot["dims"]), theta=float(rot["base"]))
        attn = AttentionSpec(hidden_size=D, num_heads=left["heads"], num_kv_heads=left["kv_heads"], head_dim=left["dim"],
                             position=position, scale=float(left["scale"]), chunk=int((left.get("mask") or {}).get("size", 0)),
                             sink=True, v_head_dim=left["vdim"], names=("q", "k", "v", "o", "sink"))
        delta = GatedDeltaSpec(hidden_size=D, num_heads=right["heads"], num_qk_heads=right["kv_heads"], dim=right["dim"],
                               vdim=right["vdim"], conv=right["conv"], decay_rank=int(right.get("decay_rank", 0)),
                               gate_rank=int(right.get("gate_rank", 0)), eps=self.eps)
        return ParallelMixerSpec(left=attn, right=delta, left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))

    def _ffn(self, mlp):
        D = self.width
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return GatedFFSpec(hidden_size=D, intermediate_size=mlp["ff"], gate="gelu_tanh")

        def clamped(rec):
            return GatedFFSpec(hidden_size=D, intermediate_size=rec["ff"], gate="clamped_swish", limit=float(rec["limit"]),
                               alpha=SWISH_ALPHA)
        r = mlp["router"]
        shared = mlp.get("shared")
        return MoESpec(hidden_size=D, experts=r["experts"], top=r["top"], expert=clamped(mlp["expert"]),
                       identity=int(r.get("identity", 0) or 0), shared=None if shared is None else clamped(shared))

    def to_spec(self) -> ModelSpec:
        D = self.width
        norm = LayerNormSpec(size=D, eps=self.eps, weight_name="", bias_name=".b")
        link = HyperConnectionSpec(streams=1, learned=False, scale=self.residual_mult)
        layers = []
        for i, layer in enumerate(self.layer_records()):
            names = [("norm", f"l{i}.norm1"), ("mixer", f"l{i}.mix."), ("ffn", f"l{i}.mlp."), ("link", f"l{i}.")]
            layers.append(ParallelLayerSpec(mixer=self._mixer(layer["mixer"]), norm=norm, link=link,
                                            ffn=self._ffn(layer.get("mlp")), names=tuple(names)))
        schedule = tuple(ScheduleEntry(layer=i, cache=i) for i in range(len(layers)))
        return ModelSpec(
            architecture="Pitenex", vocab_size=self.vocab, hidden_size=D, layers=tuple(layers), schedule=schedule,
            final_norm=norm, tie_embeddings=True, max_positions=MAX_POSITIONS, embedding_name="embed", head_name="embed",
            final_norm_prefix="final.norm", stop_ids=self.eos_token_ids, head_optional=False,
            embedding=PairHashEmbeddingSpec(self.vocab, D, buckets=self.buckets, mul_prev=self.mul_prev,
                                            mul_cur=self.mul_cur, pairs_name="bigram"),
            head=HeadSpec(self.vocab, D, scale=self.logit_scale), end_names=(("bigram", "bigram"),))

    # ---- sizes that only the checkpoint knows -------------------------------------------------------
    def with_checkpoint(self, model_dir: str) -> "PitenexConfig":
        """The configuration with the sizes that config.json leaves to the tensors' shapes filled in: the inner sizes of
        the delta rule's low-rank projections, from ``l<i>.mix.right.a1`` and ``.g1``."""
        shapes = None
        out = []
        for i, layer in enumerate(self.layer_records()):
            right = dict(layer["mixer"]["right"])
            for key, tensor in (("decay_rank", "a1"), ("gate_rank", "g1")):
                if key in right:
                    continue
                if shapes is None:
                    shapes = _checkpoint_shapes(model_dir)
                shape = shapes.get(f"l{i}.mix.right.{tensor}")
                if shape is None or len(shape) != 2:
                    raise ConfigError(f"{model_dir}: l{i}.mix.right.{tensor} is missing, so a low-rank projection's inner size is unknown")
                right[key] = int(shape[0])
            layer = dict(layer, mixer=dict(layer["mixer"], right=right))
            out.append(_freeze(layer))
        return PitenexConfig(self.vocab, self.width, self.buckets, self.mul_prev, self.mul_cur, self.eps, self.residual_mult,
                             self.logit_scale, tuple(out), self.eos_token_ids)
