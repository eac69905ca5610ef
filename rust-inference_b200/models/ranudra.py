"""Ranudra: a decoder whose layers mix latent attention (two variants) and gated linear attention, with
squared-relu feed-forwards, a residual that may be kept as several streams (hyper-connections), a run of
layers that may repeat with shared weights, and an output matrix tied to the (scaled) embedding.

config.json keys (every size and every constant that may differ between models comes from here)::

    architecture        "Ranudra"
    vocab, width        sizes of the embedding table
    embedding.scale     factor on the embedding's rows (the tied output matrix is the table without it)
    norm.eps            eps of every norm (layer norms and the RMS norms inside the mixers)
    streams             optional: number of residual streams; with it every sublayer has connection tensors
    loop                optional: {start, stop, times}: layers start .. stop-1 run ``times`` times in a row with
                        the same weights and a cache or state of their own per pass, then the rest follow
    layers[i]           {type, mixer, mlp}: type "latent_attention", "latent_attention_2" or "gla"; mixer: its
                        sizes; mlp: {kind "dense", ff} or null for a layer without feed-forward

Mixer records: latent attention has heads, dim, rot_dim, vdim, kv_rank, scale, mask.size (window; absent: all keys)
and rot {base, dims, scaling {factor, original, fast, slow} (absent: plain frequencies)}; "latent_attention" gates
each head with one sigmoid, "latent_attention_2" gates every output element and has a sink per head in the softmax.
Gated linear attention has heads, dim, vdim and tau; the inner size of its decay projection is read from ``decay_rank``
if the record has it, else from the tensor's shape when a checkpoint is loaded.

Tensor names: ``embed``, ``final.norm``, and per layer i ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``,
``l<i>.hc1|hc2.in|out|mix``.  The model itself is not written here: ``to_spec`` names the parts and the order in
which the generic model runs them (``engine/model.py``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (DenseFFSpec, EmbeddingSpec, GLASpec, HyperConnectionSpec, LatentAttentionSpec, LayerNormSpec,
                            ModelSpec, NoPositionSpec, RopePairsSpec, ScheduleEntry, StreamLayerSpec)

MIXER_TYPES = ("latent_attention", "latent_attention_2", "gla")
MAX_POSITIONS = 1 << 24          # the design has no limit of its own; the cache's size sets the real one


def _get(d, key, what, kind=(int, float)):
    if not isinstance(d, dict) or key not in d:
        raise ConfigError(f"config.json: {what} lacks {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, kind):
        raise ConfigError(f"config.json: {what}.{key} has the wrong type: {v!r}")
    return v


def _pos_int(d, key, what):
    v = _get(d, key, what, int)
    if v <= 0:
        raise ConfigError(f"config.json: {what}.{key} must be positive, got {v}")
    return v


def _freeze(v):
    if isinstance(v, list):
        return tuple(_freeze(x) for x in v)
    if isinstance(v, dict):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    return v


def _thaw(v):
    if isinstance(v, tuple) and v and all(isinstance(x, tuple) and len(x) == 2 and isinstance(x[0], str) for x in v):
        return {k: _thaw(x) for k, x in v}
    if isinstance(v, tuple):
        return [_thaw(x) for x in v]
    return v


@register_architecture("Ranudra", "ranudra")
@dataclass(frozen=True)
class RanudraConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: Tuple[tuple, ...]                    # frozen layer records of config.json
    streams: Optional[int] = None
    loop: Optional[Tuple[int, int, int]] = None  # (start, stop, times)
    eos_token_ids: Tuple[int, ...] = ()

    # ---- config.json <-> object -------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "RanudraConfig":
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (_get(lp, "start", "loop", int), _get(lp, "stop", "loop", int), _get(lp, "times", "loop", int))
        streams = d.get("streams")
        if streams is not None and (isinstance(streams, bool) or not isinstance(streams, int)):
            raise ConfigError(f"config.json: streams must be an integer, got {streams!r}")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else tuple(int(e) for e in (eos if isinstance(eos, list) else [eos]))
        return cls(vocab=_pos_int(d, "vocab", "config"), width=_pos_int(d, "width", "config"),
                   embedding_scale=float(_get(d.get("embedding"), "scale", "embedding")),
                   eps=float(_get(d.get("norm"), "eps", "norm")), layers=tuple(_freeze(l) for l in layers),
                   streams=streams, loop=loop, eos_token_ids=eos_ids)

    def layer_records(self):
        return [_thaw(l) for l in self.layers]

    def to_dict(self) -> dict:
        d = {"architecture": "Ranudra", "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": self.layer_records()}
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    # ---- checks ------------------------------------------------------------------
    def validate(self) -> None:
        if not (self.eps > 0):
            raise ConfigError("norm.eps must be positive")
        if self.streams is not None and not 1 <= self.streams <= 16:
            raise ConfigError(f"streams must be between 1 and 16, got {self.streams}")
        n = len(self.layers)
        if self.loop is not None:
            start, stop, times = self.loop
            if not (0 <= start <= stop <= n) or times < 1:
                raise ConfigError(f"loop {self.loop} does not fit {n} layers")
        for i, layer in enumerate(self.layer_records()):
            what = f"layers[{i}]"
            kind = layer.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {what}.type {kind!r} is not built (known: {', '.join(MIXER_TYPES)})")
            m = layer.get("mixer")
            for key in ("heads", "dim", "vdim"):
                _pos_int(m, key, what + ".mixer")
            if kind == "gla":
                if not float(_get(m, "tau", what + ".mixer")) > 0:
                    raise ConfigError(f"config.json: {what}.mixer.tau must be positive")
            else:
                _pos_int(m, "kv_rank", what + ".mixer")
                rot = _get(m, "rot_dim", what + ".mixer", int)
                if rot < 0 or rot % 2:
                    raise ConfigError(f"config.json: {what}.mixer.rot_dim must be even and not negative, got {rot}")
                _get(m, "scale", what + ".mixer")
                if rot:
                    r = m.get("rot")
                    if not float(_get(r, "base", what + ".mixer.rot")) > 1:
                        raise ConfigError(f"config.json: {what}.mixer.rot.base must exceed 1")
                    if r.get("dims", rot) != rot:
                        raise ConfigError(f"config.json: {what}.mixer.rot.dims {r['dims']} differs from rot_dim {rot}")
                    if r.get("scaling") is not None:
                        for key in ("factor", "original", "fast", "slow"):
                            if not float(_get(r["scaling"], key, what + ".mixer.rot.scaling")) > 0:
                                raise ConfigError(f"config.json: {what}.mixer.rot.scaling.{key} must be positive")
                if m.get("mask") is not None and _get(m["mask"], "size", what + ".mixer.mask", int) < 1:
                    raise ConfigError(f"config.json: {what}.mixer.mask.size must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {what}.mlp.kind {mlp.get('kind')!r} is not built (known: dense)")
                _pos_int(mlp, "ff", what + ".mlp")

    # ---- the model as parts --------------------------------------------------------
    def _mixer(self, kind, m):
        D = self.width
        if kind == "gla":
            return GLASpec(hidden_size=D, num_heads=m["heads"], dim=m["dim"], vdim=m["vdim"], tau=float(m["tau"]),
                           decay_rank=int(m.get("decay_rank", 0)), eps=self.eps)
        rot = m["rot_dim"]
        position = NoPositionSpec()
        if rot:
            r = m["rot"]
            sc = r.get("scaling")
            yarn = None if sc is None else (float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"]))
            position = RopePairsSpec(rotary_dim=rot, theta=float(r["base"]), yarn=yarn)
        second = kind == "latent_attention_2"
        return LatentAttentionSpec(hidden_size=D, num_heads=m["heads"], dim=m["dim"], rot_dim=rot, vdim=m["vdim"],
                                   kv_rank=m["kv_rank"], scale=float(m["scale"]), eps=self.eps, position=position,
                                   window=int((m.get("mask") or {}).get("size", 0)), sink=second,
                                   gate="element" if second else "head")

    def to_spec(self) -> ModelSpec:
        D = self.width
        S = self.streams
        norm = LayerNormSpec(size=D, eps=self.eps, weight_name="")
        link = HyperConnectionSpec(streams=S or 1, learned=S is not None)
        layers = []
        for i, layer in enumerate(self.layer_records()):
            mlp = layer.get("mlp")
            names = [("mixer", f"l{i}.mix."), ("mixer_norm", f"l{i}.norm1"), ("mixer_link", f"l{i}.hc1.")]
            if mlp is not None:
                names += [("ffn", f"l{i}.mlp."), ("ffn_norm", f"l{i}.norm2"), ("ffn_link", f"l{i}.hc2.")]
            layers.append(StreamLayerSpec(
                mixer=self._mixer(layer["type"], layer["mixer"]), mixer_norm=norm, mixer_link=link,
                ffn=None if mlp is None else DenseFFSpec(hidden_size=D, intermediate_size=mlp["ff"], activation="relu2"),
                ffn_norm=None if mlp is None else norm, ffn_link=None if mlp is None else link, names=tuple(names)))
        n = len(layers)
        start, stop, times = self.loop if self.loop is not None else (0, 0, 1)
        order = list(range(start)) + list(range(start, stop)) * times + list(range(stop, n))
        # every run of a layer has a cache entry of its own: a repeated layer shares weights, not keys or state
        schedule = tuple(ScheduleEntry(layer=i, cache=run) for run, i in enumerate(order))
        return ModelSpec(
            architecture="Ranudra", vocab_size=self.vocab, hidden_size=D, layers=tuple(layers), schedule=schedule,
            final_norm=norm, tie_embeddings=True, max_positions=MAX_POSITIONS, embedding_name="embed",
            head_name="embed", final_norm_prefix="final.norm", stop_ids=self.eos_token_ids, head_optional=False,
            embedding=EmbeddingSpec(self.vocab, D, scale=self.embedding_scale, copies=S or 1))

    # ---- sizes that only the checkpoint knows -------------------------------------------------------
    def with_checkpoint(self, model_dir: str) -> "RanudraConfig":
        """The configuration with the sizes that config.json leaves to the tensors' shapes filled in (the inner size
        of a gla layer's decay projection, from ``l<i>.mix.a1``)."""
        shapes = None
        out = []
        for i, layer in enumerate(self.layer_records()):
            if layer["type"] == "gla" and "decay_rank" not in layer["mixer"]:
                if shapes is None:
                    shapes = _checkpoint_shapes(model_dir)
                shape = shapes.get(f"l{i}.mix.a1")
                if shape is None or len(shape) != 2:
                    raise ConfigError(f"{model_dir}: l{i}.mix.a1 is missing, so the decay projection's inner size is unknown")
                layer = dict(layer, mixer=dict(layer["mixer"], decay_rank=int(shape[0])))
            out.append(_freeze(layer))
        return RanudraConfig(self.vocab, self.width, self.embedding_scale, self.eps, tuple(out), self.streams, self.loop,
                             self.eos_token_ids)


def _checkpoint_shapes(model_dir: str) -> dict:
    from ..weights.safetensors_io import Checkpoint, SafetensorsError
    try:
        ckpt = Checkpoint(model_dir)
        return {name: tuple(ckpt.shape_dtype(name)[0]) for name in ckpt.names()}
    except SafetensorsError as e:
        raise ConfigError(f"cannot read the tensor list of {model_dir}: {e}") from e
