"""The Lovurax decoder's configuration, read from its own config.json keys.

Lovurax is a pre-norm decoder over a 32-bit residual stream with root-mean-square norms, a gate on every residual sum and logits
against the embedding table times ``logit_scale``. ``layers`` lists its layers: each names its mixer by ``type`` with the mixer's
sizes under ``mixer`` and its feed-forward under ``mlp`` (``dense``: W_down act(W_up h) with the xIELU activation; null: none).
Mixers: ``retention`` (a matrix state a head that fades by its ``decay`` a token, q and k rotated in split halves over ``rot.dims`` elements),
``attention`` (grouped heads, normed queries and keys, a query temperature ``q_temp`` that grows with the position, a bias that
grows with the distance, a sigmoid of each score as that key's weight, a bias a head, an output gate) and ``latent_attention`` (keys and
values made from one cached latent vector of ``kv_rank`` numbers a token, nothing that depends on the position, a softmax, a gate a head). Every sublayer's
output is multiplied by sigmoid(W h + b) of the sublayer's own input before it joins the stream. Tensor names: ``embed``,
``l<i>.norm1`` / ``.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.rg1`` / ``.rg2`` with ``.b``, ``final.norm``. No size and no
constant that config.json gives stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .reader import ConfigError, ConfigReader
from .spec import (BlockSpec, DenseMlpSpec, GatedResidualSpec, LatentAttentionSpec, ModelSpec, NormSpec, PositionSpec, RetentionSpec, RunEntry,
                   ScaledEmbeddingSpec, ScaledHeadSpec, SigmoidAttentionSpec)

ARCHITECTURE = "Lovurax"
SLOPE_RATE = 8.0               # the design's constant in the attention's distance bias: slope_h = 2^(-8 (h + 1) / heads)


@dataclass(frozen=True)
class LovuraxLayer:
    type: str
    mixer: dict            # the mixer's sizes and constants, checked and typed
    mlp: dict | None


def _positive_float(r: ConfigReader, key: str) -> float:
    v = r.opt_float(key)
    if v is None or not v > 0:
        raise ConfigError(f"{r.source}: key '{key}' must be a positive number")
    return v


def _object(r: ConfigReader, key: str) -> ConfigReader:
    o = r.opt_object(key)
    if o is None:
        raise ConfigError(f"{r.source}: key '{key}' is absent")
    return o


def head_slopes(heads: int) -> tuple:
    return tuple(2.0 ** (-SLOPE_RATE * (h + 1) / heads) for h in range(heads))


@dataclass
class LovuraxConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: tuple
    tie_word_embeddings: bool = True
    warnings: list = field(default_factory=list)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_reader(cls, c: ConfigReader) -> "LovuraxConfig":
        vocab, width = c.positive_int("vocab"), c.positive_int("width")
        eps = _positive_float(_object(c, "norm"), "eps")
        logit_scale = c.opt_float("logit_scale")
        if logit_scale is None:
            logit_scale = 1.0
        raw = c.raw("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError(f"{c.source}: key 'layers' must be a non-empty list")
        readers = {"retention": cls._read_retention, "attention": cls._read_attention, "latent_attention": cls._read_latent}
        layers = []
        for i, item in enumerate(raw):
            lr = ConfigReader(item, f"{c.source}: layers[{i}]")
            kind = lr.opt_str("type")
            if kind not in readers:
                raise ConfigError(f"{lr.source}: key 'type' is {kind!r}; the design has {', '.join(readers)} mixers")
            layers.append(LovuraxLayer(kind, readers[kind](_object(lr, "mixer")), cls._read_mlp(lr.opt_object("mlp"))))
        return cls(vocab=vocab, width=width, eps=eps, logit_scale=float(logit_scale), layers=tuple(layers))

    @staticmethod
    def _read_retention(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "dim", "vdim")}
        decay = m.raw("decay")
        if not isinstance(decay, list) or len(decay) != out["heads"] or not all(isinstance(d, (int, float)) and 0 <= d <= 1 for d in decay):
            raise ConfigError(f"{m.source}: key 'decay' must list one number between 0 and 1 for each of the {out['heads']} heads")
        out["decay"] = tuple(float(d) for d in decay)
        rot = _object(m, "rot")
        out["rot_dims"], out["rot_base"] = rot.positive_int("dims"), _positive_float(rot, "base")
        if out["rot_dims"] % 2 or out["rot_dims"] > out["dim"]:
            raise ConfigError(f"{rot.source}: key 'dims' is {out['rot_dims']}; it must be even and at most dim {out['dim']}")
        return out

    @staticmethod
    def _read_attention(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "kv_heads", "dim", "vdim")}
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"{m.source}: {out['heads']} heads are not a multiple of {out['kv_heads']} kv_heads")
        out["scale"] = _positive_float(m, "scale")
        temp = m.opt_object("q_temp")
        out["temp_coef"], out["temp_every"] = 0.0, 1
        if temp is not None:
            coef = temp.opt_float("coef")
            if coef is None or coef < 0:
                raise ConfigError(f"{temp.source}: key 'coef' must be a number that is not negative")
            out["temp_coef"], out["temp_every"] = float(coef), temp.positive_int("every")
        return out

    @staticmethod
    def _read_latent(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "dim", "vdim", "kv_rank")}
        out["scale"] = _positive_float(m, "scale")
        return out

    @staticmethod
    def _read_mlp(f: ConfigReader | None) -> dict | None:
        if f is None:
            return None
        kind = f.opt_str("kind")
        if kind == "dense":
            return {"kind": "dense", "ff": f.positive_int("ff")}
        raise ConfigError(f"{f.source}: key 'kind' is {kind!r}; the design has dense feed-forwards")

    @classmethod
    def from_dict(cls, values: dict, source: str = "config") -> "LovuraxConfig":
        return cls.from_reader(ConfigReader(values, source))

    # ------------------------------------------------------------------ the model as parts
    def to_spec(self, tied: bool | None = None) -> ModelSpec:
        W = self.width
        norm = NormSpec(size=W, eps=self.eps, kind="rms_norm_wide")
        gate = GatedResidualSpec(hidden=W)
        names: dict = {"embed": {"table": ("embed",)}, "final_norm": {"weight": ("final.norm",)}}
        blocks = []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer.mixer
            q = p + "mix."
            if layer.type == "retention":
                mixer = RetentionSpec(hidden=W, num_heads=m["heads"], head_dim=m["dim"], v_dim=m["vdim"], decay=m["decay"], eps=self.eps,
                                      position=PositionSpec(kind="rope_neox", rotary_dim=m["rot_dims"], theta=m["rot_base"]))
                mix_names = {"in": (q + "q", q + "k", q + "v", q + "g"), "out": (q + "o",)}
            elif layer.type == "attention":
                mixer = SigmoidAttentionSpec(hidden=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
                                             scale=m["scale"], qk_norm_eps=self.eps, temp_coef=m["temp_coef"], temp_every=m["temp_every"],
                                             slopes=head_slopes(m["heads"]), head_bias=True, output_gate=True)
                mix_names = {"qkv": (q + "q", q + "k", q + "v", q + "g"), "out": (q + "o",), "q_norm": (q + "q.norm",), "k_norm": (q + "k.norm",),
                             "head_bias": (q + "pb",)}
            else:
                mixer = LatentAttentionSpec(hidden=W, num_heads=m["heads"], nope_dim=m["dim"], rope_dim=0, v_dim=m["vdim"], kv_rank=m["kv_rank"],
                                            scale=m["scale"], latent_eps=self.eps, position=None, head_gate=True)
                mix_names = {"q": (q + "q",), "uk": (q + "uk",), "uv": (q + "uv",), "out": (q + "o",), "dkv": (q + "dkv",),
                             "latent_norm": (q + "dkv.norm",), "head_gate": (q + "g",)}
            names[f"blocks.{i}.input_norm"] = {"weight": (p + "norm1",)}
            names[f"blocks.{i}.mixer"] = mix_names
            names[f"blocks.{i}.mixer_connection"] = {"gate": (p + "rg1",), "gate_bias": (p + "rg1.b",)}
            f = layer.mlp
            ff = None
            if f is not None:
                ff = DenseMlpSpec(hidden=W, intermediate=f["ff"], activation="xielu")
                names[f"blocks.{i}.feed_forward"] = {"up": (p + "mlp.up",), "down": (p + "mlp.down",), "act": (p + "mlp.act",)}
                names[f"blocks.{i}.post_mixer_norm"] = {"weight": (p + "norm2",)}
                names[f"blocks.{i}.feed_forward_connection"] = {"gate": (p + "rg2",), "gate_bias": (p + "rg2.b",)}
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, input_norm=norm, post_mixer_norm=norm if ff is not None else None,
                                    kind="pre_norm_gated", connection=gate))
        schedule = tuple(RunEntry(block=i) for i in range(len(blocks)))
        return ModelSpec(architecture=ARCHITECTURE, hidden=W, vocab=self.vocab, blocks=tuple(blocks), schedule=schedule, final_norm=norm,
                         tie_embeddings=True, max_positions=0, stop_token_ids=(), stored_dtype="bfloat16",
                         embedding=ScaledEmbeddingSpec(vocab=self.vocab, hidden=W, scale=1.0),       # the token's own row as a 32-bit stream
                         head=ScaledHeadSpec(vocab=self.vocab, hidden=W, scale=self.logit_scale), weight_names=names)
