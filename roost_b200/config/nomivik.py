"""The Nomivik decoder's configuration, read from its own config.json keys.

Nomivik is a pre-norm decoder over a 32-bit residual stream with root-mean-square norms and logits against the embedding table.
Its embedding adds a hashed table of token pairs (``embedding.bigram``: ``buckets``, ``mul_prev``, ``mul_cur``) to the token's
own row. ``layers`` lists its layers: each names its mixer by ``type`` (``rglru``: a gated linear recurrence a channel behind a
short convolution; ``parallel``: a windowed grouped-query attention with biases, a rotation of split halves, unit-norm queries
and keys, capped scores and a sink, ``left``, beside a matrix memory with exponential gates, ``right``, their normed outputs
averaged) with the mixer's sizes under ``mixer``, and its feed-forward under ``mlp`` (``dense``: a gated one with SiLU; null:
none). With ``token_side`` every layer ends by adding what a gated slice of a second token embedding gives. ``loop`` names a
range of layers that runs several times in a row with the same weights; every pass keeps a cache or state of its own, and the
embedding's output is added to the stream again before every pass but the first. Tensor names: ``embed``, ``bigram``,
``side.embed``, ``l<i>.norm1`` / ``.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``. No size and no
constant that config.json gives stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .reader import ConfigError, ConfigReader
from .spec import (BlockSpec, GatedMlpSpec, GatedRecurrenceSpec, MatrixMemorySpec, ModelSpec, NormSpec, PairHashedEmbeddingSpec,
                   ParallelMixerSpec, PositionSpec, RunEntry, ScaledEmbeddingSpec, SinkAttentionSpec, TokenInputSpec)

ARCHITECTURE = "Nomivik"
RECURRENCE_RATE = 8.0          # the design's constant in the recurrence's decay: log a = -8 r softplus(lam)
MEMORY_FLOOR = 1e-6            # the design's constant added to the matrix memory's denominator


@dataclass(frozen=True)
class NomivikLayer:
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


@dataclass
class NomivikConfig:
    vocab: int
    width: int
    eps: float
    pairs: tuple | None            # (buckets, mul_prev, mul_cur); None: the token's own row only
    side_dim: int | None           # None: no token input at the layers' ends
    layers: tuple
    loop: tuple | None             # (start, stop, times)
    tie_word_embeddings: bool = True
    warnings: list = field(default_factory=list)

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_reader(cls, c: ConfigReader) -> "NomivikConfig":
        vocab, width = c.positive_int("vocab"), c.positive_int("width")
        eps = _positive_float(_object(c, "norm"), "eps")
        pairs = None
        emb = c.opt_object("embedding")
        big = emb.opt_object("bigram") if emb is not None else None
        if big is not None:
            pairs = (big.positive_int("buckets"), big.opt_int("mul_prev"), big.opt_int("mul_cur"))
            if pairs[1] is None or pairs[2] is None or pairs[1] < 0 or pairs[2] < 0:
                raise ConfigError(f"{big.source}: 'mul_prev' and 'mul_cur' must be integers that are not negative")
        side = c.opt_object("token_side")
        side_dim = side.positive_int("dim") if side is not None else None
        raw = c.raw("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError(f"{c.source}: key 'layers' must be a non-empty list")
        layers = []
        for i, item in enumerate(raw):
            lr = ConfigReader(item, f"{c.source}: layers[{i}]")
            kind = lr.opt_str("type")
            m = _object(lr, "mixer")
            if kind == "rglru":
                mixer = cls._read_recurrence(m)
            elif kind == "parallel":
                mixer = {"left": cls._read_attention(_object(m, "left")), "right": cls._read_memory(_object(m, "right"))}
            else:
                raise ConfigError(f"{lr.source}: key 'type' is {kind!r}; the design has rglru and parallel mixers")
            layers.append(NomivikLayer(kind, mixer, cls._read_mlp(lr.opt_object("mlp"))))
        loop = None
        lp = c.opt_object("loop")
        if lp is not None:
            start, stop, times = lp.opt_int("start"), lp.opt_int("stop"), lp.positive_int("times")
            if start is None or stop is None or not 0 <= start <= stop <= len(layers):
                raise ConfigError(f"{lp.source}: 'start' and 'stop' must bound a range of the {len(layers)} layers")
            loop = (start, stop, times)
        return cls(vocab=vocab, width=width, eps=eps, pairs=pairs, side_dim=side_dim, layers=tuple(layers), loop=loop)

    @staticmethod
    def _read_recurrence(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("width", "blocks", "conv")}
        if out["width"] % out["blocks"]:
            raise ConfigError(f"{m.source}: a width of {out['width']} does not divide into {out['blocks']} blocks")
        return out

    @staticmethod
    def _read_attention(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "kv_heads", "dim", "vdim")}
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"{m.source}: {out['heads']} heads are not a multiple of {out['kv_heads']} kv_heads")
        out["scale"], out["softcap"] = _positive_float(m, "scale"), _positive_float(m, "softcap")
        out["window"] = _object(m, "mask").positive_int("size")
        rot = _object(m, "rot")
        out["rot_dims"], out["rot_base"] = rot.positive_int("dims"), _positive_float(rot, "base")
        if out["rot_dims"] % 2 or out["rot_dims"] > out["dim"]:
            raise ConfigError(f"{rot.source}: key 'dims' is {out['rot_dims']}; it must be even and at most dim {out['dim']}")
        return out

    @staticmethod
    def _read_memory(m: ConfigReader) -> dict:
        out = {k: m.positive_int(k) for k in ("heads", "dim", "vdim")}
        out["gate_cap"] = _positive_float(m, "gate_cap")
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
    def from_dict(cls, values: dict, source: str = "config") -> "NomivikConfig":
        return cls.from_reader(ConfigReader(values, source))

    # ------------------------------------------------------------------ the model as parts
    def run_order(self) -> list:
        """[(layer, whether the embedding's output is added to the stream before it)] in the order of running."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, False) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, False) for i in range(start)]
        for turn in range(times):
            order += [(i, turn > 0 and i == start) for i in range(start, stop)]
        return order + [(i, False) for i in range(stop, n)]

    def to_spec(self, tied: bool | None = None) -> ModelSpec:
        W = self.width
        norm = NormSpec(size=W, eps=self.eps, kind="rms_norm_wide")
        names: dict = {"embed": {"table": ("embed",)}, "final_norm": {"weight": ("final.norm",)}}
        if self.pairs is not None:
            names["embed"]["pairs"] = ("bigram",)
            embedding = PairHashedEmbeddingSpec(vocab=self.vocab, hidden=W, buckets=self.pairs[0], mul_prev=self.pairs[1], mul_cur=self.pairs[2])
        else:
            embedding = ScaledEmbeddingSpec(vocab=self.vocab, hidden=W, scale=1.0)     # the token's own row as a 32-bit stream
        blocks = []
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer.mixer
            if layer.type == "rglru":
                mixer = GatedRecurrenceSpec(hidden=W, width=m["width"], blocks=m["blocks"], conv_taps=m["conv"], rate=RECURRENCE_RATE)
                mix_names = {"in": (p + "mix.y", p + "mix.x"), "in_bias": (p + "mix.y.b", p + "mix.x.b"), "conv": (p + "mix.conv",),
                             "conv_bias": (p + "mix.conv.b",), "recur_gate": (p + "mix.ra",), "recur_gate_bias": (p + "mix.ra.b",),
                             "input_gate": (p + "mix.ri",), "input_gate_bias": (p + "mix.ri.b",), "lam": (p + "mix.lam",), "out": (p + "mix.o",)}
            else:
                a, r = m["left"], m["right"]
                left = SinkAttentionSpec(hidden=W, num_heads=a["heads"], num_kv_heads=a["kv_heads"], head_dim=a["dim"], v_dim=a["vdim"],
                                         scale=a["scale"], sink=True, unit_norm_eps=self.eps, window=a["window"], softcap=a["softcap"], bias=True,
                                         position=PositionSpec(kind="rope_neox", rotary_dim=a["rot_dims"], theta=a["rot_base"]))
                right = MatrixMemorySpec(hidden=W, num_heads=r["heads"], head_dim=r["dim"], v_dim=r["vdim"], gate_cap=r["gate_cap"], eps=self.eps,
                                         floor=MEMORY_FLOOR)
                mixer = ParallelMixerSpec(hidden=W, branches=(left, right), eps=self.eps)
                L, R = p + "mix.left.", p + "mix.right."
                mix_names = {"0.qkv": (L + "q", L + "k", L + "v"), "0.qkv_bias": (L + "q.b", L + "k.b", L + "v.b"), "0.out": (L + "o",),
                             "weight.0": (L + "out",),
                             "1.in": (R + "q", R + "k", R + "v", R + "g"), "1.gates": (R + "i", R + "f"), "1.gates_bias": (R + "i.b", R + "f.b"),
                             "1.norm": (R + "norm",), "1.out": (R + "o",), "weight.1": (R + "out",)}
            f = layer.mlp
            ff = None
            if f is not None:
                ff = GatedMlpSpec(hidden=W, intermediate=f["ff"], activation="silu")
                names[f"blocks.{i}.feed_forward"] = {"gate_up": (p + "mlp.gate", p + "mlp.up"), "down": (p + "mlp.down",)}
                names[f"blocks.{i}.post_mixer_norm"] = {"weight": (p + "norm2",)}
            side = None
            if self.side_dim is not None:
                d = self.side_dim
                side = TokenInputSpec(hidden=W, vocab=self.vocab, dim=d, column=i * d, columns=len(self.layers) * d, eps=self.eps)
                names[f"blocks.{i}.token_input"] = {"table": ("side.embed",), "gate": (p + "side.gate",), "proj": (p + "side.proj",),
                                                    "norm": (p + "side.norm",)}
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, input_norm=norm, post_mixer_norm=norm if ff is not None else None,
                                    kind="pre_norm_wide", token_input=side))
            names[f"blocks.{i}.input_norm"] = {"weight": (p + "norm1",)}
            names[f"blocks.{i}.mixer"] = mix_names
        # every pass of the looped range is a run of its own: the same weights, a cache or state of its own
        schedule = tuple(RunEntry(block=i, adds_embedding=again) for i, again in self.run_order())
        return ModelSpec(architecture=ARCHITECTURE, hidden=W, vocab=self.vocab, blocks=tuple(blocks), schedule=schedule, final_norm=norm,
                         tie_embeddings=True, max_positions=0, stop_token_ids=(), stored_dtype="bfloat16", embedding=embedding,
                         weight_names=names)
