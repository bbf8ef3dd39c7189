"""Typed model configuration, read from the architecture's own ``config.json`` keys.

Upstream holds every model size as a compile-time constant
(base/src/config.h:41-68, with a note to read them from config.json one day);
here no size stands in code: each value below comes from the file, and the few
keys that may be absent have the defaults that the format itself defines.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping, Optional, Tuple


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value this engine cannot run."""


@dataclass(frozen=True)
class RopeScaling:
    """``rope_scaling`` of the llama3 kind (base/src/config.h:61-65)."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def to_dict(self) -> dict:
        return {
            "rope_type": self.rope_type, "factor": self.factor,
            "low_freq_factor": self.low_freq_factor, "high_freq_factor": self.high_freq_factor,
            "original_max_position_embeddings": self.original_max_position_embeddings,
        }


def _need(d: Mapping[str, Any], key: str, typ):
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    try:
        return typ(d[key])
    except (TypeError, ValueError) as e:
        raise ConfigError(f"config.json: key {key!r} has the value {d[key]!r}, wanted {typ.__name__}") from e


@dataclass(frozen=True)
class LlamaConfig:
    """The keys of a ``LlamaForCausalLM`` config.json that decide the computation."""
    architecture: str
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    attention_bias: bool = False
    mlp_bias: bool = False
    torch_dtype: str = "bfloat16"
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)
    bos_token_id: Optional[int] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LlamaConfig":
        archs = d.get("architectures") or []
        if not archs:
            raise ConfigError("config.json: 'architectures' is missing or empty")
        heads = _need(d, "num_attention_heads", int)
        hidden = _need(d, "hidden_size", int)
        kv_heads = int(d["num_key_value_heads"]) if d.get("num_key_value_heads") is not None else heads
        if d.get("head_dim") is not None:
            head_dim = int(d["head_dim"])
        else:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size {hidden} is no multiple of "
                                  f"num_attention_heads {heads} and no head_dim is given")
            head_dim = hidden // heads
        rs = d.get("rope_scaling")
        scaling = None
        if rs:
            kind = rs.get("rope_type", rs.get("type"))
            if kind == "default":
                scaling = None
            elif kind == "llama3":
                scaling = RopeScaling(
                    rope_type="llama3",
                    factor=_need(rs, "factor", float),
                    low_freq_factor=_need(rs, "low_freq_factor", float),
                    high_freq_factor=_need(rs, "high_freq_factor", float),
                    original_max_position_embeddings=_need(rs, "original_max_position_embeddings", int),
                )
            else:
                raise ConfigError(f"config.json: rope_scaling of type {kind!r} is not supported "
                                  "(supported: 'llama3', 'default' or none)")
        eos = d.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(e) for e in eos)
        else:
            eos_ids = (int(eos),)
        cfg = cls(
            architecture=str(archs[0]),
            vocab_size=_need(d, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_need(d, "intermediate_size", int),
            num_hidden_layers=_need(d, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=_need(d, "rms_norm_eps", float),
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rope_scaling=scaling,
            max_position_embeddings=_need(d, "max_position_embeddings", int),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            hidden_act=str(d.get("hidden_act", "silu")),
            attention_bias=bool(d.get("attention_bias", False)),
            mlp_bias=bool(d.get("mlp_bias", False)),
            torch_dtype=str(d.get("torch_dtype", d.get("dtype", "bfloat16"))),
            eos_token_ids=eos_ids,
            bos_token_id=(int(d["bos_token_id"]) if d.get("bos_token_id") is not None else None),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for key in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                    "num_attention_heads", "num_key_value_heads", "head_dim",
                    "max_position_embeddings"):
            if getattr(self, key) < 1:
                raise ConfigError(f"config.json: {key} must be positive, got {getattr(self, key)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is no "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        if not (self.rms_norm_eps > 0):
            raise ConfigError("config.json: rms_norm_eps must be positive")
        if self.hidden_act != "silu":
            raise ConfigError(f"config.json: hidden_act {self.hidden_act!r} is not supported (only 'silu')")
        if self.attention_bias or self.mlp_bias:
            raise ConfigError("config.json: attention_bias / mlp_bias are not supported (the model has no bias)")
        if self.rope_scaling is not None:
            s = self.rope_scaling
            if s.high_freq_factor == s.low_freq_factor or s.factor <= 0:
                raise ConfigError("config.json: rope_scaling needs factor > 0 and "
                                  "high_freq_factor != low_freq_factor")

    def to_dict(self) -> dict:
        """A config.json that reads back to this configuration."""
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": self.hidden_act,
            "attention_bias": self.attention_bias,
            "mlp_bias": self.mlp_bias,
            "torch_dtype": self.torch_dtype,
        }
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d


@dataclass(frozen=True)
class RezusunLayerConfig:
    """One entry of ``layers``: the mixer's kind and sizes, and the feed-forward (None: the
    layer has only its mixer)."""
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


_REZUSUN_MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "rot"),   # "scale" may be left out
    "general_delta": ("heads", "dim"),
    "channel_delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}


@dataclass(frozen=True)
class RezusunConfig:
    """The keys of a Rezusun config.json: ``vocab``, ``width``, ``norm.eps``, ``layers`` (each with
    ``type``, ``mixer`` and ``mlp``) and ``loop`` (layers start .. stop - 1 run ``times`` times in a
    row).  Sizes that the file leaves to the tensors' shapes (ranks of the low-rank branches)
    are read from the checkpoint when the model is described."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[RezusunLayerConfig, ...]
    loop: Optional[Tuple[int, int, int]]
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "RezusunConfig":
        norm = d.get("norm") or {}
        layers = []
        for i, entry in enumerate(d.get("layers") or []):
            kind = entry.get("type")
            if kind not in _REZUSUN_MIXER_KEYS:
                raise ConfigError(f"config.json: layer {i} has a mixer of type {kind!r}; known: "
                                  + ", ".join(sorted(_REZUSUN_MIXER_KEYS)))
            mixer = entry.get("mixer") or {}
            for key in _REZUSUN_MIXER_KEYS[kind]:
                if mixer.get(key) is None:
                    raise ConfigError(f"config.json: layer {i} ({kind}): mixer key {key!r} is missing")
            if kind == "latent_attention":
                for key in ("base", "dims"):
                    if mixer["rot"].get(key) is None:
                        raise ConfigError(f"config.json: layer {i}: rot.{key} is missing")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: layer {i}: a feed-forward of kind {mlp.get('kind')!r} is not known "
                                      "(known: 'dense')")
                _need(mlp, "ff", int)
            layers.append(RezusunLayerConfig(str(kind), dict(mixer), dict(mlp) if mlp is not None else None))
        if not layers:
            raise ConfigError("config.json: 'layers' is missing or empty")
        loop = d.get("loop")
        loop_t = None
        if loop:
            loop_t = (_need(loop, "start", int), _need(loop, "stop", int), _need(loop, "times", int))
            a, b, n = loop_t
            if not (0 <= a <= b <= len(layers)) or n < 1:
                raise ConfigError(f"config.json: loop {dict(loop)} does not fit {len(layers)} layers")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Rezusun"])[0]),
                  vocab=_need(d, "vocab", int), width=_need(d, "width", int), norm_eps=_need(norm, "eps", float),
                  layers=tuple(layers), loop=loop_t,
                  max_position_embeddings=int(d.get("max_position_embeddings") or 131072), eos_token_ids=eos_ids)
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: vocab and width must be positive and norm.eps above zero")
        return cfg

    def layer_order(self):
        """Indices of the layers in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b, times = self.loop
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


@dataclass(frozen=True)
class SolulixLayerConfig:
    """One entry of ``layers``: the mixer's kind (``attention`` or ``delta``) and sizes, and the
    feed-forward (None: the layer has only its mixer)."""
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


_SOLULIX_MIXER_KEYS = {
    "attention": ("heads", "kv_heads", "dim", "vdim", "conv", "scale", "mask"),
    "delta": ("heads", "kv_heads", "dim", "vdim", "conv"),
}


@dataclass(frozen=True)
class SolulixConfig:
    """The keys of a Solulix config.json: ``vocab``, ``width``, ``norm.eps``, ``layers`` (each with
    ``type``, ``mixer`` and ``mlp``, the latter of ``kind`` ``dense`` or ``moe``) and ``loop``
    (layers start .. stop - 1 run ``times`` times in a row)."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[SolulixLayerConfig, ...]
    loop: Optional[Tuple[int, int, int]]
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "SolulixConfig":
        norm = d.get("norm") or {}
        layers = []
        for i, entry in enumerate(d.get("layers") or []):
            kind = entry.get("type")
            if kind not in _SOLULIX_MIXER_KEYS:
                raise ConfigError(f"config.json: layer {i} has a mixer of type {kind!r}; known: "
                                  + ", ".join(sorted(_SOLULIX_MIXER_KEYS)))
            mixer = entry.get("mixer") or {}
            for key in _SOLULIX_MIXER_KEYS[kind]:
                if mixer.get(key) is None:
                    raise ConfigError(f"config.json: layer {i} ({kind}): mixer key {key!r} is missing")
            if kind == "attention":
                for key in ("size", "keep_first"):
                    if mixer["mask"].get(key) is None:
                        raise ConfigError(f"config.json: layer {i}: mask.{key} is missing")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind") == "dense":
                    _need(mlp, "ff", int)
                elif mlp.get("kind") == "moe":
                    router = mlp.get("router") or {}
                    for key in ("experts", "top", "identity", "scale"):
                        if router.get(key) is None:
                            raise ConfigError(f"config.json: layer {i}: mlp.router.{key} is missing")
                    if (mlp.get("expert") or {}).get("ff") is None:
                        raise ConfigError(f"config.json: layer {i}: mlp.expert.ff is missing")
                    if mlp.get("shared") is not None and mlp["shared"].get("ff") is None:
                        raise ConfigError(f"config.json: layer {i}: mlp.shared.ff is missing")
                    n_all = int(router["experts"]) + int(router["identity"])
                    if not 1 <= int(router["top"]) <= n_all:
                        raise ConfigError(f"config.json: layer {i}: the router chooses {router['top']} of {n_all} experts")
                else:
                    raise ConfigError(f"config.json: layer {i}: a feed-forward of kind {mlp.get('kind')!r} is not known "
                                      "(known: 'dense', 'moe')")
            layers.append(SolulixLayerConfig(str(kind), dict(mixer), dict(mlp) if mlp is not None else None))
        if not layers:
            raise ConfigError("config.json: 'layers' is missing or empty")
        loop = d.get("loop")
        loop_t = None
        if loop:
            loop_t = (_need(loop, "start", int), _need(loop, "stop", int), _need(loop, "times", int))
            a, b, n = loop_t
            if not (0 <= a <= b <= len(layers)) or n < 1:
                raise ConfigError(f"config.json: loop {dict(loop)} does not fit {len(layers)} layers")
            if a == b:
                loop_t = None       # an empty run of layers: nothing repeats
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Solulix"])[0]),
                  vocab=_need(d, "vocab", int), width=_need(d, "width", int), norm_eps=_need(norm, "eps", float),
                  layers=tuple(layers), loop=loop_t,
                  max_position_embeddings=int(d.get("max_position_embeddings") or 131072), eos_token_ids=eos_ids)
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: vocab and width must be positive and norm.eps above zero")
        return cfg

    def passes(self):
        """(layer index, number of the pass that this run of the layer opens or None) in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop
        order = [(i, None) for i in range(a)]
        for t in range(times):
            order += [(i, t if i == a else None) for i in range(a, b)]
        return order + [(i, None) for i in range(b, n)]


def read_config_json(model_dir) -> dict:
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise ConfigError(f"{path} does not exist")
    try:
        return json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e


@dataclass(frozen=True)
class NonetarLayerConfig:
    """One entry of ``layers``: the mixer's kind (``parallel`` or ``mamba2``) and sizes, and the
    feed-forward (None: the layer has only its mixer)."""
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]


_NONETAR_MIXER_KEYS = {
    "parallel": ("left", "right", "left_scale", "right_scale"),
    "mamba2": ("heads", "vdim", "state", "groups", "norm_groups", "conv"),
}
_NONETAR_LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
_NONETAR_RIGHT_KEYS = ("width", "blocks", "conv")


@dataclass(frozen=True)
class NonetarConfig:
    """The keys of a Nonetar config.json: ``vocab``, ``width``, ``norm.eps``, ``streams`` (copies of the
    residual stream), ``logit_scale`` and ``layers`` (each with ``type``, ``mixer`` and ``mlp``, the
    latter of ``kind`` ``dense`` or null).  A ``parallel`` mixer names a ``left`` side (attention:
    ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, and optionally ``softcap`` and ``mask.size``), a
    ``right`` side (gated linear recurrence: ``width``, ``blocks``, ``conv``) and their weights in the sum;
    a ``mamba2`` mixer names ``heads``, ``vdim``, ``state``, ``groups``, ``norm_groups`` and ``conv``."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    streams: int
    logit_scale: float
    layers: Tuple[NonetarLayerConfig, ...]
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "NonetarConfig":
        norm = d.get("norm") or {}
        layers = []
        for i, entry in enumerate(d.get("layers") or []):
            kind = entry.get("type")
            if kind not in _NONETAR_MIXER_KEYS:
                raise ConfigError(f"config.json: layer {i} has a mixer of type {kind!r}; known: "
                                  + ", ".join(sorted(_NONETAR_MIXER_KEYS)))
            mixer = entry.get("mixer") or {}
            for key in _NONETAR_MIXER_KEYS[kind]:
                if mixer.get(key) is None:
                    raise ConfigError(f"config.json: layer {i} ({kind}): mixer key {key!r} is missing")
            if kind == "parallel":
                for side, keys in (("left", _NONETAR_LEFT_KEYS), ("right", _NONETAR_RIGHT_KEYS)):
                    for key in keys:
                        if mixer[side].get(key) is None:
                            raise ConfigError(f"config.json: layer {i}: mixer.{side}.{key} is missing")
                left, right = mixer["left"], mixer["right"]
                if int(left["heads"]) % int(left["kv_heads"]):
                    raise ConfigError(f"config.json: layer {i}: {left['heads']} query heads cannot be grouped over "
                                      f"{left['kv_heads']} key/value heads")
                if int(right["width"]) % int(right["blocks"]):
                    raise ConfigError(f"config.json: layer {i}: {right['width']} channels do not split into "
                                      f"{right['blocks']} equal blocks")
            else:
                if int(mixer["heads"]) % int(mixer["groups"]):
                    raise ConfigError(f"config.json: layer {i}: {mixer['heads']} heads cannot share "
                                      f"{mixer['groups']} groups evenly")
                if (int(mixer["heads"]) * int(mixer["vdim"])) % int(mixer["norm_groups"]):
                    raise ConfigError(f"config.json: layer {i}: the inner width does not split into "
                                      f"{mixer['norm_groups']} equal parts")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: layer {i}: a feed-forward of kind {mlp.get('kind')!r} is not known "
                                      "(known: 'dense')")
                _need(mlp, "ff", int)
            layers.append(NonetarLayerConfig(str(kind), dict(mixer), dict(mlp) if mlp is not None else None))
        if not layers:
            raise ConfigError("config.json: 'layers' is missing or empty")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Nonetar"])[0]),
                  vocab=_need(d, "vocab", int), width=_need(d, "width", int), norm_eps=_need(norm, "eps", float),
                  streams=int(d["streams"]) if d.get("streams") is not None else 1,
                  logit_scale=float(d["logit_scale"]) if d.get("logit_scale") is not None else 1.0,
                  layers=tuple(layers), max_position_embeddings=int(d.get("max_position_embeddings") or 131072),
                  eos_token_ids=eos_ids)
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.norm_eps > 0 or cfg.streams < 1:
            raise ConfigError("config.json: vocab, width and streams must be positive and norm.eps above zero")
        return cfg


@dataclass(frozen=True)
class TevanexLayerConfig:
    """One entry of ``layers``: the mixer's kind (``mlstm``, ``attention`` or ``attention_2``) and sizes, the
    feed-forward (None: the layer has only its mixer), and ``weights_of``: the layer whose tensors this one uses
    (None: its own)."""
    type: str
    mixer: Mapping[str, Any]
    mlp: Optional[Mapping[str, Any]]
    weights_of: Optional[int] = None


_TEVANEX_MIXER_KEYS = {
    "mlstm": ("heads", "dim", "vdim", "gate_cap"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
    "attention_2": ("heads", "kv_heads", "dim", "vdim", "scale"),
}


@dataclass(frozen=True)
class TevanexConfig:
    """The keys of a Tevanex config.json: ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``residual_mult``,
    ``logit_scale``, ``logit_softcap`` and ``layers`` (each with ``type``, ``mixer``, ``mlp`` and optionally
    ``weights_of``).  An ``mlstm`` mixer names ``heads``, ``dim``, ``vdim``, ``gate_cap``; the two attentions ``heads``,
    ``kv_heads``, ``dim``, ``vdim``, ``scale`` and optionally ``mask.size``, ``rot`` (``base``, ``dims``, and for the
    second kind ``scaling`` with ``factor``, ``original``, ``fast``, ``slow``) and ``softcap``.  A feed-forward is of
    ``kind`` ``moe``: ``expert`` (``ff``, ``limit``), ``router`` (``experts``, ``top``) and optionally ``shared``
    (``ff``, ``limit``)."""
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    logit_scale: float
    logit_softcap: float
    layers: Tuple[TevanexLayerConfig, ...]
    max_position_embeddings: int
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "TevanexConfig":
        norm = d.get("norm") or {}
        entries = list(d.get("layers") or [])
        layers = []
        for i, entry in enumerate(entries):
            kind = entry.get("type")
            if kind not in _TEVANEX_MIXER_KEYS:
                raise ConfigError(f"config.json: layer {i} has a mixer of type {kind!r}; known: "
                                  + ", ".join(sorted(_TEVANEX_MIXER_KEYS)))
            mixer = entry.get("mixer") or {}
            for key in _TEVANEX_MIXER_KEYS[kind]:
                if mixer.get(key) is None:
                    raise ConfigError(f"config.json: layer {i} ({kind}): mixer key {key!r} is missing")
            if kind != "mlstm":
                if int(mixer["kv_heads"]) < 1 or int(mixer["heads"]) % int(mixer["kv_heads"]):
                    raise ConfigError(f"config.json: layer {i}: {mixer['heads']} query heads cannot be grouped over "
                                      f"{mixer['kv_heads']} key/value heads")
                rot = mixer.get("rot")
                if rot:
                    for key in ("base", "dims"):
                        if rot.get(key) is None:
                            raise ConfigError(f"config.json: layer {i}: mixer.rot.{key} is missing")
                    if int(rot["dims"]) % 2 or int(rot["dims"]) > int(mixer["dim"]):
                        raise ConfigError(f"config.json: layer {i}: mixer.rot.dims must be even and at most mixer.dim")
                    for key in ("factor", "original", "fast", "slow") if rot.get("scaling") else ():
                        if rot["scaling"].get(key) is None:
                            raise ConfigError(f"config.json: layer {i}: mixer.rot.scaling.{key} is missing")
                if mixer.get("mask") and int(mixer["mask"].get("size") or 0) < 1:
                    raise ConfigError(f"config.json: layer {i}: mixer.mask.size must be a positive number of positions")
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp.get("kind") != "moe":
                    raise ConfigError(f"config.json: layer {i}: a feed-forward of kind {mlp.get('kind')!r} is not known "
                                      "(known: 'moe')")
                for group, keys in (("expert", ("ff", "limit")), ("router", ("experts", "top"))):
                    for key in keys:
                        if (mlp.get(group) or {}).get(key) is None:
                            raise ConfigError(f"config.json: layer {i}: mlp.{group}.{key} is missing")
                if mlp.get("shared"):
                    for key in ("ff", "limit"):
                        if mlp["shared"].get(key) is None:
                            raise ConfigError(f"config.json: layer {i}: mlp.shared.{key} is missing")
                if not 1 <= int(mlp["router"]["top"]) <= int(mlp["router"]["experts"]):
                    raise ConfigError(f"config.json: layer {i}: mlp.router.top must lie between 1 and mlp.router.experts")
            src = entry.get("weights_of")
            if src is not None:
                src = int(src)
                if not 0 <= src < len(entries) or src == i or entries[src].get("weights_of") is not None:
                    raise ConfigError(f"config.json: layer {i}: weights_of {src} must name another layer that has "
                                      "tensors of its own")
                if entries[src].get("type") != kind:
                    raise ConfigError(f"config.json: layer {i} is of type {kind!r} but uses the tensors of layer {src}, "
                                      f"which is of type {entries[src].get('type')!r}")
            layers.append(TevanexLayerConfig(str(kind), dict(mixer), dict(mlp) if mlp is not None else None, src))
        if not layers:
            raise ConfigError("config.json: 'layers' is missing or empty")
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(e) for e in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        emb = d.get("embedding") or {}
        cfg = cls(architecture=str(d.get("architecture") or (d.get("architectures") or ["Tevanex"])[0]),
                  vocab=_need(d, "vocab", int), width=_need(d, "width", int), norm_eps=_need(norm, "eps", float),
                  embedding_scale=float(emb["scale"]) if emb.get("scale") is not None else 1.0,
                  residual_mult=float(d["residual_mult"]) if d.get("residual_mult") is not None else 1.0,
                  logit_scale=float(d["logit_scale"]) if d.get("logit_scale") is not None else 1.0,
                  logit_softcap=float(d["logit_softcap"]) if d.get("logit_softcap") else 0.0,
                  layers=tuple(layers), max_position_embeddings=int(d.get("max_position_embeddings") or 131072),
                  eos_token_ids=eos_ids)
        if cfg.vocab < 1 or cfg.width < 1 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: vocab and width must be positive and norm.eps above zero")
        return cfg
