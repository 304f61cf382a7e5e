"""The Nilatar decoder: its config.json keys, its typed configuration and its ``ModelSpec``.

What the architecture is. ``x = embed[token] * embedding.scale``; a list of pre-norm layers, each
``x += ls1 * mixer(rms(x))`` and, where the layer has a feed-forward, ``x += ls2 * ff(rms(x))`` with learned
per-column scales ``ls1`` / ``ls2``; a final RMS norm and an untied head. ``layers[i].type`` names the layer's mixer:

* ``attention``: grouped-query attention without a position encoding, a sliding window (``mask.size``), a learned
  sink per head in the softmax denominator, an output gate ``sigmoid(W_g y)``; with ``kv_from: j`` the layer has no
  key and value projections and attends to layer j's cached keys and values with its own queries and window.
* ``latent_attention``: low-rank query and key/value latents with one rotated key part shared by the heads,
  interleaved-pair rotation with YaRN-scaled frequencies (``rot.scaling``), causal softmax, the same output gate.
* ``lightning``: linear attention with a decay per head (``decay``), a gated RMS norm over the heads.

The feed-forward (``mlp.kind`` = ``dense``) is ``W_down (gelu_tanh(W_gate y) * (W_up y))``.

config.json is nested: ``layers[i] = {"type", "mixer": {...}, "mlp": {"kind", "ff"} | null}``, ``embedding.scale``,
``norm.eps``, ``vocab``, ``width``. Tensors: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``,
``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``. Every size and constant comes from the
configuration; nothing here knows a particular model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ConfigReader
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class NilatarWindowed:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    kv_from: Optional[int]


@dataclass(frozen=True)
class NilatarRotation:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]]        # factor, original, fast, slow


@dataclass(frozen=True)
class NilatarLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: NilatarRotation


@dataclass(frozen=True)
class NilatarLightning:
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class NilatarLayer:
    kind: str                   # "attention" | "latent_attention" | "lightning"
    mixer: Any
    ff: Optional[int]           # the dense feed-forward's inner size, or None for a layer without one


@dataclass(frozen=True)
class NilatarConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: Tuple[NilatarLayer, ...]

    def to_dict(self) -> dict:
        """the config.json that reads back as this configuration"""
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.kind == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.window is not None:
                    mixer["mask"] = {"size": m.window}
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            elif l.kind == "latent_attention":
                rot = {"base": m.rot.base, "dims": m.rot.dims}
                if m.rot.scaling is not None:
                    rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), m.rot.scaling))
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank,
                         "kv_rank": m.kv_rank, "scale": m.scale, "rot": rot}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "decay": list(m.decay)}
            layers.append({"type": l.kind, "mixer": mixer,
                           "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers}


def _positive(what: str, v):
    if not (v > 0):
        raise ConfigError("config.json: %s must be positive, found %r" % (what, v))
    return v


def _read_windowed(raw: Mapping[str, Any], where: str, index: int) -> NilatarWindowed:
    r = ConfigReader(raw, where)
    heads = _positive(where + ".heads", r.integer("heads"))
    kv = _positive(where + ".kv_heads", r.integer("kv_heads", heads))
    if heads % kv:
        raise ConfigError("%s: heads %d is not a multiple of kv_heads %d" % (where, heads, kv))
    dim = _positive(where + ".dim", r.integer("dim"))
    vdim = _positive(where + ".vdim", r.integer("vdim", dim))
    scale = _positive(where + ".scale", r.number("scale", dim ** -0.5))
    window = None
    mraw = r.any("mask")
    if mraw is not None:
        mask = ConfigReader(mraw, where + ".mask")
        window = mask.integer("size", None)
        mask.finish(())
        if window is not None:
            _positive(where + ".mask.size", window)
    r.neutral("rot", (None,), "this mixer has no position encoding")
    kv_from = r.integer("kv_from", None)
    if kv_from is not None and not (0 <= kv_from < index):
        raise ConfigError("%s: kv_from must name an earlier layer, found %d" % (where, kv_from))
    r.finish(())
    return NilatarWindowed(heads, kv, dim, vdim, float(scale), window, kv_from)


def _read_rotation(raw: Mapping[str, Any], where: str, rot_dim: int) -> NilatarRotation:
    r = ConfigReader(raw, where)
    base = _positive(where + ".base", r.number("base", 10000.0))
    dims = r.integer("dims", rot_dim)
    if dims != rot_dim:
        raise ConfigError("%s: dims is %d, the mixer's rotated part has rot_dim = %d" % (where, dims, rot_dim))
    scaling = None
    sraw = r.any("scaling")
    if sraw is not None:
        s = ConfigReader(sraw, where + ".scaling")
        scaling = tuple(float(_positive("%s.scaling.%s" % (where, k), s.number(k)))
                        for k in ("factor", "original", "fast", "slow"))
        s.finish(())
    r.finish(())
    return NilatarRotation(float(base), dims, scaling)


def _read_latent(raw: Mapping[str, Any], where: str) -> NilatarLatent:
    r = ConfigReader(raw, where)
    heads = _positive(where + ".heads", r.integer("heads"))
    dim = _positive(where + ".dim", r.integer("dim"))
    rot_dim = r.integer("rot_dim")
    if rot_dim <= 0 or rot_dim % 2:
        raise ConfigError("%s: rot_dim must be even and positive, found %d" % (where, rot_dim))
    vdim = _positive(where + ".vdim", r.integer("vdim", dim))
    q_rank = _positive(where + ".q_rank", r.integer("q_rank"))
    kv_rank = _positive(where + ".kv_rank", r.integer("kv_rank"))
    scale = _positive(where + ".scale", r.number("scale", (dim + rot_dim) ** -0.5))
    rot = _read_rotation(r.any("rot") or {}, where + ".rot", rot_dim)
    r.neutral("mask", (None,), "latent attention sees every earlier position")
    r.finish(())
    return NilatarLatent(heads, dim, rot_dim, vdim, q_rank, kv_rank, float(scale), rot)


def _read_lightning(raw: Mapping[str, Any], where: str) -> NilatarLightning:
    r = ConfigReader(raw, where)
    heads = _positive(where + ".heads", r.integer("heads"))
    dim = _positive(where + ".dim", r.integer("dim"))
    vdim = _positive(where + ".vdim", r.integer("vdim", dim))
    draw = r.any("decay")
    if isinstance(draw, (int, float)) and not isinstance(draw, bool):
        draw = [draw] * heads
    if not isinstance(draw, (list, tuple)) or len(draw) != heads or \
            any(isinstance(x, bool) or not isinstance(x, (int, float)) for x in draw):
        raise ConfigError("%s: decay must be a list of %d numbers (one per head)" % (where, heads))
    r.neutral("mask", (None,), "linear attention has no window")
    r.neutral("rot", (None,), "linear attention has no position encoding")
    r.finish(())
    return NilatarLightning(heads, dim, vdim, tuple(float(x) for x in draw))


_MIXERS = ("attention", "latent_attention", "lightning")


def read_config(raw: Mapping[str, Any]) -> NilatarConfig:
    r = ConfigReader(raw)
    arch = r.string("architecture")
    vocab = _positive("vocab", r.integer("vocab"))
    width = _positive("width", r.integer("width"))
    norm = ConfigReader(r.any("norm") or {}, "config.json: norm")
    eps = _positive("norm.eps", norm.number("eps"))
    norm.finish(())
    emb = ConfigReader(r.any("embedding") or {}, "config.json: embedding")
    emb_scale = float(emb.number("scale", 1.0))
    emb.finish(())
    lraw = r.any("layers")
    if not isinstance(lraw, (list, tuple)) or not lraw:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers = []
    for i, l in enumerate(lraw):
        where = "config.json: layers[%d]" % i
        lr = ConfigReader(l, where)
        kind = lr.string("type")
        mraw = lr.any("mixer") or {}
        if kind == "attention":
            mixer = _read_windowed(mraw, where + ".mixer", i)
        elif kind == "latent_attention":
            mixer = _read_latent(mraw, where + ".mixer")
        elif kind == "lightning":
            mixer = _read_lightning(mraw, where + ".mixer")
        else:
            raise ConfigError("%s: type %r is not a mixer of this architecture (%s)" % (where, kind, ", ".join(_MIXERS)))
        ff = None
        fraw = lr.any("mlp")
        if fraw is not None:
            fr = ConfigReader(fraw, where + ".mlp")
            fkind = fr.string("kind", "dense")
            if fkind != "dense":
                raise ConfigError("%s.mlp: kind %r is not a feed-forward of this architecture (dense)" % (where, fkind))
            ff = _positive(where + ".mlp.ff", fr.integer("ff"))
            fr.finish(())
        lr.finish(())
        layers.append(NilatarLayer(kind, mixer, ff))
    for i, l in enumerate(layers):
        if l.kind == "attention" and l.mixer.kv_from is not None:
            src = layers[l.mixer.kv_from]
            m, s = l.mixer, src.mixer
            if src.kind != "attention" or s.kv_from is not None:
                raise ConfigError("config.json: layers[%d].mixer.kv_from names layer %d, which has no keys and values "
                                  "of its own" % (i, l.mixer.kv_from))
            if (m.kv_heads, m.dim, m.vdim) != (s.kv_heads, s.dim, s.vdim):
                raise ConfigError("config.json: layers[%d] reads the keys and values of layer %d, whose kv_heads, dim "
                                  "or vdim differ" % (i, l.mixer.kv_from))
    r.finish()
    return NilatarConfig(arch, vocab, width, float(eps), emb_scale, tuple(layers))


EMBEDDING, HEAD, FINAL_NORM = "embed", "head", "final.norm"


def build_spec(cfg: NilatarConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"eps": cfg.eps, "weight": ""})
    # what the cache of a layer keeps when later layers read its keys and values through windows of their own
    kept = {}
    for i, l in enumerate(cfg.layers):
        if l.kind == "attention":
            j = i if l.mixer.kv_from is None else l.mixer.kv_from
            w = l.mixer.window
            kept[j] = "all" if (w is None or kept.get(j) == "all") else max(w, kept.get(j, 0))
    layers, schedule = [], []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        reads = None
        if l.kind == "attention":
            reads = m.kv_from
            mixer = PartSpec("attention", {
                "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "scale": m.scale, "window": m.window, "cache_window": kept[i] if reads is None else None,
                "position": PartSpec("none", {}), "sink": "sink", "gate": "g", "shares_kv": reads is not None,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})
        elif l.kind == "latent_attention":
            scaling = None if m.rot.scaling is None else dict(zip(("factor", "original", "fast", "slow"),
                                                                  m.rot.scaling))
            position = PartSpec("rotary", {"base": m.rot.base, "rotary_dim": m.rot_dim, "pairing": "interleaved",
                                           "scaling": scaling})
            mixer = PartSpec("latent_attention", {
                "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.eps, "position": position,
                "names": {"gate": "g"}})
        else:
            mixer = PartSpec("decay_linear_attention", {
                "n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "decay": m.decay, "eps": cfg.eps})
        ff = None
        if l.ff is not None:
            ff = PartSpec("swiglu", {"intermediate": l.ff, "activation": "gelu_tanh",
                                     "names": {"gate": "gate", "up": "up", "down": "down"}})
        block = PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "feed_forward": ff,
                                     "layer_scale": {"mixer": "ls1", "feed_forward": "ls2"},
                                     "names": {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2",
                                               "feed_forward": "mlp."}})
        layers.append(LayerSpec(block, "l%d." % i))
        schedule.append(ScheduleEntry(layer=i, cache=i, reads_cache_of=reads))
    spec = ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, width=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule), final_norm=norm, final_norm_prefix=FINAL_NORM,
        embedding=PartSpec("table", {"name": EMBEDDING, "vocab": cfg.vocab, "scale": cfg.embedding_scale}),
        head=PartSpec("linear", {"name": HEAD, "vocab": cfg.vocab}),
        # a layer without a feed-forward has no use for a second norm or scale: a folder that stores them is accepted
        may_ignore=tuple(n for i, l in enumerate(cfg.layers) if l.ff is None
                         for n in ("l%d.norm2" % i, "l%d.ls2" % i)))
    spec.validate()
    return spec


register_architecture("Nilatar", build_spec, read_config)
