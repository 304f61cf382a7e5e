"""The Vozinex decoder: its config.json keys, its typed configuration and its ``ModelSpec``.

What the architecture is. Token embedding; a list of pre-norm layers, each ``x += mixer(norm1(x))`` and, where the
layer has a feed-forward, ``x += ff(norm2(x))``, the norms being layer norms with weight and bias; a final layer norm
and an untied head. The mixer is grouped-query attention whose query and key projections are each RMS-normalised over
the whole projection (all heads at once, with a gain per element) before a rotary encoding of the first ``rot.dims``
dimensions of every head (rotate-half pairing); scores are scaled by the configuration's ``scale``; a row sees the
last ``mask.size`` positions and the sequence's first ``mask.keep_first`` positions; values may have another size
than keys. The feed-forward is a mixture of experts: a 32-bit router with bias picks ``top`` experts, weighted by the
softmax over the picked logits; an expert is ``W_down relu(W_up y)^2``. A stretch of layers (``loop.start`` to
``loop.stop - 1``) runs ``loop.times`` times in a row with the same weights and a cache of its own for every pass,
and before every pass but the first the embedding output is added to the residual stream.

config.json is nested: ``layers[i] = {"type", "mixer": {...}, "mlp": {...} | null}``, ``loop``, ``norm.eps``,
``vocab``, ``width``. Tensors: ``embed``, ``l<i>.norm1`` / ``.b``, ``l<i>.mix.{q,k,v,o,q.norm,k.norm}``,
``l<i>.norm2`` / ``.b``, ``l<i>.mlp.{router,router.b,e<j>.up,e<j>.down}``, ``final.norm`` / ``.b``, ``head``.
Every size and constant comes from the configuration; nothing here knows a particular model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..config.model_config import ConfigError, ConfigReader
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


@dataclass(frozen=True)
class VozinexAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: float
    rot_dims: int
    window: Optional[int]
    keep_first: int


@dataclass(frozen=True)
class VozinexMoE:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class VozinexLayer:
    mixer: VozinexAttention
    mlp: Optional[VozinexMoE]


@dataclass(frozen=True)
class VozinexConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: Tuple[VozinexLayer, ...]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1

    def run_order(self):
        """(layer, pass) in the order the layers run; ``pass`` > 0 marks the runs of a repeated stretch"""
        order = [(i, 0) for i in range(self.loop_start)]
        for p in range(self.loop_times):
            order += [(i, p) for i in range(self.loop_start, self.loop_stop)]
        order += [(i, 0) for i in range(self.loop_stop, len(self.layers))]
        return order

    def to_dict(self) -> dict:
        """the config.json that reads back as this configuration"""
        layers = []
        for l in self.layers:
            m = l.mixer
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                     "rot": {"base": m.rot_base, "dims": m.rot_dims},
                     "mask": None if m.window is None else {"size": m.window, "keep_first": m.keep_first}}
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                       "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            layers.append({"type": "attention", "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "layers": layers,
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}


def _positive(what: str, v: int) -> int:
    if v <= 0:
        raise ConfigError("config.json: %s must be positive, found %d" % (what, v))
    return v


def _read_attention(raw: Mapping[str, Any], where: str) -> VozinexAttention:
    r = ConfigReader(raw, where)
    heads = _positive(where + ".heads", r.integer("heads"))
    kv = _positive(where + ".kv_heads", r.integer("kv_heads", heads))
    if heads % kv:
        raise ConfigError("%s: heads %d is not a multiple of kv_heads %d" % (where, heads, kv))
    dim = _positive(where + ".dim", r.integer("dim"))
    vdim = _positive(where + ".vdim", r.integer("vdim", dim))
    scale = r.number("scale", dim ** -0.5)
    if not (scale > 0.0):
        raise ConfigError("%s: scale must be positive, found %r" % (where, scale))
    rot = ConfigReader(r.any("rot") or {}, where + ".rot")
    dims = rot.integer("dims", 0)
    base = rot.number("base", 10000.0)
    rot.finish(())
    if dims < 0 or dims % 2 or dims > dim:
        raise ConfigError("%s.rot: dims must be even and lie between 0 and dim = %d, found %d" % (where, dim, dims))
    if not (base > 0.0):
        raise ConfigError("%s.rot: base must be positive, found %r" % (where, base))
    window, keep = None, 0
    mraw = r.any("mask")
    if mraw is not None:
        mask = ConfigReader(mraw, where + ".mask")
        window = mask.integer("size", None)
        keep = mask.integer("keep_first", 0)
        mask.finish(())
        if window is not None and window <= 0:
            raise ConfigError("%s.mask: size must be positive, found %d" % (where, window))
        if keep < 0:
            raise ConfigError("%s.mask: keep_first must not be negative, found %d" % (where, keep))
    r.finish(())
    return VozinexAttention(heads, kv, dim, vdim, scale, base, dims, window, keep if window is not None else 0)


def _read_moe(raw: Mapping[str, Any], where: str) -> VozinexMoE:
    r = ConfigReader(raw, where)
    kind = r.string("kind", "moe")
    if kind != "moe":
        raise ConfigError("%s: kind %r is not a feed-forward of this architecture (moe)" % (where, kind))
    ex = ConfigReader(r.any("expert") or {}, where + ".expert")
    ff = _positive(where + ".expert.ff", ex.integer("ff"))
    ex.finish(())
    ro = ConfigReader(r.any("router") or {}, where + ".router")
    experts = _positive(where + ".router.experts", ro.integer("experts"))
    top = _positive(where + ".router.top", ro.integer("top"))
    ro.finish(())
    if top > experts:
        raise ConfigError("%s.router: top %d exceeds experts %d" % (where, top, experts))
    r.finish(())
    return VozinexMoE(experts, top, ff)


def read_config(raw: Mapping[str, Any]) -> VozinexConfig:
    r = ConfigReader(raw)
    arch = r.string("architecture")
    vocab = _positive("vocab", r.integer("vocab"))
    width = _positive("width", r.integer("width"))
    norm = ConfigReader(r.any("norm") or {}, "config.json: norm")
    eps = norm.number("eps")
    norm.finish(())
    if not (eps > 0.0):
        raise ConfigError("config.json: norm.eps must be positive, found %r" % eps)
    lraw = r.any("layers")
    if not isinstance(lraw, (list, tuple)) or not lraw:
        raise ConfigError("config.json: layers must be a non-empty list")
    layers = []
    for i, l in enumerate(lraw):
        where = "config.json: layers[%d]" % i
        lr = ConfigReader(l, where)
        kind = lr.string("type")
        if kind != "attention":
            raise ConfigError("%s: type %r is not a mixer of this architecture (attention)" % (where, kind))
        mixer = _read_attention(lr.any("mixer") or {}, where + ".mixer")
        mlp = lr.any("mlp")
        layers.append(VozinexLayer(mixer, None if mlp is None else _read_moe(mlp, where + ".mlp")))
        lr.finish(())
    start = stop = 0
    times = 1
    loop = r.any("loop")
    if loop is not None:
        lp = ConfigReader(loop, "config.json: loop")
        start, stop, times = lp.integer("start", 0), lp.integer("stop", 0), lp.integer("times", 1)
        lp.finish(())
        if not (0 <= start <= stop <= len(layers)) or times < 1:
            raise ConfigError("config.json: loop must have 0 <= start <= stop <= %d layers and times >= 1, found "
                              "start %d, stop %d, times %d" % (len(layers), start, stop, times))
    r.finish()
    return VozinexConfig(arch, vocab, width, eps, tuple(layers), start, stop, times)


EMBEDDING, HEAD, FINAL_NORM = "embed", "head", "final.norm"


def build_spec(cfg: VozinexConfig) -> ModelSpec:
    norm = PartSpec("layernorm", {"eps": cfg.eps, "weight": "", "bias": ".b"})
    layers = []
    for i, l in enumerate(cfg.layers):
        m = l.mixer
        position = (PartSpec("rotary", {"base": m.rot_base, "rotary_dim": m.rot_dims}) if m.rot_dims
                    else PartSpec("none", {}))
        mixer = PartSpec("attention", {
            "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim, "scale": m.scale,
            "window": m.window, "keep_first": m.keep_first, "position": position,
            "qk_norm": {"eps": cfg.eps, "q": "q.norm", "k": "k.norm"},
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}})
        ff = None
        if l.mlp is not None:
            ff = PartSpec("moe", {
                "n_experts": l.mlp.experts, "top_k": l.mlp.top, "intermediate": l.mlp.ff, "activation": "relu2",
                "router_bias": True,
                "names": {"router": "router", "router_bias": "router.b", "up": "e%d.up", "down": "e%d.down"}})
        block = PartSpec("prenorm", {"norm1": norm, "mixer": mixer, "norm2": norm, "feed_forward": ff,
                                     "names": {"norm1": "norm1", "mixer": "mix.", "norm2": "norm2",
                                               "feed_forward": "mlp."}})
        layers.append(LayerSpec(block, "l%d." % i))
    schedule = []
    for n, (layer, p) in enumerate(cfg.run_order()):
        # every run has a cache entry of its own; a further pass over the repeated stretch begins with the embedding
        # output added to the residual stream
        schedule.append(ScheduleEntry(layer=layer, cache=n, add_embedding=p > 0 and layer == cfg.loop_start))
    spec = ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, width=cfg.width, layers=tuple(layers),
        schedule=tuple(schedule), final_norm=norm, final_norm_prefix=FINAL_NORM,
        embedding=PartSpec("table", {"name": EMBEDDING, "vocab": cfg.vocab}),
        head=PartSpec("linear", {"name": HEAD, "vocab": cfg.vocab}),
        # a layer without a feed-forward has no use for a second norm: a folder that stores one all the same is accepted
        may_ignore=tuple(n for i, l in enumerate(cfg.layers) if l.mlp is None
                         for n in ("l%d.norm2" % i, "l%d.norm2.b" % i)))
    spec.validate()
    return spec


register_architecture("Vozinex", build_spec, read_config)
