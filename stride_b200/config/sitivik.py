"""Sitivik: a decoder whose layers are listed one by one in config.json. Every layer is a pre-norm block with a layer scale on each
sublayer, h <- h + s1 * mixer(norm1(h)), then (if the layer has one) h <- h + s2 * ff(norm2(h)) with a gated silu feed-forward, then a
per-layer token input: e = a slice of a second embedding table, h <- h + norm(W_proj (gelu_tanh(W_gate h) * e)). RMS norms with plain gains;
the embedding is scaled; the head is the embedding table. The mixers:

"parallel": windowed softmax attention (biases, q/k norm over the whole projection, interleaved rotary pairs with Llama-3.1 wave scaling,
  an elementwise output gate, an output bias) beside retention (linear attention with a fixed decay per head, rotate-half pairs, every
  head's result divided by its root mean square, a silu gate); each result is RMS-normed over the width with its own gain, and the mixer's
  result is half their sum.
"attention": differential attention (two softmax maps per head over shared values, a1 - lambda a2, a norm per head, a gate per head), causal,
  no rotation, queries that grow with the logarithm of the position.
"parallel_2": chunked softmax attention with a sink of score 0 (biases, q/k norm per head, interleaved rotary pairs, an elementwise gate)
  beside the gated delta rule; the result is left_scale * left + right_scale * right.

config.json keys read here:
  architecture "Sitivik"; vocab, width; norm.eps; embedding.scale (absent: 1); token_side.dim (absent: no per-layer token input);
  layers[i]: type, mixer {...}, mlp ({kind "dense", ff} | null);
    attention members: heads, kv_heads, dim, vdim, scale, mask.size (absent: every earlier key), rot {dims, base, scaling {factor, low, high,
    original}} (absent: no rotation);
    "attention" also: diff, q_temp {coef, every} (absent: none); retention: heads, dim, vdim, decay [heads], rot {dims, base};
    gated delta rule: heads, kv_heads, dim, vdim, conv; "parallel_2" also: left_scale, right_scale.
  The ranks of the delta rule's two low-rank projections are sizes that only the tensors' shapes tell: `with_tensor_shapes` writes them
  into the mixer's entry as decay_rank and gate_rank before the configuration is parsed (a configuration without a checkpoint, for random
  weights, may name them itself; absent: vdim / 4).
Tensor names: embed, side.embed, final.norm, l<i>.{norm1,norm2,ls1,ls2}, l<i>.side.{gate,proj,norm}, l<i>.mlp.{gate,up,down},
  l<i>.mix.[left.|right.]{q,k,v,g,o} with .b, .norm and .conv behind a name, and l<i>.mix.{lq1,lk1,lq2,lk2},
  l<i>.mix.right.{b,A_log,norm,a1,a2,dt_bias,g1,g2}, l<i>.mix.{left,right}.out.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .keralorn import _get
from .llama import ConfigError
from .registry import Architecture, register_architecture

DEFAULT_MAX_POSITIONS = 32768      # config.json names no longest sequence; `max_context` of the engine overrides this


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    scaling: Optional[tuple] = None         # (factor, low, high, original)


@dataclass(frozen=True)
class SoftmaxMember:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    mask: int = 0                           # the window's or the chunk's size; 0: every earlier key
    rot: Optional[Rotation] = None
    diff: float = 0.0
    q_temp: Optional[tuple] = None          # (coef, every)


@dataclass(frozen=True)
class RetentionMember:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: Optional[Rotation] = None


@dataclass(frozen=True)
class DeltaMember:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: int = 0                     # 0: taken from the checkpoint's shapes
    gate_rank: int = 0


@dataclass(frozen=True)
class SitivikLayer:
    kind: str                               # "parallel" | "attention" | "parallel_2"
    left: Optional[SoftmaxMember]
    right: object = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    ff: int = 0                             # 0: no feed-forward


@dataclass(frozen=True)
class SitivikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    side_dim: int
    layers: tuple
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    @staticmethod
    def from_dict(j: dict) -> "SitivikConfig":
        vocab = _get(j, "vocab", "", int, True)
        width = _get(j, "width", "", int, True)
        eps = _get(j.get("norm"), "eps", "norm.", float, True)
        emb = j.get("embedding")
        embedding_scale = _get(emb, "scale", "embedding.", float) if emb else 1.0
        side = j.get("token_side")
        side_dim = _get(side, "dim", "token_side.", int, True) if side else 0
        raw_layers = j.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")

        def rotation(m, w):
            rot = m.get("rot")
            if not rot:
                return None
            dims = _get(rot, "dims", w + "rot.", int, True)
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"config.json: '{w}rot.dims' {dims} must be even and at most dim {m['dim']}")
            sc = rot.get("scaling")
            scaling = None
            if sc:
                sw = w + "rot.scaling."
                scaling = tuple(_get(sc, k, sw, float, True) for k in ("factor", "low", "high", "original"))
                if scaling[2] == scaling[1]:
                    raise ConfigError(f"config.json: '{sw}high' equals '{sw}low'")
            return Rotation(dims, _get(rot, "base", w + "rot.", float, True), scaling)

        def softmax_member(m, w, masked: bool, differential: bool = False):
            heads, kv, dim, vdim = (_get(m, k, w, int, True) for k in ("heads", "kv_heads", "dim", "vdim"))
            if heads % kv:
                raise ConfigError(f"config.json: '{w}heads' {heads} is no multiple of kv_heads {kv}")
            mask = _get(m["mask"], "size", w + "mask.", int, True) if masked and m.get("mask") else 0      # (no mask: every earlier key)
            qt = m.get("q_temp")
            q_temp = (_get(qt, "coef", w + "q_temp.", float), _get(qt, "every", w + "q_temp.", int, True)) if qt else None
            return SoftmaxMember(heads, kv, dim, vdim, _get(m, "scale", w, float), mask, rotation(m, w),
                                 _get(m, "diff", w, float) if differential else 0.0, q_temp)

        layers = []
        for i, l in enumerate(raw_layers):
            w = f"layers[{i}]."
            kind, m, mw = _get(l, "type", w), _get(l, "mixer", w), w + "mixer."
            ff = 0
            mlp = l.get("mlp")
            if mlp is not None:
                if _get(mlp, "kind", w + "mlp.") != "dense":
                    raise ConfigError(f"config.json: '{w}mlp.kind' {mlp['kind']!r} is not supported (dense)")
                ff = _get(mlp, "ff", w + "mlp.", int, True)
            if kind == "attention":
                layers.append(SitivikLayer(kind, softmax_member(m, mw, False, True), ff=ff))
            elif kind == "parallel":
                r, rw = _get(m, "right", mw), mw + "right."
                heads, dim, vdim = (_get(r, k, rw, int, True) for k in ("heads", "dim", "vdim"))
                decay = _get(r, "decay", rw)
                if not isinstance(decay, list) or len(decay) != heads or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                    raise ConfigError(f"config.json: '{rw}decay' must list {heads} numbers, one per head")
                right = RetentionMember(heads, dim, vdim, tuple(float(d) for d in decay), rotation(r, rw))
                layers.append(SitivikLayer(kind, softmax_member(_get(m, "left", mw), mw + "left.", True), right, 0.5, 0.5, ff))
            elif kind == "parallel_2":
                r, rw = _get(m, "right", mw), mw + "right."
                heads, kv, dim, vdim, taps = (_get(r, k, rw, int, True) for k in ("heads", "kv_heads", "dim", "vdim", "conv"))
                if heads % kv:
                    raise ConfigError(f"config.json: '{rw}heads' {heads} is no multiple of kv_heads {kv}")
                if taps > 8:
                    raise ConfigError(f"config.json: '{rw}conv' {taps} exceeds 8 taps, the most the kernel holds")
                ra = _get(r, "decay_rank", rw, int, True) if r.get("decay_rank") is not None else max(vdim // 4, 1)
                rg = _get(r, "gate_rank", rw, int, True) if r.get("gate_rank") is not None else max(vdim // 4, 1)
                right = DeltaMember(heads, kv, dim, vdim, taps, ra, rg)
                layers.append(SitivikLayer(kind, softmax_member(_get(m, "left", mw), mw + "left.", True), right,
                                           _get(m, "left_scale", mw, float), _get(m, "right_scale", mw, float), ff))
            else:
                raise ConfigError(f"config.json: '{w}type' {kind!r} is not supported (parallel, attention, parallel_2)")
        eos = j.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (int(eos),)
        return SitivikConfig(vocab, width, eps, embedding_scale, side_dim, tuple(layers), eos_token_ids=eos)


def with_tensor_shapes(config: dict, shapes: dict) -> dict:
    """config.json with the sizes that only the checkpoint tells: the ranks of the delta rule's low-rank projections, read from the shapes
    (name -> shape) of l<i>.mix.right.a1 and .g1 and written into a copy of the configuration as decay_rank and gate_rank."""
    import copy
    out = None
    for i, l in enumerate(config.get("layers") or []):
        if not (isinstance(l, dict) and l.get("type") == "parallel_2" and isinstance((l.get("mixer") or {}).get("right"), dict)):
            continue
        for key, name in (("decay_rank", f"l{i}.mix.right.a1"), ("gate_rank", f"l{i}.mix.right.g1")):
            if name in shapes and len(shapes[name]) == 2:
                out = out if out is not None else copy.deepcopy(config)
                out["layers"][i]["mixer"]["right"][key] = int(shapes[name][0])
    return out if out is not None else config


def _rope(rot: Optional[Rotation], dim: int):
    if rot is None:
        return None
    params = {"head_dim": dim, "rotary_dim": rot.dims, "theta": rot.base, "exact_angles": True, "scaling": {"rope_type": "default"}}
    if rot.scaling:
        factor, low, high, original = rot.scaling
        params["scaling"] = {"rope_type": "llama3", "factor": factor, "low_freq_factor": low, "high_freq_factor": high,
                             "original_max_position_embeddings": original}
    return PartSpec("rope", params)


def sitivik_model_spec(cfg: SitivikConfig) -> ModelSpec:
    W = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.eps}, {"weight": name})

    def softmax(m: SoftmaxMember, p: str, **more):
        params = {"hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "key_dim": m.dim, "value_dim": m.vdim, "scale": m.scale,
                  "norm_eps": cfg.eps, "bias": True, "position": _rope(m.rot, m.dim), "interleaved": True, "q_temp": m.q_temp}
        params.update(more)
        names = {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o", "q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b",
                 "o_bias": p + "o.b", "q_norm": p + "q.norm", "k_norm": p + "k.norm", "lq1": p + "lq1", "lk1": p + "lk1", "lq2": p + "lq2",
                 "lk2": p + "lk2"}
        return PartSpec("gated_attention", params, names)

    layers, order = [], []
    L = len(cfg.layers)
    for i, l in enumerate(cfg.layers):
        p = f"l{i}.mix."
        if l.kind == "attention":
            mixer = softmax(l.left, p, maps=2, diff=l.left.diff, gate="head")
        elif l.kind == "parallel":
            r = l.right
            left = softmax(l.left, p + "left.", window=l.left.mask, qk_norm="projection", o_bias=True, gate="element")
            right = PartSpec("retention", {"hidden_size": W, "num_heads": r.heads, "key_dim": r.dim, "value_dim": r.vdim, "decay": r.decay,
                                           "norm_eps": cfg.eps, "position": _rope(r.rot, r.dim)},
                             {k: p + "right." + k for k in ("q", "k", "v", "g", "o")})
            mixer = PartSpec("parallel_normed", {"hidden_size": W, "members": (left, right), "scales": (l.left_scale, l.right_scale), "eps": cfg.eps},
                             {"norms": (p + "left.out", p + "right.out")})
        else:
            r, q = l.right, p + "right."
            left = softmax(l.left, p + "left.", chunk=l.left.mask, qk_norm="head", sink="zero", gate="element")
            right = PartSpec("gated_delta", {"hidden_size": W, "num_heads": r.heads, "num_kv_heads": r.kv_heads, "key_dim": r.dim, "value_dim": r.vdim,
                                             "taps": r.taps, "decay_rank": r.decay_rank, "gate_rank": r.gate_rank, "norm_eps": cfg.eps},
                             {"q": q + "q", "k": q + "k", "v": q + "v", "q_conv": q + "q.conv", "k_conv": q + "k.conv", "v_conv": q + "v.conv",
                              "beta": q + "b", "a_log": q + "A_log", "dt_bias": q + "dt_bias", "a1": q + "a1", "a2": q + "a2", "g1": q + "g1",
                              "g2": q + "g2", "norm": q + "norm", "o": q + "o"})
            mixer = PartSpec("parallel", {"hidden_size": W, "members": (left, right), "scales": (l.left_scale, l.right_scale)})
        b = f"l{i}."
        parts = {"mixer": mixer, "mixer_norm": norm(b + "norm1"), "mixer_scale": PartSpec("layer_scale", {"size": W}, {"weight": b + "ls1"})}
        if l.ff:
            parts.update(feed_forward=PartSpec("swiglu", {"hidden_size": W, "intermediate_size": l.ff},
                                               {"gate": b + "mlp.gate", "up": b + "mlp.up", "down": b + "mlp.down"}),
                         feed_forward_norm=norm(b + "norm2"), feed_forward_scale=PartSpec("layer_scale", {"size": W}, {"weight": b + "ls2"}))
            layers.append(LayerSpec("prenorm_scaled", parts))
        else:
            layers.append(LayerSpec("prenorm_scaled_mixer", parts))
        order.append(i)
    if cfg.side_dim:
        # the per-layer token input is a layer of its own kind scheduled behind every layer (it holds no cache)
        for i in range(L):
            b = f"l{i}.side."
            layers.append(LayerSpec("rewrite", rewrite=PartSpec("token_side", {"hidden_size": W, "vocab_size": cfg.vocab, "dim": cfg.side_dim,
                                                                                "slices": L, "index": i, "eps": cfg.eps, "activation": "gelu_tanh"},
                                                                {"table": "side.embed", "gate": b + "gate", "proj": b + "proj", "norm": b + "norm"})))
        order = [k for i in range(L) for k in (i, L + i)]
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("lookup", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale}, {"weight": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in order),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": True}, {"weight": "head", "tied_to": "embed"}),
        max_positions=cfg.max_positions, eos_token_ids=cfg.eos_token_ids)


register_architecture(Architecture("Sitivik", SitivikConfig.from_dict, sitivik_model_spec, with_tensor_shapes), "sitivik")
