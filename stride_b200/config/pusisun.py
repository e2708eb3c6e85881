"""Pusisun: a decoder whose layers are listed one by one in config.json. Every layer norms each sublayer on both sides,
h <- h + norm1b(mixer(norm1(h))), then (if the layer has one) h <- h + norm2b(ff(norm2(h))), with RMS norms of plain gains. The mixers:
"attention", grouped-query softmax attention with biases, an RMS norm over the whole query and the whole key projection, no rotation but
a distance term slope_h (i - j) with slope_h = 2^(-8 (h + 1) / H) taken off the scores, a sliding window that keeps a request's first tokens
seen, and a learned sink per head in the softmax's denominator; "latent_attention", queries and keys/values through low-rank latents, a
rotated key part shared by all heads (rotate-half pairs, YaRN-scaled frequencies), every earlier key seen. The feed-forward is a mixture of
gated silu experts chosen by the largest router logits (with bias), weighted by the softmax over the chosen logits. The embedding is
scaled; a range of layers may run several times in a row with the same weights, each pass with its own cache: before every pass but the
first the embedding output is added to the stream, and before every pass one row of a stored table.

config.json keys read here:
  architecture "Pusisun"; vocab, width; norm.eps; embedding.scale; loop {start, stop, times} (absent: no loop);
  layers[i]: type ("attention" | "latent_attention"), mixer {...}, mlp ({kind "moe", expert {ff}, router {experts, top}} | null);
    attention mixer: heads, kv_heads, dim, vdim, scale, mask {size, keep_first} (absent: every earlier key);
    latent_attention mixer: heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot {dims (= rot_dim), base, scaling {factor, original,
                            fast, slow} (absent: unscaled frequencies)}.
Tensor names: embed, head, final.norm, loop.step, l<i>.norm1, l<i>.norm1b, l<i>.norm2, l<i>.norm2b,
  l<i>.mix.{q,q.b,k,k.b,v,v.b,q.norm,k.norm,sink,o} or l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o},
  l<i>.mlp.{router,router.b,e<j>.gate,e<j>.up,e<j>.down}.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .keralorn import _get
from .llama import ConfigError
from .registry import Architecture, register_architecture

DEFAULT_MAX_POSITIONS = 32768      # config.json names no longest sequence; `max_context` of the engine overrides this
SLOPE_BITS = 8.0                   # the distance slopes of the design's grouped attention: 2^(-8 (h + 1) / H)


@dataclass(frozen=True)
class PusisunLayer:
    kind: str                      # "attention" | "latent_attention"
    heads: int
    dim: int
    vdim: int
    scale: float
    kv_heads: int = 0              # attention
    window: int = 0
    keep_first: int = 0
    rot_dim: int = 0               # latent attention
    q_rank: int = 0
    kv_rank: int = 0
    rot_base: float = 10000.0
    rot_scaling: Optional[tuple] = None     # (factor, original, fast, slow)
    ff: int = 0                    # one expert's size; 0: no feed-forward
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class PusisunConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 0            # 0: no loop declared
    max_positions: int = DEFAULT_MAX_POSITIONS
    eos_token_ids: tuple = ()

    @staticmethod
    def from_dict(j: dict) -> "PusisunConfig":
        vocab = _get(j, "vocab", "", int, True)
        width = _get(j, "width", "", int, True)
        eps = _get(j.get("norm"), "eps", "norm.", float, True)
        emb = j.get("embedding")
        embedding_scale = _get(emb, "scale", "embedding.", float) if emb else 1.0
        raw_layers = j.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, l in enumerate(raw_layers):
            w = f"layers[{i}]."
            kind = _get(l, "type", w)
            m = _get(l, "mixer", w)
            mw = w + "mixer."
            fields = {}
            mlp = l.get("mlp")
            if mlp is not None:
                mk = _get(mlp, "kind", w + "mlp.")
                if mk != "moe":
                    raise ConfigError(f"config.json: '{w}mlp.kind' {mk!r} is not supported (moe)")
                r = _get(mlp, "router", w + "mlp.")
                rw = w + "mlp.router."
                experts, top = _get(r, "experts", rw, int, True), _get(r, "top", rw, int, True)
                if top > experts:
                    raise ConfigError(f"config.json: '{rw}' chooses {top} of {experts} experts")
                fields.update(ff=_get(_get(mlp, "expert", w + "mlp."), "ff", w + "mlp.expert.", int, True), experts=experts, top=top)
            heads, dim, vdim = (_get(m, k, mw, int, True) for k in ("heads", "dim", "vdim"))
            scale = _get(m, "scale", mw, float)
            if kind == "attention":
                kv = _get(m, "kv_heads", mw, int, True)
                if heads % kv:
                    raise ConfigError(f"config.json: '{mw}heads' {heads} is no multiple of kv_heads {kv}")
                mask = m.get("mask")
                window = keep = 0
                if mask:
                    window = _get(mask, "size", mw + "mask.", int, True)
                    keep = mask.get("keep_first") or 0
                    if not isinstance(keep, int) or isinstance(keep, bool) or keep < 0:
                        raise ConfigError(f"config.json: '{mw}mask.keep_first' must be an integer >= 0, got {keep!r}")
                layers.append(PusisunLayer("attention", heads, dim, vdim, scale, kv_heads=kv, window=window, keep_first=keep, **fields))
            elif kind == "latent_attention":
                rot_dim = _get(m, "rot_dim", mw, int)
                if rot_dim < 0 or rot_dim % 2:
                    raise ConfigError(f"config.json: '{mw}rot_dim' {rot_dim} must be even and not negative")
                base, scaling = 10000.0, None
                if rot_dim:
                    rot = _get(m, "rot", mw)
                    if _get(rot, "dims", mw + "rot.", int) != rot_dim:
                        raise ConfigError(f"config.json: '{mw}rot.dims' {rot['dims']} is not rot_dim {rot_dim}: the rotated part is rotated whole")
                    base = _get(rot, "base", mw + "rot.", float, True)
                    sc = rot.get("scaling")
                    if sc:
                        sw = mw + "rot.scaling."
                        scaling = (_get(sc, "factor", sw, float, True), _get(sc, "original", sw, float, True), _get(sc, "fast", sw, float, True),
                                   _get(sc, "slow", sw, float, True))
                layers.append(PusisunLayer("latent_attention", heads, dim, vdim, scale, rot_dim=rot_dim, q_rank=_get(m, "q_rank", mw, int, True),
                                           kv_rank=_get(m, "kv_rank", mw, int, True), rot_base=base, rot_scaling=scaling, **fields))
            else:
                raise ConfigError(f"config.json: '{w}type' {kind!r} is not supported (attention, latent_attention)")
        start = stop = times = 0
        loop = j.get("loop")
        if loop:
            start, stop, times = (_get(loop, k, "loop.", int) for k in ("start", "stop", "times"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: 'loop' {loop!r} does not fit {len(layers)} layers")
        eos = j.get("eos_token_id")
        eos = () if eos is None else tuple(eos) if isinstance(eos, list) else (int(eos),)
        return PusisunConfig(vocab, width, eps, embedding_scale, tuple(layers), start, stop, times, eos_token_ids=eos)


def pusisun_model_spec(cfg: PusisunConfig) -> ModelSpec:
    W = cfg.width

    def norm(name):
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.eps}, {"weight": name})

    def result_norm(name):
        return PartSpec("rmsnorm", {"size": W, "eps": cfg.eps}, {"weight": name})     # category branch_scale: the norm behind a sublayer

    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.kind == "attention":
            mixer = PartSpec("masked_attention",
                             {"hidden_size": W, "num_heads": l.heads, "num_kv_heads": l.kv_heads, "key_dim": l.dim, "value_dim": l.vdim,
                              "scale": l.scale, "window": l.window, "keep_first": l.keep_first, "norm_eps": cfg.eps, "qk_norm": True, "bias": True,
                              "slope_bits": SLOPE_BITS, "sink": True},
                             {"q": p + "mix.q", "k": p + "mix.k", "v": p + "mix.v", "o": p + "mix.o", "q_bias": p + "mix.q.b", "k_bias": p + "mix.k.b",
                              "v_bias": p + "mix.v.b", "q_norm": p + "mix.q.norm", "k_norm": p + "mix.k.norm", "sink": p + "mix.sink"})
        else:
            position = None
            if l.rot_dim:
                params = {"head_dim": l.rot_dim, "rotary_dim": l.rot_dim, "theta": l.rot_base}
                if l.rot_scaling is None:
                    params.update(scaling={"rope_type": "default"}, exact_angles=True)
                else:
                    f, o, fast, slow = l.rot_scaling
                    params.update(scaling={"rope_type": "yarn", "factor": f, "original": o, "fast": fast, "slow": slow})
                position = PartSpec("rope", params)
            mixer = PartSpec("latent_attention",
                             {"hidden_size": W, "num_heads": l.heads, "key_dim": l.dim, "rot_dim": l.rot_dim, "value_dim": l.vdim, "q_rank": l.q_rank,
                              "kv_rank": l.kv_rank, "scale": l.scale, "norm_eps": cfg.eps, "position": position},
                             {"dq": p + "mix.dq", "dq_norm": p + "mix.dq.norm", "uq": p + "mix.uq", "dkv": p + "mix.dkv",
                              "dkv_norm": p + "mix.dkv.norm", "uk": p + "mix.uk", "uv": p + "mix.uv", "o": p + "mix.o"})
        parts = {"mixer": mixer, "mixer_norm": norm(p + "norm1"), "mixer_scale": result_norm(p + "norm1b")}
        if l.ff:
            E = range(l.experts)
            ff = PartSpec("routed", {"hidden_size": W, "intermediate_size": l.ff, "experts": l.experts, "top": l.top, "weights_from": "logits",
                                     "expert": "silu_gated"},
                          {"router": p + "mlp.router", "correction": p + "mlp.router.b", "gate": tuple(f"{p}mlp.e{e}.gate" for e in E),
                           "up": tuple(f"{p}mlp.e{e}.up" for e in E), "down": tuple(f"{p}mlp.e{e}.down" for e in E)})
            parts.update(feed_forward=ff, feed_forward_norm=norm(p + "norm2"), feed_forward_scale=result_norm(p + "norm2b"))
            layers.append(LayerSpec("prenorm_scaled", parts))
        else:
            layers.append(LayerSpec("prenorm_scaled_mixer", parts))
    L = len(layers)
    order = list(range(L))
    if cfg.loop_times:
        # what stands in front of a pass is a layer of its own kind, one per pass (each adds its own row of the table, all but the
        # first the embedding output too); every pass of a layer is a schedule entry of its own and so has a cache of its own
        order = list(range(cfg.loop_start))
        for t in range(cfg.loop_times):
            layers.append(LayerSpec("rewrite", rewrite=PartSpec("embedding_add", {"hidden_size": W, "rows": cfg.loop_times, "row": t,
                                                                                  "add_embedding": t > 0}, {"table": "loop.step"})))
            order += [L + t] + list(range(cfg.loop_start, cfg.loop_stop))
        order += list(range(cfg.loop_stop, L))
    return ModelSpec(
        vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec("lookup", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale}, {"weight": "embed"}),
        layers=tuple(layers), schedule=tuple(ScheduleEntry(i) for i in order),
        final_norm=norm("final.norm"),
        head=PartSpec("linear", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False}, {"weight": "head", "tied_to": "embed"}),
        max_positions=cfg.max_positions, eos_token_ids=cfg.eos_token_ids)


register_architecture(Architecture("Pusisun", PusisunConfig.from_dict, pusisun_model_spec), "pusisun")
