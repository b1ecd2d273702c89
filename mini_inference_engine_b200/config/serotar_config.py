"""Serotar: a decoder whose layers norm their sublayers' OUTPUTS (x <- x + scale * norm(sublayer(x)), the sublayers read the
stream itself), with latent attention without positions as the mixer, a dense feed-forward with the xIELU activation or a
routed mixture of gated experts (scores over all router outputs, a correction for the choice, groups, identity experts, a
shared expert), a per-layer input taken from the token, and a weighted average over the results of all layers so far.  The
embedding adds a row of a second table chosen by a hash of the token and the token before it.

config.json: ``architecture`` "Serotar", ``vocab``, ``width``, ``embedding`` {scale, bigram {buckets, mul_prev, mul_cur}
(optional)}, ``norm`` {eps}, ``token_side`` {dim} (optional) and ``layers``, a list of {type, mixer, mlp}:

* type "latent_attention": mixer {heads, dim, vdim, q_rank, kv_rank, scale} -- parts.attention.LatentAttention without a
  rotated part and without a gate;
* mlp {kind "dense", ff} -- parts.feedforward.ActivatedMLP;
* mlp {kind "moe", expert {ff}, router {experts, top, identity (optional), groups {count, keep} (optional)}, shared {ff}
  (optional)} -- parts.feedforward.RoutedExperts; or null.

Tensors: 'embed', 'bigram', 'side.embed', 'head', 'final.norm', and per layer i 'l<i>.norm1', 'l<i>.norm2' (one number each),
'l<i>.ls1', 'l<i>.ls2', 'l<i>.dwa', 'l<i>.side.{gate,proj,norm}', 'l<i>.mix.*', 'l<i>.mlp.*'.  This class is the only place that
knows these names; everything else works from the ``ModelSpec`` it returns."""
from __future__ import annotations

import copy
from dataclasses import dataclass

from .model_config import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_POSITION = 1 << 20       # the design has no positions at all; the engine wants a bound

_MIXER_KEYS = ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale")


def _need(d, keys, where: str):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks key(s): {', '.join(missing)}")


@dataclass(frozen=True)
class SerotarConfig:
    vocab: int
    width: int
    embedding_scale: float
    bigram: tuple | None         # (buckets, mul_prev, mul_cur)
    norm_eps: float
    side_dim: int                # 0: no per-layer token input
    layers: tuple                # the config's own dicts, checked
    architecture: str = "Serotar"

    @classmethod
    def from_dict(cls, c: dict) -> "SerotarConfig":
        _need(c, ("vocab", "width", "norm", "layers"), "the model")
        _need(c["norm"], ("eps",), "norm")
        if not isinstance(c["layers"], list) or not c["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(c["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            if layer["type"] != "latent_attention":
                raise ConfigError(f"config.json: {where}.type {layer['type']!r} is not a mixer of this design (latent_attention)")
            _need(layer["mixer"], _MIXER_KEYS, where + ".mixer")
            if any(int(layer["mixer"][k]) < 1 for k in _MIXER_KEYS[:-1]):
                raise ConfigError(f"config.json: {where}.mixer: sizes must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ("ff",), where + ".mlp")
                elif mlp["kind"] == "moe":
                    _need(mlp, ("expert", "router"), where + ".mlp")
                    _need(mlp["expert"], ("ff",), where + ".mlp.expert")
                    r = mlp["router"]
                    _need(r, ("experts", "top"), where + ".mlp.router")
                    outputs = int(r["experts"]) + int(r.get("identity", 0))
                    if int(r["experts"]) < 1 or int(r.get("identity", 0)) < 0 or not 1 <= int(r["top"]) <= outputs:
                        raise ConfigError(f"config.json: {where}.mlp.router: top must be between 1 and experts + identity")
                    g = r.get("groups")
                    if g is not None:
                        _need(g, ("count", "keep"), where + ".mlp.router.groups")
                        count, keep = int(g["count"]), int(g["keep"])
                        if count < 1 or count > 64 or outputs % count or not 1 <= keep <= count or int(r["top"]) > keep * (outputs // count):
                            raise ConfigError(f"config.json: {where}.mlp.router.groups: {count} groups (at most 64) must divide the "
                                              f"{outputs} router outputs, and the {keep} kept must hold at least top outputs")
                    if mlp.get("shared") is not None:
                        _need(mlp["shared"], ("ff",), where + ".mlp.shared")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design (dense, moe)")
            layers.append(copy.deepcopy(layer))
        emb = c.get("embedding") or {}
        big = emb.get("bigram")
        if big is not None:
            _need(big, ("buckets", "mul_prev", "mul_cur"), "embedding.bigram")
            if int(big["buckets"]) < 1 or int(big["mul_prev"]) < 0 or int(big["mul_cur"]) < 0:
                raise ConfigError("config.json: embedding.bigram: buckets must be positive and the multipliers not negative")
        side = c.get("token_side")
        if side is not None:
            _need(side, ("dim",), "token_side")
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), embedding_scale=float(emb.get("scale", 1.0)),
                  bigram=None if big is None else (int(big["buckets"]), int(big["mul_prev"]), int(big["mul_cur"])),
                  norm_eps=float(c["norm"]["eps"]), side_dim=0 if side is None else int(side["dim"]), layers=tuple(layers),
                  architecture=str(c.get("architecture", "Serotar")))
        if cfg.vocab <= 0 or cfg.width <= 0 or cfg.side_dim < 0:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg

    def to_dict(self) -> dict:
        emb = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": emb,
             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers))}
        if self.side_dim:
            d["token_side"] = {"dim": self.side_dim}
        return d

    # ------------------------------------------------------------------ description as data
    def _feed_forward(self, mlp: dict, prefix: str) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("activated_mlp", dict(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="xielu"), prefix)
        r = mlp["router"]
        g = r.get("groups") or {"count": 1, "keep": 1}
        shared = mlp.get("shared")
        return PartSpec("routed_experts", dict(
            hidden_size=self.width, num_experts=int(r["experts"]), top=int(r["top"]), expert_size=int(mlp["expert"]["ff"]),
            activation="silu", gated=True, score="softmax", correction=True, groups=int(g["count"]), keep=int(g["keep"]),
            identity=int(r.get("identity", 0)),
            shared=None if shared is None else PartSpec("clamped_glu", dict(hidden_size=self.width, intermediate_size=int(shared["ff"]),
                                                                            limit=0.0, slope=1.0, shift=0.0))), prefix)

    def model_spec(self) -> ModelSpec:
        layers = []
        L = len(self.layers)
        aliases = {"embed.weight": "embed", "embed.pair": "bigram", "embed.side": "side.embed", "head.weight": "head",
                   "final.norm.weight": "final.norm"}
        scalar_norm = lambda prefix: PartSpec("scalar_rmsnorm", dict(size=self.width, eps=self.norm_eps), prefix)
        for i, layer in enumerate(self.layers):
            p, m = f"l{i}.", layer["mixer"]
            parts = dict(
                mixer=PartSpec("latent_attention", dict(
                    hidden_size=self.width, num_heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=0, vdim=int(m["vdim"]),
                    q_rank=int(m["q_rank"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot_dims=0, rot_base=1.0,
                    eps=self.norm_eps, gate=False), p + "mix."),
                mixer_norm=scalar_norm(p + "norm1."),
                mixer_scale=PartSpec("layer_scale", dict(size=self.width, name="ls1"), p),
                depth=PartSpec("depth_average", dict(index=i, name="dwa"), p))
            aliases[p + "norm1.weight"] = p + "norm1"
            if layer.get("mlp") is not None:
                parts["feed_forward"] = self._feed_forward(layer["mlp"], p + "mlp.")
                parts["feed_forward_norm"] = scalar_norm(p + "norm2.")
                parts["feed_forward_scale"] = PartSpec("layer_scale", dict(size=self.width, name="ls2"), p)
                aliases[p + "norm2.weight"] = p + "norm2"
            if self.side_dim:
                parts["token_input"] = PartSpec("gated_table", dict(hidden_size=self.width, dim=self.side_dim, index=i), p + "side.")
                parts["token_input_norm"] = PartSpec("rmsnorm", dict(size=self.width, eps=self.norm_eps), p + "side.norm.")
                aliases[p + "side.norm.weight"] = p + "side.norm"
            layers.append(LayerSpec("output_norm_residual", parts))
        b = self.bigram or (0, 0, 0)
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("pair_embedding", dict(vocab_size=self.vocab, hidden_size=self.width, scale=self.embedding_scale,
                                                      buckets=b[0], mul_prev=b[1], mul_cur=b[2], side_width=L * self.side_dim,
                                                      history=L + 1), "embed."),
            layers=tuple(layers), run_order=tuple(RunEntry(i, i) for i in range(L)), final_norm=scalar_norm("final.norm."),
            head=PartSpec("linear_head", dict(vocab_size=self.vocab, hidden_size=self.width), "head."),
            max_position=MAX_POSITION, eos_token_id=-1, aliases=aliases)
