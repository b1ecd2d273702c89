"""Luluzen: a pre-norm decoder (layer norm with a weight, no bias) whose layers are listed one by one in config.json, each
with a mixer of its own kind and sizes, and of which a stretch of layers may run several times with the same weights.

config.json: ``architecture`` "Luluzen", ``vocab``, ``width``, ``norm`` {eps}, ``logit_softcap`` (optional), ``loop`` {start,
stop, times} (optional) and ``layers``, a list of {type, mixer, mlp}:

* type "lightning": mixer {heads, dim, vdim, decay [one per head]} -- parts.retention.LightningAttention;
* type "parallel": mixer {left_scale, right_scale, left {heads, kv_heads, dim, vdim, scale, bias_max, q_temp {coef, every}},
  right {heads, kv_heads, dim, vdim, conv}} -- softmax attention with biases, per-head q/k norm, a temperature by position and a
  learned bias by distance (parts.attention.GatedAttention) beside a gated delta rule (parts.delta.ChannelDelta);
* type "parallel_2": mixer {left_scale, right_scale, left {heads, kv_heads, dim, vdim, scale, softcap, mask {size}, rot {base,
  dims}}, right {heads, dim, vdim, gate_cap}} -- windowed, capped, gated softmax attention with a sink beside a matrix memory
  with exponential gates (parts.matrix_memory.MatrixMemory); both kinds are joined by parts.parallel.ParallelMixers with the
  two scales;
* mlp {kind "dense", ff} -- gelu-gated feed-forward (parts.feedforward.ClampedGLU with gelu's constants) -- or {kind "moe",
  router {experts, top}, expert {ff, limit}} -- parts.feedforward.RoutedExperts with sigmoid scores on the experts' inputs --
  or null for a layer without a feed-forward.

The layers ``loop.start`` .. ``loop.stop`` - 1 run ``loop.times`` times in a row, every pass on caches and states of its own; in
front of every pass the stream is mixed with the embedding's output and shifted (parts.block.StreamMix, tensors 'loop.in' and
'loop.step').

Tensors: 'embed', 'final.norm', 'loop.in', 'loop.step', and per layer i 'l<i>.norm1', 'l<i>.norm2', 'l<i>.mix.*', 'l<i>.mlp.*'.
The output head is the embedding table.  This class is the only place that knows these names; everything else works from
the ``ModelSpec`` it returns."""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass

from .model_config import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

MAX_POSITION = 1 << 20       # the design has no position limit (angles come from the position itself); the engine wants a bound
GELU_SLOPE = 2.0 * math.sqrt(2.0 / math.pi)      # gelu_tanh(z) = z sigmoid(GELU_SLOPE (z + GELU_CUBIC z^3))
GELU_CUBIC = 0.044715


def _need(d, keys, where: str):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in d]
    if missing:
        raise ConfigError(f"config.json: {where} lacks key(s): {', '.join(missing)}")


@dataclass(frozen=True)
class LuluzenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple            # the config's own dicts, checked
    loop: tuple | None       # (start, stop, times)
    logit_softcap: float = 0.0
    architecture: str = "Luluzen"

    @classmethod
    def from_dict(cls, c: dict) -> "LuluzenConfig":
        _need(c, ("vocab", "width", "norm", "layers"), "the model")
        _need(c["norm"], ("eps",), "norm")
        if not isinstance(c["layers"], list) or not c["layers"]:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, layer in enumerate(c["layers"]):
            where = f"layers[{i}]"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer["type"] == "lightning":
                _need(m, ("heads", "dim", "vdim", "decay"), where + ".mixer")
                if len(m["decay"]) != m["heads"]:
                    raise ConfigError(f"config.json: {where}.mixer has {len(m['decay'])} decays for {m['heads']} heads")
            elif layer["type"] in ("parallel", "parallel_2"):
                _need(m, ("left", "right", "left_scale", "right_scale"), where + ".mixer")
                _need(m["left"], ("heads", "kv_heads", "dim", "vdim", "scale"), where + ".mixer.left")
                if layer["type"] == "parallel":
                    _need(m["left"], ("bias_max",), where + ".mixer.left")
                    if m["left"].get("q_temp") is not None:
                        _need(m["left"]["q_temp"], ("coef", "every"), where + ".mixer.left.q_temp")
                    _need(m["right"], ("heads", "kv_heads", "dim", "vdim", "conv"), where + ".mixer.right")
                else:
                    if m["left"].get("mask") is not None:
                        _need(m["left"]["mask"], ("size",), where + ".mixer.left.mask")
                    if m["left"].get("rot") is not None:
                        _need(m["left"]["rot"], ("base", "dims"), where + ".mixer.left.rot")
                    _need(m["right"], ("heads", "dim", "vdim"), where + ".mixer.right")
            else:
                raise ConfigError(f"config.json: {where}.type {layer['type']!r} is not a mixer of this design (lightning, parallel, parallel_2)")
            mlp = layer.get("mlp")
            if mlp is not None:
                _need(mlp, ("kind",), where + ".mlp")
                if mlp["kind"] == "dense":
                    _need(mlp, ("ff",), where + ".mlp")
                elif mlp["kind"] == "moe":
                    _need(mlp, ("router", "expert"), where + ".mlp")
                    _need(mlp["router"], ("experts", "top"), where + ".mlp.router")
                    _need(mlp["expert"], ("ff", "limit"), where + ".mlp.expert")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design (dense, moe)")
            layers.append(copy.deepcopy(layer))
        loop = None
        if c.get("loop") is not None:
            _need(c["loop"], ("start", "stop", "times"), "loop")
            loop = (int(c["loop"]["start"]), int(c["loop"]["stop"]), int(c["loop"]["times"]))
            if not 0 <= loop[0] < loop[1] <= len(layers) or loop[2] < 1:
                raise ConfigError(f"config.json: loop {c['loop']} does not name a stretch of the {len(layers)} layers run at least once")
        cfg = cls(vocab=int(c["vocab"]), width=int(c["width"]), norm_eps=float(c["norm"]["eps"]), layers=tuple(layers), loop=loop,
                  logit_softcap=float(c.get("logit_softcap") or 0.0), architecture=str(c.get("architecture", "Luluzen")))
        if cfg.vocab <= 0 or cfg.width <= 0:
            raise ConfigError("config.json: vocab and width must be positive")
        return cfg

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
             "layers": copy.deepcopy(list(self.layers))}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d

    # ------------------------------------------------------------------ description as data
    def _norm(self, prefix: str) -> PartSpec:
        return PartSpec("layernorm", dict(size=self.width, eps=self.norm_eps), prefix)

    def _mixer(self, layer: dict, prefix: str) -> PartSpec:
        m, w, eps = layer["mixer"], self.width, self.norm_eps
        if layer["type"] == "lightning":
            return PartSpec("lightning_attention", dict(hidden_size=w, num_heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                                        decay=tuple(float(d) for d in m["decay"]), eps=eps), prefix)
        left, right = m["left"], m["right"]
        common = dict(hidden_size=w, num_heads=int(left["heads"]), num_kv_heads=int(left["kv_heads"]), dim=int(left["dim"]),
                      vdim=int(left["vdim"]), scale=float(left["scale"]), eps=eps, head_temp=False)
        if layer["type"] == "parallel":
            temp = left.get("q_temp")
            attention = PartSpec("gated_attention", dict(
                common, rot_dims=0, rot_base=1.0, qk_norm="head", gate=False, bias=True,
                q_temp=(float(temp["coef"]), int(temp["every"])) if temp else None, rel_bias=(None, float(left["bias_max"]))))
            other = PartSpec("channel_delta", dict(hidden_size=w, num_heads=int(right["heads"]), num_kv_heads=int(right["kv_heads"]),
                                                   dim=int(right["dim"]), vdim=int(right["vdim"]), taps=int(right["conv"]), eps=eps))
        else:
            rot, mask = left.get("rot"), left.get("mask")
            attention = PartSpec("gated_attention", dict(
                common, rot_dims=int(rot["dims"]) if rot else 0, rot_base=float(rot["base"]) if rot else 1.0, rot_pairing="interleaved",
                qk_norm="projection", gate=True, window=int(mask["size"]) if mask else None, softcap=float(left.get("softcap") or 0.0),
                sink=True))
            other = PartSpec("matrix_memory", dict(hidden_size=w, num_heads=int(right["heads"]), dim=int(right["dim"]),
                                                   vdim=int(right["vdim"]), eps=eps, gate_cap=float(right.get("gate_cap") or 0.0)))
        return PartSpec("parallel", dict(hidden_size=w, branches={"left": attention, "right": other},
                                         scales=(float(m["left_scale"]), float(m["right_scale"]))), prefix)

    def _feed_forward(self, mlp: dict, prefix: str) -> PartSpec:
        if mlp["kind"] == "dense":
            # gelu in its tanh form is z sigmoid(2 sqrt(2/pi) (z + 0.044715 z^3)): the gated feed-forward's sigmoid with a cubic term
            return PartSpec("clamped_glu", dict(hidden_size=self.width, intermediate_size=int(mlp["ff"]), limit=-GELU_CUBIC,
                                                slope=GELU_SLOPE, shift=0.0), prefix)
        return PartSpec("routed_experts", dict(hidden_size=self.width, num_experts=int(mlp["router"]["experts"]), top=int(mlp["router"]["top"]),
                                               expert_size=int(mlp["expert"]["ff"]), activation="clamped_in", gated=True, score="sigmoid",
                                               limit=float(mlp["expert"]["limit"])), prefix)

    def run_plan(self) -> list:
        """[(layer, pass or None)] in running order: a pass number stands with the first layer of a pass of the repeated stretch."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lo, hi, times = self.loop
        plan = [(i, None) for i in range(lo)]
        for t in range(times):
            plan += [(i, t if i == lo else None) for i in range(lo, hi)]
        return plan + [(i, None) for i in range(hi, n)]

    def model_spec(self) -> ModelSpec:
        layers, aliases = [], {"embed.weight": "embed", "final.norm.weight": "final.norm"}
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            parts = dict(mixer=self._mixer(layer, p + "mix."), mixer_norm=self._norm(p + "norm1."))
            aliases[p + "norm1.weight"] = p + "norm1"
            mlp = layer.get("mlp")
            if mlp is not None:
                parts["feed_forward"] = self._feed_forward(mlp, p + "mlp.")
                parts["feed_forward_norm"] = self._norm(p + "norm2.")
                aliases[p + "norm2.weight"] = p + "norm2"
            layers.append(LayerSpec("prenorm_residual", parts))
        # the steps in front of the passes are entries of the layer list too (they share 'loop.in' and 'loop.step'); every run
        # of a layer has a cache id of its own, so every pass keeps its own keys, values and states
        run, mixes = [], {}
        for cache_id, (i, t) in enumerate(self.run_plan()):          # (a mixing step keeps nothing: its cache id is a negative number)
            if t is not None:
                if t not in mixes:
                    mixes[t] = len(layers)
                    layers.append(LayerSpec("stream_mix_step", dict(mix=PartSpec("stream_mix", dict(
                        hidden_size=self.width, rows=self.loop[2], index=t), "loop."))))
                run.append(RunEntry(mixes[t], -1 - t))
            run.append(RunEntry(i, cache_id))
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=self.width,
            embedding=PartSpec("embedding", dict(vocab_size=self.vocab, hidden_size=self.width, keep_output=self.loop is not None), "embed."),
            layers=tuple(layers), run_order=tuple(run), final_norm=self._norm("final.norm."),
            head=PartSpec("linear_head", dict(vocab_size=self.vocab, hidden_size=self.width, tied=True, softcap=self.logit_softcap), "embed."),
            max_position=MAX_POSITION, eos_token_id=-1, aliases=aliases)
