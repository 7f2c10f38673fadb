"""Typed configuration of the Gizulorn decoder, read from its own config.json keys, and its model description.

config.json: `architecture` "Gizulorn"; `vocab`, `width`; `norm.eps`; `layers`: a list whose entries give `type` (the
mixer kind: "retention" or "parallel"), `mixer` (its sizes and constants) and `mlp` (the feed-forward: `kind` "dense"
or "moe", or null for none). Tensor names: `embed`, `final.norm`, `head`, and per layer i `l<i>.norm1`, `l<i>.norm2`,
`l<i>.mix.*`, `l<i>.mlp.*`.

What the design is made of (every piece is a part of this package that another design can name with other constants):

  layer         x <- x + mixer(norm1(x)); x <- x + ff(norm2(x))        (block `pre_norm`, the second half optional)
  retention     mixer `retention`: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t per head with a fixed decay per
                head; q and k rotated by position (halves paired), k scaled by dim^-1/2; every head's o divided by its
                root mean square, times silu(W_g h), then the output product; S is request state in 32-bit
  parallel      mixer `parallel_mixers`: left_scale * left + right_scale * right, both reading the same input
    left        mixer `sink_attention`: grouped-query attention over a sliding window that also keeps the first tokens
                of the sequence, a learned per-head sink in the softmax's denominator, neighbours paired in the
                rotation, frequencies scaled by wavelength (`rope`, kind "llama3", angles in 64-bit)
    right       mixer `gated_delta`: q, k, v through a short causal convolution and silu; q, k unit vectors per head;
                S <- g * S (a decay per head and key channel), u = beta (v - S^T k), S <- S + k u^T, o = S^T q; o
                divided by its root mean square per head, times a weight and a sigmoid gate; S and the convolution's
                last inputs are request state
  feed-forward  `swiglu` (dense) or `routed_moe`: softmax router in 32-bit, the best `groups.keep` of `groups.count`
                groups of neighbouring experts, `top` experts by score, weights the scores themselves, plus a shared
                expert times sigmoid(W_sg h)
  output        the model's norm, then the output matrix `head`
"""
from __future__ import annotations
from dataclasses import dataclass, field
from typing import Any

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

MIXER_KINDS = ("retention", "parallel")
UNIT_EPS = 1e-6        # inside the root of the unit-vector norm of the delta rule's q and k: fixed by the design


def _need(m: dict, keys: tuple, where: str) -> None:
    missing = [k for k in keys if k not in m]
    if missing:
        raise ValueError(f"config.json: {where} lacks {missing}")


@dataclass(frozen=True)
class Rotation:
    base: float
    dims: int
    scaling: tuple | None = None        # (factor, low, high, original) or None

    @staticmethod
    def from_json(r: dict, dim: int, where: str) -> "Rotation":
        _need(r, ("base", "dims"), where + ".rot")
        sc = r.get("scaling")
        if sc is not None:
            _need(sc, ("factor", "low", "high", "original"), where + ".rot.scaling")
            sc = (float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"]))
            if sc[2] == sc[1]:
                raise ValueError(f"config.json: {where}.rot.scaling: low and high must differ")
        out = Rotation(float(r["base"]), int(r["dims"]), sc)
        if out.dims % 2 or not 0 <= out.dims <= dim:
            raise ValueError(f"config.json: {where}.rot.dims {out.dims} must be even and at most dim {dim}")
        return out

    def to_json(self) -> dict:
        out: dict[str, Any] = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            out["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return out

    def name(self) -> str:
        return f"rot{self.dims}@{self.base!r}" + (f"~{self.scaling!r}" if self.scaling else "")

    def spec(self) -> PartSpec:
        p: dict[str, Any] = {"head_dim": self.dims, "theta": self.base, "precise": True}
        if self.scaling is not None:
            f, lo, hi, orig = self.scaling
            p.update(kind="llama3", factor=f, low_freq_factor=lo, high_freq_factor=hi, original_max_position_embeddings=orig)
        return PartSpec("rope", p)


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: Rotation

    @staticmethod
    def from_json(m: dict, where: str) -> "RetentionConfig":
        _need(m, ("heads", "dim", "vdim", "decay", "rot"), where)
        out = RetentionConfig(int(m["heads"]), int(m["dim"]), int(m["vdim"]), tuple(float(x) for x in m["decay"]),
                              Rotation.from_json(m["rot"], int(m["dim"]), where))
        if min(out.heads, out.dim, out.vdim) <= 0:
            raise ValueError(f"config.json: {where}: heads, dim and vdim must be positive")
        if len(out.decay) != out.heads:
            raise ValueError(f"config.json: {where}.decay lists {len(out.decay)} values for {out.heads} heads")
        return out

    def to_json(self) -> dict:
        return {"decay": list(self.decay), "dim": self.dim, "heads": self.heads, "rot": self.rot.to_json(), "vdim": self.vdim}


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int
    rot: Rotation

    @staticmethod
    def from_json(m: dict, where: str) -> "SinkAttentionConfig":
        _need(m, ("heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"), where)
        _need(m["mask"], ("size",), where + ".mask")
        out = SinkAttentionConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), float(m["scale"]),
                                  int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0)),
                                  Rotation.from_json(m["rot"], int(m["dim"]), where))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) <= 0 or out.heads % out.kv_heads:
            raise ValueError(f"config.json: {where}: heads must be a positive multiple of kv_heads, dim and vdim positive")
        if out.window <= 0 or out.keep_first < 0:
            raise ValueError(f"config.json: {where}.mask: size must be positive and keep_first not negative")
        return out

    def to_json(self) -> dict:
        return {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads,
                "mask": {"keep_first": self.keep_first, "size": self.window}, "rot": self.rot.to_json(),
                "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @staticmethod
    def from_json(m: dict, where: str) -> "GatedDeltaConfig":
        _need(m, ("heads", "kv_heads", "dim", "vdim", "conv"), where)
        out = GatedDeltaConfig(int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"]), int(m["conv"]))
        if min(out.heads, out.kv_heads, out.dim, out.vdim) <= 0 or out.heads % out.kv_heads:
            raise ValueError(f"config.json: {where}: heads must be a positive multiple of kv_heads, dim and vdim positive")
        if out.conv < 1:
            raise ValueError(f"config.json: {where}.conv must be at least 1 tap")
        return out

    def to_json(self) -> dict:
        return {"conv": self.conv, "dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "vdim": self.vdim}


@dataclass(frozen=True)
class ParallelConfig:
    left: SinkAttentionConfig
    right: GatedDeltaConfig
    left_scale: float
    right_scale: float

    @staticmethod
    def from_json(m: dict, where: str) -> "ParallelConfig":
        _need(m, ("left", "right", "left_scale", "right_scale"), where)
        return ParallelConfig(SinkAttentionConfig.from_json(m["left"], where + ".left"),
                              GatedDeltaConfig.from_json(m["right"], where + ".right"),
                              float(m["left_scale"]), float(m["right_scale"]))

    def to_json(self) -> dict:
        return {"left": self.left.to_json(), "left_scale": self.left_scale, "right": self.right.to_json(),
                "right_scale": self.right_scale}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                     # "dense" or "moe"
    ff: int                       # dense: the intermediate size; moe: an expert's
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0            # 0: no shared expert

    @staticmethod
    def from_json(m: dict, where: str) -> "FeedForwardConfig":
        kind = m.get("kind")
        if kind == "dense":
            _need(m, ("ff",), where)
            out = FeedForwardConfig("dense", int(m["ff"]))
        elif kind == "moe":
            _need(m, ("router", "expert"), where)
            r = m["router"]
            _need(r, ("experts", "top"), where + ".router")
            g = r.get("groups") or {}
            shared = m.get("shared") or {}
            out = FeedForwardConfig("moe", int(m["expert"]["ff"]), int(r["experts"]), int(r["top"]),
                                    int(g.get("count", 1)), int(g.get("keep", g.get("count", 1))), int(shared.get("ff", 0)))
            if not 0 < out.top <= out.experts:
                raise ValueError(f"config.json: {where}.router: need 0 < top <= experts, got {out.top}, {out.experts}")
            if out.groups <= 0 or out.experts % out.groups or not 0 < out.keep <= out.groups:
                raise ValueError(f"config.json: {where}.router.groups: {out.experts} experts do not form {out.groups} "
                                 f"equal groups of which {out.keep} are kept")
            if out.top > out.keep * (out.experts // out.groups):
                raise ValueError(f"config.json: {where}.router: top {out.top} exceeds the experts of the {out.keep} kept groups")
        else:
            raise NotImplementedError(f"config.json: {where}.kind {kind!r} is not supported (have ['dense', 'moe'])")
        if out.ff <= 0:
            raise ValueError(f"config.json: {where}: ff must be positive")
        return out

    def to_json(self) -> dict:
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        out: dict[str, Any] = {"expert": {"ff": self.ff}, "kind": "moe",
                               "router": {"experts": self.experts, "groups": {"count": self.groups, "keep": self.keep},
                                          "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff}
        return out


@dataclass(frozen=True)
class GizulornLayer:
    type: str
    mixer: Any                     # RetentionConfig | ParallelConfig
    mlp: FeedForwardConfig | None


@dataclass(frozen=True)
class GizulornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: tuple
    max_position: int = 1 << 17      # positions are not bounded by the design; the engine sizes its tables itself

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError("config: vocab, width and the number of layers must be positive")
        if not self.norm_eps > 0:
            raise ValueError(f"config: norm.eps must be positive, got {self.norm_eps!r}")

    @staticmethod
    def from_json(c: dict) -> "GizulornConfig":
        _need(c, ("vocab", "width", "layers", "norm"), "the top level")
        layers = []
        for i, L in enumerate(c["layers"]):
            where = f"layers[{i}]"
            kind = L.get("type")
            if kind not in MIXER_KINDS:
                raise NotImplementedError(f"config.json: {where}.type {kind!r} is not supported (have {list(MIXER_KINDS)})")
            _need(L, ("mixer",), where)
            mixer = (RetentionConfig if kind == "retention" else ParallelConfig).from_json(L["mixer"], where + ".mixer")
            mlp = L.get("mlp")
            layers.append(GizulornLayer(kind, mixer, FeedForwardConfig.from_json(mlp, where + ".mlp") if mlp is not None else None))
        return GizulornConfig(int(c["vocab"]), int(c["width"]), float(c["norm"]["eps"]), tuple(layers),
                              int(c.get("max_position", 1 << 17)))

    def to_json(self) -> dict:
        return {"architecture": "Gizulorn",
                "layers": [{"mixer": L.mixer.to_json(), "mlp": L.mlp.to_json() if L.mlp else None, "type": L.type}
                           for L in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}

    def random_optional_groups(self, expected: dict) -> set:
        return {"lm_head"}

    # ---- the model description
    def _retention(self, m: RetentionConfig, positions: dict) -> PartSpec:
        positions.setdefault(m.rot.name(), m.rot.spec())
        return PartSpec("retention", {
            "hidden_size": self.width, "num_heads": m.heads, "key_dim": m.dim, "value_dim": m.vdim, "decay": m.decay,
            "key_scale": m.dim ** -0.5, "rotated": m.rot.dims, "pairing": "halves", "position": m.rot.name(),
            "eps": self.norm_eps, "gate": "silu", "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o"}})

    def _parallel(self, m: ParallelConfig, positions: dict) -> PartSpec:
        a, d = m.left, m.right
        positions.setdefault(a.rot.name(), a.rot.spec())
        left = PartSpec("sink_attention", {
            "hidden_size": self.width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "key_dim": a.dim,
            "value_dim": a.vdim, "scale": a.scale, "window": a.window, "keep_first": a.keep_first, "sink": True,
            "rotated": a.rot.dims, "pairing": "neighbours", "position": a.rot.name(),
            "names": {"q": "q", "k": "k", "v": "v", "sink": "sink", "out": "o"}})
        right = PartSpec("gated_delta", {
            "hidden_size": self.width, "num_heads": d.heads, "num_key_heads": d.kv_heads, "key_dim": d.dim,
            "value_dim": d.vdim, "taps": d.conv, "unit_eps": UNIT_EPS, "query_scale": d.dim ** -0.5, "eps": self.norm_eps,
            "names": {"q": "q", "k": "k", "v": "v", "conv": "conv", "beta": "b", "decay_log": "A_log", "decay_in": "a1",
                      "decay_out": "a2", "decay_bias": "dt_bias", "gate_in": "g1", "gate_out": "g2", "norm": "norm",
                      "out": "o"}})
        return PartSpec("parallel_mixers", {"hidden_size": self.width,
                                            "mixers": (("left", left, m.left_scale), ("right", right, m.right_scale))})

    def _ffn(self, f: FeedForwardConfig) -> PartSpec:
        if f.kind == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": f.ff,
                                       "names": ("gate", "up", "down"), "suffix": ""})
        return PartSpec("routed_moe", {
            "hidden_size": self.width, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top,
            "groups": f.groups, "keep_groups": f.keep, "shared_size": f.shared_ff, "renormalize": False,
            "names": {"router": "router", "expert": "e{}", "gate": "gate", "up": "up", "down": "down",
                      "shared": "shared", "shared_gate": "sg"}})

    def spec(self) -> ModelSpec:
        D = self.width
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": D, "eps": self.norm_eps, "name": name})
        positions: dict[str, PartSpec] = {}
        layers, schedule = [], []
        for i, L in enumerate(self.layers):
            mixer = self._retention(L.mixer, positions) if L.type == "retention" else self._parallel(L.mixer, positions)
            block = PartSpec("pre_norm", {"names": ("norm1", "mix", "norm2", "mlp"), "norms": (norm(""), norm(""))})
            layers.append(LayerSpec(f"l{i}.", block, mixer, self._ffn(L.mlp) if L.mlp is not None else None))
            schedule.append(ScheduleEntry(i, i))
        return ModelSpec(
            architecture="Gizulorn", hidden_size=D, vocab_size=self.vocab, embed_name="embed", lm_head_name="head",
            tie_embeddings=False, final_norm=norm("norm"), final_norm_name="final.norm", layers=tuple(layers),
            schedule=tuple(schedule), positions=positions, max_position=self.max_position)
