"""Typed configuration of the Pepilix decoder, read from its own config.json keys, and its model description.

config.json: `architecture` "Pepilix"; `vocab`, `width`; `embedding.scale`; `logit_scale`; `norm.eps`, `norm.groups`;
`canon.taps`; `layers`: a list whose entries give `type` (the mixer kind), `mixer` (its sizes) and `mlp` (the
feed-forward, or null). Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1`, `l<i>.norm2`, `l<i>.canon1`,
`l<i>.rg1`, `l<i>.rg1.b`, `l<i>.rg2`, `l<i>.rg2.b`, `l<i>.mix.*`, `l<i>.mlp.*`.

What the design is made of (every piece is a part of this package that another design can name with other constants):

  layer        x <- x + g1 * mixer(h1 + conv(h1)) + g2 * ff(h2),  h1 = norm1(x), h2 = norm2(x), g = sigmoid(W_g h + b_g)
               (block `parallel_gated`; the convolution is causal over time, per channel, `taps` wide, and the last
               taps - 1 inputs of every layer belong to a request's state)
  norm         RMS norm in `groups` consecutive parts of the vector, each with its own mean square (`rmsnorm`, groups)
  mixer        `latent_attention`: keys and values are read from one cached latent vector per token plus one rotated key
               part shared by the heads; a layer with `kv_from: j` has no latent projection and reads layer j's cache
  feed-forward `table_moe`: `experts` small gated feed-forwards, `top` of them per token chosen by a table indexed with
               the token id, each with weight 1 / top; activation g * sigmoid(1.702 g) * (u + 1) on clamped g, u
  output       the model's norm, the embedding table as output matrix, logits times `logit_scale`
"""
from __future__ import annotations
from dataclasses import dataclass
from typing import Any

from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

GLU_ALPHA = 1.702      # the slope inside the expert activation's sigmoid: fixed by the design
MIXER_KINDS = ("latent_attention",)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int            # unrotated query / key dimensions per head
    rot_dim: int        # rotated query / key dimensions per head (the key part is shared by all heads)
    vdim: int           # value size per head
    kv_rank: int        # size of the cached latent
    scale: float
    rot_base: float
    rot_dims: int       # how many of the rot_dim dimensions are rotated (the rest pass unchanged)
    kv_from: int | None = None

    @staticmethod
    def from_json(m: dict, where: str) -> "LatentMixerConfig":
        missing = [k for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot") if k not in m]
        if missing:
            raise ValueError(f"config.json: {where}.mixer lacks {missing}")
        rot = m["rot"]
        out = LatentMixerConfig(int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"]),
                                float(m["scale"]), float(rot["base"]), int(rot.get("dims", m["rot_dim"])),
                                None if m.get("kv_from") is None else int(m["kv_from"]))
        for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
            if getattr(out, k) <= 0:
                raise ValueError(f"config.json: {where}.mixer.{k} must be positive")
        if out.rot_dims % 2 or not 0 < out.rot_dims <= out.rot_dim:
            raise ValueError(f"config.json: {where}.mixer.rot.dims {out.rot_dims} must be even and at most rot_dim {out.rot_dim}")
        return out

    def to_json(self) -> dict:
        out: dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank,
                               "rot": {"base": self.rot_base, "dims": self.rot_dims}, "rot_dim": self.rot_dim,
                               "scale": self.scale, "vdim": self.vdim}
        if self.kv_from is not None:
            out["kv_from"] = self.kv_from
        return out


@dataclass(frozen=True)
class TableMoeConfig:
    experts: int
    top: int
    ff: int
    limit: float

    @staticmethod
    def from_json(m: dict, where: str) -> "TableMoeConfig":
        if m.get("kind", "moe") != "moe":
            raise NotImplementedError(f"config.json: {where}.mlp.kind {m.get('kind')!r} is not supported (have ['moe'])")
        try:
            out = TableMoeConfig(int(m["router"]["experts"]), int(m["router"]["top"]), int(m["expert"]["ff"]),
                                 float(m["expert"]["limit"]))
        except KeyError as e:
            raise ValueError(f"config.json: {where}.mlp lacks {e.args[0]!r}") from None
        if not 0 < out.top <= out.experts or out.ff <= 0 or not out.limit > 0:
            raise ValueError(f"config.json: {where}.mlp: need 0 < top <= experts, ff > 0, limit > 0, got {out}")
        return out

    def to_json(self) -> dict:
        return {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
                "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class PepilixLayer:
    type: str
    mixer: LatentMixerConfig
    mlp: TableMoeConfig | None


@dataclass(frozen=True)
class PepilixConfig:
    vocab: int
    width: int
    embedding_scale: float
    logit_scale: float
    norm_eps: float
    norm_groups: int
    canon_taps: int
    layers: tuple[PepilixLayer, ...]
    max_position: int = 1 << 17      # positions are not bounded by the design; the engine sizes its tables itself

    def __post_init__(self) -> None:
        if self.vocab <= 0 or self.width <= 0 or not self.layers:
            raise ValueError(f"config: vocab, width and the number of layers must be positive")
        if self.norm_groups <= 0 or self.width % self.norm_groups:
            raise ValueError(f"config: width {self.width} does not split into {self.norm_groups} equal norm groups")
        if self.canon_taps < 0:
            raise ValueError(f"config: canon.taps cannot be negative, got {self.canon_taps}")
        if not self.norm_eps > 0:
            raise ValueError(f"config: norm.eps must be positive, got {self.norm_eps!r}")
        for i, L in enumerate(self.layers):
            j = L.mixer.kv_from
            if j is None:
                continue
            if not 0 <= j < i or self.layers[j].mixer.kv_from is not None:
                raise ValueError(f"config: layer {i} reads the cache of layer {j}, which must be an earlier layer that "
                                 f"writes a cache of its own")
            own, src = L.mixer, self.layers[j].mixer
            if (own.kv_rank, own.rot_dim, own.rot_dims, own.rot_base) != (src.kv_rank, src.rot_dim, src.rot_dims, src.rot_base):
                raise ValueError(f"config: layer {i} reads the cache of layer {j} but their kv_rank, rot_dim or rotation differ")

    @staticmethod
    def from_json(c: dict) -> "PepilixConfig":
        missing = [k for k in ("vocab", "width", "layers", "norm") if k not in c]
        if missing:
            raise ValueError(f"config.json lacks {missing}")
        layers = []
        for i, L in enumerate(c["layers"]):
            kind = L.get("type", "latent_attention")
            if kind not in MIXER_KINDS:
                raise NotImplementedError(f"config.json: layers[{i}].type {kind!r} is not supported (have {list(MIXER_KINDS)})")
            mlp = L.get("mlp")
            layers.append(PepilixLayer(kind, LatentMixerConfig.from_json(L["mixer"], f"layers[{i}]"),
                                       TableMoeConfig.from_json(mlp, f"layers[{i}]") if mlp is not None else None))
        return PepilixConfig(
            vocab=int(c["vocab"]), width=int(c["width"]),
            embedding_scale=float((c.get("embedding") or {}).get("scale", 1.0)), logit_scale=float(c.get("logit_scale", 1.0)),
            norm_eps=float(c["norm"]["eps"]), norm_groups=int(c["norm"].get("groups", 1)),
            canon_taps=int((c.get("canon") or {}).get("taps", 0)),      # no `canon`: no convolution
            layers=tuple(layers),
            max_position=int(c.get("max_position", 1 << 17)))

    def to_json(self) -> dict:
        return {"architecture": "Pepilix", **({"canon": {"taps": self.canon_taps}} if self.canon_taps else {}), "embedding": {"scale": self.embedding_scale},
                "layers": [{"mixer": L.mixer.to_json(), "mlp": L.mlp.to_json() if L.mlp else None, "type": L.type}
                           for L in self.layers],
                "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps, "groups": self.norm_groups},
                "vocab": self.vocab, "width": self.width}

    def random_optional_groups(self, expected: dict) -> set[str]:
        return set()

    def spec(self) -> ModelSpec:
        D = self.width
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"size": D, "eps": self.norm_eps, "groups": self.norm_groups, "name": name})
        positions: dict[str, PartSpec] = {}
        layers, schedule = [], []
        for i, L in enumerate(self.layers):
            m = L.mixer
            # one table of angles per distinct rotation; computed in 64-bit and rounded once
            pname = f"rot{m.rot_dims}@{m.rot_base!r}"
            positions.setdefault(pname, PartSpec("rope", {"head_dim": m.rot_dims, "theta": m.rot_base, "precise": True}))
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "num_heads": m.heads, "nope_dim": m.dim, "rope_dim": m.rot_dim, "value_dim": m.vdim,
                "latent_dim": m.kv_rank, "scale": m.scale, "rotated": m.rot_dims, "eps": self.norm_eps,
                "position": pname, "own_latent": m.kv_from is None,
                "names": {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "out": "o"}})
            ffn = None
            if L.mlp is not None:
                ffn = PartSpec("table_moe", {
                    "hidden_size": D, "intermediate_size": L.mlp.ff, "num_experts": L.mlp.experts, "top": L.mlp.top,
                    "vocab_size": self.vocab, "limit": L.mlp.limit, "alpha": GLU_ALPHA,
                    "names": {"table": "table", "expert": "e{}", "gate": "gate", "up": "up", "down": "down"}})
            block = PartSpec("parallel_gated", {
                "hidden_size": D, "taps": self.canon_taps, "gated": True, "norms": (norm(""), norm("")),
                "names": {"norm1": "norm1", "norm2": "norm2", "mixer": "mix", "ffn": "mlp", "conv": "canon1",
                          "gate1": "rg1", "gate2": "rg2", "bias": "b"}})
            layers.append(LayerSpec(f"l{i}.", block, mixer, ffn))
            schedule.append(ScheduleEntry(i, i) if m.kv_from is None else ScheduleEntry(i, m.kv_from, write_cache=False))
        return ModelSpec(
            architecture="Pepilix", hidden_size=D, vocab_size=self.vocab, embed_name="embed", lm_head_name=None,
            tie_embeddings=True, final_norm=norm("norm"), final_norm_name="final.norm", layers=tuple(layers),
            schedule=tuple(schedule), positions=positions, max_position=self.max_position,
            embed_scale=self.embedding_scale if self.embedding_scale != 1.0 else None,
            logit_transform=PartSpec("scale", {"factor": self.logit_scale}) if self.logit_scale != 1.0 else None)
