"""Configuration objects mirroring the reference's config surface.

`OmChatQwen2Config` keeps the attribute names the reference reads with getattr on the hot path (omchat_arch.py:25-28,
100,161,176; internVIT_encoder.py:16-17) and adds three knobs whose defaults reproduce reference behaviour:
`mm_pixel_shuffle_ratio` (1.0 = none), `kv_page_size`, `tp_size`.
"""
from __future__ import annotations

from dataclasses import dataclass, field, asdict
from typing import List, Optional

IMAGE_TOKEN_INDEX = -200  # omchat/constants.py:8
IGNORE_INDEX = -100


@dataclass
class InternVisionConfig:
    """intern_vit_6b/configuration_intern_vit.py:63-83 defaults (InternViT-6B-448px-V1-5)."""
    num_channels: int = 3
    patch_size: int = 14
    image_size: int = 448
    qkv_bias: bool = False
    hidden_size: int = 3200
    num_attention_heads: int = 25
    intermediate_size: int = 12800
    qk_normalization: bool = True
    num_hidden_layers: int = 45
    hidden_act: str = "gelu"
    layer_norm_eps: float = 1e-6
    initializer_factor: float = 0.1
    norm_type: str = "rms_norm"  # 'layer_norm' for the InternViT-300M variant (intern_vit_300m/modeling_intern_vit.py:61-64)

    def __post_init__(self):
        if self.norm_type not in ("rms_norm", "layer_norm"):
            raise ValueError(f"unknown norm_type {self.norm_type!r}")

    @classmethod
    def intern_vit_300m(cls, **overrides) -> "InternVisionConfig":
        """intern_vit_300m/configuration_intern_vit.py:60-80 defaults: the lighter tower (LayerNorm, no QK-norm, 16 heads of 64)."""
        kw = dict(hidden_size=1024, num_attention_heads=16, intermediate_size=4096, qk_normalization=False, num_hidden_layers=24,
                  norm_type="layer_norm", initializer_factor=1.0)
        kw.update(overrides)
        return cls(**kw)

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads


@dataclass
class OmChatQwen2Config:
    """omchat_qwen2.py:16-19 (Qwen2Config fields + the mm_* attributes); defaults = Qwen2-7B + InternViT-6B."""
    model_type: str = "omchat_qwen2"
    vocab_size: int = 152064
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    max_position_embeddings: int = 32768
    # multimodal attributes read by the reference
    mm_vision_tower: Optional[str] = "InternViT-6B-448px-V1-5"
    mm_projector_type: str = "mlp2x_gelu"
    mm_hidden_size: int = 3200
    mm_vision_select_layer: int = -1
    mm_vision_select_feature: str = "patch"
    delay_load: bool = False
    image_grid_pinpoints: List[List[int]] = field(default_factory=lambda: [
        [448, 896], [896, 448], [896, 896], [1344, 448], [448, 1344], [1344, 1344]])
    tokenizer_model_max_length: Optional[int] = None
    tokenizer_padding_side: str = "right"
    tune_mm_mlp_adapter: bool = False
    mm_use_im_start_end: bool = False
    eos_token_id: int = 151645
    pad_token_id: int = 151643
    # build-specific knobs (defaults reproduce the reference)
    mm_pixel_shuffle_ratio: float = 1.0
    kv_page_size: int = 64
    tp_size: int = 1
    vision_config: InternVisionConfig = field(default_factory=InternVisionConfig)

    def __post_init__(self):
        # build_vision_tower (multimodal_encoder/builder.py:11-14) picks the tower class from the NAME: a config that names the
        # 300M tower and leaves vision_config at the 6B defaults gets the 300M defaults
        name = (self.mm_vision_tower or "").lower()
        if "internvit-300m" in name and self.vision_config == InternVisionConfig():
            self.vision_config = InternVisionConfig.intern_vit_300m()
            if self.mm_hidden_size == 3200:
                self.mm_hidden_size = self.vision_config.hidden_size

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def pixel_shuffle_down(self) -> int:
        d = round(1.0 / self.mm_pixel_shuffle_ratio)
        if d < 1 or abs(1.0 / d - self.mm_pixel_shuffle_ratio) > 1e-6:
            raise ValueError(f"mm_pixel_shuffle_ratio must be 1/k, got {self.mm_pixel_shuffle_ratio}")
        return d

    @property
    def image_tokens_per_crop(self) -> int:
        g = self.vision_config.image_size // self.vision_config.patch_size
        return (g // self.pixel_shuffle_down) ** 2

    def to_dict(self):
        return asdict(self)


@dataclass
class OmChatQwen2MoeConfig(OmChatQwen2Config):
    """omchat_qwen2_moe.py:14-17: transformers Qwen2MoeConfig fields + the mm_* attributes. Defaults = Qwen1.5-MoE-A2.7B's
    language model (Qwen2MoeConfig defaults) under the same vision tower."""
    model_type: str = "omchat_qwen2_moe"
    hidden_size: int = 2048
    intermediate_size: int = 5632
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    num_experts: int = 60
    num_experts_per_tok: int = 4
    moe_intermediate_size: int = 1408
    shared_expert_intermediate_size: int = 5632
    norm_topk_prob: bool = False
    decoder_sparse_step: int = 1
    mlp_only_layers: List[int] = field(default_factory=list)

    def layer_is_sparse(self, li: int) -> bool:
        """Qwen2MoeDecoderLayer.__init__ (transformers modeling_qwen2_moe.py:381-386)."""
        return li not in self.mlp_only_layers and self.num_experts > 0 and (li + 1) % self.decoder_sparse_step == 0


# ---------------------------------------------------------------------------------------------------------------------------
# Voduzen: a decoder-only language model described by a per-layer list (config.json: architecture "Voduzen").


@dataclass
class RotarySpec:
    """Pairwise-interleaved rotary embedding on the first `dims` dimensions of a vector: pair i = (2i, 2i + 1) turns by
    position * f_i, f_i = base^(-2i/dims). `scaling` (factor, original, fast, slow) blends f_i towards f_i / factor over a
    linear ramp in i and multiplies cos and sin by 0.1 ln(factor) + 1 (the constants 0.1 and 0.001 are fixed by the design)."""
    dims: int
    base: float
    scaling: Optional[dict] = None

    def frequencies(self):
        """(f [dims / 2] as Python floats, multiplier of cos / sin) in double precision."""
        import math
        half = self.dims // 2
        f = [self.base ** (-2.0 * i / self.dims) for i in range(half)]
        mult = 1.0
        sc = self.scaling
        if sc:
            factor, orig = float(sc["factor"]), float(sc["original"])

            def turn_dim(turns: float) -> float:
                return self.dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(self.base))
            lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
            hi = min(math.ceil(turn_dim(float(sc["slow"]))), self.dims - 1)
            span = max(hi - lo, 0.001)
            for i in range(half):
                ramp = min(max((i - lo) / span, 0.0), 1.0)
                f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
            mult = 0.1 * math.log(factor) + 1.0
        return f, mult


@dataclass
class LatentAttentionSpec:
    """Attention whose keys and values are up-projections of a cached latent of width kv_rank plus one rotated key part of
    width rot_dim shared by the heads. q_rank: queries go through a normed latent of that width (None: one projection).
    sink: the softmax denominator has one more learned term per head."""
    heads: int
    dim: int        # unrotated query / key dimensions per head
    rot_dim: int    # rotated query / key dimensions per head
    vdim: int
    kv_rank: int
    scale: float
    rot: RotarySpec = None
    q_rank: Optional[int] = None
    sink: bool = False


@dataclass
class RouterMoeSpec:
    """Mixture of experts: `experts` feed-forward experts (relu^2, no biases) of width expert_ff followed by `identity`
    identity outputs of the router; every token uses `top` of them; shared_ff: width of the always-on expert (None: none)."""
    experts: int
    identity: int
    top: int
    expert_ff: int
    shared_ff: Optional[int] = None


@dataclass
class VoduzenLayerSpec:
    type: str
    mixer: LatentAttentionSpec
    mlp: Optional[RouterMoeSpec]


@dataclass
class VoduzenConfig:
    model_type: str = "voduzen"
    vocab_size: int = 0
    hidden_size: int = 0
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    norm_eps: float = 1e-6
    layers: List[VoduzenLayerSpec] = field(default_factory=list)
    kv_page_size: int = 64       # engine knob: tokens per cache page
    eos_token_id: int = -1
    pad_token_id: int = 0

    MIXERS = ("latent_attention", "latent_attention_2")

    @classmethod
    def from_dict(cls, d: dict) -> "VoduzenConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            typ = ld["type"]
            if typ not in cls.MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {typ!r}")
            m = ld["mixer"]
            rot = m.get("rot") or {}
            rspec = RotarySpec(dims=int(rot.get("dims", m.get("rot_dim", 0))), base=float(rot.get("base", 10000.0)),
                               scaling=dict(rot["scaling"]) if rot.get("scaling") else None)
            if rspec.dims > int(m["rot_dim"]) or rspec.dims % 2:
                raise ValueError(f"layer {i}: rot.dims must be even and at most rot_dim")
            # the first kind projects queries directly and has a sink; the second sends queries through a latent, plain softmax
            mix = LatentAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), rot_dim=int(m["rot_dim"]), vdim=int(m["vdim"]),
                                      kv_rank=int(m["kv_rank"]), scale=float(m["scale"]), rot=rspec,
                                      q_rank=int(m["q_rank"]) if typ == "latent_attention_2" else None,
                                      sink=typ == "latent_attention")
            mlp = None
            md = ld.get("mlp")
            if md:
                if md.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {md.get('kind')!r}")
                r = md["router"]
                sh = md.get("shared")
                mlp = RouterMoeSpec(experts=int(r["experts"]), identity=int(r.get("identity", 0)), top=int(r["top"]),
                                    expert_ff=int(md["expert"]["ff"]), shared_ff=int(sh["ff"]) if sh else None)
            layers.append(VoduzenLayerSpec(type=typ, mixer=mix, mlp=mlp))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   logit_scale=float(d.get("logit_scale", 1.0)), norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)),
                   layers=layers, kv_page_size=int(d.get("kv_page_size", 64)), eos_token_id=int(d.get("eos_token_id", -1)),
                   pad_token_id=int(d.get("pad_token_id", 0)))

    def to_dict(self) -> dict:
        """The config.json form (round-trips through from_dict)."""
        out_layers = []
        for l in self.layers:
            m = l.mixer
            rot = {"base": m.rot.base, "dims": m.rot.dims}
            if m.rot.scaling:
                rot["scaling"] = dict(m.rot.scaling)
            md = {"dim": m.dim, "heads": m.heads, "kv_rank": m.kv_rank, "rot": rot, "rot_dim": m.rot_dim, "scale": m.scale,
                  "vdim": m.vdim}
            if m.q_rank is not None:
                md["q_rank"] = m.q_rank
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.expert_ff},
                       "router": {"experts": l.mlp.experts, "identity": l.mlp.identity, "top": l.mlp.top},
                       "shared": {"ff": l.mlp.shared_ff} if l.mlp.shared_ff else None}
            out_layers.append({"type": l.type, "mixer": md, "mlp": mlp})
        return {"architecture": "Voduzen", "vocab": self.vocab_size, "width": self.hidden_size,
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
                "layers": out_layers, "kv_page_size": self.kv_page_size, "eos_token_id": self.eos_token_id,
                "pad_token_id": self.pad_token_id}


# --------------------------------------------------------------------------------------------------------------------- Tifisun
@dataclass
class DeltaRuleSpec:
    """Gated delta rule: a [dim, vdim] fp32 state per head, decayed, corrected towards the new value along the key, read by the
    query. kv_heads query / key heads serve heads value heads. conv: taps of the causal per-channel convolution in front of
    q, k, v. channel_decay: one decay per key channel (projected through `decay_rank` columns) instead of one per head;
    gate_rank: the output gate is projected through that many columns and squashed by a sigmoid (None: one projection, silu)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    channel_decay: bool = False
    decay_rank: Optional[int] = None
    gate_rank: Optional[int] = None


@dataclass
class WindowAttentionSpec:
    """Softmax attention over a sliding window of `window` keys (the row's own included), grouped heads, no rotation. Queries and
    keys are RMS-normed over their whole projection; scores are scaled, soft-capped (softcap * tanh(s / softcap); 0 = off) and
    get a learned bias by distance: `bias_rows` table rows, the first half one per distance, the rest logarithmic up to bias_max."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    softcap: float = 0.0
    bias_max: float = 0.0

    @staticmethod
    def bucket(n: int, rows: int, far: float) -> int:
        import math
        half = rows // 2
        if n < half:
            return n
        if half < 1 or far <= half:      # no logarithmic range to spread over: everything further shares the last row
            return rows - 1
        return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


@dataclass
class DecayAttentionSpec:
    """Linear attention with one constant decay per head: S <- decay_h S + k v^T, o = S^T q, silu on q, k, v."""
    heads: int
    dim: int
    vdim: int
    decay: List[float] = field(default_factory=list)


@dataclass
class ParallelMixerSpec:
    left: WindowAttentionSpec
    right: DecayAttentionSpec


@dataclass
class DenseMlpSpec:
    """act(W_gate x + b) * (W_up x + b) -> W_down + b, act = tanh-form gelu."""
    ff: int


@dataclass
class TifisunLayerSpec:
    type: str                      # 'delta' | 'channel_delta' | 'parallel'
    mixer: object                  # DeltaRuleSpec | ParallelMixerSpec
    mlp: Optional[DenseMlpSpec]
    weights_of: Optional[int] = None   # the layer whose tensors this one uses (its cache and state are its own)



@dataclass
class TifisunConfig:
    model_type: str = "tifisun"
    vocab_size: int = 0
    hidden_size: int = 0
    embedding_scale: float = 1.0
    residual_mult: float = 1.0
    norm_eps: float = 1e-6
    layers: List[TifisunLayerSpec] = field(default_factory=list)
    kv_page_size: int = 64       # engine knob: tokens per cache page
    eos_token_id: int = -1
    pad_token_id: int = 0

    MIXERS = ("delta", "channel_delta", "parallel")

    @classmethod
    def from_dict(cls, d: dict) -> "TifisunConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            typ, m = ld["type"], ld["mixer"]
            if typ not in cls.MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {typ!r}")
            if typ == "parallel":
                l, r = m["left"], m["right"]
                left = WindowAttentionSpec(heads=int(l["heads"]), kv_heads=int(l.get("kv_heads", l["heads"])), dim=int(l["dim"]),
                                           vdim=int(l["vdim"]), scale=float(l["scale"]), window=int(l["mask"]["size"]),
                                           softcap=float(l.get("softcap") or 0.0), bias_max=float(l.get("bias_max") or 0.0))
                right = DecayAttentionSpec(heads=int(r["heads"]), dim=int(r["dim"]), vdim=int(r["vdim"]),
                                           decay=[float(x) for x in r["decay"]])
                if left.heads % left.kv_heads or len(right.decay) != right.heads or left.window < 1:
                    raise ValueError(f"layer {i}: inconsistent mixer sizes")
                mix = ParallelMixerSpec(left, right)
            else:
                mix = DeltaRuleSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads", m["heads"])), dim=int(m["dim"]),
                                    vdim=int(m["vdim"]), conv=int(m["conv"]), channel_decay=typ == "channel_delta",
                                    decay_rank=int(m["decay_rank"]) if m.get("decay_rank") else None,
                                    gate_rank=int(m["gate_rank"]) if m.get("gate_rank") else None)
                if mix.heads % mix.kv_heads or mix.conv < 1:
                    raise ValueError(f"layer {i}: inconsistent mixer sizes")
            md = ld.get("mlp")
            if md and md.get("kind", "dense") != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {md.get('kind')!r}")
            wo = ld.get("weights_of")
            if wo is not None and not (0 <= int(wo) < len(d["layers"]) and int(wo) != i and d["layers"][int(wo)]["type"] == typ):
                raise ValueError(f"layer {i}: weights_of must name another layer of the same type")
            layers.append(TifisunLayerSpec(type=typ, mixer=mix, mlp=DenseMlpSpec(ff=int(md["ff"])) if md else None,
                                           weights_of=int(wo) if wo is not None else None))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   residual_mult=float(d.get("residual_mult", 1.0)), norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)),
                   layers=layers, kv_page_size=int(d.get("kv_page_size", 64)), eos_token_id=int(d.get("eos_token_id", -1)),
                   pad_token_id=int(d.get("pad_token_id", 0)))

    def to_dict(self) -> dict:
        """The config.json form (round-trips through from_dict)."""
        out = []
        for l in self.layers:
            if l.type == "parallel":
                a, b = l.mixer.left, l.mixer.right
                md = {"left": {"bias_max": a.bias_max, "dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads,
                               "mask": {"size": a.window}, "scale": a.scale, "softcap": a.softcap, "vdim": a.vdim},
                      "right": {"decay": list(b.decay), "dim": b.dim, "heads": b.heads, "vdim": b.vdim}}
            else:
                m = l.mixer
                md = {"conv": m.conv, "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads, "vdim": m.vdim}
            e = {"type": l.type, "mixer": md, "mlp": {"ff": l.mlp.ff, "kind": "dense"} if l.mlp else None}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            out.append(e)
        return {"architecture": "Tifisun", "vocab": self.vocab_size, "width": self.hidden_size,
                "embedding": {"scale": self.embedding_scale}, "residual_mult": self.residual_mult, "norm": {"eps": self.norm_eps},
                "layers": out, "kv_page_size": self.kv_page_size, "eos_token_id": self.eos_token_id,
                "pad_token_id": self.pad_token_id}


# --------------------------------------------------------------------------------------------------------------------- Fofisun
@dataclass
class DiffAttentionSpec:
    """Differential softmax attention without rotation: every head has two score maps (queries and keys of their own, `dim` wide)
    over one set of values; o = a1 - lambda a2, RMS-normed over the head and scaled by 1 - diff, lambda = exp(lq1 . lk1) -
    exp(lq2 . lk2) + diff. conv: taps of the causal per-channel convolution behind the q, k, v projections (0: none). Queries and
    keys are RMS-normed per head and map. window: keys a row sees behind itself, itself included (None: all); keep_first: the
    first keys of the sequence stay visible behind the window. The concatenated heads pass a sigmoid gate."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    diff: float
    window: Optional[int] = None
    keep_first: int = 0
    conv: int = 0


@dataclass
class GeluMlpSpec:
    """W_down gelu(W_up x) with the erf form of gelu, no biases."""
    ff: int


@dataclass
class ClampedMoeSpec:
    """`experts` gated experts of width expert_ff, `top` per token chosen by the router's logits (weights: softmax over the chosen
    logits alone). An expert: g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit), W_down (g sigmoid(1.702 g) (u + 1)).
    shared_ff: width of an expert that every token passes, scaled by a sigmoid gate of the token (None: none)."""
    experts: int
    top: int
    expert_ff: int
    limit: float
    shared_ff: Optional[int] = None
    shared_limit: float = 0.0


@dataclass
class FofisunLayerSpec:
    type: str                      # 'attention'
    mixer: DiffAttentionSpec
    mlp: object                    # GeluMlpSpec | ClampedMoeSpec | None


@dataclass
class FofisunConfig:
    model_type: str = "fofisun"
    vocab_size: int = 0
    hidden_size: int = 0
    norm_eps: float = 1e-6
    layers: List[FofisunLayerSpec] = field(default_factory=list)
    loop_start: int = 0            # layers loop_start .. loop_stop - 1 run loop_times times in a row (the same tensors, a cache per run)
    loop_stop: int = 0
    loop_times: int = 1
    kv_page_size: int = 64         # engine knob: tokens per cache page
    eos_token_id: int = -1
    pad_token_id: int = 0

    MIXERS = ("attention",)
    POSITION_BASE = 10000.0        # sinusoidal position vectors: entry 2i / 2i + 1 = sin / cos(p * base^(-2i / width))
    SWISH_SLOPE = 1.702            # the experts' gate is g * sigmoid(SWISH_SLOPE * g)
    UP_SHIFT = 1.0                 # ... times (u + UP_SHIFT)

    def layer_runs(self) -> List[int]:
        """The layer index of every layer run, in execution order."""
        n = len(self.layers)
        if self.loop_stop <= self.loop_start:
            return list(range(n))
        return list(range(self.loop_start)) + list(range(self.loop_start, self.loop_stop)) * self.loop_times + list(range(self.loop_stop, n))

    @classmethod
    def from_dict(cls, d: dict) -> "FofisunConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            typ, m = ld["type"], ld["mixer"]
            if typ not in cls.MIXERS:
                raise ValueError(f"layer {i}: unknown mixer type {typ!r}")
            mask = m.get("mask") or {}
            mix = DiffAttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                    scale=float(m["scale"]), diff=float(m["diff"]),
                                    window=int(mask["size"]) if mask.get("size") is not None else None,
                                    keep_first=int(mask.get("keep_first") or 0), conv=int(m.get("conv") or 0))
            if mix.heads < 1 or mix.kv_heads < 1 or mix.heads % mix.kv_heads or mix.conv < 0 or mix.keep_first < 0 or \
                    (mix.window is not None and mix.window < 1):
                raise ValueError(f"layer {i}: inconsistent mixer sizes")
            md, mlp = ld.get("mlp"), None
            if md:
                kind = md.get("kind", "dense")
                if kind == "dense":
                    mlp = GeluMlpSpec(ff=int(md["ff"]))
                elif kind == "moe":
                    r, e, sh = md["router"], md["expert"], md.get("shared")
                    mlp = ClampedMoeSpec(experts=int(r["experts"]), top=int(r["top"]), expert_ff=int(e["ff"]), limit=float(e["limit"]),
                                         shared_ff=int(sh["ff"]) if sh else None, shared_limit=float(sh["limit"]) if sh else 0.0)
                    if not 1 <= mlp.top <= mlp.experts:
                        raise ValueError(f"layer {i}: top must be between 1 and the number of experts")
                else:
                    raise ValueError(f"layer {i}: unknown feed-forward kind {kind!r}")
            layers.append(FofisunLayerSpec(type=typ, mixer=mix, mlp=mlp))
        lp = d.get("loop") or {}
        start, stop, times = int(lp.get("start", 0)), int(lp.get("stop", 0)), int(lp.get("times", 1))
        if lp and not (0 <= start <= stop <= len(layers) and times >= 1):
            raise ValueError("loop: start <= stop within the layers and times >= 1 are required")
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)),
                   layers=layers, loop_start=start, loop_stop=stop, loop_times=times, kv_page_size=int(d.get("kv_page_size", 64)),
                   eos_token_id=int(d.get("eos_token_id", -1)), pad_token_id=int(d.get("pad_token_id", 0)))

    def to_dict(self) -> dict:
        """The config.json form (round-trips through from_dict)."""
        out = []
        for l in self.layers:
            m = l.mixer
            md = {"conv": m.conv, "diff": m.diff, "dim": m.dim, "heads": m.heads, "kv_heads": m.kv_heads,
                  "mask": {"keep_first": m.keep_first, "size": m.window}, "scale": m.scale, "vdim": m.vdim}
            if isinstance(l.mlp, GeluMlpSpec):
                mlp = {"ff": l.mlp.ff, "kind": "dense"}
            elif isinstance(l.mlp, ClampedMoeSpec):
                s = l.mlp
                mlp = {"expert": {"ff": s.expert_ff, "limit": s.limit}, "kind": "moe", "router": {"experts": s.experts, "top": s.top},
                       "shared": {"ff": s.shared_ff, "limit": s.shared_limit} if s.shared_ff else None}
            else:
                mlp = None
            out.append({"type": l.type, "mixer": md, "mlp": mlp})
        return {"architecture": "Fofisun", "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
                "layers": out, "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times},
                "kv_page_size": self.kv_page_size, "eos_token_id": self.eos_token_id, "pad_token_id": self.pad_token_id}


# --------------------------------------------------------------------------------------------------------------------- Vefunex
@dataclass
class SoftmaxAttentionSpec:
    """Causal softmax attention over all earlier keys with grouped heads. Which of the optional mechanisms a layer has:
    rot (RotarySpec or None): pairwise-interleaved rotation of the first rot.dims dimensions of queries and keys; q_temp_coef /
    q_temp_every: queries are multiplied by 1 + coef ln(floor((p + 1) / every) + 1) at position p (coef 0: off); value_norm: every
    head's value is divided by its root mean square before it is cached; softcap: scores become softcap tanh(score / softcap)
    (0: off); sink: one more learned term exp(sink_h) per head in the softmax denominator; gate: the concatenated heads are
    multiplied by a sigmoid of a projection of the mixer's input."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[RotarySpec] = None
    q_temp_coef: float = 0.0
    q_temp_every: int = 1
    value_norm: bool = False
    softcap: float = 0.0
    sink: bool = False
    gate: bool = False


@dataclass
class SelectiveScanSpec:
    """Selective state-space mixer: `inner` channels with `state` fp32 states each, a causal convolution of `conv` taps (with bias)
    and silu in front, step sizes through a projection of rank dt_rank; S <- exp(dt A) S + dt x B, y = S C + D x, gated by silu(z)."""
    inner: int
    state: int
    dt_rank: int
    conv: int


@dataclass
class AttentionScanMixerSpec:
    """Two mixers side by side on the same input: left_scale * attention + right_scale * selective scan."""
    left: SoftmaxAttentionSpec
    right: SelectiveScanSpec
    left_scale: float = 1.0
    right_scale: float = 1.0


@dataclass
class GatedLinearAttentionSpec:
    """Gated linear attention: per head S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t with one decay per key channel,
    alpha = sigmoid(low-rank projection + bias)^(1 / tau); queries scaled by dim^-1/2; the read-out is RMS-normed per head and gated
    by silu of a projection."""
    heads: int
    dim: int
    vdim: int
    tau: float


@dataclass
class SigmoidMoeSpec:
    """`experts` gated experts (silu, no biases) of width expert_ff; every token uses the `top` experts with the largest sigmoid
    router scores; the scores are used as they are and multiply the experts' INPUT."""
    experts: int
    top: int
    expert_ff: int


@dataclass
class VefunexLayerSpec:
    type: str                      # 'attention' | 'parallel' | 'gla'
    mixer: object                  # SoftmaxAttentionSpec | AttentionScanMixerSpec | GatedLinearAttentionSpec
    mlp: Optional[SigmoidMoeSpec]


@dataclass
class VefunexConfig:
    model_type: str = "vefunex"
    vocab_size: int = 0
    hidden_size: int = 0
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    logit_softcap: float = 0.0     # logits become cap * tanh(logits / cap) (0: off)
    canon_taps: int = 1            # taps of the convolution every sublayer's input passes (h + conv(h))
    layers: List[VefunexLayerSpec] = field(default_factory=list)
    kv_page_size: int = 64         # engine knob: tokens per cache page
    eos_token_id: int = -1
    pad_token_id: int = 0

    MIXERS = ("attention", "parallel", "gla")

    @staticmethod
    def _attention(m: dict, i: int, *, value_norm: bool, sink: bool, gate: bool) -> SoftmaxAttentionSpec:
        rot, qt = m.get("rot"), m.get("q_temp")
        spec = SoftmaxAttentionSpec(heads=int(m["heads"]), kv_heads=int(m.get("kv_heads") or m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                    scale=float(m["scale"]), rot=RotarySpec(dims=int(rot["dims"]), base=float(rot["base"])) if rot else None,
                                    q_temp_coef=float(qt["coef"]) if qt else 0.0, q_temp_every=int(qt["every"]) if qt else 1,
                                    value_norm=value_norm, softcap=float(m.get("softcap") or 0.0), sink=sink, gate=gate)
        if spec.heads < 1 or spec.kv_heads < 1 or spec.heads % spec.kv_heads or spec.q_temp_every < 1 or \
                (spec.rot is not None and (spec.rot.dims % 2 or not 0 <= spec.rot.dims <= spec.dim)):
            raise ValueError(f"layer {i}: inconsistent attention sizes")
        return spec

    @classmethod
    def from_dict(cls, d: dict) -> "VefunexConfig":
        layers = []
        for i, ld in enumerate(d["layers"]):
            typ, m = ld["type"], ld["mixer"]
            if typ == "attention":
                mix = cls._attention(m, i, value_norm=True, sink=False, gate=False)
            elif typ == "parallel":
                r = m["right"]
                right = SelectiveScanSpec(inner=int(r["inner"]), state=int(r["state"]), dt_rank=int(r["dt_rank"]), conv=int(r["conv"]))
                if min(right.inner, right.state, right.dt_rank, right.conv) < 1:
                    raise ValueError(f"layer {i}: inconsistent selective-scan sizes")
                mix = AttentionScanMixerSpec(left=cls._attention(m["left"], i, value_norm=False, sink=True, gate=True), right=right,
                                             left_scale=float(m.get("left_scale", 1.0)), right_scale=float(m.get("right_scale", 1.0)))
            elif typ == "gla":
                mix = GatedLinearAttentionSpec(heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]), tau=float(m["tau"]))
                if min(mix.heads, mix.dim, mix.vdim) < 1 or not mix.tau > 0:
                    raise ValueError(f"layer {i}: inconsistent gated-linear-attention sizes")
            else:
                raise ValueError(f"layer {i}: unknown mixer type {typ!r}")
            md, mlp = ld.get("mlp"), None
            if md:
                if md.get("kind", "moe") != "moe":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {md.get('kind')!r}")
                mlp = SigmoidMoeSpec(experts=int(md["router"]["experts"]), top=int(md["router"]["top"]), expert_ff=int(md["expert"]["ff"]))
                if not 1 <= mlp.top <= mlp.experts or mlp.expert_ff < 1:
                    raise ValueError(f"layer {i}: top must be between 1 and the number of experts")
            layers.append(VefunexLayerSpec(type=typ, mixer=mix, mlp=mlp))
        taps = int((d.get("canon") or {}).get("taps", 1))
        if taps < 1:
            raise ValueError("canon.taps must be at least 1")
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), norm_eps=float((d.get("norm") or {}).get("eps", 1e-6)),
                   residual_mult=float(d.get("residual_mult", 1.0)), logit_softcap=float(d.get("logit_softcap") or 0.0), canon_taps=taps,
                   layers=layers, kv_page_size=int(d.get("kv_page_size", 64)), eos_token_id=int(d.get("eos_token_id", -1)),
                   pad_token_id=int(d.get("pad_token_id", 0)))

    def to_dict(self) -> dict:
        """The config.json form (round-trips through from_dict)."""
        def att(a: SoftmaxAttentionSpec) -> dict:
            md = {"dim": a.dim, "heads": a.heads, "kv_heads": a.kv_heads, "scale": a.scale, "vdim": a.vdim}
            if a.rot is not None:
                md["rot"] = {"base": a.rot.base, "dims": a.rot.dims}
            if a.q_temp_coef:
                md["q_temp"] = {"coef": a.q_temp_coef, "every": a.q_temp_every}
            if a.softcap:
                md["softcap"] = a.softcap
            return md
        out = []
        for l in self.layers:
            m = l.mixer
            if l.type == "attention":
                md = att(m)
            elif l.type == "parallel":
                md = {"left": att(m.left), "left_scale": m.left_scale, "right_scale": m.right_scale,
                      "right": {"conv": m.right.conv, "dt_rank": m.right.dt_rank, "inner": m.right.inner, "state": m.right.state}}
            else:
                md = {"dim": m.dim, "heads": m.heads, "tau": m.tau, "vdim": m.vdim}
            mlp = None
            if l.mlp is not None:
                mlp = {"expert": {"ff": l.mlp.expert_ff}, "kind": "moe", "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            out.append({"type": l.type, "mixer": md, "mlp": mlp})
        return {"architecture": "Vefunex", "vocab": self.vocab_size, "width": self.hidden_size, "norm": {"eps": self.norm_eps},
                "residual_mult": self.residual_mult, "logit_softcap": self.logit_softcap, "canon": {"taps": self.canon_taps}, "layers": out,
                "kv_page_size": self.kv_page_size, "eos_token_id": self.eos_token_id, "pad_token_id": self.pad_token_id}
