"""Model configuration for DeepSeek-V4.1-Flash-shaped models.

`ModelConfig.flash()` mirrors the official configuration embedded by the
reference loader (rust/crates/ds41rt-loader/src/official-v41-config.json:24-155);
`ModelConfig.tiny()` is a CPU-sized model with the same structure used as the
numerical oracle workload.  `ModelConfig.from_official_json` parses the official
`config.json` strictly: unknown or missing text-config keys are errors, like
rust/crates/ds41rt-loader/src/v41_config.rs:87-114.
"""
from __future__ import annotations

import dataclasses
import json
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass
class RopeConfig:
    theta: float = 10000.0
    # YaRN parameters; factor == 1 disables scaling.
    factor: float = 1.0
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    original_max_position: int = 65536


@dataclass
class DSparkConfig:
    stages: int = 3
    block_size: int = 5
    noise_token_id: int = 128799
    tap_layers: Tuple[int, ...] = (37, 38, 39)
    markov_rank: int = 256
    n_experts: int = 128
    topk: int = 3
    ring_rows: int = 128


@dataclass
class EngramConfig:
    layers: Tuple[int, ...] = (1, 14)
    num_embeddings: Tuple[int, ...] = (384006168, 384016682)
    max_ngram: int = 4
    vocab_size: int = 16000000
    n_heads: int = 8
    head_dim: int = 256
    pad_token_id: int = 2
    compressed_vocab: int = 99092


@dataclass
class VisionConfig:
    layers: int = 32
    hidden: int = 1024
    heads: int = 16
    intermediate: int = 2816
    patch: int = 14
    rope_theta: float = 10000.0
    downsample: int = 3
    max_image_tokens: int = 1024
    min_pixels: int = 295936


@dataclass
class ModelConfig:
    name: str = "flash"
    vocab: int = 129280
    hidden: int = 5120
    n_layers: int = 40
    n_heads: int = 64
    head_dim: int = 512          # one KV head of this width is both K and V
    rope_dim: int = 64           # last rope_dim dims of every head are rotary
    q_lora: int = 1280
    o_groups: int = 8
    o_lora: int = 1024           # output width of each wo_a group
    window: int = 128
    norm_eps: float = 1e-20
    # compression: layer -> ratio for layers that PRODUCE a compressed source
    source_layers: Dict[int, int] = field(default_factory=lambda: {2: 2, 8: 2, 14: 2, 20: 1})
    # per-layer compress ratio (0 = window only); selects which source a layer reads
    compress_ratios: List[int] = field(default_factory=lambda: [0, 0] + [2] * 18 + [1] * 20)
    index_layers: Tuple[int, ...] = (2, 8, 14, 20, 24, 28, 32, 36)
    index_heads: int = 32
    index_dim: int = 128
    index_topk: int = 512
    candidate_layer: int = 20
    candidate_topk_blocks: int = 2048
    candidate_block: int = 8
    # prompt passes: layers below the boundary ("encoder") run over the whole prompt, the layers from it upwards
    # ("decoder") only over the last `ced_replay` prompt tokens; the boundary layer still produces its compressed source
    # for every token.  Inactive unless 0 < ced_boundary < n_layers.
    ced_boundary: int = 20
    ced_replay: int = 128
    # hyper-connections
    hc_mult: int = 4
    hc_sinkhorn_iters: int = 20
    hc_eps: float = 1e-6
    # MoE
    n_experts: int = 384
    topk: int = 6
    n_shared: int = 1
    inter: int = 2304
    route_scale: float = 1.5
    swiglu_limit: float = 10.0
    # rope: layers with compress ratio 0 use `rope_plain`, the others `rope_long`
    rope_plain: RopeConfig = field(default_factory=lambda: RopeConfig(theta=10000.0))
    rope_long: RopeConfig = field(default_factory=lambda: RopeConfig(theta=160000.0, factor=16.0))
    bos: int = 0
    eos: int = 1
    pad: int = 2
    image_token: int = 129264
    think_end_token: int = 128822
    max_context: int = 1048576
    dspark: Optional[DSparkConfig] = field(default_factory=DSparkConfig)
    engram: Optional[EngramConfig] = field(default_factory=EngramConfig)
    vision: Optional[VisionConfig] = field(default_factory=VisionConfig)

    # ------------------------------------------------------------------ derived
    @property
    def heads_per_group(self) -> int:
        return self.n_heads // self.o_groups

    @property
    def softmax_scale(self) -> float:
        return self.head_dim ** -0.5

    @property
    def index_weight_scale(self) -> float:
        # (index_dim * index_heads) ** -0.5 ; 1/64 for the flash model
        return (self.index_dim * self.index_heads) ** -0.5

    def source_of(self, layer: int) -> Optional[int]:
        """Layer whose compressed source `layer` reads (None = window only)."""
        if self.compress_ratios[layer] == 0:
            return None
        best = None
        for s in sorted(self.source_layers):
            if s <= layer:
                best = s
        return best

    def index_producer_of(self, layer: int) -> Optional[int]:
        """Nearest index layer at or below `layer` (selection reuse rule,
        rust/crates/ds41rt-daemon/src/v41_index_selection.rs:66-78)."""
        if self.source_of(layer) is None:
            return None
        best = None
        for s in self.index_layers:
            if s <= layer:
                best = s
        return best

    @property
    def ced_on(self) -> bool:
        """True when this model can prefill with the decoder layers replayed for the prompt's tail only: a boundary
        inside the stack and no compressed source produced above it."""
        b = self.ced_boundary
        return 0 < b < self.n_layers and all(s <= b for s in self.source_layers if s < self.n_layers)

    def rope_for(self, layer: int) -> RopeConfig:
        return self.rope_plain if self.compress_ratios[layer] == 0 else self.rope_long

    def validate(self) -> None:
        assert self.n_heads % self.o_groups == 0
        assert len(self.compress_ratios) >= self.n_layers
        assert self.rope_dim % 2 == 0 and self.rope_dim <= self.head_dim
        for s, r in self.source_layers.items():
            assert r in (1, 2), "compress ratio must be 1 or 2"
            assert self.compress_ratios[s] == r
        for l in range(self.n_layers):
            if self.compress_ratios[l]:
                assert self.source_of(l) is not None, f"layer {l} has no source"
                assert self.source_layers[self.source_of(l)] == self.compress_ratios[l]
                assert self.index_producer_of(l) is not None

    # ------------------------------------------------------------------ presets
    @staticmethod
    def flash(n_layers: int = 40) -> "ModelConfig":
        c = ModelConfig()
        if n_layers != 40:
            c = c.truncated(n_layers)
        c.validate()
        return c

    def truncated(self, n_layers: int) -> "ModelConfig":
        """Same architecture with only the first `n_layers` layers (used to fit
        fewer GPUs); source/index layers above the cut disappear."""
        c = dataclasses.replace(self)
        c.n_layers = n_layers
        c.name = f"{self.name}-L{n_layers}"
        c.source_layers = {k: v for k, v in self.source_layers.items() if k < n_layers}
        c.index_layers = tuple(l for l in self.index_layers if l < n_layers)
        c.compress_ratios = list(self.compress_ratios[:n_layers])
        if c.dspark is not None:
            taps = tuple(range(max(0, n_layers - 3), n_layers))
            c.dspark = dataclasses.replace(c.dspark, tap_layers=taps)
        if c.engram is not None:
            keep = [i for i, l in enumerate(c.engram.layers) if l < n_layers]
            c.engram = dataclasses.replace(
                c.engram, layers=tuple(c.engram.layers[i] for i in keep),
                num_embeddings=tuple(c.engram.num_embeddings[i] for i in keep)) if keep else None
        return c

    @staticmethod
    def tiny() -> "ModelConfig":
        """CPU oracle config: vocab 4096, hidden 512, 2 layers, q rank 192, latent
        width 128 with 32 rotary dims, 8 heads, indexer 4x32 top-64, 16 experts top-4."""
        c = ModelConfig(
            name="tiny", vocab=4096, hidden=512, n_layers=2, n_heads=8, head_dim=128, rope_dim=32,
            q_lora=192, o_groups=2, o_lora=128, window=32,
            source_layers={0: 2, 1: 1}, compress_ratios=[2, 1], index_layers=(0, 1),
            index_heads=4, index_dim=32, index_topk=64,
            candidate_layer=-1, candidate_topk_blocks=0, candidate_block=8,
            n_experts=16, topk=4, inter=256,
            rope_plain=RopeConfig(theta=10000.0), rope_long=RopeConfig(theta=10000.0),
            image_token=4095, think_end_token=4094, max_context=4096,
            dspark=DSparkConfig(stages=1, block_size=5, noise_token_id=4093, tap_layers=(0, 1),
                                markov_rank=32, n_experts=8, topk=2, ring_rows=32),
            engram=None, vision=None)
        c.validate()
        return c

    @staticmethod
    def small() -> "ModelConfig":
        """GPU test config whose dims exercise the tensor-core tile shapes
        (hidden 1024, latent 512 like the real model) while staying small."""
        c = ModelConfig(
            name="small", vocab=8192, hidden=1024, n_layers=4, n_heads=16, head_dim=512, rope_dim=64,
            q_lora=256, o_groups=2, o_lora=256, window=128,
            source_layers={1: 2, 2: 1}, compress_ratios=[0, 2, 1, 1], index_layers=(1, 2),
            index_heads=8, index_dim=128, index_topk=128,
            candidate_layer=-1, candidate_topk_blocks=0,
            n_experts=32, topk=4, inter=512,
            image_token=8191, think_end_token=8190, max_context=65536,
            dspark=DSparkConfig(stages=1, noise_token_id=8189, tap_layers=(1, 2, 3), markov_rank=64,
                                n_experts=8, topk=2),
            engram=None, vision=None)
        c.validate()
        return c

    # ------------------------------------------------------------------ official
    _TEXT_KEYS = {
        "model_type", "vocab_size", "hidden_size", "moe_intermediate_size", "num_hidden_layers",
        "num_attention_heads", "num_key_value_heads", "head_dim", "qk_rope_head_dim", "q_lora_rank",
        "o_lora_rank", "o_groups", "hidden_act", "swiglu_limit", "rms_norm_eps", "attention_bias",
        "attention_dropout", "initializer_range", "use_cache", "tie_word_embeddings",
        "max_position_embeddings", "rope_theta", "rope_scaling", "n_routed_experts", "n_shared_experts",
        "num_experts_per_tok", "scoring_func", "topk_method", "norm_topk_prob", "routed_scaling_factor",
        "sliding_window", "compress_ratios", "compress_rope_theta", "kv_source_layer_ids",
        "index_source_layer_ids", "index_n_heads", "index_head_dim", "index_topk",
        "candidate_source_layer_id", "candidate_topk_blocks", "candidate_block_size", "hc_mult",
        "hc_sinkhorn_iters", "hc_eps", "engram_layer_ids", "engram_num_embeddings",
        "engram_max_ngram_size", "engram_vocab_size", "engram_n_heads", "engram_head_dim",
        "engram_pad_token_id", "engram_compressed_vocab_size", "num_nextn_predict_layers",
        "dspark_block_size", "dspark_noise_token_id", "dspark_target_layer_ids", "dspark_markov_rank",
        "dspark_n_routed_experts", "dspark_num_experts_per_tok",
    }

    @staticmethod
    def from_official_json(text: str) -> "ModelConfig":
        doc = json.loads(text)
        for key in ("text_config", "vision_config", "quantization_config"):
            if key not in doc:
                raise ValueError(f"official config: missing '{key}'")
        t = doc["text_config"]
        unknown = set(t) - ModelConfig._TEXT_KEYS
        missing = ModelConfig._TEXT_KEYS - set(t)
        if unknown:
            raise ValueError(f"official config: unknown text_config keys {sorted(unknown)}")
        if missing:
            raise ValueError(f"official config: missing text_config keys {sorted(missing)}")
        if t["scoring_func"] != "sqrtsoftplus" or t["num_key_value_heads"] != 1:
            raise ValueError("official config: unsupported router scoring or KV head count")
        n = t["num_hidden_layers"]
        ratios = list(t["compress_ratios"])
        sources = {int(l): ratios[int(l)] for l in t["kv_source_layer_ids"]}
        rs = t["rope_scaling"]
        v = doc["vision_config"]
        c = ModelConfig(
            name="flash", vocab=t["vocab_size"], hidden=t["hidden_size"], n_layers=n,
            n_heads=t["num_attention_heads"], head_dim=t["head_dim"], rope_dim=t["qk_rope_head_dim"],
            q_lora=t["q_lora_rank"], o_groups=t["o_groups"], o_lora=t["o_lora_rank"],
            window=t["sliding_window"], norm_eps=t["rms_norm_eps"], source_layers=sources,
            compress_ratios=ratios, index_layers=tuple(t["index_source_layer_ids"]),
            index_heads=t["index_n_heads"], index_dim=t["index_head_dim"], index_topk=t["index_topk"],
            candidate_layer=t["candidate_source_layer_id"], candidate_topk_blocks=t["candidate_topk_blocks"],
            candidate_block=t["candidate_block_size"], hc_mult=t["hc_mult"],
            hc_sinkhorn_iters=t["hc_sinkhorn_iters"], hc_eps=t["hc_eps"], n_experts=t["n_routed_experts"],
            topk=t["num_experts_per_tok"], n_shared=t["n_shared_experts"], inter=t["moe_intermediate_size"],
            route_scale=t["routed_scaling_factor"], swiglu_limit=t["swiglu_limit"],
            rope_plain=RopeConfig(theta=float(t["rope_theta"])),
            rope_long=RopeConfig(theta=float(t["compress_rope_theta"]), factor=float(rs["factor"]),
                                 beta_fast=float(rs["beta_fast"]), beta_slow=float(rs["beta_slow"]),
                                 original_max_position=int(rs["original_max_position_embeddings"])),
            bos=doc.get("bos_token_id", 0), eos=doc.get("eos_token_id", 1), pad=doc.get("pad_token_id", 2),
            image_token=doc.get("image_token_id", 129264), max_context=t["max_position_embeddings"],
            dspark=DSparkConfig(stages=t["num_nextn_predict_layers"], block_size=t["dspark_block_size"],
                                noise_token_id=t["dspark_noise_token_id"],
                                tap_layers=tuple(t["dspark_target_layer_ids"]),
                                markov_rank=t["dspark_markov_rank"], n_experts=t["dspark_n_routed_experts"],
                                topk=t["dspark_num_experts_per_tok"]),
            engram=EngramConfig(layers=tuple(t["engram_layer_ids"]),
                                num_embeddings=tuple(t["engram_num_embeddings"]),
                                max_ngram=t["engram_max_ngram_size"], vocab_size=t["engram_vocab_size"],
                                n_heads=t["engram_n_heads"], head_dim=t["engram_head_dim"],
                                pad_token_id=t["engram_pad_token_id"],
                                compressed_vocab=t["engram_compressed_vocab_size"]),
            vision=VisionConfig(layers=v["num_hidden_layers"], hidden=v["hidden_size"],
                                heads=v["num_attention_heads"], intermediate=v["intermediate_size"],
                                patch=v["patch_size"], rope_theta=float(v["rope_theta"]),
                                downsample=v["downsample_ratio"], max_image_tokens=v["max_image_tokens"],
                                min_pixels=v["min_pixels"]))
        c.validate()
        return c


def rope_inv_freq(rope: RopeConfig, dim: int) -> List[float]:
    """Inverse frequencies for `dim` rotary dims (dim/2 pairs) with YaRN
    correction when factor > 1 (native/cuda/kernels/v41_attention_ops.cu:328-341)."""
    half = dim // 2
    base = [rope.theta ** (-2.0 * i / dim) for i in range(half)]
    if rope.factor <= 1.0:
        return base

    def corr_dim(rot: float) -> float:
        return dim * math.log(rope.original_max_position / (rot * 2 * math.pi)) / (2 * math.log(rope.theta))

    low = max(math.floor(corr_dim(rope.beta_fast)), 0)
    high = min(math.ceil(corr_dim(rope.beta_slow)), dim - 1)
    if high == low:
        high += 0.001
    out = []
    for i in range(half):
        ramp = min(max((i - low) / (high - low), 0.0), 1.0)
        mask = 1.0 - ramp            # 1 -> keep extrapolated (high-frequency) value
        out.append(base[i] / rope.factor * (1 - mask) + base[i] * mask)
    return out
