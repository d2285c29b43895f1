"""Model targets: architecture facts, derived byte sizes and tensor-parallel sharding.

A `Target` carries everything the engine needs to size pools and pick kernels. Presets cover the five
benchmark configurations (tiny hybrid MoE, 27B-class dense NVFP4, Flash-Next-class hybrid MoE,
Nemotron-class Mamba-2 hybrid MoE) plus the reference's 27B hybrid layer set. The reference's equivalent is
hibana/target.py:24-173 (dataclass + shard()) and the per-model config modules
(hibana/model/qwen38_config.py:14-31, hibana/model/flashnext/config.py:15-50,
hibana/model/nemotron/config.py:33-73).
"""
from __future__ import annotations

from dataclasses import dataclass, field, replace
from typing import Optional

# Layer kinds of the mixer / FFN sequence.
ATTN, GATED_ATTN, MAMBA2, GDN = "attn", "gated_attn", "mamba2", "gdn"
MLP, MOE, LATENT_MOE, NONE = "mlp", "moe", "latent_moe", "none"


@dataclass(frozen=True)
class Target:
    name: str
    family: str                      # dense | hybrid_moe | flashnext | nemotron | qwen38 | bolt
    hidden: int
    vocab: int
    layers: tuple                    # tuple of (mixer kind, ffn kind)
    # attention
    q_heads: int = 0
    kv_heads: int = 0
    head_dim: int = 128
    rope_theta: float = 1e6
    rotary_frac: float = 1.0         # fraction of head_dim that is rotated (NeoX halves)
    qk_norm: bool = False
    gemma_norm: bool = False         # (1 + w) RMSNorm weights
    # dense FFN
    ffn: int = 0
    # Mamba-2
    mamba_heads: int = 0
    mamba_head_dim: int = 0
    mamba_state: int = 0
    mamba_groups: int = 1
    conv_width: int = 4
    mamba_chunk: int = 128
    # gated delta rule
    gdn_k_heads: int = 0
    gdn_v_heads: int = 0
    gdn_head_dim: int = 128
    # MoE
    experts: int = 0
    top_k: int = 0
    expert_ffn: int = 0
    shared_ffn: int = 0              # 0 = no shared expert
    router: str = "softmax"          # softmax | sigmoid
    router_scale: float = 1.0
    moe_act: str = "swiglu"          # swiglu | relu2
    latent: int = 0                  # latent MoE width (0 = experts act on hidden)
    # speculation
    mtp_layers: int = 0
    mtp_depth: int = 0
    # numerics / formats
    weight_format: str = "bf16"      # bf16 | nvfp4 | w3
    kv_dtype: str = "bf16"           # bf16 | fp8
    norm_eps: float = 1e-6
    max_context: int = 262144
    hyper_streams: int = 0           # > 1: hyper-connections (that many residual streams per token, models/hyper.py)
    hyper_rank: int = 64             # width of the low-rank gate projections of a hyper-connection site
    prefill_chunk: int = 2048
    tie_embeddings: bool = False
    vision: tuple = ()               # (image, patch, width, depth, heads, mlp) of the vision encoder; () = text only
    qsa_ratio: int = 0               # > 0: sparse attention indexer (models/qsa.py): tokens per compressed index key
    qsa_budget: int = 2048           # KV tokens a query row attends to through the indexer (plus its own group's tail)
    qsa_heads: int = 4               # index query heads (128 wide)
    ple_layers: tuple = ()           # block indices that add the per-layer n-gram embedding (models/ple.py) to the streams
    ple_heads: int = 4               # table heads per n-gram order (2- and 3-grams)
    ple_kernel: int = 4              # taps of its dilated convolution
    ple_rows: int = 1 << 18          # table rows per head (the synthetic table; a checkpoint brings its own sizes)
    ple_eos: int = 1                 # end-of-sequence id that cuts an n-gram context
    moe_specs: tuple = ()            # ((block index, experts, expert width), ...): blocks whose MoE differs from the default
    tp_size: int = 1
    tp_rank: int = 0

    def block(self, index: int) -> "Target":
        """The geometry block `index` is built with (heterogeneous MoE blocks override experts / width)."""
        for i, experts, width in self.moe_specs:
            if i == index:
                return replace(self, experts=experts, expert_ffn=width)
        return self

    # ---- derived
    @property
    def rot_dim(self) -> int:
        r = int(self.head_dim * self.rotary_frac)
        return r - (r % 2)

    @property
    def attn_layers(self) -> int:
        return sum(1 for m, _ in self.layers if m in (ATTN, GATED_ATTN))

    @property
    def recurrent_layers(self) -> int:
        return sum(1 for m, _ in self.layers if m in (MAMBA2, GDN))

    @property
    def kv_bytes_per_token(self) -> int:
        esz = 1 if self.kv_dtype == "fp8" else 2
        return self.attn_layers * 2 * self.kv_heads * self.head_dim * esz

    @property
    def mamba_inner(self) -> int:
        return self.mamba_heads * self.mamba_head_dim

    @property
    def mamba_conv_dim(self) -> int:
        return self.mamba_inner + 2 * self.mamba_groups * self.mamba_state

    @property
    def gdn_conv_dim(self) -> int:
        return (2 * self.gdn_k_heads + self.gdn_v_heads) * self.gdn_head_dim

    @property
    def state_bytes_per_slot(self) -> int:
        """Recurrent state (fp32 SSM / delta-rule state + bf16 conv window) of one sequence."""
        total = 0
        for mixer, _ in self.layers:
            if mixer == MAMBA2:
                total += self.mamba_heads * self.mamba_head_dim * self.mamba_state * 4
                total += self.mamba_conv_dim * (self.conv_width - 1) * 2
            elif mixer == GDN:
                total += self.gdn_v_heads * self.gdn_head_dim * self.gdn_head_dim * 4
                total += self.gdn_conv_dim * (self.conv_width - 1) * 2
        if self.ple_layers:      # the per-layer embedding's convolution window (3 = its dilation) and token history
            total += max(self.hyper_streams, 1) * self.hidden * (self.ple_kernel - 1) * 3 * 2 + 16
        return total

    def param_count(self) -> int:
        h = self.hidden
        n = self.vocab * h * (1 if self.tie_embeddings else 2)
        for mixer, ffn in self.layers:
            if mixer in (ATTN, GATED_ATTN):
                qw = self.q_heads * self.head_dim * (2 if mixer == GATED_ATTN else 1)
                n += h * (qw + 2 * self.kv_heads * self.head_dim) + self.q_heads * self.head_dim * h
            elif mixer == MAMBA2:
                n += h * (2 * self.mamba_inner + 2 * self.mamba_groups * self.mamba_state + self.mamba_heads)
                n += self.mamba_inner * h
            elif mixer == GDN:
                n += h * (self.gdn_conv_dim + self.gdn_v_heads * self.gdn_head_dim + 2 * self.gdn_v_heads)
                n += self.gdn_v_heads * self.gdn_head_dim * h
            if ffn == MLP:
                n += 3 * h * self.ffn
            elif ffn in (MOE, LATENT_MOE):
                width = self.latent or h
                mult = 3 if self.moe_act == "swiglu" else 2
                n += self.experts * mult * width * self.expert_ffn + h * self.experts
                n += mult * h * self.shared_ffn
                if self.latent:
                    n += 2 * h * self.latent
        return n

    def shard(self, size: int, rank: int = 0) -> "Target":
        """Per-rank geometry under tensor parallelism: heads and FFN widths divide; kv heads replicate when
        there are fewer of them than ranks (reference: hibana/target.py:114-122)."""
        if size == 1:
            return self
        def div(v: int) -> int:
            if v == 0:
                return 0
            if v % size:
                raise ValueError(f"{self.name}: {v} does not divide by tp={size}")
            return v // size
        kv = self.kv_heads // size if self.kv_heads >= size else (1 if self.kv_heads else 0)
        return replace(self, q_heads=div(self.q_heads), kv_heads=kv, ffn=div(self.ffn),
                       mamba_heads=div(self.mamba_heads),
                       mamba_groups=max(1, self.mamba_groups // size) if self.mamba_groups else 0,
                       gdn_k_heads=div(self.gdn_k_heads), gdn_v_heads=div(self.gdn_v_heads),
                       shared_ffn=div(self.shared_ffn), tp_size=size, tp_rank=rank)


def _pattern(n: int, mixers: list, ffn: str) -> tuple:
    return tuple((mixers[i % len(mixers)], ffn) for i in range(n))


def tiny_hybrid_moe() -> Target:
    """CPU-oracle configuration: [Mamba2, attn, Mamba2, attn] each followed by an 8-expert top-2 MoE."""
    return Target(name="tiny-hybrid-moe", family="hybrid_moe", hidden=256, vocab=4096,
                  layers=_pattern(4, [MAMBA2, ATTN], MOE), q_heads=4, kv_heads=2, head_dim=64, rope_theta=1e4,
                  mamba_heads=8, mamba_head_dim=32, mamba_state=64, mamba_groups=1, conv_width=4, mamba_chunk=64,
                  experts=8, top_k=2, expert_ffn=512, shared_ffn=512, router="softmax", mtp_layers=1, mtp_depth=2,
                  max_context=4096, prefill_chunk=256)


def dense_27b() -> Target:
    """27B-class dense decoder, NVFP4 weights, bf16 KV."""
    return Target(name="dense-27b", family="dense", hidden=5120, vocab=151936, layers=_pattern(64, [ATTN], MLP),
                  q_heads=40, kv_heads=8, head_dim=128, rope_theta=1e6, ffn=17408, weight_format="nvfp4")


def dense_tiny() -> Target:
    """Small dense decoder with the 27B layer structure (tests, smoke)."""
    return Target(name="dense-tiny", family="dense", hidden=512, vocab=2048, layers=_pattern(2, [ATTN], MLP),
                  q_heads=4, kv_heads=2, head_dim=128, rope_theta=1e6, ffn=1024, weight_format="nvfp4",
                  max_context=4096, prefill_chunk=512)


def qwen38_hybrid() -> Target:
    """The reference's 27B: 48 gated-delta-rule + 16 gated full-attention layers (every 4th)."""
    return Target(name="qwen38", family="qwen38", hidden=5120, vocab=248320,
                  layers=_pattern(64, [GDN, GDN, GDN, GATED_ATTN], MLP), q_heads=24, kv_heads=4, head_dim=256,
                  rope_theta=1e7, rotary_frac=0.25, qk_norm=True, gemma_norm=True, ffn=17408, gdn_k_heads=16,
                  gdn_v_heads=48, gdn_head_dim=128, mtp_layers=1, mtp_depth=3, weight_format="nvfp4", kv_dtype="fp8")


def flashnext() -> Target:
    """Flash-Next-class 125B hybrid MoE (reference dimensions)."""
    return Target(name="flashnext", family="flashnext", hidden=2560, vocab=248320,
                  layers=_pattern(48, [GDN, GDN, GDN, GATED_ATTN], MOE), q_heads=24, kv_heads=2, head_dim=256,
                  rope_theta=1e7, rotary_frac=0.25, qk_norm=True, gemma_norm=True, gdn_k_heads=16, gdn_v_heads=48,
                  gdn_head_dim=128, experts=512, top_k=10, expert_ffn=640, shared_ffn=640, router="softmax",
                  mtp_layers=1, mtp_depth=3, weight_format="nvfp4", kv_dtype="fp8", prefill_chunk=4096,
                  hyper_streams=4, hyper_rank=320, qsa_ratio=4, qsa_budget=2048, qsa_heads=4, ple_layers=(0,))


NEMOTRON_PATTERN = "MEMEMEM*EMEMEMEM*EMEMEMEM*EMEMEMEMEM*EMEMEMEMEM*EMEMEMEMEM*EMEMEMEMEM*EMEMEMEM*EMEMEMEME"


def nemotron() -> Target:
    """Nemotron-class 120B-A12B: 88 blocks by pattern (M = Mamba-2, E = latent MoE, * = attention)."""
    kinds = {"M": (MAMBA2, NONE), "E": (NONE, LATENT_MOE), "*": (ATTN, NONE)}
    layers = tuple(kinds[c] for c in NEMOTRON_PATTERN)
    return Target(name="nemotron", family="nemotron", hidden=4096, vocab=131072, layers=layers, q_heads=32,
                  kv_heads=2, head_dim=128, rotary_frac=0.0, mamba_heads=128, mamba_head_dim=64, mamba_state=128,
                  mamba_groups=8, conv_width=4, mamba_chunk=128, experts=512, top_k=22, expert_ffn=2688,
                  shared_ffn=5376, router="sigmoid", router_scale=5.0, moe_act="relu2", latent=1024, mtp_layers=1,
                  mtp_depth=3, weight_format="nvfp4", kv_dtype="fp8", norm_eps=1e-5, prefill_chunk=4096,
                  vision=(448, 16, 1280, 32, 16, 5120))


# Bolt: (block index, routed experts, expert width) of its 40 MoE blocks, and the blocks that are attention
# (architecture facts of the published config; every other block is Mamba-2).
BOLT_MOE = ((1, 240, 2048), (3, 240, 1536), (5, 240, 2048), (8, 304, 2304), (10, 240, 2304), (12, 240, 2048),
            (14, 240, 2048), (17, 304, 2304), (19, 304, 2048), (21, 432, 2560), (23, 432, 2304), (26, 240, 2048),
            (28, 432, 2304), (30, 304, 2560), (32, 304, 2304), (34, 432, 2304), (37, 368, 2304), (39, 368, 2048),
            (41, 368, 2304), (43, 432, 2560), (45, 368, 2560), (48, 496, 2560), (50, 432, 2560), (52, 240, 2304),
            (54, 368, 2304), (56, 368, 2560), (59, 304, 2048), (61, 240, 2304), (63, 240, 2304), (65, 240, 2048),
            (67, 240, 2048), (70, 368, 2048), (72, 368, 2304), (74, 432, 2304), (76, 432, 2560), (79, 496, 2560),
            (81, 432, 2560), (83, 432, 2560), (85, 496, 2560), (87, 368, 2560))
BOLT_ATTENTION = (7, 16, 25, 36, 47, 58, 69, 78)


def bolt() -> Target:
    """Bolt-class 74B-A9B: Nemotron geometry with heterogeneous MoE blocks (240 to 496 experts of width 1536 to
    2560, top-9), weights in GGML blocks (IQ2 experts, Q8_0 elsewhere) served in place. Reference:
    hibana/model/bolt/config.py:13-41."""
    moe = {i for i, _, _ in BOLT_MOE}
    layers = tuple((ATTN, NONE) if i in BOLT_ATTENTION else (NONE, LATENT_MOE) if i in moe else (MAMBA2, NONE)
                   for i in range(88))
    return Target(name="bolt", family="bolt", hidden=4096, vocab=131072, layers=layers, q_heads=32, kv_heads=2,
                  head_dim=128, rotary_frac=0.0, mamba_heads=128, mamba_head_dim=64, mamba_state=128, mamba_groups=8,
                  conv_width=4, mamba_chunk=128, experts=240, top_k=9, expert_ffn=2048, shared_ffn=5376,
                  router="sigmoid", router_scale=5.0, moe_act="relu2", latent=1024, weight_format="ggml",
                  kv_dtype="fp8", norm_eps=1e-5, prefill_chunk=2048, moe_specs=BOLT_MOE)


PRESETS = {
    "tiny": tiny_hybrid_moe, "tiny-hybrid-moe": tiny_hybrid_moe, "dense-27b": dense_27b, "27b-dense": dense_27b,
    "dense-tiny": dense_tiny, "qwen38": qwen38_hybrid, "27b": qwen38_hybrid, "flashnext": flashnext,
    "nemotron": nemotron, "bolt": bolt,
}


def get_target(name: str) -> Target:
    try:
        return PRESETS[name]()
    except KeyError:
        raise ValueError(f"unknown target {name!r}; known: {sorted(PRESETS)}") from None


def scaled(t: Target, *, layers: Optional[int] = None, **overrides) -> Target:
    """A down-scaled copy (same structure, fewer layers / other dims) for tests."""
    if t.ple_layers and overrides.get("hidden", t.hidden) < t.hidden:
        overrides.setdefault("ple_rows", 4096)        # a narrower copy gets a table to match
    if layers is not None:
        overrides["layers"] = t.layers[:layers]
        overrides.setdefault("moe_specs", tuple(sp for sp in t.moe_specs if sp[0] < layers))
    return replace(t, **overrides)
