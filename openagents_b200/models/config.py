"""Model shapes and their GGUF metadata mapping.

The presets are the shapes the benchmark configurations name; the server detects a family from
``general.architecture`` the way the reference's model registry is described to
(reference: docs/muse/muse-glimmer.md:118-126).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass, replace


@dataclass(frozen=True)
class ModelConfig:
    arch: str = "llama"            # llama | gpt2 | gpt-oss
    n_layers: int = 2
    d_model: int = 256
    n_heads: int = 4
    n_kv_heads: int = 2
    head_dim: int = 64
    ffn: int = 688
    vocab: int = 32000
    context: int = 2048
    rope_theta: float = 10000.0
    rope_style: str = "pairs"      # "pairs": (2i, 2i+1) rotate together; "half": (i, i + hd/2)
    norm_eps: float = 1e-5
    tied_embeddings: bool = False
    # mixture of experts (gpt-oss)
    n_experts: int = 0
    top_k: int = 0
    sliding_window: int = 0        # 0 = every layer attends to the full context
    swa_every: int = 2             # layer i uses the window when sliding_window > 0 and i % swa_every == 0
    attn_sinks: bool = False
    qkv_bias: bool = False
    name: str = "tiny-llama"

    @property
    def q_dim(self) -> int:
        return self.n_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv_heads * self.head_dim

    def layer_uses_window(self, i: int) -> bool:
        return self.sliding_window > 0 and i % self.swa_every == 0

    def n_params(self) -> int:
        d, f, v = self.d_model, self.ffn, self.vocab
        if self.arch == "gpt2":
            per = 4 * d * d + 2 * d * f + 9 * d + f
            return self.n_layers * per + v * d + self.context * d + 2 * d
        attn = d * self.q_dim * 2 + d * self.kv_dim * 2
        mlp = 3 * d * f * max(1, self.n_experts)
        emb = v * d * (1 if self.tied_embeddings else 2)
        return self.n_layers * (attn + mlp + 2 * d) + emb + d

    def to_gguf_metadata(self) -> dict:
        a = self.arch
        md = {
            "general.architecture": a,
            "general.name": self.name,
            f"{a}.block_count": self.n_layers,
            f"{a}.embedding_length": self.d_model,
            f"{a}.feed_forward_length": self.ffn,
            f"{a}.attention.head_count": self.n_heads,
            f"{a}.attention.head_count_kv": self.n_kv_heads,
            f"{a}.attention.key_length": self.head_dim,
            f"{a}.attention.layer_norm_rms_epsilon": float(self.norm_eps),
            f"{a}.rope.freq_base": float(self.rope_theta),
            f"{a}.context_length": self.context,
            f"{a}.vocab_size": self.vocab,
            "b200.rope_style": self.rope_style,
            "b200.tied_embeddings": self.tied_embeddings,
        }
        if self.n_experts:
            md[f"{a}.expert_count"] = self.n_experts
            md[f"{a}.expert_used_count"] = self.top_k
        if self.sliding_window:
            md[f"{a}.attention.sliding_window"] = self.sliding_window
            md["b200.swa_every"] = self.swa_every
        md["b200.attn_sinks"] = self.attn_sinks
        md["b200.qkv_bias"] = self.qkv_bias
        return md

    @staticmethod
    def from_gguf_metadata(md: dict) -> "ModelConfig":
        a = md.get("general.architecture")
        if a not in ("llama", "gpt2", "gpt-oss"):
            raise ValueError(f"unsupported architecture {a!r}")
        g = lambda k, dflt=None: md.get(f"{a}.{k}", dflt)
        n_heads = int(g("attention.head_count"))
        d = int(g("embedding_length"))
        hd = int(g("attention.key_length", d // n_heads))
        return ModelConfig(
            arch=a, n_layers=int(g("block_count")), d_model=d, n_heads=n_heads,
            n_kv_heads=int(g("attention.head_count_kv", n_heads)), head_dim=hd,
            ffn=int(g("feed_forward_length")), vocab=int(g("vocab_size", 0)),
            context=int(g("context_length", 2048)), rope_theta=float(g("rope.freq_base", 10000.0)),
            rope_style=md.get("b200.rope_style", "half" if a == "gpt-oss" else "pairs"),
            norm_eps=float(g("attention.layer_norm_rms_epsilon", g("attention.layer_norm_epsilon", 1e-5))),
            tied_embeddings=bool(md.get("b200.tied_embeddings", a == "gpt2")),
            n_experts=int(g("expert_count", 0)), top_k=int(g("expert_used_count", 0)),
            sliding_window=int(g("attention.sliding_window", 0)), swa_every=int(md.get("b200.swa_every", 2)),
            attn_sinks=bool(md.get("b200.attn_sinks", a == "gpt-oss")),
            qkv_bias=bool(md.get("b200.qkv_bias", a == "gpt2")),
            name=md.get("general.name", a))

    def with_(self, **kw) -> "ModelConfig":
        return replace(self, **kw)

    def as_dict(self) -> dict:
        return asdict(self)


TINY_LLAMA = ModelConfig()
LLAMA3_8B = ModelConfig(arch="llama", n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                        ffn=14336, vocab=128256, context=8192, rope_theta=500000.0, name="llama-3-8b-shape")
LLAMA3_70B = ModelConfig(arch="llama", n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128,
                         ffn=28672, vocab=128256, context=16384, rope_theta=500000.0, name="llama-3-70b-shape")
GPT2_SMALL = ModelConfig(arch="gpt2", n_layers=12, d_model=768, n_heads=12, n_kv_heads=12, head_dim=64,
                         ffn=3072, vocab=50257, context=1024, tied_embeddings=True, qkv_bias=True,
                         name="gpt2-small-shape")
GPT_OSS_20B = ModelConfig(arch="gpt-oss", n_layers=24, d_model=2880, n_heads=64, n_kv_heads=8, head_dim=64,
                          ffn=2880, vocab=201088, context=8192, rope_theta=150000.0, rope_style="half",
                          n_experts=32, top_k=4, sliding_window=128, swa_every=2, attn_sinks=True,
                          name="gpt-oss-20b-shape")

PRESETS = {c.name: c for c in (TINY_LLAMA, LLAMA3_8B, LLAMA3_70B, GPT2_SMALL, GPT_OSS_20B)}
