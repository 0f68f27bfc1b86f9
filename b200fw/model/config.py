"""Model hyper-parameters (the HF ``config.json`` fields the reference reads,
src/engines/train_engine.py:604-628) and the architectures named by the benchmark configs."""
from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Dict


@dataclass
class ModelConfig:
    vocab_size: int = 151936
    hidden_size: int = 1024
    num_layers: int = 28
    num_heads: int = 16
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    max_position_embeddings: int = 32768
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    tie_word_embeddings: bool = True
    init_std: float = 0.02

    def to_hf(self) -> Dict:
        return {
            "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
            "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
            "num_hidden_layers": self.num_layers, "num_attention_heads": self.num_heads,
            "num_key_value_heads": self.num_kv_heads, "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "max_position_embeddings": self.max_position_embeddings, "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta, "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu", "torch_dtype": "bfloat16",
        }

    @classmethod
    def from_hf(cls, d: Dict) -> "ModelConfig":
        required = {"hidden_size", "num_attention_heads", "num_hidden_layers", "intermediate_size", "vocab_size"}
        missing = required - set(d)
        if missing:
            raise ValueError(f"config.json is missing required fields: {sorted(missing)}")
        return cls(
            vocab_size=d["vocab_size"], hidden_size=d["hidden_size"], num_layers=d["num_hidden_layers"],
            num_heads=d["num_attention_heads"], num_kv_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            head_dim=d.get("head_dim", d["hidden_size"] // d["num_attention_heads"]),
            intermediate_size=d["intermediate_size"],
            max_position_embeddings=d.get("max_position_embeddings", 32768),
            rms_norm_eps=d.get("rms_norm_eps", 1e-6), rope_theta=d.get("rope_theta", 1e6),
            tie_word_embeddings=d.get("tie_word_embeddings", False),
        )

    def num_params(self) -> int:
        H, I, D = self.hidden_size, self.intermediate_size, self.head_dim
        per_layer = H * D * (self.num_heads * 2 + self.num_kv_heads * 2) + 3 * H * I + 2 * H + 2 * D
        emb = self.vocab_size * H * (1 if self.tie_word_embeddings else 2)
        return self.num_layers * per_layer + emb + H

    def asdict(self) -> Dict:
        return asdict(self)


PRESETS: Dict[str, ModelConfig] = {
    # 4 layers, hidden 256, 4q/2kv heads of 64, FFN 704, vocab 8192, tied (CPU/gloo plumbing config)
    "tiny": ModelConfig(vocab_size=8192, hidden_size=256, num_layers=4, num_heads=4, num_kv_heads=2, head_dim=64,
                        intermediate_size=704, max_position_embeddings=4096, tie_word_embeddings=True),
    # same shape family with head_dim 128 so that the CUDA kernels apply
    "tiny128": ModelConfig(vocab_size=8192, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
                           head_dim=128, intermediate_size=768, max_position_embeddings=4096,
                           tie_word_embeddings=True),
    "qwen3-0.6b": ModelConfig(vocab_size=151936, hidden_size=1024, num_layers=28, num_heads=16, num_kv_heads=8,
                              head_dim=128, intermediate_size=3072, tie_word_embeddings=True),
    "qwen3-4b": ModelConfig(vocab_size=151936, hidden_size=2560, num_layers=36, num_heads=32, num_kv_heads=8,
                            head_dim=128, intermediate_size=9728, tie_word_embeddings=True),
    "qwen3-8b": ModelConfig(vocab_size=151936, hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8,
                            head_dim=128, intermediate_size=12288, tie_word_embeddings=False),
    "qwen3-32b": ModelConfig(vocab_size=151936, hidden_size=5120, num_layers=64, num_heads=64, num_kv_heads=8,
                             head_dim=128, intermediate_size=25600, tie_word_embeddings=False),
}
