"""Architecture descriptions (no torch, no CUDA library: importable anywhere)."""
from __future__ import annotations

from dataclasses import dataclass, replace


@dataclass
class ModelArgs:
    """gpu/model.py:39-49, plus `tie_embeddings`."""

    dim: int = 2560
    n_layers: int = 30
    n_heads: int = 20
    n_kv_heads: int = 5
    vocab_size: int = 128256
    ffn_dim: int = 6912
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    use_kernel: bool = True
    tie_embeddings: bool = True

    @property
    def head_dim(self) -> int:
        return self.dim // self.n_heads


# The architectures the benchmark configurations name.
PRESETS = {
    "2b": ModelArgs(),
    "3b": ModelArgs(dim=3200, n_layers=26, n_heads=32, n_kv_heads=32, vocab_size=32002, ffn_dim=8640,
                    rope_theta=10000.0, tie_embeddings=False),
    "8b": ModelArgs(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, vocab_size=128256, ffn_dim=14336,
                    tie_embeddings=False),
    "100b": ModelArgs(dim=10240, n_layers=80, n_heads=80, n_kv_heads=8, vocab_size=128256, ffn_dim=32768,
                      tie_embeddings=False),
    # small shapes for tests
    "tiny": ModelArgs(dim=256, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=512, ffn_dim=384),
}


def preset(name: str, **overrides) -> ModelArgs:
    return replace(PRESETS[name], **overrides)
