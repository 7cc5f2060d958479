"""Model geometries of the decode path: pure data, importable without the CUDA libraries.

A geometry is what the reference packages hard-code as module constants (``HIDDEN``, ``LAYERS``, ``KV_HEADS`` ... in
prime_kernels/decode_megakernel/__init__.py:37-43 and prime_kernels/decode_megakernel_360m/__init__.py:26-34 of
the reference project), made a value so one kernel family serves SmolLM2 135M / 360M / 1.7B.
"""
from __future__ import annotations

from dataclasses import dataclass

HEAD_DIM = 64


@dataclass(frozen=True)
class Geometry:
    name: str
    hidden: int
    intermediate: int
    layers: int
    q_heads: int
    kv_heads: int
    vocab: int = 49152
    rope_theta: float = 100000.0
    eps: float = 1e-5
    weight_format: int = 0   # 0 = bf16, 1 = MXFP8 packed rows

    @property
    def qkv_rows(self) -> int:
        return (self.q_heads + 2 * self.kv_heads) * HEAD_DIM

    def with_format(self, weight_format: int) -> "Geometry":
        return Geometry(self.name, self.hidden, self.intermediate, self.layers, self.q_heads, self.kv_heads,
                        self.vocab, self.rope_theta, self.eps, weight_format)

    def weight_bytes(self) -> int:
        """Bytes of every weight a decode step reads once (projections, norms, tied lm_head), bf16 or packed MXFP8."""
        h, i = self.hidden, self.intermediate

        def mat(rows, k):
            return rows * ((k + k // 32 + 15) // 16 * 16 if self.weight_format else 2 * k)

        per_layer = mat(self.qkv_rows, h) + mat(h, self.q_heads * HEAD_DIM) + mat(2 * i, h) + mat(h, i) + 2 * 2 * h
        return self.layers * per_layer + mat(self.vocab, h) + 2 * h

    def kv_bytes_per_position(self) -> int:
        """K and V bytes of one cache position over all layers."""
        return self.layers * self.kv_heads * HEAD_DIM * 2 * 2


SMOLLM2_135M = Geometry("smollm2-135m", 576, 1536, 30, 9, 3)
SMOLLM2_360M = Geometry("smollm2-360m", 960, 2560, 32, 15, 5)
SMOLLM2_1P7B = Geometry("smollm2-1.7b", 2048, 8192, 24, 32, 32, rope_theta=130000.0)
GEOMETRIES = {g.name: g for g in (SMOLLM2_135M, SMOLLM2_360M, SMOLLM2_1P7B)}
