"""KV-cache geometry and byte layout (engine/src/bruce.cu:43-65, 5473-5503)."""
from __future__ import annotations

from dataclasses import dataclass, replace

F32, F16 = 0, 1


@dataclass(frozen=True)
class Geom:
    n_head: int = 32
    n_kv: int = 8
    head_dim: int = 128
    window: int = 4096
    slot_ctx: int = 8192          # positions per slot of a full-attention layer (g_kv_nctx)
    n_slots: int = 1
    q_dtype: int = F16
    out_dtype: int = F16
    softmax_scale: float = 0.0    # 0 => 1/sqrt(head_dim)

    @property
    def group(self) -> int:
        return self.n_head // self.n_kv

    @property
    def rec(self) -> int:
        """Bytes of one (kv head, position) record: HD/32 fp16 scales, then HD int8 values."""
        return self.head_dim + 2 * (self.head_dim // 32)

    @property
    def pos_bytes(self) -> int:
        """K+V bytes per cached position per layer (2176 in both geometries)."""
        return 2 * self.n_kv * self.rec

    def pstride(self, is_swa: bool) -> int:
        return 2 * self.window if is_swa else self.slot_ctx

    def layer_bytes(self, is_swa: bool) -> int:
        return self.n_slots * self.pstride(is_swa) * self.n_kv * self.rec

    def slot_offset(self, slot: int, is_swa: bool) -> int:
        """Byte offset of a slot's partition inside a layer buffer (bruce.cu:5493-5503)."""
        return slot * self.pstride(is_swa) * self.n_kv * self.rec

    def with_(self, **kw) -> "Geom":
        return replace(self, **kw)


# graded geometry: 32 q-heads / 8 KV heads, head_dim 128, window 4096
G_B = Geom()
# the reference's native geometry (bruce.cu:43-53): 16 / 4 / 256, window 1024, fp32 q and out
G_R = Geom(n_head=16, n_kv=4, head_dim=256, window=1024, q_dtype=F32, out_dtype=F32)
