"""Gated sliding-window attention mixer with grouped key/value heads: ONE fused GEMM [q ; k ; v ; gate] on the block's normed
input -> (rotary of k + cache store, one kernel) -> attention over the paged cache (rotary of q, window, softmax with an
optional sink, sigmoid output gate: one kernel) -> o GEMM."""
import torch

from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.window_attn import window_attention, window_kv_store


class WindowAttentionMixer:
    def __init__(self, spec, weight, eps: float, cache_key):
        self.spec, self.weight = spec, weight
        self.cache_width, self.cache_slot = cache_key          # which cache tensor and which of its slots this layer uses

    def forward(self, h: torch.Tensor, caches: dict, block_table: torch.Tensor, st) -> torch.Tensor:
        m, w = self.spec, self.weight
        T, H, G, dk, dv = h.shape[0], m.heads, m.kv_heads, m.dim, m.vdim
        proj = linear(h, w.in_proj)                             # [T, H dk | G dk | G dv | H dv]
        q_end, k_end, v_end = H * dk, (H + G) * dk, (H + G) * dk + G * dv
        out = torch.empty((T, H * dv), dtype=h.dtype, device=h.device)
        if st.ignore_kvcache:
            out.zero_()
        else:
            cos, sin = st.rotary[(m.rot_base, m.rot_dims)] if m.rot_dims > 0 else (None, None)
            cache = caches[self.cache_width]
            window_kv_store(proj[:, q_end:k_end], proj[:, k_end:v_end], cache, self.cache_slot, block_table, st, G, dk, dv,
                            m.rot_dims, cos, sin)
            window_attention(proj[:, :q_end], proj[:, v_end:], cache, self.cache_slot, block_table, st, out, H, G, dk, dv,
                             m.rot_dims, m.window, m.scale, m.sink, cos, sin)
        return linear(out, w.o)
