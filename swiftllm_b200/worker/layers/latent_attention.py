"""Latent-attention mixer: queries through a normed low-rank latent, keys / values through ONE normed latent per token that
all heads share, plus one rotated key part; sliding-window causal softmax; a sigmoid gate per head on the output.

Only the latent c [r] and the rotated key part [dr] are cached.  Keys and values are never expanded: with W_uk[h] [dn, r] and
W_uv[h] [dv, r]
    q_nope[h] . (W_uk[h] c_j) = (W_uk[h]^T q_nope[h]) . c_j = q_lat[h] . c_j         (one batched GEMM over heads)
    sum_j p_j (W_uv[h] c_j)   = W_uv[h] (sum_j p_j c_j)    = W_uv[h] out_lat[h]      (one batched GEMM over heads)
so the attention kernel reads each cached row once for all heads.  Op sequence per step:
    fused [dq ; g ; dkv] GEMM -> RMS norm of the query latent -> uq GEMM -> (own latent: norm + rotary + cache store, one kernel)
    -> q_lat batched GEMM -> latent attention (rotary of q, window, softmax, gate: one kernel) -> uv batched GEMM -> o GEMM."""
import torch

from swiftllm_b200.worker.kernels.latent_attn import latent_attention, latent_kv_store
from swiftllm_b200.worker.kernels.linear import linear
from swiftllm_b200.worker.kernels.parallel_block import rmsnorm_strided


class LatentAttentionMixer:
    def __init__(self, spec, weight, eps: float, cache_key):
        self.spec, self.weight, self.eps = spec, weight, eps
        self.cache_width, self.cache_slot = cache_key          # which cache tensor and which of its slots this layer uses

    def forward(self, h: torch.Tensor, caches: dict, block_table: torch.Tensor, st) -> torch.Tensor:
        m, w = self.spec, self.weight
        T, H, dn, dr, r = h.shape[0], m.heads, m.dim, m.rot_dim, m.kv_rank
        proj = linear(h, w.in_proj)                             # [T, q_rank | H | (r + dr)]
        cq = rmsnorm_strided(proj[:, :m.q_rank], w.dq_norm, self.eps)
        gate = proj[:, m.q_rank:m.q_rank + H]
        q = linear(cq, w.uq).view(T, H, dn + dr)
        out_lat = torch.empty((T, H, r), dtype=h.dtype, device=h.device)
        if st.ignore_kvcache:
            out_lat.zero_()
        else:
            cos, sin = st.rotary[(m.rot_base, m.rot_dims)] if m.rot_dims > 0 else (None, None)
            cache = caches[self.cache_width]
            if m.kv_from is None:
                latent_kv_store(proj[:, m.q_rank + H:], w.dkv_norm, cache, self.cache_slot, block_table, st, r, dr, m.rot_dims,
                                self.eps, cos, sin)
            q_lat = torch.empty((T, H, r), dtype=h.dtype, device=h.device)
            torch.bmm(q[:, :, :dn].transpose(0, 1), w.uk, out=q_lat.transpose(0, 1))
            latent_attention(q_lat, q[:, :, dn:], gate, cache, self.cache_slot, block_table, st, out_lat, m.rot_dims, m.window,
                             m.scale, cos, sin)
        v = torch.empty((T, H, m.vdim), dtype=h.dtype, device=h.device)
        torch.bmm(out_lat.transpose(0, 1), w.uv.transpose(1, 2), out=v.transpose(0, 1))
        return linear(v.view(T, H * m.vdim), w.o)
