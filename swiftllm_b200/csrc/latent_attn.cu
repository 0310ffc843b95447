// Latent ("compressed KV") attention over a paged cache that holds, per token and caching layer, ONE row shared by all heads:
//     [ c (r values: the RMS-normed KV latent) | k_rot (dr values: the rotated key part, rotary already applied) ].
// Keys and values are never expanded: the caller folds the key up-projection into the query (q_lat[h] = W_uk[h]^T q_nope[h])
// and applies the value up-projection to the attention-weighted sum of latents, so per head
//     score(i, j) = (q_lat[i,h] . c[j] + rope(q_rot[i,h]) . k_rot[j]) * scale,   out_lat[i,h] = sum_j softmax_j(score) c[j].
// Every token of the step is a query with its own (block-table row, position): prompt portions and single decoded tokens go
// through the same kernel, so the result for a position does not depend on how its sequence was cut into steps.  A query at
// position p attends to the positions max(0, p - window + 1) .. p (window <= 0: all of 0 .. p).
// Softmax, the norm of the latent and the rotation run in fp32 for every storage type.
#include "typed_io.cuh"

namespace sllm {

// ------------------------------------------------------------------ cache store
// One CTA per token: c = rmsnorm(dkv[:r]) * norm_w, k_rot = interleaved rotary of dkv[r : r + dr] (the first rot_dims entries
// in pairs (2i, 2i+1), angle table cos/sin [T, rot_dims / 2]); both written to the token's row of cache slot `slot`.
template <typename T>
__global__ void __launch_bounds__(128) latent_kv_store_kernel(
    const T* __restrict__ dkv, int64_t row_stride, const T* __restrict__ norm_w, const float* __restrict__ cosb,
    const float* __restrict__ sinb, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
    const int* __restrict__ block_table, int max_blocks_per_seq, T* __restrict__ cache, int n_slots, int slot, int block_size,
    int r, int dr, int rot_dims, float eps) {
    __shared__ float red[32];
    const int64_t t = blockIdx.x;
    const T* row = dkv + t * row_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < r; i += blockDim.x) { const float v = ldf(row + i); ss += v * v; }
    const float denom = sqrtf(block_sum(ss, red) / (float)r + eps);
    const int pos = tok_pos[t];
    const int blk = block_table[(int64_t)tok_seq[t] * max_blocks_per_seq + pos / block_size];
    T* dst = cache + (((int64_t)blk * n_slots + slot) * block_size + pos % block_size) * (r + dr);
    for (int i = threadIdx.x; i < r; i += blockDim.x) stf(dst + i, ldf(row + i) / denom * ldf(norm_w + i));
    const int half = rot_dims >> 1;
    for (int j = threadIdx.x; j < dr; j += blockDim.x) {
        float o;
        if (j < rot_dims) {
            const int i = j >> 1;
            const float u = ldf(row + r + 2 * i), v = ldf(row + r + 2 * i + 1);
            const float c = cosb[t * half + i], s = sinb[t * half + i];
            o = (j & 1) ? v * c + u * s : u * c - v * s;
        } else {
            o = ldf(row + r + j);
        }
        stf(dst + r + j, o);
    }
}

// ------------------------------------------------------------------ attention
constexpr int LA_TILE = 32;        // keys per tile: one per lane in the score phase
constexpr int LA_MAX_HPB = 8;      // heads (warps) per CTA; they share the staged key tile

// grid (tokens, ceil(H / hpb)), hpb warps.  KR: per-lane accumulator registers, r <= 32 * KR.
template <typename T, int KR>
__global__ void __launch_bounds__(LA_MAX_HPB * 32) latent_attn_kernel(
    const T* __restrict__ q_lat, int64_t ql_stride_t, int64_t ql_stride_h,      // [T, H, r]
    const T* __restrict__ q_rot, int64_t qr_stride_t, int64_t qr_stride_h,      // [T, H, dr] (un-rotated; rotated here)
    const float* __restrict__ cosb, const float* __restrict__ sinb,            // [T, rot_dims / 2]
    const T* __restrict__ gate, int64_t gate_stride_t,                          // [T, H] logits of the output gate, or null
    const T* __restrict__ cache, int n_slots, int slot, int block_size,
    const int* __restrict__ block_table, int max_blocks_per_seq, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, T* __restrict__ out, int64_t out_stride_t, int64_t out_stride_h,
    int H, int r, int dr, int rot_dims, int window, float scale) {
    extern __shared__ float smem[];
    const int D = r + dr, DP = D + 1;
    const int hpb = blockDim.x >> 5;
    float* qs = smem;                      // [hpb][D]
    float* tile = smem + hpb * D;          // [LA_TILE][DP]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y * hpb + warp;
    const bool live = h < H;
    const int pos = tok_pos[t];
    const int* bt = block_table + (int64_t)tok_seq[t] * max_blocks_per_seq;

    if (live) {
        float* qw = qs + warp * D;
        const T* ql = q_lat + t * ql_stride_t + (int64_t)h * ql_stride_h;
        const T* qr = q_rot + t * qr_stride_t + (int64_t)h * qr_stride_h;
        for (int d = lane; d < r; d += 32) qw[d] = ldf(ql + d) * scale;
        const int half = rot_dims >> 1;
        for (int j = lane; j < dr; j += 32) {
            float o;
            if (j < rot_dims) {
                const int i = j >> 1;
                const float u = ldf(qr + 2 * i), v = ldf(qr + 2 * i + 1);
                const float c = cosb[t * half + i], s = sinb[t * half + i];
                o = (j & 1) ? v * c + u * s : u * c - v * s;
            } else {
                o = ldf(qr + j);
            }
            qw[r + j] = o * scale;
        }
    }

    float m = -INFINITY, l = 0.f;
    float acc[KR];
#pragma unroll
    for (int k = 0; k < KR; k++) acc[k] = 0.f;

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    for (int base = lo; base <= pos; base += LA_TILE) {
        __syncthreads();                   // the previous tile is no longer read (and qs is written, first time round)
        const int nkeys = min(LA_TILE, pos - base + 1);
        for (int jj = warp; jj < nkeys; jj += hpb) {
            const int kp = base + jj;
            const T* src = cache + (((int64_t)bt[kp / block_size] * n_slots + slot) * block_size + kp % block_size) * D;
            for (int d = lane; d < D; d += 32) tile[jj * DP + d] = ldf(src + d);
        }
        __syncthreads();
        if (!live) continue;
        const float* qw = qs + warp * D;
        float s = -INFINITY;
        if (lane < nkeys) {
            const float* kr = tile + lane * DP;
            float a = 0.f;
            for (int d = 0; d < D; d++) a += qw[d] * kr[d];
            s = a;
        }
        const float m_new = fmaxf(m, warp_max(s));          // finite: key `base` is always visible
        const float alpha = expf(m - m_new);                // 0 on the first tile (m = -inf)
        const float p = lane < nkeys ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int k = 0; k < KR; k++) acc[k] *= alpha;
        for (int jj = 0; jj < nkeys; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* kr = tile + jj * DP;
#pragma unroll
            for (int k = 0; k < KR; k++) {
                const int d = lane + 32 * k;
                if (d < r) acc[k] += pj * kr[d];
            }
        }
        m = m_new;
    }
    if (!live) return;
    float g = 1.f;
    if (gate != nullptr) g = 1.f / (1.f + expf(-ldf(gate + t * gate_stride_t + h)));
    T* o = out + t * out_stride_t + (int64_t)h * out_stride_h;
#pragma unroll
    for (int k = 0; k < KR; k++) {
        const int d = lane + 32 * k;
        if (d < r) stf(o + d, acc[k] / l * g);
    }
}

template <typename T, int KR>
static int launch_latent_attn(const void* q_lat, int64_t ql_st, int64_t ql_sh, const void* q_rot, int64_t qr_st, int64_t qr_sh,
                              const void* cosb, const void* sinb, const void* gate, int64_t gate_st, const void* cache,
                              int n_slots, int slot, int block_size, const void* block_table, int max_blocks_per_seq,
                              const void* tok_seq, const void* tok_pos, void* out, int64_t out_st, int64_t out_sh,
                              int64_t num_tokens, int H, int r, int dr, int rot_dims, int window, float scale,
                              cudaStream_t stream) {
    const int hpb = H < LA_MAX_HPB ? H : LA_MAX_HPB;
    const int D = r + dr;
    const size_t smem = ((size_t)hpb * D + (size_t)LA_TILE * (D + 1)) * sizeof(float);
    SLLM_REQUIRE(smem <= 200 * 1024, "latent_attention: r + dr = %d needs %zu bytes of shared memory", D, smem);
    static unsigned long long configured = 0;
    auto kern = latent_attn_kernel<T, KR>;
    if (smem > 48 * 1024 && first_use_on_this_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        SLLM_REQUIRE(e == cudaSuccess, "latent_attention: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    dim3 grid((unsigned)num_tokens, (unsigned)cdiv(H, hpb));
    kern<<<grid, hpb * 32, smem, stream>>>(
        (const T*)q_lat, ql_st, ql_sh, (const T*)q_rot, qr_st, qr_sh, (const float*)cosb, (const float*)sinb, (const T*)gate,
        gate_st, (const T*)cache, n_slots, slot, block_size, (const int*)block_table, max_blocks_per_seq, (const int*)tok_seq,
        (const int*)tok_pos, (T*)out, out_st, out_sh, H, r, dr, rot_dims, window, scale);
    return check_launch("latent_attention");
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_latent_kv_store(const void* dkv, int64_t row_stride, const void* norm_weight, const void* cosb, const void* sinb,
                         const void* tok_seq, const void* tok_pos, const void* block_table, int max_blocks_per_seq,
                         void* cache, int n_slots, int slot, int block_size, int64_t num_tokens, int r, int dr, int rot_dims,
                         float eps, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && r > 0 && dr >= 0 && rot_dims >= 0 && rot_dims <= dr && rot_dims % 2 == 0 &&
                 row_stride >= r + dr, "latent_kv_store: bad shape (r %d, dr %d, rot_dims %d)", r, dr, rot_dims);
    SLLM_REQUIRE(n_slots > 0 && slot >= 0 && slot < n_slots && block_size > 0 && max_blocks_per_seq > 0,
                 "latent_kv_store: bad cache geometry");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(dkv && norm_weight && tok_seq && tok_pos && block_table && cache && (rot_dims == 0 || (cosb && sinb)),
                 "latent_kv_store: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (latent_kv_store_kernel<T><<<(unsigned)num_tokens, 128, 0, (cudaStream_t)stream>>>(
        (const T*)dkv, row_stride, (const T*)norm_weight, (const float*)cosb, (const float*)sinb, (const int*)tok_seq,
        (const int*)tok_pos, (const int*)block_table, max_blocks_per_seq, (T*)cache, n_slots, slot, block_size, r, dr,
        rot_dims, eps)));
    return check_launch("latent_kv_store");
}

int sllm_latent_attention(const void* q_lat, int64_t q_lat_stride_t, int64_t q_lat_stride_h, const void* q_rot,
                          int64_t q_rot_stride_t, int64_t q_rot_stride_h, const void* cosb, const void* sinb,
                          const void* gate, int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                          const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos,
                          void* out, int64_t out_stride_t, int64_t out_stride_h, int64_t num_tokens, int num_heads, int r,
                          int dr, int rot_dims, int window, float scale, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && num_heads > 0 && r > 0 && r <= 512 && dr >= 0 && rot_dims >= 0 && rot_dims <= dr &&
                 rot_dims % 2 == 0, "latent_attention: bad shape (heads %d, r %d <= 512, dr %d, rot_dims %d)", num_heads, r, dr,
                 rot_dims);
    SLLM_REQUIRE(n_slots > 0 && slot >= 0 && slot < n_slots && block_size > 0 && max_blocks_per_seq > 0,
                 "latent_attention: bad cache geometry");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(q_lat && (dr == 0 || q_rot) && cache && block_table && tok_seq && tok_pos && out &&
                 (rot_dims == 0 || (cosb && sinb)), "latent_attention: null pointer");
#define SLLM_LA_ARGS q_lat, q_lat_stride_t, q_lat_stride_h, q_rot, q_rot_stride_t, q_rot_stride_h, cosb, sinb, gate,            \
                     gate_stride_t, cache, n_slots, slot, block_size, block_table, max_blocks_per_seq, tok_seq, tok_pos, out,   \
                     out_stride_t, out_stride_h, num_tokens, num_heads, r, dr, rot_dims, window, scale, (cudaStream_t)stream
    SLLM_DISPATCH_DTYPE_F32(dtype, {
        if (r <= 64) return (launch_latent_attn<T, 2>(SLLM_LA_ARGS));
        if (r <= 128) return (launch_latent_attn<T, 4>(SLLM_LA_ARGS));
        if (r <= 256) return (launch_latent_attn<T, 8>(SLLM_LA_ARGS));
        return (launch_latent_attn<T, 16>(SLLM_LA_ARGS));
    });
#undef SLLM_LA_ARGS
    return 0;
}

}  // extern "C"
