// Gated sliding-window attention with grouped key/value heads and an optional softmax sink, over a paged cache that holds per
// token and layer ONE row [ k (G heads x dk, rotary applied) | v (G heads x dv) ].
//   score(i, j) = rope(q[i,h]) . k[j, g(h)] * scale          g(h) = h / (H / G)
//   p(i, j)     = exp(score) / (sink + sum_j' exp(score))     sink = 1 when the softmax has a value-less sink of score 0, else 0
//   out[i, h]   = sigmoid(gate[i, h, :]) * sum_j p(i, j) v[j, g(h)]          (element-wise gate; no gate when null)
// Every token of the step is a query with its own (block-table row, position): prompt portions and single decoded tokens go
// through the same kernel, so the result at a position does not depend on how its sequence was cut into steps.  A query at
// position p sees the positions max(0, p - window + 1) .. p (window <= 0: all of 0 .. p).  Rotary pairs are interleaved
// ((2i, 2i+1), the first rot_dims entries of a head; the rest pass through).  Softmax, rotation and the weighted sum of values
// run in fp32 for every storage type.
#include "typed_io.cuh"

namespace sllm {

// ------------------------------------------------------------------ cache store
// One CTA per token: rotate k, copy v, write the token's row of cache slot `slot`.
template <typename T>
__global__ void __launch_bounds__(128) window_kv_store_kernel(
    const T* __restrict__ k, int64_t k_stride, const T* __restrict__ v, int64_t v_stride, const float* __restrict__ cosb,
    const float* __restrict__ sinb, const int* __restrict__ tok_seq, const int* __restrict__ tok_pos,
    const int* __restrict__ block_table, int max_blocks_per_seq, T* __restrict__ cache, int n_slots, int slot, int block_size,
    int G, int dk, int dv, int rot_dims) {
    const int64_t t = blockIdx.x;
    const int pos = tok_pos[t];
    const int blk = block_table[(int64_t)tok_seq[t] * max_blocks_per_seq + pos / block_size];
    const int kw = G * dk, vw = G * dv;
    T* dst = cache + (((int64_t)blk * n_slots + slot) * block_size + pos % block_size) * (kw + vw);
    const T* kr = k + t * k_stride;
    const T* vr = v + t * v_stride;
    const int half = rot_dims >> 1;
    for (int c = threadIdx.x; c < kw; c += blockDim.x) {
        const int j = c % dk, base = c - j;
        float o;
        if (j < rot_dims) {
            const int i = j >> 1;
            const float a = ldf(kr + base + 2 * i), b = ldf(kr + base + 2 * i + 1);
            const float cs = cosb[t * half + i], sn = sinb[t * half + i];
            o = (j & 1) ? b * cs + a * sn : a * cs - b * sn;
        } else {
            o = ldf(kr + c);
        }
        stf(dst + c, o);
    }
    for (int c = threadIdx.x; c < vw; c += blockDim.x) dst[kw + c] = vr[c];
}

// ------------------------------------------------------------------ attention (fp32 CUDA cores)
constexpr int WA_TILE = 32;        // keys per tile: one per lane in the score phase
constexpr int WA_MAX_HPB = 8;      // query heads (warps) per CTA: heads of ONE key/value group, they share the staged tile

// grid (tokens, H / hpb), hpb warps; hpb divides H / G.  KR: per-lane accumulator registers, dv <= 32 * KR.
template <typename T, int KR>
__global__ void __launch_bounds__(WA_MAX_HPB * 32) window_attn_kernel(
    const T* __restrict__ q, int64_t q_stride_t,                                 // [T, H, dk] (un-rotated; rotated here)
    const float* __restrict__ cosb, const float* __restrict__ sinb,            // [T, rot_dims / 2]
    const T* __restrict__ gate, int64_t gate_stride_t,                          // [T, H, dv] gate logits, or null
    const T* __restrict__ cache, int n_slots, int slot, int block_size,
    const int* __restrict__ block_table, int max_blocks_per_seq, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, T* __restrict__ out, int64_t out_stride_t,  // [T, H, dv]
    int H, int G, int dk, int dv, int rot_dims, int window, float scale, float sink) {
    extern __shared__ float smem[];
    const int KP = dk + 1;
    const int hpb = blockDim.x >> 5;
    float* qs = smem;                          // [hpb][dk]
    float* kt = qs + hpb * dk;                 // [WA_TILE][dk + 1]
    float* vt = kt + WA_TILE * KP;             // [WA_TILE][dv]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t t = blockIdx.x;
    const int h = blockIdx.y * hpb + warp;
    const int g = (blockIdx.y * hpb) / (H / G);
    const int pos = tok_pos[t];
    const int* bt = block_table + (int64_t)tok_seq[t] * max_blocks_per_seq;
    const int row = G * (dk + dv);

    {
        float* qw = qs + warp * dk;
        const T* qr = q + t * q_stride_t + (int64_t)h * dk;
        const int half = rot_dims >> 1;
        for (int j = lane; j < dk; j += 32) {
            float o;
            if (j < rot_dims) {
                const int i = j >> 1;
                const float a = ldf(qr + 2 * i), b = ldf(qr + 2 * i + 1);
                const float cs = cosb[t * half + i], sn = sinb[t * half + i];
                o = (j & 1) ? b * cs + a * sn : a * cs - b * sn;
            } else {
                o = ldf(qr + j);
            }
            qw[j] = o * scale;
        }
    }

    // a sink takes part in the normalisation only: it enters the running (maximum, sum) as a key of score 0 without a value
    float m = sink > 0.f ? 0.f : -INFINITY, l = sink;
    float acc[KR];
#pragma unroll
    for (int k = 0; k < KR; k++) acc[k] = 0.f;

    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    for (int base = lo; base <= pos; base += WA_TILE) {
        __syncthreads();                       // the previous tile is no longer read (and qs is written, first time round)
        const int nkeys = min(WA_TILE, pos - base + 1);
        for (int jj = warp; jj < nkeys; jj += hpb) {
            const int kp = base + jj;
            const T* src = cache + (((int64_t)bt[kp / block_size] * n_slots + slot) * block_size + kp % block_size) * row;
            const T* ks = src + g * dk;
            const T* vs = src + G * dk + g * dv;
            for (int d = lane; d < dk; d += 32) kt[jj * KP + d] = ldf(ks + d);
            for (int d = lane; d < dv; d += 32) vt[jj * dv + d] = ldf(vs + d);
        }
        __syncthreads();
        const float* qw = qs + warp * dk;
        float s = -INFINITY;
        if (lane < nkeys) {
            const float* kr = kt + lane * KP;
            float a = 0.f;
            for (int d = 0; d < dk; d++) a += qw[d] * kr[d];
            s = a;
        }
        const float m_new = fmaxf(m, warp_max(s));          // finite: key `base` is always visible
        const float alpha = expf(m - m_new);                // 0 on the first tile without a sink (m = -inf)
        const float p = lane < nkeys ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(p);
#pragma unroll
        for (int k = 0; k < KR; k++) acc[k] *= alpha;
        for (int jj = 0; jj < nkeys; jj++) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const float* vr = vt + jj * dv;
#pragma unroll
            for (int k = 0; k < KR; k++) {
                const int d = lane + 32 * k;
                if (d < dv) acc[k] += pj * vr[d];
            }
        }
        m = m_new;
    }
    const float denom = l;
    T* o = out + t * out_stride_t + (int64_t)h * dv;
    const T* gr = gate != nullptr ? gate + t * gate_stride_t + (int64_t)h * dv : nullptr;
#pragma unroll
    for (int k = 0; k < KR; k++) {
        const int d = lane + 32 * k;
        if (d < dv) {
            float y = acc[k] / denom;
            if (gr != nullptr) y *= 1.f / (1.f + expf(-ldf(gr + d)));
            stf(o + d, y);
        }
    }
}

static int heads_per_cta(int hq) {
    for (int n = WA_MAX_HPB; n > 1; n--)
        if (hq % n == 0) return n;
    return 1;
}

template <typename T, int KR>
static int launch_window_attn(const void* q, int64_t q_stride_t, const void* cosb, const void* sinb, const void* gate,
                              int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                              const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos, void* out,
                              int64_t out_stride_t, int64_t num_tokens, int H, int G, int dk, int dv, int rot_dims, int window,
                              float scale, float sink, cudaStream_t stream) {
    static unsigned long long attr_mask = 0;
    const int hpb = heads_per_cta(H / G);
    const size_t smem = ((size_t)hpb * dk + (size_t)WA_TILE * (dk + 1) + (size_t)WA_TILE * dv) * sizeof(float);
    SLLM_REQUIRE(smem <= 200 * 1024, "window_attention: head sizes %d / %d need %zu bytes of shared memory", dk, dv, smem);
    auto kern = window_attn_kernel<T, KR>;
    if (first_use_on_this_device(attr_mask))
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    kern<<<dim3((unsigned)num_tokens, (unsigned)(H / hpb)), hpb * 32, smem, stream>>>(
        (const T*)q, q_stride_t, (const float*)cosb, (const float*)sinb, (const T*)gate, gate_stride_t, (const T*)cache, n_slots,
        slot, block_size, (const int*)block_table, max_blocks_per_seq, (const int*)tok_seq, (const int*)tok_pos, (T*)out,
        out_stride_t, H, G, dk, dv, rot_dims, window, scale, sink);
    return check_launch("window_attention");
}

}  // namespace sllm

using namespace sllm;

extern "C" {

int sllm_window_kv_store(const void* k, int64_t k_row_stride, const void* v, int64_t v_row_stride, const void* cosb,
                         const void* sinb, const void* tok_seq, const void* tok_pos, const void* block_table,
                         int max_blocks_per_seq, void* cache, int n_slots, int slot, int block_size, int64_t num_tokens,
                         int num_kv_heads, int dk, int dv, int rot_dims, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && num_kv_heads > 0 && dk > 0 && dv > 0 && rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0,
                 "window_kv_store: bad shape (kv heads %d, dk %d, dv %d, rot_dims %d)", num_kv_heads, dk, dv, rot_dims);
    SLLM_REQUIRE(slot >= 0 && slot < n_slots && block_size > 0, "window_kv_store: bad cache slot %d of %d", slot, n_slots);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(k && v && tok_seq && tok_pos && block_table && cache && (rot_dims == 0 || (cosb && sinb)),
                 "window_kv_store: null pointer");
    SLLM_DISPATCH_DTYPE_F32(dtype, (window_kv_store_kernel<T><<<(unsigned)num_tokens, 128, 0, (cudaStream_t)stream>>>(
        (const T*)k, k_row_stride, (const T*)v, v_row_stride, (const float*)cosb, (const float*)sinb, (const int*)tok_seq,
        (const int*)tok_pos, (const int*)block_table, max_blocks_per_seq, (T*)cache, n_slots, slot, block_size, num_kv_heads,
        dk, dv, rot_dims)));
    return check_launch("window_kv_store");
}

int sllm_window_attention(const void* q, int64_t q_stride_t, const void* cosb, const void* sinb, const void* gate,
                          int64_t gate_stride_t, const void* cache, int n_slots, int slot, int block_size,
                          const void* block_table, int max_blocks_per_seq, const void* tok_seq, const void* tok_pos, void* out,
                          int64_t out_stride_t, int64_t num_tokens, int num_heads, int num_kv_heads, int dk, int dv,
                          int rot_dims, int window, float scale, int sink, sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && dk > 0 && dv > 0 &&
                 dv <= 256 && rot_dims >= 0 && rot_dims <= dk && rot_dims % 2 == 0,
                 "window_attention: bad shape (heads %d / %d, dk %d, dv %d <= 256, rot_dims %d)", num_heads, num_kv_heads, dk,
                 dv, rot_dims);
    SLLM_REQUIRE(slot >= 0 && slot < n_slots && block_size > 0, "window_attention: bad cache slot %d of %d", slot, n_slots);
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(q && tok_seq && tok_pos && block_table && cache && out && (rot_dims == 0 || (cosb && sinb)),
                 "window_attention: null pointer");
    const float sinkw = sink ? 1.f : 0.f;
#define WA_LAUNCH(KR)                                                                                                      \
    SLLM_DISPATCH_DTYPE_F32(dtype, return (launch_window_attn<T, KR>(q, q_stride_t, cosb, sinb, gate, gate_stride_t, cache,   \
        n_slots, slot, block_size, block_table, max_blocks_per_seq, tok_seq, tok_pos, out, out_stride_t, num_tokens,        \
        num_heads, num_kv_heads, dk, dv, rot_dims, window, scale, sinkw, (cudaStream_t)stream)))
    if (dv <= 32) { WA_LAUNCH(1); }
    else if (dv <= 64) { WA_LAUNCH(2); }
    else if (dv <= 128) { WA_LAUNCH(4); }
    else { WA_LAUNCH(8); }
#undef WA_LAUNCH
    return 0;
}

}  // extern "C"
