// Latent ("compressed KV") attention over a paged cache that holds, per token and caching layer, ONE row shared by all heads:
//     [ c (r values: the RMS-normed KV latent) | k_rot (dr values: the rotated key part, rotary already applied) ].
// Keys and values are never expanded: the caller folds the key up-projection into the query (q_lat[h] = W_uk[h]^T q_nope[h])
// and applies the value up-projection to the attention-weighted sum of latents, so per head
//     score(i, j) = (q_lat[i,h] . c[j] + rope(q_rot[i,h]) . k_rot[j]) * scale,   out_lat[i,h] = sum_j softmax_j(score) c[j].
// Every token of the step is a query with its own (block-table row, position): prompt portions and single decoded tokens go
// through the same kernel, so the result for a position does not depend on how its sequence was cut into steps.  A query at
// position p attends to the positions max(0, p - window + 1) .. p (window <= 0: all of 0 .. p).
// Softmax, the norm of the latent and the rotation run in fp32 for every storage type.
#include "mma_helpers.cuh"
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


// ------------------------------------------------------------------ attention, tensor-core path (16-bit storage)
// One CTA per (token, group of 16 heads): the heads are the M dimension of the MMA tiles (all heads share the keys), 8 warps.
// Per tile of LM_KT keys (raw cache rows, cp.async into shared memory, rows past the last visible key zero-filled):
//   S[16, KT]  = Q[16, D] K^T          warp w: key columns 8w..8w+7, mma.m16n8k16 over D (two accumulators: even / odd slices)
//   online softmax in fp32             warp w: heads 2w, 2w+1, two keys per lane; P rounded to 16 bits (l sums the rounded P)
//   O[16, r]  += P[16, KT] K[:, :r]    warp w: latent columns 8(w + 8i).., B fragments by ldmatrix.trans from the same key tile
// Needs r % 16 == 0 and dr % 16 == 0 (16-byte rows for cp.async / ldmatrix) and a tile that fits in shared memory; other shapes and
// float storage take the kernel above.
constexpr int LM_KT = 64;
constexpr int LM_NW = 8;           // warps per CTA = key column tiles per key tile (LM_KT / 8)

template <typename T, int NT>      // NT: latent column tiles (8 wide) per warp, r <= 64 * NT
__global__ void __launch_bounds__(LM_NW * 32) latent_attn_mma_kernel(
    const T* __restrict__ q_lat, int64_t ql_stride_t, int64_t ql_stride_h, const T* __restrict__ q_rot, int64_t qr_stride_t,
    int64_t qr_stride_h, const float* __restrict__ cosb, const float* __restrict__ sinb, const T* __restrict__ gate,
    int64_t gate_stride_t, const T* __restrict__ cache, int n_slots, int slot, int block_size,
    const int* __restrict__ block_table, int max_blocks_per_seq, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, T* __restrict__ out, int64_t out_stride_t, int64_t out_stride_h, int H, int r, int dr,
    int rot_dims, int window, float scale, int nsplit, float* __restrict__ partial) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int D = r + dr, LD = D + 8, LP = LM_KT + 8, LS = LM_KT + 1;
    T* Qs = reinterpret_cast<T*>(smem_raw);                 // [16][LD]
    T* Ks = Qs + 16 * LD;                                   // [KT][LD]
    T* Ps = Ks + LM_KT * LD;                                // [16][LP]
    float* Sf = reinterpret_cast<float*>(Ps + 16 * LP);     // [16][LS]
    float* ms = Sf + 16 * LS;                               // [16] running max
    float* ls = ms + 16;                                    // [16] running sum
    float* al = ls + 16;                                    // [16] rescale factor of the current tile
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
    const int64_t t = blockIdx.x;
    const int h0 = blockIdx.y * 16;
    const int pos = tok_pos[t];
    const int* bt = block_table + (int64_t)tok_seq[t] * max_blocks_per_seq;

    // queries of this head group: [q_lat | rotary(q_rot)], rows past H are zero
    for (int hl = warp; hl < 16; hl += LM_NW) {
        const int h = h0 + hl;
        T* qw = Qs + hl * LD;
        if (h < H) {
            const T* ql = q_lat + t * ql_stride_t + (int64_t)h * ql_stride_h;
            const T* qr = q_rot + t * qr_stride_t + (int64_t)h * qr_stride_h;
            for (int d = lane; d < r; d += 32) qw[d] = ql[d];
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
                stf(qw + r + j, o);
            }
        } else {
            for (int d = lane; d < D; d += 32) stf(qw + d, 0.f);
        }
    }
    if (threadIdx.x < 16) { ms[threadIdx.x] = -INFINITY; ls[threadIdx.x] = 0.f; }

    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; i++) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    const int n_col_tiles = r >> 3;
    const int chunks = D >> 3;             // 16-byte chunks per cache row
    const uint32_t qs_a = smem_u32(Qs), ks_a = smem_u32(Ks), ps_a = smem_u32(Ps);

    // gridDim.z CTAs share the visible keys of a (token, head group): CTA z takes a contiguous run of key tiles and, when
    // nsplit > 1, leaves (unnormalised sum, running max, running sum) in `partial` for latent_attn_combine_kernel
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int tiles = (pos - lo + LM_KT) / LM_KT;
    const int per_split = (tiles + nsplit - 1) / nsplit;
    const int tile_end = min(tiles, ((int)blockIdx.z + 1) * per_split);
    for (int tile = blockIdx.z * per_split; tile < tile_end; tile++) {
        const int base = lo + tile * LM_KT;
        __syncthreads();                   // Ks / Ps of the previous tile are no longer read; Qs and the stats are written
        const int nkeys = min(LM_KT, pos - base + 1);
        {
            // this warp's rows are LM_NW positions apart: walk (block, offset) instead of dividing for every row
            int kb = (base + warp) / block_size, ko = (base + warp) - kb * block_size;
            for (int jj = warp; jj < LM_KT; jj += LM_NW) {
                const bool valid = jj < nkeys;
                const T* src = valid ? cache + (((int64_t)bt[kb] * n_slots + slot) * block_size + ko) * D : cache;
                const uint32_t dst = ks_a + (uint32_t)(jj * LD) * 2u;
                for (int c = lane; c < chunks; c += 32) cp_async16(dst + c * 16, src + c * 8, valid ? 16 : 0);
                ko += LM_NW;
                while (ko >= block_size) { ko -= block_size; kb++; }
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        // ---- S = Q K^T: this warp's key columns 8w..8w+7
        {
            // two accumulators (even / odd 16-wide slices of D): half the length of the dependent MMA chain; one x4 load
            // brings the B fragments of both slices
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, u0[4] = {0.f, 0.f, 0.f, 0.f};
            const int j = lane >> 3;                                              // matrix of the x4 load this lane addresses
            const uint32_t a_addr = qs_a + (uint32_t)((lane & 15) * LD + 8 * (lane >> 4)) * 2u;
            const uint32_t b_row = ks_a + (uint32_t)((8 * warp + (lane & 7)) * LD + 8 * (j & 1)) * 2u;
            int kk = 0;
            for (; kk + 32 <= D; kk += 32) {
                uint32_t a[4], c[4], b0, b1, d0, d1;
                ldmatrix_x4(a_addr + kk * 2, a[0], a[1], a[2], a[3]);
                ldmatrix_x4(a_addr + kk * 2 + 32, c[0], c[1], c[2], c[3]);
                ldmatrix_x4(b_row + kk * 2 + 32 * (j >> 1), b0, b1, d0, d1);
                mma_16816<T>(s0, a, b0, b1);
                mma_16816<T>(u0, c, d0, d1);
            }
            if (kk < D) {
                uint32_t a[4], b0, b1, d0, d1;
                ldmatrix_x4(a_addr + kk * 2, a[0], a[1], a[2], a[3]);
                ldmatrix_x4(b_row + kk * 2, b0, b1, d0, d1);                      // upper two matrices repeat the lower: unused
                mma_16816<T>(s0, a, b0, b1);
            }
            const int c0 = 8 * warp + 2 * tq;
            Sf[g * LS + c0] = s0[0] + u0[0]; Sf[g * LS + c0 + 1] = s0[1] + u0[1];
            Sf[(g + 8) * LS + c0] = s0[2] + u0[2]; Sf[(g + 8) * LS + c0 + 1] = s0[3] + u0[3];
        }
        __syncthreads();

        // ---- online softmax: this warp's heads 2w, 2w+1
        for (int row = 2 * warp; row < 2 * warp + 2; row++) {
            const float x0 = lane < nkeys ? Sf[row * LS + lane] * scale : -INFINITY;
            const float x1 = lane + 32 < nkeys ? Sf[row * LS + lane + 32] * scale : -INFINITY;
            const float m_old = ms[row];
            const float m_new = fmaxf(m_old, warp_max(fmaxf(x0, x1)));            // finite: key `base` is always visible
            const T p0 = Traits<T>::from_f(lane < nkeys ? expf(x0 - m_new) : 0.f);
            const T p1 = Traits<T>::from_f(lane + 32 < nkeys ? expf(x1 - m_new) : 0.f);
            Ps[row * LP + lane] = p0;
            Ps[row * LP + lane + 32] = p1;
            const float sum = warp_sum(Traits<T>::to_f(p0) + Traits<T>::to_f(p1));
            __syncwarp();
            if (lane == 0) {
                const float alpha = expf(m_old - m_new);                          // 0 on the first tile
                ms[row] = m_new; ls[row] = ls[row] * alpha + sum; al[row] = alpha;
            }
        }
        __syncthreads();

        // ---- O = O * alpha + P K[:, :r]: this warp's latent column tiles w, w + 8, ...
        {
            const float a_lo = al[g], a_hi = al[g + 8];
#pragma unroll
            for (int i = 0; i < NT; i++) { acc[i][0] *= a_lo; acc[i][1] *= a_lo; acc[i][2] *= a_hi; acc[i][3] *= a_hi; }
            const int j = lane >> 3;
            const uint32_t a_addr = ps_a + (uint32_t)((lane & 15) * LP + 8 * (lane >> 4)) * 2u;
            for (int ks = 0; ks < LM_KT && ks < nkeys; ks += 16) {
                uint32_t a[4];
                ldmatrix_x4(a_addr + ks * 2, a[0], a[1], a[2], a[3]);
                const uint32_t row_addr = ks_a + (uint32_t)((ks + 8 * (j & 1) + (lane & 7)) * LD) * 2u;
#pragma unroll
                for (int i = 0; i < NT; i += 2) {
                    const int ct0 = warp + LM_NW * i, ct1 = warp + LM_NW * (i + 1);
                    if (ct0 >= n_col_tiles) break;
                    const int ct = (j >> 1) ? (ct1 < n_col_tiles ? ct1 : ct0) : ct0;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(row_addr + ct * 16, b0, b1, b2, b3);
                    mma_16816<T>(acc[i], a, b0, b1);
                    if (ct1 < n_col_tiles) mma_16816<T>(acc[i + 1], a, b2, b3);
                }
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NT; i++) {
        const int ct = warp + LM_NW * i;
        if (ct >= n_col_tiles) break;
#pragma unroll
        for (int half = 0; half < 2; half++) {
            const int hl = g + 8 * half, h = h0 + hl;
            if (h >= H) continue;
            if (nsplit > 1) {
                float* pr = partial + ((t * H + h) * nsplit + blockIdx.z) * (r + 2);
                pr[ct * 8 + 2 * tq] = acc[i][2 * half];
                pr[ct * 8 + 2 * tq + 1] = acc[i][2 * half + 1];
                if (ct == 0 && tq == 0) { pr[r] = ms[hl]; pr[r + 1] = ls[hl]; }
                continue;
            }
            float gt = 1.f;
            if (gate != nullptr) gt = 1.f / (1.f + expf(-ldf(gate + t * gate_stride_t + h)));
            const float f = gt / ls[hl];
            T* o = out + t * out_stride_t + (int64_t)h * out_stride_h + ct * 8 + 2 * tq;
            stf(o, acc[i][2 * half] * f);
            stf(o + 1, acc[i][2 * half + 1] * f);
        }
    }
}

// One warp per (token, head): merge the key splits.  partial [T, H, nsplit, r + 2] = (sum_j e^(s_j - m) c_j, m, sum_j e^(s_j - m));
// a split that saw no key has m = -inf and contributes nothing.
template <typename T>
__global__ void __launch_bounds__(128) latent_attn_combine_kernel(const float* __restrict__ partial, const T* __restrict__ gate,
                                                                  int64_t gate_stride_t, T* __restrict__ out, int64_t out_stride_t,
                                                                  int64_t out_stride_h, int64_t num_tokens, int H, int r, int nsplit) {
    const int lane = threadIdx.x & 31;
    const int64_t idx = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (idx >= num_tokens * H) return;
    const int64_t t = idx / H;
    const int h = (int)(idx - t * H);
    const float* pr = partial + idx * nsplit * (r + 2);
    float M = -INFINITY;
    for (int z = 0; z < nsplit; z++) M = fmaxf(M, pr[z * (r + 2) + r]);
    float L = 0.f;
    for (int z = 0; z < nsplit; z++) L += expf(pr[z * (r + 2) + r] - M) * pr[z * (r + 2) + r + 1];
    float gt = 1.f;
    if (gate != nullptr) gt = 1.f / (1.f + expf(-ldf(gate + t * gate_stride_t + h)));
    T* o = out + t * out_stride_t + (int64_t)h * out_stride_h;
    for (int d = lane; d < r; d += 32) {
        float a = 0.f;
        for (int z = 0; z < nsplit; z++) a += expf(pr[z * (r + 2) + r] - M) * pr[z * (r + 2) + d];
        stf(o + d, a / L * gt);
    }
}

template <typename T, int NT>
static int launch_latent_attn_mma(const void* q_lat, int64_t ql_st, int64_t ql_sh, const void* q_rot, int64_t qr_st, int64_t qr_sh,
                                  const void* cosb, const void* sinb, const void* gate, int64_t gate_st, const void* cache,
                                  int n_slots, int slot, int block_size, const void* block_table, int max_blocks_per_seq,
                                  const void* tok_seq, const void* tok_pos, void* out, int64_t out_st, int64_t out_sh,
                                  int64_t num_tokens, int H, int r, int dr, int rot_dims, int window, float scale,
                                  cudaStream_t stream, int nsplit, void* partial) {
    const int D = r + dr;
    const size_t smem = ((size_t)(16 + LM_KT) * (D + 8) + 16 * (LM_KT + 8)) * 2 + (16 * (LM_KT + 1) + 48) * sizeof(float);
    SLLM_REQUIRE(smem <= 200 * 1024, "latent_attention: r + dr = %d needs %zu bytes of shared memory", D, smem);
    static unsigned long long configured = 0;
    auto kern = latent_attn_mma_kernel<T, NT>;
    if (first_use_on_this_device(configured)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        SLLM_REQUIRE(e == cudaSuccess, "latent_attention: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    }
    dim3 grid((unsigned)num_tokens, (unsigned)cdiv(H, 16), (unsigned)nsplit);
    kern<<<grid, LM_NW * 32, smem, stream>>>(
        (const T*)q_lat, ql_st, ql_sh, (const T*)q_rot, qr_st, qr_sh, (const float*)cosb, (const float*)sinb, (const T*)gate,
        gate_st, (const T*)cache, n_slots, slot, block_size, (const int*)block_table, max_blocks_per_seq, (const int*)tok_seq,
        (const int*)tok_pos, (T*)out, out_st, out_sh, H, r, dr, rot_dims, window, scale, nsplit, (float*)partial);
    if (int rc = check_launch("latent_attention (mma)")) return rc;
    if (nsplit > 1) {
        latent_attn_combine_kernel<T><<<(unsigned)cdiv(num_tokens * H, 4), 128, 0, stream>>>(
            (const float*)partial, (const T*)gate, gate_st, (T*)out, out_st, out_sh, num_tokens, H, r, nsplit);
        return check_launch("latent_attention (combine)");
    }
    return 0;
}

template <typename T> struct LatentMma {
    template <typename... A> static int run(int r, A... a) {
        if (r <= 128) return launch_latent_attn_mma<T, 2>(a...);
        if (r <= 256) return launch_latent_attn_mma<T, 4>(a...);
        if (r <= 512) return launch_latent_attn_mma<T, 8>(a...);
        return launch_latent_attn_mma<T, 16>(a...);
    }
};
template <> struct LatentMma<float> {
    template <typename... A> static int run(int, A...) { set_error("latent_attention: no tensor-core path for float storage"); return 1; }
};

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

// tests and A/B timing: 1 = always take the CUDA-core kernel (process-wide; set through sllm_latent_attention_set_simt)
static int sllm_latent_attention_force_simt = 0;

extern "C" {

int sllm_latent_attention_set_simt(int on) {
    const int old = sllm_latent_attention_force_simt;
    sllm_latent_attention_force_simt = on ? 1 : 0;
    return old;
}

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
                          int dr, int rot_dims, int window, float scale, int num_splits, void* split_workspace,
                          sllm_dtype_t dtype, sllm_stream_t stream) {
    SLLM_REQUIRE(num_tokens >= 0 && num_heads > 0 && r > 0 && r <= 1024 && dr >= 0 && rot_dims >= 0 && rot_dims <= dr &&
                 rot_dims % 2 == 0, "latent_attention: bad shape (heads %d, r %d <= 1024, dr %d, rot_dims %d)", num_heads, r, dr,
                 rot_dims);
    SLLM_REQUIRE(n_slots > 0 && slot >= 0 && slot < n_slots && block_size > 0 && max_blocks_per_seq > 0,
                 "latent_attention: bad cache geometry");
    if (num_tokens == 0) return 0;
    SLLM_REQUIRE(q_lat && (dr == 0 || q_rot) && cache && block_table && tok_seq && tok_pos && out &&
                 (rot_dims == 0 || (cosb && sinb)), "latent_attention: null pointer");
#define SLLM_LA_ARGS q_lat, q_lat_stride_t, q_lat_stride_h, q_rot, q_rot_stride_t, q_rot_stride_h, cosb, sinb, gate,            \
                     gate_stride_t, cache, n_slots, slot, block_size, block_table, max_blocks_per_seq, tok_seq, tok_pos, out,   \
                     out_stride_t, out_stride_h, num_tokens, num_heads, r, dr, rot_dims, window, scale, (cudaStream_t)stream
    // 16-bit storage and 16-element-aligned rows: tensor cores; everything else: the fp32 CUDA-core kernel
    const size_t mma_smem = ((size_t)(16 + LM_KT) * (r + dr + 8) + 16 * (LM_KT + 8)) * 2 + (16 * (LM_KT + 1) + 48) * sizeof(float);
    const bool mma = dtype != SLLM_F32 && r % 16 == 0 && dr % 16 == 0 && mma_smem <= 200 * 1024 && !sllm_latent_attention_force_simt;
    if (mma) {
        const int nsplit = (num_splits > 1 && split_workspace != nullptr) ? (num_splits > 64 ? 64 : num_splits) : 1;
        SLLM_DISPATCH_DTYPE_F32(dtype, return (LatentMma<T>::run(r, SLLM_LA_ARGS, nsplit, split_workspace)));
    }
    SLLM_DISPATCH_DTYPE_F32(dtype, {
        if (r <= 64) return (launch_latent_attn<T, 2>(SLLM_LA_ARGS));
        if (r <= 128) return (launch_latent_attn<T, 4>(SLLM_LA_ARGS));
        if (r <= 256) return (launch_latent_attn<T, 8>(SLLM_LA_ARGS));
        if (r <= 512) return (launch_latent_attn<T, 16>(SLLM_LA_ARGS));
        return (launch_latent_attn<T, 32>(SLLM_LA_ARGS));
    });
#undef SLLM_LA_ARGS
    return 0;
}

}  // extern "C"
