// Per-head RMSNorm of q and k, rotation, and the write of keys and values into pages.
//
// Input is the fused projection row [q heads | k heads | v heads] of every token.  One
// warp takes one (token, head):
//   q head: q = RMSNorm(q; q_norm, eps) -> rotate -> q_out[token, head, :]
//   k head: k = RMSNorm(k; k_norm, eps) -> rotate -> k_pool[page, kv head, slot, :]
//   v head: copy                                   -> v_pool[page, kv head, slot, :]
// with page = block_table[seq, pos / page_size], slot = pos % page_size.
// Rotation (half-split): for j < rotary_dim / 2, angle = pos * inv_freq[j] in float,
//   out[j] = x[j] cos - x[j + half] sin, out[j + half] = x[j + half] cos + x[j] sin;
// numbers from rotary_dim on pass through.  Norm weights are float; either may be null
// (no norm).  With write_kv == 0 only q is produced (a layer that reads another layer's
// cache).  Everything is computed in float and rounded once to T.
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 512;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) qk_rope_cache_kernel(
    const T* __restrict__ qkv, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ inv_freq, int rotary_dim, const int* __restrict__ positions,
    const int* __restrict__ seq_index, const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, T* __restrict__ q_out, int n_tokens, int nq, int nkv, int hd,
    int row_stride, int write_kv, int* __restrict__ status) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * heads_total) return;
    const int t = (int)(item / heads_total);
    const int head = (int)(item % heads_total);
    float* buf = smem + warp * hd;
    const T* src = qkv + (size_t)t * row_stride + (size_t)head * hd;

    const int pos = positions[t];
    T* dst;
    const float* norm_w;
    bool rotate = true;
    if (head < nq) {
        dst = q_out + ((size_t)t * nq + head) * hd;
        norm_w = q_norm;
    } else {
        const int kvh = (head - nq) % nkv;
        const bool is_v = head >= nq + nkv;
        const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
        if (page < 0) {  // the host reserves pages before the step; never write through a hole
            if (lane == 0) atomicExch(status, 1);
            return;
        }
        const size_t off = (((size_t)page * nkv + kvh) * page_size + pos % page_size) * hd;
        dst = (is_v ? v_pool : k_pool) + off;
        norm_w = is_v ? nullptr : k_norm;
        rotate = !is_v;
    }

    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) {
        const float v = to_float(src[d]);
        buf[d] = v;
        ss += v * v;
    }
    if (norm_w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)hd + eps);
        __syncwarp();
        for (int d = lane; d < hd; d += 32) buf[d] = buf[d] * inv * norm_w[d];
    }
    __syncwarp();
    const int half = rotary_dim >> 1;
    if (rotate && half > 0) {
        for (int j = lane; j < half; j += 32) {
            const float angle = (float)pos * inv_freq[j];
            float sn, cs;
            sincosf(angle, &sn, &cs);
            const float a = buf[j], b = buf[j + half];
            dst[j] = from_float<T>(a * cs - b * sn);
            dst[j + half] = from_float<T>(b * cs + a * sn);
        }
        for (int d = rotary_dim + lane; d < hd; d += 32) dst[d] = from_float<T>(buf[d]);
    } else {
        for (int d = lane; d < hd; d += 32) dst[d] = from_float<T>(buf[d]);
    }
}
}  // namespace

RMX_API int rmx_qk_rope_cache(const void* qkv, const float* q_norm, const float* k_norm, float eps,
                              const float* inv_freq, int rotary_dim, const int* positions, const int* seq_index,
                              const int* block_table, int table_stride, int page_size, void* k_pool, void* v_pool,
                              void* q_out, int n_tokens, int nq, int nkv, int hd, int row_stride, int write_kv,
                              int* status, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && hd > 0 && hd <= MAX_HD, "qk_rope_cache: head_dim %d must be in 1..%d", hd, MAX_HD);
    RMX_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
                "qk_rope_cache: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    RMX_REQUIRE(page_size > 0 && table_stride > 0, "qk_rope_cache: bad page geometry");
    RMX_REQUIRE(row_stride >= (nq + (write_kv ? 2 * nkv : 0)) * hd, "qk_rope_cache: row stride %d too small", row_stride);
    RMX_REQUIRE(rotary_dim == 0 || inv_freq != nullptr, "qk_rope_cache: rotation without a table");
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const long long items = (long long)n_tokens * heads_total;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * hd * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        qk_rope_cache_kernel<float><<<blocks, WARPS * 32, smem, s>>>(
            (const float*)qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table,
            table_stride, page_size, (float*)k_pool, (float*)v_pool, (float*)q_out, n_tokens, nq, nkv, hd, row_stride, write_kv, status);
    else if (dtype == RMX_BF16)
        qk_rope_cache_kernel<__nv_bfloat16><<<blocks, WARPS * 32, smem, s>>>(
            (const __nv_bfloat16*)qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table,
            table_stride, page_size, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens,
            nq, nkv, hd, row_stride, write_kv, status);
    else
        RMX_FAIL("qk_rope_cache: unknown dtype %d", dtype);
    RMX_CHECK_LAUNCH("qk_rope_cache");
    return 0;
}
