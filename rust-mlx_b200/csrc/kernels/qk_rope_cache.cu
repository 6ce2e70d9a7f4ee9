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
//
// The cosines and sines of a step's positions are the same for every head and every layer:
// rope_table_kernel forms them once per step ([token][cos of j | sin of j], float, with the same
// float product and the same sincosf), and the kernels here read them when the table is given.
#include "common.cuh"
#include "rope128.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 512;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32) qk_rope_cache_kernel(
    const T* __restrict__ qkv, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ inv_freq, int rotary_dim, const int* __restrict__ positions,
    const int* __restrict__ seq_index, const int* __restrict__ block_table, int table_stride, int page_size,
    T* __restrict__ k_pool, T* __restrict__ v_pool, T* __restrict__ q_out, int n_tokens, int nq, int nkv, int hd,
    int row_stride, int write_kv, int* __restrict__ status, const float* __restrict__ cos_sin) {
    extern __shared__ float smem[];
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
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
            float sn, cs;
            if (cos_sin) {
                cs = cos_sin[(size_t)t * rotary_dim + j];
                sn = cos_sin[(size_t)t * rotary_dim + half + j];
            } else {
                sincosf((float)pos * inv_freq[j], &sn, &cs);
            }
            const float a = buf[j], b = buf[j + half];
            dst[j] = from_float<T>(a * cs - b * sn);
            dst[j + half] = from_float<T>(b * cs + a * sn);
        }
        for (int d = rotary_dim + lane; d < hd; d += 32) dst[d] = from_float<T>(buf[d]);
    } else {
        for (int d = lane; d < hd; d += 32) dst[d] = from_float<T>(buf[d]);
    }
}

// cos_sin[t][j] = cos(pos_t * inv_freq[j]), cos_sin[t][half + j] = sin(...): once per step.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_sin, int n_tokens, int half) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n_tokens * half) return;
    const int t = idx / half, j = idx - t * half;
    float sn, cs;
    sincosf((float)positions[t] * inv_freq[j], &sn, &cs);
    cos_sin[(size_t)t * 2 * half + j] = cs;
    cos_sin[(size_t)t * 2 * half + half + j] = sn;
}

// bfloat16, head size 128, all 128 numbers rotated, table given: a lane holds four neighbouring numbers of the
// head; the partner of number j is j + 64, sixteen lanes away.  A warp takes PER_WARP (token, head) items and
// issues all their loads before it works on the first, so that their latencies overlap.
constexpr int PER_WARP = 4;

__global__ void __launch_bounds__(WARPS * 32) qk_rope_cache_128_kernel(
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ cos_sin, const int* __restrict__ positions, const int* __restrict__ seq_index,
    const int* __restrict__ block_table, int table_stride, int page_size, __nv_bfloat16* __restrict__ k_pool,
    __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ q_out, int n_tokens, int nq, int nkv, int row_stride,
    int write_kv, int* __restrict__ status) {
    constexpr int hd = 128;
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const int total = n_tokens * heads_total;   // the launcher keeps this below 2^31
    const int first = (blockIdx.x * WARPS + warp) * PER_WARP;
    if (first >= total) return;
    uint2 raw[PER_WARP];
    __nv_bfloat16* dst[PER_WARP];
    const float* norm_w[PER_WARP];
    int tok[PER_WARP];
    bool rotate[PER_WARP], live[PER_WARP];
#pragma unroll
    for (int u = 0; u < PER_WARP; ++u) {
        const int item = first + u;
        live[u] = item < total;
        const int t = live[u] ? item / heads_total : 0;
        const int head = live[u] ? item - t * heads_total : 0;
        tok[u] = t;
        raw[u] = *reinterpret_cast<const uint2*>(qkv + (size_t)t * row_stride + (size_t)head * hd + lane * 4);
        rotate[u] = true;
        if (head < nq) {
            dst[u] = q_out + ((size_t)t * nq + head) * hd;
            norm_w[u] = q_norm;
        } else {
            const int pos = positions[t];
            const int kvh = (head - nq) % nkv;
            const bool is_v = head >= nq + nkv;
            const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
            if (page < 0) {  // the host reserves pages before the step; never write through a hole
                if (lane == 0 && live[u]) atomicExch(status, 1);
                live[u] = false;
            }
            dst[u] = (is_v ? v_pool : k_pool) + (((size_t)(page < 0 ? 0 : page) * nkv + kvh) * page_size + pos % page_size) * hd;
            norm_w[u] = is_v ? nullptr : k_norm;
            rotate[u] = !is_v;
        }
    }
#pragma unroll
    for (int u = 0; u < PER_WARP; ++u) {
        if (!live[u]) continue;
        if (!rotate[u]) {  // values pass through
            *reinterpret_cast<uint2*>(dst[u] + lane * 4) = raw[u];
            continue;
        }
        const uint2 packed = rope128_head(raw[u], norm_w[u], eps, cos_sin + (size_t)tok[u] * hd, lane);
        *reinterpret_cast<uint2*>(dst[u] + lane * 4) = packed;
    }
}
// The same for many tokens (prompt portions): a warp takes one token and HEADS_PER_WARP neighbouring heads of it,
// two heads a pass (sixteen lanes a head, eight neighbouring numbers a lane, 16-byte loads and stores; the partner
// of number j is j + 64, eight lanes away).  The token's position, page and its cosines and sines are read once a
// warp, and all loads of the warp's heads are under way before the first is worked on.
constexpr int HEADS_PER_WARP = 8;

__global__ void __launch_bounds__(WARPS * 32, 8) qk_rope_cache_128_wide_kernel(
    const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_norm, const float* __restrict__ k_norm, float eps,
    const float* __restrict__ cos_sin, const int* __restrict__ positions, const int* __restrict__ seq_index,
    const int* __restrict__ block_table, int table_stride, int page_size, __nv_bfloat16* __restrict__ k_pool,
    __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ q_out, int n_tokens, int nq, int nkv, int row_stride,
    int write_kv, int* __restrict__ status) {
    constexpr int hd = 128, PASSES = HEADS_PER_WARP / 2;
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const int groups = (heads_total + HEADS_PER_WARP - 1) / HEADS_PER_WARP;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)n_tokens * groups) return;
    const int t = (int)(item / groups), head0 = (int)(item - (long long)t * groups) * HEADS_PER_WARP;
    const int sub = lane >> 4, l16 = lane & 15;       // which of the pass's two heads, and where in it
    const __nv_bfloat16* src = qkv + (size_t)t * row_stride + l16 * 8;
    uint4 raw[PASSES];
#pragma unroll
    for (int u = 0; u < PASSES; ++u) {
        const int head = head0 + 2 * u + sub;
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (head < heads_total) raw[u] = *reinterpret_cast<const uint4*>(src + (size_t)head * hd);
    }
    // cosines and sines of the pairs (j, j + 64) that this lane's eight numbers belong to
    const int j = (l16 & 7) * 8;
    float cs[8], sn[8];
    {
        const float4 c0 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + j);
        const float4 c1 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + j + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + 64 + j);
        const float4 s1 = *reinterpret_cast<const float4*>(cos_sin + (size_t)t * hd + 64 + j + 4);
        cs[0] = c0.x; cs[1] = c0.y; cs[2] = c0.z; cs[3] = c0.w; cs[4] = c1.x; cs[5] = c1.y; cs[6] = c1.z; cs[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
    long long slot_row = -1;   // the row of the pools' [pages * nkv * page_size] rows that kv head 0 of this token has
    if (head0 + HEADS_PER_WARP > nq && write_kv) {
        const int pos = positions[t];
        const int page = block_table[(size_t)seq_index[t] * table_stride + pos / page_size];
        if (page < 0) {  // the host reserves pages before the step; never write through a hole
            if (lane == 0) atomicExch(status, 1);
        } else {
            slot_row = (long long)page * nkv * page_size + pos % page_size;
        }
    }
#pragma unroll
    for (int u = 0; u < PASSES; ++u) {
        const int head = head0 + 2 * u + sub;
        const bool live = head < heads_total;
        const bool is_q = head < nq, is_v = head >= nq + nkv;
        __nv_bfloat16* dst = nullptr;
        if (live) {
            if (is_q) dst = q_out + ((size_t)t * nq + head) * hd + l16 * 8;
            else if (slot_row >= 0)
                dst = (is_v ? v_pool : k_pool) + (size_t)(slot_row + (long long)((head - nq) % nkv) * page_size) * hd + l16 * 8;
        }
        const uint32_t rw[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&rw[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
        // every lane takes part in the shuffles, whatever its head is
        const bool normed = live && !is_v && (is_q ? q_norm != nullptr : k_norm != nullptr);
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (normed) {
            const float inv = rsqrtf(ss / (float)hd + eps);
            const float* w = (is_q ? q_norm : k_norm) + l16 * 8;   // (the same 512 bytes for every warp: they stay in L1)
            const float4 a = *reinterpret_cast<const float4*>(w), b = *reinterpret_cast<const float4*>(w + 4);
            v[0] = v[0] * inv * a.x; v[1] = v[1] * inv * a.y; v[2] = v[2] * inv * a.z; v[3] = v[3] * inv * a.w;
            v[4] = v[4] * inv * b.x; v[5] = v[5] * inv * b.y; v[6] = v[6] * inv * b.z; v[7] = v[7] * inv * b.w;
        }
        float out[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 8);
            // lanes 0..7 of a head hold x[j] (partner x[j + 64] eight lanes on): out = a cos - b sin
            // lanes 8..15 hold x[j + 64] (partner x[j]):                          out = b cos + a sin
            out[i] = is_v ? v[i] : (l16 < 8 ? v[i] * cs[i] - other * sn[i] : v[i] * cs[i] + other * sn[i]);
        }
        if (dst) {
            if (is_v) {
                *reinterpret_cast<uint4*>(dst) = raw[u];   // values pass through
            } else {
                uint32_t ow[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    __nv_bfloat162 r = __floats2bfloat162_rn(out[2 * i], out[2 * i + 1]);
                    ow[i] = *reinterpret_cast<uint32_t*>(&r);
                }
                *reinterpret_cast<uint4*>(dst) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
            }
        }
    }
}
}  // namespace

RMX_API int rmx_rope_table(const int* positions, const float* inv_freq, float* cos_sin, int n_tokens, int rotary_dim,
                           void* stream) {
    if (n_tokens == 0 || rotary_dim == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && rotary_dim > 0 && rotary_dim % 2 == 0, "rope_table: bad sizes");
    const int half = rotary_dim / 2, total = n_tokens * half;
    RMX_CHECK_LAUNCHED(launch_dependent(rope_table_kernel, dim3((total + 255) / 256), dim3(256), 0, (cudaStream_t)stream, positions,
                                        inv_freq, cos_sin, n_tokens, half), "rope_table");
    return 0;
}

RMX_API int rmx_qk_rope_cache(const void* qkv, const float* q_norm, const float* k_norm, float eps,
                              const float* inv_freq, int rotary_dim, const int* positions, const int* seq_index,
                              const int* block_table, int table_stride, int page_size, void* k_pool, void* v_pool,
                              void* q_out, int n_tokens, int nq, int nkv, int hd, int row_stride, int write_kv,
                              int* status, const float* cos_sin, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && hd > 0 && hd <= MAX_HD, "qk_rope_cache: head_dim %d must be in 1..%d", hd, MAX_HD);
    RMX_REQUIRE(rotary_dim >= 0 && rotary_dim <= hd && rotary_dim % 2 == 0,
                "qk_rope_cache: rotary_dim %d must be even and at most head_dim %d", rotary_dim, hd);
    RMX_REQUIRE(page_size > 0 && table_stride > 0, "qk_rope_cache: bad page geometry");
    RMX_REQUIRE(row_stride >= (nq + (write_kv ? 2 * nkv : 0)) * hd, "qk_rope_cache: row stride %d too small", row_stride);
    RMX_REQUIRE(rotary_dim == 0 || inv_freq != nullptr || cos_sin != nullptr, "qk_rope_cache: rotation without a table");
    const int heads_total = nq + (write_kv ? 2 * nkv : 0);
    const long long items = (long long)n_tokens * heads_total;
    const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
    const size_t smem = (size_t)WARPS * hd * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_BF16 && hd == 128 && rotary_dim == 128 && cos_sin != nullptr && row_stride % 4 == 0 &&
        ((uintptr_t)qkv & 7) == 0 && items < (1LL << 30)) {
        if (n_tokens >= 256 && row_stride % 8 == 0 && ((uintptr_t)qkv & 15) == 0) {   // prompt portions
            const long long warps = (long long)n_tokens * ((heads_total + HEADS_PER_WARP - 1) / HEADS_PER_WARP);
            RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_128_wide_kernel, dim3((unsigned)((warps + WARPS - 1) / WARPS)), dim3(WARPS * 32), 0, s,
                (const __nv_bfloat16*)qkv, q_norm, k_norm, eps, cos_sin, positions, seq_index, block_table, table_stride, page_size,
                (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens, nq, nkv, row_stride, write_kv, status),
                "qk_rope_cache_128_wide");
            return 0;
        }
        const unsigned blocks128 = (unsigned)((items + (long long)WARPS * PER_WARP - 1) / (WARPS * PER_WARP));
        RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_128_kernel, dim3(blocks128), dim3(WARPS * 32), 0, s,
            (const __nv_bfloat16*)qkv, q_norm, k_norm, eps, cos_sin, positions, seq_index, block_table, table_stride, page_size,
            (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens, nq, nkv, row_stride, write_kv, status),
            "qk_rope_cache_128");
        return 0;
    }
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_kernel<float>, dim3(blocks), dim3(WARPS * 32), smem, s,
            (const float*)qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table,
            table_stride, page_size, (float*)k_pool, (float*)v_pool, (float*)q_out, n_tokens, nq, nkv, hd, row_stride, write_kv, status, cos_sin), "qk_rope_cache");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(qk_rope_cache_kernel<__nv_bfloat16>, dim3(blocks), dim3(WARPS * 32), smem, s,
            (const __nv_bfloat16*)qkv, q_norm, k_norm, eps, inv_freq, rotary_dim, positions, seq_index, block_table,
            table_stride, page_size, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool, (__nv_bfloat16*)q_out, n_tokens,
            nq, nkv, hd, row_stride, write_kv, status, cos_sin), "qk_rope_cache");
    else
        RMX_FAIL("qk_rope_cache: unknown dtype %d", dtype);
    RMX_CHECK_LAUNCH("qk_rope_cache");
    return 0;
}
