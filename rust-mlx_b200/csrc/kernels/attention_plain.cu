// Attention over the paged cache on the FMA units, one warp per (token, query head).
//
// This kernel serves the 32-bit path for prompts and decoding alike, and is the
// fallback of the bfloat16 path.  A query at position p reads keys lo .. p, lo = 0 or
// p - window + 1, through its request's block table.  Keys are visited in blocks of 32
// aligned to absolute positions (block b holds positions 32b .. 32b+31) in ascending
// order, with an online softmax in float.  The order in which numbers are added
// depends on p (and the window) only: not on how the prompt was cut into steps, on the
// other tokens of the batch, on the page size or on which pages hold the keys.
//
// Grid: (tokens, kv heads); a block has one warp per query head of the group, so the
// group's warps read the same keys from shared memory.
#include "common.cuh"

namespace {
constexpr int KB = 32;  // keys per block

template <typename T>
__global__ void attention_plain_kernel(const T* __restrict__ q, const T* __restrict__ k_pool,
                                       const T* __restrict__ v_pool, const int* __restrict__ positions,
                                       const int* __restrict__ seq_index, const int* __restrict__ block_table,
                                       int table_stride, int page_size, T* __restrict__ out, int nq, int nkv,
                                       int hd, int window, float scale, int* __restrict__ status) {
    extern __shared__ float smem[];
    const int group = nq / nkv;
    const int t = blockIdx.x, kvh = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = kvh * group + warp;
    const int kstride = hd + 1;
    float* Ks = smem;                          // [KB][hd + 1]
    float* Vs = Ks + KB * kstride;             // [KB][hd]
    float* Qs = Vs + KB * hd;                  // [group][hd]
    const int pos = positions[t];
    const int* table = block_table + (size_t)seq_index[t] * table_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;

    for (int d = lane; d < hd; d += 32) Qs[warp * hd + d] = to_float(q[((size_t)t * nq + head) * hd + d]) * scale;

    const int per_lane = (hd + 31) / 32;
    float acc[16];  // head_dim up to 512
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int b = lo / KB; b <= pos / KB; ++b) {
        const int base = b * KB;
        __syncthreads();
        for (int idx = threadIdx.x; idx < KB * hd; idx += blockDim.x) {
            const int j = idx / hd, d = idx - j * hd;
            const int kp = base + j;
            float kv = 0.f, vv = 0.f;
            if (kp >= lo && kp <= pos) {
                const int page = table[kp / page_size];
                if (page >= 0) {
                    const size_t off = (((size_t)page * nkv + kvh) * page_size + kp % page_size) * hd + d;
                    kv = to_float(k_pool[off]);
                    vv = to_float(v_pool[off]);
                } else if (d == 0) {
                    atomicExch(status, 2);  // a key that should be there has no page
                }
            }
            Ks[j * kstride + d] = kv;
            Vs[j * hd + d] = vv;
        }
        __syncthreads();
        const int kp = base + lane;
        const bool valid = kp >= lo && kp <= pos;
        float s = 0.f;
        const float* qrow = Qs + warp * hd;
        const float* krow = Ks + lane * kstride;
        for (int d = 0; d < hd; ++d) s = fmaf(qrow[d], krow[d], s);
        s = valid ? s : -INFINITY;
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = expf(m - m_new);  // first block: exp(-inf) = 0
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int i = 0; i < 16; ++i) acc[i] *= corr;
        for (int j = 0; j < KB; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int d = lane + 32 * i;
                if (i < per_lane && d < hd) acc[i] = fmaf(pj, Vs[j * hd + d], acc[i]);
            }
        }
    }
    const float inv_l = 1.f / l;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const int d = lane + 32 * i;
        if (i < per_lane && d < hd) out[((size_t)t * nq + head) * hd + d] = from_float<T>(acc[i] * inv_l);
    }
}
}  // namespace

RMX_API int rmx_attention_plain(const void* q, const void* k_pool, const void* v_pool, const int* positions,
                                const int* seq_index, const int* block_table, int table_stride, int page_size,
                                void* out, int n_tokens, int nq, int nkv, int hd, int window, float scale,
                                int* status, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_plain: %d query heads over %d kv heads", nq, nkv);
    const int group = nq / nkv;
    RMX_REQUIRE(group <= 32, "attention_plain: more than 32 query heads per kv head (%d)", group);
    RMX_REQUIRE(hd > 0 && hd <= 512, "attention_plain: head_dim %d must be in 1..512", hd);
    RMX_REQUIRE(page_size > 0 && table_stride > 0 && window >= 0, "attention_plain: bad page geometry");
    RMX_REQUIRE(nkv <= 65535, "attention_plain: too many kv heads");
    const size_t smem = ((size_t)KB * (hd + 1) + (size_t)KB * hd + (size_t)group * hd) * sizeof(float);
    RMX_REQUIRE(smem <= 200 * 1024, "attention_plain: head_dim %d with group %d needs too much shared memory", hd, group);
    dim3 grid(n_tokens, nkv);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_plain_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_plain_kernel<float><<<grid, group * 32, smem, s>>>(
            (const float*)q, (const float*)k_pool, (const float*)v_pool, positions, seq_index, block_table, table_stride,
            page_size, (float*)out, nq, nkv, hd, window, scale, status);
    } else if (dtype == RMX_BF16) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(attention_plain_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attention_plain_kernel<__nv_bfloat16><<<grid, group * 32, smem, s>>>(
            (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, positions, seq_index,
            block_table, table_stride, page_size, (__nv_bfloat16*)out, nq, nkv, hd, window, scale, status);
    } else {
        RMX_FAIL("attention_plain: unknown dtype %d", dtype);
    }
    RMX_CHECK_LAUNCH("attention_plain");
    return 0;
}
