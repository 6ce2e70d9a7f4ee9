// Embedding gather, residual add + RMSNorm, and SwiGLU.
//
// The residual stream is float32 in every run; activations that kernels hand to one
// another are in the compute type T (float or bfloat16).  Sums of squares, rsqrt and the
// scaling are done in float and rounded once.
#include <type_traits>

#include "common.cuh"

// Four consecutive numbers as floats (the address is 16-byte aligned for float, 8 for bfloat16).
__device__ __forceinline__ void load4(const float* p, float4& v) { v = *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float4& v) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    v = make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, const float4& v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float4& v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a);
    raw.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}
// Threads of a block that takes one row: four numbers per thread, a whole number of warps.
static inline int block_threads(int width) {
    int t = ((width + 3) / 4 + 31) / 32 * 32;
    return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

// h[t, :] = table[ids[t], :] as float.  An id outside the table writes zeros (the host
// rejects such ids before the step; the kernel never reads outside the table).
// from_last (or null): where from_last[t] != 0 the token's id is not ids[t] but the one the last step's sampling
// left for the token's sequence, last_tokens[slots[seq_index[t]]] (the host launched this step before it read it).
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ h, int width, int vocab, const int* __restrict__ from_last,
                                 const int* __restrict__ seq_index, const int* __restrict__ slots,
                                 const int* __restrict__ last_tokens) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int t = blockIdx.x;
    const int id = (from_last && from_last[t]) ? last_tokens[slots[seq_index[t]]] : ids[t];
    const bool ok = id >= 0 && id < vocab;
    const T* row = table + (size_t)(ok ? id : 0) * width;
    float* out = h + (size_t)t * width;
    if ((width & 3) == 0) {  // four numbers per thread and pass
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (ok) load4(row + i, v);
            *reinterpret_cast<float4*>(out + i) = v;
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) out[i] = ok ? to_float(row[i]) : 0.f;
    }
}

RMX_API int rmx_embedding(const int* ids, const void* table, float* h, int n_tokens, int width, int vocab,
                          const int* from_last, const int* seq_index, const int* slots, const int* last_tokens,
                          int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && width > 0 && vocab > 0, "embedding: bad sizes");
    RMX_REQUIRE(from_last == nullptr || (seq_index && slots && last_tokens), "embedding: from_last needs seq_index, slots and last_tokens");
    const int threads = block_threads(width);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, s, ids, (const float*)table, h, width,
                                            vocab, from_last, seq_index, slots, last_tokens), "embedding");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(embedding_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, s, ids,
                                            (const __nv_bfloat16*)table, h, width, vocab, from_last, seq_index, slots, last_tokens), "embedding");
    else
        RMX_FAIL("embedding: unknown dtype %d", dtype);
    RMX_CHECK_LAUNCH("embedding");
    return 0;
}

// One block per output row.  src_row = rows ? rows[r] : r.
//   v = h[src_row] + delta[src_row]          (float; delta may be null)
//   if (write_h) h[src_row] = v
//   x[r] = v * rsqrt(mean(v^2) + eps) * w     (rounded once to T)
// The reduction order depends on the width and the block size only.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                   const int* __restrict__ rows, const float* __restrict__ w, float eps,
                                   T* __restrict__ x, int width, int write_h) {
    __shared__ float scratch[32];
    extern __shared__ __align__(16) float vals[];
    // what follows (a product) may take its place and fetch its weights now: it waits for this kernel, and so for the
    // one before it, before it touches what they write
    allow_dependents();
    wait_for_prior_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * width;
    const T* drow = delta ? delta + (size_t)src * width : nullptr;
    T* xrow = x + (size_t)r * width;
    float ss = 0.f;
    if ((width & 3) == 0) {
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(hrow + i);
            if (drow) {
                float4 d;
                load4(drow + i, d);
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            }
            *reinterpret_cast<float4*>(vals + i) = v;
            if (write_h) *reinterpret_cast<float4*>(hrow + i) = v;
            ss += v.x * v.x;
            ss += v.y * v.y;
            ss += v.z * v.z;
            ss += v.w * v.w;
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
        for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(vals + i);
            const float4 g = *reinterpret_cast<const float4*>(w + i);
            store4(xrow + i, make_float4(v.x * inv * g.x, v.y * inv * g.y, v.z * inv * g.z, v.w * inv * g.w));
        }
    } else {
        for (int i = threadIdx.x; i < width; i += blockDim.x) {
            float v = hrow[i];
            if (drow) v += to_float(drow[i]);
            vals[i] = v;
            if (write_h) hrow[i] = v;
            ss += v * v;
        }
        const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
        for (int i = threadIdx.x; i < width; i += blockDim.x) xrow[i] = from_float<T>(vals[i] * inv * w[i]);
    }
}

// The same for rows of up to CHUNKS * 4 * blockDim numbers (a multiple of 4): every thread keeps its CHUNKS groups
// of four in registers, all their loads under way at once, and the blocks are small enough for several to share an
// SM.  The reduction order depends on the width and the block size only, as above.
template <typename T, int CHUNKS>
__global__ void add_rmsnorm_rows_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                        const int* __restrict__ rows, const float* __restrict__ w, float eps,
                                        T* __restrict__ x, int width, int write_h) {
    __shared__ float scratch[32];
    // the norm's weight does not come from the kernel before this one: it is fetched before the wait for it
    float4 g[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        g[c] = i < width ? *reinterpret_cast<const float4*>(w + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    // what follows (a product) may take its place and fetch its weights now: it waits for this kernel, and so for the
    // one before it, before it touches what they write
    allow_dependents();
    wait_for_prior_kernels();
    const int r = blockIdx.x;
    const int src = rows ? rows[r] : r;
    float* hrow = h + (size_t)src * width;
    const T* drow = delta ? delta + (size_t)src * width : nullptr;
    T* xrow = x + (size_t)r * width;
    float4 v[CHUNKS], d[CHUNKS];
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        v[c] = d[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < width) {
            v[c] = *reinterpret_cast<const float4*>(hrow + i);
            if (drow) load4(drow + i, d[c]);
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        v[c].x += d[c].x; v[c].y += d[c].y; v[c].z += d[c].z; v[c].w += d[c].w;
        if (write_h && i < width) *reinterpret_cast<float4*>(hrow + i) = v[c];
        ss += v[c].x * v[c].x;
        ss += v[c].y * v[c].y;
        ss += v[c].z * v[c].z;
        ss += v[c].w * v[c].w;
    }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)width + eps);
#pragma unroll
    for (int c = 0; c < CHUNKS; ++c) {
        const int i = (c * blockDim.x + threadIdx.x) * 4;
        if (i < width)
            store4(xrow + i, make_float4(v[c].x * inv * g[c].x, v[c].y * inv * g[c].y, v[c].z * inv * g[c].z, v[c].w * inv * g[c].w));
    }
}

template <typename T>
int launch_add_rmsnorm(float* h, const T* delta, const int* rows, const float* w, float eps, T* x, int n_rows, int width,
                       int write_h, cudaStream_t s) {
    const int groups = width / 4;
    // Which arrangement runs decides the order in which a row's squares are added.  In the 32-bit path that order
    // may depend on the width only (the same bits however a step is cut), so the number of rows chooses between
    // the arrangements for bfloat16 alone.
    const bool by_rows = !std::is_same<T, float>::value;
    if ((width & 3) == 0 && groups <= 1024 && (n_rows <= 256 || !by_rows)) {
        // few rows (decoding): as many threads as the row has groups of four, so that a row's latency is one load
        const int threads = (groups + 31) / 32 * 32;
        RMX_CHECK_LAUNCHED(launch_dependent(add_rmsnorm_rows_kernel<T, 1>, dim3(n_rows), dim3(threads), 0, s, h, delta, rows, w, eps,
                                            x, width, write_h), "add_rmsnorm");
        return 0;
    }
    constexpr int CHUNKS = 4;
    if ((width & 3) == 0 && groups <= CHUNKS * 1024) {
        // many rows: as few threads as hold the row in CHUNKS groups each (at least a warp), several blocks an SM
        int threads = ((groups + CHUNKS - 1) / CHUNKS + 31) / 32 * 32;
        threads = threads < 32 ? 32 : threads;
        RMX_CHECK_LAUNCHED(launch_dependent(add_rmsnorm_rows_kernel<T, CHUNKS>, dim3(n_rows), dim3(threads), 0, s, h, delta, rows, w, eps,
                                            x, width, write_h), "add_rmsnorm");
        return 0;
    }
    const int threads = block_threads(width);
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    RMX_CHECK_LAUNCHED(launch_dependent(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(threads), smem, s, h, delta, rows, w, eps, x, width,
                                        write_h), "add_rmsnorm");
    return 0;
}

RMX_API int rmx_add_rmsnorm(float* h, const void* delta, const int* rows, const float* w, float eps, void* x,
                            int n_rows, int width, int write_h, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && width > 0, "add_rmsnorm: bad sizes");
    RMX_REQUIRE((size_t)width * 4 <= 160 * 1024, "add_rmsnorm: width %d is beyond 40960", width);
    RMX_REQUIRE(!(rows && write_h), "add_rmsnorm: rows and write_h do not go together");
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    if (dtype == RMX_F32) rc = launch_add_rmsnorm<float>(h, (const float*)delta, rows, w, eps, (float*)x, n_rows, width, write_h, s);
    else if (dtype == RMX_BF16)
        rc = launch_add_rmsnorm<__nv_bfloat16>(h, (const __nv_bfloat16*)delta, rows, w, eps, (__nv_bfloat16*)x, n_rows, width, write_h, s);
    else RMX_FAIL("add_rmsnorm: unknown dtype %d", dtype);
    if (rc != 0) return rc;
    RMX_CHECK_LAUNCH("add_rmsnorm");
    return 0;
}

// out[t, j] = silu(gate_up[t, j]) * gate_up[t, inter + j], silu(z) = z / (1 + exp(-z)),
// in float with one rounding.
__device__ __forceinline__ float silu_mul(float g, float u) { return g / (1.f + expf(-g)) * u; }

// Where gate j and up j lie in a row of 2 * inter numbers: concatenated [gate | up] (block == 0), or in blocks of
// `block` gate numbers followed by their `block` up numbers.
__device__ __forceinline__ void gate_up_at(int j, int inter, int block, int& gi, int& ui) {
    if (block == 0) {
        gi = j;
        ui = inter + j;
    } else {
        gi = (j / block) * 2 * block + j % block;
        ui = gi + block;
    }
}

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int block, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t t = idx / inter;
    const int j = (int)(idx - t * inter);
    int gi, ui;
    gate_up_at(j, inter, block, gi, ui);
    const float g = to_float(gate_up[t * 2 * inter + gi]);
    const float u = to_float(gate_up[t * 2 * inter + ui]);
    out[idx] = from_float<T>(silu_mul(g, u));
}

// four outputs per thread; inter is a multiple of 4
template <typename T>
__global__ void swiglu_kernel4(const T* __restrict__ gate_up, T* __restrict__ out, int inter, int block, size_t total4) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    const int per_row = inter >> 2;
    const size_t t = idx / per_row;
    const int j = (int)(idx - t * per_row) * 4;
    int gi, ui;
    gate_up_at(j, inter, block, gi, ui);   // four neighbours stay together: block is a multiple of 4
    float4 g, u;
    load4(gate_up + t * 2 * inter + gi, g);
    load4(gate_up + t * 2 * inter + ui, u);
    store4(out + t * inter + j, make_float4(silu_mul(g.x, u.x), silu_mul(g.y, u.y), silu_mul(g.z, u.z), silu_mul(g.w, u.w)));
}

// bfloat16, sixteen outputs per thread as two groups of eight (16-byte loads and stores); inter and block are
// multiples of 8.  blockIdx.x is the token, blockIdx.y the part of its row.  The exponential and the division are
// the fast ones (about two units in the last place of a float): the result is rounded to bfloat16, eight bits.
__device__ __forceinline__ float silu_mul_fast(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }

__global__ void swiglu_kernel8(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out, int inter,
                               int block) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int per_row = inter >> 3;
    const __nv_bfloat16* src = gate_up + (size_t)blockIdx.x * 2 * inter;
    __nv_bfloat16* dst = out + (size_t)blockIdx.x * inter;
    uint4 g[2], u[2];
    int j[2];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        const int item = (blockIdx.y * 2 + c) * blockDim.x + threadIdx.x;
        j[c] = item < per_row ? item * 8 : -1;
        if (j[c] >= 0) {
            int gi, ui;
            gate_up_at(j[c], inter, block, gi, ui);
            g[c] = *reinterpret_cast<const uint4*>(src + gi);
            u[c] = *reinterpret_cast<const uint4*>(src + ui);
        }
    }
#pragma unroll
    for (int c = 0; c < 2; ++c) {
        if (j[c] < 0) continue;
        const uint32_t gw[4] = {g[c].x, g[c].y, g[c].z, g[c].w}, uw[4] = {u[c].x, u[c].y, u[c].z, u[c].w};
        uint32_t ow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[i]));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[i]));
            __nv_bfloat162 r = __floats2bfloat162_rn(silu_mul_fast(a.x, b.x), silu_mul_fast(a.y, b.y));
            ow[i] = *reinterpret_cast<uint32_t*>(&r);
        }
        *reinterpret_cast<uint4*>(dst + j[c]) = make_uint4(ow[0], ow[1], ow[2], ow[3]);
    }
}

RMX_API int rmx_swiglu(const void* gate_up, void* out, int n_tokens, int inter, int block, int dtype, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(n_tokens > 0 && inter > 0, "swiglu: bad sizes");
    RMX_REQUIRE(block == 0 || (block > 0 && inter % block == 0), "swiglu: blocks of %d do not divide %d", block, inter);
    const bool vec = (inter & 3) == 0 && (block & 3) == 0;
    const int threads = 256;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_BF16 && (inter & 7) == 0 && (block & 7) == 0 && ((uintptr_t)gate_up & 15) == 0 && ((uintptr_t)out & 15) == 0) {
        const int per_row = inter / 8;
        const int t8 = per_row >= 512 ? 256 : 128;
        RMX_CHECK_LAUNCHED(launch_dependent(swiglu_kernel8, dim3(n_tokens, (per_row + 2 * t8 - 1) / (2 * t8)), dim3(t8), 0, s,
                                            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block), "swiglu");
        return 0;
    }
    const size_t total = (size_t)n_tokens * inter / (vec ? 4 : 1);
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    if (dtype == RMX_F32) {
        if (vec) RMX_CHECK_LAUNCHED(launch_dependent(swiglu_kernel4<float>, dim3(blocks), dim3(threads), 0, s, (const float*)gate_up, (float*)out, inter, block, total), "swiglu");
        else swiglu_kernel<float><<<blocks, threads, 0, s>>>((const float*)gate_up, (float*)out, inter, block, total);
    } else if (dtype == RMX_BF16) {
        if (vec) RMX_CHECK_LAUNCHED(launch_dependent(swiglu_kernel4<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, total), "swiglu");
        else swiglu_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>((const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, block, total);
    } else {
        RMX_FAIL("swiglu: unknown dtype %d", dtype);
    }
    RMX_CHECK_LAUNCH("swiglu");
    return 0;
}

// h[t, :] += delta[t, :] (float add, delta in T): closes the residual stream when no norm follows.
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ h, const T* __restrict__ delta, size_t total) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < total) h[idx] += to_float(delta[idx]);
}

RMX_API int rmx_add_residual(float* h, const void* delta, int n_rows, int width, int dtype, void* stream) {
    if (n_rows == 0) return 0;
    const size_t total = (size_t)n_rows * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        add_residual_kernel<float><<<blocks, threads, 0, s>>>(h, (const float*)delta, total);
    else if (dtype == RMX_BF16)
        add_residual_kernel<__nv_bfloat16><<<blocks, threads, 0, s>>>(h, (const __nv_bfloat16*)delta, total);
    else
        RMX_FAIL("add_residual: unknown dtype %d", dtype);
    RMX_CHECK_LAUNCH("add_residual");
    return 0;
}

// x[t, j] = x[t, j] + bias[j] (float add, one rounding): the bias of a projection, added to the product as the
// reference does (src/weights.rs:198-200).  `ld` is the distance between rows of x.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int width, int ld, size_t total) {
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const size_t row = idx / width;
    const int col = (int)(idx - row * width);
    T* at = x + row * ld + col;
    *at = from_float<T>(to_float(*at) + bias[col]);
}

RMX_API int rmx_add_bias(void* x, const float* bias, int n_rows, int width, int ld, int dtype, void* stream) {
    if (n_rows == 0 || width == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && width > 0 && ld >= width && x && bias, "add_bias: bad sizes or a null pointer");
    const size_t total = (size_t)n_rows * width;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RMX_F32)
        RMX_CHECK_LAUNCHED(launch_dependent(add_bias_kernel<float>, dim3(blocks), dim3(threads), 0, s, (float*)x, bias, width, ld, total), "add_bias");
    else if (dtype == RMX_BF16)
        RMX_CHECK_LAUNCHED(launch_dependent(add_bias_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, (__nv_bfloat16*)x, bias, width, ld, total), "add_bias");
    else
        RMX_FAIL("add_bias: unknown dtype %d", dtype);
    return 0;
}
