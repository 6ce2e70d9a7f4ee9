// bfloat16 matrix product on the Blackwell tensor cores for few rows (decoding):
//   C[M, N] = A[M, K] . W[N, K]^T,  M <= 64 rows of activations against a large weight.
//
// With so few rows the product is bound by reading W once.  The kernel swaps the roles of
// the operands so that the weight fills the 128-row side of the tensor-core instruction:
//   D[128 weight rows, MPAD tokens] += Wtile[128, 64] . Atile[MPAD, 64]^T     (tcgen05.mma, kind::f16)
// A block owns one tile of 128 weight rows (and, with split-K, one slice of K).  One thread
// streams W and A tiles of 64 k into a ring of shared-memory stages with TMA (128-byte
// swizzle); one thread issues the MMAs, whose accumulator lives in tensor memory; when
// the last MMA has completed, the four warps read the accumulator (tcgen05.ld, one weight
// row per thread) and write C, coalesced over the weight rows.  With split-K the slices
// leave float partial sums in a scratch buffer and the last block to finish a tile adds
// them in slice order (a counter per tile says who is last), so the result does not
// depend on the order in which blocks run.
//
// Every wait on a barrier gives up after a bounded number of polls, records an error in
// the status word and lets the block run to its end (tensor memory is always freed).
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "tcgen05.cuh"

namespace {
constexpr int TILE_N = 128;   // weight rows per block: the M side of the instruction
constexpr int TILE_K = 64;    // 64 bfloat16 = 128 bytes: one swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 128;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

struct GemmParams {
    void* c;                 // [M, ldc] bfloat16 or float
    float* partial;          // [splits, MPAD, n_tiles * 128] floats (splits > 1)
    unsigned int* counters;  // [n_tiles], zero between launches (splits > 1)
    int* status;
    int M, N, K, ldc, splits, k_blocks, out_float;
    uint32_t spin_limit;     // polls after which a wait on a barrier gives up (SPIN_LIMIT; a test passes a small number)
    int no_loads;            // test only: the producer issues no copies, so that every wait for a tile runs out
    int dependent;           // launched as a programmatic dependent: wait for the grid before before reading A
    int epilogue;            // 0: C = product.  1: the tile's rows are 64 gate rows then their 64 up rows;
                             //    C[M, N / 2] = silu(gate) * up, formed in float and rounded once.
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Store a float into the shared memory of another block of the cluster, at the place that `local` has here.
__device__ __forceinline__ void st_cluster(float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_addr(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(remote), "f"(v) : "memory");
}

// CLUSTER: the slices of K of one tile form a thread-block cluster (grid.y == cluster size == splits); they
// hand their partial sums to the first block through distributed shared memory, no global scratch.
template <int MPAD, int STAGES, bool CLUSTER>
__global__ void __launch_bounds__(THREADS) gemm_swapab_kernel(const __grid_constant__ CUtensorMap map_w,
                                                              const __grid_constant__ CUtensorMap map_a,
                                                              const GemmParams p) {
    constexpr int W_BYTES = TILE_N * TILE_K * 2, A_BYTES = MPAD * TILE_K * 2;
    constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    constexpr int TMEM_COLS = MPAD < 32 ? 32 : MPAD;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // tiles must sit on 1024-byte boundaries for the 128-byte swizzle
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int s_failed, s_last;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int per_split = (p.k_blocks + p.splits - 1) / p.splits;
    const int kb_begin = split * per_split, kb_end = min(p.k_blocks, kb_begin + per_split);
    const int n_kb = max(0, kb_end - kb_begin);

    if (tid == 0) {
        s_failed = 0;
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&acc_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_tensormap(&map_w);
        prefetch_tensormap(&map_a);
        // the kernels that follow may be launched now: they wait for this grid before they read its output
        asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    }
    if (warp == 1) {  // one warp allocates the accumulator's columns of tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_addr(&tmem_base_smem)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_acc = tmem_base_smem;

    const uint32_t spin_limit = p.spin_limit;
    if (warp == 0 && lane == 0 && !p.no_loads) {
        // ---- producer: stream W and A tiles through the ring.  The weights do not depend on the kernel
        // before this one, so the first stages' W tiles are on their way before the wait for that kernel.
        const int ahead = n_kb < STAGES ? n_kb : STAGES;
        for (int i = 0; i < ahead; ++i) {
            mbar_expect_tx(&full_bar[i], STAGE_BYTES);
            tma_load_2d(tiles + i * STAGE_BYTES, &map_w, &full_bar[i], (kb_begin + i) * TILE_K, tile * TILE_N);
        }
        if (p.dependent) asm volatile("griddepcontrol.wait;\n" ::: "memory");
        for (int i = 0; i < ahead; ++i)
            tma_load_2d(tiles + i * STAGE_BYTES + W_BYTES, &map_a, &full_bar[i], (kb_begin + i) * TILE_K, 0);
        for (int i = ahead; i < n_kb; ++i) {
            const int s = i % STAGES, round = i / STAGES;
            if (!mbar_wait(&empty_bar[s], (round - 1) & 1, spin_limit)) { atomicExch(&s_failed, 1); break; }
            unsigned char* dst = tiles + s * STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            const int k0 = (kb_begin + i) * TILE_K;
            tma_load_2d(dst, &map_w, &full_bar[s], k0, tile * TILE_N);
            tma_load_2d(dst + W_BYTES, &map_a, &full_bar[s], k0, 0);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        const uint32_t idesc = umma_idesc(MPAD);
        for (int i = 0; i < n_kb; ++i) {
            const int s = i % STAGES, round = i / STAGES;
            if (!mbar_wait(&full_bar[s], round & 1, spin_limit)) { atomicExch(&s_failed, 1); break; }
            tcgen05_fence_after();
            const uint32_t w_addr = smem_addr(tiles + s * STAGE_BYTES), a_addr = w_addr + W_BYTES;
#pragma unroll
            for (int k = 0; k < TILE_K / UMMA_K; ++k)
                umma_mma(tmem_acc, umma_desc(w_addr + k * UMMA_K * 2), umma_desc(a_addr + k * UMMA_K * 2), idesc, i > 0 || k > 0);
            umma_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
        }
        umma_commit(&acc_bar);            // the accumulator is complete once every MMA has finished
    }
    __syncwarp();

    // ---- epilogue: every thread owns one weight row of the tile
    bool ok = n_kb == 0 || mbar_wait(&acc_bar, 0, spin_limit);
    if (!ok) atomicExch(&s_failed, 1);
    tcgen05_fence_after();
    const int n = tile * TILE_N + warp * 32 + lane;
    float acc[MPAD];
    if (n_kb > 0 && ok) {
#pragma unroll
        for (int c = 0; c < MPAD; c += 16) {
            uint32_t r[16];
            tmem_ld16(tmem_acc + ((uint32_t)(warp * 32) << 16) + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[c + j] = __uint_as_float(r[j]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < MPAD; ++j) acc[j] = 0.f;
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_acc), "r"(TMEM_COLS));
    const bool failed = s_failed != 0;
    if (failed && tid == 0) atomicExch(p.status, 3);
    // (a block that failed still joins the cluster's barriers, or the tile's counter, below)

    if constexpr (CLUSTER && MPAD >= 32) {
        // More than 16 rows: the slices share the summing.  Row t belongs to block t mod splits of the cluster; every
        // block hands each of its rows to the row's owner (its own rows to itself) through distributed shared memory,
        // and every owner adds the slices of its rows in slice order and writes them.  A block's work then does not
        // grow with the number of slices (one block adding everything reads splits x rows numbers a thread), and the
        // room it needs is a fraction of the stages, so that up to eight slices can share a tile at any row count.
        // (The loop over a block's rows is not unrolled on purpose: this code runs once a block, and what it costs is
        // fetching its instructions.  With up to 16 rows the first block adds everything: it is faster there, and the
        // other blocks leave their SMs sooner.)
        const uint32_t rank = cluster_ctarank();
        const int S = p.splits, cap = (MPAD + S - 1) / S;    // cap: rows a block can own
        float* recv = reinterpret_cast<float*>(tiles);       // [S slices][cap rows][128]
        float* ex = recv + (size_t)S * cap * TILE_N;          // [64]: SwiGLU's exchange between the halves of the block
        cluster_sync();
        {
            uint32_t owner = 0;
            float* at = recv + (size_t)rank * cap * TILE_N + tid;   // row t is its owner's j-th: `at` moves on with j
#pragma unroll
            for (int t = 0; t < MPAD; ++t) {
                if (t < p.M) st_cluster(at, owner, acc[t]);
                if (++owner == (uint32_t)S) { owner = 0; at += TILE_N; }
            }
        }
        cluster_sync();
        if (failed) return;
        const size_t slice = (size_t)cap * TILE_N;
        for (int j = 0, t = (int)rank; t < p.M; ++j, t += S) {
            const float* src = recv + (size_t)j * TILE_N + tid;
            float sum = 0.f;
            for (int z = 0; z < S; ++z) sum += src[z * slice];
            if (p.epilogue == 1) {
                // the upper half of the block (up rows) hands its sums to the lower half (gate rows)
                if (tid >= 64) ex[tid - 64] = sum;
                __syncthreads();
                const int col = tile * 64 + tid;
                if (tid < 64 && col < p.N / 2) {
                    const float v = sum / (1.f + expf(-sum)) * ex[tid];
                    if (p.out_float) reinterpret_cast<float*>(p.c)[(size_t)t * p.ldc + col] = v;
                    else reinterpret_cast<__nv_bfloat16*>(p.c)[(size_t)t * p.ldc + col] = __float2bfloat16_rn(v);
                }
                __syncthreads();
            } else if (n < p.N) {
                if (p.out_float) reinterpret_cast<float*>(p.c)[(size_t)t * p.ldc + n] = sum;
                else reinterpret_cast<__nv_bfloat16*>(p.c)[(size_t)t * p.ldc + n] = __float2bfloat16_rn(sum);
            }
        }
        return;
    } else if constexpr (CLUSTER) {
        // every block's MMAs are done (its shared-memory stages are free); the slices hand their sums to the
        // first block of the cluster, which adds them in slice order
        float* slots = reinterpret_cast<float*>(tiles);   // [splits - 1][MPAD][128] in the first block
        const uint32_t rank = cluster_ctarank();
        cluster_sync();
        if (rank != 0) {
#pragma unroll
            for (int t = 0; t < MPAD; ++t)
                if (t < p.M) st_cluster(slots + ((rank - 1) * MPAD + t) * TILE_N + tid, 0, acc[t]);
        }
        cluster_sync();
        if (rank != 0 || failed) return;
        for (int z = 1; z < p.splits; ++z) {
#pragma unroll
            for (int t = 0; t < MPAD; ++t)
                if (t < p.M) acc[t] += slots[((z - 1) * MPAD + t) * TILE_N + tid];
        }
    } else if (p.splits > 1) {
        // leave this slice's sums, then the last block of the tile adds the slices in order
        const size_t ldp = (size_t)gridDim.x * TILE_N;
        float* mine = p.partial + (size_t)split * MPAD * ldp;
#pragma unroll
        for (int t = 0; t < MPAD; ++t)
            if (t < p.M) mine[(size_t)t * ldp + n] = acc[t];
        __threadfence();
        __syncthreads();
        // a block that gave up still counts, so that the counter is zero again for the next launch
        if (tid == 0) {
            s_last = atomicAdd(&p.counters[tile], 1u) == (unsigned)p.splits - 1;
            if (s_last) p.counters[tile] = 0;
        }
        __syncthreads();
        if (!s_last || failed) return;
        __threadfence();
#pragma unroll
        for (int t = 0; t < MPAD; ++t) acc[t] = 0.f;
        for (int z = 0; z < p.splits; ++z) {
            const float* src = p.partial + (size_t)z * MPAD * ldp;
#pragma unroll
            for (int t = 0; t < MPAD; ++t)
                if (t < p.M) acc[t] += __ldcg(src + (size_t)t * ldp + n);
        }
    } else if (failed) {
        return;
    }
    if (p.epilogue == 1) {
        // the upper half of the block (up rows) hands its sums to the lower half (gate rows) through the
        // shared-memory stages, which are free by now
        float* ex = reinterpret_cast<float*>(tiles);   // [MPAD][64]
        if (CLUSTER) __syncthreads();                  // the first block has read the other slices' sums from there
        if (tid >= 64) {
#pragma unroll
            for (int t = 0; t < MPAD; ++t) ex[t * 64 + tid - 64] = acc[t];
        }
        __syncthreads();
        const int col = tile * 64 + tid;
        if (tid < 64 && col < p.N / 2) {
#pragma unroll
            for (int t = 0; t < MPAD; ++t) {
                if (t < p.M) {
                    const float g = acc[t], u = ex[t * 64 + tid];
                    const float v = g / (1.f + expf(-g)) * u;
                    if (p.out_float) reinterpret_cast<float*>(p.c)[(size_t)t * p.ldc + col] = v;
                    else reinterpret_cast<__nv_bfloat16*>(p.c)[(size_t)t * p.ldc + col] = __float2bfloat16_rn(v);
                }
            }
        }
        return;
    }
    if (n < p.N) {
        if (p.out_float) {
            float* c = reinterpret_cast<float*>(p.c);
#pragma unroll
            for (int t = 0; t < MPAD; ++t)
                if (t < p.M) c[(size_t)t * p.ldc + n] = acc[t];
        } else {
            __nv_bfloat16* c = reinterpret_cast<__nv_bfloat16*>(p.c);
#pragma unroll
            for (int t = 0; t < MPAD; ++t)
                if (t < p.M) c[(size_t)t * p.ldc + n] = __float2bfloat16_rn(acc[t]);
        }
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiled)ptr;
    }
    return fn;
}

// A [rows, cols] row-major bfloat16 matrix with leading dimension ld, copied in boxes of [box_rows, 64] with
// the 128-byte swizzle; rows and columns outside the matrix read as zeros.
struct MapKey {
    const void* base;
    int rows, cols, ld, box_rows;
    bool operator==(const MapKey& o) const {
        return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = std::hash<const void*>()(k.base);
        for (int v : {k.rows, k.cols, k.ld, k.box_rows}) h = h * 1000003u ^ std::hash<int>()(v);
        return h;
    }
};

}  // namespace

// Tensor maps depend on the address and the shape only; weights keep theirs, so encoded maps are kept.
int rmx_make_tensor_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    static std::mutex lock;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{base, rows, cols, ld, box_rows};
    std::lock_guard<std::mutex> guard(lock);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *map = it->second;
        return 0;
    }
    if (rmx_encode_tensor_map(map, base, rows, cols, ld, box_rows) != 0) return -1;
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *map);
    return 0;
}

int rmx_encode_tensor_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    EncodeTiled fn = encode_tiled();
    if (!fn) RMX_FAIL("gemm_tcgen05: the driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)TILE_K, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RMX_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return 0;
}

namespace {
template <int MPAD, int STAGES, bool CLUSTER>
int launch_as(const CUtensorMap& mw, const CUtensorMap& ma, const GemmParams& p, int n_tiles, bool dependent, cudaStream_t s) {
    constexpr size_t smem = (size_t)STAGES * (TILE_N * TILE_K * 2 + MPAD * TILE_K * 2) + 1024;
    // a function's attributes are kept per device: raise the limit once on each
    static bool raised[64] = {};
    if (rmx_first_on_device(raised)) {
        cudaError_t e = cudaFuncSetAttribute(gemm_swapab_kernel<MPAD, STAGES, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RMX_FAIL("gemm_tcgen05: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles, p.splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    int n_attrs = 0;
    if (CLUSTER) {
        attrs[n_attrs].id = cudaLaunchAttributeClusterDimension;
        attrs[n_attrs].val.clusterDim.x = 1;
        attrs[n_attrs].val.clusterDim.y = p.splits;
        attrs[n_attrs].val.clusterDim.z = 1;
        ++n_attrs;
    }
    if (dependent) {
        attrs[n_attrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n_attrs].val.programmaticStreamSerializationAllowed = 1;
        ++n_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = n_attrs;
    GemmParams q = p;
    q.dependent = dependent ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_swapab_kernel<MPAD, STAGES, CLUSTER>, mw, ma, q);
    if (e != cudaSuccess) RMX_FAIL("gemm_tcgen05: launch failed: %s", cudaGetErrorString(e));
    return 0;
}

// cluster: reduce split-K through distributed shared memory (2..8 slices whose sums fit the first block's stages)
template <int MPAD, int STAGES>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, const GemmParams& p, int n_tiles, cudaStream_t s,
           bool cluster = false, bool dependent = false) {
    if (cluster) return launch_as<MPAD, STAGES, true>(mw, ma, p, n_tiles, dependent, s);
    return launch_as<MPAD, STAGES, false>(mw, ma, p, n_tiles, dependent, s);
}
}  // namespace

// What the kernel takes: up to 64 rows, K a multiple of 8 (TMA rows are 16-byte multiples), 16-byte aligned bases.
RMX_API int rmx_gemm_tcgen05_supports(int M, int N, int K) { return M >= 1 && M <= 64 && N >= 1 && K >= 8 && K % 8 == 0; }

// Scratch for split-K: floats for partial sums and one counter per tile of 128 weight rows.
RMX_API long long rmx_gemm_tcgen05_scratch_floats(int M, int N, int splits) {
    const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    return splits <= 1 ? 0 : (long long)splits * mpad * ((N + TILE_N - 1) / TILE_N) * TILE_N;
}

namespace {
int gemm_tcgen05_run(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                     int out_float, int splits, float* partial, unsigned int* counters, int* status,
                     int flags, cudaStream_t s, uint32_t spin_limit = SPIN_LIMIT, int no_loads = 0) {
    if (M == 0 || N == 0) return 0;
    RMX_REQUIRE(rmx_gemm_tcgen05_supports(M, N, K), "gemm_tcgen05: M=%d N=%d K=%d is outside 1..64 rows, K %% 8 == 0", M, N, K);
    RMX_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0,
                "gemm_tcgen05: operands must be 16-byte aligned with leading dimensions that are multiples of 8");
    const int k_blocks = (K + TILE_K - 1) / TILE_K;
    RMX_REQUIRE(splits >= 1 && splits <= k_blocks && splits <= 65535, "gemm_tcgen05: %d splits for %d k-blocks", splits, k_blocks);
    const int n_tiles = (N + TILE_N - 1) / TILE_N;
    const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    // flags: 1 = reduce split-K inside a cluster when it can be (no scratch needed); 2 = programmatic dependent launch
    const int stages = mpad == 64 ? 4 : (mpad == 16 ? 6 : 5);
    // what the cluster's reduction needs of a block's stages: up to 16 rows, the other slices' sums of all rows in the
    // first block; above, every slice's sums of the rows a block owns (and a line for SwiGLU)
    const size_t reduce_bytes = mpad <= 16 ? (size_t)(splits - 1) * mpad * TILE_N * 4
                                           : ((size_t)splits * ((mpad + splits - 1) / splits) * TILE_N + 64) * 4;
    const bool fits = reduce_bytes <= (size_t)stages * (TILE_N * TILE_K * 2 + mpad * TILE_K * 2);
    const bool cluster = (flags & 1) && splits >= 2 && splits <= 8 && fits;
    const bool dependent = (flags & 2) != 0;
    const int epilogue = (flags & 4) ? 1 : 0;   // flags: 4 = SwiGLU over blocks of 64 gate rows and 64 up rows
    RMX_REQUIRE(epilogue != 1 || N % 128 == 0, "gemm_tcgen05: the SwiGLU epilogue needs N to be a multiple of 128, got %d", N);
    RMX_REQUIRE(splits == 1 || cluster || (partial && counters), "gemm_tcgen05: split-K needs scratch");
    CUtensorMap mw, ma;
    if (rmx_make_tensor_map(&mw, W, N, K, ldw, TILE_N) != 0) return -1;
    if (rmx_make_tensor_map(&ma, A, M, K, lda, mpad) != 0) return -1;
    GemmParams p;
    p.c = C; p.partial = partial; p.counters = counters; p.status = status;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.splits = splits; p.k_blocks = k_blocks; p.out_float = out_float;
    p.dependent = 0; p.epilogue = epilogue; p.spin_limit = spin_limit; p.no_loads = no_loads;
    // stages sized so that two blocks fit an SM: more blocks in flight smooth the last wave
    if (mpad == 16) return launch<16, 6>(mw, ma, p, n_tiles, s, cluster, dependent);
    if (mpad == 32) return launch<32, 5>(mw, ma, p, n_tiles, s, cluster, dependent);
    return launch<64, 4>(mw, ma, p, n_tiles, s, cluster, dependent);
}
}  // namespace

// C[M, N] = A[M, K] . W[N, K]^T.  out_float: C is float (logits), else bfloat16.  With splits > 1, `partial` holds
// rmx_gemm_tcgen05_scratch_floats floats and `counters` ceil(N / 128) zeroed unsigned ints (left zero again).
RMX_API int rmx_gemm_tcgen05(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw, int ldc,
                             int out_float, int splits, float* partial, unsigned int* counters, int* status,
                             int flags, void* stream) {
    return gemm_tcgen05_run(A, W, C, M, N, K, lda, ldw, ldc, out_float, splits, partial, counters, status, flags, (cudaStream_t)stream);
}

// For tests of the give-up path: the same kernel with the same arguments, except that its producer issues no
// copies and every wait gives up after `spin_limit` polls.  No tile ever arrives, so the thread that issues the
// MMAs gives up at its first wait; the block records status 3, writes no output, frees its tensor memory, joins
// its cluster's barriers (or counts itself at the tile's counter, which is zero again afterwards) and returns.
// Nothing is left in flight: there was no copy and no MMA.
RMX_API int rmx_gemm_tcgen05_wait_probe(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw,
                                        int ldc, int out_float, int splits, float* partial, unsigned int* counters,
                                        int* status, int flags, int spin_limit, void* stream) {
    RMX_REQUIRE(spin_limit >= 1 && spin_limit <= (1 << 20), "gemm_tcgen05_wait_probe: a limit of 1 to 2^20 polls, got %d", spin_limit);
    return gemm_tcgen05_run(A, W, C, M, N, K, lda, ldw, ldc, out_float, splits, partial, counters, status, flags & ~2,
                            (cudaStream_t)stream, (uint32_t)spin_limit, 1);
}

// ---------------------------------------------------------------------------------------------
// The same product for callers that cannot allocate: scratch in the library's own memory.
// See rmx_no_alloc.h for who needs this and what it promises.
#include "rmx_no_alloc.h"

namespace {
// File-scope device memory: loaded with the library on every GPU that uses it and kept until exit.
static __device__ __align__(256) float g_static_partial[RMX_STATIC_SCRATCH_FLOATS];
static __device__ __align__(256) unsigned int g_static_counters[RMX_STATIC_SCRATCH_TILES];
static __device__ __align__(256) int g_static_status[64];

constexpr int MAX_DEVICES = 64;
struct StaticScratch {
    float* partial = nullptr;
    unsigned int* counters = nullptr;
    int* status = nullptr;
};
StaticScratch g_scratch[MAX_DEVICES];
std::mutex g_scratch_lock;

// In host code the arrays' names stand for the symbols, not for device addresses: ask the runtime for
// the addresses once per device, with that device current.
int static_scratch(StaticScratch* out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) RMX_FAIL("gemm_tcgen05_static: no current device: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= MAX_DEVICES) RMX_FAIL("gemm_tcgen05_static: device %d is beyond %d", dev, MAX_DEVICES);
    std::lock_guard<std::mutex> guard(g_scratch_lock);
    StaticScratch& s = g_scratch[dev];
    if (!s.partial) {
        void *p = nullptr, *c = nullptr, *st = nullptr;
        if ((e = cudaGetSymbolAddress(&p, g_static_partial)) != cudaSuccess ||
            (e = cudaGetSymbolAddress(&c, g_static_counters)) != cudaSuccess ||
            (e = cudaGetSymbolAddress(&st, g_static_status)) != cudaSuccess)
            RMX_FAIL("gemm_tcgen05_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
        s.partial = (float*)p;
        s.counters = (unsigned int*)c;
        s.status = (int*)st;
    }
    *out = s;
    return 0;
}
}  // namespace

RMX_API int rmx_gemm_tcgen05_static(const void* A, const void* W, void* C, int M, int N, int K, int lda, int ldw,
                                    int ldc, int out_float, int splits, void* stream) {
    if (M == 0 || N == 0) return 0;
    RMX_REQUIRE(rmx_gemm_tcgen05_supports(M, N, K), "gemm_tcgen05_static: M=%d N=%d K=%d is outside 1..64 rows, K %% 8 == 0", M, N, K);
    RMX_REQUIRE(lda % 8 == 0 && ldw % 8 == 0 && ((uintptr_t)A & 15) == 0 && ((uintptr_t)W & 15) == 0,
                "gemm_tcgen05_static: operands must be 16-byte aligned with leading dimensions that are multiples of 8");
    const int k_blocks = (K + TILE_K - 1) / TILE_K;
    const int n_tiles = (N + TILE_N - 1) / TILE_N;
    RMX_REQUIRE(n_tiles <= RMX_STATIC_SCRATCH_TILES, "gemm_tcgen05_static: N=%d is beyond the %d rows the library's scratch covers",
                N, RMX_STATIC_SCRATCH_TILES * TILE_N);
    const int mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    if (splits <= 0) {  // as many slices as fit the scratch, up to one block per SM slot, at least 8 k-blocks each
        const long long room = RMX_STATIC_SCRATCH_FLOATS / ((long long)mpad * n_tiles * TILE_N);
        long long pick = room;
        if (pick > k_blocks / 8) pick = k_blocks / 8;
        int dev = 0, sms = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            RMX_FAIL("gemm_tcgen05_static: the device's SM count cannot be read");
        if (pick > 2 * sms / n_tiles) pick = 2 * sms / n_tiles;   // two blocks fit an SM
        splits = pick < 1 ? 1 : (int)pick;
    }
    RMX_REQUIRE(splits >= 1 && splits <= k_blocks && splits <= 65535, "gemm_tcgen05_static: %d splits for %d k-blocks", splits, k_blocks);
    const long long need = splits <= 1 ? 0 : rmx_gemm_tcgen05_scratch_floats(M, N, splits);
    RMX_REQUIRE(need <= RMX_STATIC_SCRATCH_FLOATS,
                "gemm_tcgen05_static: %d splits of M=%d N=%d need %lld floats of scratch, the library holds %d; use fewer splits",
                splits, M, N, need, RMX_STATIC_SCRATCH_FLOATS);
    StaticScratch scratch;
    if (static_scratch(&scratch) != 0) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    // what must start at zero: the tiles' counters (a call that was cut short may have left some set) and the status word
    cudaError_t e = cudaMemsetAsync(scratch.counters, 0, sizeof(unsigned int) * n_tiles, s);
    if (e == cudaSuccess) e = cudaMemsetAsync(scratch.status, 0, sizeof(int), s);
    if (e != cudaSuccess) RMX_FAIL("gemm_tcgen05_static: clearing the scratch failed: %s", cudaGetErrorString(e));
    CUtensorMap mw, ma;
    if (rmx_encode_tensor_map(&mw, W, N, K, ldw, TILE_N) != 0) return -1;
    if (rmx_encode_tensor_map(&ma, A, M, K, lda, mpad) != 0) return -1;
    GemmParams p;
    p.c = C; p.partial = scratch.partial; p.counters = scratch.counters; p.status = scratch.status;
    p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.splits = splits; p.k_blocks = k_blocks; p.out_float = out_float;
    p.dependent = 0; p.epilogue = 0; p.spin_limit = SPIN_LIMIT; p.no_loads = 0;
    if (mpad == 16) return launch<16, 5>(mw, ma, p, n_tiles, s);
    if (mpad == 32) return launch<32, 5>(mw, ma, p, n_tiles, s);
    return launch<64, 4>(mw, ma, p, n_tiles, s);
}

RMX_API int rmx_gemm_tcgen05_static_status(void* stream) {
    StaticScratch scratch;
    if (static_scratch(&scratch) != 0) return -1;
    int host = 0;
    cudaError_t e = cudaMemcpyAsync(&host, scratch.status, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) RMX_FAIL("gemm_tcgen05_static_status: %s", cudaGetErrorString(e));
    return host;
}
