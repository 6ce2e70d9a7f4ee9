// Attention for prompt portions on the Blackwell tensor cores (tcgen05), head sizes 64 and 128, bfloat16.
//
// A block takes one kv head and one tile of 128 query rows of one sequence; a row is a (token, query
// head of the group) pair, 128 / group tokens by `group` heads, so the heads that share a kv head share
// every key and value tile.  Keys are visited in tiles of 64 aligned to absolute positions.
//
// A block takes two neighbouring tiles, which share every key and value tile it fetches (or one, for steps so
// small that SMs would be left without work).  Key tiles go in pairs: one step of every role is 128 keys.
//
//   warp 0   producer: Q once, then pairs of key tiles and of value tiles by TMA (tensor-map boxes, 128-byte
//            swizzle) into two rings, the keys a pair ahead of the values
//   warp 1   issues S = Q K^T: the scores of a pair of key tiles are one group of MMAs of 128 columns (an MMA of
//            128 rows by 64 columns takes as long as one of 128 columns; the pair's key tiles lie in neighbouring
//            slots of the ring, which makes them one operand of 128 rows).  There is one score buffer in tensor
//            memory; the two query tiles take it in turns: as soon as a tile's softmax warps have their scores
//            in registers, the other tile's next scores are formed in it
//   warp 2   issues O += P V with P read from tensor memory.  (Two issuing warps: the tensor cores take an MMA
//            only when an earlier one has left their queue, so a warp that issues is held for as long as they
//            run; while one is held or waits for a barrier, the other issues.  Both run their loop with every
//            lane and elect one to issue, so that the operand descriptors stay in uniform registers.)
//   warp 3   spare
//   warps 4-7 and 8-11  softmax of the first and the second query tile: every thread owns one row (one lane of
//            tensor memory) and holds its 128 scores of a pair in registers.  The reference m that exponentials
//            are taken against moves only when a score exceeds it by more than 2^8, so a pair is first tried in one
//            pass against the reference as it stands (exponent, largest exponent seen, sum, probabilities as
//            bfloat16 into tensor memory), and done the long way (maximum, new reference, O rescaled, the same pass
//            again) only where that pass meets a larger score or a row has no reference yet.  A pair that needs a
//            mask (the diagonal, the window's edge) is masked in tensor memory first and then treated like any other
//
// Code size: the kernel's code is fetched anew at every launch (the kernels between two launches push it out of
// the instruction caches), and straight-line code is fetched at a few instructions a microsecond: 30 KB of
// unrolled paths that a block runs once or twice cost 100 us a launch when they were there.  So there is one
// instance of the pass over a pair's scores, and everything that runs once a block or rarely is a rolled loop.
//
// Registers: the roles' warpgroup gives most of its registers to the softmax warpgroups (setmaxnreg).
// Tensor memory (all 512 columns): scores 128, O of each query tile 128, P of each query tile 64 (128 keys as
// bfloat16).  Tiles late in a sequence see more keys: blocks start in the order of their tiles' lengths, all kv
// heads of the longest tile first, so that the longest blocks do not run last.  V is used as it lies in the cache,
// [key][d], through an MN-major operand descriptor.  Every wait on a barrier is bounded: a block that gives up
// records status 3, frees its tensor memory and ends.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {
constexpr int BM = 128, BN = 64;
constexpr int BOX_BYTES = 128;              // a row of a copied box: 64 numbers of d
constexpr int Q_BOX = BM * BOX_BYTES, KV_BOX = BN * BOX_BYTES;   // 16 KB and 8 KB: a tile's rows by 64 numbers of d
constexpr int K_PAIRS = 3, V_PAIRS = 2;     // rings of pairs of key tiles and of value tiles (the keys are asked for earlier: the scores run a pair ahead)
constexpr int K_SLOTS = 2 * K_PAIRS, V_SLOTS = 2 * V_PAIRS;
constexpr int THREADS = 384;   // a warpgroup of roles (producer, two MMA issuers, a spare warp) and one of softmax warps for each query tile
// Registers a thread: what the block is launched with (384 threads: 65536 / 384, rounded down to a multiple of 8), and
// what the warpgroups have after trading.  A warpgroup that asks for more waits, without a limit, until others of its
// own block have given that much back: the roles' warpgroup must free at least what the two softmax warpgroups take.
constexpr int LAUNCH_REGS = 168, ROLE_REGS = 56, SOFTMAX_REGS = 224;
static_assert((LAUNCH_REGS - ROLE_REGS) * 128 >= (SOFTMAX_REGS - LAUNCH_REGS) * (THREADS - 128), "the softmax warpgroups would wait for registers that nobody frees");
constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr float LOG2E = 1.4426950408889634f;
// Tensor memory: the scores of a pair of key tiles in columns 0..127, one buffer that the two query tiles take in
// turns (a tile's softmax warps read their scores into registers and hand it on); O of tile t, HD columns, from
// 128 + HD t; P of tile t, bfloat16, 128 keys in 64 columns, after them.
constexpr int TMEM_COLS = 512;              // two query tiles: all of an SM's tensor memory
constexpr int S_COL = 0, O_COL = 128, P_COLS = 64;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_3d(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n"
        ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
// Operand descriptors for tiles with the 128-byte swizzle.  K-major: rows of 128 bytes (64 elements of the
// reduction), groups of 8 rows 1024 bytes apart.  MN-major: rows of 128 bytes hold 64 elements of the M/N
// side, 8 rows (steps of the reduction) per 1024-byte group; `lbo` is the distance between blocks of 64
// M/N elements, `sbo` between groups of 8 reduction steps.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t addr) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
// bfloat16 x bfloat16 -> float, M = 128; b_mn: the B operand is MN-major.
__device__ __forceinline__ uint32_t idesc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t id, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(id), "r"((uint32_t)accumulate) : "memory");
}
// The same with the A operand in tensor memory (rows are lanes; 16 bfloat16 of the reduction are 8 columns).
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t id, bool accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(id), "r"((uint32_t)accumulate) : "memory");
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,"
        "%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
// 2^x on the special-function unit (x <= 0 here; -inf gives 0).
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Two floats in one 64-bit register, for the instructions that work on such pairs, and the maximum of three.
__device__ __forceinline__ uint64_t pair(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpair(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;\n" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma_pair(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ uint64_t add_pair(uint64_t a, uint64_t b) {
    uint64_t r;
    asm("add.rn.f32x2 %0, %1, %2;\n" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;\n" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct Params {
    __nv_bfloat16* out;        // [tokens, nq, HD]
    const int* q_start;        // [seqs + 1]
    const int* positions;      // [tokens]
    const int* block_table;    // [seqs, table_stride]
    int* status;
    int n_seqs, nq, nkv, group, tq, table_stride, page_size, page_shift, window, box_rows;
    int per_block;   // query tiles a block takes: 2 (they share each key tile) or, for small steps, 1 (more blocks)
    float scale_log2;
    // With n_splits > 1 (a step so small that whole tiles would leave SMs without work) blockIdx.z takes one of that
    // many runs of the tile's key tiles and leaves its share, O not yet divided by the row's sum, with the row's
    // (reference maximum, sum); a second kernel adds the shares.
    int n_splits, n_rows;          // n_rows = tokens * nq
    float* part_o;                 // [n_splits][n_rows][HD]
    float* part_ml;                // [n_splits][n_rows][2]
};

// One block: two neighbouring query tiles (A and B, 128 rows each) of one sequence against one kv head.  Both use
// every key and value tile the block fetches, and while the softmax warps of one tile work the tensor cores
// serve the other.
template <int HD>
__global__ void __launch_bounds__(THREADS, 1) attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                   const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v,
                                                                   const Params p) {
    constexpr int BOXES = HD / 64;                      // boxes of 64 numbers of d in a head
    constexpr int Q_BYTES = BOXES * Q_BOX, KV_BYTES = BOXES * KV_BOX;   // a query tile; a key tile, and the same a value tile
    constexpr int O_COLS = HD, P_COL = O_COL + 2 * O_COLS;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = base;                               // [2 tiles][2 boxes][128 rows][128 B]
    // keys: [2 halves of d][K_SLOTS slots][64 rows][128 B], so that the same half of two neighbouring slots is one
    // run of 128 rows; values: [V_SLOTS slots][2 halves of d][64 rows][128 B]
    unsigned char* kv_smem = q_smem + 2 * Q_BYTES;
    unsigned char* k_smem = kv_smem;
    unsigned char* v_smem = kv_smem + K_SLOTS * KV_BYTES;
    // keys and values come and go by pairs of slots (a pair of key tiles is one step of every role)
    __shared__ __align__(8) uint64_t q_full, k_full[K_PAIRS], k_empty[K_PAIRS], v_full[V_PAIRS], v_empty[V_PAIRS], s_full[2], s_read[2], p_full[2], pv_done[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int s_failed, s_tile[3], s_warp_total[THREADS / 32];

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // (the same in every lane, and known to be)
    const int kvh = blockIdx.x;   // the kv head runs fastest, so that blocks start in the order of their tiles
    if (tid == 0) {
        s_failed = 0;
        mbar_init(&q_full, 1);
        for (int i = 0; i < K_PAIRS; ++i) {
            mbar_init(&k_full[i], 1);
            mbar_init(&k_empty[i], 1);
        }
        for (int i = 0; i < V_PAIRS; ++i) {
            mbar_init(&v_full[i], 1);
            mbar_init(&v_empty[i], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&s_full[t], 1);
            mbar_init(&p_full[t], 4);      // one arrival per softmax warp of the tile
            mbar_init(&s_read[t], 4);
            mbar_init(&pv_done[t], 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
        s_tile[0] = -1;
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&tmem_base_smem)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::);
    }
    // Which sequence and which pair of its tiles this block has: pairs are counted sequence by sequence, and handed
    // out from the last to the first (tiles late in a sequence see the most keys).  A block's start is a chain of
    // loads that wait for one another (the sequences' tokens, then the tile's position and its pages, then the
    // copies), each most of a microsecond, so whatever needs nothing from them runs while they are under way: the
    // first sequences' token counts are asked for before the stages are zeroed.
    const int pair_tokens = p.per_block * p.tq;
    int first_a = 0, first_n = 0;
    if (tid < p.n_seqs) {
        first_a = p.q_start[tid];
        first_n = p.q_start[tid + 1] - first_a;
    }
    // the key and value stages start as zeros: a part of a tile that is never fetched (beyond the sequence's end, a
    // page the request does not hold) must hold finite numbers, because a probability of zero still multiplies it
    for (int idx = tid; idx < (K_SLOTS + V_SLOTS) * KV_BYTES / 16; idx += THREADS)
        reinterpret_cast<uint4*>(kv_smem)[idx] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    {
        int before_all = 0;
        for (int chunk = 0; chunk < p.n_seqs; chunk += THREADS) {
            const int sq = chunk + tid;
            int a = first_a, n = first_n, pairs = 0;
            if (chunk > 0 && sq < p.n_seqs) {
                a = p.q_start[sq];
                n = p.q_start[sq + 1] - a;
            }
            if (sq < p.n_seqs) pairs = (n + pair_tokens - 1) / pair_tokens;
            int incl = pairs;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            __syncthreads();
            if (lane == 31) s_warp_total[warp] = incl;
            __syncthreads();
            int before = before_all, total = 0;
#pragma unroll
            for (int w = 0; w < THREADS / 32; ++w) {
                if (w < warp) before += s_warp_total[w];
                total += s_warp_total[w];
            }
            const int mine = (int)(gridDim.y - 1 - blockIdx.y) - (before + incl - pairs);
            if (pairs > 0 && mine >= 0 && mine < pairs) {
                s_tile[0] = sq;
                s_tile[1] = a + mine * pair_tokens;
                s_tile[2] = min(pair_tokens, n - mine * pair_tokens);
            }
            before_all += total;
        }
    }
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_base_smem;
    const int seq = s_tile[0], tok0 = s_tile[1], n_tok = s_tile[2];
    const bool two = n_tok > p.tq;   // the second tile has rows
    const int* table = seq >= 0 ? p.block_table + (size_t)seq * p.table_stride : nullptr;
    // The queries need the tile's first token only, and without a window the pages are read from the table's start:
    // both are asked for before the tile's position is here.
    int early[3] = {-1, -1, -1};   // the producer's first three runs of 32 table entries
    if (warp == 0 && seq >= 0) {
        if (lane == 0) {
            mbar_expect_tx(&q_full, two ? 2 * Q_BYTES : Q_BYTES);
            for (int t = 0; t < (two ? 2 : 1); ++t) {
#pragma unroll
                for (int x = 0; x < BOXES; ++x)
                    tma_3d(q_smem + t * Q_BYTES + x * Q_BOX, &map_q, &q_full, 64 * x, kvh * p.group, tok0 + t * p.tq);
            }
        }
        if (p.window == 0 && p.n_splits == 1) {
#pragma unroll
            for (int i = 0; i < 3; ++i) early[i] = 32 * i + lane < p.table_stride ? table[32 * i + lane] : -1;
        }
    }
    int n_kt = 0, kt_lo = 0, pos0 = 0, pos_last = 0, lo_first = 0;
    if (seq >= 0) {
        pos0 = p.positions[tok0];
        lo_first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
        pos_last = pos0 + n_tok - 1;
        kt_lo = lo_first / BN;
        n_kt = pos_last / BN - kt_lo + 1;
        if (p.n_splits > 1) {   // this block's run of the key tiles (it may be empty)
            const int per = (n_kt + p.n_splits - 1) / p.n_splits;
            const int first = min(n_kt, (int)blockIdx.z * per), last = min(n_kt, first + per);
            kt_lo += first;
            n_kt = last - first;
        }
    }
    const int n_pairs = (n_kt + 1) / 2;
    // (the softmax warps hold a row's 128 scores in registers: the warpgroup of roles hands them most of its own,
    // every warp of a warpgroup as the first thing in its branch)

    if (warp == 0 && seq >= 0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(ROLE_REGS));
        // ---- producer.  A copy brings one box (a page's keys or values of one tile, or 64 of them if pages are
        // larger) of one half of d; the copies of a pair of tiles (at most 32) are issued by as many lanes at once,
        // because a thread that issues them one after another takes longer than the tensor cores take for the
        // pair.  The warp holds the part of the block table that the copies are about to need in registers (three
        // runs of 32 entries, the last one still on its way), so that no copy waits for a load of its page's number
        // from global memory.
        constexpr uint32_t FULL = 0xffffffffu;
        int win = ((kt_lo * BN) >> p.page_shift) & ~31;   // the table entry that lane 0 of `cur` holds
        auto entries = [&](int first) {
            const int e = first + lane;
            return e < p.table_stride ? table[e] : -1;
        };
        const bool had = p.window == 0 && p.n_splits == 1;   // (then win is 0 and the entries were asked for above)
        int cur = had ? early[0] : entries(win), nxt = had ? early[1] : entries(win + 32), far = had ? early[2] : entries(win + 64);
        auto wait = [&](uint64_t* bar, uint32_t parity) {
            int done = lane == 0 ? (int)mbar_wait(bar, parity) : 1;
            return __shfl_sync(FULL, done, 0) != 0;
        };
        // this lane's copy within a pair: which tile of the pair, which box of the tile, which half of d
        const int boxes = BN / p.box_rows, per_tile = BOXES * boxes;
        const int my_tile = lane / per_tile, my_box = (lane % per_tile) / BOXES, my_half = lane % BOXES;
        const uint32_t copy_bytes = p.box_rows * 64 * 2u;
        // the copies of tiles first .. first + n - 1 (keys when `keys`, else values) into their slots, counted by `bar`
        auto fetch = [&](int first, int n, bool keys, uint64_t* bar) {
            // move the table's registers on so that the pair's last entry lies in them (no pair reaches back more
            // than 32 entries behind the furthest entry asked for so far)
            const int e_last = min((kt_lo + first + n) * BN - 1, pos_last) >> p.page_shift;
            while (e_last >= win + 64) {
                cur = nxt;
                nxt = far;
                win += 32;
                far = entries(win + 64);
            }
            const int i = first + my_tile, kp = (kt_lo + i) * BN + my_box * p.box_rows, e = kp >> p.page_shift;
            const int a = __shfl_sync(FULL, cur, e & 31), b = __shfl_sync(FULL, nxt, e & 31);
            const int page = e < win + 32 ? a : b;
            bool mine = my_tile < n && kp <= pos_last && kp + p.box_rows > lo_first;
            if (mine && page < 0) {   // a page the request does not hold: an error of the caller
                atomicExch(p.status, 2);
                mine = false;
            }
            const uint32_t copies = __popc(__ballot_sync(FULL, mine));
            if (lane == 0) mbar_expect_tx(bar, copies * copy_bytes);
            __syncwarp();
            if (mine) {
                const int st = i % (keys ? K_SLOTS : V_SLOTS);
                const int row = (page * p.nkv + kvh) * p.page_size + (kp & (p.page_size - 1));
                unsigned char* dst = keys ? k_smem + st * KV_BOX + my_half * (K_SLOTS * KV_BOX)
                                          : v_smem + st * KV_BYTES + my_half * KV_BOX;
                tma_2d(dst + my_box * p.box_rows * 128, keys ? &map_k : &map_v, bar, my_half * 64, row);
            }
            __syncwarp();
        };
        bool ok = true;
        // A pair's key slots are free once the scores of the pair K_PAIRS before are formed, its value slots once the
        // probabilities of the pair V_PAIRS before have been multiplied with them.  The keys are asked for a pair
        // ahead of the values (the scores of a pair are formed while the softmax of the pair before still runs).
        auto keys_of = [&](int j) {
            if (j >= K_PAIRS && !wait(&k_empty[j % K_PAIRS], (j / K_PAIRS - 1) & 1)) return false;
            fetch(2 * j, min(2, n_kt - 2 * j), true, &k_full[j % K_PAIRS]);
            return true;
        };
        if (n_pairs > 0) ok = keys_of(0);
        for (int j = 0; j < n_pairs && ok; ++j) {
            if (j + 1 < n_pairs && !keys_of(j + 1)) { ok = false; break; }
            if (j >= V_PAIRS && !wait(&v_empty[j % V_PAIRS], (j / V_PAIRS - 1) & 1)) { ok = false; break; }
            fetch(2 * j, min(2, n_kt - 2 * j), false, &v_full[j % V_PAIRS]);
        }
        if (!ok && lane == 0) atomicExch(&s_failed, 1);
    } else if ((warp == 1 || warp == 2) && seq >= 0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(ROLE_REGS));
        // ---- issuers of the MMAs: warp 1 the scores, warp 2 O += P V.  While one waits (for a barrier, or because
        // the tensor cores' queue is full: an MMA is taken only when an earlier one has left it) the other issues.
        // The whole warp runs the loop with everything it computes the same in every lane (so that operand
        // descriptors can live in the warp's uniform registers), and one elected lane issues.
        constexpr uint32_t FULL = 0xffffffffu;
        const uint32_t tm = __shfl_sync(FULL, tmem, 0);
        const int n_pairs_u = __shfl_sync(FULL, n_pairs, 0), n_kt_u = __shfl_sync(FULL, n_kt, 0);
        const int n_t = __shfl_sync(FULL, two ? 2 : 1, 0);
        const uint32_t q_addr = __shfl_sync(FULL, smem_u32(q_smem), 0);
        const int jobs = n_pairs_u * n_t;   // a job is (pair of key tiles, query tile), pair by pair, tile by tile
        auto wait = [&](uint64_t* bar, uint32_t parity) {
            int done = lane == 0 ? (int)mbar_wait(bar, parity) : 1;
            return __shfl_sync(FULL, done, 0) != 0;
        };
        bool ok = true;
        if (warp == 1) {
            // S = Q K^T of the pair j of key tiles (two neighbouring slots: 128 rows of keys) for query tile t into
            // the score columns: the reduction runs over d, 8 steps of 16; d 0..63 lie in the first half of the key
            // region, 64..127 in the second.  (If the pair's second tile does not exist, its columns are never
            // used.)  The score columns pass from job to job: job k's scores may be formed once the warps of job
            // k - 1 have theirs in registers.
            const uint32_t id_s = idesc(2 * BN, false);
            const uint64_t q_desc0 = desc_kmajor(q_addr);
            const uint64_t k_desc0 = desc_kmajor(q_addr + 2 * Q_BYTES);
            ok = wait(&q_full, 0);
            int t = 0, j = 0;
            for (int k = 0; k < jobs && ok; ++k) {
                if (t == 0 && !wait(&k_full[j % K_PAIRS], (j / K_PAIRS) & 1)) { ok = false; break; }
                if (k > 0) {
                    const int pt = t == 0 ? n_t - 1 : t - 1, pj = t == 0 ? j - 1 : j;
                    if (!wait(&s_read[pt], pj & 1)) { ok = false; break; }
                }
                fence_after();
                const uint64_t q_desc = q_desc0 + (uint64_t)((t * Q_BYTES) >> 4);
                const uint64_t k_desc = k_desc0 + (uint64_t)(((j % K_PAIRS) * 2 * KV_BOX) >> 4);
                const uint32_t d_addr = tm + S_COL;
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < HD / 16; ++kk)
                        umma(d_addr, q_desc + (uint64_t)(((kk >> 2) * Q_BOX + (kk & 3) * 32) >> 4),
                             k_desc + (uint64_t)(((kk >> 2) * (K_SLOTS * KV_BOX) + (kk & 3) * 32) >> 4), id_s, kk > 0);
                    umma_commit(&s_full[t]);
                    if (t == n_t - 1) umma_commit(&k_empty[j % K_PAIRS]);   // the pair's keys are free after the last tile's scores
                }
                __syncwarp();
                if (++t == n_t) { t = 0; ++j; }
            }
        } else {
            // O += P V of the pair's tiles: the probabilities come from tensor memory (16 keys are 8 columns), the
            // reduction runs over a tile's 64 keys in 4 steps of 16; V is [key][d], MN-major: blocks of 64 d are 8 KB
            // apart, groups of 8 keys 1 KB
            const uint32_t id_o = idesc(HD, true);
            const uint64_t v_desc0 = desc_mnmajor(q_addr + 2 * Q_BYTES + K_SLOTS * KV_BYTES, KV_BOX, 1024);
            int t = 0, j = 0;
            for (int k = 0; k < jobs && ok; ++k) {
                if (t == 0 && !wait(&v_full[j % V_PAIRS], (j / V_PAIRS) & 1)) { ok = false; break; }
                if (!wait(&p_full[t], j & 1)) { ok = false; break; }
                fence_after();
                const int tiles = min(2, n_kt_u - 2 * j);
                const uint32_t d_addr = tm + O_COL + t * O_COLS, a_addr = tm + P_COL + t * P_COLS;
                const uint64_t v_desc = v_desc0 + (uint64_t)((((2 * j) % V_SLOTS) * KV_BYTES) >> 4);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < BN / 16; ++kk)
                        umma_ts(d_addr, a_addr + kk * 8, v_desc + (uint64_t)((kk * 2048) >> 4), id_o, j > 0 || kk > 0);
                    if (tiles == 2) {
#pragma unroll
                        for (int kk = 0; kk < BN / 16; ++kk)
                            umma_ts(d_addr, a_addr + (BN / 16 + kk) * 8, v_desc + (uint64_t)((KV_BYTES + kk * 2048) >> 4), id_o, true);
                    }
                    umma_commit(&pv_done[t]);
                    if (t == n_t - 1) umma_commit(&v_empty[j % V_PAIRS]);   // every query tile is done with the pair's values
                }
                __syncwarp();
                if (++t == n_t) { t = 0; ++j; }
            }
        }
        if (!ok && lane == 0) atomicExch(&s_failed, 1);
    } else if (warp < 4 && seq >= 0) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;\n" ::"n"(ROLE_REGS));   // the spare warps of the roles' warpgroup
    } else if (warp >= 4 && seq >= 0 && (warp < 8 || two)) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;\n" ::"n"(SOFTMAX_REGS));
        // ---- softmax of query tile t: thread owns row r of the tile = lane r of tensor memory
        const int t = warp < 8 ? 0 : 1;
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t lane_base = tmem + ((uint32_t)(quad * 32) << 16);
        const uint32_t s_addr = lane_base + S_COL, o_addr = lane_base + O_COL + t * O_COLS, p_addr = lane_base + P_COL + t * P_COLS;
        const int tile_tok0 = tok0 + t * p.tq;
        const int tile_tokens = min(p.tq, n_tok - t * p.tq);
        const int rows_valid = tile_tokens * p.group;
        const bool row_ok = r < rows_valid;
        const int tok = row_ok ? r / p.group : 0;
        const int row_pos = pos0 + t * p.tq + tok;
        const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
        const uint64_t scale2 = pair(p.scale_log2, p.scale_log2);
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int j = 0; j < n_pairs; ++j) {
            const int tiles = min(2, n_kt - 2 * j);
            const int k0 = (kt_lo + 2 * j) * BN;   // the pair's first key
            ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], j & 1));
            if (!ok) break;
            fence_after();
            // A pair that some row of this warp does not see whole (the diagonal, the window's edge, rows past the
            // tile's end, a missing second key tile) is masked first, in a rolled loop that takes the scores through
            // registers back into tensor memory with -inf where the row must not look: such pairs are few, and the
            // code for all that follows is the same for every pair (code that a block runs once costs more to
            // fetch than to run).
            const bool whole = __all_sync(0xffffffffu, row_ok && k0 + tiles * BN - 1 <= row_pos && k0 >= row_lo);
            if (!whole) {
                // key k0 + i is seen if lo <= i <= hi
                const int lo = row_lo - k0, hi = row_ok ? min(row_pos - k0, tiles * BN - 1) : -1 << 20;
#pragma unroll 1
                for (int c = 0; c < 2 * BN; c += 32) {
                    uint32_t w[32];
                    tmem_ld32(s_addr + c, w);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) w[i] = (c + i >= lo && c + i <= hi) ? w[i] : 0xff800000u;   // -inf
                    tmem_st32(s_addr + c, w);
                }
                tmem_st_wait();
            }
            // the row's scores of the pair, all in registers
            uint32_t v[4][32];
#define SCORE(i) __uint_as_float(v[(i) >> 5][(i) & 31])
            tmem_ld32(s_addr, v[0]);
            tmem_ld32(s_addr + 32, v[1]);
            tmem_ld_wait();
            tmem_ld32(s_addr + 64, v[2]);   // (of a pair's missing second tile: never used)
            tmem_ld32(s_addr + 96, v[3]);
            tmem_ld_wait();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&s_read[t]);   // the scores are in registers: their columns may go to the next job
            if (j > 0) {
                // the MMAs of the pair before have read its probabilities and added into O: both may be written now
                ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[t], (j - 1) & 1));
                if (!ok) break;
                fence_after();
            }
            // Exponents against the reference `ref` and the row's sum, two numbers at a time (fma and add on pairs of
            // floats); the probabilities go into tensor memory as bfloat16, 32 keys in 16 columns.  With `track` the
            // largest exponent is kept as well.
            auto emit = [&](float ref, float& largest) {
                const uint64_t ref2 = pair(-ref, -ref);
                uint64_t sum_a = pair(0.f, 0.f), sum_b = pair(0.f, 0.f);
                float x0 = -INFINITY, x1 = -INFINITY, x2 = -INFINITY, x3 = -INFINITY;
                uint32_t pk[2][16];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (c < 2 || tiles == 2) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            float e0, e1, e2, e3;
                            unpair(fma_pair(pair(SCORE(32 * c + i), SCORE(32 * c + i + 1)), scale2, ref2), e0, e1);
                            unpair(fma_pair(pair(SCORE(32 * c + i + 2), SCORE(32 * c + i + 3)), scale2, ref2), e2, e3);
                            if (i & 4) {
                                x2 = max3(x2, e0, e1);
                                x3 = max3(x3, e2, e3);
                            } else {
                                x0 = max3(x0, e0, e1);
                                x1 = max3(x1, e2, e3);
                            }
                            const float a0 = ex2(e0), a1 = ex2(e1), a2 = ex2(e2), a3 = ex2(e3);
                            sum_a = add_pair(sum_a, pair(a0, a1));
                            sum_b = add_pair(sum_b, pair(a2, a3));
                            pk[c & 1][i / 2] = pack_bf16(a0, a1);
                            pk[c & 1][i / 2 + 1] = pack_bf16(a2, a3);
                            // (a chunk is stored while the next one's exponentials are on their way: a store right
                            // after its own chunk would hold them back until the chunk's last exponential is there)
                            if (c > 0 && i == 16) tmem_st16(p_addr + 16 * (c - 1), pk[(c - 1) & 1]);
                        }
                    }
                }
                tmem_st16(p_addr + 16 * (tiles == 2 ? 3 : 1), pk[1]);
                float sum_even, sum_odd;
                unpair(add_pair(sum_a, sum_b), sum_even, sum_odd);
                largest = fmaxf(fmaxf(x0, x1), fmaxf(x2, x3));
                return sum_even + sum_odd;
            };
            // m is the reference the exponentials are taken against, not the true maximum: it moves only when a
            // score exceeds it by more than 8 (probabilities then stay below 2^8, far from overflow), so that O, which
            // sits in tensor memory, has to be rescaled only rarely.  A pair is therefore tried against the reference
            // as it stands, in one pass that also keeps the largest exponent; only if that shows a score more than 8
            // above the reference (or a row has no reference yet) is the pair done the long way: maximum, new
            // reference, O rescaled, and the same pass once more.
            bool long_way = !__all_sync(0xffffffffu, m != -INFINITY);
            float ref = m, corr = 1.f, sum;
#pragma unroll 1
            for (;;) {
                if (long_way) {
                    float c0 = -INFINITY, c1 = -INFINITY, c2 = -INFINITY, c3 = -INFINITY;   // four chains, so that none waits for the last
#pragma unroll
                    for (int i = 0; i < 2 * BN; i += 8) {
                        if (i < BN || tiles == 2) {
                            c0 = max3(c0, SCORE(i), SCORE(i + 1));
                            c1 = max3(c1, SCORE(i + 2), SCORE(i + 3));
                            c2 = max3(c2, SCORE(i + 4), SCORE(i + 5));
                            c3 = max3(c3, SCORE(i + 6), SCORE(i + 7));
                        }
                    }
                    float mx = fmaxf(fmaxf(c0, c1), fmaxf(c2, c3));
                    mx = mx == -INFINITY ? mx : mx * p.scale_log2;
                    const float m_new = (m == -INFINITY || mx > m + 8.f) ? fmaxf(m, mx) : m;
                    corr = m_new == -INFINITY ? 1.f : ex2(m - m_new);
                    ref = m_new == -INFINITY ? 0.f : m_new;
                    m = m_new;
                    if (j > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
                        // the reference of some row of this warp moved: rescale O
#pragma unroll 1
                        for (int c = 0; c < HD; c += 32) {
                            uint32_t o[32];
                            tmem_ld32(o_addr + c, o);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                            tmem_st32(o_addr + c, o);
                        }
                    }
                }
                float largest;
                sum = emit(ref, largest);
                if (long_way || !__any_sync(0xffffffffu, largest > 8.f)) break;
                long_way = true;
            }
            l = l * corr + sum;
#undef SCORE
            // positions past the sequence's end lie in a fetched page but were never written: their values must
            // not reach the sum, not even multiplied by zero.  Only the tile that holds the end has such keys; the
            // first query tile's warps clear them (both tiles' MMAs wait for these warps' arrival or come after it).
            if (t == 0 && k0 + tiles * BN - 1 > pos_last) {
                // (the values must have arrived, or they would land on top of the zeros)
                ok = __all_sync(0xffffffffu, mbar_wait(&v_full[j % V_PAIRS], (j / V_PAIRS) & 1));
                if (!ok) break;
                const int kt_end = pos_last / BN - kt_lo;   // the tile that holds the end, counted from this block's first
                unsigned char* vd = v_smem + (kt_end % V_SLOTS) * KV_BYTES;
                const int first_bad = pos_last + 1 - (kt_lo + kt_end) * BN;
                constexpr int CHUNKS = HD / 8;   // chunks of 16 bytes in a row: eight in every box
                for (int idx = quad * 32 + lane; idx < (BN - first_bad) * CHUNKS; idx += 128) {
                    const int row = first_bad + idx / CHUNKS, c = idx % CHUNKS;
                    *reinterpret_cast<uint4*>(vd + (c >> 3) * KV_BOX + row * 128 + ((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            tmem_st_wait();
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[t]);
        }
        if (ok && n_kt > 0) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[t], (n_pairs - 1) & 1));
        if (ok) {
            fence_after();
            const int g = r - tok * p.group;
            const size_t row = (size_t)(tile_tok0 + tok) * p.nq + kvh * p.group + g;
            if (p.n_splits > 1) {
                // this run's share of the row (a run without keys leaves maximum -inf and sum 0, and no numbers)
                float* dst = p.part_o + ((size_t)blockIdx.z * p.n_rows + row) * HD;
                if (n_kt > 0) {
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {   // (rolled, like every loop that runs once a block: code that is fetched once costs more than it saves)
                        uint32_t v[32];
                        tmem_ld32(o_addr + c, v);
                        tmem_ld_wait();
                        if (row_ok) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(dst + c + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                                      __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        }
                    }
                }
                if (row_ok) *reinterpret_cast<float2*>(p.part_ml + ((size_t)blockIdx.z * p.n_rows + row) * 2) = make_float2(m, l);
            } else if (n_kt > 0) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                __nv_bfloat16* dst = p.out + row * HD;
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(o_addr + c, v);
                    tmem_ld_wait();
                    if (row_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 o4;
                            o4.x = pack_bf16(__uint_as_float(v[j]) * inv, __uint_as_float(v[j + 1]) * inv);
                            o4.y = pack_bf16(__uint_as_float(v[j + 2]) * inv, __uint_as_float(v[j + 3]) * inv);
                            o4.z = pack_bf16(__uint_as_float(v[j + 4]) * inv, __uint_as_float(v[j + 5]) * inv);
                            o4.w = pack_bf16(__uint_as_float(v[j + 6]) * inv, __uint_as_float(v[j + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + c + j) = o4;
                        }
                    }
                }
            }
        }
        if (!ok) atomicExch(&s_failed, 1);
    }
    __syncwarp();
    fence_before();
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(TMEM_COLS));
    if (tid == 0 && s_failed) atomicExch(p.status, 3);
}

// out[row] = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z over the runs z of the row's keys, in run order.
// A warp a row; a lane has HD / 32 neighbouring numbers of it.
template <int HD>
__global__ void __launch_bounds__(128) attention_tcgen05_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                      __nv_bfloat16* __restrict__ out, int n_rows, int n_splits,
                                                                      int first_row, int rows) {
    constexpr int PER = HD / 32;
    const int lane = threadIdx.x & 31;
    if (blockIdx.x * 4 + (threadIdx.x >> 5) >= rows) return;
    const int row = first_row + blockIdx.x * 4 + (threadIdx.x >> 5);
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, part_ml[((size_t)z * n_rows + row) * 2]);
    float L = 0.f;
    float acc[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = 0.f;
    for (int z = 0; z < n_splits; ++z) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((size_t)z * n_rows + row) * 2);
        if (ml.x == -INFINITY) continue;
        const float f = exp2f(ml.x - M);
        const float* src = part_o + ((size_t)z * n_rows + row) * HD + lane * PER;
        L += f * ml.y;
#pragma unroll
        for (int i = 0; i < PER; i += 2) {
            const float2 v = *reinterpret_cast<const float2*>(src + i);
            acc[i] += f * v.x;
            acc[i + 1] += f * v.y;
        }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    __nv_bfloat16* dst = out + (size_t)row * HD + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; i += 2) *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16(acc[i] * inv, acc[i + 1] * inv);
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encoder() {
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

struct MapKey {
    const void* base;
    long long a, b;
    int c, d;
    bool operator==(const MapKey& o) const { return base == o.base && a == o.a && b == o.b && c == o.c && d == o.d; }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.base) ^ (std::hash<long long>()(k.a) * 31) ^ (std::hash<long long>()(k.b) * 131) ^
               (size_t)(k.c * 7 + k.d);
    }
};
std::mutex g_lock;
std::unordered_map<MapKey, CUtensorMap, MapHash> g_maps;

// A pool of one layer as [rows, hd] bfloat16; boxes of [box_rows, 64].
int pool_map(CUtensorMap* map, const void* base, long long rows, int box_rows, int hd) {
    std::lock_guard<std::mutex> guard(g_lock);
    const MapKey key{base, rows, hd, box_rows, 2};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *map = it->second; return 0; }
    EncodeTiled fn = encoder();
    if (!fn) RMX_FAIL("attention_tcgen05: the driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RMX_FAIL("attention_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, *map);
    return 0;
}

// The queries [tokens, nq, hd]; boxes of [tq tokens, group heads, 64]: a tile's rows come out token by token, the
// group's heads side by side.
int q_map(CUtensorMap* map, const void* base, long long tokens, int nq, int group, int tq, int hd) {
    std::lock_guard<std::mutex> guard(g_lock);
    const MapKey key{base, tokens, (long long)nq * 1024 + hd, group, 3};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *map = it->second; return 0; }
    EncodeTiled fn = encoder();
    if (!fn) RMX_FAIL("attention_tcgen05: the driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nq, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)nq * hd * 2};
    cuuint32_t box[3] = {64, (cuuint32_t)group, (cuuint32_t)tq};
    cuuint32_t elem[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RMX_FAIL("attention_tcgen05: cuTensorMapEncodeTiled (queries) failed with code %d", (int)r);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, *map);
    return 0;
}
template <int HD>
int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const Params& p, int n_tiles, int first_token,
           int run_tokens, cudaStream_t stream) {
    constexpr size_t smem = 1024 + (size_t)(HD / 64) * (2 * Q_BOX + (K_SLOTS + V_SLOTS) * KV_BOX);
    static bool raised[64] = {};
    if (rmx_first_on_device(raised)) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RMX_FAIL("attention_tcgen05: shared memory of %zu bytes refused: %s", smem, cudaGetErrorString(e));
        cudaFuncAttributes fa;
        e = cudaFuncGetAttributes(&fa, attention_tcgen05_kernel<HD>);
        if (e != cudaSuccess || fa.numRegs != LAUNCH_REGS)   // the trade of registers between the warpgroups is worked out for this number
            RMX_FAIL("attention_tcgen05: built with %d registers a thread, not %d", e == cudaSuccess ? fa.numRegs : -1, LAUNCH_REGS);
    }
    // blocks are handed to the SMs in the order x, then y: all kv heads of the tile that sees the most keys first
    attention_tcgen05_kernel<HD><<<dim3(p.nkv, n_tiles, p.n_splits), THREADS, smem, stream>>>(mq, mk, mv, p);
    RMX_CHECK_LAUNCH("attention_tcgen05");
    if (p.n_splits > 1) {
        attention_tcgen05_merge_kernel<HD><<<(run_tokens * p.nq + 3) / 4, 128, 0, stream>>>(p.part_o, p.part_ml, p.out, p.n_rows, p.n_splits,
                                                                                          first_token * p.nq, run_tokens * p.nq);
        RMX_CHECK_LAUNCH("attention_tcgen05_merge");
    }
    return 0;
}
}  // namespace

// Head size 64 or 128, a group that divides 128, pages of at least 8 positions (a power of two).
RMX_API int rmx_attention_tcgen05_supports(int hd, int group, int page_size) {
    return (hd == 64 || hd == 128) && group >= 1 && group <= 16 && (group & (group - 1)) == 0 && page_size >= 8 &&
           (page_size & (page_size - 1)) == 0;
}

RMX_API int rmx_attention_tcgen05_tile_tokens(int group) { return BM / group; }

// tiles_per_block: 2 (a block takes two neighbouring query tiles of 128 rows, which share every key tile it fetches)
// or 1 (twice the blocks: for steps so small that two tiles a block would leave SMs without work).
// n_tiles: the number of blocks: sum over sequences of ceil(tokens / (tiles_per_block * 128 / group)).
// pool_pages: pages in k_pool / v_pool.
// n_splits > 1: every tile's keys in that many runs, one block each (blockIdx.z), added by a second kernel; part_o
// [n_splits, n_tokens * nq, hd] and part_ml [n_splits, n_tokens * nq, 2] floats are their scratch; the sequences
// given hold the step's tokens first_token .. first_token + run_tokens - 1 (only their rows of `out` are written).
RMX_API int rmx_attention_tcgen05(const void* q, const void* k_pool, const void* v_pool, const int* q_start,
                                  const int* positions, const int* block_table, int table_stride, int page_size,
                                  void* out, int n_seqs, int n_tokens, int n_tiles, int tiles_per_block, int nq, int nkv,
                                  int hd, int window, float scale, int pool_pages, int n_splits, float* part_o, float* part_ml,
                                  int first_token, int run_tokens, int* status, void* stream) {
    if (n_tokens == 0) return 0;
    RMX_REQUIRE(tiles_per_block == 1 || tiles_per_block == 2, "attention_tcgen05: a block takes 1 or 2 tiles, not %d", tiles_per_block);
    RMX_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_tcgen05: %d query heads over %d kv heads", nq, nkv);
    const int group = nq / nkv;
    RMX_REQUIRE(rmx_attention_tcgen05_supports(hd, group, page_size),
                "attention_tcgen05: head_dim %d, group %d, page size %d is not built", hd, group, page_size);
    RMX_REQUIRE(table_stride > 0 && window >= 0 && n_tiles > 0 && n_tiles <= 65535 && n_seqs > 0 && pool_pages > 0,
                "attention_tcgen05: bad geometry");
    RMX_REQUIRE(scale > 0.f, "attention_tcgen05: the scale must be positive (the maximum is taken before scaling)");
    RMX_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)k_pool & 127) == 0 && ((uintptr_t)v_pool & 127) == 0,
                "attention_tcgen05: operands must be aligned");
    Params p;
    p.out = (__nv_bfloat16*)out; p.q_start = q_start; p.positions = positions; p.block_table = block_table; p.status = status;
    p.n_seqs = n_seqs; p.nq = nq; p.nkv = nkv; p.group = group; p.tq = BM / group; p.table_stride = table_stride;
    p.page_size = page_size; p.window = window; p.box_rows = page_size < BN ? page_size : BN;
    p.per_block = tiles_per_block;
    RMX_REQUIRE(n_splits >= 1 && n_splits <= 64 && (n_splits == 1 || (part_o && part_ml)), "attention_tcgen05: %d runs of keys need room for their shares", n_splits);
    p.n_splits = n_splits; p.n_rows = n_tokens * nq; p.part_o = part_o; p.part_ml = part_ml;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.scale_log2 = scale * LOG2E;
    CUtensorMap mq, mk, mv;
    const long long pool_rows = (long long)pool_pages * nkv * page_size;
    if (q_map(&mq, q, n_tokens, nq, group, p.tq, hd) != 0) return -1;
    if (pool_map(&mk, k_pool, pool_rows, p.box_rows, hd) != 0) return -1;
    if (pool_map(&mv, v_pool, pool_rows, p.box_rows, hd) != 0) return -1;
    if (n_splits > 1)
        RMX_REQUIRE(first_token >= 0 && run_tokens > 0 && first_token + run_tokens <= n_tokens, "attention_tcgen05: the tokens of this launch are not among the step's");
    return hd == 64 ? launch<64>(mq, mk, mv, p, n_tiles, first_token, run_tokens, (cudaStream_t)stream)
                    : launch<128>(mq, mk, mv, p, n_tiles, first_token, run_tokens, (cudaStream_t)stream);
}
