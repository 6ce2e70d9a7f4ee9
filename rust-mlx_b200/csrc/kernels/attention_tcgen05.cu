// Attention for prompt portions on the Blackwell tensor cores (tcgen05), head size 128, bfloat16.
//
// A block takes one kv head and one tile of 128 query rows of one sequence; a row is a (token, query
// head of the group) pair, 128 / group tokens by `group` heads, so the heads that share a kv head share
// every key and value tile.  Keys are visited in tiles of 64 aligned to absolute positions.
//
// A block takes two neighbouring tiles, which share every key and value tile it fetches (or one, for steps so
// small that SMs would be left without work).
//
//   warp 0   producer: Q once and then K/V tiles by TMA (tensor-map boxes, 128-byte swizzle) into a ring
//   warps 1 and 10  issue the MMAs (warp 10 the scores, warp 1 O += P V, so that neither waits for what the
//            other waits for): S = Q K^T into tensor memory, for two neighbouring key tiles at once (an MMA of 128
//            rows by 64 columns takes as long as one of 128 columns, so the scores of a pair of key tiles cost
//            what one tile's would; the pair's key tiles lie in neighbouring slots of the ring, which makes them
//            one operand of 128 rows); the next pair's scores are formed as soon as the softmax warps have read
//            this pair's into registers; later O += P V, tile by tile
//   warps 2-5 and 6-9  softmax of the first and the second query tile: every thread owns one row (one lane
//            of tensor memory): it reads its 64 scores, masks where the tile touches the diagonal or the
//            window's edge, keeps the running maximum and sum in float, writes its probabilities as bfloat16
//            into shared memory for the second MMA, and rescales its row of O when the maximum moved
//
// S and O live in tensor memory (per query tile 128 columns of scores, a pair of key tiles, and 128 of O).  Tiles
// late in a sequence see more keys: blocks start in the order of their tiles' lengths, all kv heads of the longest
// tile first, so that the longest blocks do not run last.  V is used as it lies in the cache, [key][d], through an
// MN-major operand descriptor.  Every wait on a barrier is bounded: a block that gives up records status 3,
// frees its tensor memory and ends.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {
constexpr int HD = 128, BM = 128, BN = 64;
constexpr int STAGES = 4;                   // slots of the key/value ring, one key tile (and its value tile) each; pairs 0|1 and 2|3
constexpr int THREADS = 352;   // producer, O += P V issuer, 4 softmax warps for each of the block's two query tiles, score issuer
constexpr uint32_t SPIN_LIMIT = 1u << 24;
constexpr float LOG2E = 1.4426950408889634f;
constexpr int Q_BYTES = BM * HD * 2;        // 32 KB: two boxes of [128 rows][64 columns]
constexpr int KV_BYTES = BN * HD * 2;       // 16 KB per key tile, the same per value tile
constexpr int P_BYTES = BM * BN * 2;        // 16 KB
constexpr int TILE_COLS = 256;              // per query tile: S of a pair of key tiles in columns 0..63 and 64..127, O in 128..255
constexpr int TMEM_COLS = 512;              // two query tiles: all of an SM's tensor memory
constexpr int O_COL = 128;

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
__global__ void __launch_bounds__(THREADS) attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                   const __grid_constant__ CUtensorMap map_k,
                                                                   const __grid_constant__ CUtensorMap map_v,
                                                                   const Params p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = base;                               // [2 tiles][2 boxes][128 rows][128 B]
    // keys: [2 halves of d][STAGES slots][64 rows][128 B], so that the same half of two neighbouring slots is one
    // run of 128 rows; values: [STAGES slots][2 halves of d][64 rows][128 B]
    unsigned char* kv_smem = q_smem + 2 * Q_BYTES;
    unsigned char* k_smem = kv_smem;
    unsigned char* v_smem = kv_smem + STAGES * KV_BYTES;
    unsigned char* p_smem = kv_smem + STAGES * 2 * KV_BYTES;    // [2 tiles][128 rows][128 B]
    // keys come and go by pairs of slots (a pair's scores are one group of MMAs), values slot by slot
    __shared__ __align__(8) uint64_t q_full, k_full[2], k_empty[2], v_full[STAGES], v_empty[STAGES], s_full[2], s_read[2], p_full[2], o_done[2];
    __shared__ uint32_t tmem_base_smem;
    __shared__ int s_failed, s_tile[3], s_warp_total[THREADS / 32];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x;   // the kv head runs fastest, so that blocks start in the order of their tiles
    if (tid == 0) {
        s_failed = 0;
        mbar_init(&q_full, 1);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&v_full[s], 1);
            mbar_init(&v_empty[s], 1);
        }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&k_full[t], 1);
            mbar_init(&k_empty[t], 1);
            mbar_init(&s_full[t], 1);
            mbar_init(&s_read[t], 4);      // one arrival per softmax warp of the tile
            mbar_init(&p_full[t], 128);
            mbar_init(&o_done[t], 1);
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
    // which sequence and which pair of its tiles this block has: pairs are counted sequence by sequence, and handed
    // out from the last to the first (tiles late in a sequence see the most keys)
    {
        const int pair_tokens = p.per_block * p.tq;
        int before_all = 0;
        for (int chunk = 0; chunk < p.n_seqs; chunk += THREADS) {
            const int sq = chunk + tid;
            int a = 0, n = 0, pairs = 0;
            if (sq < p.n_seqs) {
                a = p.q_start[sq];
                n = p.q_start[sq + 1] - a;
                pairs = (n + pair_tokens - 1) / pair_tokens;
            }
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
    // the key and value stages start as zeros: a part of a tile that is never fetched (beyond the sequence's end, a
    // page the request does not hold) must hold finite numbers, because a probability of zero still multiplies it
    for (int idx = tid; idx < STAGES * 2 * KV_BYTES / 16; idx += THREADS)
        reinterpret_cast<uint4*>(kv_smem)[idx] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    fence_before();
    __syncthreads();
    fence_after();
    const uint32_t tmem = tmem_base_smem;
    const int seq = s_tile[0], tok0 = s_tile[1], n_tok = s_tile[2];
    int n_kt = 0, kt_lo = 0, pos0 = 0, pos_last = 0, lo_first = 0;
    const int* table = nullptr;
    if (seq >= 0) {
        pos0 = p.positions[tok0];
        table = p.block_table + (size_t)seq * p.table_stride;
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
    const bool two = n_tok > p.tq;   // the second tile has rows

    if (warp == 0 && seq >= 0) {
        // ---- producer.  A copy brings one box (a page's keys or values of one tile, or 64 of them if pages are
        // larger) of one half of d; the copies of a group (a pair of key tiles, or one value tile: at most 32) are
        // issued by as many lanes at once, because a thread that issues them one after another takes longer than the
        // tensor cores take for the tile.  The warp holds the part of the block table that the copies are about to
        // need in registers (three runs of 32 entries, the last one still on its way), so that no copy waits for a
        // load of its page's number from global memory.
        constexpr uint32_t FULL = 0xffffffffu;
        if (lane == 0) {
            mbar_expect_tx(&q_full, two ? 2 * Q_BYTES : Q_BYTES);
            for (int t = 0; t < (two ? 2 : 1); ++t) {
                tma_3d(q_smem + t * Q_BYTES, &map_q, &q_full, 0, kvh * p.group, tok0 + t * p.tq);
                tma_3d(q_smem + t * Q_BYTES + Q_BYTES / 2, &map_q, &q_full, 64, kvh * p.group, tok0 + t * p.tq);
            }
        }
        int win = ((kt_lo * BN) >> p.page_shift) & ~31;   // the table entry that lane 0 of `cur` holds
        auto entries = [&](int first) {
            const int e = first + lane;
            return e < p.table_stride ? table[e] : -1;
        };
        int cur = entries(win), nxt = entries(win + 32), far = entries(win + 64);
        auto wait = [&](uint64_t* bar, uint32_t parity) {
            int done = lane == 0 ? (int)mbar_wait(bar, parity) : 1;
            return __shfl_sync(FULL, done, 0) != 0;
        };
        // this lane's copy within a group: which tile of the group, which box of the tile, which half of d
        const int boxes = BN / p.box_rows, per_tile = 2 * boxes;
        const int my_tile = lane / per_tile, my_box = (lane % per_tile) >> 1, my_half = lane & 1;
        const uint32_t copy_bytes = p.box_rows * 64 * 2u;
        // the copies of tiles first .. first + n - 1 (keys when `keys`, else values) into their slots, counted by `bar`
        auto fetch = [&](int first, int n, bool keys, uint64_t* bar) {
            // move the table's registers on so that the group's last entry lies in them (no group reaches back more
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
                const int st = i % STAGES;
                const int row = (page * p.nkv + kvh) * p.page_size + (kp & (p.page_size - 1));
                unsigned char* dst = keys ? k_smem + st * (KV_BYTES / 2) + my_half * (STAGES * KV_BYTES / 2)
                                          : v_smem + st * KV_BYTES + my_half * (KV_BYTES / 2);
                tma_2d(dst + my_box * p.box_rows * 128, keys ? &map_k : &map_v, bar, my_half * 64, row);
            }
            __syncwarp();
        };
        bool ok = true;
        for (int i = 0; i < n_kt && ok; ++i) {
            if ((i & 1) == 0) {   // the keys of the pair of tiles i, i + 1: their slots are free once the scores of the pair before last are formed
                const int j = i >> 1;
                if (j >= 2 && !wait(&k_empty[j & 1], ((j >> 1) - 1) & 1)) { ok = false; break; }
                fetch(i, min(2, n_kt - i), true, &k_full[j & 1]);
            }
            const int st = i % STAGES, round = i / STAGES;
            if (round > 0 && !wait(&v_empty[st], (round - 1) & 1)) { ok = false; break; }
            fetch(i, 1, false, &v_full[st]);
        }
        if (!ok && lane == 0) atomicExch(&s_failed, 1);
    } else if (warp == 10 && lane == 0 && seq >= 0) {
        // ---- issuer of the score MMAs.  One thread issues them all, so what it executes per MMA counts: the operand
        // descriptors are formed before the loop (those of Q do not change; those of K differ by the pair's address,
        // which is added to the descriptor's low bits), and the loops are unrolled.
        const uint32_t id_s = idesc(2 * BN, false);
        const int n_t = two ? 2 : 1;
        uint64_t q_desc[2][HD / 16];
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk)
                q_desc[t][kk] = desc_kmajor(smem_u32(q_smem + t * Q_BYTES) + (kk >> 2) * (Q_BYTES / 2) + (kk & 3) * 32);
        const uint64_t k_desc0 = desc_kmajor(smem_u32(k_smem));
        const int n_pairs = (n_kt + 1) / 2;
        bool ok = mbar_wait(&q_full, 0);
        for (int j = 0; j < n_pairs && ok; ++j) {
            // S = Q K^T of the key tiles 2 j and 2 j + 1 (slots 2 (j & 1) and the next: 128 rows of keys) for each query
            // tile into its 128 score columns: the reduction runs over d, 8 steps of 16; d 0..63 lie in the first half
            // of the key region, 64..127 in the second.  (If the pair's second tile does not exist, its columns are
            // never read.)  The columns are free once the softmax warps have read the pair before into registers.
            if (!mbar_wait(&k_full[j & 1], (j >> 1) & 1)) { ok = false; break; }
            fence_after();
            const uint64_t k_desc = k_desc0 + (uint64_t)(((j & 1) * 2 * (KV_BYTES / 2)) >> 4);
            for (int t = 0; t < n_t && ok; ++t) {
                if (j > 0 && !mbar_wait(&s_read[t], (j - 1) & 1)) { ok = false; break; }
                fence_after();
                const uint32_t d_addr = tmem + t * TILE_COLS;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    umma(d_addr, t == 0 ? q_desc[0][kk] : q_desc[1][kk],
                         k_desc + (uint64_t)(((kk >> 2) * (STAGES * KV_BYTES / 2) + (kk & 3) * 32) >> 4), id_s, kk > 0);
                umma_commit(&s_full[t]);
            }
            umma_commit(&k_empty[j & 1]);   // the pair's key slots are free once these MMAs have finished
        }
        if (!ok) atomicExch(&s_failed, 1);
    } else if (warp == 1 && lane == 0 && seq >= 0) {
        // ---- issuer of O += P V: the reduction runs over a tile's 64 keys, 4 steps of 16; V is [key][d], MN-major:
        // blocks of 64 d are 8 KB apart, groups of 8 keys 1 KB
        const uint32_t id_o = idesc(HD, true);
        const int n_t = two ? 2 : 1;
        uint64_t p_desc[2][BN / 16];
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int kk = 0; kk < BN / 16; ++kk) p_desc[t][kk] = desc_kmajor(smem_u32(p_smem + t * P_BYTES) + kk * 32);
        const uint64_t v_desc0 = desc_mnmajor(smem_u32(v_smem), KV_BYTES / 2, 1024);
        bool ok = true;
        for (int i = 0; i < n_kt && ok; ++i) {
            const int st = i % STAGES;
            if (!mbar_wait(&v_full[st], (i / STAGES) & 1)) { ok = false; break; }
            const uint64_t v_desc = v_desc0 + (uint64_t)((st * KV_BYTES) >> 4);
            for (int t = 0; t < n_t && ok; ++t) {
                if (!mbar_wait(&p_full[t], i & 1)) { ok = false; break; }
                fence_after();
                const uint32_t d_addr = tmem + t * TILE_COLS + O_COL;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk)
                    umma(d_addr, t == 0 ? p_desc[0][kk] : p_desc[1][kk], v_desc + (uint64_t)((kk * 2048) >> 4), id_o, i > 0 || kk > 0);
                umma_commit(&o_done[t]);
            }
            umma_commit(&v_empty[st]);   // both query tiles are done with this slot's values once these MMAs have finished
        }
        if (!ok) atomicExch(&s_failed, 1);
    } else if (warp >= 2 && warp < 10 && seq >= 0 && (warp < 6 || two)) {
        // ---- softmax of query tile t: thread owns row r of the tile = lane r of tensor memory
        const int t = warp < 6 ? 0 : 1;
        const int quad = warp & 3;
        const int r = quad * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quad * 32) << 16) + t * TILE_COLS;
        const int tile_tok0 = tok0 + t * p.tq;
        const int tile_tokens = min(p.tq, n_tok - t * p.tq);
        const int rows_valid = tile_tokens * p.group;
        const bool row_ok = r < rows_valid;
        const int tok = row_ok ? r / p.group : 0;
        const int row_pos = pos0 + t * p.tq + tok;
        const int row_lo = p.window > 0 ? max(0, row_pos - p.window + 1) : 0;
        unsigned char* p_tile = p_smem + t * P_BYTES;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        for (int i = 0; i < n_kt; ++i) {
            const int kt = kt_lo + i;
            if ((i & 1) == 0) {   // the scores of the pair of key tiles i, i + 1
                ok = __all_sync(0xffffffffu, mbar_wait(&s_full[t], (i >> 1) & 1));
                if (!ok) break;
                fence_after();
            }
            float s[BN];
            {
                // both halves of the tile's scores are asked for before either is waited for
                uint32_t v0[32], v1[32];
                tmem_ld32(lane_addr + (i & 1) * BN, v0);
                tmem_ld32(lane_addr + (i & 1) * BN + 32, v1);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    s[j] = __uint_as_float(v0[j]);
                    s[32 + j] = __uint_as_float(v1[j]);
                }
            }
            if ((i & 1) || i + 1 == n_kt) {   // the pair's scores are in registers: the next pair's may overwrite them
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s_read[t]);
            }
            // a tile that every row of this warp sees whole (below the diagonal, inside the window) needs no mask:
            // the maximum is taken over the raw scores and the scale goes into the exponent's multiply-add
            const bool whole = __all_sync(0xffffffffu, row_ok && kt * BN + BN - 1 <= row_pos && kt * BN >= row_lo);
            float mx = -INFINITY;
            if (whole) {
#pragma unroll
                for (int j = 0; j < BN; j += 2) mx = max3(mx, s[j], s[j + 1]);
                mx *= p.scale_log2;
            } else {
#pragma unroll
                for (int j = 0; j < BN; ++j) {
                    const int kp = kt * BN + j;
                    const bool seen = row_ok && kp <= row_pos && kp >= row_lo;
                    s[j] = seen ? s[j] : -INFINITY;
                    mx = fmaxf(mx, s[j]);
                }
                mx = mx == -INFINITY ? mx : mx * p.scale_log2;
            }
            // m is the reference the exponentials are taken against, not the true maximum: it moves only when a
            // score exceeds it by more than 8 (probabilities then stay below 2^8, far from overflow), so that O, which
            // sits in tensor memory, has to be rescaled only rarely
            const float m_new = (m == -INFINITY || mx > m + 8.f) ? fmaxf(m, mx) : m;
            const float corr = m_new == -INFINITY ? 1.f : ex2(m - m_new);
            const float neg_ref = m_new == -INFINITY ? 0.f : -m_new;
            m = m_new;
            // exponents and the row's sum two numbers at a time (fma and add on pairs of floats)
            const uint64_t scale2 = pair(p.scale_log2, p.scale_log2), ref2 = pair(neg_ref, neg_ref);
            uint64_t sum2 = pair(0.f, 0.f);
            uint32_t pk[BN / 2];
#pragma unroll
            for (int j = 0; j < BN; j += 2) {
                float e0, e1;
                unpair(fma_pair(pair(s[j], s[j + 1]), scale2, ref2), e0, e1);
                const float a = ex2(e0), b = ex2(e1);
                sum2 = add_pair(sum2, pair(a, b));
                pk[j / 2] = pack_bf16(a, b);
            }
            float sum_even, sum_odd;
            unpair(sum2, sum_even, sum_odd);
            l = l * corr + (sum_even + sum_odd);
            if (i > 0) {
                // the MMA that used the last probabilities and added into O has finished
                ok = __all_sync(0xffffffffu, mbar_wait(&o_done[t], (i - 1) & 1));
                if (!ok) break;
                fence_after();
                if (__any_sync(0xffffffffu, corr != 1.f)) {   // the maximum of some row of this warp moved: rescale O
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(lane_addr + O_COL + c, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
                        tmem_st32(lane_addr + O_COL + c, v);
                    }
                    tmem_st_wait();
                }
            }
            // probabilities of this row: 64 bfloat16 = one 128-byte row with its 16-byte chunks swizzled
            unsigned char* prow = p_tile + r * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
            // positions past the sequence's end lie in a fetched page but were never written: their values must
            // not reach the sum, not even multiplied by zero.  Only the tile that holds the end has such keys; the
            // first query tile's warps clear them (both tiles' MMAs wait for these warps' arrival or come after it).
            if (t == 0 && kt * BN + BN - 1 > pos_last) {
                // (the values must have arrived, or they would land on top of the zeros)
                ok = __all_sync(0xffffffffu, mbar_wait(&v_full[i % STAGES], (i / STAGES) & 1));
                if (!ok) break;
                unsigned char* vd = v_smem + (i % STAGES) * KV_BYTES;
                const int first_bad = pos_last + 1 - kt * BN;
                for (int idx = quad * 32 + lane; idx < (BN - first_bad) * 16; idx += 128) {
                    const int row = first_bad + idx / 16, c = idx % 16;   // 16 chunks of 16 bytes per row: two boxes of 8
                    *reinterpret_cast<uint4*>(vd + (c >> 3) * (KV_BYTES / 2) + row * 128 + ((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            fence_before();
            mbar_arrive(&p_full[t]);
        }
        if (ok && n_kt > 0) ok = __all_sync(0xffffffffu, mbar_wait(&o_done[t], (n_kt - 1) & 1));
        if (ok) {
            fence_after();
            const int g = r - tok * p.group;
            const size_t row = (size_t)(tile_tok0 + tok) * p.nq + kvh * p.group + g;
            if (p.n_splits > 1) {
                // this run's share of the row (a run without keys leaves maximum -inf and sum 0, and no numbers)
                float* dst = p.part_o + ((size_t)blockIdx.z * p.n_rows + row) * HD;
                if (n_kt > 0) {
#pragma unroll
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t v[32];
                        tmem_ld32(lane_addr + O_COL + c, v);
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
#pragma unroll
                for (int c = 0; c < HD; c += 32) {
                    uint32_t v[32];
                    tmem_ld32(lane_addr + O_COL + c, v);
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
__global__ void __launch_bounds__(128) attention_tcgen05_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                                      __nv_bfloat16* __restrict__ out, int n_rows, int n_splits,
                                                                      int first_row, int rows) {
    const int lane = threadIdx.x & 31;
    if (blockIdx.x * 4 + (threadIdx.x >> 5) >= rows) return;
    const int row = first_row + blockIdx.x * 4 + (threadIdx.x >> 5);
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, part_ml[((size_t)z * n_rows + row) * 2]);
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int z = 0; z < n_splits; ++z) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + ((size_t)z * n_rows + row) * 2);
        if (ml.x == -INFINITY) continue;
        const float f = exp2f(ml.x - M);
        const float4 v = *reinterpret_cast<const float4*>(part_o + ((size_t)z * n_rows + row) * HD + lane * 4);
        L += f * ml.y;
        acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    uint2 o;
    o.x = pack_bf16(acc.x * inv, acc.y * inv);
    o.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + (size_t)row * HD + lane * 4) = o;
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

// A pool of one layer as [rows, 128] bfloat16; boxes of [box_rows, 64].
int pool_map(CUtensorMap* map, const void* base, long long rows, int box_rows) {
    std::lock_guard<std::mutex> guard(g_lock);
    const MapKey key{base, rows, 0, box_rows, 2};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *map = it->second; return 0; }
    EncodeTiled fn = encoder();
    if (!fn) RMX_FAIL("attention_tcgen05: the driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
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

// The queries [tokens, nq, 128]; boxes of [tq tokens, group heads, 64]: a tile's rows come out token by token, the
// group's heads side by side.
int q_map(CUtensorMap* map, const void* base, long long tokens, int nq, int group, int tq) {
    std::lock_guard<std::mutex> guard(g_lock);
    const MapKey key{base, tokens, nq, group, 3};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *map = it->second; return 0; }
    EncodeTiled fn = encoder();
    if (!fn) RMX_FAIL("attention_tcgen05: the driver has no cuTensorMapEncodeTiled");
    cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nq, (cuuint64_t)tokens};
    cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)nq * HD * 2};
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
}  // namespace

// Head size 128, a group that divides 128, pages of at least 8 positions (a power of two).
RMX_API int rmx_attention_tcgen05_supports(int hd, int group, int page_size) {
    return hd == 128 && group >= 1 && group <= 16 && (group & (group - 1)) == 0 && page_size >= 8 &&
           (page_size & (page_size - 1)) == 0;
}

RMX_API int rmx_attention_tcgen05_tile_tokens(int group) { return BM / group; }

// tiles_per_block: 2 (a block takes two neighbouring query tiles of 128 rows, which share every key tile it fetches)
// or 1 (twice the blocks: for steps so small that two tiles a block would leave SMs without work).
// n_tiles: the number of blocks: sum over sequences of ceil(tokens / (tiles_per_block * 128 / group)).
// pool_pages: pages in k_pool / v_pool.
// n_splits > 1: every tile's keys in that many runs, one block each (blockIdx.z), added by a second kernel; part_o
// [n_splits, n_tokens * nq, 128] and part_ml [n_splits, n_tokens * nq, 2] floats are their scratch; the sequences
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
    if (q_map(&mq, q, n_tokens, nq, group, p.tq) != 0) return -1;
    if (pool_map(&mk, k_pool, pool_rows, p.box_rows) != 0) return -1;
    if (pool_map(&mv, v_pool, pool_rows, p.box_rows) != 0) return -1;
    constexpr size_t smem = 1024 + 2 * Q_BYTES + (size_t)STAGES * 2 * KV_BYTES + 2 * P_BYTES;
    static bool raised[64] = {};
    if (rmx_first_on_device(raised)) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RMX_FAIL("attention_tcgen05: shared memory of %zu bytes refused: %s", smem, cudaGetErrorString(e));
    }
    // blocks are handed to the SMs in the order x, then y: all kv heads of the tile that sees the most keys first
    attention_tcgen05_kernel<<<dim3(nkv, n_tiles, n_splits), THREADS, smem, (cudaStream_t)stream>>>(mq, mk, mv, p);
    RMX_CHECK_LAUNCH("attention_tcgen05");
    if (n_splits > 1) {
        RMX_REQUIRE(first_token >= 0 && run_tokens > 0 && first_token + run_tokens <= n_tokens, "attention_tcgen05: the tokens of this launch are not among the step's");
        attention_tcgen05_merge_kernel<<<(run_tokens * nq + 3) / 4, 128, 0, (cudaStream_t)stream>>>(part_o, part_ml, (__nv_bfloat16*)out, p.n_rows, n_splits,
                                                                                                  first_token * nq, run_tokens * nq);
        RMX_CHECK_LAUNCH("attention_tcgen05_merge");
    }
    return 0;
}
