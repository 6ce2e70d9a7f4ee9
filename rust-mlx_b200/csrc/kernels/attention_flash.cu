// Flash attention over the paged cache for bfloat16, on the tensor cores (mma.sync m16n8k16),
// serving prompt portions and decoded tokens in one launch.
//
// A block takes one kv head and one tile of query rows of one sequence.  A row is a
// (token, query head of the group) pair, so the heads that share a kv head share every key
// and value the block loads: TQ = 64 / group tokens by `group` heads per tile.  Keys are
// visited in tiles of 64 aligned to absolute positions, brought to shared memory with
// cp.async (two stages), through the request's block table.  Scores, the running maximum,
// the exponentials, their sum and the output accumulate in float.  A row at position p
// sees keys lo .. p (lo = p - window + 1 or 0).  With n_splits > 1 (long contexts, few
// rows: decoding) grid.z blocks share a tile's keys and write unnormalised partial
// results, which attention_merge_kernel combines.
//
// Two arrangements of the four warps.  Rows: each warp owns 16 of the tile's 64 rows and
// all 64 keys of a key tile (prompt portions).  Keys (KEYSPLIT, used when every tile has at
// most 16 rows, i.e. decoding): all warps hold the same 16 rows and each takes 16 of the 64
// keys, so that one token's work is spread over the block; the warps' partial results are
// combined through shared memory at the end.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "rope128.cuh"

namespace {
constexpr int BM = 64, BN = 64, NWARPS = 4, THREADS = NWARPS * 32;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

struct FlashParams {
    const __nv_bfloat16* q;        // [tokens, nq, HD]
    const __nv_bfloat16* k_pool;   // [pages, nkv, page_size, HD]
    const __nv_bfloat16* v_pool;
    const int* q_start;            // [seqs + 1] first flat token of every sequence
    const int* positions;          // [tokens]
    const int* block_table;        // [seqs, table_stride]
    __nv_bfloat16* out;            // [tokens, nq, HD]
    float* part_o;                 // [splits, tokens * nq, HD]   (splits > 1)
    float* part_ml;                // [splits, tokens * nq, 2]
    unsigned int* counters;        // [seqs * nkv] zeros, or null: who is the last split of a (sequence, kv head)
    int* status;
    int n_seqs, n_tokens, nq, nkv, group, tq, table_stride, page_size, page_shift, window, n_splits;
    float scale_log2;
    int cluster;                   // the splits of a (sequence, kv head) are one thread-block cluster (decoding by TMA)
    // Decoding by TMA, heads of 128, one token a sequence: the kernel may take the projection's rows as they come
    // ([q heads | k heads | v heads] of every token) and, while it waits for its first keys, norm and rotate its own
    // query heads and its token's key and store key and value into their page (see rope128.cuh)
    const __nv_bfloat16* qkv;      // [tokens, qkv_stride], or null: `q` holds finished queries and the pages are written
    const float* q_norm;           // [128] or null
    const float* k_norm;
    const float* cos_sin;          // [tokens][128]
    __nv_bfloat16* k_store;        // the pools again, to write; null: the layer reads another layer's cache
    __nv_bfloat16* v_store;
    float eps;
    int qkv_stride;
};

template <int HD, bool KEYSPLIT>
__global__ void __launch_bounds__(THREADS) attention_flash_kernel(const FlashParams p) {
    constexpr int NT = KEYSPLIT ? 2 : BN / 8;   // score tiles of 8 keys per warp and key tile
    constexpr int QROWS = KEYSPLIT ? 16 : BM;   // query rows kept in shared memory
    constexpr int STAGES = KEYSPLIT ? 3 : 2;    // key tiles in the ring: decoding is bound by loads in flight
    constexpr int STRIDE = HD + 8;          // 16 bytes of padding: ldmatrix rows fall into different banks
    constexpr int CHUNKS = HD / 8;          // 16-byte chunks per row
    constexpr int KSTEPS = HD / 16;
    constexpr int DTILES = HD / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);  // [QROWS][STRIDE]
    __nv_bfloat16* Ks = Qs + QROWS * STRIDE;                          // [STAGES][BN][STRIDE]
    __nv_bfloat16* Vs = Ks + STAGES * BN * STRIDE;                    // [STAGES][BN][STRIDE]
    __shared__ int s_tile[3];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, split = blockIdx.z;

    // which sequence and which of its tiles this block has: tiles are counted sequence by
    // sequence; the threads scan the sequences' tile counts together
    {
        __shared__ int s_warp_total[NWARPS];
        if (tid == 0) s_tile[0] = -1;
        int base = 0;
        for (int chunk = 0; chunk < p.n_seqs; chunk += THREADS) {
            const int sq = chunk + tid;
            int a = 0, n = 0, tiles = 0;
            if (sq < p.n_seqs) {
                a = p.q_start[sq];
                n = p.q_start[sq + 1] - a;
                tiles = (n + p.tq - 1) / p.tq;
            }
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int v = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += v;
            }
            __syncthreads();
            if (lane == 31) s_warp_total[warp] = incl;
            __syncthreads();
            int before = base, total = 0;
#pragma unroll
            for (int w = 0; w < NWARPS; ++w) {
                if (w < warp) before += s_warp_total[w];
                total += s_warp_total[w];
            }
            const int first_tile = before + incl - tiles;
            const int mine = (int)blockIdx.x - first_tile;
            if (tiles > 0 && mine >= 0 && mine < tiles) {
                s_tile[0] = sq;
                s_tile[1] = a + mine * p.tq;
                s_tile[2] = min(p.tq, n - mine * p.tq);
            }
            base += total;
        }
    }
    __syncthreads();
    const int seq = s_tile[0], tok0 = s_tile[1], n_tok = s_tile[2];
    if (seq < 0) return;  // the grid is an upper bound
    const int pos0 = p.positions[tok0];
    const int rows_valid = n_tok * p.group;
    const int* table = p.block_table + (size_t)seq * p.table_stride;

    // keys this tile needs: from the first row's lower bound to the last row's position
    const int lo_first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int pos_last = pos0 + n_tok - 1;
    const int kt_lo = lo_first / BN, kt_hi = pos_last / BN;
    const int n_kt = kt_hi - kt_lo + 1;
    const int per_split = (n_kt + p.n_splits - 1) / p.n_splits;
    const int kt_begin = kt_lo + split * per_split;
    const int kt_end = min(kt_hi + 1, kt_begin + per_split);

    // ---- Q tile to shared memory (rows beyond the tile are zeros)
    for (int idx = tid; idx < QROWS * CHUNKS; idx += THREADS) {
        const int r = idx / CHUNKS, c = idx - r * CHUNKS;
        const bool valid = r < rows_valid;
        const int tok = valid ? r / p.group : 0, g = valid ? r - tok * p.group : 0;
        const __nv_bfloat16* src = p.q + ((size_t)(tok0 + tok) * p.nq + kvh * p.group + g) * HD + c * 8;
        cp_async16(Qs + r * STRIDE + c * 8, src, valid);
    }
    cp_async_commit();

    const int page_mask = p.page_size - 1;
    const size_t head_off = (size_t)kvh * p.page_size * HD;
    const size_t page_elems = (size_t)p.nkv * p.page_size * HD;
    auto load_kv = [&](int kt, int stage) {
        __nv_bfloat16* kd = Ks + stage * BN * STRIDE;
        __nv_bfloat16* vd = Vs + stage * BN * STRIDE;
        for (int idx = tid; idx < BN * CHUNKS; idx += THREADS) {
            const int j = idx / CHUNKS, c = idx - j * CHUNKS;
            const int kp = kt * BN + j;
            bool valid = kp >= lo_first && kp <= pos_last;
            size_t off = 0;
            if (valid) {
                const int page = table[kp >> p.page_shift];
                if (page < 0) {
                    valid = false;
                    if (c == 0) atomicExch(p.status, 2);
                } else {
                    off = (size_t)page * page_elems + head_off + (size_t)((kp & page_mask) * HD + c * 8);
                }
            }
            cp_async16(kd + j * STRIDE + c * 8, p.k_pool + off, valid);
            cp_async16(vd + j * STRIDE + c * 8, p.v_pool + off, valid);
        }
    };

#pragma unroll
    for (int st = 0; st < STAGES - 1; ++st) {
        if (kt_begin + st < kt_end) load_kv(kt_begin + st, st);
        cp_async_commit();
    }

    // ---- this warp's rows
    const int row_base = KEYSPLIT ? 0 : warp * 16;
    const int key_base = KEYSPLIT ? warp * 16 : 0;              // this warp's keys inside a key tile
    const int r_lo = row_base + (lane >> 2), r_hi = r_lo + 8;   // the two rows this thread holds in C fragments
    const bool warp_active = row_base < rows_valid;
    int row_pos[2], row_lo[2];
    bool row_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = i == 0 ? r_lo : r_hi;
        row_ok[i] = r < rows_valid;
        row_pos[i] = pos0 + (row_ok[i] ? r / p.group : 0);
        row_lo[i] = p.window > 0 ? max(0, row_pos[i] - p.window + 1) : 0;
    }

    cp_async_wait<STAGES - 1>();  // Q has landed (the oldest group)
    __syncthreads();
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
        ldmatrix_x4(qf[kk], Qs + (row_base + (lane & 15)) * STRIDE + kk * 16 + (lane >> 4) * 8);

    float o[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int kt = kt_begin; kt < kt_end; ++kt) {
        const int stage = (kt - kt_begin) % STAGES;
        if (kt + STAGES - 1 < kt_end) load_kv(kt + STAGES - 1, (kt - kt_begin + STAGES - 1) % STAGES);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (warp_active) {
            const __nv_bfloat16* kbase = Ks + stage * BN * STRIDE;
            const __nv_bfloat16* vbase = Vs + stage * BN * STRIDE;
            float s[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int jp = 0; jp < NT / 2; ++jp) {
                    uint32_t kf[4];
                    const int key = key_base + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
                    const int dcol = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(kf, kbase + key * STRIDE + dcol);
                    mma_bf16(s[2 * jp], qf[kk], kf[0], kf[1]);
                    mma_bf16(s[2 * jp + 1], qf[kk], kf[2], kf[3]);
                }
            }
            // mask, scale, online softmax (in base 2)
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const int kp = kt * BN + key_base + j * 8 + (lane & 3) * 2 + (e & 1);
                    const bool ok = row_ok[i] && kp <= row_pos[i] && kp >= row_lo[i];
                    s[j][e] = ok ? s[j][e] * p.scale_log2 : -INFINITY;
                    mx[i] = fmaxf(mx[i], s[j][e]);
                }
            }
            float corr[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m[i], mx[i]);
                corr[i] = m_new == -INFINITY ? 1.f : exp2f(m[i] - m_new);
                m[i] = m_new;
                l[i] *= corr[i];
            }
            const float mref[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = e >> 1;
                    const float pv = exp2f(s[j][e] - mref[i]);  // -inf -> 0
                    s[j][e] = pv;
                    l[i] += pv;
                }
            }
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                o[d][0] *= corr[0]; o[d][1] *= corr[0];
                o[d][2] *= corr[1]; o[d][3] *= corr[1];
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < DTILES / 2; ++dp) {
                    uint32_t vf[4];
                    const int key = key_base + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int dcol = dp * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(vf, vbase + key * STRIDE + dcol);
                    mma_bf16(o[2 * dp], pf, vf[0], vf[1]);
                    mma_bf16(o[2 * dp + 1], pf, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();  // the stage is free for the load after next
    }
    cp_async_wait<0>();
    allow_dependents();   // what follows may start fetching its weights while the results are written

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    if constexpr (KEYSPLIT) {
        // the four warps hold partial results for the same rows: combine them in warp order
        float* so = reinterpret_cast<float*>(Ks);             // [NWARPS][16][HD]   (key tiles are done)
        float* sml = so + NWARPS * 16 * HD;                   // [NWARPS][16][2]
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = (lane >> 2) + 8 * i;
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                const int col = d * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(so + (warp * 16 + r) * HD + col) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
            }
            if ((lane & 3) == 0) {
                sml[(warp * 16 + r) * 2] = m[i];
                sml[(warp * 16 + r) * 2 + 1] = l[i];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < rows_valid * HD; idx += THREADS) {
            const int r = idx / HD, d = idx - r * HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, sml[(w * 16 + r) * 2]);
            float L = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < NWARPS; ++w) {
                const float mw = sml[(w * 16 + r) * 2];
                const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
                L += f * sml[(w * 16 + r) * 2 + 1];
                acc += f * so[(w * 16 + r) * HD + d];
            }
            const int tok = r / p.group, g = r - tok * p.group;
            const size_t row = (size_t)(tok0 + tok) * p.nq + kvh * p.group + g;
            if (p.n_splits == 1) {
                p.out[row * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
            } else {
                const size_t prow = (size_t)split * p.n_tokens * p.nq + row;
                p.part_o[prow * HD + d] = acc;
                if (d == 0) {
                    p.part_ml[prow * 2] = M;
                    p.part_ml[prow * 2 + 1] = L;
                }
            }
        }
        return;
    }
    if (!warp_active) return;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = i == 0 ? r_lo : r_hi;
        if (!row_ok[i]) continue;
        const int tok = r / p.group, g = r - tok * p.group;
        const size_t row = (size_t)(tok0 + tok) * p.nq + kvh * p.group + g;
        if (p.n_splits == 1) {
            const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
            __nv_bfloat16* dst = p.out + row * HD;
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                const int col = d * 8 + (lane & 3) * 2;
                *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
            }
        } else {
            const size_t prow = (size_t)split * p.n_tokens * p.nq + row;
            float* dst = p.part_o + prow * HD;
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                const int col = d * 8 + (lane & 3) * 2;
                *reinterpret_cast<float2*>(dst + col) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
            }
            if ((lane & 3) == 0) {
                p.part_ml[prow * 2] = m[i];
                p.part_ml[prow * 2 + 1] = l[i];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same attention with keys and values fetched by TMA, for head sizes 64 and 128 and pages of at least 8
// positions.  A fifth warp is the producer: one thread fetches a key tile with a few tensor-map copies
// (cp.async.bulk.tensor, boxes of up to 64 rows by 64 columns, 128-byte swizzle, completion on an mbarrier)
// into a ring of stages; the four computing warps read the tiles with ldmatrix at the swizzled places and
// never spend an instruction on addresses or wait for one another.  Both arrangements of the warps: rows
// (prompt portions) and keys (decoding: every tile has at most 16 rows, the work is reading keys and values).
constexpr int DSTAGES = 3;
constexpr int DTHREADS = (NWARPS + 1) * 32;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
// Polls until the phase with the given parity has completed; gives up after a bounded number of polls.
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
__device__ __forceinline__ void tma_box(void* smem, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
        ::"r"(smem_u32(smem)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The address, in the cluster's shared window, of what `local` is in the block of the given rank.
__device__ __forceinline__ uint32_t in_block(const void* local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    return remote;
}
// Element (row, col) of a key or value tile held as HD/64 blocks of [64 rows][64 columns], rows of 128
// bytes whose 16-byte chunks are exchanged by the row's low three bits (the 128-byte swizzle of TMA).
template <int HD>
__device__ __forceinline__ const __nv_bfloat16* swz(const __nv_bfloat16* tile, int row, int col) {
    return tile + (col >> 6) * (64 * 64) + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3);
}

// FINISH: built for p.qkv (decoding that finishes the projection itself); the other builds carry none of that code.
template <int HD, bool KEYSPLIT, bool FINISH = false>
__global__ void __launch_bounds__(DTHREADS, 2) attention_tma_kernel(const __grid_constant__ CUtensorMap map_k,
                                                                const __grid_constant__ CUtensorMap map_v,
                                                                const FlashParams p, int box_rows) {
    constexpr int STRIDE = HD + 8, CHUNKS = HD / 8, KSTEPS = HD / 16, DTILES = HD / 8;
    constexpr int NT = KEYSPLIT ? 2 : BN / 8;              // score tiles of 8 keys per warp and key tile
    constexpr int QROWS = KEYSPLIT ? 16 : BM;
    constexpr int STAGES = KEYSPLIT ? DSTAGES : 2;         // decoding is bound by loads in flight, prompts by arithmetic
    constexpr int TILE_ELEMS = 64 * HD;                    // one key tile (or value tile)
    extern __shared__ unsigned char smem_decode_raw[];
    // the stages sit on a 1024-byte boundary, as the 128-byte swizzle asks
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_decode_raw) + 1023) & ~(uintptr_t)1023);
    __nv_bfloat16* KV = reinterpret_cast<__nv_bfloat16*>(base);                        // [STAGES][K tile | V tile]
    __nv_bfloat16* Qs = KV + STAGES * 2 * TILE_ELEMS;                                  // [QROWS][STRIDE]
    // decoding with its splits as a cluster: where the other splits leave their shares of this block's output columns
    float4* recv = reinterpret_cast<float4*>(Qs + QROWS * STRIDE);                     // [splits][ceil(16 * HD / 4 / splits)]
    float2* recv_ml = reinterpret_cast<float2*>(recv + 16 * HD / 4 + 8);               // [8 splits][16 rows] (max, sum)
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES];
    __shared__ int s_failed, s_tile[3];
    constexpr int TABLE_KEPT = 512;
    __shared__ int s_table[KEYSPLIT ? TABLE_KEPT : 1];   // decoding: the head of the sequence's block table

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.y, split = blockIdx.z;
    if (tid == 0) {
        s_failed = 0;
        for (int st = 0; st < STAGES; ++st) {
            mbar_init(&full_bar[st], 1);
            mbar_init(&empty_bar[st], NWARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_v) : "memory");
    }
    // the stages start as zeros so that a part of a tile that is never fetched (a page the request does not
    // hold) has finite numbers in it
    for (int idx = tid; idx < STAGES * 2 * TILE_ELEMS / 8; idx += DTHREADS)
        reinterpret_cast<uint4*>(KV)[idx] = make_uint4(0u, 0u, 0u, 0u);
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncthreads();
    // (the matching wait stands before the first store into another block's shared memory: every block of the
    // cluster has started by then)
    if (KEYSPLIT && p.cluster) asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    // Everything above needs nothing from the kernels before this one; the queries do, and so do the keys and
    // values of the step's own tokens where a kernel before this one stores them.  A kernel that finishes the
    // projection itself (FINISH) stores its token's key and value itself and patches them into the tile it
    // fetched: whatever else it reads of the pools was written by earlier steps, and the step's tables and
    // positions were uploaded before the step's first kernel.  So there only the warps that read the projection
    // wait, and the producer's copies of keys and values run while the kernel before this one still ends.
    allow_dependents();
    if (!FINISH) wait_for_prior_kernels();
    int seq, tok0, n_tok, pos0;
    if constexpr (KEYSPLIT) {   // one tile per sequence
        seq = blockIdx.x;
        // loads that do not wait for one another: the table's head, the sequence's tokens, and the position of
        // token number `seq`, which is the sequence's first token whenever every sequence brings one token
        if (warp == NWARPS) {
            const int* row = p.block_table + (size_t)seq * p.table_stride;
            for (int j = lane; j < min(p.table_stride, TABLE_KEPT); j += 32) s_table[j] = row[j];
        }
        const int a = p.q_start[seq], b = p.q_start[seq + 1], guess = p.positions[seq];
        tok0 = a;
        n_tok = b - a;
        pos0 = tok0 == seq ? guess : p.positions[tok0];
    } else {
        // which sequence and which of its tiles this block has: the threads scan the sequences' tile counts together
        __shared__ int s_warp_total[NWARPS + 1];
        if (tid == 0) s_tile[0] = -1;
        int before_all = 0;
        for (int chunk = 0; chunk < p.n_seqs; chunk += DTHREADS) {
            const int sq = chunk + tid;
            int a = 0, n = 0, tiles = 0;
            if (sq < p.n_seqs) {
                a = p.q_start[sq];
                n = p.q_start[sq + 1] - a;
                tiles = (n + p.tq - 1) / p.tq;
            }
            int incl = tiles;
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
            for (int w = 0; w < NWARPS + 1; ++w) {
                if (w < warp) before += s_warp_total[w];
                total += s_warp_total[w];
            }
            const int mine = (int)blockIdx.x - (before + incl - tiles);
            if (tiles > 0 && mine >= 0 && mine < tiles) {
                s_tile[0] = sq;
                s_tile[1] = a + mine * p.tq;
                s_tile[2] = min(p.tq, n - mine * p.tq);
            }
            before_all += total;
        }
        __syncthreads();
        seq = s_tile[0]; tok0 = s_tile[1]; n_tok = s_tile[2];
        if (seq < 0) return;  // the grid is an upper bound
        pos0 = p.positions[tok0];
    }
    const int rows_valid = n_tok * p.group;
    const int* table = p.block_table + (size_t)seq * p.table_stride;
    const int lo_first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int pos_last = pos0 + n_tok - 1;
    const int kt_lo = lo_first / BN, kt_hi = pos_last / BN;
    const int per_split = (kt_hi - kt_lo + 1 + p.n_splits - 1) / p.n_splits;
    const int kt_begin = kt_lo + split * per_split;
    const int kt_end = min(kt_hi + 1, kt_begin + per_split);
    const int n_mine = kt_begin < kt_end ? kt_end - kt_begin : 0;

    // Q rows (zeros beyond the tile's rows), fetched by the computing warps; the producer does not wait for them
    uint2 k_new = make_uint2(0u, 0u), v_new = make_uint2(0u, 0u);   // the token's own key and value (fused decoding)
    bool have_new = false;
    if (warp < NWARPS) {
        if constexpr (FINISH) {
            wait_for_prior_kernels();
            // one token a sequence: its `group` query heads are the tile's rows; a warp takes a head at a time
            const __nv_bfloat16* row = p.qkv + (size_t)tok0 * p.qkv_stride;
            const float* cs = p.cos_sin + (size_t)tok0 * 128;
            for (int g = warp; g < QROWS; g += NWARPS) {
                uint2 qv = make_uint2(0u, 0u);
                if (g < p.group)
                    qv = rope128_head(*reinterpret_cast<const uint2*>(row + (size_t)(kvh * p.group + g) * 128 + lane * 4), p.q_norm, p.eps, cs, lane);
                *reinterpret_cast<uint2*>(Qs + g * STRIDE + lane * 4) = qv;
            }
            // the block whose keys end with the token's own forms its key and stores key and value: the warp that
            // will work on the 16 keys around the token's place keeps them, to put them into the tile it gets by
            // TMA (which may have read the page before these stores landed)
            if (p.k_store != nullptr && kt_hi >= kt_begin && kt_hi < kt_end && warp == ((pos0 & (BN - 1)) >> 4)) {
                k_new = rope128_head(*reinterpret_cast<const uint2*>(row + (size_t)(p.nq + kvh) * 128 + lane * 4), p.k_norm, p.eps, cs, lane);
                v_new = *reinterpret_cast<const uint2*>(row + (size_t)(p.nq + p.nkv + kvh) * 128 + lane * 4);
                have_new = true;
                const int page = table[pos0 >> p.page_shift];
                if (page < 0) {  // the host reserves pages before the step; never write through a hole
                    if (lane == 0) atomicExch(p.status, 1);
                } else {
                    const size_t at = (((size_t)page * p.nkv + kvh) * p.page_size + (pos0 & (p.page_size - 1))) * 128 + lane * 4;
                    *reinterpret_cast<uint2*>(p.k_store + at) = k_new;
                    *reinterpret_cast<uint2*>(p.v_store + at) = v_new;
                }
            }
        } else {
            for (int idx = tid; idx < QROWS * CHUNKS; idx += NWARPS * 32) {
                const int r = idx / CHUNKS, c = idx - r * CHUNKS;
                const bool valid = r < rows_valid;
                const int tok = valid ? r / p.group : 0, g = valid ? r - tok * p.group : 0;
                cp_async16(Qs + r * STRIDE + c * 8, p.q + ((size_t)(tok0 + tok) * p.nq + kvh * p.group + g) * HD + c * 8, valid);
            }
            cp_async_commit();
        }
    }

    if (warp == NWARPS) {
        __syncwarp();   // the table's head is in shared memory
        // ---- producer: per tile, 64 / box_rows boxes of rows by HD / 64 boxes of columns, for K and for V: at most
        // 32 copies, which as many lanes issue at once (one thread issuing them in turn is slower than the tiles
        // are used up when pages are small)
        constexpr int PER_BOX = 2 * (HD / 64);
        const int boxes = BN / box_rows;
        const int my_box = lane / PER_BOX, my_cb = (lane % PER_BOX) >> 1;
        const bool my_v = lane & 1;
        auto entry = [&](int j) { return KEYSPLIT && j < TABLE_KEPT ? s_table[j] : table[j]; };
        for (int i = 0; i < n_mine; ++i) {
            const int st = i % STAGES, round = i / STAGES, kt = kt_begin + i;
            int ok = 1;
            if (round > 0 && lane == 0) ok = mbar_wait(&empty_bar[st], (round - 1) & 1);
            if (!__shfl_sync(0xffffffffu, ok, 0)) {
                if (lane == 0) atomicExch(&s_failed, 1);
                break;
            }
            const int kp = kt * BN + my_box * box_rows;
            bool mine = my_box < boxes && kp <= pos_last && kp + box_rows > lo_first;
            const int page = mine ? entry(kp >> p.page_shift) : 0;
            if (mine && page < 0) {
                atomicExch(p.status, 2);
                mine = false;
            }
            const uint32_t copies = __popc(__ballot_sync(0xffffffffu, mine));
            if (lane == 0) mbar_expect_tx(&full_bar[st], copies * (uint32_t)box_rows * 64u * 2u);
            __syncwarp();
            if (mine) {
                __nv_bfloat16* dst = KV + st * 2 * TILE_ELEMS + (my_v ? TILE_ELEMS : 0) + my_cb * 64 * 64 + my_box * box_rows * 64;
                const int row = (page * p.nkv + kvh) * p.page_size + (kp & (p.page_size - 1));
                tma_box(dst, my_v ? &map_v : &map_k, &full_bar[st], my_cb * 64, row);
            }
            __syncwarp();
        }
        __syncwarp();
    } else {
        cp_async_wait<0>();
        asm volatile("bar.sync 1, %0;\n" ::"n"(NWARPS * 32) : "memory");   // the computing warps among themselves
    }

    // ---- computing warps.  Rows: each warp owns 16 of the tile's rows and all 64 keys.  Keys (KEYSPLIT): the same
    // 16 rows in every warp, 16 of the 64 keys each.
    const int cw = warp & 3;
    const int row_base = KEYSPLIT ? 0 : cw * 16;
    const int key_base = KEYSPLIT ? cw * 16 : 0;
    const bool warp_active = warp < NWARPS && row_base < rows_valid;
    int row_pos[2], row_lo[2];
    bool row_ok[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = row_base + (lane >> 2) + 8 * i;
        row_ok[i] = r < rows_valid;
        row_pos[i] = pos0 + (row_ok[i] ? r / p.group : 0);
        row_lo[i] = p.window > 0 ? max(0, row_pos[i] - p.window + 1) : 0;
    }
    uint32_t qf[KSTEPS][4];
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
        ldmatrix_x4(qf[kk], Qs + (row_base + (lane & 15)) * STRIDE + kk * 16 + (lane >> 4) * 8);
    float o[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int i = 0; i < n_mine && warp < NWARPS; ++i) {
        const int kt = kt_begin + i, stage = i % STAGES;
        if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[stage], (i / STAGES) & 1))) { atomicExch(&s_failed, 1); break; }
        if (FINISH && have_new && kt == kt_hi) {
            // the token's own key and value into the tile, whatever the TMA found at their place
            if constexpr (HD == 128) {
                __nv_bfloat16* kb = KV + stage * 2 * TILE_ELEMS;
                const int r = pos0 & (BN - 1), col = lane * 4;
                __nv_bfloat16* kp = const_cast<__nv_bfloat16*>(swz<HD>(kb, r, col & ~7)) + (col & 7);
                __nv_bfloat16* vp = const_cast<__nv_bfloat16*>(swz<HD>(kb + TILE_ELEMS, r, col & ~7)) + (col & 7);
                *reinterpret_cast<uint2*>(kp) = k_new;
                *reinterpret_cast<uint2*>(vp) = v_new;
            }
            __syncwarp();
        }
        if (warp_active) {
            const __nv_bfloat16* kbase = KV + stage * 2 * TILE_ELEMS;
            const __nv_bfloat16* vbase = kbase + TILE_ELEMS;
            float s[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int jp = 0; jp < NT / 2; ++jp) {
                    uint32_t kf[4];
                    const int key = key_base + jp * 16 + (lane & 7) + ((lane >> 4) << 3);
                    const int dcol = kk * 16 + ((lane >> 3) & 1) * 8;
                    ldmatrix_x4(kf, swz<HD>(kbase, key, dcol));
                    mma_bf16(s[2 * jp], qf[kk], kf[0], kf[1]);
                    mma_bf16(s[2 * jp + 1], qf[kk], kf[2], kf[3]);
                }
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    const int kp = kt * BN + key_base + j * 8 + (lane & 3) * 2 + (e & 1);
                    const bool ok = row_ok[r] && kp <= row_pos[r] && kp >= row_lo[r];
                    s[j][e] = ok ? s[j][e] * p.scale_log2 : -INFINITY;
                    mx[r] = fmaxf(mx[r], s[j][e]);
                }
            }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m[r], mx[r]);
                corr[r] = m_new == -INFINITY ? 1.f : exp2f(m[r] - m_new);
                m[r] = m_new;
                l[r] *= corr[r];
            }
            const float mref[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float pv = exp2f(s[j][e] - mref[e >> 1]);
                    s[j][e] = pv;
                    l[e >> 1] += pv;
                }
            }
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                o[d][0] *= corr[0]; o[d][1] *= corr[0];
                o[d][2] *= corr[1]; o[d][3] *= corr[1];
            }
            // positions past the sequence's end lie in a fetched page but were never written: whatever is there
            // must not reach the sum, not even multiplied by zero.  Only the tile that holds the end has such keys.
            const bool tail = kt * BN + BN - 1 > pos_last;
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
                pf[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                pf[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pf[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int dp = 0; dp < DTILES / 2; ++dp) {
                    uint32_t vf[4];
                    const int key = key_base + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int dcol = dp * 16 + (lane >> 4) * 8;
                    ldmatrix_x4_trans(vf, swz<HD>(vbase, key, dcol));
                    if (tail) {
                        // a value register holds keys k0 + {0, 1}; the odd registers the keys 8 further on
                        const int k0 = kt * BN + key_base + kk * 16 + (lane & 3) * 2;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const int ka = k0 + (q & 1) * 8;
                            if (ka > pos_last) vf[q] &= 0xffff0000u;
                            if (ka + 1 > pos_last) vf[q] &= 0x0000ffffu;
                        }
                    }
                    mma_bf16(o[2 * dp], pf, vf[0], vf[1]);
                    mma_bf16(o[2 * dp + 1], pf, vf[2], vf[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    if (tid == 0 && s_failed) atomicExch(p.status, 3);

    if constexpr (!KEYSPLIT) {
        if (!warp_active) return;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int r = row_base + (lane >> 2) + 8 * i;
            if (!row_ok[i]) continue;
            const int tok = r / p.group, g = r - tok * p.group;
            const size_t row = (size_t)(tok0 + tok) * p.nq + kvh * p.group + g;
            if (p.n_splits == 1) {
                const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
                __nv_bfloat16* dst = p.out + row * HD;
#pragma unroll
                for (int d = 0; d < DTILES; ++d) {
                    const int col = d * 8 + (lane & 3) * 2;
                    *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
                }
            } else {
                const size_t prow = (size_t)split * p.n_tokens * p.nq + row;
                float* dst = p.part_o + prow * HD;
#pragma unroll
                for (int d = 0; d < DTILES; ++d) {
                    const int col = d * 8 + (lane & 3) * 2;
                    *reinterpret_cast<float2*>(dst + col) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
                }
                if ((lane & 3) == 0) {
                    p.part_ml[prow * 2] = m[i];
                    p.part_ml[prow * 2 + 1] = l[i];
                }
            }
        }
        return;
    }

    // KEYSPLIT: combine the four warps' partial results in warp order
    float* so = reinterpret_cast<float*>(KV);             // [NWARPS][16][HD]
    float* sml = so + NWARPS * 16 * HD;                   // [NWARPS][16][2]
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 2 && warp < NWARPS; ++i) {
        const int r = (lane >> 2) + 8 * i;
        if (r >= rows_valid) continue;
#pragma unroll
        for (int d = 0; d < DTILES; ++d) {
            const int col = d * 8 + (lane & 3) * 2;
            *reinterpret_cast<float2*>(so + (warp * 16 + r) * HD + col) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
        }
        if ((lane & 3) == 0) {
            sml[(warp * 16 + r) * 2] = m[i];
            sml[(warp * 16 + r) * 2 + 1] = l[i];
        }
    }
    __syncthreads();
    if (p.cluster) {
        // The splits of this (sequence, kv head) are one cluster, and the output's groups of four columns are dealt
        // out among its blocks: group number i falls to block i % n.  Every block adds its four warps' results and
        // stores each group's sum, with its row's (max, sum), into the shared memory of the block the group falls
        // to; after one cluster barrier each block holds all splits' shares of its groups and adds them in split
        // order.  Nothing is read from another block's memory, so no block waits for a second barrier.
        const int n = p.n_splits, per_block = (16 * (HD / 4) + n - 1) / n;
        uint32_t rank;
        asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");   // all blocks of the cluster run
        for (int it = tid; it < rows_valid * (HD / 4); it += DTHREADS) {
            const int r = it / (HD / 4), d = (it - r * (HD / 4)) * 4;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, sml[(w * 16 + r) * 2]);
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int w = 0; w < NWARPS; ++w) {
                const float mw = sml[(w * 16 + r) * 2];
                const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
                const float4 v = *reinterpret_cast<const float4*>(so + (w * 16 + r) * HD + d);
                L += f * sml[(w * 16 + r) * 2 + 1];
                acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
            }
            const uint32_t to = (uint32_t)(it % n);
            const uint32_t dst = in_block(recv + rank * per_block + it / n, to);
            asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(dst), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
            if (d == 0) {
                for (int z = 0; z < n; ++z) {
                    const uint32_t dml = in_block(recv_ml + rank * 16 + r, (uint32_t)z);
                    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};\n" ::"r"(dml), "f"(M), "f"(L) : "memory");
                }
            }
        }
        cluster_sync_all();
        for (int j = tid; j < per_block; j += DTHREADS) {
            const int it = j * n + (int)rank;
            if (it >= rows_valid * (HD / 4)) break;
            const int r = it / (HD / 4), d = (it - r * (HD / 4)) * 4;
            float M = -INFINITY;
            for (int z = 0; z < n; ++z) M = fmaxf(M, recv_ml[z * 16 + r].x);
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int z = 0; z < n; ++z) {      // in split order
                const float2 ml = recv_ml[z * 16 + r];
                const float f = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
                const float4 v = recv[z * per_block + j];
                L += f * ml.y;
                acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
            }
            const float inv = L > 0.f ? 1.f / L : 0.f;
            const int tok = r / p.group, g = r - tok * p.group;
            const size_t row = (size_t)(tok0 + tok) * p.nq + kvh * p.group + g;
            uint2 packed;
            packed.x = pack_bf16(acc.x * inv, acc.y * inv);
            packed.y = pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(p.out + row * HD + d) = packed;
        }
        return;
    }
    for (int idx = tid; idx < rows_valid * HD; idx += DTHREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, sml[(w * 16 + r) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < NWARPS; ++w) {
            const float mw = sml[(w * 16 + r) * 2];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += f * sml[(w * 16 + r) * 2 + 1];
            acc += f * so[(w * 16 + r) * HD + d];
        }
        const int tok = r / p.group, g = r - tok * p.group;
        const size_t row = (size_t)(tok0 + tok) * p.nq + kvh * p.group + g;
        if (p.n_splits == 1) {
            p.out[row * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t prow = (size_t)split * p.n_tokens * p.nq + row;
            p.part_o[prow * HD + d] = acc;
            if (d == 0) {
                p.part_ml[prow * 2] = M;
                p.part_ml[prow * 2 + 1] = L;
            }
        }
    }
    if (p.n_splits == 1 || p.counters == nullptr) return;
    // the last split of this (sequence, kv head) to finish combines all of them, in split order
    __shared__ int s_last;
    __threadfence();
    __syncthreads();
    if (tid == 0) s_last = atomicAdd(&p.counters[seq * p.nkv + kvh], 1u) == (unsigned)p.n_splits - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // Two rounds of loads, each of loads that do not wait for one another: first every split's (m, l) of every
    // row, from which each row's factors 2^(m_z - M) / L follow; then the partial outputs, four floats at a time.
    const size_t rows_all = (size_t)p.n_tokens * p.nq;
    float* factor = reinterpret_cast<float*>(KV);          // [n_splits][16]; the partial sums in KV are spent
    for (int idx = tid; idx < p.n_splits * rows_valid; idx += DTHREADS) {
        const int z = idx / rows_valid, r = idx - z * rows_valid;
        const int tok = r / p.group, g = r - tok * p.group;
        const size_t row = (size_t)(tok0 + tok) * p.nq + kvh * p.group + g;
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + (z * rows_all + row) * 2));
        factor[z * 16 + r] = ml.x;
        factor[(p.n_splits + z) * 16 + r] = ml.y;
    }
    __syncthreads();
    if (tid < rows_valid) {
        float M = -INFINITY;
        for (int z = 0; z < p.n_splits; ++z) M = fmaxf(M, factor[z * 16 + tid]);
        float L = 0.f;
        for (int z = 0; z < p.n_splits; ++z) {      // in split order
            const float mz = factor[z * 16 + tid];
            const float f = mz == -INFINITY ? 0.f : exp2f(mz - M);
            L += f * factor[(p.n_splits + z) * 16 + tid];
            factor[z * 16 + tid] = f;
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
        for (int z = 0; z < p.n_splits; ++z) factor[z * 16 + tid] *= inv;
    }
    __syncthreads();
    for (int idx = tid; idx < rows_valid * (HD / 4); idx += DTHREADS) {
        const int r = idx / (HD / 4), d = (idx - r * (HD / 4)) * 4;
        const int tok = r / p.group, g = r - tok * p.group;
        const size_t row = (size_t)(tok0 + tok) * p.nq + kvh * p.group + g;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int z = 0; z < p.n_splits; ++z) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + (z * rows_all + row) * HD + d));
            const float f = factor[z * 16 + r];
            acc.x += f * v.x; acc.y += f * v.y; acc.z += f * v.z; acc.w += f * v.w;
        }
        uint2 packed;
        packed.x = pack_bf16(acc.x, acc.y);
        packed.y = pack_bf16(acc.z, acc.w);
        *reinterpret_cast<uint2*>(p.out + row * HD + d) = packed;
    }
    if (tid == 0) p.counters[seq * p.nkv + kvh] = 0;   // zero again for the next launch
}

// out[row] = sum_z 2^(m_z - M) o_z / sum_z 2^(m_z - M) l_z over the splits, in split order, for the rows from
// first_row on that the grid covers (the other rows of the step belong to another call).
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       __nv_bfloat16* __restrict__ out, int rows, int hd, int n_splits, int first_row) {
    allow_dependents();
    const int row = first_row + blockIdx.x;
    float M = -INFINITY;
    for (int z = 0; z < n_splits; ++z) M = fmaxf(M, part_ml[((size_t)z * rows + row) * 2]);
    float L = 0.f;
    for (int z = 0; z < n_splits; ++z) {
        const float mz = part_ml[((size_t)z * rows + row) * 2];
        if (mz != -INFINITY) L += exp2f(mz - M) * part_ml[((size_t)z * rows + row) * 2 + 1];
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = threadIdx.x; d < hd; d += blockDim.x) {
        float acc = 0.f;
        for (int z = 0; z < n_splits; ++z) {
            const float mz = part_ml[((size_t)z * rows + row) * 2];
            if (mz != -INFINITY) acc += exp2f(mz - M) * part_o[((size_t)z * rows + row) * hd + d];
        }
        out[(size_t)row * hd + d] = __float2bfloat16_rn(acc * inv);
    }
}

template <int HD, bool KEYSPLIT>
int launch_flash_as(const FlashParams& p, int n_tiles, cudaStream_t s) {
    constexpr int QROWS = KEYSPLIT ? 16 : BM, STAGES = KEYSPLIT ? 3 : 2;
    constexpr size_t tiles = (size_t)(QROWS + 2 * STAGES * BN) * (HD + 8) * sizeof(__nv_bfloat16);
    constexpr size_t merge = (size_t)QROWS * (HD + 8) * sizeof(__nv_bfloat16) + (size_t)NWARPS * 16 * (HD + 2) * sizeof(float);
    constexpr size_t smem = tiles > merge ? tiles : merge;
    static bool raised[64] = {};  // per instantiation and device: the attribute is set once
    if (smem > 48 * 1024 && rmx_first_on_device(raised)) {
        cudaError_t e = cudaFuncSetAttribute(attention_flash_kernel<HD, KEYSPLIT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RMX_FAIL("attention_flash: shared memory of %zu bytes refused: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid(n_tiles, p.nkv, p.n_splits);
    attention_flash_kernel<HD, KEYSPLIT><<<grid, THREADS, smem, s>>>(p);
    RMX_CHECK_LAUNCH("attention_flash");
    return 0;
}

template <int HD>
int launch_flash(const FlashParams& p, int n_tiles, bool keysplit, cudaStream_t s) {
    return keysplit ? launch_flash_as<HD, true>(p, n_tiles, s) : launch_flash_as<HD, false>(p, n_tiles, s);
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A pool of one layer seen as [pages * kv_heads * page_size rows, hd columns]; boxes of [box_rows, 64], 128-byte swizzle.
// Maps depend on the address and the geometry only, and pools keep theirs: encoded maps are kept.
int pool_map(CUtensorMap* map, const void* base, long long rows, int hd, int box_rows) {
    struct Key {
        const void* base; long long rows; int hd, box_rows;
        bool operator==(const Key& o) const { return base == o.base && rows == o.rows && hd == o.hd && box_rows == o.box_rows; }
    };
    struct Hash {
        size_t operator()(const Key& k) const {
            return std::hash<const void*>()(k.base) ^ (std::hash<long long>()(k.rows) * 31) ^ (size_t)(k.hd * 7 + k.box_rows);
        }
    };
    static std::mutex lock;
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    static EncodeTiled fn = nullptr;
    std::lock_guard<std::mutex> guard(lock);
    const Key key{base, rows, hd, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) {
        *map = it->second;
        return 0;
    }
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            RMX_FAIL("attention_decode: the driver has no cuTensorMapEncodeTiled");
        fn = (EncodeTiled)ptr;
    }
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) RMX_FAIL("attention_decode: cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *map);
    return 0;
}

template <int HD, bool KEYSPLIT, bool FINISH = false>
int launch_tma_as(const FlashParams& p, int n_tiles, long long pool_rows, cudaStream_t s) {
    const int box_rows = p.page_size < BN ? p.page_size : BN;
    CUtensorMap mk, mv;
    if (pool_map(&mk, p.k_pool, pool_rows, HD, box_rows) != 0) return -1;
    if (pool_map(&mv, p.v_pool, pool_rows, HD, box_rows) != 0) return -1;
    constexpr int QROWS = KEYSPLIT ? 16 : BM, STAGES = KEYSPLIT ? DSTAGES : 2;
    // stages, Q rows and, for decoding, the cluster's receive buffers (16 rows of HD floats and 8 x 16 pairs)
    constexpr size_t smem = 1024 + (size_t)STAGES * 2 * 64 * HD * 2 + (size_t)QROWS * (HD + 8) * 2 +
                            (KEYSPLIT ? (size_t)16 * HD * 4 + 8 * 16 + 8 * 16 * 8 : 0);
    static bool raised[64] = {};
    if (rmx_first_on_device(raised)) {
        cudaError_t e = cudaFuncSetAttribute(attention_tma_kernel<HD, KEYSPLIT, FINISH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) RMX_FAIL("attention_tma: shared memory of %zu bytes refused: %s", smem, cudaGetErrorString(e));
    }
    dim3 grid(n_tiles, p.nkv, p.n_splits);
    if (p.cluster) {
        // the splits of one (sequence, kv head) as a cluster, and still a programmatic dependent of the kernel before
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(DTHREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = s;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = p.n_splits;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = rmx_dependent_launch_enabled() ? 2 : 1;
        RMX_CHECK_LAUNCHED(cudaLaunchKernelEx(&cfg, attention_tma_kernel<HD, KEYSPLIT, FINISH>, mk, mv, p, box_rows), "attention_tma (cluster)");
        return 0;
    }
    RMX_CHECK_LAUNCHED(launch_dependent(attention_tma_kernel<HD, KEYSPLIT, FINISH>, grid, dim3(DTHREADS), smem, s, mk, mv, p, box_rows),
                       "attention_tma");
    return 0;
}

// Whether this device can hold a cluster of `size` blocks of the decoding kernel at once (asked once per size).
template <int HD>
bool cluster_possible(int size) {
    static int known[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};   // 0: not asked, 1: yes, -1: no
    if (size < 2 || size > 8) return false;
    if (known[size] == 0) {
        constexpr size_t smem = 1024 + (size_t)DSTAGES * 2 * 64 * HD * 2 + (size_t)16 * (HD + 8) * 2 + (size_t)16 * HD * 4 + 8 * 16 + 8 * 16 * 8;
        cudaFuncSetAttribute(attention_tma_kernel<HD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(1, 1, size);
        cfg.blockDim = dim3(DTHREADS);
        cfg.dynamicSmemBytes = smem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = size;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        int clusters = 0;
        const cudaError_t e = cudaOccupancyMaxActiveClusters(&clusters, attention_tma_kernel<HD, true>, &cfg);
        if (e != cudaSuccess) cudaGetLastError();
        known[size] = e == cudaSuccess && clusters > 0 ? 1 : -1;
    }
    return known[size] > 0;
}

template <int HD>
int launch_tma(const FlashParams& p, int n_tiles, bool keysplit, long long pool_rows, cudaStream_t s) {
    if constexpr (HD == 128)
        if (keysplit && p.qkv) return launch_tma_as<HD, true, true>(p, n_tiles, pool_rows, s);
    return keysplit ? launch_tma_as<HD, true>(p, n_tiles, pool_rows, s) : launch_tma_as<HD, false>(p, n_tiles, pool_rows, s);
}
}  // namespace

// Which head sizes the tensor-core kernel is built for; others take attention_plain.
RMX_API int rmx_attention_flash_supports(int hd, int group) {
    const bool hd_ok = hd == 16 || hd == 32 || hd == 64 || hd == 96 || hd == 128;
    return hd_ok && group >= 1 && group <= 16 ? 1 : 0;
}

// qkv (or null): the projection's rows [tokens, qkv_stride] = [q heads | k heads | v heads] before norm and rotation;
// then q is not read, and the kernel norms (q_norm, k_norm: [128] floats or null, eps) and rotates (cos_sin:
// [tokens][128], cosines then sines) each sequence's one token itself and, with write_kv, stores its key and value.
// max_q_len: the most tokens any sequence brings to this step (0: unknown).  pool_pages: pages in k_pool / v_pool
// (0: unknown; the TMA path for decoding is then not taken).
// n_tiles: the number of query tiles of the batch, sum over sequences of ceil(tokens / (64 / group)).
// counters: seqs * nkv zeroed unsigned ints (left zero), or null; lets the decoding kernel combine its splits itself.
// part_o / part_ml are needed when n_splits > 1: [n_splits, tokens * nq, hd] and [n_splits, tokens * nq, 2] floats.
RMX_API int rmx_attention_flash(const void* q, const void* k_pool, const void* v_pool, const int* q_start,
                                const int* positions, const int* block_table, int table_stride, int page_size,
                                void* out, float* part_o, float* part_ml, unsigned int* counters, int n_seqs, int n_tokens, int n_tiles,
                                int nq, int nkv, int hd, int window, float scale, int n_splits, int max_q_len,
                                int pool_pages, const void* qkv, int qkv_stride, const float* q_norm, const float* k_norm,
                                float eps, const float* cos_sin, int write_kv, int first_token, int run_tokens, int* status,
                                void* stream) {
    if (n_tokens == 0) return 0;
    // first_token, run_tokens: the tokens of the sequences given here (a step's sequences may be given in several
    // calls, each with a run of them; q, out and the partial sums are those of the whole step)
    RMX_REQUIRE(first_token >= 0 && run_tokens > 0 && first_token + run_tokens <= n_tokens, "attention_flash: tokens %d + %d of %d",
                first_token, run_tokens, n_tokens);
    RMX_REQUIRE(nq > 0 && nkv > 0 && nq % nkv == 0, "attention_flash: %d query heads over %d kv heads", nq, nkv);
    const int group = nq / nkv;
    RMX_REQUIRE(rmx_attention_flash_supports(hd, group), "attention_flash: head_dim %d with group %d is not built", hd, group);
    RMX_REQUIRE(page_size > 0 && table_stride > 0 && window >= 0 && n_tiles > 0 && n_seqs > 0, "attention_flash: bad geometry");
    RMX_REQUIRE((page_size & (page_size - 1)) == 0, "attention_flash: page size %d is no power of two", page_size);
    RMX_REQUIRE(n_splits >= 1 && n_splits <= 65535 && nkv <= 65535, "attention_flash: bad grid");
    RMX_REQUIRE(n_splits == 1 || (part_o && part_ml), "attention_flash: splits need partial buffers");
    FlashParams p;
    p.q = (const __nv_bfloat16*)q; p.k_pool = (const __nv_bfloat16*)k_pool; p.v_pool = (const __nv_bfloat16*)v_pool;
    p.q_start = q_start; p.positions = positions; p.block_table = block_table; p.out = (__nv_bfloat16*)out;
    p.part_o = part_o; p.part_ml = part_ml; p.status = status; p.counters = nullptr; p.cluster = 0;
    p.qkv = (const __nv_bfloat16*)qkv; p.qkv_stride = qkv_stride; p.q_norm = q_norm; p.k_norm = k_norm; p.eps = eps; p.cos_sin = cos_sin;
    p.k_store = qkv && write_kv ? (__nv_bfloat16*)const_cast<void*>(k_pool) : nullptr;
    p.v_store = qkv && write_kv ? (__nv_bfloat16*)const_cast<void*>(v_pool) : nullptr;
    p.n_seqs = n_seqs; p.n_tokens = n_tokens; p.nq = nq; p.nkv = nkv; p.group = group; p.tq = BM / group;
    p.table_stride = table_stride; p.page_size = page_size; p.window = window; p.n_splits = n_splits;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
    p.scale_log2 = scale * LOG2E;
    cudaStream_t s = (cudaStream_t)stream;
    // every tile has at most 16 rows (decoding, or very short portions): spread keys over the warps
    const bool keysplit = max_q_len > 0 && max_q_len * group <= 16;
    int rc;
    // at the head sizes of real models keys and values come by TMA (pool_pages tells the pool's extent)
    const bool by_tma = pool_pages > 0 && page_size >= 8 && (hd == 64 || hd == 128) && (!keysplit || n_tiles == n_seqs) &&
                        ((uintptr_t)k_pool & 127) == 0 && ((uintptr_t)v_pool & 127) == 0;
    if (qkv) {
        RMX_REQUIRE(by_tma && keysplit && hd == 128 && max_q_len == 1 && n_tokens == n_seqs && cos_sin != nullptr,
                    "attention_flash: the projection's rows are taken as they come only when decoding one token a sequence by TMA with heads of 128");
        RMX_REQUIRE(qkv_stride >= (nq + 2 * nkv) * 128 && qkv_stride % 4 == 0 && ((uintptr_t)qkv & 7) == 0, "attention_flash: bad projection rows");
    } else {
        RMX_REQUIRE(q != nullptr, "attention_flash: no queries");
    }
    if (by_tma) {
        const long long pool_rows = (long long)pool_pages * nkv * page_size;
        // The decoding arrangement combines its splits itself: up to 8 as a thread-block cluster, through
        // distributed shared memory; more (up to 128) through the partial buffers, the last block to finish adding
        // them, if the caller gave counters.
        if (keysplit && n_splits >= 2 && n_splits <= 8 && (hd == 64 ? cluster_possible<64>(n_splits) : cluster_possible<128>(n_splits)))
            p.cluster = 1;
        else if (keysplit && n_splits <= 128) p.counters = counters;
        rc = hd == 64 ? launch_tma<64>(p, n_tiles, keysplit, pool_rows, s) : launch_tma<128>(p, n_tiles, keysplit, pool_rows, s);
        if (rc == 0 && (p.cluster || p.counters)) return 0;
        p.cluster = 0;
    } else
    switch (hd) {
        case 16: rc = launch_flash<16>(p, n_tiles, keysplit, s); break;
        case 32: rc = launch_flash<32>(p, n_tiles, keysplit, s); break;
        case 64: rc = launch_flash<64>(p, n_tiles, keysplit, s); break;
        case 96: rc = launch_flash<96>(p, n_tiles, keysplit, s); break;
        default: rc = launch_flash<128>(p, n_tiles, keysplit, s); break;
    }
    if (rc != 0) return rc;
    if (n_splits > 1) {
        attention_merge_kernel<<<run_tokens * nq, hd >= 128 ? 128 : 64, 0, s>>>(part_o, part_ml, (__nv_bfloat16*)out, n_tokens * nq, hd, n_splits,
                                                                                first_token * nq);
        RMX_CHECK_LAUNCH("attention_merge");
    }
    return 0;
}

RMX_API int rmx_attention_flash_tile_tokens(int group) { return BM / group; }

// Whether a decoding step (one token a sequence) may hand rmx_attention_flash the projection's rows as they come.
RMX_API int rmx_attention_flash_takes_projection(int hd, int group, int page_size, int rotary_dim) {
    return hd == 128 && rotary_dim == 128 && group >= 1 && group <= 16 && page_size >= 8 && (page_size & (page_size - 1)) == 0 ? 1 : 0;
}
