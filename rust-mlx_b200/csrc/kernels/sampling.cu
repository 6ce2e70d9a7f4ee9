// Choosing the next token from float logits: greedy (lowest id wins a tie, the rule of
// the reference's greedy head, kernels/greedy_reduce.metal:10-14) and temperature
// sampling, p = softmax(logits / temperature), by inversion of the cumulative sum with
// a uniform number that the host derives from (seed, request, step).
//
// One block per row.  All sums are formed in an order fixed by the vocabulary size and
// the block size, so a row's choice does not depend on the other rows of the batch.
#include "common.cuh"

namespace {
constexpr int THREADS = 1024;

__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, int ld,
                                                         const float* __restrict__ temperature,
                                                         const float* __restrict__ uniform, int* __restrict__ out,
                                                         int vocab, const int* __restrict__ slots,
                                                         int* __restrict__ last_tokens) {
    __shared__ float s_val[THREADS];
    __shared__ int s_idx[THREADS];
    __shared__ int s_choice;
    allow_dependents();        // (what follows waits for this kernel before it touches memory)
    wait_for_prior_kernels();
    const int r = blockIdx.x, tid = threadIdx.x;
    const float* row = logits + (size_t)r * ld;

    // argmax, lowest index on ties; NaN never wins
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    auto take = [&](float v, int i) {
        if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
    };
    // four logits a load where the row starts on a 16-byte boundary, several loads in flight
    const int n4 = (reinterpret_cast<uintptr_t>(row) & 15) == 0 ? vocab / 4 : 0;
#pragma unroll 4
    for (int i = tid; i < n4; i += THREADS) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(row) + i);
        take(v.x, 4 * i);
        take(v.y, 4 * i + 1);
        take(v.z, 4 * i + 2);
        take(v.w, 4 * i + 3);
    }
    for (int i = 4 * n4 + tid; i < vocab; i += THREADS) take(row[i], i);
    s_val[tid] = best;
    s_idx[tid] = best_i;
    __syncthreads();
    for (int stride = THREADS / 2; stride > 0; stride >>= 1) {
        if (tid < stride) {
            const float v = s_val[tid + stride];
            const int i = s_idx[tid + stride];
            if (v > s_val[tid] || (v == s_val[tid] && i < s_idx[tid])) { s_val[tid] = v; s_idx[tid] = i; }
        }
        __syncthreads();
    }
    const float row_max = s_val[0];
    const int arg = s_idx[0] == 0x7fffffff ? 0 : s_idx[0];
    const float temp = temperature ? temperature[r] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) {
            out[r] = arg;
            if (last_tokens) last_tokens[slots[r]] = arg;
        }
        return;
    }
    __syncthreads();

    // every thread owns a contiguous chunk; chunk sums, then an inclusive scan over threads
    const float inv_t = 1.f / temp;
    const int chunk = (vocab + THREADS - 1) / THREADS;
    const int c0 = min(vocab, tid * chunk), c1 = min(vocab, c0 + chunk);
    float sum = 0.f;
    for (int i = c0; i < c1; ++i) sum += expf((row[i] - row_max) * inv_t);
    s_val[tid] = sum;
    __syncthreads();
    if (tid == 0) {
        float run = 0.f;
        for (int i = 0; i < THREADS; ++i) { run += s_val[i]; s_val[i] = run; }
        s_choice = -1;
    }
    __syncthreads();
    const float total = s_val[THREADS - 1];
    const float target = uniform[r] * total;
    const float before = tid == 0 ? 0.f : s_val[tid - 1];
    if (c1 > c0 && target >= before && target < s_val[tid]) {
        float run = before;
        int pick = c1 - 1;
        for (int i = c0; i < c1; ++i) {
            run += expf((row[i] - row_max) * inv_t);
            if (target < run) { pick = i; break; }
        }
        s_choice = pick;
    }
    __syncthreads();
    if (tid == 0) {
        const int choice = s_choice >= 0 ? s_choice : arg;  // target == total by rounding: the likeliest token
        out[r] = choice;
        if (last_tokens) last_tokens[slots[r]] = choice;
    }
}
}  // namespace

// slots / last_tokens (both or neither): the choice of row r is also left at last_tokens[slots[r]], where the next
// step's embedding can find it without a trip through the host.
RMX_API int rmx_sample(const float* logits, int ld, const float* temperature, const float* uniform, int* out,
                       int n_rows, int vocab, const int* slots, int* last_tokens, void* stream) {
    if (n_rows == 0) return 0;
    RMX_REQUIRE(n_rows > 0 && vocab > 0 && ld >= vocab, "sample: bad sizes");
    RMX_REQUIRE(temperature == nullptr || uniform != nullptr, "sample: temperatures without uniform numbers");
    RMX_REQUIRE((slots == nullptr) == (last_tokens == nullptr), "sample: slots and last_tokens go together");
    RMX_CHECK_LAUNCHED(launch_dependent(sample_kernel, dim3(n_rows), dim3(THREADS), 0, (cudaStream_t)stream, logits, ld, temperature,
                                        uniform, out, vocab, slots, last_tokens), "sample");
    return 0;
}
