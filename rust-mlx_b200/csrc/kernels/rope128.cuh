// One head of 128 bfloat16 numbers in a warp: lane l holds numbers 4 l .. 4 l + 3.  RMSNorm over the head (float,
// weight `norm_w` or none), then the half-split rotation with the cosines and sines of the token's position
// (`cos_sin`: 64 cosines then 64 sines; number j pairs with j + 64, which lies sixteen lanes away), one rounding
// to bfloat16.  Shared by the kernel that does this for all tokens of a step and by the decoding attention,
// which does it for its own token while it waits for its first keys: the same instructions, the same bits.
#pragma once
#include "common.cuh"

__device__ __forceinline__ uint2 rope128_head(uint2 raw, const float* __restrict__ norm_w, float eps,
                                              const float* __restrict__ cos_sin, int lane) {
    constexpr int hd = 128;
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    float v[4] = {lo.x, lo.y, hi.x, hi.y};
    if (norm_w) {
        float ss = v[0] * v[0];
        ss += v[1] * v[1];
        ss += v[2] * v[2];
        ss += v[3] * v[3];
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)hd + eps);
        const float4 w = *reinterpret_cast<const float4*>(norm_w + lane * 4);
        v[0] = v[0] * inv * w.x; v[1] = v[1] * inv * w.y; v[2] = v[2] * inv * w.z; v[3] = v[3] * inv * w.w;
    }
    const int j = (lane & 15) * 4;   // index of the pair (j, j + 64) this lane's numbers belong to
    const float4 cs = *reinterpret_cast<const float4*>(cos_sin + j);
    const float4 sn = *reinterpret_cast<const float4*>(cos_sin + 64 + j);
    const float c[4] = {cs.x, cs.y, cs.z, cs.w}, s_[4] = {sn.x, sn.y, sn.z, sn.w};
    float out[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, v[i], 16);
        // lanes 0..15 hold x[j] (partner x[j + 64] comes from lane + 16): out = a cos - b sin
        // lanes 16..31 hold x[j + 64] (partner x[j]):                      out = b cos + a sin
        out[i] = lane < 16 ? v[i] * c[i] - other * s_[i] : v[i] * c[i] + other * s_[i];
    }
    __nv_bfloat162 o01 = __floats2bfloat162_rn(out[0], out[1]), o23 = __floats2bfloat162_rn(out[2], out[3]);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&o01);
    packed.y = *reinterpret_cast<uint32_t*>(&o23);
    return packed;
}
