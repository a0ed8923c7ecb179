// RoPE index and trigonometry helpers shared by the glue kernels and the attention kernel that
// folds RoPE in.
#pragma once
#include "common.cuh"

namespace smelt {

// RoPE helpers (Resources/Shaders/attention.metal:11-115).
__device__ __forceinline__ void rope_indices(int layout, int dim, int half_rope, int head_dim, int& d0, int& d1,
                                             int& c0, int& c1) {
    if (layout == 1) { d0 = dim; d1 = dim + half_rope; c0 = d0; c1 = d1; }
    else if (layout == 2) { d0 = dim; d1 = dim + head_dim / 2; c0 = dim; c1 = dim + half_rope; }
    else { d0 = dim * 2; d1 = d0 + 1; c0 = d0; c1 = d1; }
}
__device__ __forceinline__ void rope_trig(int pair, int half_rope, uint32_t position, float base_log2, int math_mode,
                                          const __half* cos_t, const __half* sin_t, int c0i, int c1i, float& c0,
                                          float& s0, float& c1, float& s1) {
    if (math_mode == 1) {
        // exp2, cos and sin are evaluated in double and rounded once, i.e. correctly rounded
        // fp32 results, so the host oracle and the device agree bit for bit even at angles of
        // tens of thousands of radians where one fp32 ulp of the frequency moves the phase.
        const float d = (float)pair / (float)half_rope;
        const float inv_freq = (float)exp2((double)(-d * base_log2));
        const float angle = (float)position * inv_freq;
        double sd, cd;
        sincos((double)angle, &sd, &cd);
        const float s = (float)sd, c = (float)cd;
        c0 = c; s0 = s; c1 = c; s1 = s;
    } else {
        c0 = __half2float(cos_t[c0i]); s0 = __half2float(sin_t[c0i]);
        c1 = __half2float(cos_t[c1i]); s1 = __half2float(sin_t[c1i]);
    }
}

}  // namespace smelt
