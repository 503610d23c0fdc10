// Routed experts: which experts a token uses and with what weight.
//
//   moe_route       one warp a row.  scores = softmax(logits) over all E experts (float32), or with score_kind 1 the sigmoid of
//                   every logit by itself.  The experts form `groups`
//                   equal groups of neighbours; a group's score is its largest score, and only experts of the `keep` best
//                   groups can be chosen (groups <= 1 or keep >= groups: all can).  The `top` largest scores among those are
//                   chosen (of equal scores the lower index first); their weights are the scores themselves, not
//                   renormalised.  weights [rows, E] receives the score of a chosen expert and 0 for every other; chosen
//                   [rows, top] the indices, best first.
//   moe_scale       act[r, e, j] *= weights[r, e] over act [rows, E, ff]: after this, one product with every expert's output
//                   matrix side by side is the weighted sum of the chosen experts' outputs (the others contribute zeros).
#include "api.h"
#include "common.cuh"

namespace citlali {

constexpr int kMaxExpertsPerLane = 16;      // E <= 512

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ logits, float* __restrict__ weights, int32_t* __restrict__ chosen, int rows, int E,
                 int groups, int keep, int top, float weight_scale, int score_kind) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* z = logits + (size_t)row * E;
    float s[kMaxExpertsPerLane];
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j) {
        const int e = lane + 32 * j;
        s[j] = e < E ? z[e] : -INFINITY;
        m = fmaxf(m, s[j]);
    }
    if (score_kind == 1) {
#pragma unroll
        for (int j = 0; j < kMaxExpertsPerLane; ++j) s[j] = lane + 32 * j < E ? 1.0f / (1.0f + expf(-s[j])) : 0.0f;
    } else {
        m = warp_max(m);
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < kMaxExpertsPerLane; ++j) {
            const int e = lane + 32 * j;
            s[j] = e < E ? expf(s[j] - m) : 0.0f;
            sum += s[j];
        }
        sum = warp_sum(sum);
#pragma unroll
        for (int j = 0; j < kMaxExpertsPerLane; ++j) s[j] = s[j] / sum;
    }
    // which experts may be chosen: bit j of `open` for expert lane + 32 j
    unsigned open = 0;
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j)
        if (lane + 32 * j < E) open |= 1u << j;
    if (groups > 1 && keep < groups) {
        const int per = E / groups;
        unsigned kept_mine = 0;                              // groups are looked at one after another; `keep` rounds
        // a group's score: the largest score in it.  Lane l keeps the scores of groups l, l + 32, ... (at most 16 each).
        float gs[kMaxExpertsPerLane];
#pragma unroll
        for (int j = 0; j < kMaxExpertsPerLane; ++j) gs[j] = -INFINITY;
        for (int grp = 0; grp < groups; ++grp) {
            float best = -INFINITY;
#pragma unroll
            for (int j = 0; j < kMaxExpertsPerLane; ++j) {
                const int e = lane + 32 * j;
                if (e < E && e / per == grp) best = fmaxf(best, s[j]);
            }
            best = warp_max(best);
#pragma unroll
            for (int j = 0; j < kMaxExpertsPerLane; ++j)
                if (grp == lane + 32 * j) gs[j] = best;
        }
        for (int round = 0; round < keep; ++round) {
            float best = -INFINITY;
            int arg = 0x7fffffff;
#pragma unroll
            for (int j = 0; j < kMaxExpertsPerLane; ++j) {
                const int grp = lane + 32 * j;
                if (grp < groups && !(kept_mine >> j & 1u) && (gs[j] > best || (gs[j] == best && grp < arg))) { best = gs[j]; arg = grp; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
                if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
            }
#pragma unroll
            for (int j = 0; j < kMaxExpertsPerLane; ++j)
                if (arg == lane + 32 * j) kept_mine |= 1u << j;
        }
        // an expert is open if its group was kept: ask the lane that holds the group's bit
        unsigned allowed = 0;
#pragma unroll
        for (int j = 0; j < kMaxExpertsPerLane; ++j) {
            const int e = lane + 32 * j;
            const int grp = e < E ? e / per : 0;
            const unsigned bits = __shfl_sync(0xffffffffu, kept_mine, grp & 31);
            if (e < E && (bits >> (grp >> 5) & 1u)) allowed |= 1u << j;
        }
        open = allowed;
    }
    unsigned taken = 0;
    for (int round = 0; round < top; ++round) {
        float best = -INFINITY;
        int arg = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < kMaxExpertsPerLane; ++j) {
            const int e = lane + 32 * j;
            if ((open >> j & 1u) && !(taken >> j & 1u) && (s[j] > best || (s[j] == best && e < arg))) { best = s[j]; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
#pragma unroll
        for (int j = 0; j < kMaxExpertsPerLane; ++j)
            if (arg == lane + 32 * j) taken |= 1u << j;
        if (lane == 0 && chosen) chosen[(size_t)row * top + round] = arg;
    }
#pragma unroll
    for (int j = 0; j < kMaxExpertsPerLane; ++j) {
        const int e = lane + 32 * j;
        if (e < E) weights[(size_t)row * E + e] = (taken >> j & 1u) ? s[j] * weight_scale : 0.0f;
    }
}

template <typename T>
__global__ void moe_scale_kernel(T* __restrict__ act, const float* __restrict__ weights, int E, int ff) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const int n = E * ff;
    T* a = act + (size_t)row * n;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        const float w = weights[(size_t)row * E + i / ff];
        stf(a, i, w == 0.0f ? 0.0f : ldf(a, i) * w);
    }
}

// The same for bfloat16 rows whose experts' widths are multiples of 8: 16-byte words, each within one expert.
__global__ void moe_scale_vec_kernel(__nv_bfloat16* __restrict__ act, const float* __restrict__ weights, int E, int ff) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const int words = E * ff / 8;
    uint4* a = reinterpret_cast<uint4*>(act + (size_t)row * E * ff);
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < words; i += gridDim.y * blockDim.x) {
        const float w = weights[(size_t)row * E + (i * 8) / ff];
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (w != 0.0f) {
            v = a[i];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h[e]);
                h[e] = __floats2bfloat162_rn(f.x * w, f.y * w);
            }
        }
        a[i] = v;
    }
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_moe_route(const float* logits, float* weights, int32_t* chosen, int rows, int E, int groups, int keep,
                                 int top, float weight_scale, int score_kind, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (score_kind != 0 && score_kind != 1) {
        set_last_error("moe_route: score kind %d is neither softmax (0) nor sigmoid (1)", score_kind);
        return kBadShape;
    }
    if (E <= 0 || E > 32 * kMaxExpertsPerLane || top <= 0 || top > E) {
        set_last_error("moe_route: %d experts (at most %d), %d chosen", E, 32 * kMaxExpertsPerLane, top);
        return kBadShape;
    }
    if (groups > 1 && (E % groups != 0 || keep <= 0 || (keep < groups && keep * (E / groups) < top))) {
        set_last_error("moe_route: %d experts in %d groups of which %d are kept cannot give %d experts", E, groups, keep, top);
        return kBadShape;
    }
    launch_kernel(moe_route_kernel, (rows + 3) / 4, 128, 0, stream, logits, weights, chosen, rows, E, groups, keep, top, weight_scale,
                  score_kind);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_moe_scale(void* act, int dtype, const float* weights, int rows, int E, int ff, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == kBF16 && ff % 8 == 0 && ((uintptr_t)act & 15u) == 0) {
        const int by = (E * ff / 8 + 255) / 256;
        dim3 grid(rows, by < 64 ? by : 64);
        launch_kernel(moe_scale_vec_kernel, grid, 256, 0, stream, (__nv_bfloat16*)act, weights, E, ff);
        return CITLALI_LAUNCH_CHECK();
    }
    return CITLALI_DISPATCH_FLOAT(dtype, T, [&] {
        const int by = (E * ff + 255) / 256;
        dim3 grid(rows, by < 64 ? by : 64);
        launch_kernel(moe_scale_kernel<T>, grid, 256, 0, stream, (T*)act, weights, E, ff);
        return CITLALI_LAUNCH_CHECK();
    });
}
