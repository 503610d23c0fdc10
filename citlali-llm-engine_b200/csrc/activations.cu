// Activations that take a bias, two parameters or a clamp, each one pass over a product's result.
//
//   bias_xielu        out = xielu(z + bias):  u > 0: ap u^2 + u / 2;  u <= 0: an (exp(u) - 1 - u) + u / 2, with
//                     ap = softplus(p) and an = 1/2 + softplus(q) made by the caller.  float32 inside, rounded at the store.
//   add_row_bias      y[r] += bias over float32 rows (a product's bias where nothing behind the product takes it along).
//   expert_gate       the gated activation of E experts and an optional expert that every row uses, from one product whose
//                     columns are, expert after expert, gate and up alternating in runs:
//                         kind 0:  silu(g) u
//                         kind 1:  g' = min(g, limit), u' = clamp(u, -limit, limit);  g' sigmoid(alpha g') (u' + 1)
//                         kind 2:  gelu_tanh(g) u,  gelu_tanh(z) = z / 2 (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))
//                     after an optional bias on gate and up,
//                     times the row's weight for the expert (zero: the expert's activations are zeros and its inputs are
//                     not read), or, with weight_input, of the activation of gate and up each times that weight (the
//                     expert applied to its weighted input).  The expert for every row comes last, has a width, run and
//                     limit of its own and weight 1.
#include "api.h"
#include "common.cuh"

namespace citlali {

__device__ __forceinline__ float xielu(float u, float ap, float an) {
    return u > 0.0f ? fmaf(ap * u, u, 0.5f * u) : fmaf(an, expm1f(u) - u, 0.5f * u);
}
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                       __uint_as_float(u.y & 0xffff0000u));
}
__device__ __forceinline__ void store4(float* p, const float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

// A block row (and a share of its columns); VEC: four neighbouring columns a thread (n a multiple of four, 16-byte rows).
template <typename TZ, typename TO, bool VEC>
__global__ void __launch_bounds__(256)
bias_xielu_kernel(const TZ* __restrict__ z, const float* __restrict__ bias, float ap, float an, TO* __restrict__ out, int n) {
    dependents_may_launch();
    wait_for_predecessor();
    const TZ* zr = z + (size_t)blockIdx.x * n;
    TO* o = out + (size_t)blockIdx.x * n;
    if constexpr (VEC) {
        for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < n; c += gridDim.y * blockDim.x * 4) {
            float4 u = load4(zr + c);
            if (bias) {
                const float4 b = *reinterpret_cast<const float4*>(bias + c);
                u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
            store4(o + c, make_float4(xielu(u.x, ap, an), xielu(u.y, ap, an), xielu(u.z, ap, an), xielu(u.w, ap, an)));
        }
    } else {
        for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
            float u = ldf(zr, c);
            if (bias) u += bias[c];
            stf(o, c, xielu(u, ap, an));
        }
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256)
add_row_bias_kernel(float* __restrict__ y, const float* __restrict__ bias, size_t total, int n) {
    dependents_may_launch();
    wait_for_predecessor();
    if constexpr (VEC) {                                      // rows of a multiple of four floats: 16-byte words
        for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += (size_t)gridDim.x * blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(y + i);
            const float4 b = *reinterpret_cast<const float4*>(bias + i % n);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            *reinterpret_cast<float4*>(y + i) = v;
        }
    } else {
        for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
            y[i] += bias[i % n];
    }
}

__device__ __forceinline__ float gated(float g, float u, int kind, float limit, float alpha) {
    if (kind == 0) return g / (1.0f + expf(-g)) * u;
    if (kind == 2) return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * fmaf(0.044715f * g * g, g, g))) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
}

template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
expert_gate_kernel(const TZ* __restrict__ gu, const float* __restrict__ weights, TO* __restrict__ act, int E, int ff, int run,
                   int kind, float limit, float alpha, int tail_ff, int tail_run, float tail_limit,
                   const float* __restrict__ bias, int weight_input) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const int routed = E * ff, n = routed + tail_ff;
    const TZ* in = gu + (size_t)row * 2 * n;
    TO* o = act + (size_t)row * n;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += gridDim.y * blockDim.x) {
        float r = 0.0f;
        if (i < routed) {
            const int e = i / ff, j = i % ff;
            const float w = weights[(size_t)row * E + e];
            if (w != 0.0f) {
                const size_t at = (size_t)e * 2 * ff + (size_t)(j / run) * 2 * run + j % run;
                float g = ldf(in, at), u = ldf(in, at + run);
                if (bias) { g += bias[at]; u += bias[at + run]; }
                r = weight_input ? gated(w * g, w * u, kind, limit, alpha) : w * gated(g, u, kind, limit, alpha);
            }
        } else {
            const int j = i - routed;
            const size_t at = (size_t)2 * routed + (size_t)(j / tail_run) * 2 * tail_run + j % tail_run;
            float g = ldf(in, at), u = ldf(in, at + tail_run);
            if (bias) { g += bias[at]; u += bias[at + tail_run]; }
            r = gated(g, u, kind, tail_limit, alpha);
        }
        stf(o, i, r);
    }
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_bias_xielu(const void* z, int z_dtype, const float* bias, float ap, float an, void* out, int out_dtype,
                                  int rows, int n, cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return 0;
    const bool vec = n % 4 == 0 && (((uintptr_t)z | (uintptr_t)out | (uintptr_t)bias) & 15u) == 0;
    const int per_block = vec ? 1024 : 256;
    const int by = (n + per_block - 1) / per_block;
    const dim3 grid(rows, by < 64 ? by : 64);
    return CITLALI_DISPATCH_FLOAT(z_dtype, TZ, [&] {
        return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
            if (vec) launch_kernel(bias_xielu_kernel<TZ, TO, true>, grid, 256, 0, stream, (const TZ*)z, bias, ap, an, (TO*)out, n);
            else launch_kernel(bias_xielu_kernel<TZ, TO, false>, grid, 256, 0, stream, (const TZ*)z, bias, ap, an, (TO*)out, n);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_add_row_bias(float* y, const float* bias, int rows, int n, cudaStream_t stream) {
    if (rows <= 0 || n <= 0) return 0;
    const size_t total = (size_t)rows * n;
    const bool vec = n % 4 == 0 && (((uintptr_t)y | (uintptr_t)bias) & 15u) == 0;
    const size_t blocks = (total / (vec ? 4 : 1) + 255) / 256;
    const int grid = (int)(blocks < 16384 ? blocks : 16384);
    if (vec) launch_kernel(add_row_bias_kernel<true>, grid, 256, 0, stream, y, bias, total, n);
    else launch_kernel(add_row_bias_kernel<false>, grid, 256, 0, stream, y, bias, total, n);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_expert_gate(const void* gate_up, int in_dtype, const float* weights, void* act, int act_dtype, int rows,
                                   int E, int ff, int run, int kind, float limit, float alpha, int tail_ff, int tail_run,
                                   float tail_limit, const float* bias, int weight_input, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (E < 0 || ff < 0 || tail_ff < 0 || (E > 0 && (ff <= 0 || run <= 0 || ff % run != 0 || weights == nullptr)) ||
        (tail_ff > 0 && (tail_run <= 0 || tail_ff % tail_run != 0)) || kind < 0 || kind > 2 || E * ff + tail_ff <= 0) {
        set_last_error("expert_gate: %d experts of %d in runs of %d, an expert for all of %d in runs of %d, kind %d", E, ff, run,
                       tail_ff, tail_run, kind);
        return kBadShape;
    }
    const int n = E * ff + tail_ff;
    const int by = (n + 255) / 256;
    dim3 grid(rows, by < 64 ? by : 64);
    return CITLALI_DISPATCH_FLOAT(in_dtype, TZ, [&] {
        return CITLALI_DISPATCH_FLOAT(act_dtype, TO, [&] {
            launch_kernel(expert_gate_kernel<TZ, TO>, grid, 256, 0, stream, (const TZ*)gate_up, weights, (TO*)act, E, ff,
                          run > 0 ? run : 1, kind, limit, alpha, tail_ff, tail_run > 0 ? tail_run : 1, tail_limit, bias, weight_input);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}
