// Kernels of a layer whose norm sits on the sub-layer's OUTPUT:  x <- x + layer_norm(sublayer(x)).
//
//   layer_norm_add   x[r] += (y[r] - mean) / sqrt(var + eps) * w  (var = mean of squared deviations, no bias), all
//                    32-bit; optionally the updated row is also left in the compute dtype for the sub-layer that reads
//                    it next, so that the residual is read once.
//   layer_norm_rows  out[i] = layer_norm(x[index[i]]) * w, rounded once (the model's last norm).
//   cast_rows        float32 -> the compute dtype.
//   scaled_sum       out = a * l + b * r (two mixers side by side).
// One block a row; the row waits in shared memory between the passes (mean, then deviations, then the store), so every
// row is read from global memory once.
#include "api.h"
#include "common.cuh"

namespace citlali {

template <typename TG, typename TE>
__global__ void __launch_bounds__(256)
layer_norm_add_kernel(const float* __restrict__ y, const TG* __restrict__ gain, float* __restrict__ x, TE* __restrict__ emit,
                      int hidden, float eps) {
    extern __shared__ float row_s[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = y + (size_t)row * hidden;
    float s = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i];
        row_s[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_s[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    float* dst = x + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = dst[i] + (row_s[i] - mean) * inv * ldf(gain, i);
        dst[i] = v;
        if (emit) stf(emit, (size_t)row * hidden + i, v);
    }
}

template <typename TG, typename TO>
__global__ void __launch_bounds__(256)
layer_norm_rows_kernel(const float* __restrict__ x, const TG* __restrict__ gain, const TG* __restrict__ bias,
                       const int32_t* __restrict__ row_index, TO* __restrict__ out, int hidden, float eps) {
    extern __shared__ float row_s[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = x + (size_t)(row_index ? row_index[row] : row) * hidden;
    float s = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i];
        row_s[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_s[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        stf(out, (size_t)row * hidden + i, (row_s[i] - mean) * inv * ldf(gain, i) + (bias ? ldf(bias, i) : 0.0f));
}

// The same two kernels for rows that are multiples of 4 and at most 8192 elements: a thread keeps its part of the row in
// registers (two 16-byte words at most), so the row is read once with 16-byte loads; few rows get up to 1024 threads each.
template <typename TE>
__device__ __forceinline__ void store4(TE* p, size_t at, const float4& v) {
    if constexpr (sizeof(TE) == 2) {
        uint2 w;
        *reinterpret_cast<__nv_bfloat162*>(&w.x) = __floats2bfloat162_rn(v.x, v.y);
        *reinterpret_cast<__nv_bfloat162*>(&w.y) = __floats2bfloat162_rn(v.z, v.w);
        *reinterpret_cast<uint2*>(p + at) = w;
    } else {
        *reinterpret_cast<float4*>(p + at) = v;
    }
}
template <typename TG>
__device__ __forceinline__ float4 load4(const TG* p, size_t at) {
    if constexpr (sizeof(TG) == 2) {
        const uint2 w = *reinterpret_cast<const uint2*>(p + at);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w.y));
        return make_float4(lo.x, lo.y, hi.x, hi.y);
    } else {
        return *reinterpret_cast<const float4*>(p + at);
    }
}

// ADD: x += norm(y) and emit; otherwise out = norm(x[index]).
template <typename TG, typename TO, bool ADD>
__global__ void __launch_bounds__(1024)
layer_norm_vec_kernel(const float* __restrict__ src_rows, const TG* __restrict__ gain, const TG* __restrict__ bias,
                      const int32_t* __restrict__ row_index, float* __restrict__ x, TO* __restrict__ out, int hidden, float eps) {
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = src_rows + (size_t)((!ADD && row_index) ? row_index[row] : row) * hidden;
    const int quads = hidden >> 2;
    float4 v[2];
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int qd = threadIdx.x + j * blockDim.x;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (qd < quads) v[j] = *reinterpret_cast<const float4*>(src + qd * 4);
        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int qd = threadIdx.x + j * blockDim.x;
        if (qd < quads) {
            v[j].x -= mean; v[j].y -= mean; v[j].z -= mean; v[j].w -= mean;
            ss = fmaf(v[j].x, v[j].x, ss); ss = fmaf(v[j].y, v[j].y, ss); ss = fmaf(v[j].z, v[j].z, ss); ss = fmaf(v[j].w, v[j].w, ss);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int qd = threadIdx.x + j * blockDim.x;
        if (qd < quads) {
            const float4 g = load4(gain, (size_t)qd * 4);
            float4 r = make_float4(v[j].x * inv * g.x, v[j].y * inv * g.y, v[j].z * inv * g.z, v[j].w * inv * g.w);
            if (bias) {
                const float4 b = load4(bias, (size_t)qd * 4);
                r.x += b.x; r.y += b.y; r.z += b.z; r.w += b.w;
            }
            const size_t at = (size_t)row * hidden + qd * 4;
            if (ADD) {
                const float4 old = *reinterpret_cast<const float4*>(x + at);
                r.x += old.x; r.y += old.y; r.z += old.z; r.w += old.w;
                *reinterpret_cast<float4*>(x + at) = r;
                if (out) store4(out, at, r);
            } else {
                store4(out, at, r);
            }
        }
    }
}

// threads a row for the kernel above: one 16-byte word a thread up to 1024 threads.  The number follows the row's length
// alone, so a row's sums are taken in one order whatever the step's size.
static int vec_threads(int rows, int hidden) {
    (void)rows;
    int t = ((hidden / 4 + 31) / 32) * 32;
    return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}
static bool vec_ok(int hidden, const void* a, const void* b, const void* c, const void* d) {
    return hidden % 4 == 0 && hidden <= 8192 && (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d) & 15u) == 0;
}

template <typename TO>
__global__ void cast_rows_kernel(const float* __restrict__ x, TO* __restrict__ out, size_t n) {
    dependents_may_launch();
    wait_for_predecessor();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) stf(out, i, x[i]);
}

__global__ void scaled_sum_kernel(float a, const float* __restrict__ l, float b, const float* __restrict__ r,
                                  float* __restrict__ out, size_t n) {
    dependents_may_launch();
    wait_for_predecessor();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = a * l[i] + b * r[i];
}

// A norm on a sub-layer's output, the sum, and the norm in front of the next sub-layer in one pass over the row:
//   x[r] += layer_norm(y[r] + in_bias) * g1 + b1;   emit[r] = x[r] (rounded);   out2[r] = layer_norm(x[r]) * g2 + b2.
// in_bias, b1, emit and the second norm (g2 null: none; b2 may be null) are optional; gains and biases are float32.  One
// block a row whose thread count follows the row's length alone; the row waits in shared memory between the passes.
template <typename TE>
__global__ void __launch_bounds__(1024)
layer_norm_chain_kernel(const float* __restrict__ y, const float* __restrict__ in_bias, const float* __restrict__ g1,
                        const float* __restrict__ b1, float* __restrict__ x, TE* __restrict__ emit, const float* __restrict__ g2,
                        const float* __restrict__ b2, TE* __restrict__ out2, int hidden, float eps1, float eps2) {
    extern __shared__ float row_s[];
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = y + (size_t)row * hidden;
    float s = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = src[i] + (in_bias ? in_bias[i] : 0.0f);
        row_s[i] = v;
        s += v;
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_s[i] - mean;
        ss = fmaf(d, d, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps1);
    float* dst = x + (size_t)row * hidden;
    float s2 = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = dst[i] + ((row_s[i] - mean) * inv * g1[i] + (b1 ? b1[i] : 0.0f));
        dst[i] = v;
        if (emit) stf(emit, (size_t)row * hidden + i, v);
        row_s[i] = v;
        s2 += v;
    }
    if (g2 == nullptr) return;
    const float mean2 = block_sum(s2, scratch) / (float)hidden;
    float ss2 = 0.0f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float d = row_s[i] - mean2;
        ss2 = fmaf(d, d, ss2);
    }
    const float inv2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)hidden + eps2);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        stf(out2, (size_t)row * hidden + i, (row_s[i] - mean2) * inv2 * g2[i] + (b2 ? b2[i] : 0.0f));
}

__device__ __forceinline__ void store4(float* p, size_t i, const float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* p, size_t i, const float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<const uint32_t*>(&lo);
    u.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p + i) = u;
}

// The same chain for rows whose length is a multiple of four and at most 4096 NV: a thread keeps NV runs of four
// elements in registers through all passes (16-byte loads and stores, no copy of the row in shared memory).  The order of
// the sums follows the row's length alone.
template <typename TE, int NV>
__global__ void __launch_bounds__(1024)
layer_norm_chain_vec_kernel(const float* __restrict__ y, const float* __restrict__ in_bias, const float* __restrict__ g1,
                            const float* __restrict__ b1, float* __restrict__ x, TE* __restrict__ emit,
                            const float* __restrict__ g2, const float* __restrict__ b2, TE* __restrict__ out2, int hidden,
                            float eps1, float eps2) {
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int nvec = hidden / 4;
    const size_t base = (size_t)blockIdx.x * hidden;
    float4 v[NV];
    float s = 0.0f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        const int i = c * blockDim.x + threadIdx.x;
        v[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (i < nvec) {
            v[c] = *reinterpret_cast<const float4*>(y + base + 4 * i);
            if (in_bias) {
                const float4 b = *reinterpret_cast<const float4*>(in_bias + 4 * i);
                v[c].x += b.x; v[c].y += b.y; v[c].z += b.z; v[c].w += b.w;
            }
            s += (v[c].x + v[c].y) + (v[c].z + v[c].w);
        }
    }
    const float mean = block_sum(s, scratch) / (float)hidden;
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        if (c * blockDim.x + threadIdx.x < nvec) {
            const float dx = v[c].x - mean, dy = v[c].y - mean, dz = v[c].z - mean, dw = v[c].w - mean;
            ss += fmaf(dx, dx, dy * dy) + fmaf(dz, dz, dw * dw);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)hidden + eps1);
    float s2 = 0.0f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        const int i = c * blockDim.x + threadIdx.x;
        if (i < nvec) {
            const float4 g = *reinterpret_cast<const float4*>(g1 + 4 * i);
            const float4 b = b1 ? *reinterpret_cast<const float4*>(b1 + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            float4 r = *reinterpret_cast<const float4*>(x + base + 4 * i);
            r.x += (v[c].x - mean) * inv * g.x + b.x;
            r.y += (v[c].y - mean) * inv * g.y + b.y;
            r.z += (v[c].z - mean) * inv * g.z + b.z;
            r.w += (v[c].w - mean) * inv * g.w + b.w;
            *reinterpret_cast<float4*>(x + base + 4 * i) = r;
            if (emit) store4(emit, base + 4 * i, r);
            v[c] = r;
            s2 += (r.x + r.y) + (r.z + r.w);
        }
    }
    if (g2 == nullptr) return;
    const float mean2 = block_sum(s2, scratch) / (float)hidden;
    float ss2 = 0.0f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        if (c * blockDim.x + threadIdx.x < nvec) {
            const float dx = v[c].x - mean2, dy = v[c].y - mean2, dz = v[c].z - mean2, dw = v[c].w - mean2;
            ss2 += fmaf(dx, dx, dy * dy) + fmaf(dz, dz, dw * dw);
        }
    }
    const float inv2 = 1.0f / sqrtf(block_sum(ss2, scratch) / (float)hidden + eps2);
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        const int i = c * blockDim.x + threadIdx.x;
        if (i < nvec) {
            const float4 g = *reinterpret_cast<const float4*>(g2 + 4 * i);
            const float4 b = b2 ? *reinterpret_cast<const float4*>(b2 + 4 * i) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            store4(out2, base + 4 * i, make_float4((v[c].x - mean2) * inv2 * g.x + b.x, (v[c].y - mean2) * inv2 * g.y + b.y,
                                                   (v[c].z - mean2) * inv2 * g.z + b.z, (v[c].w - mean2) * inv2 * g.w + b.w));
        }
    }
}

static int grid_for(size_t n) {
    const size_t blocks = (n + 255) / 256;
    return (int)(blocks < 8192 ? (blocks ? blocks : 1) : 8192);
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_layer_norm_add(const float* y, const void* gain, int gain_dtype, float* x, void* emit, int emit_dtype,
                                      int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (hidden <= 0 || smem > 200 * 1024) {
        set_last_error("layer_norm_add: rows of %d elements do not fit a block's shared memory", hidden);
        return kTooLarge;
    }
    if (vec_ok(hidden, y, gain, x, emit)) {
        return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
            return CITLALI_DISPATCH_FLOAT(emit_dtype, TE, [&] {
                launch_kernel(layer_norm_vec_kernel<TG, TE, true>, rows, vec_threads(rows, hidden), 0, stream, y, (const TG*)gain,
                              (const TG*)nullptr, (const int32_t*)nullptr, x, (TE*)emit, hidden, eps);
                return CITLALI_LAUNCH_CHECK();
            });
        });
    }
    return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
        return CITLALI_DISPATCH_FLOAT(emit_dtype, TE, [&] {
            auto kernel = layer_norm_add_kernel<TG, TE>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            launch_kernel(kernel, rows, 256, smem, stream, y, (const TG*)gain, x, (TE*)emit, hidden, eps);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_layer_norm_rows(const float* x, const void* gain, const void* bias, int gain_dtype, const int32_t* row_index,
                                       void* out, int out_dtype, int rows, int hidden, float eps, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (hidden <= 0 || smem > 200 * 1024) {
        set_last_error("layer_norm_rows: rows of %d elements do not fit a block's shared memory", hidden);
        return kTooLarge;
    }
    if (vec_ok(hidden, x, gain, out, bias)) {
        return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
            return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
                launch_kernel(layer_norm_vec_kernel<TG, TO, false>, rows, vec_threads(rows, hidden), 0, stream, x, (const TG*)gain,
                              (const TG*)bias, row_index, (float*)nullptr, (TO*)out, hidden, eps);
                return CITLALI_LAUNCH_CHECK();
            });
        });
    }
    return CITLALI_DISPATCH_FLOAT(gain_dtype, TG, [&] {
        return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
            auto kernel = layer_norm_rows_kernel<TG, TO>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) return (int)e;
            }
            launch_kernel(kernel, rows, 256, smem, stream, x, (const TG*)gain, (const TG*)bias, row_index, (TO*)out, hidden, eps);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_cast_rows(const float* x, void* out, int out_dtype, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    return CITLALI_DISPATCH_FLOAT(out_dtype, TO, [&] {
        launch_kernel(cast_rows_kernel<TO>, grid_for(n), 256, 0, stream, x, (TO*)out, n);
        return CITLALI_LAUNCH_CHECK();
    });
}

extern "C" int citlali_scaled_sum(float a, const float* l, float b, const float* r, float* out, size_t n, cudaStream_t stream) {
    if (n == 0) return 0;
    launch_kernel(scaled_sum_kernel, grid_for(n), 256, 0, stream, a, l, b, r, out, n);
    return CITLALI_LAUNCH_CHECK();
}

extern "C" int citlali_layer_norm_chain(const float* y, const float* in_bias, const float* g1, const float* b1, float* x,
                                        void* emit, const float* g2, const float* b2, void* out2, int out_dtype, int rows,
                                        int hidden, float eps1, float eps2, cudaStream_t stream) {
    if (rows <= 0) return 0;
    const size_t smem = (size_t)hidden * sizeof(float);
    if (hidden <= 0 || smem > 200 * 1024 || g1 == nullptr || (g2 != nullptr && out2 == nullptr)) {
        set_last_error("layer_norm_chain: rows of %d elements; the first gain and, with a second norm, its output are needed", hidden);
        return kBadShape;
    }
    int threads = ((hidden / 4 + 31) / 32) * 32;             // follows the row's length alone: one order of sums a row
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
    const uintptr_t together = (uintptr_t)y | (uintptr_t)in_bias | (uintptr_t)g1 | (uintptr_t)b1 | (uintptr_t)x | (uintptr_t)emit |
                               (uintptr_t)g2 | (uintptr_t)b2 | (uintptr_t)out2;
    if (hidden % 4 == 0 && hidden <= 4 * 4096 && (together & 15u) == 0) {
        const int nv = (hidden / 4 + threads - 1) / threads;             // 1, 2, 3 or 4 runs of four elements a thread
        return CITLALI_DISPATCH_FLOAT(out_dtype, TE, [&] {
            if (nv <= 1) launch_kernel(layer_norm_chain_vec_kernel<TE, 1>, rows, threads, 0, stream, y, in_bias, g1, b1, x, (TE*)emit, g2, b2, (TE*)out2, hidden, eps1, eps2);
            else if (nv <= 2) launch_kernel(layer_norm_chain_vec_kernel<TE, 2>, rows, threads, 0, stream, y, in_bias, g1, b1, x, (TE*)emit, g2, b2, (TE*)out2, hidden, eps1, eps2);
            else launch_kernel(layer_norm_chain_vec_kernel<TE, 4>, rows, threads, 0, stream, y, in_bias, g1, b1, x, (TE*)emit, g2, b2, (TE*)out2, hidden, eps1, eps2);
            return CITLALI_LAUNCH_CHECK();
        });
    }
    return CITLALI_DISPATCH_FLOAT(out_dtype, TE, [&] {
        auto kernel = layer_norm_chain_kernel<TE>;
        if (smem > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return (int)e;
        }
        launch_kernel(kernel, rows, threads, smem, stream, y, in_bias, g1, b1, x, (TE*)emit, g2, b2, (TE*)out2, hidden, eps1, eps2);
        return CITLALI_LAUNCH_CHECK();
    });
}
