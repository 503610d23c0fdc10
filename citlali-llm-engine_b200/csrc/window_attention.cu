// Attention over a sliding window that also keeps a sequence's first tokens, for heads whose keys and values may differ
// in size, with a short causal convolution in front of q, k and v.
//
//   conv_heads_prepare   one warp a (row, head): the convolution over time of the head's channels (earlier tokens from the
//                        step's rows or from the sequence's kept inputs), for q and k heads an RMS norm with a weight
//                        shared by the heads and the rotation of the first rot_dims elements in neighbouring pairs
//                        (2i, 2i+1) by position * inv_freq[i]; q goes to a buffer, k and v to the row's place in the
//                        paged cache.  All float32 until the one rounding at the store.  An optional bias a channel is
//                        added to what the convolution gives (with one tap: to the projection itself).
//   attention_window     one block a (row, query head): keys j <= pos with pos - j < window or j < keep_first (window 0:
//                        every key); scores, softmax and the weighted sum in float32; with a soft cap c the scaled score s
//                        becomes c tanh(s / c) before the softmax; with a gate the head's output element i is multiplied
//                        by sigmoid(gate[row, head vd + i]).  The keys are dealt to 32 groups of
//                        eight lanes by their place among the visible keys, each group keeps a running softmax of its own,
//                        and the groups are merged in one fixed order: a row's result does not depend on the step it came
//                        in, and no score is ever stored, so the number of keys has no limit.
#include "api.h"
#include "common.cuh"

namespace citlali {

constexpr int kHeadWarps = 8;
constexpr int kMaxPerLane = 8;         // head sizes up to 256

template <typename T, typename TQ>
__global__ void __launch_bounds__(kHeadWarps * 32)
conv_heads_prepare_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ taps_w, int taps,
                          const float* __restrict__ state, size_t state_stride, size_t conv_off,
                          const float* __restrict__ q_gain, const float* __restrict__ k_gain, const float* __restrict__ inv_freq,
                          int rot_dims, const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                          const int32_t* __restrict__ page_table, int table_stride, T* __restrict__ k_pool, T* __restrict__ v_pool,
                          int page_size, TQ* __restrict__ q_out, int nq, int nkv, int d, int vd, float eps, int write_cache,
                          const float* __restrict__ bias) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, lane = threadIdx.x & 31;
    const int head = blockIdx.y * kHeadWarps + (threadIdx.x >> 5);
    if (head >= nq + 2 * nkv) return;
    const bool is_q = head < nq, is_v = head >= nq + nkv;
    if (!is_q && !write_cache) return;
    const int C = (nq + nkv) * d + nkv * vd;
    const int n = is_v ? vd : d;
    const int c0 = is_v ? (nq + nkv) * d + (head - nq - nkv) * vd : head * d;
    const int slot = row_slot[row], pos = row_pos[row];
    int in_step = 0;
    while (in_step < taps - 1 && row - in_step - 1 >= 0 && row_slot[row - in_step - 1] == slot) ++in_step;
    const float* kept = state ? state + (size_t)slot * state_stride + conv_off : nullptr;
    float x[kMaxPerLane];
    float ss = 0.0f;
    // a lane holds the neighbouring elements 2 lane, 2 lane + 1 (+ 64 j): a rotation pair stays in one lane
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const int i = (j >> 1) * 64 + 2 * lane + (j & 1);
        float acc = 0.0f;
        if (i < n) {
            const int c = c0 + i;
            for (int back = taps - 1; back >= 0; --back) {
                float u;
                if (back <= in_step) u = proj[(size_t)(row - back) * proj_stride + c];
                else u = kept[(size_t)(taps - 1 - back + in_step) * C + c];
                acc = fmaf(taps_w[(size_t)c * taps + (taps - 1 - back)], u, acc);
            }
            if (bias) acc += bias[c];
        }
        x[j] = acc;
        ss = fmaf(acc, acc, ss);
    }
    size_t cache_at = 0;
    if (!is_q) {
        const int page = page_table[(size_t)slot * table_stride + pos / page_size];
        const int kvh = is_v ? head - nq - nkv : head - nq;
        cache_at = (((size_t)page * nkv + kvh) * page_size + pos % page_size) * (size_t)n;
    }
    if (is_v) {
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
            const int i = (j >> 1) * 64 + 2 * lane + (j & 1);
            if (i < n) stf(v_pool, cache_at + i, x[j]);
        }
        return;
    }
    const float* gain = is_q ? q_gain : k_gain;
    if (gain) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)d + eps);
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
            const int i = (j >> 1) * 64 + 2 * lane + (j & 1);
            if (i < n) x[j] = x[j] * inv * gain[i];
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; j += 2) {
        const int i = (j >> 1) * 64 + 2 * lane;
        if (i < rot_dims) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i >> 1], &sn, &cs);
            const float a = x[j], b = x[j + 1];
            x[j] = a * cs - b * sn;
            x[j + 1] = b * cs + a * sn;
        }
    }
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
        const int i = (j >> 1) * 64 + 2 * lane + (j & 1);
        if (i < n) {
            if (is_q) stf(q_out, (size_t)row * nq * d + (size_t)head * d + i, x[j]);
            else stf(k_pool, cache_at + i, x[j]);
        }
    }
}

// Eight lanes share a key: lane part p of them holds the key's (and the value's) elements p, p + 8, ... (or, for bfloat16
// heads that are multiples of 8, the 16-byte pieces p, p + 8, ...).  A warp takes four keys at a time, a block's eight warps
// the keys t = 4 warp + 32 i ...; every group of eight lanes keeps a running maximum, sum and weighted value sum of its own
// keys (online softmax), and the 32 groups of the block are merged once at the end in group order.  Which keys a group gets
// depends on the row's position, the window and the kept tokens alone.
constexpr int kWinWarps = 8;

// PL: elements of a head a lane holds (heads up to 8 PL).  VEC: bfloat16 pools and head sizes that are multiples of 8; a lane
// then holds the 16-byte pieces part, part + 8, ..., and the keys of two or four turns are fetched before any of them is used
// (a group of lanes is alone with the latency of its loads; two blocks share an SM for heads up to 128).
template <int PL>
__device__ __forceinline__ int slice_element(int c, int part, bool vec) { return vec ? (part + 8 * (c >> 3)) * 8 + (c & 7) : part + 8 * c; }

template <int PL>
__device__ __forceinline__ void unpack_pieces(const uint4 (&raw)[PL / 8 > 0 ? PL / 8 : 1], float (&x)[PL]) {
#pragma unroll
    for (int c = 0; c < PL / 8; ++c) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[c]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            x[c * 8 + 2 * e] = f.x;
            x[c * 8 + 2 * e + 1] = f.y;
        }
    }
}

template <typename T, typename TQ, int PL, bool VEC>
__global__ void __launch_bounds__(kWinWarps * 32, PL <= 16 ? 2 : 1)
attention_window_kernel(const TQ* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                        const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ row_slot,
                        const int32_t* __restrict__ row_pos, TQ* __restrict__ out, int nq, int nkv, int d, int vd,
                        int page_size, int window, int keep_first, float scale, float softcap, const float* __restrict__ gate,
                        size_t gate_stride) {
    extern __shared__ float smem[];                            // [32 groups][vd] weighted sums, then [32] maxima, [32] sums
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, head = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int part = lane & 7, group = warp * 4 + (lane >> 3);
    const int g = head / (nq / nkv);
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int first = min(keep_first, lo);                     // kept keys 0..first-1, then the window lo..pos
    const int n = first + pos - lo + 1;
    const int32_t* pages = page_table + (size_t)row_slot[row] * table_stride;
    float qs[PL], acc[PL];
#pragma unroll
    for (int c = 0; c < PL; ++c) {
        const int i = slice_element<PL>(c, part, VEC);
        qs[c] = i < d ? ldf(q + (size_t)row * nq * d + (size_t)head * d, i) * scale : 0.0f;
        acc[c] = 0.0f;
    }
    float m = -INFINITY, l = 0.0f;
    const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;
    auto take = [&](float s, const float (&v)[PL]) {           // one key's score and value into the group's running softmax
        if (softcap > 0.0f) s = softcap * tanhf(s * inv_cap);
        if (s > m) {                                           // the maximum grows: what the group has is scaled down
            const float f = expf(m - s);                       // (zero the first time)
            l *= f;
#pragma unroll
            for (int c = 0; c < PL; ++c) acc[c] *= f;
            m = s;
        }
        const float p = expf(s - m);
        l += p;
#pragma unroll
        for (int c = 0; c < PL; ++c) acc[c] = fmaf(p, v[c], acc[c]);
    };
    auto place = [&](int t) -> size_t {                        // where the t-th visible key lies in the pools (in rows)
        const int key = t < first ? t : lo + (t - first);
        return ((size_t)pages[key / page_size] * nkv + g) * page_size + key % page_size;
    };
    constexpr int STEP = kWinWarps * 4;                        // keys the block takes a turn
    if constexpr (VEC) {
        constexpr int U = PL <= 8 ? 4 : 2, W = PL / 8;       // keys in flight a group: as many as two blocks' registers allow
        for (int base = warp * 4; base < n; base += STEP * U) {        // the same trips for all lanes of a warp
            uint4 kr[U][W], vr[U][W];
            bool on[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = base + u * STEP + (lane >> 3);
                on[u] = t < n;
                const size_t at = on[u] ? place(t) : 0;
#pragma unroll
                for (int c = 0; c < W; ++c) {
                    const int piece = part + 8 * c;
                    kr[u][c] = (on[u] && piece * 8 < d) ? *reinterpret_cast<const uint4*>(k_pool + at * d + piece * 8) : make_uint4(0, 0, 0, 0);
                    vr[u][c] = (on[u] && piece * 8 < vd) ? *reinterpret_cast<const uint4*>(v_pool + at * vd + piece * 8) : make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (base + u * STEP >= n) break;               // (warp-uniform) no lane of the warp has a key in this turn
                float x[PL];
                unpack_pieces<PL>(kr[u], x);
                float s = 0.0f;
#pragma unroll
                for (int c = 0; c < PL; ++c) s = fmaf(qs[c], x[c], s);
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                if (on[u]) {
                    unpack_pieces<PL>(vr[u], x);
                    take(s, x);
                }
            }
        }
    } else {
        for (int base = warp * 4; base < n; base += STEP) {
            const int t = base + (lane >> 3);
            const bool on = t < n;
            const size_t at = on ? place(t) : 0;
            float x[PL];
            float s = 0.0f;
#pragma unroll
            for (int c = 0; c < PL; ++c) {
                const int i = part + 8 * c;
                x[c] = (on && i < d) ? ldf(k_pool, at * d + i) : 0.0f;
                s = fmaf(qs[c], x[c], s);
            }
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (on) {
#pragma unroll
                for (int c = 0; c < PL; ++c) {
                    const int i = part + 8 * c;
                    x[c] = i < vd ? ldf(v_pool, at * vd + i) : 0.0f;
                }
                take(s, x);
            }
        }
    }
    // the block's 32 groups, merged in group order
    float* sums = smem;
    float* gm = smem + 32 * vd;
    float* gl = gm + 32;
#pragma unroll
    for (int c = 0; c < PL; ++c) {
        const int i = slice_element<PL>(c, part, VEC);
        if (i < vd) sums[group * vd + i] = acc[c];
    }
    if (part == 0) { gm[group] = m; gl[group] = l; }
    __syncthreads();
    float top = -INFINITY;
    for (int j = 0; j < 32; ++j) top = fmaxf(top, gm[j]);
    for (int i = threadIdx.x; i < vd; i += blockDim.x) {
        float z = 0.0f, a = 0.0f;
        for (int j = 0; j < 32; ++j) {
            if (gm[j] == -INFINITY) continue;                  // a group without keys
            const float f = expf(gm[j] - top);
            z = fmaf(f, gl[j], z);
            a = fmaf(f, sums[j * vd + i], a);
        }
        float r = a / z;
        if (gate) r *= 1.0f / (1.0f + expf(-gate[(size_t)row * gate_stride + (size_t)head * vd + i]));
        stf(out, (size_t)row * nq * vd + (size_t)head * vd + i, r);
    }
}

template <typename T, typename TQ, int PL, bool VEC>
static int launch_window(const void* q, const void* k_pool, const void* v_pool, const int32_t* page_table, int table_stride,
                         const int32_t* row_slot, const int32_t* row_pos, void* out, int rows, int nq, int nkv, int d, int vd,
                         int page_size, int window, int keep_first, float scale, float softcap, const float* gate,
                         size_t gate_stride, cudaStream_t stream) {
    const size_t smem = (size_t)(32 * vd + 64) * sizeof(float);
    dim3 grid(rows, nq);
    launch_kernel(attention_window_kernel<T, TQ, PL, VEC>, grid, kWinWarps * 32, smem, stream, (const TQ*)q, (const T*)k_pool,
                  (const T*)v_pool, page_table, table_stride, row_slot, row_pos, (TQ*)out, nq, nkv, d, vd, page_size, window,
                  keep_first, scale, softcap, gate, gate_stride);
    return CITLALI_LAUNCH_CHECK();
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_conv_heads_prepare(const float* proj, int proj_stride, const float* taps_w, int taps, float* state,
                                          size_t state_stride, size_t conv_off, const float* q_gain, const float* k_gain,
                                          const float* inv_freq, int rot_dims, const int32_t* row_slot, const int32_t* row_pos,
                                          const int32_t* page_table, int table_stride, void* k_pool, void* v_pool,
                                          int cache_dtype, int page_size, void* q_out, int q_dtype, int rows, int nq, int nkv,
                                          int d, int vd, float eps, int write_cache, const float* bias,
                                          cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || d <= 0 || vd <= 0 || d > 32 * kMaxPerLane || vd > 32 * kMaxPerLane || taps < 1 || page_size <= 0) {
        set_last_error("conv_heads_prepare: %d and %d heads of %d (values %d, at most %d), %d taps", nq, nkv, d, vd,
                       32 * kMaxPerLane, taps);
        return kBadShape;
    }
    if (rot_dims < 0 || rot_dims % 2 != 0 || rot_dims > d || (taps > 1 && state == nullptr)) {
        set_last_error("conv_heads_prepare: %d rotated elements must be even and at most the head size %d; taps need a state",
                       rot_dims, d);
        return kBadShape;
    }
    const int heads = nq + 2 * nkv;
    dim3 grid(rows, (heads + kHeadWarps - 1) / kHeadWarps);
    return CITLALI_DISPATCH_FLOAT(cache_dtype, T, [&] {
        return CITLALI_DISPATCH_FLOAT(q_dtype, TQ, [&] {
            launch_kernel(conv_heads_prepare_kernel<T, TQ>, grid, kHeadWarps * 32, 0, stream, proj, proj_stride, taps_w, taps,
                          (const float*)state, state_stride, conv_off, q_gain, k_gain, inv_freq, rot_dims, row_slot, row_pos,
                          page_table, table_stride, (T*)k_pool, (T*)v_pool, page_size, (TQ*)q_out, nq, nkv, d, vd, eps,
                          write_cache, bias);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_attention_window(const void* q, int q_dtype, const void* k_pool, const void* v_pool, int cache_dtype,
                                        const int32_t* page_table, int table_stride, const int32_t* row_slot,
                                        const int32_t* row_pos, void* out, int rows, int nq, int nkv, int d, int vd,
                                        int page_size, int window, int keep_first, int max_keys, float scale,
                                        float softcap, const float* gate, size_t gate_stride, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (nq <= 0 || nkv <= 0 || nq % nkv != 0 || d <= 0 || vd <= 0 || nq > 65535 || window < 0 || keep_first < 0) {
        set_last_error("attention_window: %d query heads over %d key/value heads of %d (values %d), window %d, %d kept", nq, nkv,
                       d, vd, window, keep_first);
        return kBadShape;
    }
    (void)max_keys;
    const int big = d > vd ? d : vd;
    if (big > 256) {
        set_last_error("attention_window: heads of %d (values %d) exceed 256", d, vd);
        return kTooLarge;
    }
    // 16-byte pieces for bfloat16 pools and heads that are multiples of 8 (rows of the pools then start on 16-byte boundaries)
    const bool vec = cache_dtype == kBF16 && d % 8 == 0 && vd % 8 == 0 && ((uintptr_t)k_pool & 15u) == 0 && ((uintptr_t)v_pool & 15u) == 0;
#define CITLALI_WINDOW(T, TQ)                                                                                             \
    do {                                                                                                                  \
        if (vec) {                                                                                                        \
            if constexpr (sizeof(T) == 2) {                                                                               \
                if (big <= 64) return launch_window<T, TQ, 8, true>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, out, rows, nq, nkv, d, vd, page_size, window, keep_first, scale, softcap, gate, gate_stride, stream); \
                if (big <= 128) return launch_window<T, TQ, 16, true>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, out, rows, nq, nkv, d, vd, page_size, window, keep_first, scale, softcap, gate, gate_stride, stream); \
                return launch_window<T, TQ, 32, true>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, out, rows, nq, nkv, d, vd, page_size, window, keep_first, scale, softcap, gate, gate_stride, stream); \
            }                                                                                                             \
        }                                                                                                                 \
        if (big <= 64) return launch_window<T, TQ, 8, false>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, out, rows, nq, nkv, d, vd, page_size, window, keep_first, scale, softcap, gate, gate_stride, stream); \
        if (big <= 128) return launch_window<T, TQ, 16, false>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, out, rows, nq, nkv, d, vd, page_size, window, keep_first, scale, softcap, gate, gate_stride, stream); \
        return launch_window<T, TQ, 32, false>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, out, rows, nq, nkv, d, vd, page_size, window, keep_first, scale, softcap, gate, gate_stride, stream); \
    } while (0)
    return CITLALI_DISPATCH_FLOAT(cache_dtype, T, [&] {
        return CITLALI_DISPATCH_FLOAT(q_dtype, TQ, [&]() -> int { CITLALI_WINDOW(T, TQ); });
    });
#undef CITLALI_WINDOW
}
