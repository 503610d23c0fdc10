// Attention whose weights are sigmoids of scores that the heads share among themselves, with a distance bias, a query
// temperature and a gate on every head's output.
//
//   biased_heads_prepare  proj [rows, C] float32 = q (H D) | k (G D) | v (G V) | gate (H), any of the last three absent,
//                         plus a bias a column.  q is multiplied by the row's temperature
//                         1 + coef ln(floor((pos + 1) / every) + 1) and goes to a buffer, k and v go to the row's place
//                         in the paged cache, the gate's sigmoid to a float32 buffer.
//   sigmoid_attention     one block a row (or a row and a run of keys), all heads together, since every head's weight
//                         needs every head's score.  For key j visible from position i (0 <= i - j < window; window 0:
//                         every earlier key):
//                             s_g = (q_g . k_{g / (H/G)}) scale - slope_g (i - j),   slope_g = 2^(-slope_exp (g + 1) / H)
//                             m_h = sum_g talk[h, g] s_g + head_bias[h]
//                             out_h += sigmoid(m_h) v_{h / (H/G)}
//                         and at the end out_h *= gate[row, h].  Nothing is normalised over the keys.  Scores, the mix,
//                         the sigmoid and the sums are float32.  A row's visible keys are cut into runs of kRunKeys
//                         counted from the window's first key; a run is summed key by key in ascending order and the
//                         runs are added in ascending order, whether one block walks them all or each has a block of its
//                         own (then a second kernel adds their partial sums): a row's result depends on its position and
//                         the window alone, not on the step it came in.
#include "api.h"
#include "common.cuh"

namespace citlali {

constexpr int kTileKeys = 32;          // keys whose scores wait in shared memory at a time
constexpr int kRunKeys = 32;           // keys of a run (a multiple of kTileKeys)
constexpr int kSigThreads = 256;

// Eight consecutive elements as floats, by 16-byte loads (the address is a multiple of eight elements).
__device__ __forceinline__ void load8(const float* p, float (&x)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&x)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[2 * i] = __uint_as_float(w[i] << 16);
        x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename T, typename TQ>
__global__ void __launch_bounds__(256)
biased_heads_prepare_kernel(const float* __restrict__ proj, const float* __restrict__ bias, const int32_t* __restrict__ row_slot,
                            const int32_t* __restrict__ row_pos, const int32_t* __restrict__ page_table, int table_stride,
                            T* __restrict__ k_pool, T* __restrict__ v_pool, int page_size, TQ* __restrict__ q_out,
                            float* __restrict__ gate_out, int rows, int H, int G, int D, int V, int has_kv, int has_gate,
                            float temp_coef, int temp_every) {
    dependents_may_launch();
    wait_for_predecessor();
    const int nq = H * D, nk = has_kv ? G * D : 0, nv = has_kv ? G * V : 0;
    const int C = nq + nk + nv + (has_gate ? H : 0);
    const size_t total = (size_t)rows * C;
    for (size_t at = (size_t)blockIdx.x * blockDim.x + threadIdx.x; at < total; at += (size_t)gridDim.x * blockDim.x) {
        const int row = (int)(at / C), c = (int)(at % C);
        float x = proj[at];
        if (bias) x += bias[c];
        const int pos = row_pos[row];
        if (c < nq) {
            if (temp_every > 0) x *= 1.0f + temp_coef * logf((float)((pos + 1) / temp_every + 1));
            stf(q_out, (size_t)row * nq + c, x);
        } else if (c < nq + nk + nv) {
            const bool is_v = c >= nq + nk;
            const int cc = is_v ? c - nq - nk : c - nq;
            const int n = is_v ? V : D;
            const int head = cc / n, i = cc % n;
            const int page = page_table[(size_t)row_slot[row] * table_stride + pos / page_size];
            const size_t to = (((size_t)page * G + head) * page_size + pos % page_size) * (size_t)n + i;
            if (is_v) stf(v_pool, to, x); else stf(k_pool, to, x);
        } else {
            gate_out[(size_t)row * H + (c - nq - nk - nv)] = 1.0f / (1.0f + expf(-x));
        }
    }
}

// PL: elements of a key a lane holds (D <= 32 PL).  ACC: outputs a thread owns (H V <= 256 ACC).  VEC (D and V multiples
// of eight): keys and values come in 16-byte pieces; eight lanes share a key's score (four keys a warp at a time) and a
// thread owns eight neighbouring outputs of one head.  Either way an output's keys are added in ascending order.
template <typename T, typename TQ, int PL, int ACC, bool VEC>
__global__ void __launch_bounds__(kSigThreads)
sigmoid_attention_kernel(const TQ* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ row_slot,
                         const int32_t* __restrict__ row_pos, const float* __restrict__ talk, const float* __restrict__ head_bias,
                         const float* __restrict__ gate, TQ* __restrict__ out, float* __restrict__ partial, int H, int G, int D,
                         int V, int page_size, int window, float scale, float slope_exp) {
    extern __shared__ __align__(16) float smem[];
    constexpr int NACC = VEC ? (ACC >= 8 ? ACC : 8) : ACC;
    float* qs = smem;                                  // [H, D]
    float* tk = qs + H * D;                            // [H (g), H (h)]: the mix, transposed
    float* hb = tk + H * H;                            // [H]
    float* sl = hb + H;                                // [H]
    float* raw = sl + H;                               // [kTileKeys, H]
    float* wts = raw + kTileKeys * H;                  // [kTileKeys, H]
    int* rowbase = reinterpret_cast<int*>(wts + kTileKeys * H);     // [kTileKeys]: page * G * page_size + place in the page
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int n = pos - lo + 1;
    const int runs = (n + kRunKeys - 1) / kRunKeys;
    const bool split = gridDim.y > 1;
    if (split && (int)blockIdx.y >= runs) return;
    const int HV = H * V, per = H / G;
    for (int i = tid; i < H * D; i += kSigThreads) qs[i] = ldf(q, (size_t)row * H * D + i);
    for (int i = tid; i < H * H; i += kSigThreads) tk[i] = talk ? talk[(i % H) * H + i / H] : ((i / H == i % H) ? 1.0f : 0.0f);
    for (int i = tid; i < H; i += kSigThreads) {
        hb[i] = head_bias ? head_bias[i] : 0.0f;
        sl[i] = slope_exp > 0.0f ? exp2f(-slope_exp * (float)(i + 1) / (float)H) : 0.0f;
    }
    __syncthreads();
    const int32_t* pages = page_table + (size_t)row_slot[row] * table_stride;
    float total[NACC];
#pragma unroll
    for (int a = 0; a < NACC; ++a) total[a] = 0.0f;
    const int run_first = split ? blockIdx.y : 0, run_last = split ? blockIdx.y + 1 : runs;
    for (int run = run_first; run < run_last; ++run) {
        float acc[NACC];
#pragma unroll
        for (int a = 0; a < NACC; ++a) acc[a] = 0.0f;
        const int k0 = lo + run * kRunKeys;
        const int k1 = min(k0 + kRunKeys, pos + 1);
        for (int t0 = k0; t0 < k1; t0 += kTileKeys) {
            const int tn = min(kTileKeys, k1 - t0);
            if constexpr (VEC) {
                // scores of the tile's keys: eight lanes a key, a lane the elements 8 l, 8 l + 64, ... of it
                constexpr int PL8 = PL / 2;
                const int jj = warp * 4 + (lane >> 3), l8 = lane & 7;
                const bool ok = jj < tn;
                const int key = t0 + jj;
                const int base = ok ? pages[key / page_size] * G * page_size + key % page_size : 0;
                if (ok && l8 == 0) rowbase[jj] = base;
                for (int g2 = 0; g2 < G; ++g2) {
                    const size_t at = ((size_t)base + (size_t)g2 * page_size) * (size_t)D;
                    float kr[PL8][8];
#pragma unroll
                    for (int c = 0; c < PL8; ++c) {
                        const int i = 8 * l8 + 64 * c;
                        if (ok && i < D) load8(k_pool + at + i, kr[c]);
                        else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) kr[c][e] = 0.0f;
                        }
                    }
                    for (int hh = 0; hh < per; ++hh) {
                        const int h = g2 * per + hh;
                        float s = 0.0f;
#pragma unroll
                        for (int c = 0; c < PL8; ++c) {
                            const int i = 8 * l8 + 64 * c;
                            if (i < D) {
                                const float4 qa = *reinterpret_cast<const float4*>(qs + h * D + i);
                                const float4 qb = *reinterpret_cast<const float4*>(qs + h * D + i + 4);
                                s = fmaf(qa.x, kr[c][0], s); s = fmaf(qa.y, kr[c][1], s); s = fmaf(qa.z, kr[c][2], s);
                                s = fmaf(qa.w, kr[c][3], s); s = fmaf(qb.x, kr[c][4], s); s = fmaf(qb.y, kr[c][5], s);
                                s = fmaf(qb.z, kr[c][6], s); s = fmaf(qb.w, kr[c][7], s);
                            }
                        }
                        s += __shfl_xor_sync(0xffffffffu, s, 1);
                        s += __shfl_xor_sync(0xffffffffu, s, 2);
                        s += __shfl_xor_sync(0xffffffffu, s, 4);
                        if (ok && l8 == 0) raw[jj * H + h] = s * scale - sl[h] * (float)(pos - key);
                    }
                }
            } else {
                // scores of the tile's keys: a warp a key, a lane the elements lane, lane + 32, ... of it
                for (int jj = warp; jj < tn; jj += kSigThreads / 32) {
                    const int key = t0 + jj;
                    const int base = pages[key / page_size] * G * page_size + key % page_size;
                    if (lane == 0) rowbase[jj] = base;
                    for (int g2 = 0; g2 < G; ++g2) {
                        const size_t at = ((size_t)base + (size_t)g2 * page_size) * (size_t)D;
                        float kr[PL];
#pragma unroll
                        for (int c = 0; c < PL; ++c) {
                            const int i = lane + 32 * c;
                            kr[c] = i < D ? ldf(k_pool, at + i) : 0.0f;
                        }
                        for (int hh = 0; hh < per; ++hh) {
                            const int h = g2 * per + hh;
                            float s = 0.0f;
#pragma unroll
                            for (int c = 0; c < PL; ++c) {
                                const int i = lane + 32 * c;
                                if (i < D) s = fmaf(qs[h * D + i], kr[c], s);
                            }
                            s = warp_sum(s);
                            if (lane == 0) raw[jj * H + h] = s * scale - sl[h] * (float)(pos - key);
                        }
                    }
                }
            }
            __syncthreads();
            // the heads' scores mixed, the head's bias, the sigmoid
            for (int i = tid; i < tn * H; i += kSigThreads) {
                const int jj = i / H, h = i % H;
                float m = 0.0f;
                for (int g = 0; g < H; ++g) m = fmaf(tk[g * H + h], raw[jj * H + g], m);
                m += hb[h];
                wts[i] = 1.0f / (1.0f + expf(-m));
            }
            __syncthreads();
            if constexpr (VEC) {
                // the weighted values: a thread owns outputs 8 o .. 8 o + 7 for o = tid, tid + 256, ...
                const int vchunks = V / 8, owners = H * vchunks;
#pragma unroll
                for (int a = 0; a < NACC / 8; ++a) {
                    const int o = tid + kSigThreads * a;
                    if (o < owners) {
                        const int h = o / vchunks, e = (o % vchunks) * 8;
                        const size_t col = (size_t)(h / per) * page_size;
#pragma unroll 8
                        for (int jj = 0; jj < tn; ++jj) {
                            float vv[8];
                            load8(v_pool + ((size_t)rowbase[jj] + col) * (size_t)V + e, vv);
                            const float w = wts[jj * H + h];
#pragma unroll
                            for (int x = 0; x < 8; ++x) acc[a * 8 + x] = fmaf(w, vv[x], acc[a * 8 + x]);
                        }
                    }
                }
            } else {
                // the weighted values: a thread owns outputs tid, tid + 256, ...
#pragma unroll
                for (int a = 0; a < ACC; ++a) {
                    const int o = tid + kSigThreads * a;
                    if (o < HV) {
                        const int h = o / V, e = o % V;
                        const size_t col = (size_t)(h / per) * page_size;
                        float s = acc[a];
#pragma unroll 4
                        for (int jj = 0; jj < tn; ++jj)
                            s = fmaf(wts[jj * H + h], ldf(v_pool, ((size_t)rowbase[jj] + col) * (size_t)V + e), s);
                        acc[a] = s;
                    }
                }
            }
            __syncthreads();
        }
#pragma unroll
        for (int a = 0; a < NACC; ++a) total[a] += acc[a];
    }
#pragma unroll
    for (int a = 0; a < NACC; ++a) {
        const int o = VEC ? (tid + kSigThreads * (a / 8)) * 8 + a % 8 : tid + kSigThreads * a;
        if (o < HV) {
            if (split) partial[((size_t)row * gridDim.y + blockIdx.y) * HV + o] = total[a];
            else stf(out, (size_t)row * HV + o, gate ? total[a] * gate[(size_t)row * H + o / V] : total[a]);
        }
    }
}

// The runs' partial sums added in run order, then the gate.
template <typename TQ>
__global__ void __launch_bounds__(256)
sigmoid_attention_merge_kernel(const float* __restrict__ partial, const int32_t* __restrict__ row_pos, const float* __restrict__ gate,
                               TQ* __restrict__ out, int H, int V, int window, int max_runs) {
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x, HV = H * V;
    const int pos = row_pos[row];
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int runs = (pos - lo + 1 + kRunKeys - 1) / kRunKeys;
    for (int o = blockIdx.y * blockDim.x + threadIdx.x; o < HV; o += gridDim.y * blockDim.x) {
        float total = 0.0f;
        for (int r = 0; r < runs; ++r) total += partial[((size_t)row * max_runs + r) * HV + o];
        stf(out, (size_t)row * HV + o, gate ? total * gate[(size_t)row * H + o / V] : total);
    }
}

template <typename T, typename TQ, int PL, int ACC, bool VEC>
static int launch_sigmoid(const void* q, const void* k_pool, const void* v_pool, const int32_t* page_table, int table_stride,
                          const int32_t* row_slot, const int32_t* row_pos, const float* talk, const float* head_bias,
                          const float* gate, void* out, float* partial, int rows, int runs, int H, int G, int D, int V,
                          int page_size, int window, float scale, float slope_exp, cudaStream_t stream) {
    const size_t smem = (size_t)(H * D + H * H + 2 * H + 2 * kTileKeys * H) * sizeof(float) + kTileKeys * sizeof(int);
    auto kernel = sigmoid_attention_kernel<T, TQ, PL, ACC, VEC>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    launch_kernel(kernel, dim3(rows, runs), kSigThreads, smem, stream, (const TQ*)q, (const T*)k_pool, (const T*)v_pool,
                  page_table, table_stride, row_slot, row_pos, talk, head_bias, gate, (TQ*)out, partial, H, G, D, V, page_size,
                  window, scale, slope_exp);
    return CITLALI_LAUNCH_CHECK();
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_biased_heads_prepare(const float* proj, const float* bias, const int32_t* row_slot, const int32_t* row_pos,
                                            const int32_t* page_table, int table_stride, void* k_pool, void* v_pool,
                                            int cache_dtype, int page_size, void* q_out, int q_dtype, float* gate_out, int rows,
                                            int H, int G, int D, int V, int has_kv, int has_gate, float temp_coef,
                                            int temp_every, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || G <= 0 || D <= 0 || V <= 0 || page_size <= 0 || (has_gate && gate_out == nullptr) ||
        (has_kv && (k_pool == nullptr || v_pool == nullptr))) {
        set_last_error("biased_heads_prepare: %d and %d heads of %d (values %d), pages of %d; a gate and keys need their buffers",
                       H, G, D, V, page_size);
        return kBadShape;
    }
    const size_t total = (size_t)rows * (H * D + (has_kv ? G * (D + V) : 0) + (has_gate ? H : 0));
    const size_t blocks = (total + 255) / 256;
    const int grid = (int)(blocks < 16384 ? blocks : 16384);
    return CITLALI_DISPATCH_FLOAT(cache_dtype, T, [&] {
        return CITLALI_DISPATCH_FLOAT(q_dtype, TQ, [&] {
            launch_kernel(biased_heads_prepare_kernel<T, TQ>, grid, 256, 0, stream, proj, bias, row_slot, row_pos, page_table,
                          table_stride, (T*)k_pool, (T*)v_pool, page_size, (TQ*)q_out, gate_out, rows, H, G, D, V, has_kv,
                          has_gate, temp_coef, temp_every);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_sigmoid_attention_run_keys(void) { return kRunKeys; }

// `runs` 1: one block a row walks all its keys; more: a block a (row, run of kRunKeys keys) into `partial`
// [rows, runs, H V] float32, which a second kernel adds up (runs must cover the longest row: runs * kRunKeys >= its keys).
extern "C" int citlali_sigmoid_attention(const void* q, int q_dtype, const void* k_pool, const void* v_pool, int cache_dtype,
                                         const int32_t* page_table, int table_stride, const int32_t* row_slot,
                                         const int32_t* row_pos, const float* talk, const float* head_bias, const float* gate,
                                         void* out, float* partial, int runs, int rows, int H, int G, int D, int V,
                                         int page_size, int window, float scale, float slope_exp, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || V <= 0 || window < 0 || page_size <= 0 || runs < 1 || runs > 65535 ||
        (runs > 1 && partial == nullptr)) {
        set_last_error("sigmoid_attention: %d query heads over %d key/value heads of %d (values %d), window %d, %d runs", H, G,
                       D, V, window, runs);
        return kBadShape;
    }
    if (D > 256 || H * V > 256 * 32) {
        set_last_error("sigmoid_attention: heads of %d exceed 256, or %d heads of %d values exceed %d outputs a row", D, H, V,
                       256 * 32);
        return kTooLarge;
    }
    const size_t smem = (size_t)(H * D + H * H + 2 * H + 2 * kTileKeys * H) * sizeof(float) + kTileKeys * sizeof(int);
    if (smem > 200 * 1024) {
        set_last_error("sigmoid_attention: %d heads of %d need %zu bytes of shared memory", H, D, smem);
        return kTooLarge;
    }
    const int HV = H * V;
    const bool vec = D % 8 == 0 && V % 8 == 0 && ((uintptr_t)k_pool & 15u) == 0 && ((uintptr_t)v_pool & 15u) == 0;
#define CITLALI_SIG(T, TQ, PL, VEC)                                                                                            \
    do {                                                                                                                    \
        if (HV <= 256 * 2) return launch_sigmoid<T, TQ, PL, 2, VEC>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, talk, head_bias, gate, out, partial, rows, runs, H, G, D, V, page_size, window, scale, slope_exp, stream); \
        if (HV <= 256 * 8) return launch_sigmoid<T, TQ, PL, 8, VEC>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, talk, head_bias, gate, out, partial, rows, runs, H, G, D, V, page_size, window, scale, slope_exp, stream); \
        return launch_sigmoid<T, TQ, PL, 32, VEC>(q, k_pool, v_pool, page_table, table_stride, row_slot, row_pos, talk, head_bias, gate, out, partial, rows, runs, H, G, D, V, page_size, window, scale, slope_exp, stream); \
    } while (0)
    if (q_dtype != cache_dtype) {
        set_last_error("sigmoid_attention: queries and the cache must have one type");
        return kBadShape;
    }
    int rc = CITLALI_DISPATCH_FLOAT(cache_dtype, T, [&] {
        return [&]() -> int {
            using TQ = T;
            if (vec) {
                if (D <= 64) CITLALI_SIG(T, TQ, 2, true);
                if (D <= 128) CITLALI_SIG(T, TQ, 4, true);
                CITLALI_SIG(T, TQ, 8, true);
            }
            if (D <= 64) CITLALI_SIG(T, TQ, 2, false);
            if (D <= 128) CITLALI_SIG(T, TQ, 4, false);
            CITLALI_SIG(T, TQ, 8, false);
        }();
    });
#undef CITLALI_SIG
    if (rc != 0 || runs == 1) return rc;
    return CITLALI_DISPATCH_FLOAT(q_dtype, TQ, [&] {
        const int by = (HV + 255) / 256;
        launch_kernel(sigmoid_attention_merge_kernel<TQ>, dim3(rows, by), 256, 0, stream, (const float*)partial, row_pos, gate,
                      (TQ*)out, H, V, window, runs);
        return CITLALI_LAUNCH_CHECK();
    });
}
