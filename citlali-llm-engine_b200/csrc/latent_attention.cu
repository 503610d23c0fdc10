// Attention through a shared latent: per token the cache holds one vector [c | r], the normed latent c (R numbers)
// and one rotated key part r (P numbers) that all heads share.  A head's key is [W_uk c | r] and its value W_uv c, so
//   score = q_plain . (W_uk c) + q_rot . r = (W_uk^T q_plain) . c + q_rot . r,
//   out   = W_uv (sum_j p_j c_j):
// the heads' matrices are applied to the query before and to the weighted latent after the walk over the cache, and
// the walk itself reads R + P numbers a token whatever the number of heads.
//
//   latent_prepare     one block a row: RMS norm of the query latent and of c (plain weights), rotation of r by the
//                      row's position (angle = float(position) * inv_freq[i]; element pairs (2i, 2i+1), or with
//                      rot_halves (i, i + rot_dims / 2)), cache write.
//   heads_product      y[row, h, :] = x[row, h, :] . M_h for a matrix per head given by strides (W_uk as stored, or
//                      W_uv transposed); optional extras: a tail of the row rotated and copied behind the product
//                      (the query's rotated part), or a sigmoid gate on the result (a number an element, or with
//                      gate_per_head a number a head).  bfloat16 matrices run on the
//                      tensor cores (heads_product_mma), float32 ones on CUDA cores.
//   latent_attention   one warp a (row, head): keys lo..pos in ascending order, lo = 0 or pos - window + 1, online
//                      softmax in float32 whose denominator also counts exp(sink) once.
#include "api.h"
#include "common.cuh"
#include "mma_common.cuh"

namespace citlali {

// Element i of a vector of n whose first rot_dims elements turn by the position: the pair of i is i ^ 1 (neighbours) or,
// with halves, i +- rot_dims / 2; the pair's first element u becomes u cos - v sin, its second v cos + u sin.
template <typename TX>
__device__ __forceinline__ float rotated_element(const TX* __restrict__ src, int i, int rot_dims, int halves, int pos,
                                                 const float* __restrict__ inv_freq) {
    const float self = ldf(src, i);
    if (i >= rot_dims) return self;
    const int half = rot_dims >> 1;
    const bool first = halves ? i < half : !(i & 1);
    const int f = halves ? (first ? i : i - half) : i >> 1;
    const float other = ldf(src, halves ? (first ? i + half : i - half) : i ^ 1);
    float sn, cs;
    sincosf((float)pos * inv_freq[f], &sn, &cs);
    return first ? self * cs - other * sn : self * cs + other * sn;
}

// proj [rows, proj_stride] float32: query latent (RQ) | c (R) | r (P) | ...   (has_kv = 0: no c and r in the row).
template <typename TC, typename TQ>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(const float* __restrict__ proj, int proj_stride, int RQ, int R, int P, int has_kv,
                      const float* __restrict__ q_weight, const float* __restrict__ c_weight,
                      const float* __restrict__ inv_freq, int rot_dims, const int32_t* __restrict__ row_slot,
                      const int32_t* __restrict__ row_pos, const int32_t* __restrict__ page_table, int table_stride,
                      TC* __restrict__ pool, int page_size, TQ* __restrict__ cq, float eps, int rot_halves) {
    __shared__ float scratch[32];
    dependents_may_launch();
    wait_for_predecessor();
    const int row = blockIdx.x;
    const float* src = proj + (size_t)row * proj_stride;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < RQ; i += blockDim.x) ss = fmaf(src[i], src[i], ss);
    ss = block_sum(ss, scratch);
    float inv = 1.0f / sqrtf(ss / (float)RQ + eps);
    for (int i = threadIdx.x; i < RQ; i += blockDim.x) stf(cq, (size_t)row * RQ + i, src[i] * inv * q_weight[i]);
    if (!has_kv) return;
    const float* c = src + RQ;
    ss = 0.0f;
    for (int i = threadIdx.x; i < R; i += blockDim.x) ss = fmaf(c[i], c[i], ss);
    ss = block_sum(ss, scratch);
    inv = 1.0f / sqrtf(ss / (float)R + eps);
    const int pos = row_pos[row];
    const int page = page_table[(size_t)row_slot[row] * table_stride + pos / page_size];
    TC* dst = pool + ((size_t)page * page_size + pos % page_size) * (R + P);
    for (int i = threadIdx.x; i < R; i += blockDim.x) stf(dst, i, c[i] * inv * c_weight[i]);
    const float* r = c + R;
    if (rot_halves) {
        for (int i = threadIdx.x; i < P; i += blockDim.x) stf(dst, R + i, rotated_element(r, i, rot_dims, 1, pos, inv_freq));
        return;
    }
    for (int i = threadIdx.x; i < P / 2; i += blockDim.x) {
        float a = r[2 * i], b = r[2 * i + 1];
        if (2 * i + 1 < rot_dims) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            const float a2 = a * cs - b * sn, b2 = b * cs + a * sn;
            a = a2; b = b2;
        }
        stf(dst, R + 2 * i, a);
        stf(dst, R + 2 * i + 1, b);
    }
    if ((P & 1) && threadIdx.x == 0) stf(dst, R + P - 1, r[P - 1]);
}

// x[row, h, K .. K + tail) rotated by the row's position (pairs (2i, 2i+1) below rot_dims) and written to
// y[row, h, N .. N + tail), for `count` rows from row0 on; the block's threads share the work.
template <typename TX, typename TY>
__device__ __forceinline__ void rotate_tail(const TX* __restrict__ x, size_t x_row, int x_head, TY* __restrict__ y, size_t y_row,
                                            int y_head, int h, int row0, int count, int rows, int K, int N, int tail,
                                            const float* __restrict__ inv_freq, int rot_dims,
                                            const int32_t* __restrict__ row_pos, int rot_halves) {
    if (rot_halves) {
        for (int e = threadIdx.x; e < count * tail; e += blockDim.x) {
            const int r = e / tail, i = e % tail, row = row0 + r;
            if (row >= rows) continue;
            const TX* src = x + (size_t)row * x_row + (size_t)h * x_head + K;
            stf(y + (size_t)row * y_row + (size_t)h * y_head + N, i,
                rotated_element(src, i, rot_dims, 1, rot_dims > 0 ? row_pos[row] : 0, inv_freq));
        }
        return;
    }
    const int pairs = (tail + 1) / 2;
    for (int e = threadIdx.x; e < count * pairs; e += blockDim.x) {
        const int r = e / pairs, i = e % pairs, row = row0 + r;
        if (row >= rows) continue;
        const TX* src = x + (size_t)row * x_row + (size_t)h * x_head + K;
        TY* dst = y + (size_t)row * y_row + (size_t)h * y_head + N;
        float a = ldf(src, 2 * i);
        if (2 * i + 1 >= tail) { stf(dst, 2 * i, a); continue; }
        float b = ldf(src, 2 * i + 1);
        if (2 * i + 1 < rot_dims) {
            float sn, cs;
            sincosf((float)row_pos[row] * inv_freq[i], &sn, &cs);
            const float a2 = a * cs - b * sn, b2 = b * cs + a * sn;
            a = a2; b = b2;
        }
        stf(dst, 2 * i, a);
        stf(dst, 2 * i + 1, b);
    }
}

// y[row, h, n] = sum_k x[row * x_row + h * x_head + k] * M[h * m_head + k * m_k + n * m_n],  n < N, k < K.
// k ascending, float accumulation.  A block: 8 rows x 64 columns of one head; tiles of 32 k through shared memory.
// tail > 0: x[row, h, K .. K + tail) is rotated by the row's position (pairs (2i, 2i+1) below rot_dims) and written to
// y[row, h, N .. N + tail).  gate: y *= sigmoid(gate[row * gate_stride + h * N + n]).
template <typename TX, typename TM, typename TY>
__global__ void __launch_bounds__(256)
heads_product_kernel(const TX* __restrict__ x, size_t x_row, int x_head, const TM* __restrict__ M, size_t m_head, int m_k,
                     int m_n, TY* __restrict__ y, size_t y_row, int y_head, int rows, int K, int N, int tail,
                     const float* __restrict__ inv_freq, int rot_dims, const int32_t* __restrict__ row_pos,
                     const float* __restrict__ gate, size_t gate_stride, int rot_halves, int gate_per_head) {
    __shared__ float xs[8][33];
    __shared__ float ms[32][65];
    dependents_may_launch();
    wait_for_predecessor();
    const int h = blockIdx.y, row0 = blockIdx.x * 8, n0 = blockIdx.z * 64;
    const int tn = threadIdx.x & 63, tr = threadIdx.x >> 6;             // thread: column tn, rows tr and tr + 4
    float acc0 = 0.0f, acc1 = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 32) {
        {
            const int r = threadIdx.x >> 5, k = threadIdx.x & 31;
            xs[r][k] = (row0 + r < rows && k0 + k < K) ? ldf(x, (size_t)(row0 + r) * x_row + (size_t)h * x_head + k0 + k) : 0.0f;
        }
        for (int e = threadIdx.x; e < 32 * 64; e += 256) {
            // the faster index of the tile follows the matrix's contiguous axis
            const int k = m_n == 1 ? e >> 6 : e & 31, n = m_n == 1 ? e & 63 : e >> 5;
            ms[k][n] = (k0 + k < K && n0 + n < N) ? ldf(M, (size_t)h * m_head + (size_t)(k0 + k) * m_k + (size_t)(n0 + n) * m_n) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const float m = ms[k][tn];
            acc0 = fmaf(xs[tr][k], m, acc0);
            acc1 = fmaf(xs[tr + 4][k], m, acc1);
        }
        __syncthreads();
    }
    const int n = n0 + tn;
    if (n < N) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = row0 + tr + 4 * half;
            if (row >= rows) continue;
            float v = half ? acc1 : acc0;
            if (gate) v *= 1.0f / (1.0f + expf(-gate[(size_t)row * gate_stride + (gate_per_head ? (size_t)h : (size_t)h * N + n)]));
            stf(y, (size_t)row * y_row + (size_t)h * y_head + n, v);
        }
    }
    if (tail > 0 && blockIdx.z == 0)
        rotate_tail(x, x_row, x_head, y, y_row, y_head, h, row0, 8, rows, K, N, tail, inv_freq, rot_dims, row_pos, rot_halves);
}

// The same product on the tensor cores for bfloat16 matrices: a block of four warps computes 64 rows x 64 columns of one
// head (a warp: 16 rows), x and M_h pass through shared memory as bfloat16 in tiles of 64 k (M_h laid [n][k] whatever
// its strides; 16-byte loads along the matrix's contiguous axis where alignment allows), m16n8k16 MMAs with float
// accumulators, k ascending.
template <typename TX, typename TY>
__global__ void __launch_bounds__(128)
heads_product_mma_kernel(const TX* __restrict__ x, size_t x_row, int x_head, const __nv_bfloat16* __restrict__ M,
                         size_t m_head, int m_k, int m_n, TY* __restrict__ y, size_t y_row, int y_head, int rows, int K,
                         int N, int tail, const float* __restrict__ inv_freq, int rot_dims,
                         const int32_t* __restrict__ row_pos, const float* __restrict__ gate, size_t gate_stride,
                         int rot_halves, int gate_per_head) {
    constexpr int KT = 64, LD = KT + 8;
    __shared__ __align__(16) __nv_bfloat16 xs[64][LD];
    __shared__ __align__(16) __nv_bfloat16 ms[64][LD];
    dependents_may_launch();
    wait_for_predecessor();
    const int h = blockIdx.y, row0 = blockIdx.x * 64, n0 = blockIdx.z * 64;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f;
    const uint32_t xs_a = (uint32_t)__cvta_generic_to_shared(&xs[0][0]), ms_a = (uint32_t)__cvta_generic_to_shared(&ms[0][0]);
    const __nv_bfloat16* Mh = M + (size_t)h * m_head;
    const bool x_vec = sizeof(TX) == 4 && x_row % 4 == 0 && x_head % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const bool m_vec = (reinterpret_cast<uintptr_t>(M) & 15) == 0 && m_head % 8 == 0 && (m_k == 1 ? m_n % 8 == 0 : m_k % 8 == 0);
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.0f);
    for (int k0 = 0; k0 < K; k0 += KT) {
        // x: 64 rows x 64 k in pieces of four
        for (int e = threadIdx.x; e < 64 * (KT / 4); e += 128) {
            const int r = e / (KT / 4), k = (e % (KT / 4)) * 4, row = row0 + r;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (row < rows) {
                const TX* src = x + (size_t)row * x_row + (size_t)h * x_head + k0 + k;
                if constexpr (sizeof(TX) == 4) {
                    if (x_vec && k0 + k + 4 <= K) {
                        const float4 f = *reinterpret_cast<const float4*>(src);
                        v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                    } else {
                        for (int j = 0; j < 4; ++j) if (k0 + k + j < K) v[j] = ldf(src, j);
                    }
                } else {
                    for (int j = 0; j < 4; ++j) if (k0 + k + j < K) v[j] = ldf(src, j);
                }
            }
            *reinterpret_cast<uint2*>(&xs[r][k]) = make_uint2(fa::pack_bf16(v[0], v[1]), fa::pack_bf16(v[2], v[3]));
        }
        // M_h: 64 n x 64 k in pieces of eight along the matrix's contiguous axis
        for (int e = threadIdx.x; e < 64 * (KT / 8); e += 128) {
            if (m_k == 1) {                                   // k contiguous: a piece is eight k of one n
                const int n = e / (KT / 8), k = (e % (KT / 8)) * 8;
                const __nv_bfloat16* src = Mh + (size_t)(n0 + n) * m_n + k0 + k;
                if (m_vec && n0 + n < N && k0 + k + 8 <= K) {
                    *reinterpret_cast<uint4*>(&ms[n][k]) = *reinterpret_cast<const uint4*>(src);
                } else {
                    for (int j = 0; j < 8; ++j) ms[n][k + j] = (n0 + n < N && k0 + k + j < K) ? src[j] : zero;
                }
            } else {                                          // n contiguous (or neither): a piece is eight n of one k
                const int k = e / 8, n = (e % 8) * 8;
                const __nv_bfloat16* src = Mh + (size_t)(k0 + k) * m_k + (size_t)(n0 + n) * m_n;
                if (m_vec && m_n == 1 && k0 + k < K && n0 + n + 8 <= N) {
                    const uint4 w = *reinterpret_cast<const uint4*>(src);
                    const __nv_bfloat16* wv = reinterpret_cast<const __nv_bfloat16*>(&w);
                    for (int j = 0; j < 8; ++j) ms[n + j][k] = wv[j];
                } else {
                    for (int j = 0; j < 8; ++j) ms[n + j][k] = (k0 + k < K && n0 + n + j < N) ? src[(size_t)j * m_n] : zero;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < KT; kk += 16) {
            uint32_t a0, a1, a2, a3;
            fa::ldmatrix_x4(xs_a + (uint32_t)(((warp * 16 + (lane & 15)) * LD + kk + (lane >> 4) * 8) * 2), a0, a1, a2, a3);
#pragma unroll
            for (int n = 0; n < 8; n += 2) {
                uint32_t b0, b1, b2, b3;
                fa::ldmatrix_x4(ms_a + (uint32_t)(((n * 8 + ((lane >> 4) << 3) + (lane & 7)) * LD + kk + ((lane >> 3) & 1) * 8) * 2),
                                b0, b1, b2, b3);
                fa::mma_16816(acc[n], a0, a1, a2, a3, b0, b1);
                fa::mma_16816(acc[n + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();
    }
    // a lane holds two neighbouring columns of a row: stored as one word where the output's rows and heads start on even
    // elements (8 bytes of float32, 4 of bfloat16)
    const bool pairs = y_row % 2 == 0 && y_head % 2 == 0 && (reinterpret_cast<uintptr_t>(y) & (2 * sizeof(TY) - 1)) == 0;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int row = row0 + warp * 16 + g + half * 8, col = n0 + n * 8 + t * 2;
            if (row >= rows || col >= N) continue;
            float v0 = acc[n][2 * half], v1 = acc[n][2 * half + 1];
            if (gate) {
                const float* gr = gate + (size_t)row * gate_stride + (gate_per_head ? (size_t)h : (size_t)h * N + col);
                v0 *= 1.0f / (1.0f + expf(-gr[0]));
                if (col + 1 < N) v1 *= 1.0f / (1.0f + expf(-gr[gate_per_head ? 0 : 1]));
            }
            TY* dst = y + (size_t)row * y_row + (size_t)h * y_head + col;
            if (pairs && col + 1 < N) {
                if constexpr (sizeof(TY) == 4) *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
                else *reinterpret_cast<uint32_t*>(dst) = fa::pack_bf16(v0, v1);
            } else {
                stf(dst, 0, v0);
                if (col + 1 < N) stf(dst, 1, v1);
            }
        }
    if (tail > 0 && blockIdx.z == 0)
        rotate_tail(x, x_row, x_head, y, y_row, y_head, h, row0, 64, rows, K, N, tail, inv_freq, rot_dims, row_pos, rot_halves);
}

// q [rows, H, E] float32 (E = R + P: the query in the latent's coordinates, then its rotated part); the cache's pool
// [page, page_size, E]; out [rows, H, R] float32 = sum_j p_j c_j.  NC * 32 >= E.
template <typename TC, int NC>
__global__ void __launch_bounds__(128)
latent_attention_kernel(const float* __restrict__ q, const TC* __restrict__ pool, const int32_t* __restrict__ page_table,
                        int table_stride, const int32_t* __restrict__ row_slot, const int32_t* __restrict__ row_pos,
                        const float* __restrict__ sink, float* __restrict__ out, int rows, int H, int R, int E,
                        int page_size, int window, float scale) {
    dependents_may_launch();
    wait_for_predecessor();
    const int lane = threadIdx.x & 31;
    const long unit = (long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (unit >= (long)rows * H) return;
    const int row = (int)(unit / H), h = (int)(unit % H);          // the warps of a block share a row's keys
    const int pos = row_pos[row];
    const int32_t* table = page_table + (size_t)row_slot[row] * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    float qv[NC], acc[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) {
        const int i = j * 32 + lane;
        qv[j] = i < E ? q[((size_t)row * H + h) * E + i] * scale : 0.0f;
        acc[j] = 0.0f;
    }
    float top = -INFINITY, denom = 0.0f;
    for (int key = lo; key <= pos; ++key) {
        const TC* kv = pool + ((size_t)table[key / page_size] * page_size + key % page_size) * E;
        float kvv[NC];
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < NC; ++j) {
            const int i = j * 32 + lane;
            kvv[j] = i < E ? ldf(kv, i) : 0.0f;
            s = fmaf(qv[j], kvv[j], s);
        }
        s = warp_sum(s);
        const float new_top = fmaxf(top, s);
        const float shrink = expf(top - new_top), p = expf(s - new_top);     // exp(-inf) = 0 on the first key
        denom = denom * shrink + p;
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[j] = fmaf(p, kvv[j], acc[j] * shrink);
        top = new_top;
    }
    if (sink) {
        const float sk = sink[h], new_top = fmaxf(top, sk);
        const float shrink = expf(top - new_top);
        denom = denom * shrink + expf(sk - new_top);
#pragma unroll
        for (int j = 0; j < NC; ++j) acc[j] *= shrink;
    }
    const float inv = 1.0f / denom;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
        const int i = j * 32 + lane;
        if (i < R) out[((size_t)row * H + h) * R + i] = acc[j] * inv;
    }
}

}  // namespace citlali

using namespace citlali;

extern "C" int citlali_latent_prepare(const float* proj, int proj_stride, int RQ, int R, int P, int has_kv,
                                      const float* q_weight, const float* c_weight, const float* inv_freq, int rot_dims,
                                      const int32_t* row_slot, const int32_t* row_pos, const int32_t* page_table,
                                      int table_stride, void* pool, int cache_dtype, int page_size, void* cq, int cq_dtype,
                                      int rows, float eps, int rot_halves, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (rot_dims < 0 || rot_dims > P || (rot_dims & 1)) {
        set_last_error("latent_prepare: %d rotated dimensions of a key part of %d", rot_dims, P);
        return kBadShape;
    }
    return CITLALI_DISPATCH_FLOAT(cache_dtype, TC, [&] {
        return CITLALI_DISPATCH_FLOAT(cq_dtype, TQ, [&] {
            launch_kernel(latent_prepare_kernel<TC, TQ>, rows, 256, 0, stream, proj, proj_stride, RQ, R, P, has_kv, q_weight,
                          c_weight, inv_freq, rot_dims, row_slot, row_pos, page_table, table_stride, (TC*)pool, page_size,
                          (TQ*)cq, eps, rot_halves);
            return CITLALI_LAUNCH_CHECK();
        });
    });
}

extern "C" int citlali_heads_product(const void* x, int x_dtype, size_t x_row, int x_head, const void* M, int m_dtype,
                                     size_t m_head, int m_k, int m_n, void* y, int y_dtype, size_t y_row, int y_head,
                                     int rows, int heads, int K, int N, int tail, const float* inv_freq, int rot_dims,
                                     const int32_t* row_pos, const float* gate, size_t gate_stride, int rot_halves,
                                     int gate_per_head, cudaStream_t stream) {
    if (rows <= 0 || heads <= 0) return 0;
    if (heads > 65535 || (N + 63) / 64 > 65535) {
        set_last_error("heads_product: %d heads or %d columns exceed the grid", heads, N);
        return kTooLarge;
    }
    if (tail > 0 && (rot_dims > tail || (rot_dims & 1) || (rot_dims > 0 && (!inv_freq || !row_pos)))) {
        set_last_error("heads_product: %d rotated dimensions of a tail of %d", rot_dims, tail);
        return kBadShape;
    }
    if (m_dtype == kBF16) {
        dim3 grid((rows + 63) / 64, heads, (N + 63) / 64);
        return CITLALI_DISPATCH_FLOAT(x_dtype, TX, [&] {
            return CITLALI_DISPATCH_FLOAT(y_dtype, TY, [&] {
                launch_kernel(heads_product_mma_kernel<TX, TY>, grid, 128, 0, stream, (const TX*)x, x_row, x_head,
                              (const __nv_bfloat16*)M, m_head, m_k, m_n, (TY*)y, y_row, y_head, rows, K, N, tail, inv_freq,
                              rot_dims, row_pos, gate, gate_stride, rot_halves, gate_per_head);
                return CITLALI_LAUNCH_CHECK();
            });
        });
    }
    dim3 grid((rows + 7) / 8, heads, (N + 63) / 64);
    return CITLALI_DISPATCH_FLOAT(x_dtype, TX, [&] {
        return CITLALI_DISPATCH_FLOAT(m_dtype, TM, [&] {
            return CITLALI_DISPATCH_FLOAT(y_dtype, TY, [&] {
                launch_kernel(heads_product_kernel<TX, TM, TY>, grid, 256, 0, stream, (const TX*)x, x_row, x_head, (const TM*)M,
                              m_head, m_k, m_n, (TY*)y, y_row, y_head, rows, K, N, tail, inv_freq, rot_dims, row_pos, gate,
                              gate_stride, rot_halves, gate_per_head);
                return CITLALI_LAUNCH_CHECK();
            });
        });
    });
}

extern "C" int citlali_latent_attention(const float* q, const void* pool, int cache_dtype, const int32_t* page_table,
                                        int table_stride, const int32_t* row_slot, const int32_t* row_pos,
                                        const float* sink, float* out, int rows, int H, int R, int E, int page_size,
                                        int window, float scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (E > 1024 || R > E) {
        set_last_error("latent_attention: a cached vector of %d (latent %d) exceeds 1024", E, R);
        return kTooLarge;
    }
    const long units = (long)rows * H;
    const int blocks = (int)((units + 3) / 4);
    const int nc = (E + 31) / 32;
#define CITLALI_LATENT(TC, NC)                                                                                        \
    launch_kernel(latent_attention_kernel<TC, NC>, blocks, 128, 0, stream, q, (const TC*)pool, page_table, table_stride, \
                  row_slot, row_pos, sink, out, rows, H, R, E, page_size, window, scale)
#define CITLALI_LATENT_SIZES(TC)                    \
    if (nc <= 2) CITLALI_LATENT(TC, 2);             \
    else if (nc <= 4) CITLALI_LATENT(TC, 4);        \
    else if (nc <= 6) CITLALI_LATENT(TC, 6);        \
    else if (nc <= 8) CITLALI_LATENT(TC, 8);        \
    else if (nc <= 12) CITLALI_LATENT(TC, 12);      \
    else if (nc <= 16) CITLALI_LATENT(TC, 16);      \
    else if (nc <= 20) CITLALI_LATENT(TC, 20);      \
    else if (nc <= 24) CITLALI_LATENT(TC, 24);      \
    else CITLALI_LATENT(TC, 32)
    if (cache_dtype == kF32) { CITLALI_LATENT_SIZES(float); }
    else if (cache_dtype == kBF16) { CITLALI_LATENT_SIZES(__nv_bfloat16); }
    else {
        set_last_error("latent_attention: dtype code %d is neither float32 (0) nor bfloat16 (1)", cache_dtype);
        return kBadDType;
    }
#undef CITLALI_LATENT_SIZES
#undef CITLALI_LATENT
    return CITLALI_LAUNCH_CHECK();
}
