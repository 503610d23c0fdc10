// Sigmoid attention of runs of new tokens on the tensor cores (bfloat16 cache, pages of 64 keys), in two kernels, because
// a head's weight needs every head's score and no block can keep the outputs of all heads:
//
//   sigmoid_weights  a block takes 8 consecutive rows of a sequence, ALL heads, and a run of key pages.  Two of its eight warps
//                    share 16 of a page's 64 keys: each fetches them per key/value head (cp.async, straight on to
//                    registers), computes K Q_g^T for its half of the heads g with mma.sync m16n8k16 (keys are M, the 8 rows
//                    are N), takes the scale and the distance term in float32 and leaves s_g in shared memory.  When all
//                    heads are there, the two warps mix them on the CUDA cores, eight output heads at a time, m_h = sum_g talk[h, g] s_g + head_bias[h],
//                    takes the sigmoid (0 where the key is not visible) and writes the weights in bfloat16 to
//                    W [head, group of 8 rows, column, 8 rows]; column 0 is the first key of the first page that the
//                    16 rows around the group can see.
//   sigmoid_values   a block takes 64 rows and one head, walks the pages its rows see, and adds W V with the same MMA into
//                    float32 registers (W tiles come by cp.async into a buffer a warp, values a page at a time for the
//                    block), then multiplies by the gate and writes the row.
//
// The sums over keys go in the order of the pages, so a row's result depends on its position and the window alone.
#include "api.h"
#include "common.cuh"
#include "mma_common.cuh"

namespace citlali {
namespace sgt {

using namespace fa;

constexpr int kKeys = 64;            // keys of a tile: one cache page
constexpr int kRows = 8;             // rows of a weights block
constexpr int kTilesPerBlock = 8;    // pages a weights block walks
constexpr int kValueRows = 64;       // rows of a values block
constexpr int kWRow = 48;            // bytes between keys in a warp's buffer of weights (16 rows used, spread over the banks)

__device__ __forceinline__ void ldmatrix_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}

__host__ __device__ inline int padded_heads(int H) { return (H + 7) / 8 * 8; }

inline size_t weights_smem(int H, int D) {
    const int hp = padded_heads(H);
    return (size_t)H * kRows * (D * 2 + 16) + (size_t)2 * kKeys * (D * 2 + 16) + (size_t)4 * H * 16 * kRows * sizeof(float) +
           (size_t)(2 * H * hp + hp + H) * sizeof(float);
}

// c += a * b on two floats at once.
__device__ __forceinline__ void fma2(float2& c, const float2 a, const float2 b) {
    c.x = fmaf(a.x, b.x, c.x);
    c.y = fmaf(a.y, b.y, c.y);
}
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// DK: head size / 16.
template <int DK>
__global__ void __launch_bounds__(256, 2)
sigmoid_weights_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                       const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ seq_start,
                       const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_past,
                       const float* __restrict__ talk, const float* __restrict__ head_bias, __nv_bfloat16* __restrict__ W,
                       int ldc, int groups_total, int H, int G, int window, float scale, float slope_exp) {
    constexpr int D = DK * 16;
    constexpr int kRowBytes = D * 2 + 16;
    constexpr int kChunks = D / 8;
    extern __shared__ __align__(16) uint8_t smem[];
    const int hp = padded_heads(H), per = H / G;
    uint8_t* q_bytes = smem;                                               // [H, 8 rows, D (+8)]
    uint8_t* k_bytes = q_bytes + (size_t)H * kRows * kRowBytes;            // [4 warps][2][16 keys, D (+8)]
    float* s_all = reinterpret_cast<float*>(k_bytes + 2 * kKeys * kRowBytes);  // [4 warps][H, 16 keys, 8 rows]
    float* t_mix = s_all + 4 * H * 16 * kRows;                             // [H (g), hp (h), 2]: talk transposed, each twice
    float* t_bias = t_mix + 2 * H * hp;                                    // [hp], times -log2(e)
    float* t_slope = t_bias + hp;                                          // [H]
    const uint32_t s_q = (uint32_t)__cvta_generic_to_shared(q_bytes), s_k = (uint32_t)__cvta_generic_to_shared(k_bytes);

    dependents_may_launch();
    wait_for_predecessor();
    const int seq = blockIdx.z, q0 = blockIdx.y * kRows;
    const int row0 = seq_start[seq], n_new = seq_start[seq + 1] - row0;
    if (q0 >= n_new) return;
    const int past = seq_past[seq];
    const int q16 = q0 / 16 * 16;
    const int first16 = past + q16, last16 = past + min(q16 + 16, n_new) - 1;
    const int tlo = window > 0 ? max(0, first16 - window + 1) / kKeys : 0, thi = last16 / kKeys;
    const int t_begin = tlo + blockIdx.x * kTilesPerBlock, t_end = min(thi + 1, t_begin + kTilesPerBlock);
    if (t_begin > thi) return;
    const size_t group = (size_t)(row0 / kRows + seq + blockIdx.y);
    const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    for (int c = tid; c < H * kRows * kChunks; c += 256) {
        const int ch = c % kChunks, r = (c / kChunks) % kRows, h = c / (kChunks * kRows);
        const int at = (h * kRows + r) * kRowBytes + ch * 16;
        if (q0 + r < n_new) cp_async16(s_q + at, q + ((size_t)(row0 + q0 + r) * H + h) * D + ch * 8);
        else *reinterpret_cast<uint4*>(q_bytes + at) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
    for (int i = tid; i < H * hp; i += 256) {
        const int g = i / hp, h = i % hp;
        t_mix[2 * i] = t_mix[2 * i + 1] = h < H ? (talk ? talk[h * H + g] : (h == g ? 1.0f : 0.0f)) : 0.0f;
    }
    for (int i = tid; i < hp; i += 256) t_bias[i] = (head_bias && i < H) ? -1.4426950408889634f * head_bias[i] : 0.0f;
    for (int i = tid; i < H; i += 256) t_slope[i] = slope_exp > 0.0f ? exp2f(-slope_exp * (float)(i + 1) / (float)H) : 0.0f;

    // Two warps share 16 of the page's keys: each computes the scores of its half of the heads (split between key/value
    // heads where there are several), then each mixes every other run of eight output heads.
    const int slice = warp & 3, half = warp >> 2;
    const int h_mid = G >= 2 ? (G + 1) / 2 * per : (H + 1) / 2;
    const int h_lo = half ? h_mid : 0, h_hi = half ? H : h_mid;
    const int kv_lo = h_lo / per, nkv = h_hi > h_lo ? (h_hi - 1) / per - kv_lo + 1 : 0;
    const int tiles = t_end - t_begin, jobs = tiles * nkv;
    float* s_w = s_all + (size_t)slice * H * 16 * kRows;
    const int c_key = lane >> 2, c_row = (lane & 3) * 2;        // this lane's place in an accumulator tile
    const int m_key = lane >> 1, m_row = (lane & 1) * 4;        // and in the mix: a key and four rows
    // a warp fetches its 16 keys of a (page, key/value head) into its own buffer; they leave it for registers at once, so the
    // next ones are fetched while the warp works
    const uint32_t my_k = s_k + warp * 16 * kRowBytes;
    auto load_keys = [&](int n) {
        const int t = t_begin + n / nkv, kv = kv_lo + n % nkv;
        const size_t base = (((size_t)pages[t] * G + kv) * kKeys + slice * 16) * D;
        for (int c = lane; c < 16 * kChunks; c += 32) {
            const int r = c / kChunks, ch = c % kChunks;
            cp_async16(my_k + r * kRowBytes + ch * 16, k_pool + base + (size_t)r * D + ch * 8);
        }
    };
    auto pair_barrier = [&]() { asm volatile("bar.sync %0, 64;" ::"r"(1 + slice) : "memory"); };
    if (jobs > 0) load_keys(0);
    cp_async_commit();
    cp_async_wait<1>();                                        // the queries
    __syncthreads();
    int n = 0;
    for (int ti = 0; ti < tiles; ++ti) {
        const int t = t_begin + ti;
        // distances of this lane's four places in an accumulator tile (the same for every head)
        const int key0 = t * kKeys + slice * 16 + c_key, pos0 = past + q0 + c_row;
        const float d00 = (float)(pos0 - key0), d01 = d00 + 1.0f, d10 = d00 - 8.0f, d11 = d00 - 7.0f;
        for (int k = 0; k < nkv; ++k, ++n) {
            const int kv = kv_lo + k;
            cp_async_wait<0>();
            __syncwarp();
            uint32_t kf[DK][4];
            {
                const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
                const int cbyte = (lane >> 4) * 16;
#pragma unroll
                for (int ks = 0; ks < DK; ++ks)
                    ldmatrix_x4(my_k + r * kRowBytes + ks * 32 + cbyte, kf[ks][0], kf[ks][1], kf[ks][2], kf[ks][3]);
            }
            __syncwarp();
            if (n + 1 < jobs) load_keys(n + 1);
            cp_async_commit();
            const int g_end = min(h_hi, (kv + 1) * per);
            for (int g = max(h_lo, kv * per); g < g_end; ++g) {
                float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f}, odd[4] = {0.0f, 0.0f, 0.0f, 0.0f};      // two chains of MMAs
                const uint32_t qb = s_q + (g * kRows + (lane & 7)) * kRowBytes + ((lane >> 3) & 1) * 16;
#pragma unroll
                for (int ks = 0; ks < DK; ++ks) {
                    uint32_t b0, b1;
                    ldmatrix_x2(qb + ks * 32, b0, b1);
                    if (ks & 1) mma_16816(odd, kf[ks][0], kf[ks][1], kf[ks][2], kf[ks][3], b0, b1);
                    else mma_16816(acc, kf[ks][0], kf[ks][1], kf[ks][2], kf[ks][3], b0, b1);
                }
                const float slope = t_slope[g];
                float2 lo2, hi2;
                lo2.x = (acc[0] + odd[0]) * scale - slope * d00;
                lo2.y = (acc[1] + odd[1]) * scale - slope * d01;
                hi2.x = (acc[2] + odd[2]) * scale - slope * d10;
                hi2.y = (acc[3] + odd[3]) * scale - slope * d11;
                *reinterpret_cast<float2*>(s_w + (g * 16 + c_key) * kRows + c_row) = lo2;
                *reinterpret_cast<float2*>(s_w + (g * 16 + c_key + 8) * kRows + c_row) = hi2;
            }
        }
        pair_barrier();
        // all heads' scores of this page are there.  The mix: this lane's key and four rows, eight output heads at a time
        const int key = t * kKeys + slice * 16 + m_key;
        bool visible[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = q0 + m_row + i, pos = past + r;
            visible[i] = r < n_new && key <= pos && (window <= 0 || key > pos - window);
        }
        const size_t col = (size_t)(t - tlo) * kKeys + slice * 16 + m_key;
        __nv_bfloat16* w_at = W + ((size_t)group * ldc + col) * kRows + m_row;
        const size_t w_head = (size_t)groups_total * ldc * kRows;
        for (int hc = half * 8; hc < hp; hc += 16) {
            float2 m[8][2];
#pragma unroll
            for (int j = 0; j < 8; ++j) { m[j][0] = make_float2(0.0f, 0.0f); m[j][1] = make_float2(0.0f, 0.0f); }
            const float* s_at = s_w + m_key * kRows + m_row;
            const float* t_at = t_mix + 2 * hc;
#pragma unroll 4
            for (int g = 0; g < H; ++g) {
                const float4 s4 = *reinterpret_cast<const float4*>(s_at + g * 16 * kRows);
                const float2 s01 = make_float2(s4.x, s4.y), s23 = make_float2(s4.z, s4.w);
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    const float4 tt = *reinterpret_cast<const float4*>(t_at + (size_t)g * 2 * hp + 2 * j);
                    const float2 ta = make_float2(tt.x, tt.y), tb = make_float2(tt.z, tt.w);
                    fma2(m[j][0], ta, s01); fma2(m[j][1], ta, s23);
                    fma2(m[j + 1][0], tb, s01); fma2(m[j + 1][1], tb, s23);
                }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int h = hc + j;
                const float b = t_bias[h];
                const float x[4] = {m[j][0].x, m[j][0].y, m[j][1].x, m[j][1].y};
                float w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {            // 1 / (1 + 2^(-(m + bias) log2 e)), 0 for a key that is not visible
                    w[i] = fast_rcp(1.0f + fast_exp2(fmaf(x[i], -1.4426950408889634f, b)));
                    w[i] = visible[i] ? w[i] : 0.0f;
                }
                uint2 packed;
                packed.x = pack_bf16(w[0], w[1]);
                packed.y = pack_bf16(w[2], w[3]);
                if (h < H) *reinterpret_cast<uint2*>(w_at + (size_t)h * w_head) = packed;
            }
        }
        pair_barrier();                                        // the scores are read before the next page's are written
    }
    cp_async_wait<0>();
}

// VK: value size / 16.
template <int VK>
__global__ void __launch_bounds__(128)
sigmoid_values_kernel(const __nv_bfloat16* __restrict__ W, int ldc, int groups_total, const __nv_bfloat16* __restrict__ v_pool,
                      const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ seq_start,
                      const int32_t* __restrict__ seq_slot, const int32_t* __restrict__ seq_past,
                      const float* __restrict__ gate, __nv_bfloat16* __restrict__ out, int H, int G, int window) {
    constexpr int V = VK * 16;
    constexpr int kRowBytes = V * 2 + 16;
    constexpr int kTileBytes = kKeys * kRowBytes;
    constexpr int kChunks = V / 8;
    constexpr int kWBytes = kKeys * kWRow;
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t s_v = (uint32_t)__cvta_generic_to_shared(smem);          // [2][64 keys, V (+8)]
    const uint32_t s_w = s_v + 2 * kTileBytes;                              // [4 warps][2][64 keys, 16 rows (+8)]

    dependents_may_launch();
    wait_for_predecessor();
    const int seq = blockIdx.z, head = blockIdx.x;
    const int row0 = seq_start[seq], n_new = seq_start[seq + 1] - row0;
    const int q0 = (gridDim.y - 1 - blockIdx.y) * kValueRows;              // the last rows see the most keys: first
    if (q0 >= n_new) return;
    const int past = seq_past[seq];
    const int kvh = head / (H / G);
    const int32_t* pages = page_table + (size_t)seq_slot[seq] * table_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int tlo_b = window > 0 ? max(0, past + q0 - window + 1) / kKeys : 0;
    const int thi_b = (past + min(q0 + kValueRows, n_new) - 1) / kKeys;
    const int qw = q0 + warp * 16;
    const bool active = qw < n_new;
    const int tlo_w = window > 0 ? max(0, past + qw - window + 1) / kKeys : 0;
    const int thi_w = active ? (past + min(qw + 16, n_new) - 1) / kKeys : -1;
    const bool second = qw + kRows < n_new;                                 // the warp's rows 8..15 exist
    const size_t group = (size_t)(row0 / kRows + seq + qw / kRows);
    const uint32_t my_w = s_w + warp * 2 * kWBytes;

    auto load_tile = [&](int t, int buf) {
        const size_t base = ((size_t)pages[t] * G + kvh) * kKeys * V;
        for (int c = tid; c < kKeys * kChunks; c += 128) {
            const int r = c / kChunks, ch = c % kChunks;
            cp_async16(s_v + buf * kTileBytes + r * kRowBytes + ch * 16, v_pool + base + (size_t)r * V + ch * 8);
        }
        if (t >= tlo_w && t <= thi_w) {
            const size_t col = (size_t)(t - tlo_w) * kKeys;
            for (int c = lane; c < kKeys * 2; c += 32) {
                const int key = c >> 1, half = c & 1;
                const uint32_t dst = my_w + buf * kWBytes + key * kWRow + half * 16;
                if (half == 0 || second)
                    cp_async16(dst, W + (((size_t)head * groups_total + group + half) * ldc + col + key) * kRows);
                else
                    *reinterpret_cast<uint4*>(smem + (dst - s_v)) = make_uint4(0, 0, 0, 0);
            }
        }
    };
    load_tile(tlo_b, 0);
    cp_async_commit();

    float o[2 * VK][4];
#pragma unroll
    for (int i = 0; i < 2 * VK; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f; }
    for (int t = tlo_b; t <= thi_b; ++t) {
        const int buf = (t - tlo_b) & 1;
        if (t + 1 <= thi_b) load_tile(t + 1, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        if (t >= tlo_w && t <= thi_w) {
            const uint32_t vb = s_v + buf * kTileBytes, wb = my_w + buf * kWBytes;
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk) {
                uint32_t a0, a1, a2, a3;
                {
                    const int mi = lane >> 3, key = kk * 16 + (mi >> 1) * 8 + (lane & 7);
                    ldmatrix_x4_trans(wb + key * kWRow + (mi & 1) * 16, a0, a1, a2, a3);
                }
#pragma unroll
                for (int np = 0; np < VK; ++np) {
                    const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                    const int cbyte = np * 32 + (lane >> 4) * 16;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans(vb + r * kRowBytes + cbyte, b0, b1, b2, b3);
                    mma_16816(o[2 * np], a0, a1, a2, a3, b0, b1);
                    mma_16816(o[2 * np + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();
    if (!active) return;
    const int r0 = qw + (lane >> 2), r1 = r0 + 8;
    const int colv = (lane & 3) * 2;
    const float g0 = (gate && r0 < n_new) ? gate[(size_t)(row0 + r0) * H + head] : 1.0f;
    const float g1 = (gate && r1 < n_new) ? gate[(size_t)(row0 + r1) * H + head] : 1.0f;
#pragma unroll
    for (int i = 0; i < 2 * VK; ++i) {
        if (r0 < n_new)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r0) * H + head) * V + i * 8 + colv) = pack_bf16(o[i][0] * g0, o[i][1] * g0);
        if (r1 < n_new)
            *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + r1) * H + head) * V + i * 8 + colv) = pack_bf16(o[i][2] * g1, o[i][3] * g1);
    }
}

template <int DK>
static int launch_weights(dim3 grid, size_t smem, cudaStream_t stream, const void* q, const void* k_pool, const int32_t* page_table,
                          int table_stride, const int32_t* seq_start, const int32_t* seq_slot, const int32_t* seq_past,
                          const float* talk, const float* head_bias, void* W, int ldc, int groups_total, int H, int G, int window,
                          float scale, float slope_exp) {
    auto kernel = sigmoid_weights_kernel<DK>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    launch_kernel(kernel, grid, 256, smem, stream, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, page_table, table_stride,
                  seq_start, seq_slot, seq_past, talk, head_bias, (__nv_bfloat16*)W, ldc, groups_total, H, G, window, scale,
                  slope_exp);
    return CITLALI_LAUNCH_CHECK();
}

template <int VK>
static int launch_values(dim3 grid, cudaStream_t stream, const void* W, int ldc, int groups_total, const void* v_pool,
                         const int32_t* page_table, int table_stride, const int32_t* seq_start, const int32_t* seq_slot,
                         const int32_t* seq_past, const float* gate, void* out, int H, int G, int window) {
    constexpr int smem = 2 * kKeys * (VK * 32 + 16) + 4 * 2 * kKeys * kWRow;
    auto kernel = sigmoid_values_kernel<VK>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    launch_kernel(kernel, grid, 128, smem, stream, (const __nv_bfloat16*)W, ldc, groups_total, (const __nv_bfloat16*)v_pool,
                  page_table, table_stride, seq_start, seq_slot, seq_past, gate, (__nv_bfloat16*)out, H, G, window);
    return CITLALI_LAUNCH_CHECK();
}

static bool size_has_kernel(int n) { return n >= 16 && n % 16 == 0 && (n <= 128 || n == 256); }

}  // namespace sgt
}  // namespace citlali

using namespace citlali;

// 1 if citlali_sigmoid_attention_mma has kernels for these sizes (bfloat16 only).
extern "C" int citlali_sigmoid_attention_mma_supports(int H, int G, int D, int V, int page_size) {
    if (page_size != sgt::kKeys || H <= 0 || G <= 0 || H % G != 0) return 0;
    if (!sgt::size_has_kernel(D) || !sgt::size_has_kernel(V)) return 0;
    return sgt::weights_smem(H, D) <= 200 * 1024 ? 1 : 0;
}

// Columns (keys) a row group's weights take, and row groups, for `rows` rows of `sequences` sequences whose rows see at most
// `max_keys` keys; the scratch holds H * groups * columns * 8 bfloat16.
extern "C" int citlali_sigmoid_attention_mma_columns(int window, int max_keys) {
    int tiles = (max_keys + sgt::kKeys - 1) / sgt::kKeys;
    if (window > 0) {
        const int banded = (window + 14) / sgt::kKeys + 2;
        if (banded < tiles) tiles = banded;
    }
    return (tiles < 1 ? 1 : tiles) * sgt::kKeys;
}
extern "C" int citlali_sigmoid_attention_mma_groups(int rows, int sequences) { return rows / sgt::kRows + sequences + 1; }

// Sigmoid attention (see citlali_sigmoid_attention) of the new tokens of `sequences` sequences, as citlali_attention_prefill
// takes them; bfloat16 q, cache and out; `weights` is scratch of H * groups * columns * 8 bfloat16 (the two functions above).
extern "C" int citlali_sigmoid_attention_mma(const void* q, const void* k_pool, const void* v_pool, const int32_t* page_table,
                                             int table_stride, const int32_t* seq_start, const int32_t* seq_slot,
                                             const int32_t* seq_past, const float* talk, const float* head_bias,
                                             const float* gate, void* out, void* weights, int columns, int groups, int sequences,
                                             int max_new, int H, int G, int D, int V, int page_size, int window, float scale,
                                             float slope_exp, cudaStream_t stream) {
    if (sequences <= 0 || max_new <= 0) return 0;
    if (!citlali_sigmoid_attention_mma_supports(H, G, D, V, page_size) || window < 0 || columns <= 0 || columns % sgt::kKeys != 0 ||
        weights == nullptr || sequences > 65535 || (max_new + sgt::kRows - 1) / sgt::kRows > 65535) {
        set_last_error("sigmoid_attention_mma: no kernel for %d heads over %d of %d (values %d) with pages of %d, or bad scratch",
                       H, G, D, V, page_size);
        return kBadShape;
    }
    if (((uintptr_t)q & 15u) || ((uintptr_t)weights & 15u) || ((uintptr_t)out & 3u)) {
        set_last_error("sigmoid_attention_mma: q and the scratch must be 16-byte aligned");
        return kBadAlignment;
    }
    const int chunks = (columns / sgt::kKeys + sgt::kTilesPerBlock - 1) / sgt::kTilesPerBlock;
    const dim3 wgrid(chunks, (max_new + sgt::kRows - 1) / sgt::kRows, sequences);
    const size_t wsmem = sgt::weights_smem(H, D);
    int rc = kBadShape;
#define CITLALI_SGW(N) case N: rc = sgt::launch_weights<N>(wgrid, wsmem, stream, q, k_pool, page_table, table_stride, seq_start, \
                                                            seq_slot, seq_past, talk, head_bias, weights, columns, groups, H, G, \
                                                            window, scale, slope_exp); break
    switch (D / 16) { CITLALI_SGW(1); CITLALI_SGW(2); CITLALI_SGW(3); CITLALI_SGW(4); CITLALI_SGW(5); CITLALI_SGW(6); CITLALI_SGW(7);
                      CITLALI_SGW(8); CITLALI_SGW(16); }
#undef CITLALI_SGW
    if (rc != 0) return rc;
    const dim3 vgrid(H, (max_new + sgt::kValueRows - 1) / sgt::kValueRows, sequences);
#define CITLALI_SGV(N) case N: return sgt::launch_values<N>(vgrid, stream, weights, columns, groups, v_pool, page_table, table_stride, \
                                                            seq_start, seq_slot, seq_past, gate, out, H, G, window)
    switch (V / 16) { CITLALI_SGV(1); CITLALI_SGV(2); CITLALI_SGV(3); CITLALI_SGV(4); CITLALI_SGV(5); CITLALI_SGV(6); CITLALI_SGV(7);
                      CITLALI_SGV(8); CITLALI_SGV(16); }
#undef CITLALI_SGV
    return kBadShape;
}
