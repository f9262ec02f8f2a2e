// Latent attention: every head's keys and values are products of ONE cached vector per position.
//
// A position's cache row is [c (R numbers: the down-projection's first R outputs, unit RMS times a weight) |
// k_rot (Dr numbers, rotated by position)], one row for all heads: [pages, 1, 1, page_size, R + Dr].
// Head h's key is [Wuk_h c | k_rot] and its value Wuv_h c. Because both are linear in c, the products with the
// per-head matrices move to the query's and the output's side:
//
//   score(i, j) = scale * ((Wuk_h^T q_h[:Dn]) . c_j + rot(q_h[Dn:]) . k_rot_j)          q~ = Wuk_h^T q_h[:Dn], R numbers
//   out_h(i)    = Wuv_h (sum_j p(i, j) c_j)                                             o~ = sum_j p c_j,     R numbers
//
// so attention itself runs over the cache rows alone, as multi-query attention with keys of R + Dr and values of R
// channels (the values ARE the keys' first R channels). The two small per-head products are batched matrix products
// outside this file. Visible keys: j <= i, and i - j < window when window > 0. With `sink` a learned number per
// head joins the softmax's denominator (exp(sink_h), once, with no key and no value). With `gate` a head's output is
// multiplied by sigmoid(gate[t, h]). Scores, the softmax and the sums are float32.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kMaxRank = 1024;    // R of the generic kernel: 32 accumulators a lane

// One block per token: the latent's norm, the rotation of the shared key part and of every head's rotated query part,
// and the cache write. down: [T, R + Dr]; q: [T, H, Dn + Dr]; q_rot: [T, H, Dr]. The rotation couples channel i with
// i + dims/2 for i < dims/2 (dims <= Dr; channels from dims on pass); table: [positions, dims/2] (cos, sin).
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ down, int64_t ld_down, const T* __restrict__ q, int64_t ld_q,
                                      const float* __restrict__ norm_w, const float2* __restrict__ table,
                                      const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_of_token,
                                      const int32_t* __restrict__ page_table, int P, T* __restrict__ pool,
                                      T* __restrict__ q_rot, int H, int Dn, int Dr, int R, int dims, int page_size,
                                      float eps, int write_kv) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = dims / 2;
    const float2* cs = table != nullptr ? table + (int64_t)pos * half : nullptr;
    pdl_wait();
    if (write_kv) {
        const T* dr = down + (int64_t)t * ld_down;
        float ss = 0.0f;
        for (int c = threadIdx.x; c < R; c += blockDim.x) {
            const float v = to_f32(dr[c]);
            ss += v * v;
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)R + eps);
        const int page = page_table[(int64_t)seq_of_token[t] * P + pos / page_size];
        T* row = pool + ((int64_t)page * page_size + pos % page_size) * (R + Dr);
        for (int c = threadIdx.x; c < R; c += blockDim.x) row[c] = from_f32<T>(to_f32(dr[c]) * inv * norm_w[c]);
        for (int i = threadIdx.x; i < Dr; i += blockDim.x) {
            float v = to_f32(dr[R + i]);
            if (cs != nullptr && i < dims) {
                const bool low = i < half;
                const float2 a = cs[low ? i : i - half];
                const float o = to_f32(dr[R + (low ? i + half : i - half)]);
                v = low ? v * a.x - o * a.y : v * a.x + o * a.y;
            }
            row[R + i] = from_f32<T>(v);
        }
    }
    for (int idx = threadIdx.x; idx < H * Dr; idx += blockDim.x) {
        const int h = idx / Dr, i = idx - h * Dr;
        const T* src = q + (int64_t)t * ld_q + (int64_t)h * (Dn + Dr) + Dn;
        float v = to_f32(src[i]);
        if (cs != nullptr && i < dims) {
            const bool low = i < half;
            const float2 a = cs[low ? i : i - half];
            const float o = to_f32(src[low ? i + half : i - half]);
            v = low ? v * a.x - o * a.y : v * a.x + o * a.y;
        }
        q_rot[((int64_t)t * H + h) * Dr + i] = from_f32<T>(v);
    }
}

// The same for bfloat16 rows in whole 16-byte pieces (R, Dr, Dn multiples of 8, dims a multiple of 16): a thread moves 8
// channels at a time, a rotation's two partner pieces together.
__device__ __forceinline__ void unpack8(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
    uint4 o;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    return o;
}
// dst[i..i+8) and dst[i + half..) from src's two pieces, turned by cs[i..i+8) (cos, sin)
__device__ __forceinline__ void rotate_pieces(const __nv_bfloat16* src, __nv_bfloat16* dst, const float2* cs, int i, int half) {
    float lo[8], hi[8], a[8], b[8];
    unpack8(*reinterpret_cast<const uint4*>(src + i), lo);
    unpack8(*reinterpret_cast<const uint4*>(src + i + half), hi);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const float2 t = cs[i + j];
        a[j] = lo[j] * t.x - hi[j] * t.y;
        b[j] = hi[j] * t.x + lo[j] * t.y;
    }
    *reinterpret_cast<uint4*>(dst + i) = pack8(a);
    *reinterpret_cast<uint4*>(dst + i + half) = pack8(b);
}

__global__ void latent_prepare_vec_kernel(const __nv_bfloat16* __restrict__ down, int64_t ld_down, const __nv_bfloat16* __restrict__ q,
                                          int64_t ld_q, const float* __restrict__ norm_w, const float2* __restrict__ table,
                                          const int32_t* __restrict__ positions, const int32_t* __restrict__ seq_of_token,
                                          const int32_t* __restrict__ page_table, int P, __nv_bfloat16* __restrict__ pool,
                                          __nv_bfloat16* __restrict__ q_rot, int H, int Dn, int Dr, int R, int dims, int page_size,
                                          float eps, int write_kv) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int half = dims / 2;
    const float2* cs = table != nullptr ? table + (int64_t)pos * half : nullptr;
    const int pairs = cs != nullptr ? half / 8 : 0;          // pieces that turn with a partner
    const int plain = Dr / 8 - 2 * pairs;                    // pieces that pass
    pdl_wait();
    if (write_kv) {
        const __nv_bfloat16* dr = down + (int64_t)t * ld_down;
        float v[4][8];
        float ss = 0.0f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = (threadIdx.x + u * blockDim.x) * 8;
            if (c < R) {
                unpack8(*reinterpret_cast<const uint4*>(dr + c), v[u]);
#pragma unroll
                for (int j = 0; j < 8; ++j) ss += v[u][j] * v[u][j];
            }
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)R + eps);
        const int page = page_table[(int64_t)seq_of_token[t] * P + pos / page_size];
        __nv_bfloat16* row = pool + ((int64_t)page * page_size + pos % page_size) * (R + Dr);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = (threadIdx.x + u * blockDim.x) * 8;
            if (c < R) {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[u][j] = v[u][j] * inv * norm_w[c + j];
                *reinterpret_cast<uint4*>(row + c) = pack8(v[u]);
            }
        }
        for (int i = threadIdx.x; i < pairs + plain; i += blockDim.x) {
            if (i < pairs) rotate_pieces(dr + R, row + R, cs, i * 8, half);
            else *reinterpret_cast<uint4*>(row + R + dims + (i - pairs) * 8) = *reinterpret_cast<const uint4*>(dr + R + dims + (i - pairs) * 8);
        }
    }
    const int per_head = pairs + plain;
    for (int idx = threadIdx.x; idx < H * per_head; idx += blockDim.x) {
        const int h = idx / per_head, i = idx - h * per_head;
        const __nv_bfloat16* src = q + (int64_t)t * ld_q + (int64_t)h * (Dn + Dr) + Dn;
        __nv_bfloat16* dst = q_rot + ((int64_t)t * H + h) * Dr;
        if (i < pairs) rotate_pieces(src, dst, cs, i * 8, half);
        else *reinterpret_cast<uint4*>(dst + dims + (i - pairs) * 8) = *reinterpret_cast<const uint4*>(src + dims + (i - pairs) * 8);
    }
}

// One warp per (token, head). Scores with lanes over keys, weighted sums with lanes over channels.
template <typename T>
__global__ void latent_attention_generic_kernel(const T* __restrict__ q_lat, int64_t qs_t, int64_t qs_h,
                                                const T* __restrict__ q_rot, const T* __restrict__ pool,
                                                const int32_t* __restrict__ page_table, int P,
                                                const int32_t* __restrict__ seq_of_token,
                                                const int32_t* __restrict__ positions, const T* __restrict__ gate,
                                                int64_t ld_gate, const float* __restrict__ sink, T* __restrict__ out,
                                                int64_t os_t, int64_t os_h, int Tn, int H, int R, int Dr, int page_size,
                                                float scale, int window) {
    extern __shared__ float q_sm[];   // [warps][R + Dr]
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
    if (item >= (int64_t)Tn * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int pos = positions[t];
    const int32_t* table = page_table + (int64_t)seq_of_token[t] * P;
    const int W = R + Dr;
    float* qs = q_sm + warp * W;
    const T* ql = q_lat + (int64_t)t * qs_t + (int64_t)h * qs_h;
    const T* qr = q_rot + ((int64_t)t * H + h) * Dr;
    for (int d = lane; d < R; d += 32) qs[d] = to_f32(ql[d]) * scale;
    for (int d = lane; d < Dr; d += 32) qs[R + d] = to_f32(qr[d]) * scale;
    __syncwarp();

    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    float m = -INFINITY, l = 0.0f;
    if (sink != nullptr) {      // the denominator starts with exp(sink - m) = 1 at m = sink
        m = sink[h];
        l = 1.0f;
    }
    float acc[kMaxRank / 32];
#pragma unroll
    for (int u = 0; u < kMaxRank / 32; ++u) acc[u] = 0.0f;

    for (int j0 = lo; j0 <= pos; j0 += 32) {
        const int j = j0 + lane;
        float s = -INFINITY;
        if (j <= pos) {
            const int page = table[j / page_size];
            const T* kr = pool + ((int64_t)page * page_size + j % page_size) * W;
            float dot = 0.0f;
            for (int d = 0; d < W; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = j <= pos ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);   // 0 on the first block without a sink (m = -inf)
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int u = 0; u < kMaxRank / 32; ++u) acc[u] *= corr;
        const int cnt = min(32, pos - j0 + 1);
        for (int jj = 0; jj < cnt; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int jk = j0 + jj;
            const int page = table[jk / page_size];
            const T* vr = pool + ((int64_t)page * page_size + jk % page_size) * W;
#pragma unroll
            for (int u = 0; u < kMaxRank / 32; ++u) {
                const int d = lane + 32 * u;
                if (d < R) acc[u] = fmaf(pj, to_f32(vr[d]), acc[u]);
            }
        }
    }
    float g = 1.0f;
    if (gate != nullptr) g = 1.0f / (1.0f + expf(-to_f32(gate[(int64_t)t * ld_gate + h])));
    const float norm = g / l;
    T* orow = out + (int64_t)t * os_t + (int64_t)h * os_h;
#pragma unroll
    for (int u = 0; u < kMaxRank / 32; ++u) {
        const int d = lane + 32 * u;
        if (d < R) orow[d] = from_f32<T>(acc[u] * norm);
    }
}

// out[b][M, N] = x[b][M, K] . w[b][N, K]^T for b < batch, every operand with a row stride and a batch stride: the
// per-head products on either side of the attention (CUDA-core FMAs, sums in an order that depends on K alone).
constexpr int BM = 64, BN = 64, BK = 32;

template <typename T>
__global__ void __launch_bounds__(256)
gemm_batched_kernel(const T* __restrict__ x, int64_t ldx, int64_t sx, const T* __restrict__ w, int64_t ldw, int64_t sw,
                    T* __restrict__ out, int64_t ldo, int64_t so, int M, int N, int K) {
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.z;
    x += (int64_t)b * sx;
    w += (int64_t)b * sw;
    out += (int64_t)b * so;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int idx = threadIdx.x; idx < BM * BK; idx += 256) {
            const int r = idx >> 5, k = idx & 31;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            xs[k][r] = (gm < M && gk < K) ? to_f32(x[(int64_t)gm * ldx + gk]) : 0.0f;
            ws[k][r] = (gn < N && gk < K) ? to_f32(w[(int64_t)gn * ldw + gk]) : 0.0f;
        }
        __syncthreads();
        float part[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) part[i][j] = 0.0f;
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], bb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bb[j] = ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[i][j] = fmaf(a[i], bb[j], part[i][j]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] += part[i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) out[(int64_t)gm * ldo + gn] = from_f32<T>(acc[i][j]);
        }
    }
}

// The same product for few rows (M <= 16: single tokens): a weight-streaming kernel. A block keeps x[b] (M x K, float32)
// in shared memory; each of its warps owns output columns n and walks w[b][n] once, every lane summing its k's for all M
// rows, then the warp reduces (an order that depends on K alone).
template <typename T>
__global__ void __launch_bounds__(256)
gemm_batched_few_rows_kernel(const T* __restrict__ x, int64_t ldx, int64_t sx, const T* __restrict__ w, int64_t ldw, int64_t sw,
                             T* __restrict__ out, int64_t ldo, int64_t so, int M, int N, int K, int cols_per_block) {
    extern __shared__ float xs_rows[];          // [M][K]
    pdl_launch_dependents();
    pdl_wait();
    const int b = blockIdx.y;
    x += (int64_t)b * sx;
    w += (int64_t)b * sw;
    out += (int64_t)b * so;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
#pragma unroll
        for (int m = 0; m < 16; ++m)
            if (m < M) xs_rows[m * K + k] = to_f32(x[(int64_t)m * ldx + k]);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int n_lo = blockIdx.x * cols_per_block, n_hi = min(N, n_lo + cols_per_block);
    for (int n = n_lo + warp; n < n_hi; n += warps) {
        const T* wn = w + (int64_t)n * ldw;
        float acc[16];
#pragma unroll
        for (int m = 0; m < 16; ++m) acc[m] = 0.0f;
        for (int k0 = lane; k0 < K; k0 += 128) {           // four weights in flight a lane
            float wv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) wv[u] = k0 + 32 * u < K ? to_f32(wn[k0 + 32 * u]) : 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int k = k0 + 32 * u;
                if (k < K) {
#pragma unroll
                    for (int m = 0; m < 16; ++m)
                        if (m < M) acc[m] = fmaf(xs_rows[m * K + k], wv[u], acc[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < 16; ++m) {
            if (m < M) {
                const float v = warp_sum(acc[m]);
                if (lane == 0) out[(int64_t)m * ldo + n] = from_f32<T>(v);
            }
        }
    }
}

}  // namespace

XS_API int xs_latent_prepare(const void* down, int64_t ld_down, const void* q, int64_t ld_q, const float* norm_w,
                             const float* table, const int32_t* positions, const int32_t* seq_of_token,
                             const int32_t* page_table, int P, void* pool, void* q_rot, int T, int H, int Dn, int Dr, int R,
                             int dims, int page_size, float eps, int write_kv, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(H > 0 && Dn > 0 && Dr >= 0 && R > 0, "latent_prepare: %d heads of %d + %d, rank %d", H, Dn, Dr, R);
    XS_REQUIRE(dims >= 0 && dims % 2 == 0 && dims <= Dr, "latent_prepare: %d rotated channels of %d", dims, Dr);
    XS_REQUIRE(!write_kv || (pool != nullptr && page_table != nullptr && P > 0), "latent_prepare: no cache to write to");
    const int turned = table != nullptr ? dims : 0;
    if (dtype == XS_BF16 && R % 8 == 0 && R <= 4096 && Dr % 8 == 0 && Dn % 8 == 0 && turned % 16 == 0 && ld_down % 8 == 0 && ld_q % 8 == 0 &&
        (uintptr_t)down % 16 == 0 && (uintptr_t)q % 16 == 0 && (uintptr_t)pool % 16 == 0 && (uintptr_t)q_rot % 16 == 0) {
        xs_launch(latent_prepare_vec_kernel, dim3(T), dim3(128), 0, stream, (const __nv_bfloat16*)down, ld_down,
                  (const __nv_bfloat16*)q, ld_q, norm_w, (const float2*)table, positions, seq_of_token, page_table, P,
                  (__nv_bfloat16*)pool, (__nv_bfloat16*)q_rot, H, Dn, Dr, R, turned, page_size, eps, write_kv);
        XS_LAUNCH_CHECK("latent_prepare");
        return 0;
    }
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(latent_prepare_kernel<TT>, dim3(T), dim3(128), 0, stream, (const TT*)down, ld_down,
                                (const TT*)q, ld_q, norm_w, (const float2*)table, positions, seq_of_token, page_table, P,
                                (TT*)pool, (TT*)q_rot, H, Dn, Dr, R, dims, page_size, eps, write_kv));
    XS_LAUNCH_CHECK("latent_prepare");
    return 0;
}

XS_API int xs_latent_attention_generic(const void* q_lat, int64_t qs_t, int64_t qs_h, const void* q_rot, const void* pool,
                                       const int32_t* page_table, int P, const int32_t* seq_of_token,
                                       const int32_t* positions, const void* gate, int64_t ld_gate, const float* sink,
                                       void* out, int64_t os_t, int64_t os_h, int T, int H, int R, int Dr, int page_size,
                                       float scale, int window, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(H > 0 && R > 0 && R <= kMaxRank && Dr >= 0, "latent attention: %d heads, rank %d (at most %d), %d rotated", H, R,
               kMaxRank, Dr);
    XS_REQUIRE(window >= 0 && page_size > 0 && P > 0, "latent attention: window %d, page size %d, %d pages", window, page_size, P);
    const int warps = 4;
    const int blocks = ceil_div_i((int64_t)T * H, warps);
    const size_t smem = (size_t)warps * (R + Dr) * sizeof(float);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(latent_attention_generic_kernel<TT>, dim3(blocks), dim3(warps * 32), smem, stream,
                                (const TT*)q_lat, qs_t, qs_h, (const TT*)q_rot, (const TT*)pool, page_table, P, seq_of_token,
                                positions, (const TT*)gate, ld_gate, sink, (TT*)out, os_t, os_h, T, H, R, Dr, page_size,
                                scale, window));
    XS_LAUNCH_CHECK("latent_attention_generic");
    return 0;
}

XS_API int xs_gemm_batched(const void* x, int64_t ldx, int64_t sx, const void* w, int64_t ldw, int64_t sw, void* out,
                           int64_t ldo, int64_t so, int batch, int M, int N, int K, int dtype, cudaStream_t stream) {
    if (M == 0 || N == 0 || batch == 0) return 0;
    XS_REQUIRE(batch > 0 && batch <= 65535 && M > 0 && N > 0 && K > 0, "gemm_batched: %d x (%d x %d x %d)", batch, M, N, K);
    XS_REQUIRE(ldx >= K && ldw >= K && ldo >= N, "gemm_batched: a row stride is shorter than its row");
    if (M <= 16 && (size_t)M * K * 4 <= 48 * 1024) {
        const int cols = 8;         // columns a block owns (8 warps, one each)
        XS_DISPATCH_DTYPE(dtype, TT,
                          xs_launch(gemm_batched_few_rows_kernel<TT>, dim3(ceil_div_i(N, cols), batch), dim3(256),
                                    (size_t)M * K * sizeof(float), stream, (const TT*)x, ldx, sx, (const TT*)w, ldw, sw, (TT*)out,
                                    ldo, so, M, N, K, cols));
        XS_LAUNCH_CHECK("gemm_batched (few rows)");
        return 0;
    }
    const dim3 grid(ceil_div_i(N, BN), ceil_div_i(M, BM), batch);
    XS_REQUIRE(grid.y <= 65535, "gemm_batched: %d rows exceed the grid limit", M);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(gemm_batched_kernel<TT>, grid, dim3(256), 0, stream, (const TT*)x, ldx, sx, (const TT*)w,
                                ldw, sw, (TT*)out, ldo, so, M, N, K));
    XS_LAUNCH_CHECK("gemm_batched");
    return 0;
}

// ================================================================================================================
// The same attention on tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 sums), for prompts and for single
// tokens alike. A CTA of eight warps owns 64 query rows of one sequence, a row being a (token, head) pair (token-major, so
// that a tile's rows stand at neighbouring positions and share their keys; in a decode step the rows are the heads of
// the sequence's one token). It walks the visible keys one cache page (64 positions) at a time: the page's rows
// [64, R + Dr] come into shared memory by cp.async; warp (wm, wn) forms the scores of rows 16 wm .. 16 wm + 15 with keys
// 32 wn .. 32 wn + 31 from the query tile in shared memory (ldmatrix), the two warps of a row group exchange their row
// maxima and their probabilities (bfloat16) through shared memory, and each then adds P V for its half of the R value
// columns (the values are the first R columns of the same rows, read with ldmatrix.trans). With `splits` > 1 the
// key pages of a sequence are cut over that many CTAs (single tokens: few rows, long ranges), which leave maximum, sum
// and unnormalised output per row in scratch for a combine kernel. The sink joins the denominator at the very end.
namespace {

__device__ __forceinline__ float log2e() { return 1.4426950408889634f; }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

struct LatentMmaArgs {
    const __nv_bfloat16* q_lat;     // (token, head) rows of R, strides qs_t, qs_h
    int64_t qs_t, qs_h;
    const __nv_bfloat16* q_rot;     // [T, H, Dr]
    const __nv_bfloat16* pool;      // [pages, 64, R + Dr]
    const int32_t* page_table;      // [n_seqs, P]
    int P;
    const int32_t* cu_seqlens;      // [n_seqs + 1]
    const int32_t* kv_lens;         // [n_seqs] keys of each sequence after the step
    const __nv_bfloat16* gate;      // [T, >= H] logits or null
    int64_t ld_gate;
    const float* sink;              // [H] or null
    __nv_bfloat16* out;             // (token, head) rows of R, strides os_t, os_h
    int64_t os_t, os_h;
    float* scratch;                 // splits > 1: [T * H, splits, R + 2] (maximum, sum, output)
    int H, R, Dr, window, splits;
    float scale_log2;               // scale * log2(e)
    int qrows;                      // query rows a CTA owns: 64, or 16 (the kernel of single tokens) when no sequence brings more than 32
};

constexpr int kKeys = 64;      // keys a step: one cache page

template <int RT>     // value columns a warp owns: up to 64 RT (R <= 128 RT)
__global__ void __launch_bounds__(256, 1) latent_attention_mma_kernel(const LatentMmaArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int W = a.R + a.Dr;
    const int WP = (W + 15) & ~15;
    const int ldw = WP + 8;                                  // elements between rows of the query and key tiles
    __nv_bfloat16* sQ = (__nv_bfloat16*)smem;                // [qrows][ldw]
    __nv_bfloat16* sK = sQ + a.qrows * ldw;                  // [64][ldw]
    __nv_bfloat16* sP = sK + kKeys * ldw;                    // [4][16][72]
    float* sRed = (float*)(sP + 4 * 16 * 72);                // [2][64]
    pdl_launch_dependents();
    const int seq = blockIdx.y, split = blockIdx.z;
    const int t0 = a.cu_seqlens[seq], q_len = a.cu_seqlens[seq + 1] - t0, kv_len = a.kv_lens[seq];
    const int m0 = blockIdx.x * a.qrows;
    if (m0 >= q_len * a.H) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wm = warp & 3, wn = warp >> 2;
    const int first_pos = kv_len - q_len;                    // position of the step's first token
    const int tok_first = m0 / a.H, tok_last = min(q_len - 1, (m0 + a.qrows - 1) / a.H);
    const int j_hi = first_pos + tok_last;
    const int j_lo = a.window > 0 ? max(0, first_pos + tok_first - a.window + 1) : 0;
    int b_lo = j_lo / kKeys, b_hi = j_hi / kKeys + 1;        // pages [b_lo, b_hi)
    if (a.splits > 1) {
        const int per = (b_hi - b_lo + a.splits - 1) / a.splits;
        b_lo = b_lo + split * per;
        b_hi = min(b_hi, b_lo + per);
    }
    const int32_t* table = a.page_table + (int64_t)seq * a.P;
    // zero the padding columns of both tiles once (loads never write them)
    for (int idx = threadIdx.x; idx < (a.qrows + kKeys) * (ldw - W); idx += blockDim.x) {
        const int r = idx / (ldw - W), c = W + idx % (ldw - W);
        sQ[r * ldw + c] = __float2bfloat16_rn(0.0f);         // (rows from qrows on in this index space are the key tile's)
    }
    pdl_wait();
    // the query tile: row rho -> token rho / H, head rho % H; rows past the sequence's last are zero
    for (int idx = threadIdx.x; idx < a.qrows * (W / 8); idx += blockDim.x) {
        const int r = idx / (W / 8), c = (idx % (W / 8)) * 8;
        const int rho = m0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (rho < q_len * a.H) {
            const int tok = t0 + rho / a.H, h = rho % a.H;
            v = c < a.R ? *(const uint4*)(a.q_lat + (int64_t)tok * a.qs_t + (int64_t)h * a.qs_h + c)
                        : *(const uint4*)(a.q_rot + ((int64_t)tok * a.H + h) * a.Dr + (c - a.R));
        }
        *(uint4*)(sQ + r * ldw + c) = v;
    }
    // this thread's two rows (of the warp's 16) and their positions
    const int r_lo = wm * 16 + (lane >> 2), r_hi = r_lo + 8;
    const int rho_lo = m0 + r_lo, rho_hi = m0 + r_hi;
    const bool active = wm * 16 < a.qrows && m0 + wm * 16 < q_len * a.H;      // single tokens with few heads fill one row group only
    const int pos_lo = rho_lo < q_len * a.H ? first_pos + rho_lo / a.H : -1;
    const int pos_hi = rho_hi < q_len * a.H ? first_pos + rho_hi / a.H : -1;
    const int min_lo = a.window > 0 ? pos_lo - a.window + 1 : 0, min_hi = a.window > 0 ? pos_hi - a.window + 1 : 0;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
    const int ch = ((a.R / 2 + 15) / 16) * 16;               // value columns of a warp
    const int col0 = wn * ch;
    const int RP = (a.R + 15) & ~15;
    float o[8 * RT][4];
#pragma unroll
    for (int i = 0; i < 8 * RT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const uint32_t sQ_u = (uint32_t)__cvta_generic_to_shared(sQ), sK_u = (uint32_t)__cvta_generic_to_shared(sK);
    const uint32_t sP_u = (uint32_t)__cvta_generic_to_shared(sP + wm * 16 * 72);

    for (int b = b_lo; b < b_hi; ++b) {
        __syncthreads();                                     // the last page's values have been read
        const __nv_bfloat16* page = a.pool + (int64_t)table[b] * kKeys * W;
        for (int idx = threadIdx.x; idx < kKeys * (W / 8); idx += blockDim.x) {
            const int r = idx / (W / 8), c = (idx % (W / 8)) * 8;
            cp_async16(sK_u + (uint32_t)(r * ldw + c) * 2, page + (int64_t)r * W + c);
        }
        cp_async_wait_all();
        __syncthreads();
        // scores of 16 rows x 32 keys
        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
        for (int kk = 0; active && kk < WP; kk += 16) {      // (a row group past the sequence's rows has nothing to add)
            uint32_t qa[4], kb0[4], kb1[4];
            ldmatrix_x4(qa, sQ_u + (uint32_t)((wm * 16 + (lane & 15)) * ldw + kk + (lane >> 4) * 8) * 2);
            const int krow = wn * 32 + (lane & 7) + ((lane >> 4) << 3), kcol = kk + ((lane >> 3) & 1) * 8;
            ldmatrix_x4(kb0, sK_u + (uint32_t)(krow * ldw + kcol) * 2);
            ldmatrix_x4(kb1, sK_u + (uint32_t)((krow + 16) * ldw + kcol) * 2);
            mma_bf16(s[0], qa, kb0[0], kb0[1]);
            mma_bf16(s[1], qa, kb0[2], kb0[3]);
            mma_bf16(s[2], qa, kb1[0], kb1[1]);
            mma_bf16(s[3], qa, kb1[2], kb1[3]);
        }
        // scale, mask, this warp's row maxima
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int j = b * kKeys + wn * 32 + nt * 8 + (lane & 3) * 2 + e;
                s[nt][e] = (j <= pos_lo && j >= min_lo) ? s[nt][e] * a.scale_log2 : -INFINITY;
                s[nt][2 + e] = (j <= pos_hi && j >= min_hi) ? s[nt][2 + e] * a.scale_log2 : -INFINITY;
                mx_lo = fmaxf(mx_lo, s[nt][e]);
                mx_hi = fmaxf(mx_hi, s[nt][2 + e]);
            }
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        if ((lane & 3) == 0) {
            sRed[wn * 64 + r_lo] = mx_lo;
            sRed[wn * 64 + r_hi] = mx_hi;
        }
        __syncthreads();
        const float new_lo = fmaxf(m_lo, fmaxf(sRed[r_lo], sRed[64 + r_lo]));
        const float new_hi = fmaxf(m_hi, fmaxf(sRed[r_hi], sRed[64 + r_hi]));
        const float use_lo = new_lo == -INFINITY ? 0.0f : new_lo, use_hi = new_hi == -INFINITY ? 0.0f : new_hi;
        const float corr_lo = exp2f(m_lo - use_lo), corr_hi = exp2f(m_hi - use_hi);     // 0 while the old maximum is -inf
        m_lo = new_lo;
        m_hi = new_hi;
        l_lo *= corr_lo;
        l_hi *= corr_hi;
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) {
            const float p0 = exp2f(s[nt][0] - use_lo), p1 = exp2f(s[nt][1] - use_lo);
            const float p2 = exp2f(s[nt][2] - use_hi), p3 = exp2f(s[nt][3] - use_hi);
            // the sums run over the probabilities as the products see them (rounded to bfloat16)
            const __nv_bfloat162 v01 = __floats2bfloat162_rn(p0, p1), v23 = __floats2bfloat162_rn(p2, p3);
            l_lo += __bfloat162float(v01.x) + __bfloat162float(v01.y);
            l_hi += __bfloat162float(v23.x) + __bfloat162float(v23.y);
            const int kc = wn * 32 + nt * 8 + (lane & 3) * 2;
            *(__nv_bfloat162*)(sP + (wm * 16 + (lane >> 2)) * 72 + kc) = v01;
            *(__nv_bfloat162*)(sP + (wm * 16 + (lane >> 2) + 8) * 72 + kc) = v23;
        }
#pragma unroll
        for (int i = 0; i < 8 * RT; ++i) {
            o[i][0] *= corr_lo;
            o[i][1] *= corr_lo;
            o[i][2] *= corr_hi;
            o[i][3] *= corr_hi;
        }
        __syncthreads();                                     // both halves of P are written
        // O += P V over this warp's value columns
#pragma unroll
        for (int ks = 0; ks < kKeys / 16; ++ks) {
            if (!active) break;
            uint32_t pa[4];
            ldmatrix_x4(pa, sP_u + (uint32_t)((lane & 15) * 72 + ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int np = 0; np < 4 * RT; ++np) {
                const int c = col0 + np * 16;
                if (np * 16 < ch && c < RP) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, sK_u + (uint32_t)((ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldw + c + (lane >> 4) * 8) * 2);
                    mma_bf16(o[2 * np], pa, vb[0], vb[1]);
                    mma_bf16(o[2 * np + 1], pa, vb[2], vb[3]);
                }
            }
        }
    }
    // row sums: over the quad, then over the two warps of the row group
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    __syncthreads();
    if ((lane & 3) == 0) {
        sRed[wn * 64 + r_lo] = l_lo;
        sRed[wn * 64 + r_hi] = l_hi;
    }
    __syncthreads();
    l_lo = sRed[r_lo] + sRed[64 + r_lo];
    l_hi = sRed[r_hi] + sRed[64 + r_hi];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int rho = half ? rho_hi : rho_lo;
        if (rho >= q_len * a.H) continue;
        const int tok = t0 + rho / a.H, h = rho % a.H;
        const float m = half ? m_hi : m_lo;
        float l = half ? l_hi : l_lo;
        if (a.splits > 1) {
            float* dst = a.scratch + (((int64_t)tok * a.H + h) * a.splits + split) * (a.R + 2);
            if (wn == 0 && (lane & 3) == 0) {
                dst[0] = m;
                dst[1] = l;
            }
#pragma unroll
            for (int i = 0; i < 8 * RT; ++i) {
                const int c = col0 + i * 8 + (lane & 3) * 2;
                if (i * 8 < ch && c < a.R) {
                    dst[2 + c] = o[i][2 * half];
                    dst[2 + c + 1] = o[i][2 * half + 1];
                }
            }
            continue;
        }
        if (a.sink != nullptr) l += exp2f(a.sink[h] * log2e() - m);
        float norm = 1.0f / l;
        if (a.gate != nullptr) norm *= 1.0f / (1.0f + expf(-__bfloat162float(a.gate[(int64_t)tok * a.ld_gate + h])));
        __nv_bfloat16* dst = a.out + (int64_t)tok * a.os_t + (int64_t)h * a.os_h;
#pragma unroll
        for (int i = 0; i < 8 * RT; ++i) {
            const int c = col0 + i * 8 + (lane & 3) * 2;
            if (i * 8 < ch && c < a.R)
                *(__nv_bfloat162*)(dst + c) = __floats2bfloat162_rn(o[i][2 * half] * norm, o[i][2 * half + 1] * norm);
        }
    }
}

// Single tokens (at most 32 query rows a sequence): 16 rows a CTA, all eight warps on them. Warp w forms the scores of
// keys 8 w .. 8 w + 7 of the page (two accumulators over alternate k steps), the warps exchange row maxima and the
// probabilities through shared memory, and warp w then adds P V for its eighth of the value columns. A CTA holds 103 KB
// of shared memory at 576 channels a row, so two share an SM and a sequence's pages are cut over twice as many CTAs.
__global__ void __launch_bounds__(256, 2) latent_attention_mma16_kernel(const LatentMmaArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int W = a.R + a.Dr;
    const int WP = (W + 15) & ~15;
    const int ldw = WP + 8;
    __nv_bfloat16* sQ = (__nv_bfloat16*)smem;                // [16][ldw]
    __nv_bfloat16* sK = sQ + 16 * ldw;                       // [64][ldw]
    __nv_bfloat16* sP = sK + kKeys * ldw;                    // [16][72]
    float* sRed = (float*)(sP + 16 * 72);                    // [8][16]
    pdl_launch_dependents();
    const int seq = blockIdx.y, split = blockIdx.z;
    const int t0 = a.cu_seqlens[seq], q_len = a.cu_seqlens[seq + 1] - t0, kv_len = a.kv_lens[seq];
    const int m0 = blockIdx.x * 16;
    if (m0 >= q_len * a.H) return;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int first_pos = kv_len - q_len;
    const int tok_first = m0 / a.H, tok_last = min(q_len - 1, (m0 + 15) / a.H);
    const int j_hi = first_pos + tok_last;
    const int j_lo = a.window > 0 ? max(0, first_pos + tok_first - a.window + 1) : 0;
    int b_lo = j_lo / kKeys, b_hi = j_hi / kKeys + 1;
    if (a.splits > 1) {
        const int per = (b_hi - b_lo + a.splits - 1) / a.splits;
        b_lo = b_lo + split * per;
        b_hi = min(b_hi, b_lo + per);
    }
    const int32_t* table = a.page_table + (int64_t)seq * a.P;
    for (int idx = threadIdx.x; idx < (16 + kKeys) * (ldw - W); idx += blockDim.x) {
        const int r = idx / (ldw - W), c = W + idx % (ldw - W);
        sQ[r * ldw + c] = __float2bfloat16_rn(0.0f);
    }
    pdl_wait();
    for (int idx = threadIdx.x; idx < 16 * (W / 8); idx += blockDim.x) {
        const int r = idx / (W / 8), c = (idx % (W / 8)) * 8;
        const int rho = m0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (rho < q_len * a.H) {
            const int tok = t0 + rho / a.H, h = rho % a.H;
            v = c < a.R ? *(const uint4*)(a.q_lat + (int64_t)tok * a.qs_t + (int64_t)h * a.qs_h + c)
                        : *(const uint4*)(a.q_rot + ((int64_t)tok * a.H + h) * a.Dr + (c - a.R));
        }
        *(uint4*)(sQ + r * ldw + c) = v;
    }
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    const int rho_lo = m0 + r_lo, rho_hi = m0 + r_hi;
    const int pos_lo = rho_lo < q_len * a.H ? first_pos + rho_lo / a.H : -1;
    const int pos_hi = rho_hi < q_len * a.H ? first_pos + rho_hi / a.H : -1;
    const int min_lo = a.window > 0 ? pos_lo - a.window + 1 : 0, min_hi = a.window > 0 ? pos_hi - a.window + 1 : 0;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.0f, l_hi = 0.0f;
    const int cw = (((a.R + 7) / 8 + 15) / 16) * 16;         // value columns of a warp
    const int col0 = w * cw;
    const int RP = (a.R + 15) & ~15;
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    const uint32_t sQ_u = (uint32_t)__cvta_generic_to_shared(sQ), sK_u = (uint32_t)__cvta_generic_to_shared(sK);
    const uint32_t sP_u = (uint32_t)__cvta_generic_to_shared(sP);

    for (int b = b_lo; b < b_hi; ++b) {
        __syncthreads();
        const __nv_bfloat16* page = a.pool + (int64_t)table[b] * kKeys * W;
        for (int r = w; r < kKeys; r += 8)                   // a warp a row: no division on the way
            for (int c = lane * 8; c < W; c += 256) cp_async16(sK_u + (uint32_t)(r * ldw + c) * 2, page + (int64_t)r * W + c);
        cp_async_wait_all();
        __syncthreads();
        float s0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, s1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int kk = 0; kk < WP; kk += 32) {
            uint32_t qa[4], kb[4];
            ldmatrix_x4(kb, sK_u + (uint32_t)((w * 8 + (lane & 7)) * ldw + kk + (lane >> 3) * 8) * 2);
            ldmatrix_x4(qa, sQ_u + (uint32_t)((lane & 15) * ldw + kk + (lane >> 4) * 8) * 2);
            mma_bf16(s0, qa, kb[0], kb[1]);
            if (kk + 16 < WP) {
                ldmatrix_x4(qa, sQ_u + (uint32_t)((lane & 15) * ldw + kk + 16 + (lane >> 4) * 8) * 2);
                mma_bf16(s1, qa, kb[2], kb[3]);
            }
        }
        float sc[4];
        float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int j = b * kKeys + w * 8 + (lane & 3) * 2 + e;
            sc[e] = (j <= pos_lo && j >= min_lo) ? (s0[e] + s1[e]) * a.scale_log2 : -INFINITY;
            sc[2 + e] = (j <= pos_hi && j >= min_hi) ? (s0[2 + e] + s1[2 + e]) * a.scale_log2 : -INFINITY;
            mx_lo = fmaxf(mx_lo, sc[e]);
            mx_hi = fmaxf(mx_hi, sc[2 + e]);
        }
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
        mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
        mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
        if ((lane & 3) == 0) {
            sRed[w * 16 + r_lo] = mx_lo;
            sRed[w * 16 + r_hi] = mx_hi;
        }
        __syncthreads();
        float new_lo = m_lo, new_hi = m_hi;
#pragma unroll
        for (int x = 0; x < 8; ++x) {
            new_lo = fmaxf(new_lo, sRed[x * 16 + r_lo]);
            new_hi = fmaxf(new_hi, sRed[x * 16 + r_hi]);
        }
        const float use_lo = new_lo == -INFINITY ? 0.0f : new_lo, use_hi = new_hi == -INFINITY ? 0.0f : new_hi;
        const float corr_lo = exp2f(m_lo - use_lo), corr_hi = exp2f(m_hi - use_hi);
        m_lo = new_lo;
        m_hi = new_hi;
        {
            const __nv_bfloat162 v01 = __floats2bfloat162_rn(exp2f(sc[0] - use_lo), exp2f(sc[1] - use_lo));
            const __nv_bfloat162 v23 = __floats2bfloat162_rn(exp2f(sc[2] - use_hi), exp2f(sc[3] - use_hi));
            l_lo = l_lo * corr_lo + __bfloat162float(v01.x) + __bfloat162float(v01.y);
            l_hi = l_hi * corr_hi + __bfloat162float(v23.x) + __bfloat162float(v23.y);
            const int kc = w * 8 + (lane & 3) * 2;
            *(__nv_bfloat162*)(sP + r_lo * 72 + kc) = v01;
            *(__nv_bfloat162*)(sP + r_hi * 72 + kc) = v23;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o[i][0] *= corr_lo;
            o[i][1] *= corr_lo;
            o[i][2] *= corr_hi;
            o[i][3] *= corr_hi;
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < kKeys / 16; ++ks) {
            uint32_t pa[4];
            ldmatrix_x4(pa, sP_u + (uint32_t)((lane & 15) * 72 + ks * 16 + (lane >> 4) * 8) * 2);
#pragma unroll
            for (int np = 0; np < 4; ++np) {
                const int c = col0 + np * 16;
                if (np * 16 < cw && c < RP) {
                    uint32_t vb[4];
                    ldmatrix_x4_trans(vb, sK_u + (uint32_t)((ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ldw + c + (lane >> 4) * 8) * 2);
                    mma_bf16(o[2 * np], pa, vb[0], vb[1]);
                    mma_bf16(o[2 * np + 1], pa, vb[2], vb[3]);
                }
            }
        }
    }
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    __syncthreads();
    if ((lane & 3) == 0) {
        sRed[w * 16 + r_lo] = l_lo;
        sRed[w * 16 + r_hi] = l_hi;
    }
    __syncthreads();
    l_lo = l_hi = 0.0f;
#pragma unroll
    for (int x = 0; x < 8; ++x) {
        l_lo += sRed[x * 16 + r_lo];
        l_hi += sRed[x * 16 + r_hi];
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int rho = half ? rho_hi : rho_lo;
        if (rho >= q_len * a.H) continue;
        const int tok = t0 + rho / a.H, h = rho % a.H;
        const float m = half ? m_hi : m_lo;
        float l = half ? l_hi : l_lo;
        if (a.splits > 1) {
            float* dst = a.scratch + (((int64_t)tok * a.H + h) * a.splits + split) * (a.R + 2);
            if (w == 0 && (lane & 3) == 0) {
                dst[0] = m;
                dst[1] = l;
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int c = col0 + i * 8 + (lane & 3) * 2;
                if (i * 8 < cw && c < a.R) {
                    dst[2 + c] = o[i][2 * half];
                    dst[2 + c + 1] = o[i][2 * half + 1];
                }
            }
            continue;
        }
        if (a.sink != nullptr) l += exp2f(a.sink[h] * log2e() - m);
        float norm = 1.0f / l;
        if (a.gate != nullptr) norm *= 1.0f / (1.0f + expf(-__bfloat162float(a.gate[(int64_t)tok * a.ld_gate + h])));
        __nv_bfloat16* dst = a.out + (int64_t)tok * a.os_t + (int64_t)h * a.os_h;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int c = col0 + i * 8 + (lane & 3) * 2;
            if (i * 8 < cw && c < a.R)
                *(__nv_bfloat162*)(dst + c) = __floats2bfloat162_rn(o[i][2 * half] * norm, o[i][2 * half + 1] * norm);
        }
    }
}

// One block per (token, head): the splits' maxima, sums and outputs into the final row.
__global__ void latent_attention_combine_kernel(const float* __restrict__ scratch, const float* __restrict__ sink,
                                                const __nv_bfloat16* __restrict__ gate, int64_t ld_gate,
                                                __nv_bfloat16* __restrict__ out, int64_t os_t, int64_t os_h, int H, int R,
                                                int splits) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float weight[64];      // of each split: 2^(its maximum - the row's), then divided by the row's sum
    __shared__ float norm_sm;
    const int tok = blockIdx.x / H, h = blockIdx.x % H;
    const float* src = scratch + (int64_t)blockIdx.x * splits * (R + 2);
    if (threadIdx.x < 32) {           // splits <= 64: two per lane, all loads in flight at once
        const int s0 = threadIdx.x, s1 = threadIdx.x + 32;
        const float m0 = s0 < splits ? src[(int64_t)s0 * (R + 2)] : -INFINITY, m1 = s1 < splits ? src[(int64_t)s1 * (R + 2)] : -INFINITY;
        const float l0 = s0 < splits ? src[(int64_t)s0 * (R + 2) + 1] : 0.0f, l1 = s1 < splits ? src[(int64_t)s1 * (R + 2) + 1] : 0.0f;
        const float M = warp_max(fmaxf(m0, m1));
        const float w0 = exp2f(m0 - M), w1 = exp2f(m1 - M);
        float L = warp_sum(l0 * w0 + l1 * w1);
        if (sink != nullptr) L += exp2f(sink[h] * log2e() - M);
        weight[s0] = w0;
        weight[s1] = w1;
        if (threadIdx.x == 0) {
            float norm = 1.0f / L;
            if (gate != nullptr) norm *= 1.0f / (1.0f + expf(-__bfloat162float(gate[(int64_t)tok * ld_gate + h])));
            norm_sm = norm;
        }
    }
    __syncthreads();
    const float norm = norm_sm;
    __nv_bfloat16* dst = out + (int64_t)tok * os_t + (int64_t)h * os_h;
    for (int c = threadIdx.x; c < R; c += blockDim.x) {
        float v = 0.0f;
#pragma unroll 8
        for (int s = 0; s < splits; ++s) v = fmaf(src[(int64_t)s * (R + 2) + 2 + c], weight[s], v);
        dst[c] = __float2bfloat16_rn(v * norm);
    }
}

}  // namespace

XS_API int xs_latent_attention_mma_supports(int R, int Dr, int page_size) {
    return R >= 16 && R % 8 == 0 && Dr >= 0 && Dr % 8 == 0 && R <= 512 && page_size == 64 &&
           (size_t)(2 * 64 * (((R + Dr + 15) & ~15) + 8) * 2 + 4 * 16 * 72 * 2 + 2 * 64 * 4) <= 227 * 1024;
}

// Query rows a CTA owns, and how many such CTAs fit an SM (what the key splits of single tokens are sized by).
XS_API int xs_latent_attention_mma_rows(int max_q_len, int H) { return (int64_t)max_q_len * H <= 32 ? 16 : 64; }
XS_API int xs_latent_attention_mma_ctas_per_sm(int max_q_len, int H, int R, int Dr) {
    const int WP = (R + Dr + 15) & ~15;
    const size_t smem = (size_t)(xs_latent_attention_mma_rows(max_q_len, H) + 64) * (WP + 8) * 2 + 4 * 16 * 72 * 2 + 2 * 64 * 4 + 1024;
    const int fit = (int)((227 * 1024) / smem);
    return fit < 1 ? 1 : fit > 2 ? 2 : fit;
}

XS_API int64_t xs_latent_attention_mma_scratch_bytes(int64_t rows, int R, int splits) {
    return splits > 1 ? rows * splits * (R + 2) * (int64_t)sizeof(float) : 0;
}

// max_q_len: the most tokens a sequence brings (the grid's bound); scratch for splits > 1.
XS_API int xs_latent_attention_mma(const void* q_lat, int64_t qs_t, int64_t qs_h, const void* q_rot, const void* pool,
                                   const int32_t* page_table, int P, const int32_t* cu_seqlens, const int32_t* kv_lens,
                                   const void* gate, int64_t ld_gate, const float* sink, void* out, int64_t os_t, int64_t os_h,
                                   void* scratch, int64_t scratch_bytes, int T, int n_seqs, int max_q_len, int H, int R, int Dr,
                                   int page_size, float scale, int window, int splits, cudaStream_t stream) {
    if (T == 0 || n_seqs == 0) return 0;
    XS_REQUIRE(xs_latent_attention_mma_supports(R, Dr, page_size), "latent attention (mma): rank %d, %d rotated, pages of %d", R, Dr,
               page_size);
    XS_REQUIRE(H > 0 && window >= 0 && splits >= 1 && splits <= 65535 && n_seqs <= 65535 && max_q_len > 0,
               "latent attention (mma): %d heads, window %d, %d splits, %d sequences", H, window, splits, n_seqs);
    XS_REQUIRE(qs_t % 8 == 0 && qs_h % 8 == 0 && os_t % 2 == 0 && os_h % 2 == 0 && (uintptr_t)q_lat % 16 == 0 &&
                   (uintptr_t)q_rot % 16 == 0 && (uintptr_t)pool % 16 == 0 && (uintptr_t)out % 4 == 0,
               "latent attention (mma): operands are not aligned");
    XS_REQUIRE(splits == 1 || (scratch != nullptr && scratch_bytes >= xs_latent_attention_mma_scratch_bytes((int64_t)T * H, R, splits)),
               "latent attention (mma): %d splits need %lld bytes of scratch", splits,
               (long long)xs_latent_attention_mma_scratch_bytes((int64_t)T * H, R, splits));
    LatentMmaArgs a = {(const __nv_bfloat16*)q_lat, qs_t, qs_h, (const __nv_bfloat16*)q_rot, (const __nv_bfloat16*)pool,
                       page_table, P, cu_seqlens, kv_lens, (const __nv_bfloat16*)gate, ld_gate, sink, (__nv_bfloat16*)out,
                       os_t, os_h, (float*)scratch, H, R, Dr, window, splits, scale * 1.4426950408889634f,
                       xs_latent_attention_mma_rows(max_q_len, H)};
    const int WP = (R + Dr + 15) & ~15;
    const size_t smem = (size_t)(a.qrows + 64) * (WP + 8) * 2 + 4 * 16 * 72 * 2 + 2 * 64 * 4;
    const dim3 grid(ceil_div_i((int64_t)max_q_len * H, a.qrows), n_seqs, splits);
#define XS_GO(RT)                                                                                                       \
    do {                                                                                                                \
        static bool opted = false;                                                                                      \
        if (!opted) {                                                                                                   \
            cudaFuncSetAttribute(latent_attention_mma_kernel<RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); \
            opted = true;                                                                                               \
        }                                                                                                               \
        xs_launch(latent_attention_mma_kernel<RT>, grid, dim3(256), smem, stream, a);                                   \
    } while (0)
    if (a.qrows == 16) {
        static bool opted16 = false;
        if (!opted16) {
            cudaFuncSetAttribute(latent_attention_mma16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
            opted16 = true;
        }
        const size_t smem16 = (size_t)(16 + 64) * (WP + 8) * 2 + 16 * 72 * 2 + 8 * 16 * 4;
        xs_launch(latent_attention_mma16_kernel, grid, dim3(256), smem16, stream, a);
    } else if (R <= 128) XS_GO(1);
    else if (R <= 256) XS_GO(2);
    else XS_GO(4);
#undef XS_GO
    XS_LAUNCH_CHECK("latent_attention_mma");
    if (splits > 1) {
        xs_launch(latent_attention_combine_kernel, dim3(T * H), dim3(128), 0, stream, (const float*)scratch, sink,
                  (const __nv_bfloat16*)gate, ld_gate, (__nv_bfloat16*)out, os_t, os_h, H, R, splits);
        XS_LAUNCH_CHECK("latent_attention_combine");
    }
    return 0;
}
