// Pieces of a layer's frame that are neither a product nor a mixer:
//
//   embed_pos          h[t] = table[id[t]] * scale + rows[position[t]]: a token table plus a learned row per position
//   causal_conv        y[t, c] = (x[t, c] if residual) + act(sum_j taps[c, j] x[t - (n - 1) + j, c]) over a sequence's earlier
//                      tokens, the inputs before a step coming from the sequence's state [n - 1, C], which then moves on
//   gated_add          h[t, c] += branch[t, c] * sigmoid(logit[t, c] + bias[c]): a branch joins the float32 stream through
//                      a gate
//   depth_average      out[t, c] = sum_j coef[j] * hist[j, t, c]: what a layer hands on as a weighted sum of the embedding's
//                      and every earlier layer's results
//   rmsnorm_accumulate acc[t, :] (+)= scale * x[t, :] / sqrt(mean(x[t, :]^2) + eps) * w: branches that run side by side are
//                      normed and summed in float32
//   side_gate          x[t, j] = gelu_tanh(x[t, j]) * table[id[t], off + j]: a slice of a second token table, gated
//   rmsnorm_rows       y[t, :n] = x[t, :n] / sqrt(mean(x[t, :n]^2) + eps) * w over columns of a wider matrix
//   sigmoid_mul        o[t, c] *= sigmoid(g[t, c])
//   cast_rows          dst[t, :n] = src[t, :n] (float32 to the activation type) into columns of a wider matrix
//
// All sums are float32 in a fixed order per element, whatever else is in the batch.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kMaxTaps = 16;
constexpr int kMaxTerms = 512;

template <typename T>
__global__ void embed_pos_kernel(const T* __restrict__ table, const T* __restrict__ rows, const int32_t* __restrict__ ids,
                                 const int32_t* __restrict__ positions, float* __restrict__ h, int H, float scale) {
    pdl_launch_dependents();
    const int t = blockIdx.x;
    const int64_t id = ids[t], pos = positions[t];
    pdl_wait();
    const T* a = table + id * H;
    const T* b = rows + pos * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) h[(int64_t)t * H + c] = fmaf(to_f32(a[c]), scale, to_f32(b[c]));
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return z / (1.0f + expf(-1.5957691216057308f * (z + 0.044715f * z * z * z)));     // 0.5 (1 + tanh(a)) = 1 / (1 + exp(-2 a))
}

// x[t, j] = gelu_tanh(x[t, j]) * table[id[t], off + j] in place: the gate of a token-side input times the token's slice of
// the second table. x: [T, d] rows `ldx` apart; table: [vocab, ld_table] of x's element type.
template <typename T>
__global__ void side_gate_kernel(T* __restrict__ x, int64_t ldx, const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 int64_t ld_table, int off, int64_t total, int d) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / d;
        const int j = (int)(i - t * d);
        const float e = to_f32(table[(int64_t)ids[t] * ld_table + off + j]);
        x[t * ldx + j] = from_f32<T>(gelu_tanh_f(to_f32(x[t * ldx + j])) * e);
    }
}

template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ x, int64_t ldx, const float* __restrict__ w, T* __restrict__ y,
                                    int64_t ldy, int n, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const T* xr = x + (int64_t)blockIdx.x * ldx;
    T* yr = y + (int64_t)blockIdx.x * ldy;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
        const float v = to_f32(xr[c]);
        ss = fmaf(v, v, ss);
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) yr[c] = from_f32<T>(to_f32(xr[c]) * inv * w[c]);
}

template <typename T>
__global__ void sigmoid_mul_kernel(T* __restrict__ o, int64_t ldo, const T* __restrict__ g, int64_t ldg, int64_t total, int n) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / n;
        const int c = (int)(i - t * n);
        const float gv = to_f32(g[t * ldg + c]);
        o[t * ldo + c] = from_f32<T>(to_f32(o[t * ldo + c]) / (1.0f + expf(-gv)));
    }
}

template <typename T>
__global__ void cast_rows_kernel(const float* __restrict__ src, int64_t lds, T* __restrict__ dst, int64_t ldd, int64_t total, int n) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / n;
        const int c = (int)(i - t * n);
        dst[t * ldd + c] = from_f32<T>(src[t * lds + c]);
    }
}

// SiLU of a filter's sum. In front of a rounding to bfloat16 the fast exponential and division do (a few units in the last
// place of float32); float32 activations take the exact ones.
template <typename T>
__device__ __forceinline__ float silu_f(float v) {
    if constexpr (sizeof(T) == 4) return v / (1.0f + expf(-v));
    else return __fdividef(v, 1.0f + __expf(-v));
}

template <typename T>
__global__ void causal_conv_kernel(const T* __restrict__ x, int64_t ldx, const float* __restrict__ taps_w,
                                   T* __restrict__ state, const int32_t* __restrict__ seq_of_token,
                                   const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                                   T* __restrict__ out, int64_t ldo, int C, int taps, int act, int residual, int move_state) {
    pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (c >= C) return;
    float w[kMaxTaps];                              // by how far back the tap looks (static indices: registers)
#pragma unroll
    for (int b = 0; b < kMaxTaps; ++b) w[b] = b < taps ? taps_w[(int64_t)c * taps + (taps - 1 - b)] : 0.0f;
    const int seq = seq_of_token[t];
    const int local = t - cu_seqlens[seq];
    const int64_t slot = slots[seq];
    pdl_wait();
    float acc = 0.0f, cur = 0.0f;
#pragma unroll
    for (int back = kMaxTaps - 1; back >= 0; --back) {
        if (back < taps) {
            float v;
            if (local - back >= 0)
                v = to_f32(x[(int64_t)(t - back) * ldx + c]);
            else      // state row n - 1 - j holds the input j positions before the step (j = back - local)
                v = to_f32(state[(slot * (taps - 1) + (taps - 1 - (back - local))) * C + c]);
            if (back == 0) cur = v;
            acc = fmaf(w[back], v, acc);
            // A step of one token a sequence moves the state on here: the input `back` positions before this token is
            // back + 1 before the next, a row that this thread has read already (it walks from the far end).
            if (move_state && back < taps - 1) state[(slot * (taps - 1) + (taps - 2 - back)) * C + c] = from_f32<T>(v);
        }
    }
    if (act == 1) acc = silu_f<T>(acc);
    if (residual) acc = __fadd_rn(acc, cur);          // (never fused with the activation's last product: the same bits in both kernels)
    out[(int64_t)t * ldo + c] = from_f32<T>(acc);
}

// four channels at a time, held as floats
template <typename T>
struct ConvVec;
template <>
struct ConvVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <>
struct ConvVec<__nv_bfloat16> {
    static constexpr int N = 4;                    // (eight channels a thread cost the registers of two more CTAs an SM)
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
        uint2 r;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 2; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint2*>(p) = r;
    }
};

constexpr int kTileTaps = 8;     // the tiled kernel's filters have at most this many taps
constexpr int kTileTokens = 8;   // tokens a thread

// The same sums in the same order as causal_conv_kernel, for long steps: a thread takes four channels and kTileTokens
// tokens, loads the rows it needs once (all loads in flight together) and keeps them in registers, with its channels' taps
// (contiguous in memory: 16 bytes a load). Only a sequence's first TAPS - 1 tokens of a step go to its state.
template <typename T, int TAPS>
__global__ void __launch_bounds__(128) causal_conv_tile_kernel(const T* __restrict__ x, int64_t ldx, const float* __restrict__ taps_w,
                                                               const T* __restrict__ state, const int32_t* __restrict__ seq_of_token,
                                                               const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                                                               T* __restrict__ out, int64_t ldo, int C, int act, int residual,
                                                               int n_tokens) {
    constexpr int V = ConvVec<T>::N, ROWS = kTileTokens + TAPS - 1;
    pdl_launch_dependents();
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * V;
    const int t0 = blockIdx.x * kTileTokens;
    if (c >= C) return;
    float w[V * TAPS];                              // channel v's tap k at [v * TAPS + k]
    {
        const float4* w4 = reinterpret_cast<const float4*>(taps_w + (int64_t)c * TAPS);
#pragma unroll
        for (int i = 0; i < V * TAPS / 4; ++i) {
            const float4 r = w4[i];
            w[4 * i] = r.x; w[4 * i + 1] = r.y; w[4 * i + 2] = r.z; w[4 * i + 3] = r.w;
        }
    }
    // every token's place in its sequence, all loads together (a chain of two loads a token otherwise)
    int seq[kTileTokens], local[kTileTokens];
#pragma unroll
    for (int i = 0; i < kTileTokens; ++i) seq[i] = seq_of_token[min(t0 + i, n_tokens - 1)];
#pragma unroll
    for (int i = 0; i < kTileTokens; ++i) local[i] = min(t0 + i, n_tokens - 1) - cu_seqlens[seq[i]];
    pdl_wait();
    float rows[ROWS][V];                            // row r is token t0 - (TAPS - 1) + r
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int t = t0 - (TAPS - 1) + r;
        if (t >= 0 && t < n_tokens)
            ConvVec<T>::load(x + (int64_t)t * ldx + c, rows[r]);
        else {
#pragma unroll
            for (int v = 0; v < V; ++v) rows[r][v] = 0.0f;
        }
    }
#pragma unroll
    for (int i = 0; i < kTileTokens; ++i) {
        const int t = t0 + i;
        if (t < n_tokens) {
            float acc[V];
#pragma unroll
            for (int v = 0; v < V; ++v) acc[v] = 0.0f;
#pragma unroll
            for (int back = TAPS - 1; back >= 0; --back) {
                if (local[i] - back >= 0) {
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[v] = fmaf(w[v * TAPS + TAPS - 1 - back], rows[i + TAPS - 1 - back][v], acc[v]);
                } else {
                    float sv[V];
                    ConvVec<T>::load(state + ((int64_t)slots[seq[i]] * (TAPS - 1) + (TAPS - 1 - (back - local[i]))) * C + c, sv);
#pragma unroll
                    for (int v = 0; v < V; ++v) acc[v] = fmaf(w[v * TAPS + TAPS - 1 - back], sv[v], acc[v]);
                }
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                if (act == 1) acc[v] = silu_f<T>(acc[v]);
                if (residual) acc[v] = __fadd_rn(acc[v], rows[i + TAPS - 1][v]);
            }
            ConvVec<T>::store(out + (int64_t)t * ldo + c, acc);
        }
    }
}

// After the convolution: a sequence's state becomes its last n - 1 inputs (the step's, and the old state's where the step
// brought fewer).
template <typename T>
__global__ void causal_conv_state_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ state,
                                         const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots, int C,
                                         int taps) {
    pdl_launch_dependents();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    const int seq = blockIdx.x;
    if (c >= C) return;
    const int t0 = cu_seqlens[seq], n = cu_seqlens[seq + 1] - t0;
    const int64_t slot = slots[seq];
    pdl_wait();
    if (n <= 0) return;
    T* st = state + slot * (taps - 1) * C + c;
    T keep[kMaxTaps];
    for (int j = 0; j < taps - 1; ++j) {
        const int local = n - (taps - 1) + j;       // the input that row j holds after the step
        keep[j] = local >= 0 ? x[(int64_t)(t0 + local) * ldx + c] : st[(int64_t)(j + n) * C];
    }
    for (int j = 0; j < taps - 1; ++j) st[(int64_t)j * C] = keep[j];
}

template <typename TB>
__global__ void gated_add_kernel(float* __restrict__ h, const TB* __restrict__ branch, const float* __restrict__ logits,
                                 int64_t ld_logits, const float* __restrict__ bias, int64_t total, int W) {
    pdl_launch_dependents();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const int64_t t = i / W;
    const int c = (int)(i - t * W);
    const float z = logits[t * ld_logits + c] + (bias != nullptr ? bias[c] : 0.0f);
    h[i] += to_f32(branch[i]) / (1.0f + expf(-z));
}

__global__ void depth_average_kernel(const float* __restrict__ hist, int64_t plane, const float* __restrict__ coef, int terms,
                                     float* __restrict__ out, int64_t total) {
    __shared__ float cs[kMaxTerms];
    pdl_launch_dependents();
    for (int j = threadIdx.x; j < terms; j += blockDim.x) cs[j] = coef[j];
    __syncthreads();
    pdl_wait();
    const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= total) return;
    if (i + 4 <= total && (plane & 3) == 0) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < terms; ++j) {
            const float4 v = *reinterpret_cast<const float4*>(hist + (int64_t)j * plane + i);
            acc.x = fmaf(cs[j], v.x, acc.x); acc.y = fmaf(cs[j], v.y, acc.y);
            acc.z = fmaf(cs[j], v.z, acc.z); acc.w = fmaf(cs[j], v.w, acc.w);
        }
        *reinterpret_cast<float4*>(out + i) = acc;
        return;
    }
    for (int64_t e = i; e < total && e < i + 4; ++e) {
        float acc = 0.0f;
        for (int j = 0; j < terms; ++j) acc = fmaf(cs[j], hist[(int64_t)j * plane + e], acc);
        out[e] = acc;
    }
}

// One block a row; the row's sum of squares in a fixed order (block_sum), then acc (+)= scale * x / rms * w.
template <typename T>
__global__ void rmsnorm_accumulate_kernel(const T* __restrict__ x, const float* __restrict__ w, float* __restrict__ acc, int W,
                                          float eps, float scale, int add) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const T* xr = x + (int64_t)blockIdx.x * W;
    float* ar = acc + (int64_t)blockIdx.x * W;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = to_f32(xr[c]);
        ss = fmaf(v, v, ss);
    }
    const float inv = scale / sqrtf(block_sum(ss, scratch) / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = to_f32(xr[c]) * inv * w[c];
        ar[c] = add ? ar[c] + v : v;
    }
}


// The same three for bfloat16 rows in whole 16-byte pieces (n and the row strides multiples of 8, aligned pointers): 8 elements a
// thread and load.
__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float (&v)[8]) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h2[j]);
        v[2 * j] = f.x;
        v[2 * j + 1] = f.y;
    }
}
__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
    uint4 o;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) h2[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
    return o;
}

// One block a row, the row held in registers (up to 4 pieces a thread: n <= 32 * blockDim.x).
__global__ void rmsnorm_rows_vec_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx, const float* __restrict__ w,
                                        __nv_bfloat16* __restrict__ y, int64_t ldy, int n, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const __nv_bfloat16* xr = x + (int64_t)blockIdx.x * ldx;
    __nv_bfloat16* yr = y + (int64_t)blockIdx.x * ldy;
    float v[4][8];
    float ss = 0.0f;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int c = (threadIdx.x + u * blockDim.x) * 8;
        if (c < n) {
            unpack_bf16x8(*reinterpret_cast<const uint4*>(xr + c), v[u]);
#pragma unroll
            for (int j = 0; j < 8; ++j) ss = fmaf(v[u][j], v[u][j], ss);
        }
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)n + eps);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const int c = (threadIdx.x + u * blockDim.x) * 8;
        if (c < n) {
            const float4 w0 = *reinterpret_cast<const float4*>(w + c), w1 = *reinterpret_cast<const float4*>(w + c + 4);
            const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int j = 0; j < 8; ++j) v[u][j] = v[u][j] * inv * ww[j];
            *reinterpret_cast<uint4*>(yr + c) = pack_bf16x8(v[u]);
        }
    }
}

__global__ void sigmoid_mul_vec_kernel(__nv_bfloat16* __restrict__ o, int64_t ldo, const __nv_bfloat16* __restrict__ g, int64_t ldg,
                                       int64_t total8, int n8) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / n8;
        const int c = (int)(i - t * n8) * 8;
        float a[8], b[8];
        unpack_bf16x8(*reinterpret_cast<const uint4*>(o + t * ldo + c), a);
        unpack_bf16x8(*reinterpret_cast<const uint4*>(g + t * ldg + c), b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = a[j] / (1.0f + expf(-b[j]));
        *reinterpret_cast<uint4*>(o + t * ldo + c) = pack_bf16x8(a);
    }
}

__global__ void cast_rows_vec_kernel(const float* __restrict__ src, int64_t lds, __nv_bfloat16* __restrict__ dst, int64_t ldd,
                                     int64_t total8, int n8) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / n8;
        const int c = (int)(i - t * n8) * 8;
        const float4 a = *reinterpret_cast<const float4*>(src + t * lds + c), b = *reinterpret_cast<const float4*>(src + t * lds + c + 4);
        const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
        *reinterpret_cast<uint4*>(dst + t * ldd + c) = pack_bf16x8(v);
    }
}

}  // namespace

XS_API int xs_embed_pos(const void* table, const void* rows, int dtype, const int32_t* ids, const int32_t* positions, float* h,
                        int T, int H, float scale, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && H > 0, "embed_pos: %d tokens of width %d", T, H);
    XS_DISPATCH_DTYPE(dtype, TT, xs_launch(embed_pos_kernel<TT>, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream, (const TT*)table,
                                           (const TT*)rows, ids, positions, h, H, scale));
    XS_LAUNCH_CHECK("embed_pos");
    return 0;
}

// x: [T, d] rows `ldx` apart, in place; table: [vocab, ld_table] of the same element type, columns off .. off + d - 1.
XS_API int xs_side_gate(void* x, int64_t ldx, const int32_t* ids, const void* table, int64_t ld_table, int off, int T, int d,
                        int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && d > 0 && ldx >= d && off >= 0 && off + d <= ld_table, "side_gate: %d tokens, columns %d + %d of %lld", T, off, d,
               (long long)ld_table);
    const int64_t total = (int64_t)T * d;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    XS_DISPATCH_DTYPE(dtype, TT, xs_launch(side_gate_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (TT*)x, ldx, ids, (const TT*)table,
                                           ld_table, off, total, d));
    XS_LAUNCH_CHECK("side_gate");
    return 0;
}

XS_API int xs_rmsnorm_rows(const void* x, int64_t ldx, const float* w, void* y, int64_t ldy, int T, int n, float eps, int dtype,
                           cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && n > 0 && ldx >= n && ldy >= n, "rmsnorm_rows: %d rows of %d", T, n);
    if (dtype == XS_BF16 && n % 8 == 0 && n <= 8192 && ldx % 8 == 0 && ldy % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)y % 16 == 0 &&
        (uintptr_t)w % 16 == 0) {
        xs_launch(rmsnorm_rows_vec_kernel, dim3(T), dim3(n > 4096 ? 256 : 128), 0, stream, (const __nv_bfloat16*)x, ldx, w,
                  (__nv_bfloat16*)y, ldy, n, eps);
        XS_LAUNCH_CHECK("rmsnorm_rows");
        return 0;
    }
    XS_DISPATCH_DTYPE(dtype, TT, xs_launch(rmsnorm_rows_kernel<TT>, dim3(T), dim3(n >= 1024 ? 256 : 128), 0, stream, (const TT*)x, ldx,
                                           w, (TT*)y, ldy, n, eps));
    XS_LAUNCH_CHECK("rmsnorm_rows");
    return 0;
}

XS_API int xs_sigmoid_mul(void* o, int64_t ldo, const void* g, int64_t ldg, int T, int n, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && n > 0 && ldo >= n && ldg >= n, "sigmoid_mul: %d rows of %d", T, n);
    if (dtype == XS_BF16 && n % 8 == 0 && ldo % 8 == 0 && ldg % 8 == 0 && (uintptr_t)o % 16 == 0 && (uintptr_t)g % 16 == 0) {
        const int64_t total8 = (int64_t)T * (n / 8);
        const int blocks8 = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        xs_launch(sigmoid_mul_vec_kernel, dim3(blocks8), dim3(256), 0, stream, (__nv_bfloat16*)o, ldo, (const __nv_bfloat16*)g, ldg,
                  total8, n / 8);
        XS_LAUNCH_CHECK("sigmoid_mul");
        return 0;
    }
    const int64_t total = (int64_t)T * n;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    XS_DISPATCH_DTYPE(dtype, TT, xs_launch(sigmoid_mul_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (TT*)o, ldo, (const TT*)g, ldg,
                                           total, n));
    XS_LAUNCH_CHECK("sigmoid_mul");
    return 0;
}

XS_API int xs_cast_rows(const float* src, int64_t lds, void* dst, int64_t ldd, int T, int n, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && n > 0 && lds >= n && ldd >= n, "cast_rows: %d rows of %d", T, n);
    if (dtype == XS_BF16 && n % 8 == 0 && lds % 4 == 0 && ldd % 8 == 0 && (uintptr_t)src % 16 == 0 && (uintptr_t)dst % 16 == 0) {
        const int64_t total8 = (int64_t)T * (n / 8);
        const int blocks8 = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        xs_launch(cast_rows_vec_kernel, dim3(blocks8), dim3(256), 0, stream, src, lds, (__nv_bfloat16*)dst, ldd, total8, n / 8);
        XS_LAUNCH_CHECK("cast_rows");
        return 0;
    }
    const int64_t total = (int64_t)T * n;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    XS_DISPATCH_DTYPE(dtype, TT, xs_launch(cast_rows_kernel<TT>, dim3(blocks), dim3(256), 0, stream, src, lds, (TT*)dst, ldd, total, n));
    XS_LAUNCH_CHECK("cast_rows");
    return 0;
}

// x: [T, >= C] rows `ldx` apart; out likewise `ldo` apart; state: [*, taps - 1, C] in x's element type. act 0: none, 1: silu
// of the filter's sum. residual 1: the token's own input is added behind the activation.
XS_API int xs_causal_conv(const void* x, int64_t ldx, const float* taps_w, void* state, const int32_t* seq_of_token,
                          const int32_t* cu_seqlens, const int32_t* slots, void* out, int64_t ldo, int T, int n_seqs, int C,
                          int taps, int act, int residual, int all_single, int dtype, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(!all_single || T == n_seqs, "causal_conv: %d tokens for %d sequences of one token each", T, n_seqs);
    XS_REQUIRE(C > 0 && taps >= 1 && taps <= kMaxTaps, "causal_conv: %d channels, %d taps (at most %d)", C, taps, kMaxTaps);
    XS_REQUIRE(T > 0 && n_seqs > 0 && C <= 65535 * 128 && (act == 0 || act == 1), "causal_conv: %d tokens in %d sequences, %d channels",
               T, n_seqs, C);
    const int tiles = ceil_div_i(C, 128);
    const int vec = 4;                             // channels a thread
    const bool aligned = C % vec == 0 && ldx % vec == 0 && ldo % vec == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                         (uintptr_t)state % 16 == 0 && (uintptr_t)taps_w % 16 == 0;
    if (aligned && taps <= kTileTaps && T >= 256 && !all_single) {
#define XS_TILE(TT, N)                                                                                                         \
    xs_launch(causal_conv_tile_kernel<TT, N>, dim3(ceil_div_i(T, kTileTokens), ceil_div_i(C, 128 * vec)), dim3(128), 0, stream, \
              (const TT*)x, ldx, taps_w, (const TT*)state, seq_of_token, cu_seqlens, slots, (TT*)out, ldo, C, act, residual, T)
        XS_DISPATCH_DTYPE(dtype, TT, do {
            if (taps == 1) XS_TILE(TT, 1);
            else if (taps == 2) XS_TILE(TT, 2);
            else if (taps == 3) XS_TILE(TT, 3);
            else if (taps == 4) XS_TILE(TT, 4);
            else if (taps == 5) XS_TILE(TT, 5);
            else if (taps == 6) XS_TILE(TT, 6);
            else if (taps == 7) XS_TILE(TT, 7);
            else XS_TILE(TT, 8);
        } while (0));
#undef XS_TILE
    } else {
        XS_DISPATCH_DTYPE(dtype, TT,
                          xs_launch(causal_conv_kernel<TT>, dim3(T, tiles), dim3(128), 0, stream, (const TT*)x, ldx, taps_w,
                                    (TT*)state, seq_of_token, cu_seqlens, slots, (TT*)out, ldo, C, taps, act, residual,
                                    all_single && taps > 1 ? 1 : 0));
        if (all_single) {
            XS_LAUNCH_CHECK("causal_conv");
            return 0;
        }
    }
    XS_LAUNCH_CHECK("causal_conv");
    if (taps > 1) {
        XS_DISPATCH_DTYPE(dtype, TT,
                          xs_launch(causal_conv_state_kernel<TT>, dim3(n_seqs, tiles), dim3(128), 0, stream, (const TT*)x, ldx,
                                    (TT*)state, cu_seqlens, slots, C, taps));
        XS_LAUNCH_CHECK("causal_conv (state)");
    }
    return 0;
}

XS_API int xs_gated_add(float* h, const void* branch, int branch_dtype, const float* logits, int64_t ld_logits, const float* bias,
                        int T, int W, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && W > 0 && ld_logits >= W, "gated_add: %d rows of %d, gate rows %lld apart", T, W, (long long)ld_logits);
    const int64_t total = (int64_t)T * W;
    XS_DISPATCH_DTYPE(branch_dtype, TB,
                      xs_launch(gated_add_kernel<TB>, dim3(ceil_div_i(total, 256)), dim3(256), 0, stream, h, (const TB*)branch,
                                logits, ld_logits, bias, total, W));
    XS_LAUNCH_CHECK("gated_add");
    return 0;
}

// hist: `terms` planes of `plane` floats each, of which the first `total` are summed into out.
XS_API int xs_depth_average(const float* hist, int64_t plane, const float* coef, int terms, float* out, int64_t total,
                            cudaStream_t stream) {
    if (total == 0) return 0;
    XS_REQUIRE(terms > 0 && terms <= kMaxTerms && total > 0 && plane >= total, "depth_average: %d terms (at most %d) of %lld",
               terms, kMaxTerms, (long long)total);
    XS_REQUIRE(((uintptr_t)hist % 16 == 0) && ((uintptr_t)out % 16 == 0), "depth_average: buffers must be 16-byte aligned");
    xs_launch(depth_average_kernel, dim3(ceil_div_i(ceil_div_i(total, 4), 256)), dim3(256), 0, stream, hist, plane, coef, terms, out,
              total);
    XS_LAUNCH_CHECK("depth_average");
    return 0;
}

XS_API int xs_rmsnorm_accumulate(const void* x, int dtype, const float* w, float* acc, int T, int W, float eps, float scale,
                                 int add, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && W > 0, "rmsnorm_accumulate: %d rows of %d", T, W);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(rmsnorm_accumulate_kernel<TT>, dim3(T), dim3(W >= 2048 ? 256 : 128), 0, stream, (const TT*)x, w, acc,
                                W, eps, scale, add));
    XS_LAUNCH_CHECK("rmsnorm_accumulate");
    return 0;
}
