// Residual add + layer norm without a bias, fused as the RMSNorm kernel of norm_embed.cu is:
//
//   LN(x, w, eps) = (x - mean(x)) * (mean((x - mean(x))^2) + eps)^(-1/2) * w        over the last dimension
//
// For each output row i (source row r = rows ? rows[i] : i):
//   v = h[r]                                   float32
//   if m:      b = m[r];  if post_w: b = LN(b, post_w, eps_post)
//              v = v + b;  h[r] = v            the residual sum stays float32
//   if w:      y[i] = LN(v, w, eps)            written in y's element type
// The mean is taken first and the variance from the deviations (two passes over a row that lives in
// shared memory), all in float32, whatever the element type of m and y.
#include "common.cuh"

namespace {

template <typename TM, typename TY>
__global__ void add_layernorm_kernel(float* __restrict__ h, const TM* __restrict__ m, const float* __restrict__ post_w,
                                     const float* __restrict__ w, TY* __restrict__ y, const int32_t* __restrict__ rows,
                                     int H, float eps_post, float eps) {
    extern __shared__ float row[];
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float* hr = h + r * H;
    const float inv_h = 1.0f / (float)H;
    if (m != nullptr) {
        const TM* mr = m + r * H;
        float s = 0.0f;
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            const float b = to_f32(mr[c]);
            row[c] = b;
            s += b;
        }
        if (post_w != nullptr) {
            const float mean = block_sum(s, scratch) * inv_h;
            float q = 0.0f;
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float d = row[c] - mean;
                q += d * d;
            }
            const float inv = 1.0f / sqrtf(block_sum(q, scratch) * inv_h + eps_post);
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float v = hr[c] + (row[c] - mean) * inv * post_w[c];
                row[c] = v;
                hr[c] = v;
            }
        } else {
            for (int c = threadIdx.x; c < H; c += blockDim.x) {
                const float v = hr[c] + row[c];
                row[c] = v;
                hr[c] = v;
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) row[c] = hr[c];
    }
    if (w == nullptr) return;
    float s = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) s += row[c];
    const float mean = block_sum(s, scratch) * inv_h;
    float q = 0.0f;
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        const float d = row[c] - mean;
        q += d * d;
    }
    const float inv = 1.0f / sqrtf(block_sum(q, scratch) * inv_h + eps);
    TY* yr = y + (int64_t)i * H;
    for (int c = threadIdx.x; c < H; c += blockDim.x) yr[c] = from_f32<TY>((row[c] - mean) * inv * w[c]);
}

// The same for widths that are a multiple of 4 and at most 16 * 1024: a thread keeps up to four float4 of the row in
// registers, so the row is read once and every pass after the first runs on registers.
template <typename TM>
__device__ __forceinline__ float4 ln_load4(const TM* p);
template <>
__device__ __forceinline__ float4 ln_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <>
__device__ __forceinline__ float4 ln_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 raw = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void ln_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void ln_store4(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&a);
    raw.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}

// mean and 1 / sqrt(variance + eps) of the row held as v[NV] by the block's threads (zeros beyond the row)
template <int NV>
__device__ __forceinline__ void ln_stats(const float4 (&v)[NV], int chunks, int H, float eps, float* scratch, float& mean, float& inv) {
    float s = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) s += v[k].x + v[k].y + v[k].z + v[k].w;
    mean = block_sum(s, scratch) / (float)H;
    float q = 0.0f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        if ((int)(threadIdx.x + k * blockDim.x) < chunks) {
            const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, d = v[k].w - mean;
            q += a * a + b * b + c * c + d * d;
        }
    }
    inv = 1.0f / sqrtf(block_sum(q, scratch) / (float)H + eps);
}

template <typename TM, typename TY, int NV>
__global__ void add_layernorm_vec_kernel(float* __restrict__ h, const TM* __restrict__ m, const float* __restrict__ post_w,
                                         const float* __restrict__ w, TY* __restrict__ y, const int32_t* __restrict__ rows,
                                         int H, float eps_post, float eps) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float* hr = h + r * H;
    const int chunks = H >> 2;
    float4 v[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        v[k] = c < chunks ? ln_load4<float>(hr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (m != nullptr) {
        const TM* mr = m + r * H;
        float4 b[NV];
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            b[k] = c < chunks ? ln_load4<TM>(mr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        float mean = 0.0f, inv = 1.0f;
        if (post_w != nullptr) ln_stats<NV>(b, chunks, H, eps_post, scratch, mean, inv);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int c = threadIdx.x + k * blockDim.x;
            if (c >= chunks) continue;
            if (post_w != nullptr) {
                const float4 pw = ln_load4<float>(post_w + 4 * c);
                v[k].x += (b[k].x - mean) * inv * pw.x;
                v[k].y += (b[k].y - mean) * inv * pw.y;
                v[k].z += (b[k].z - mean) * inv * pw.z;
                v[k].w += (b[k].w - mean) * inv * pw.w;
            } else {
                v[k].x += b[k].x;
                v[k].y += b[k].y;
                v[k].z += b[k].z;
                v[k].w += b[k].w;
            }
            ln_store4(hr + 4 * c, v[k]);
        }
    }
    if (w == nullptr) return;
    float mean, inv;
    ln_stats<NV>(v, chunks, H, eps, scratch, mean, inv);
    TY* yr = y + (int64_t)i * H;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int c = threadIdx.x + k * blockDim.x;
        if (c >= chunks) continue;
        const float4 ww = ln_load4<float>(w + 4 * c);
        ln_store4(yr + 4 * c, make_float4((v[k].x - mean) * inv * ww.x, (v[k].y - mean) * inv * ww.y,
                                          (v[k].z - mean) * inv * ww.z, (v[k].w - mean) * inv * ww.w));
    }
}

// y[t, g, :] = x[t, g, :] / sqrt(mean(x[t, g, :]^2) + eps) * w[g, :]: a unit-RMS norm in `groups` equal parts of a
// row (x float32, y in the activation type). One block per (row, part).
// With `gate` (rows of the activation type, `ld_gate` apart): y is also multiplied by sigmoid(gate[t, g, :]), or with
// gate_act 1 by silu(gate[t, g, :]) = gate * sigmoid(gate).
template <typename TY>
__global__ void grouped_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, TY* __restrict__ y,
                                       int width, int part, float eps, const TY* __restrict__ gate, int64_t ld_gate,
                                       int gate_act) {
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int64_t base = (int64_t)blockIdx.x * width + (int64_t)blockIdx.y * part;
    const float* xr = x + base;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < part; c += blockDim.x) ss += xr[c] * xr[c];
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)part + eps);
    const float* wr = w + (int64_t)blockIdx.y * part;
    if (gate != nullptr) {
        const TY* gr = gate + (int64_t)blockIdx.x * ld_gate + (int64_t)blockIdx.y * part;
        for (int c = threadIdx.x; c < part; c += blockDim.x) {
            const float gv = to_f32(gr[c]);
            y[base + c] = from_f32<TY>(xr[c] * inv * wr[c] * (gate_act == 1 ? gv : 1.0f) / (1.0f + expf(-gv)));
        }
        return;
    }
    for (int c = threadIdx.x; c < part; c += blockDim.x) y[base + c] = from_f32<TY>(xr[c] * inv * wr[c]);
}

// The same for parts of at most 1024 elements: one block a row, a warp a part (warps take parts in turn), so that a row of
// many short parts (the heads of a recurrent layer) is one block instead of one tiny block a part.
template <typename TY>
__global__ void grouped_rmsnorm_warp_kernel(const float* __restrict__ x, const float* __restrict__ w, TY* __restrict__ y,
                                            int width, int part, int groups, float eps, const TY* __restrict__ gate,
                                            int64_t ld_gate, int gate_act) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int64_t row = blockIdx.x;
    for (int g = warp; g < groups; g += warps) {
        const int64_t base = row * width + (int64_t)g * part;
        const float* xr = x + base;
        float v[32];                                   // up to 1024 elements a part
        float ss = 0.0f;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const int c = lane + 32 * k;
            v[k] = c < part ? xr[c] : 0.0f;
            ss += v[k] * v[k];
            if (32 * (k + 1) >= part) break;
        }
        const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)part + eps);
        const float* wr = w + (int64_t)g * part;
        const TY* gr = gate != nullptr ? gate + row * ld_gate + (int64_t)g * part : nullptr;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const int c = lane + 32 * k;
            if (c < part) {
                float o = v[k] * inv * wr[c];
                if (gr != nullptr) {
                    const float gv = to_f32(gr[c]);
                    o *= (gate_act == 1 ? gv : 1.0f) / (1.0f + expf(-gv));
                }
                y[base + c] = from_f32<TY>(o);
            }
            if (32 * (k + 1) >= part) break;
        }
    }
}

}  // namespace

XS_API int xs_add_layernorm(float* h, const void* m, int m_dtype, const float* post_w, const float* w, void* y,
                            int y_dtype, const int32_t* rows, int n_rows, int H, float eps_post, float eps,
                            cudaStream_t stream) {
    if (n_rows == 0) return 0;
    XS_REQUIRE(n_rows > 0 && H > 0, "add_layernorm: %d rows of width %d", n_rows, H);
    XS_REQUIRE((size_t)H * 4 <= 200 * 1024, "add_layernorm: width %d does not fit shared memory (limit 51200)", H);
    XS_REQUIRE(w == nullptr || y != nullptr, "add_layernorm: a norm weight without an output");
    const bool aligned = H % 4 == 0 && ((uintptr_t)h % 16 == 0) && ((uintptr_t)m % 16 == 0) && ((uintptr_t)y % 16 == 0) &&
                         ((uintptr_t)w % 16 == 0) && ((uintptr_t)post_w % 16 == 0);
    if (aligned && H <= 16 * 1024) {
        const int chunks = H / 4;
        const int vthreads = chunks <= 128 ? 128 : chunks <= 1024 ? 256 : chunks <= 2048 ? 512 : 1024;
        const int nv = (chunks + vthreads - 1) / vthreads;
#define XS_VEC(TM, TY, NV)                                                                                              \
    xs_launch(add_layernorm_vec_kernel<TM, TY, NV>, dim3(n_rows), dim3(vthreads), 0, stream, h, (const TM*)m, post_w, \
              w, (TY*)y, rows, H, eps_post, eps)
#define XS_VEC_NV(TM, TY)                       \
    do {                                        \
        if (nv <= 1) XS_VEC(TM, TY, 1);         \
        else if (nv == 2) XS_VEC(TM, TY, 2);    \
        else XS_VEC(TM, TY, 4);                 \
    } while (0)
        XS_DISPATCH_DTYPE(m_dtype, TM, XS_DISPATCH_DTYPE(y_dtype, TY, XS_VEC_NV(TM, TY)));
#undef XS_VEC_NV
#undef XS_VEC
        XS_LAUNCH_CHECK("add_layernorm");
        return 0;
    }
    const size_t smem = (size_t)H * sizeof(float);
    const int threads = H >= 4096 ? 512 : H >= 512 ? 256 : 128;
#define XS_GO(TM, TY)                                                                                          \
    do {                                                                                                       \
        if (smem > 48 * 1024)                                                                                  \
            cudaFuncSetAttribute(add_layernorm_kernel<TM, TY>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                                 (int)smem);                                                                   \
        xs_launch(add_layernorm_kernel<TM, TY>, dim3(n_rows), dim3(threads), smem, stream, h, (const TM*)m,    \
                  post_w, w, (TY*)y, rows, H, eps_post, eps);                                                  \
    } while (0)
    XS_DISPATCH_DTYPE(m_dtype, TM, XS_DISPATCH_DTYPE(y_dtype, TY, XS_GO(TM, TY)));
#undef XS_GO
    XS_LAUNCH_CHECK("add_layernorm");
    return 0;
}

XS_API int xs_grouped_rmsnorm(const float* x, const float* w, void* y, int y_dtype, int rows, int width, int groups,
                              float eps, const void* gate, int64_t ld_gate, int gate_act, cudaStream_t stream) {
    if (rows == 0) return 0;
    XS_REQUIRE(gate_act == 0 || gate_act == 1, "grouped_rmsnorm: gate activation %d (0 sigmoid, 1 silu)", gate_act);
    XS_REQUIRE(rows > 0 && width > 0 && groups > 0 && width % groups == 0, "grouped_rmsnorm: %d rows of %d in %d parts",
               rows, width, groups);
    XS_REQUIRE(groups <= 65535, "grouped_rmsnorm: %d parts exceed the grid limit", groups);
    const int part = width / groups;
    if (part <= 1024 && groups > 1) {
        const int warps = groups < 8 ? groups : 8;
        XS_DISPATCH_DTYPE(y_dtype, TY,
                          xs_launch(grouped_rmsnorm_warp_kernel<TY>, dim3(rows), dim3(32 * warps), 0, stream, x, w, (TY*)y, width,
                                    part, groups, eps, (const TY*)gate, ld_gate, gate_act));
        XS_LAUNCH_CHECK("grouped_rmsnorm");
        return 0;
    }
    const int threads = part >= 1024 ? 256 : 128;
    XS_DISPATCH_DTYPE(y_dtype, TY,
                      xs_launch(grouped_rmsnorm_kernel<TY>, dim3(rows, groups), dim3(threads), 0, stream, x, w, (TY*)y,
                                width, part, eps, (const TY*)gate, ld_gate, gate_act));
    XS_LAUNCH_CHECK("grouped_rmsnorm");
    return 0;
}
