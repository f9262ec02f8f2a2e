// The gated delta rule: per head a memory S [D, P] (float32, zero at a sequence's start) that every token first decays,
// then corrects towards its value along its key, and then reads with its query:
//
//   kn = k / sqrt(|k|^2 + unit_eps)          qn = q / sqrt(|q|^2 + unit_eps) * q_scale
//   g  = exp(-exp(A_log_h) * softplus(a + dt_bias_h))          beta = sigmoid(b)
//   S <- g S;   u = beta (v - S^T kn);   S <- S + kn u^T;   o = S^T qn
//
// Heads share keys and queries in groups (head h reads key head h / (heads / key heads)). q, k and v come in the
// activation type (behind their projections, short convolutions and activations); the unit norms, a, b, the decay, beta,
// the memory and every sum are float32 in both precision modes.
//
// A CTA walks one (sequence, head, tile of value columns) in order. A column's D rows of S live in the registers of PARTS
// neighbouring lanes (ROWS rows each), so the two sums over a column that a token needs (with kn and with qn) are one pass over
// the registers and a shuffle; written with u folded in, a token costs that pass and one more:
//   r = S^T kn, s = S^T qn (old S);  u = beta (v - g r);  o = g s + u (kn . qn);  S <- g S + kn u^T
// Tokens are staged eight at a time in shared memory (normed keys and queries, kn . qn, g, beta, the tile's values).
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kStage = 8;      // tokens staged at a time

__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

struct GdArgs {
    const void* qkv;           // [T, ld]: q | k | v behind their convolutions
    int64_t ld;
    int q_col, k_col, v_col;
    const float* ab;           // [T, ld_ab]: a (heads) | b (heads), float32
    int64_t ld_ab;
    const float* a_log;
    const float* dt_bias;
    float* state;              // [slots, heads, D, P]
    const int32_t* cu_seqlens;
    const int32_t* slots;
    float* y;                  // [T, heads * P]
    int heads, key_heads, D, P;
    float q_scale, unit_eps;
};

template <typename T, int ROWS, int PARTS>
__global__ void __launch_bounds__(128) gated_delta_kernel(GdArgs a) {
    extern __shared__ __align__(16) float smem[];
    const int D = a.D, Pn = a.P;
    const int DP = ROWS * PARTS;                   // rows of S as the registers hold them (>= D; the surplus stays zero)
    const int cols = blockDim.x / PARTS;           // value columns of this CTA
    float* qs = smem;                              // [kStage][DP]
    float* ks = qs + kStage * DP;                  // [kStage][DP]
    float* vs = ks + kStage * DP;                  // [kStage][cols]
    float* sc = vs + kStage * cols;                // [kStage][4]: g, beta, kn . qn
    pdl_launch_dependents();
    const int h = blockIdx.y, seq = blockIdx.z;
    const int kh = h / (a.heads / a.key_heads);
    const int part = threadIdx.x % PARTS, col_local = threadIdx.x / PARTS;
    const int col = blockIdx.x * cols + col_local;
    const bool live = col < Pn;
    const int t0 = a.cu_seqlens[seq], t1 = a.cu_seqlens[seq + 1];
    const int64_t slot = a.slots[seq];
    const float decay_rate = -expf(a.a_log[h]), dt_b = a.dt_bias[h];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    pdl_wait();
    if (t1 <= t0) return;
    float S[ROWS];
    float* sg = a.state + ((slot * a.heads + h) * D) * (int64_t)Pn;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int d = part * ROWS + r;
        S[r] = (live && d < D) ? sg[(int64_t)d * Pn + col] : 0.0f;
    }
    const T* qkv = (const T*)a.qkv;
    for (int base = t0; base < t1; base += kStage) {
        const int n = min(kStage, t1 - base);
        __syncthreads();                           // the last stage's readers are done
        // a warp a token: its key and query, their norms and their product
        for (int i = warp; i < n; i += warps) {
            const T* row = qkv + (int64_t)(base + i) * a.ld;
            float qq = 0.0f, kk = 0.0f;
            for (int d = lane; d < DP; d += 32) {
                const float qv = d < D ? to_f32(row[a.q_col + kh * D + d]) : 0.0f;
                const float kv = d < D ? to_f32(row[a.k_col + kh * D + d]) : 0.0f;
                qs[i * DP + d] = qv;
                ks[i * DP + d] = kv;
                qq = fmaf(qv, qv, qq);
                kk = fmaf(kv, kv, kk);
            }
            qq = warp_sum(qq);
            kk = warp_sum(kk);
            const float qn = a.q_scale / sqrtf(qq + a.unit_eps), kn = 1.0f / sqrtf(kk + a.unit_eps);
            float dot = 0.0f;
            for (int d = lane; d < DP; d += 32) {
                const float qv = qs[i * DP + d] * qn, kv = ks[i * DP + d] * kn;
                qs[i * DP + d] = qv;
                ks[i * DP + d] = kv;
                dot = fmaf(qv, kv, dot);
            }
            dot = warp_sum(dot);
            if (lane == 0) {
                const float* ab = a.ab + (int64_t)(base + i) * a.ld_ab;
                sc[i * 4 + 0] = expf(decay_rate * softplus_f(ab[h] + dt_b));
                sc[i * 4 + 1] = 1.0f / (1.0f + expf(-ab[a.heads + h]));
                sc[i * 4 + 2] = dot;
            }
        }
        for (int idx = threadIdx.x; idx < n * cols; idx += blockDim.x) {
            const int i = idx / cols, c = idx - i * cols;
            const int gc = blockIdx.x * cols + c;
            vs[i * cols + c] = gc < Pn ? to_f32(qkv[(int64_t)(base + i) * a.ld + a.v_col + h * Pn + gc]) : 0.0f;
        }
        __syncthreads();
        for (int i = 0; i < n; ++i) {
            const float4* k4 = reinterpret_cast<const float4*>(ks + i * DP + part * ROWS);
            const float4* q4 = reinterpret_cast<const float4*>(qs + i * DP + part * ROWS);
            float r0 = 0.0f, r1 = 0.0f, s0 = 0.0f, s1 = 0.0f;
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                const float4 kv = k4[r], qv = q4[r];
                r0 = fmaf(S[4 * r], kv.x, r0); r1 = fmaf(S[4 * r + 1], kv.y, r1);
                r0 = fmaf(S[4 * r + 2], kv.z, r0); r1 = fmaf(S[4 * r + 3], kv.w, r1);
                s0 = fmaf(S[4 * r], qv.x, s0); s1 = fmaf(S[4 * r + 1], qv.y, s1);
                s0 = fmaf(S[4 * r + 2], qv.z, s0); s1 = fmaf(S[4 * r + 3], qv.w, s1);
            }
            float rk = r0 + r1, sq = s0 + s1;
#pragma unroll
            for (int o = 1; o < PARTS; o <<= 1) {
                rk += __shfl_xor_sync(0xffffffffu, rk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
            }
            const float g = sc[i * 4 + 0], beta = sc[i * 4 + 1], kq = sc[i * 4 + 2];
            const float u = beta * (vs[i * cols + col_local] - g * rk);
            if (live && part == 0) a.y[(int64_t)(base + i) * (a.heads * Pn) + h * Pn + col] = fmaf(u, kq, g * sq);
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                const float4 kv = k4[r];
                S[4 * r] = fmaf(kv.x, u, g * S[4 * r]);
                S[4 * r + 1] = fmaf(kv.y, u, g * S[4 * r + 1]);
                S[4 * r + 2] = fmaf(kv.z, u, g * S[4 * r + 2]);
                S[4 * r + 3] = fmaf(kv.w, u, g * S[4 * r + 3]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int d = part * ROWS + r;
        if (live && d < D) sg[(int64_t)d * Pn + col] = S[r];
    }
}

template <typename T, int ROWS, int PARTS>
int launch(const GdArgs& a, int n_seqs, cudaStream_t stream) {
    int threads = ((a.P * PARTS + 31) / 32) * 32;
    if (threads > 128) threads = 128;
    const int cols = threads / PARTS;
    const size_t smem = (size_t)(2 * kStage * ROWS * PARTS + kStage * cols + kStage * 4) * sizeof(float);
    xs_launch(gated_delta_kernel<T, ROWS, PARTS>, dim3(ceil_div_i(a.P, cols), a.heads, n_seqs), dim3(threads), smem, stream, a);
    return 0;
}

}  // namespace

XS_API int xs_gated_delta_scan(const void* qkv, int64_t ld, int q_col, int k_col, int v_col, const float* ab, int64_t ld_ab,
                               const float* a_log, const float* dt_bias, float* state, const int32_t* cu_seqlens,
                               const int32_t* slots, float* y, int n_seqs, int heads, int key_heads, int D, int P, float q_scale,
                               float unit_eps, int dtype, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    XS_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && heads > 0 && heads <= 65535 && key_heads > 0 && heads % key_heads == 0,
               "gated_delta: %d sequences, %d heads over %d key heads", n_seqs, heads, key_heads);
    XS_REQUIRE(D > 0 && D <= 256 && P > 0, "gated_delta: key size %d (at most 256), value size %d", D, P);
    XS_REQUIRE(ld_ab >= 2 * heads, "gated_delta: gate rows %lld apart for %d heads", (long long)ld_ab, heads);
    GdArgs a{qkv, ld, q_col, k_col, v_col, ab, ld_ab, a_log, dt_bias, state, cu_seqlens, slots, y, heads, key_heads, D, P,
             q_scale, unit_eps};
#define XS_GO(TT)                                                     \
    do {                                                              \
        if (D <= 16) launch<TT, 16, 1>(a, n_seqs, stream);            \
        else if (D <= 32) launch<TT, 32, 1>(a, n_seqs, stream);       \
        else if (D <= 64) launch<TT, 32, 2>(a, n_seqs, stream);       \
        else if (D <= 128) launch<TT, 64, 2>(a, n_seqs, stream);      \
        else launch<TT, 64, 4>(a, n_seqs, stream);                    \
    } while (0)
    XS_DISPATCH_DTYPE(dtype, TT, XS_GO(TT));
#undef XS_GO
    XS_LAUNCH_CHECK("gated_delta_scan");
    return 0;
}
