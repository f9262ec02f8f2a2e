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
// lanes of one warp (ROWS rows each), so the two sums over a column that a token needs (with kn and with qn) are one pass over
// the registers and a few shuffles; written with u folded in, a token costs that pass and one more:
//   r = S^T kn, s = S^T qn (old S);  u = beta (v - g r);  o = g s + u (kn . qn);  S <- g S + kn u^T
// The recurrence is a chain of dependent operations per entry of S, so a token's time is latency, not arithmetic. The warps
// that hold S (consumers) therefore do nothing else: kProducers further warps stage the next tokens (normed keys and
// queries, kn . qn, g, beta, the tile's values) into the other of two buffers in shared memory while the consumers walk
// the current one, and the two sides meet at one barrier a buffer.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kRows = 16;      // rows of S whose products with a key are summed in one chain of four accumulators
constexpr int kProducers = 4;  // warps that stage tokens
constexpr int kBatch = 4;      // tokens whose loads a producer warp has in flight together

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

// tokens a buffer: the longer, the better a producer's load latencies are spread; bounded by shared memory (the widest
// case, checked where the kernel is launched, is under the 48 KB every kernel may have). Brief steps need no long buffer.
template <int DP, int JOIN>
constexpr int stage_tokens() { return JOIN > 1 ? 8 : DP <= 64 ? 32 : DP <= 128 ? 16 : 8; }

template <typename T, int BLOCKS, int JOIN>
__global__ void __launch_bounds__(128 + 32 * kProducers, 2) gated_delta_kernel(GdArgs a) {
    extern __shared__ __align__(16) float smem[];
    constexpr int ROWS = kRows * JOIN;             // rows of S a lane keeps
    constexpr int PARTS = BLOCKS / JOIN;           // lanes a column
    constexpr int DP = kRows * BLOCKS;             // rows of S as the registers hold them (>= D; the surplus stays zero)
    constexpr int STAGE = stage_tokens<DP, JOIN>();
    constexpr int NR = (DP + 31) / 32;             // entries of a key a producer lane keeps
    const int D = a.D, Pn = a.P;
    const int consumers = (int)blockDim.x - 32 * kProducers;
    const int cols = consumers / PARTS;            // value columns of this CTA
    float* qs = smem;                              // [2][STAGE][DP]
    float* ks = qs + 2 * STAGE * DP;               // [2][STAGE][DP]
    float* vs = ks + 2 * STAGE * DP;               // [2][STAGE][cols]
    float* sc = vs + 2 * STAGE * cols;             // [2][STAGE][4]: g, beta, kn . qn
    pdl_launch_dependents();
    const int h = blockIdx.y, seq = blockIdx.z;
    const int kh = h / (a.heads / a.key_heads);
    const bool producer = (int)threadIdx.x >= consumers;
    const int lane = threadIdx.x & 31;
    const int t0 = a.cu_seqlens[seq], t1 = a.cu_seqlens[seq + 1];
    const int64_t slot = a.slots[seq];
    pdl_wait();
    if (t1 <= t0) return;
    const int stages = (t1 - t0 + STAGE - 1) / STAGE;
    const T* qkv = (const T*)a.qkv;

    if (producer) {
        const int pt = (int)threadIdx.x - consumers, pwarp = pt >> 5;
        const float decay_rate = -expf(a.a_log[h]), dt_b = a.dt_bias[h];
        for (int s = 0; s <= stages; ++s) {
            if (s < stages) {
                const int base = t0 + s * STAGE, n = min(STAGE, t1 - base);
                float* qb = qs + (s & 1) * STAGE * DP;
                float* kb = ks + (s & 1) * STAGE * DP;
                float* vb = vs + (s & 1) * STAGE * cols;
                float* sb = sc + (s & 1) * STAGE * 4;
                // a token a thread: its decay and its step size
                if (pt < n) {
                    const float* ab = a.ab + (int64_t)(base + pt) * a.ld_ab;
                    sb[pt * 4 + 0] = expf(decay_rate * softplus_f(ab[h] + dt_b));
                    sb[pt * 4 + 1] = 1.0f / (1.0f + expf(-ab[a.heads + h]));
                }
                // the tile's values
#pragma unroll 4
                for (int idx = pt; idx < n * cols; idx += 32 * kProducers) {
                    const int i = idx / cols, c = idx - i * cols;
                    const int gc = blockIdx.x * cols + c;
                    vb[idx] = gc < Pn ? to_f32(qkv[(int64_t)(base + i) * a.ld + a.v_col + h * Pn + gc]) : 0.0f;
                }
                // a warp a token, kBatch tokens' loads together: key and query, their norms and their product
                for (int g0 = pwarp * kBatch; g0 < n; g0 += kProducers * kBatch) {
                    float qv[kBatch][NR], kv[kBatch][NR];
#pragma unroll
                    for (int j = 0; j < kBatch; ++j) {
                        const T* row = qkv + (int64_t)(base + min(g0 + j, n - 1)) * a.ld;
#pragma unroll
                        for (int r = 0; r < NR; ++r) {
                            const int d = lane + 32 * r;
                            qv[j][r] = d < D ? to_f32(row[a.q_col + kh * D + d]) : 0.0f;
                            kv[j][r] = d < D ? to_f32(row[a.k_col + kh * D + d]) : 0.0f;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < kBatch; ++j) {
                        float qq = 0.0f, kk = 0.0f, qk = 0.0f;
#pragma unroll
                        for (int r = 0; r < NR; ++r) {
                            qq = fmaf(qv[j][r], qv[j][r], qq);
                            kk = fmaf(kv[j][r], kv[j][r], kk);
                            qk = fmaf(qv[j][r], kv[j][r], qk);
                        }
                        qq = warp_sum(qq);
                        kk = warp_sum(kk);
                        qk = warp_sum(qk);
                        const float qn = a.q_scale / sqrtf(qq + a.unit_eps), kn = 1.0f / sqrtf(kk + a.unit_eps);
                        const int i = g0 + j;
                        if (i < n) {
#pragma unroll
                            for (int r = 0; r < NR; ++r) {
                                const int d = lane + 32 * r;
                                if (d < DP) {
                                    qb[i * DP + d] = qv[j][r] * qn;
                                    kb[i * DP + d] = kv[j][r] * kn;
                                }
                            }
                            if (lane == 0) sb[i * 4 + 2] = qk * qn * kn;
                        }
                    }
                }
            }
            __syncthreads();                       // buffer s is full; the consumers are done with the one before it
        }
        return;
    }

    const int part = lane % PARTS, col_local = (int)threadIdx.x / PARTS;
    const int col = blockIdx.x * cols + col_local;
    const bool live = col < Pn;
    float S[ROWS];
    float* sg = a.state + ((slot * a.heads + h) * D) * (int64_t)Pn;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int d = part * ROWS + r;
        S[r] = (live && d < D) ? sg[(int64_t)d * Pn + col] : 0.0f;
    }
    __syncthreads();                               // buffer 0 is full
    for (int s = 0; s < stages; ++s) {
        const int base = t0 + s * STAGE, n = min(STAGE, t1 - base);
        const float* qb = qs + (s & 1) * STAGE * DP + part * ROWS;
        const float* kb = ks + (s & 1) * STAGE * DP + part * ROWS;
        const float* vb = vs + (s & 1) * STAGE * cols + col_local;
        const float* sb = sc + (s & 1) * STAGE * 4;
        float* yo = a.y + (int64_t)base * (a.heads * Pn) + h * Pn + col;
#pragma unroll(JOIN == 1 ? 2 : 1)
        for (int i = 0; i < n; ++i) {
            const float4* k4 = reinterpret_cast<const float4*>(kb + i * DP);
            const float4* q4 = reinterpret_cast<const float4*>(qb + i * DP);
            // Blocks of kRows rows are summed each in four chains, and the blocks' sums pairwise, neighbours first: within
            // the lane for the JOIN blocks it keeps, by shuffles across the lanes of a column. The tree is the same
            // whatever JOIN is, so every JOIN gives the same bits.
            float pr[JOIN], ps[JOIN];
#pragma unroll
            for (int j = 0; j < JOIN; ++j) {
                float r0 = 0.0f, r1 = 0.0f, r2 = 0.0f, r3 = 0.0f, s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
                for (int r = j * (kRows / 4); r < (j + 1) * (kRows / 4); ++r) {
                    const float4 kv = k4[r], qv = q4[r];
                    r0 = fmaf(S[4 * r], kv.x, r0); r1 = fmaf(S[4 * r + 1], kv.y, r1);
                    r2 = fmaf(S[4 * r + 2], kv.z, r2); r3 = fmaf(S[4 * r + 3], kv.w, r3);
                    s0 = fmaf(S[4 * r], qv.x, s0); s1 = fmaf(S[4 * r + 1], qv.y, s1);
                    s2 = fmaf(S[4 * r + 2], qv.z, s2); s3 = fmaf(S[4 * r + 3], qv.w, s3);
                }
                pr[j] = (r0 + r1) + (r2 + r3);
                ps[j] = (s0 + s1) + (s2 + s3);
            }
#pragma unroll
            for (int w = 1; w < JOIN; w <<= 1)
#pragma unroll
                for (int m = 0; m < JOIN; m += 2 * w) {
                    pr[m] += pr[m + w];
                    ps[m] += ps[m + w];
                }
            float rk = pr[0], sq = ps[0];
#pragma unroll
            for (int o = 1; o < PARTS; o <<= 1) {
                rk += __shfl_xor_sync(0xffffffffu, rk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
            }
            const float4 gbk = *reinterpret_cast<const float4*>(sb + i * 4);   // g, beta, kn . qn
            const float g = gbk.x;
            const float u = gbk.y * (vb[i * cols] - g * rk);
            if (live && part == 0) yo[(int64_t)i * (a.heads * Pn)] = fmaf(u, gbk.z, g * sq);
#pragma unroll
            for (int r = 0; r < ROWS / 4; ++r) {
                const float4 kv = k4[r];
                S[4 * r] = fmaf(kv.x, u, g * S[4 * r]);
                S[4 * r + 1] = fmaf(kv.y, u, g * S[4 * r + 1]);
                S[4 * r + 2] = fmaf(kv.z, u, g * S[4 * r + 2]);
                S[4 * r + 3] = fmaf(kv.w, u, g * S[4 * r + 3]);
            }
        }
        __syncthreads();                           // this buffer may be filled again; the next one is full
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int d = part * ROWS + r;
        if (live && d < D) sg[(int64_t)d * Pn + col] = S[r];
    }
}

template <typename T, int BLOCKS, int JOIN>
int launch(const GdArgs& a, int n_seqs, cudaStream_t stream) {
    constexpr int DP = kRows * BLOCKS, STAGE = stage_tokens<DP, JOIN>(), PARTS = BLOCKS / JOIN;
    int consumers = ((a.P * PARTS + 31) / 32) * 32;
    if (consumers > 128) consumers = 128;
    const int cols = consumers / PARTS;
    const size_t smem = (size_t)(4 * STAGE * DP + 2 * STAGE * cols + 2 * STAGE * 4) * sizeof(float);
    static_assert((4 * STAGE * DP + 2 * STAGE * (128 / PARTS) + 2 * STAGE * 4) * sizeof(float) <= 48 * 1024, "two buffers of tokens fit");
    xs_launch(gated_delta_kernel<T, BLOCKS, JOIN>, dim3(ceil_div_i(a.P, cols), a.heads, n_seqs),
              dim3(consumers + 32 * kProducers), smem, stream, a);
    return 0;
}

}  // namespace

XS_API int xs_gated_delta_scan(const void* qkv, int64_t ld, int q_col, int k_col, int v_col, const float* ab, int64_t ld_ab,
                               const float* a_log, const float* dt_bias, float* state, const int32_t* cu_seqlens,
                               const int32_t* slots, float* y, int n_seqs, int heads, int key_heads, int D, int P, float q_scale,
                               float unit_eps, int tokens, int dtype, cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    XS_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && heads > 0 && heads <= 65535 && key_heads > 0 && heads % key_heads == 0,
               "gated_delta: %d sequences, %d heads over %d key heads", n_seqs, heads, key_heads);
    XS_REQUIRE(D > 0 && D <= 256 && P > 0, "gated_delta: key size %d (at most 256), value size %d", D, P);
    XS_REQUIRE(ld_ab >= 2 * heads, "gated_delta: gate rows %lld apart for %d heads", (long long)ld_ab, heads);
    GdArgs a{qkv, ld, q_col, k_col, v_col, ab, ld_ab, a_log, dt_bias, state, cu_seqlens, slots, y, heads, key_heads, D, P,
             q_scale, unit_eps};
    // A sequence's time is a chain a token long, so long steps spread a column's rows over as many lanes as there are blocks
    // of kRows rows (short chains, many CTAs). Steps of a token or two a sequence are bound by reading and writing S:
    // there a lane keeps two blocks, and a CTA twice the columns.
    const bool brief = tokens <= 2 * n_seqs;
#define XS_GO(TT)                                                                                    \
    do {                                                                                             \
        if (D <= 16) launch<TT, 1, 1>(a, n_seqs, stream);                                            \
        else if (D <= 32) brief ? launch<TT, 2, 2>(a, n_seqs, stream) : launch<TT, 2, 1>(a, n_seqs, stream);       \
        else if (D <= 64) brief ? launch<TT, 4, 2>(a, n_seqs, stream) : launch<TT, 4, 1>(a, n_seqs, stream);       \
        else if (D <= 128) brief ? launch<TT, 8, 2>(a, n_seqs, stream) : launch<TT, 8, 1>(a, n_seqs, stream);      \
        else brief ? launch<TT, 16, 2>(a, n_seqs, stream) : launch<TT, 16, 1>(a, n_seqs, stream);    \
    } while (0)
    XS_DISPATCH_DTYPE(dtype, TT, XS_GO(TT));
#undef XS_GO
    XS_LAUNCH_CHECK("gated_delta_scan");
    return 0;
}
