// A linear-attention memory with a constant decay per head ("lightning attention"):
//
//   S_t = decay_h * S_(t-1) + k_t v_t^T        S: [D, E] float32 per (sequence, head), zero at a sequence's start
//   o_t = S_t^T q_t                            with q, k, v = silu of the projections' outputs
//
// The projections come in the activation type; silu, the decay, the state and every sum are float32. A CTA walks one
// (sequence, head, block of 32 value columns) in order: 8 warps, warp g holding a run of neighbouring rows of the block's columns in
// registers (lane = column), so that a token's k and q are read from shared memory as broadcasts, four at a time. Tokens are
// staged 16 at a time: the next 16 tokens' q, k and v are fetched into registers before the current 16 are walked, and go through silu into
// the other of two shared buffers behind them. A token's output is the sum of the 8 warps' partial sums, added in a fixed
// order after the walk.
//
// Long pieces of a prompt run as chunks side by side in three launches: every chunk from the empty state (leaving its end
// state), a carry over each sequence's chunks in order (S <- decay^len S + local, which is what the recurrence unrolls to;
// each chunk is left with the state it starts from), and the chunks again from their true states, writing the outputs.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kCols = 32;        // value columns a CTA
constexpr int kWarps = 8;        // row groups
constexpr int kBatch = 16;       // tokens staged at a time

enum ScanMode : int { kSequences = 0, kChunkLocal = 1, kChunkFinal = 2 };

struct LightningArgs {
    const void* qkv;             // rows `ld` apart: q [H * D] at q_col, k [H * D] at k_col, v [H * E] at v_col
    int64_t ld;
    int q_col, k_col, v_col;
    const float* decay;          // [H]
    float* state;                // [slots, H, D, E]
    const int32_t* cu_seqlens;   // [sequences + 1]
    const int32_t* slots;        // [sequences]
    float* y;                    // [T, H * E]
    const int32_t* chunks;       // [n, 3] (sequence, first token, tokens), or null
    float* chunk_state;          // [n, H, D, E]
    int H, D, E, mode;
};

// In front of inputs of 8 bits of mantissa the fast exponential and division do (a few units in the last place of float32);
// float32 inputs take the exact ones.
template <typename T>
__device__ __forceinline__ float silu_of(T raw) {
    const float v = to_f32(raw);
    if constexpr (sizeof(T) == 4) return v / (1.0f + expf(-v));
    else return __fdividef(v, 1.0f + __expf(-v));
}

// NR: rows of the state a thread holds (D <= 8 NR): warp g holds rows g NR .. g NR + NR - 1, so that a token's k and q come
// from shared memory four at a time, as broadcasts. A staged token is q [8 NR], k [8 NR] (zeros from D on) and v [32].
template <typename T, int NR>
__global__ void __launch_bounds__(kWarps * 32) lightning_scan_kernel(const LightningArgs a) {
    extern __shared__ __align__(16) float smem[];
    constexpr int DP = kWarps * NR;
    constexpr int row = 2 * DP + kCols;
    const int D = a.D, E = a.E;
    float* stage = smem;                              // [2][kBatch][row]
    float* part = smem + 2 * kBatch * row;            // [2][kBatch][kWarps][kCols]
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int h = blockIdx.y, c0 = blockIdx.x * kCols, col = c0 + lane;
    int t0, n, slot;
    if (a.mode == kSequences) {
        t0 = a.cu_seqlens[blockIdx.z];
        n = a.cu_seqlens[blockIdx.z + 1] - t0;
        slot = a.slots[blockIdx.z];
    } else {
        const int32_t* ch = a.chunks + 3 * (int64_t)blockIdx.z;
        t0 = ch[1];
        n = ch[2];
        slot = 0;
    }
    if (n <= 0) return;
    const float decay = a.decay[h];
    const T* base = (const T*)a.qkv;
    const bool outputs = a.mode != kChunkLocal;        // (a chunk's pass from the empty state leaves its end state only)
    constexpr int NL = NR + 2;                         // staged elements a thread fetches: kBatch * row / 256
    T fetched[NL];

    auto fetch = [&](int b0) {
#pragma unroll
        for (int u = 0; u < NL; ++u) {
            const int e = threadIdx.x + u * (kWarps * 32);
            const int tt = e / row, j = e - tt * row;
            T v = from_f32<T>(0.0f);
            if (b0 + tt < n) {
                const T* r = base + (int64_t)(t0 + b0 + tt) * a.ld;
                if (j < DP) {
                    if (j < D && outputs) v = r[a.q_col + h * D + j];
                } else if (j < 2 * DP) {
                    if (j - DP < D) v = r[a.k_col + h * D + (j - DP)];
                } else if (c0 + (j - 2 * DP) < E) {
                    v = r[a.v_col + h * E + c0 + (j - 2 * DP)];
                }
            }
            fetched[u] = v;
        }
    };
    auto put = [&](float* buf) {
#pragma unroll
        for (int u = 0; u < NL; ++u) buf[threadIdx.x + u * (kWarps * 32)] = silu_of(fetched[u]);
    };

    pdl_wait();
    float S[NR];
    {
        const float* from = a.mode == kSequences ? a.state + (((int64_t)slot * a.H + h) * D) * E
                            : a.mode == kChunkFinal ? a.chunk_state + (((int64_t)blockIdx.z * a.H + h) * D) * E : nullptr;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = g * NR + i;
            S[i] = (from != nullptr && r < D && col < E) ? from[(int64_t)r * E + col] : 0.0f;
        }
    }
    fetch(0);
    put(stage);
    __syncthreads();

    // one token: S <- decay S + k v, and (with outputs) this warp's share of S^T q
    auto token = [&](const float* q, float* pp_t) {
        const float4* k4 = reinterpret_cast<const float4*>(q + DP + g * NR);
        const float4* q4 = reinterpret_cast<const float4*>(q + g * NR);
        const float v = q[2 * DP + lane];
        float acc0 = 0.0f, acc1 = 0.0f;
#pragma unroll
        for (int i = 0; i < NR / 4; ++i) {
            const float4 kk = k4[i];
            S[4 * i + 0] = fmaf(decay, S[4 * i + 0], kk.x * v);
            S[4 * i + 1] = fmaf(decay, S[4 * i + 1], kk.y * v);
            S[4 * i + 2] = fmaf(decay, S[4 * i + 2], kk.z * v);
            S[4 * i + 3] = fmaf(decay, S[4 * i + 3], kk.w * v);
            if (outputs) {
                const float4 qq = q4[i];
                acc0 = fmaf(S[4 * i + 0], qq.x, acc0);
                acc1 = fmaf(S[4 * i + 1], qq.y, acc1);
                acc0 = fmaf(S[4 * i + 2], qq.z, acc0);
                acc1 = fmaf(S[4 * i + 3], qq.w, acc1);
            }
        }
        if (outputs) pp_t[g * kCols + lane] = acc0 + acc1;
    };

    int which = 0;
    for (int b0 = 0; b0 < n; b0 += kBatch) {
        const int cnt = min(kBatch, n - b0);
        const bool more = b0 + kBatch < n;
        if (more) fetch(b0 + kBatch);
        const float* buf = stage + which * kBatch * row;
        float* pp = part + which * kBatch * kWarps * kCols;
        if (cnt == kBatch) {
#pragma unroll 4
            for (int tt = 0; tt < kBatch; ++tt) token(buf + tt * row, pp + tt * kWarps * kCols);
        } else {
            for (int tt = 0; tt < cnt; ++tt) token(buf + tt * row, pp + tt * kWarps * kCols);
        }
        if (more) put(stage + (which ^ 1) * kBatch * row);
        __syncthreads();
        if (outputs) {
            // the 8 row groups' sums of each (token, column), added in the order of the groups
            for (int e = threadIdx.x; e < cnt * kCols; e += kWarps * 32) {
                const int tt = e / kCols, c = e - tt * kCols;
                if (c0 + c < E) {
                    float o = 0.0f;
#pragma unroll
                    for (int w = 0; w < kWarps; ++w) o += pp[(tt * kWarps + w) * kCols + c];
                    a.y[(int64_t)(t0 + b0 + tt) * a.H * E + (int64_t)h * E + c0 + c] = o;
                }
            }
        }
        which ^= 1;
    }
    if (a.mode != kChunkFinal) {
        float* to = a.mode == kSequences ? a.state + (((int64_t)slot * a.H + h) * D) * E
                                         : a.chunk_state + (((int64_t)blockIdx.z * a.H + h) * D) * E;
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int r = g * NR + i;
            if (r < D && col < E) to[(int64_t)r * E + col] = S[i];
        }
    }
}

// Per sequence, in the order of its chunks: the chunk's local end state gives way to the state the chunk starts from, and the
// running state moves on by decay^len times itself plus the local end state; the last one is the sequence's new state.
__global__ void lightning_carry_kernel(const float* __restrict__ decay, float* __restrict__ state, const int32_t* __restrict__ slots,
                                       const int32_t* __restrict__ chunks, const int32_t* __restrict__ first_chunk,
                                       float* __restrict__ chunk_state, int H, int64_t per_head) {
    pdl_launch_dependents();
    pdl_wait();
    const int seq = blockIdx.z, h = blockIdx.y;
    const int c_lo = first_chunk[seq], c_hi = first_chunk[seq + 1];
    if (c_lo >= c_hi) return;
    const float d = decay[h];
    float* st = state + ((int64_t)slots[seq] * H + h) * per_head;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < per_head; e += (int64_t)gridDim.x * blockDim.x) {
        float run = st[e];
        for (int c = c_lo; c < c_hi; ++c) {
            float* cs = chunk_state + ((int64_t)c * H + h) * per_head + e;
            const float local = *cs;
            *cs = run;
            run = fmaf(powf(d, (float)chunks[3 * c + 2]), run, local);
        }
        st[e] = run;
    }
}

template <typename T>
int launch_scan(const LightningArgs& a, int items, cudaStream_t stream) {
    const dim3 grid(ceil_div_i(a.E, kCols), a.H, items);
#define XS_GO(NR)                                                                                                        \
    do {                                                                                                                 \
        const size_t smem = (size_t)(2 * kBatch * (2 * kWarps * NR + kCols) + 2 * kBatch * kWarps * kCols) * sizeof(float); \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(lightning_scan_kernel<T, NR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        xs_launch(lightning_scan_kernel<T, NR>, grid, dim3(kWarps * 32), smem, stream, a);                               \
    } while (0)
    if (a.D <= 32) XS_GO(4);
    else if (a.D <= 64) XS_GO(8);
    else if (a.D <= 128) XS_GO(16);
    else XS_GO(32);
#undef XS_GO
    return 0;
}

}  // namespace

// qkv: [T, *] rows `ld` apart in the element type `dtype`; state [slots, H, D, E] and y [T, H * E] float32. With `chunks`
// ([n_chunks, 3] int32: sequence, first token, tokens; `first_chunk` [n_seqs + 1]; `chunk_state` [n_chunks, H, D, E] float32)
// the chunks run side by side in three launches.
XS_API int xs_lightning_scan(const void* qkv, int64_t ld, int q_col, int k_col, int v_col, const float* decay, float* state,
                             const int32_t* cu_seqlens, const int32_t* slots, float* y, int n_seqs, int H, int D, int E, int dtype,
                             const int32_t* chunks, const int32_t* first_chunk, int n_chunks, float* chunk_state,
                             cudaStream_t stream) {
    if (n_seqs == 0) return 0;
    XS_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && H > 0 && H <= 65535 && D > 0 && D <= 256 && E > 0,
               "lightning: %d sequences, %d heads of %d x %d (keys of at most 256)", n_seqs, H, D, E);
    XS_REQUIRE(chunks == nullptr || (first_chunk != nullptr && chunk_state != nullptr && n_chunks > 0 && n_chunks <= 65535),
               "lightning: %d chunks without their scratch", n_chunks);
    LightningArgs a = {qkv, ld, q_col, k_col, v_col, decay, state, cu_seqlens, slots, y, chunks, chunk_state, H, D, E, kSequences};
    if (chunks == nullptr) {
        XS_DISPATCH_DTYPE(dtype, TT, launch_scan<TT>(a, n_seqs, stream));
        XS_LAUNCH_CHECK("lightning_scan");
        return 0;
    }
    a.mode = kChunkLocal;
    XS_DISPATCH_DTYPE(dtype, TT, launch_scan<TT>(a, n_chunks, stream));
    XS_LAUNCH_CHECK("lightning_scan (chunks, local)");
    const int64_t per_head = (int64_t)D * E;
    xs_launch(lightning_carry_kernel, dim3(ceil_div_i(per_head, 256), H, n_seqs), dim3(256), 0, stream, decay, state, slots, chunks,
              first_chunk, chunk_state, H, per_head);
    XS_LAUNCH_CHECK("lightning_carry");
    a.mode = kChunkFinal;
    XS_DISPATCH_DTYPE(dtype, TT, launch_scan<TT>(a, n_chunks, stream));
    XS_LAUNCH_CHECK("lightning_scan (chunks, final)");
    return 0;
}
