// Routed experts (a mixture of small gated feed-forwards) and the clamped gated unit's activation.
//
// A step's tokens each choose `top` of E experts. Four kernels, none of which needs the host to know a count:
//   route    per token: the `top` largest float32 router logits (ties: the lower index), softmax over them alone
//   plan     one CTA: rows (token, choice) counted per expert, each given a place in an order sorted by expert, and
//            the list of row tiles (expert, first row, rows) that the products walk; its length stays on the device
//   product  out[row] = W[expert of row] x[source of row], tile by tile of the plan; the grid is sized by the most
//            tiles that T * top rows over E experts can make, surplus CTAs leave at once
//            (first product: rows gathered from the tokens, epilogue silu(gate) * up; second: rows in place)
//   combine  y[t] = sum_k weight[t, k] * out[place of (t, k)], in float32, in the order of k
// The generic product sums each output's K terms in an order that depends on K alone, as gemm_generic.cu does.
#include "common.cuh"

namespace {

constexpr int kMaxTop = 16;
constexpr int kLocalExperts = 64;

__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------- clamped gated unit
// out[t, f] = g * sigmoid(alpha g) * (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit); a row of gu is
// [F gate | F up], or with interleave 8 blocks of 8 gate columns and the 8 up columns of the same outputs.
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int F, int64_t ld,
                                   float limit, float alpha, float shift, int interleave) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / F;
        const int f = (int)(i - t * F);
        const int64_t gi = interleave ? (int64_t)(f / interleave) * 2 * interleave + f % interleave : f;
        const int64_t ui = interleave ? gi + interleave : (int64_t)F + f;
        const float g = fminf(to_f32(gu[t * ld + gi]), limit);
        const float u = fminf(fmaxf(to_f32(gu[t * ld + ui]), -limit), limit);
        out[i] = from_f32<T>(g * sigmoid_f(alpha * g) * (u + shift));
    }
}

// 8 outputs a thread, 16-byte loads and stores (bfloat16, F a multiple of 8, rows 16-byte aligned).
__global__ void clamped_glu_bf16x8_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, int64_t total8,
                                          int F8, int64_t ld, float limit, float alpha, float shift, int interleave) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = i / F8;
        const int j = (int)(i - t * F8);
        const __nv_bfloat16* row = gu + t * ld;
        const uint4 g = *reinterpret_cast<const uint4*>(row + (interleave ? 16 * j : 8 * j));
        const uint4 u = *reinterpret_cast<const uint4*>(row + (interleave ? 16 * j + 8 : 8 * (int64_t)F8 + 8 * j));
        const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
        const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
        uint4 o;
        __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 gf = __bfloat1622float2(gp[k]), uf = __bfloat1622float2(up[k]);
            gf.x = fminf(gf.x, limit);
            gf.y = fminf(gf.y, limit);
            uf.x = fminf(fmaxf(uf.x, -limit), limit);
            uf.y = fminf(fmaxf(uf.y, -limit), limit);
            op[k] = __floats2bfloat162_rn(gf.x * sigmoid_f(alpha * gf.x) * (uf.x + shift), gf.y * sigmoid_f(alpha * gf.y) * (uf.y + shift));
        }
        *reinterpret_cast<uint4*>(out + t * 8 * (int64_t)F8 + 8 * j) = o;
    }
}

// ------------------------------------------------------------------------------------------------- squared ReLU
// out = max(x, 0)^2, the square taken in float32.
template <typename T>
__global__ void relu_squared_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(x[i]), 0.0f);
        out[i] = from_f32<T>(v * v);
    }
}

__global__ void relu_squared_bf16x8_kernel(const uint4* __restrict__ x, uint4* __restrict__ out, int64_t total8) {
    pdl_launch_dependents();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
        uint4 raw = x[i];
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 f = __bfloat1622float2(p[k]);
            f.x = fmaxf(f.x, 0.0f);
            f.y = fmaxf(f.y, 0.0f);
            p[k] = __floats2bfloat162_rn(f.x * f.x, f.y * f.y);
        }
        out[i] = raw;
    }
}

// ----------------------------------------------------------------------------------------------------- router logits
// logits[t, e] = x[t] . w[e] in float32: a warp per (token, expert) pair walks both rows (16-byte loads where the rows
// allow, eight loads in flight a lane); a lane's partial sums and the warp's reduction run in an order that depends on
// K alone, whatever else is in the batch.
template <typename T>
__global__ void moe_logits_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w, float* __restrict__ logits,
                                  int Tn, int E, int K, int vec) {
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int64_t pair = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= (int64_t)Tn * E) return;
    const int t = (int)(pair / E), e = (int)(pair % E);
    const T* xr = x + (int64_t)t * ldx;
    const T* we = w + (int64_t)e * K;
    pdl_wait();
    float acc = 0.0f;
    if (vec) {          // bfloat16 rows in whole 16-byte pieces
        const uint4* x8 = reinterpret_cast<const uint4*>(xr);
        const uint4* w8 = reinterpret_cast<const uint4*>(we);
#pragma unroll 4
        for (int i = lane; i < (K >> 3); i += 32) {
            const uint4 a = x8[i], b = w8[i];
            const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 af = __bfloat1622float2(a2[j]), bf = __bfloat1622float2(b2[j]);
                acc = fmaf(af.x, bf.x, acc);
                acc = fmaf(af.y, bf.y, acc);
            }
        }
    } else {
#pragma unroll 8
        for (int k = lane; k < K; k += 32) acc = fmaf(to_f32(xr[k]), to_f32(we[k]), acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) logits[pair] = acc;
}

// ------------------------------------------------------------------------------------------------------------ route
__global__ void moe_route_kernel(const float* __restrict__ logits, int ld, int T, int E, int top, float scale,
                                 int32_t* __restrict__ ids, float* __restrict__ wts) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const float* zg = logits + (int64_t)t * ld;
    float zl[kLocalExperts];            // up to 64 logits are read once, all loads in flight
    if (E <= kLocalExperts) {
#pragma unroll
        for (int e = 0; e < kLocalExperts; ++e) zl[e] = e < E ? zg[e] : 0.0f;
    }
    int chosen[kMaxTop];
    float val[kMaxTop];
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float bv = 0.0f;
        for (int e = 0; e < E; ++e) {
            bool taken = false;
            for (int j = 0; j < k; ++j) taken |= chosen[j] == e;
            if (taken) continue;
            const float v = E <= kLocalExperts ? zl[e] : zg[e];
            if (best < 0 || v > bv) {
                best = e;
                bv = v;
            }
        }
        chosen[k] = best;
        val[k] = bv;
    }
    float sum = 0.0f;
    const float largest = val[0];
    for (int k = 0; k < top; ++k) {
        val[k] = expf(val[k] - largest);
        sum += val[k];
    }
    for (int k = 0; k < top; ++k) {
        ids[(int64_t)t * top + k] = chosen[k];
        wts[(int64_t)t * top + k] = val[k] / sum * scale;
    }
}

// A warp per token (E <= 256): a lane holds logits lane, lane + 32, ...; each of the `top` rounds finds the largest logit
// left (ties: the lower index) by a reduction over the warp.
__global__ void moe_route_warp_kernel(const float* __restrict__ logits, int ld, int T, int E, int top, float scale,
                                      int32_t* __restrict__ ids, float* __restrict__ wts) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (t >= T) return;
    const float* z = logits + (int64_t)t * ld;
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = lane + 32 * j < E ? z[lane + 32 * j] : -INFINITY;
    float mine = 0.0f, largest = 0.0f, sum = 0.0f;
    int mine_id = 0;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 1 << 30;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int e = lane + 32 * j;
            if (e < E && (v[j] > bv || (v[j] == bv && e < bi))) {
                bv = v[j];
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (lane + 32 * j == bi) v[j] = -INFINITY;       // taken (a logit of -inf itself is never chosen twice: its index is)
        if (k == 0) largest = bv;
        const float p = expf(bv - largest);
        sum += p;
        if (lane == k) {
            mine = p;
            mine_id = bi;
        }
    }
    if (lane < top) {
        ids[(int64_t)t * top + lane] = mine_id;
        wts[(int64_t)t * top + lane] = mine / sum * scale;
    }
}

// Routing by sigmoid scores with a limit on groups. A token's scores are s = sigmoid(logits); its choice scores c = s +
// correction (a number per expert). The experts form `groups` equal groups of neighbours; a group's score is the sum of its
// `group_top` largest choice scores, and only experts of the `keep` best groups can be chosen (the others count as minus
// infinity, so negative choice scores still beat them). The `top` largest choice scores are chosen (ties: the lower index,
// for groups and for experts); the weights are the chosen experts' s times `scale`, not normed to sum 1 unless `renorm`.
// `score` 1: s is the softmax over all E logits instead of their sigmoids. Experts from `real` on have no weights (their
// output is their input): a choice of one is written as id -1, with its weight.
// A warp per token; the token's s and c stand in shared memory (2 E floats a warp).
__global__ void moe_route_grouped_kernel(const float* __restrict__ logits, int ld, int T, int E, int top,
                                         const float* __restrict__ correction, int groups, int keep, int group_top, float scale,
                                         int renorm, int score, int real, int32_t* __restrict__ ids, float* __restrict__ wts) {
    extern __shared__ float route_smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    float* s = route_smem + (size_t)warp * (2 * E + groups);
    float* c = s + E;
    float* gs = c + E;
    const float* z = logits + (int64_t)t * ld;
    // score 1: the scores are the softmax over all E logits (largest first taken off, sum in the warp's fixed order)
    float z_max = -INFINITY, z_sum = 1.0f;
    if (score == 1) {
        for (int e = lane; e < E; e += 32) z_max = fmaxf(z_max, z[e]);
        z_max = warp_max(z_max);
        z_sum = 0.0f;
        for (int e = lane; e < E; e += 32) z_sum += expf(z[e] - z_max);
        z_sum = warp_sum(z_sum);
    }
    for (int e = lane; e < E; e += 32) {
        const float v = score == 1 ? expf(z[e] - z_max) / z_sum : 1.0f / (1.0f + expf(-z[e]));
        s[e] = v;
        c[e] = v + (correction != nullptr ? correction[e] : 0.0f);
    }
    __syncwarp();
    const int per = E / groups;
    if (groups > 1 && keep < groups) {
        for (int g = lane; g < groups; g += 32) {
            // the sum of the group's `group_top` largest choice scores: pick them one after another
            float sum = 0.0f;
            int taken[8];
            const int n = min(group_top, per);
            for (int k = 0; k < n; ++k) {
                float bv = -INFINITY;
                int bi = -1;
                for (int j = 0; j < per; ++j) {
                    bool used = false;
                    for (int q = 0; q < k; ++q) used |= taken[q] == j;
                    if (!used && (bi < 0 || c[g * per + j] > bv)) {
                        bv = c[g * per + j];
                        bi = j;
                    }
                }
                taken[k] = bi;
                sum += bv;
            }
            gs[g] = sum;
        }
        __syncwarp();
        // groups that are not among the `keep` best: rank = how many groups beat this one (ties: the lower index wins)
        for (int g = lane; g < groups; g += 32) {
            int rank = 0;
            for (int o = 0; o < groups; ++o) rank += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
            if (rank >= keep)
                for (int j = 0; j < per; ++j) c[g * per + j] = -INFINITY;
        }
        __syncwarp();
    }
    float mine = 0.0f, sum = 0.0f;
    int mine_id = 0;
    for (int k = 0; k < top; ++k) {
        float bv = -INFINITY;
        int bi = 1 << 30;
        for (int e = lane; e < E; e += 32) {
            const float v = c[e];
            if (v > bv || (v == bv && e < bi)) {
                bv = v;
                bi = e;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) {
                bv = ov;
                bi = oi;
            }
        }
        if (bi >= E) bi = 0;                    // (only a row of NaNs comes here)
        const float w = s[bi];
        __syncwarp();
        if (lane == 0) c[bi] = -INFINITY;       // taken (enough experts are open, so none at minus infinity is ever chosen)
        __syncwarp();
        sum += w;
        if (lane == k) {
            mine = w;
            mine_id = bi;
        }
    }
    if (lane < top) {
        ids[(int64_t)t * top + lane] = mine_id < real ? mine_id : -1;        // (an expert without weights: its input passes)
        wts[(int64_t)t * top + lane] = (renorm ? mine / sum : mine) * scale;
    }
}

// ------------------------------------------------------------------------------------------------------------- plan
// meta: [0] number of tiles; then per tile 3 words (expert, first row, rows) from meta[4] on.
// pad: every expert's rows start at a multiple of tile_rows (places that no row takes get source -1; rows_cap places).
__global__ void moe_plan_kernel(const int32_t* __restrict__ ids, int n, int E, int tile_rows, int pad, int rows_cap,
                                int32_t* __restrict__ place, int32_t* __restrict__ source, int32_t* __restrict__ meta) {
    extern __shared__ int32_t sm[];      // count[E], first[E], next[E]
    int32_t* count = sm;
    int32_t* first = sm + E;
    int32_t* next = sm + 2 * E;
    pdl_launch_dependents();
    pdl_wait();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    if (pad)
        for (int i = threadIdx.x; i < rows_cap; i += blockDim.x) source[i] = -1;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        if (ids[i] >= 0) atomicAdd(&count[ids[i]], 1);      // (a row without an expert, id -1, takes no place)
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            first[e] = at;
            next[e] = at;
            for (int r = 0; r < count[e]; r += tile_rows) {
                int32_t* m = meta + 4 + 3 * tiles;
                m[0] = e;
                m[1] = at + r;
                m[2] = min(tile_rows, count[e] - r);
                ++tiles;
            }
            at += count[e];
            if (pad) at = (at + tile_rows - 1) / tile_rows * tile_rows;
        }
        meta[0] = tiles;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        if (ids[i] < 0) {
            place[i] = -1;
            continue;
        }
        const int p = atomicAdd(&next[ids[i]], 1);
        place[i] = p;
        source[p] = i;
    }
}

// ---------------------------------------------------------------------------------------------------------- product
// out[row, :] = W[e] . x[src(row)] for the rows of one tile; W is [E, N(,2), K] stacked. GLU: W[e] is [2 N, K], gate
// rows first, and out = silu(gate) * up. src(row) = source[row] / top when `source` is given (rows gathered from the
// tokens), else row.
constexpr int TM = 64, TN = 64, TK = 32;

template <typename TX, typename TO, bool GLU>
__global__ void __launch_bounds__(256)
moe_gemm_kernel(const TX* __restrict__ x, int64_t ldx, const TX* __restrict__ w, TO* __restrict__ out, int64_t ldo,
                const int32_t* __restrict__ source, int top, const int32_t* __restrict__ meta, int N, int K, float limit,
                float alpha, float shift) {
    __shared__ float xs[TK][TM + 1];
    __shared__ float ws[GLU ? 2 : 1][TK][TN + 1];
    __shared__ int64_t src_row[TM];
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.y >= meta[0]) return;
    const int32_t* mt = meta + 4 + 3 * blockIdx.y;
    const int e = mt[0], row0 = mt[1], rows = mt[2];
    const int n0 = blockIdx.x * TN;
    const TX* we = w + (int64_t)e * (GLU ? 2 : 1) * N * K;
    if (threadIdx.x < TM) {
        const int r = row0 + threadIdx.x;
        src_row[threadIdx.x] = threadIdx.x < rows ? (source != nullptr ? source[r] / top : r) : -1;
    }
    __syncthreads();
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[GLU ? 2 : 1][4][4];
#pragma unroll
    for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[g][i][j] = 0.0f;
    for (int k0 = 0; k0 < K; k0 += TK) {
        for (int idx = threadIdx.x; idx < TM * TK; idx += 256) {
            const int r = idx >> 5, k = idx & 31;
            const int gn = n0 + r, gk = k0 + k;
            const int64_t sr = src_row[r];
            xs[k][r] = (sr >= 0 && gk < K) ? to_f32(x[sr * ldx + gk]) : 0.0f;
            ws[0][k][r] = (gn < N && gk < K) ? to_f32(we[(int64_t)gn * K + gk]) : 0.0f;
            if (GLU) ws[GLU ? 1 : 0][k][r] = (gn < N && gk < K) ? to_f32(we[(int64_t)(N + gn) * K + gk]) : 0.0f;
        }
        __syncthreads();
        float part[GLU ? 2 : 1][4][4];
#pragma unroll
        for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) part[g][i][j] = 0.0f;
#pragma unroll
        for (int k = 0; k < TK; ++k) {
            float a[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[k][ty * 4 + i];
#pragma unroll
            for (int g = 0; g < (GLU ? 2 : 1); ++g) {
                float b[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = ws[g][k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) part[g][i][j] = fmaf(a[i], b[j], part[g][i][j]);
            }
        }
#pragma unroll
        for (int g = 0; g < (GLU ? 2 : 1); ++g)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[g][i][j] += part[g][i][j];
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[0][i][j];
            if (GLU) {
                // the gate and the up product are rounded to the activation type first, as two separate products' would be
                float g = to_f32(from_f32<TO>(v)), u = to_f32(from_f32<TO>(acc[GLU ? 1 : 0][i][j]));
                if (limit > 0.0f) {          // the clamped unit: g = min(gate, limit), u = clamp(up, -limit, limit)
                    g = fminf(g, limit);
                    u = fminf(fmaxf(u, -limit), limit);
                    v = g * sigmoid_f(alpha * g) * (u + shift);
                } else {
                    v = g * sigmoid_f(g) * u;
                }
            }
            out[(int64_t)(row0 + r) * ldo + gn] = from_f32<TO>(v);
        }
    }
}

// ----------------------------------------------------------------------------------------------------------- gather
// sorted[r, :] = x[source[r] / top, :] (zeros where source[r] < 0), 16 bytes a thread.
__global__ void moe_gather_kernel(const uint4* __restrict__ x, int64_t ldx16, const int32_t* __restrict__ source, int top,
                                  uint4* __restrict__ sorted, int K16) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int src = source[r];
    const uint4* from = x + (int64_t)(src < 0 ? 0 : src / top) * ldx16;
    for (int c = threadIdx.x; c < K16; c += blockDim.x)
        sorted[(int64_t)r * K16 + c] = src < 0 ? make_uint4(0u, 0u, 0u, 0u) : from[c];
}

// ---------------------------------------------------------------------------------------------------------- combine
template <typename TI, typename TO>
__global__ void moe_combine_kernel(const TI* __restrict__ rows_out, const int32_t* __restrict__ place,
                                   const float* __restrict__ wts, TO* __restrict__ y, int H, int top,
                                   const TI* __restrict__ shared, const float* __restrict__ shared_gate, int ld_gate,
                                   const TI* __restrict__ passed, int64_t ld_passed) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    // a unit that every token uses joins the sum, times sigmoid of the token's gate logit (1 without one)
    const float sg = shared == nullptr ? 0.0f : shared_gate == nullptr ? 1.0f : sigmoid_f(shared_gate[(int64_t)t * ld_gate]);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
        float v = shared == nullptr ? 0.0f : sg * to_f32(shared[(int64_t)t * H + c]);
        for (int k = 0; k < top; ++k) {
            // (a choice without a place is an expert that hands its input through: `passed` holds the tokens' inputs)
            const int pl = place[(int64_t)t * top + k];
            const float r = pl >= 0 ? to_f32(rows_out[(int64_t)pl * H + c]) : passed != nullptr ? to_f32(passed[(int64_t)t * ld_passed + c]) : 0.0f;
            v = fmaf(wts[(int64_t)t * top + k], r, v);
        }
        y[(int64_t)t * H + c] = from_f32<TO>(v);
    }
}

}  // namespace

XS_API int xs_clamped_glu(const void* gu, void* out, int dtype, int T, int F, int64_t ld, float limit, float alpha,
                          float shift, int interleave, cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && F > 0 && ld >= 2 * (int64_t)F, "clamped_glu: %d rows, %d columns, stride %lld", T, F, (long long)ld);
    XS_REQUIRE(interleave == 0 || (interleave == 8 && F % 8 == 0), "clamped_glu: interleave %d with %d columns", interleave, F);
    if (dtype == XS_BF16 && F % 8 == 0 && ld % 8 == 0 && (uintptr_t)gu % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const int64_t total8 = (int64_t)T * (F / 8);
        const int blocks8 = (int)((total8 + 255) / 256 < 148 * 32 ? (total8 + 255) / 256 : 148 * 32);
        xs_launch(clamped_glu_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (const __nv_bfloat16*)gu, (__nv_bfloat16*)out,
                  total8, F / 8, ld, limit, alpha, shift, interleave);
        XS_LAUNCH_CHECK("clamped_glu");
        return 0;
    }
    const int64_t total = (int64_t)T * F;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(clamped_glu_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (const TT*)gu, (TT*)out, total,
                                F, ld, limit, alpha, shift, interleave));
    XS_LAUNCH_CHECK("clamped_glu");
    return 0;
}

XS_API int xs_relu_squared(const void* x, void* out, int dtype, int64_t total, cudaStream_t stream) {
    if (total == 0) return 0;
    XS_REQUIRE(total > 0, "relu_squared: %lld elements", (long long)total);
    if (dtype == XS_BF16 && total % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0) {
        const int64_t total8 = total / 8;
        const int blocks8 = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
        xs_launch(relu_squared_bf16x8_kernel, dim3(blocks8), dim3(256), 0, stream, (const uint4*)x, (uint4*)out, total8);
        XS_LAUNCH_CHECK("relu_squared");
        return 0;
    }
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    XS_DISPATCH_DTYPE(dtype, TT, xs_launch(relu_squared_kernel<TT>, dim3(blocks), dim3(256), 0, stream, (const TT*)x, (TT*)out, total));
    XS_LAUNCH_CHECK("relu_squared");
    return 0;
}

XS_API int xs_moe_logits(const void* x, int64_t ldx, const void* w, float* logits, int T, int E, int K, int dtype,
                         cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && E > 0 && K > 0, "moe_logits: %d tokens, %d experts, width %d", T, E, K);
    const int vec = dtype == XS_BF16 && K % 8 == 0 && ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)w % 16 == 0;
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(moe_logits_kernel<TT>, dim3(ceil_div_i((int64_t)T * E, 4)), dim3(128), 0, stream, (const TT*)x, ldx,
                                (const TT*)w, logits, T, E, K, vec));
    XS_LAUNCH_CHECK("moe_logits");
    return 0;
}

// logits: rows of `ld` >= E floats, of which the first E are the experts' (a caller may keep other per-token numbers behind
// them). The weights are the softmax over the chosen logits (which is the softmax over all of them, divided by the chosen
// ones' sum) times `scale`.
XS_API int xs_moe_route(const float* logits, int ld, int T, int E, int top, float scale, int32_t* ids, float* wts,
                        cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && E > 0 && top > 0 && top <= E && top <= kMaxTop && ld >= E,
               "moe_route: %d tokens, %d experts (row stride %d), top %d (at most %d)", T, E, ld, top, kMaxTop);
    if (E <= 256 && E > top)
        xs_launch(moe_route_warp_kernel, dim3(ceil_div_i(T, 4)), dim3(128), 0, stream, logits, ld, T, E, top, scale, ids, wts);
    else
        xs_launch(moe_route_kernel, dim3(ceil_div_i(T, 32)), dim3(32), 0, stream, logits, ld, T, E, top, scale, ids, wts);
    XS_LAUNCH_CHECK("moe_route");
    return 0;
}

XS_API int xs_moe_route_grouped(const float* logits, int ld, int T, int E, int top, const float* correction, int groups, int keep,
                                int group_top, float scale, int renorm, int score, int real, int32_t* ids, float* wts,
                                cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && E > 0 && top > 0 && top <= E && top <= kMaxTop && ld >= E,
               "moe_route_grouped: %d tokens, %d experts (row stride %d), top %d (at most %d)", T, E, ld, top, kMaxTop);
    XS_REQUIRE(groups > 0 && E % groups == 0 && keep > 0 && keep <= groups && group_top > 0 && group_top <= 8,
               "moe_route_grouped: %d experts in %d groups of which %d are kept (a group's %d largest count)", E, groups, keep, group_top);
    XS_REQUIRE((int64_t)keep * (E / groups) >= top, "moe_route_grouped: %d groups of %d experts cannot give %d choices", keep, E / groups, top);
    XS_REQUIRE((score == 0 || score == 1) && real > 0 && real <= E, "moe_route_grouped: score %d (0 sigmoid, 1 softmax), %d of %d experts with weights",
               score, real, E);
    const size_t per_warp = (size_t)(2 * E + groups) * sizeof(float);
    XS_REQUIRE(per_warp <= 40 * 1024, "moe_route_grouped: %d experts are more than the kernel's shared memory holds", E);
    const int warps = per_warp * 4 <= 40 * 1024 ? 4 : 1;
    xs_launch(moe_route_grouped_kernel, dim3(ceil_div_i(T, warps)), dim3(32 * warps), per_warp * warps, stream, logits, ld, T, E, top,
              correction, groups, keep, group_top, scale, renorm, score, real, ids, wts);
    XS_LAUNCH_CHECK("moe_route_grouped");
    return 0;
}

XS_API int xs_moe_tile_rows() { return TM; }

// How many tiles n rows over E experts can make at most: whole tiles, and a partly filled one per expert.
XS_API int xs_moe_max_tiles(int n, int E) { return n / TM + (n < E ? n : E); }

// tile_rows 0: the generic product's tiles, rows packed. tile_rows > 0: tiles of that many rows, every expert's rows
// padded to whole tiles; `source` then has rows_cap >= tile_rows * xs_moe_max_tiles_of(n, E, tile_rows) places.
XS_API int xs_moe_max_tiles_of(int n, int E, int tile_rows) { return n / tile_rows + (n < E ? n : E); }

XS_API int xs_moe_plan(const int32_t* ids, int n, int E, int tile_rows, int rows_cap, int32_t* place, int32_t* source,
                       int32_t* meta, cudaStream_t stream) {
    if (n == 0) return 0;
    XS_REQUIRE(n > 0 && E > 0 && E <= 4096, "moe_plan: %d rows, %d experts (at most 4096)", n, E);
    XS_REQUIRE(tile_rows == 0 || rows_cap >= tile_rows * xs_moe_max_tiles_of(n, E, tile_rows), "moe_plan: %d places for %d rows in tiles of %d",
               rows_cap, n, tile_rows);
    xs_launch(moe_plan_kernel, dim3(1), dim3(1024), (size_t)3 * E * sizeof(int32_t), stream, ids, n, E,
              tile_rows > 0 ? tile_rows : TM, tile_rows > 0 ? 1 : 0, rows_cap, place, source, meta);
    XS_LAUNCH_CHECK("moe_plan");
    return 0;
}

// x and w share an element type; out is float32 or that type. glu: w is [E, 2 N, K] and out = silu(gate) * up, or with
// limit > 0 the clamped unit's g * sigmoid(alpha g) * (u + shift), g = min(gate, limit), u = clamp(up, -limit, limit).
XS_API int xs_moe_gemm(const void* x, int64_t ldx, const void* w, void* out, int64_t ldo, const int32_t* source, int top,
                       const int32_t* meta, int max_tiles, int N, int K, int glu, float limit, float alpha, float shift,
                       int in_dtype, int out_dtype, cudaStream_t stream) {
    if (max_tiles == 0) return 0;
    XS_REQUIRE(max_tiles > 0 && max_tiles <= 65535 && N > 0 && K > 0 && top > 0, "moe_gemm: %d tiles, N %d, K %d", max_tiles, N, K);
    XS_REQUIRE(in_dtype == out_dtype, "moe_gemm: element types in %d, out %d", in_dtype, out_dtype);
    const dim3 grid(ceil_div_i(N, TN), max_tiles);
#define XS_GO(TT)                                                                                                   \
    do {                                                                                                            \
        if (glu)                                                                                                    \
            xs_launch(moe_gemm_kernel<TT, TT, true>, grid, dim3(256), 0, stream, (const TT*)x, ldx, (const TT*)w,   \
                      (TT*)out, ldo, source, top, meta, N, K, limit, alpha, shift);                                                      \
        else                                                                                                        \
            xs_launch(moe_gemm_kernel<TT, TT, false>, grid, dim3(256), 0, stream, (const TT*)x, ldx, (const TT*)w,  \
                      (TT*)out, ldo, source, top, meta, N, K, limit, alpha, shift);                                                      \
    } while (0)
    XS_DISPATCH_DTYPE(in_dtype, TT, XS_GO(TT));
#undef XS_GO
    XS_LAUNCH_CHECK("moe_gemm");
    return 0;
}

// x rows of K bfloat16 (K a multiple of 8, rows 16-byte aligned) into the plan's padded order.
XS_API int xs_moe_gather(const void* x, int64_t ldx, const int32_t* source, int top, void* sorted, int rows_cap, int K,
                         cudaStream_t stream) {
    if (rows_cap == 0) return 0;
    XS_REQUIRE(K > 0 && K % 8 == 0 && ldx % 8 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)sorted % 16 == 0 && top > 0,
               "moe_gather: rows of %d (stride %lld) are not 16-byte pieces", K, (long long)ldx);
    xs_launch(moe_gather_kernel, dim3(rows_cap), dim3(K / 8 >= 256 ? 256 : 128), 0, stream, (const uint4*)x, ldx / 8, source, top,
              (uint4*)sorted, K / 8);
    XS_LAUNCH_CHECK("moe_gather");
    return 0;
}

XS_API int xs_moe_combine(const void* rows_out, const int32_t* place, const float* wts, void* y, int T, int H, int top,
                          const void* shared, const float* shared_gate, int ld_gate, const void* passed, int64_t ld_passed, int dtype,
                          cudaStream_t stream) {
    if (T == 0) return 0;
    XS_REQUIRE(T > 0 && H > 0 && top > 0, "moe_combine: %d tokens of %d, top %d", T, H, top);
    XS_DISPATCH_DTYPE(dtype, TT,
                      xs_launch(moe_combine_kernel<TT, TT>, dim3(T), dim3(H >= 1024 ? 256 : 128), 0, stream,
                                (const TT*)rows_out, place, wts, (TT*)y, H, top, (const TT*)shared, shared_gate, ld_gate,
                                (const TT*)passed, ld_passed));
    XS_LAUNCH_CHECK("moe_combine");
    return 0;
}
