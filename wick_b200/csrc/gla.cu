// Gated linear attention: a recurrence per head whose state is a matrix of key channels by value elements, with a decay
// per key channel and token, for steps of any shape over per-sequence state records.
//
// The input projection's float32 partial sums hold, per token, [q: H dk | k: H dk | v: H dv | g: H dv | low: r]
// (H heads, dk key channels, dv value elements, r the rank of the decay's two-step projection).
//
//   prepare : q <- q * q_scale;  z = W2 low + b (H dk numbers);  a = exp(-softplus(-z) / tau) = sigmoid(z)^(1 / tau);
//             the token's row [q | k | a | v] goes out as float32
//   scan    : S_t = diag(a_t) S_(t-1) + k_t v_t^T  (dk x dv per head);  o_t = S_t^T q_t
//   out     : every head's o is divided by its root mean square over dv (eps inside the root) and multiplied by a weight
//             of dv numbers that the heads share, then by silu(g); the result goes out in the activation type
//
// A sequence's record (float32) is the state as [H][dv][dk] (a column of S, the dk numbers that meet one element of v,
// lies together).  Everything here is float32 arithmetic; a token's numbers depend on its own sequence alone.  A step of
// few tokens adds them in the same order whatever its shape; a long prompt step scanned in chunks (below) rounds the
// state differently, and no more than that.
#include "common.cuh"

namespace wick {

constexpr int GLA_ROWS = 16;                    // state numbers a thread keeps of one column, at most
constexpr int GLA_COLS = 4;                     // columns of the state a thread keeps

__device__ __forceinline__ bool gla_chunk_of(int slot, int n_seqs, const int* __restrict__ cu_seqlens, int chunk, int& b, int& first,
                                             int& len) {
    int at = 0;
    for (b = 0; b < n_seqs; ++b) {
        const int t0 = cu_seqlens[b], q = cu_seqlens[b + 1] - t0, nc = (q + chunk - 1) / chunk;
        if (slot < at + nc) {
            const int c = slot - at;
            first = t0 + c * chunk;
            len = min(chunk, q - c * chunk);
            return true;
        }
        at += nc;
    }
    return false;
}

template <int BYTES>
__device__ __forceinline__ void gla_cp_async(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(d), "l"(src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void gla_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT>
__device__ __forceinline__ void gla_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory"); }

__device__ __forceinline__ float gla_sum_parts(const float* __restrict__ parts, int splits, int64_t split_stride, int64_t at) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += parts[s * split_stride + at];
    return v;
}

constexpr int GLA_PREP_THREADS = 256;             // channels a block of the preparation takes
constexpr int GLA_PREP_RANK = 32;                 // a thread keeps its row of W2 in registers up to this rank

// grid (ceil(tokens / PB), ceil(H dk / 256) + ceil(H dv / 256)): a block takes 256 key channels (q, k and the decay) or 256
// value elements of PB tokens, so that a thread's row of W2 is read once for all of them and its PB tokens' numbers are on
// their way from memory at once.  out row: [q * q_scale | k | a | v], 3 H dk + H dv numbers.
template <int PB, bool ONE>
__global__ void __launch_bounds__(GLA_PREP_THREADS)
gla_prepare_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, int cols, int HK, int HV, int rank,
                   const float* __restrict__ w2, const float* __restrict__ b2, float q_scale, float inv_tau,
                   float* __restrict__ out, int n, int stage) {
    extern __shared__ float low[];                                       // [PB][rank], then (stage) the block's rows of W2
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    // (ONE: the projection came as one sum; a plain load each, so that a thread's loads are all on their way before the first is used)
    auto ld = [&](int64_t at) { return ONE ? parts[at] : gla_sum_parts(parts, splits, split_stride, at); };
    const int tid = threadIdx.x, t0 = blockIdx.x * PB, nt = min(PB, n - t0);
    const int tiles_k = (HK + GLA_PREP_THREADS - 1) / GLA_PREP_THREADS;
    const int low_col = 2 * HK + 2 * HV, channels = 3 * HK + HV;
    if ((int)blockIdx.y >= tiles_k) {
        const int c = ((int)blockIdx.y - tiles_k) * GLA_PREP_THREADS + tid;
        if (c >= HV) return;
        float v[PB];
#pragma unroll
        for (int i = 0; i < PB; ++i) v[i] = i < nt ? ld((int64_t)(t0 + i) * cols + 2 * HK + c) : 0.f;
#pragma unroll
        for (int i = 0; i < PB; ++i)
            if (i < nt) out[(int64_t)(t0 + i) * channels + 3 * HK + c] = v[i];
        return;
    }
    const int c = blockIdx.y * GLA_PREP_THREADS + tid;
    float qv[PB], kv[PB];
#pragma unroll
    for (int i = 0; i < PB; ++i) {
        const bool in = i < nt && c < HK;
        const int64_t row = (int64_t)(t0 + i) * cols;
        qv[i] = in ? ld(row + c) : 0.f;
        kv[i] = in ? ld(row + HK + c) : 0.f;
    }
    for (int idx = tid; idx < nt * rank; idx += GLA_PREP_THREADS) {
        const int i = idx / rank, j = idx - i * rank;
        low[idx] = ld((int64_t)(t0 + i) * cols + low_col + j);
    }
    // The block's 256 rows of W2 lie together in memory: they come in whole lines and wait in shared memory, a row's
    // numbers an odd count apart (thread c then reads row c without meeting its neighbours' banks).
    float* wt = low + PB * rank;
    const int ws = rank | 1, c0 = blockIdx.y * GLA_PREP_THREADS;
    if (stage) {
        const int64_t most = (int64_t)(HK - c0) * rank;
        for (int idx = tid; idx < GLA_PREP_THREADS * rank && idx < most; idx += GLA_PREP_THREADS) {
            const int r = idx / rank;
            wt[r * ws + (idx - r * rank)] = w2[(int64_t)c0 * rank + idx];
        }
    }
    __syncthreads();
    if (c >= HK) return;
    const float* wr = stage ? wt + tid * ws : w2 + (int64_t)c * rank;
    const float bias = b2 ? b2[c] : 0.f;
    const bool held = rank <= GLA_PREP_RANK;
    float w[GLA_PREP_RANK];
#pragma unroll
    for (int j = 0; j < GLA_PREP_RANK; ++j) w[j] = (held && j < rank) ? wr[j] : 0.f;
#pragma unroll
    for (int i = 0; i < PB; ++i) {
        if (i >= nt) break;
        const float* li = low + i * rank;
        float z = bias;
        if (held) {
#pragma unroll
            for (int j = 0; j < GLA_PREP_RANK; ++j)
                if (j < rank) z = fmaf(w[j], li[j], z);
        } else {
            for (int j = 0; j < rank; ++j) z = fmaf(wr[j], li[j], z);
        }
        float* o = out + (int64_t)(t0 + i) * channels;
        o[c] = qv[i] * q_scale;
        o[HK + c] = kv[i];
        // log sigmoid(z) = -softplus(-z)
        const float sp = -z > 20.0f ? -z : log1pf(expf(-z));
        o[2 * HK + c] = expf(-sp * inv_tau);
    }
}

// The sums of four columns over the LN threads that share them (see the state-space scan: the same exchange).
template <int LN>
__device__ __forceinline__ float gla_sum_columns(float (&a)[4], int sub, int& col, bool& writes) {
    constexpr unsigned ALL = 0xffffffffu;
    if (LN < 4) {
#pragma unroll
        for (int o = LN / 2; o > 0; o >>= 1)
#pragma unroll
            for (int c = 0; c < 4; ++c) a[c] += __shfl_xor_sync(ALL, a[c], o);
        col = -1;
        writes = sub == 0;
        return 0.f;
    }
    constexpr int O1 = LN >= 4 ? LN / 2 : 1, O2 = LN >= 4 ? LN / 4 : 1;
    const bool hi = (sub & O1) != 0, hi2 = (sub & O2) != 0;
    const float k0 = (hi ? a[2] : a[0]) + __shfl_xor_sync(ALL, hi ? a[0] : a[2], O1);
    const float k1 = (hi ? a[3] : a[1]) + __shfl_xor_sync(ALL, hi ? a[1] : a[3], O1);
    float m = (hi2 ? k1 : k0) + __shfl_xor_sync(ALL, hi2 ? k0 : k1, O2);
#pragma unroll
    for (int o = LN / 8; o > 0; o >>= 1) m += __shfl_xor_sync(ALL, m, o);
    col = (hi ? 2 : 0) + (hi2 ? 1 : 0);
    writes = (sub & (O2 - 1)) == 0;
    return m;
}

// A thread keeps a tile of S in registers: GLA_COLS columns (elements of v) by up to GLA_ROWS key channels, the channels in
// groups of four neighbours, group r of thread `sub` being the channels (r LN + sub) 4 .. + 3; the LN threads that share four
// columns are neighbours in a warp.  Tokens pass in runs of `run` through shared memory: v [run][cpb], k, q and a [run][NP]
// (NP: dk rounded up to whole groups, zeros beyond dk), o [run][cpb]; a thread reads them as vectors of four.
//   MODE 0, grid (sequences * H, ceil(dv / cpb)): a sequence's new tokens one after the other, from its record's state and
//           back into it.
// A long prompt is cut into chunks that run side by side (the recurrence is linear in the state):
//   MODE 1, grid (chunks * H, ...): a chunk from a state of zeros; its last state goes to `chunk_state` [chunks][H][dv][dk] and
//           the products of its decays to `chunk_decay` [chunks][H][dk].  gla_chunk_join_kernel then walks a sequence's chunks
//           and leaves in `chunk_state` the state each chunk starts from, and the last one in the record.
//   MODE 2, the same grid: a chunk from the state it starts from, o out.
template <int LN, int MODE>
__global__ void __launch_bounds__(128)
gla_scan_kernel(const float* __restrict__ qkav, int channels, int H, int P, int N, float* __restrict__ state, int64_t record,
                const int* __restrict__ slots, const int* __restrict__ cu_seqlens, float* __restrict__ y, int run, int n_seqs,
                int chunk, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    extern __shared__ float4 gla_smem4[];
    float* smem = reinterpret_cast<float*>(gla_smem4);
    pdl_trigger();
    pdl_wait();
    qkav = fresh(qkav);
    state = fresh(state);
    chunk_state = fresh(chunk_state);
    constexpr int CT = GLA_COLS, R4 = GLA_ROWS / 4;
    const int CPB = (int)blockDim.x / LN * CT;                          // columns a block takes
    const int unit = blockIdx.x / H, h = blockIdx.x - unit * H;
    int b = unit, t0, q;
    if (MODE == 0) {
        t0 = cu_seqlens[b];
        q = cu_seqlens[b + 1] - t0;
        if (q <= 0) return;
    } else if (!gla_chunk_of(unit, n_seqs, cu_seqlens, chunk, b, t0, q)) {
        return;
    }
    const int tid = threadIdx.x, sub = tid % LN, lc = tid / LN, pc0 = blockIdx.y * CPB, col0 = pc0 + lc * CT;
    const int per4 = (N + 4 * LN - 1) / (4 * LN), NP = per4 * 4 * LN, HK = H * N, inner = H * P;
    const int stage = (run * (CPB + 3 * NP) + 3) & ~3;
    float* ys = smem + 2 * stage;                                        // [run][CPB]
    float* sp = MODE == 0 ? state + (int64_t)slots[b] * record + ((int64_t)h * P + col0) * N
                          : chunk_state + (((int64_t)unit * H + h) * P + col0) * N;
    const bool whole = (N & 3) == 0 && (reinterpret_cast<size_t>(sp) & 15) == 0;
    const bool vec = ((channels | P | N) & 3) == 0 && ((reinterpret_cast<size_t>(qkav) | reinterpret_cast<size_t>(y)) & 15) == 0;
    float S[R4][4][CT];
    float dec[R4][4];
#pragma unroll
    for (int r = 0; r < R4; ++r) {
#pragma unroll
        for (int j = 0; j < 4; ++j) dec[r][j] = 1.f;
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const int n = (r * LN + sub) * 4;
            const bool in = MODE != 1 && r < per4 && col0 + c < P;
            if (in && whole && n < N) {
                const float4 v = *reinterpret_cast<const float4*>(sp + (int64_t)c * N + n);
                S[r][0][c] = v.x, S[r][1][c] = v.y, S[r][2][c] = v.z, S[r][3][c] = v.w;
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) S[r][j][c] = (in && n + j < N) ? sp[(int64_t)c * N + n + j] : 0.f;
            }
        }
    }
    // What lies beyond the head's columns and key channels stays zero in both stages: the copies never write there.
    if (NP != N || pc0 + CPB > P) {
        for (int idx = tid; idx < 2 * stage; idx += blockDim.x) smem[idx] = 0.f;
        __syncthreads();
    }
    auto copy_run = [&](int st, int i0, int len) {
        float* vs = smem + st * stage;                                   // [run][CPB]
        float* ks = vs + run * CPB;                                      // [run][NP]
        float* qs = ks + run * NP;                                       // [run][NP]
        float* as = qs + run * NP;                                       // [run][NP]
        const float* src = qkav + (int64_t)(t0 + i0) * channels;
        if (vec) {
            const int c4 = CPB / 4, n4 = NP / 4;
            for (int idx = tid; idx < len * c4; idx += blockDim.x) {
                const int i = idx / c4, c = (idx - i * c4) * 4;
                if (pc0 + c < P) gla_cp_async<16>(vs + i * CPB + c, src + (int64_t)i * channels + 3 * HK + h * P + pc0 + c);
            }
            for (int idx = tid; idx < len * n4; idx += blockDim.x) {
                const int i = idx / n4, n = (idx - i * n4) * 4;
                if (n < N) {
                    const float* rowp = src + (int64_t)i * channels + h * N + n;
                    if (MODE != 1) gla_cp_async<16>(qs + i * NP + n, rowp);
                    gla_cp_async<16>(ks + i * NP + n, rowp + HK);
                    gla_cp_async<16>(as + i * NP + n, rowp + 2 * HK);
                }
            }
        } else {
            for (int idx = tid; idx < len * CPB; idx += blockDim.x) {
                const int i = idx / CPB, c = idx - i * CPB;
                if (pc0 + c < P) gla_cp_async<4>(vs + idx, src + (int64_t)i * channels + 3 * HK + h * P + pc0 + c);
            }
            for (int idx = tid; idx < len * NP; idx += blockDim.x) {
                const int i = idx / NP, n = idx - i * NP;
                if (n < N) {
                    const float* rowp = src + (int64_t)i * channels + h * N + n;
                    if (MODE != 1) gla_cp_async<4>(qs + idx, rowp);
                    gla_cp_async<4>(ks + idx, rowp + HK);
                    gla_cp_async<4>(as + idx, rowp + 2 * HK);
                }
            }
        }
        gla_cp_commit();
    };
    copy_run(0, 0, min(run, q));
    for (int i0 = 0, st = 0; i0 < q; i0 += run, st ^= 1) {
        const int len = min(run, q - i0), next = min(run, q - i0 - run);
        if (next > 0) {
            copy_run(st ^ 1, i0 + run, next);
            gla_cp_wait<1>();
        } else {
            gla_cp_wait<0>();
        }
        __syncthreads();
        const float* vs = smem + st * stage;
        const float* ks = vs + run * CPB;
        const float* qs = ks + run * NP;
        const float* as = qs + run * NP;
        for (int i = 0; i < len; ++i) {
            const float4 xv = *reinterpret_cast<const float4*>(vs + i * CPB + lc * CT);
            const float x[CT] = {xv.x, xv.y, xv.z, xv.w};
            const float4* ki = reinterpret_cast<const float4*>(ks + i * NP) + sub;
            const float4* qi = reinterpret_cast<const float4*>(qs + i * NP) + sub;
            const float4* ai = reinterpret_cast<const float4*>(as + i * NP) + sub;
            float acc[CT] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < R4; ++r) {
                if (r < per4) {
                    const float4 kv = ki[r * LN], av = ai[r * LN];
                    const float kk[4] = {kv.x, kv.y, kv.z, kv.w}, aa[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (MODE == 1) dec[r][j] *= aa[j];
#pragma unroll
                        for (int c = 0; c < CT; ++c) S[r][j][c] = fmaf(aa[j], S[r][j][c], kk[j] * x[c]);
                    }
                    if (MODE != 1) {
                        const float4 qv = qi[r * LN];
                        const float qq[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int c = 0; c < CT; ++c) acc[c] = fmaf(S[r][j][c], qq[j], acc[c]);
                    }
                }
            }
            if (MODE != 1) {
                int c1;
                bool writes;
                const float m = gla_sum_columns<LN>(acc, sub, c1, writes);
                float* yi = ys + i * CPB + lc * CT;
                if (LN < 4) {
                    if (writes) *reinterpret_cast<float4*>(yi) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                } else if (writes) {
                    yi[c1] = m;
                }
            }
        }
        __syncthreads();                                 // (the run's results are whole; nobody reads this stage any more)
        if (MODE == 1) continue;
        float* dst = y + (int64_t)(t0 + i0) * inner + h * P + pc0;
        if (vec) {
            const int c4 = CPB / 4;
            for (int idx = tid; idx < len * c4; idx += blockDim.x) {
                const int i = idx / c4, c = (idx - i * c4) * 4;
                if (pc0 + c < P) *reinterpret_cast<float4*>(dst + (int64_t)i * inner + c) = *reinterpret_cast<const float4*>(ys + i * CPB + c);
            }
        } else {
            for (int idx = tid; idx < len * CPB; idx += blockDim.x) {
                const int i = idx / CPB, c = idx - i * CPB;
                if (pc0 + c < P) dst[(int64_t)i * inner + c] = ys[idx];
            }
        }
    }
    if (MODE == 2) return;
#pragma unroll
    for (int r = 0; r < R4; ++r)
#pragma unroll
        for (int c = 0; c < CT; ++c) {
            const int n = (r * LN + sub) * 4;
            if (r >= per4 || col0 + c >= P) continue;
            if (whole && n < N) {
                *reinterpret_cast<float4*>(sp + (int64_t)c * N + n) = make_float4(S[r][0][c], S[r][1][c], S[r][2][c], S[r][3][c]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (n + j < N) sp[(int64_t)c * N + n + j] = S[r][j][c];
            }
        }
    if (MODE == 1 && lc == 0 && blockIdx.y == 0) {
#pragma unroll
        for (int r = 0; r < R4; ++r)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = (r * LN + sub) * 4 + j;
                if (r < per4 && n < N) chunk_decay[((int64_t)unit * H + h) * N + n] = dec[r][j];
            }
    }
}

// grid (sequences, ceil(H dv dk / 256)).  Walks a sequence's chunks in order: what a chunk starts from replaces its own last
// state in `chunk_state`, and S <- (products of the chunk's decays, per key channel) S + (the chunk's last state from zeros)
// goes on to the next one; after the last chunk S is the record's new state.
__global__ void __launch_bounds__(256)
gla_chunk_join_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay, int H, int P, int N,
                      float* __restrict__ state, int64_t record, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                      int chunk) {
    pdl_trigger();
    pdl_wait();
    chunk_state = fresh(chunk_state);
    chunk_decay = fresh(chunk_decay);
    state = fresh(state);
    const int b = blockIdx.x;
    const int64_t e = (int64_t)blockIdx.y * blockDim.x + threadIdx.x, all = (int64_t)H * P * N;
    if (e >= all) return;
    const int q = cu_seqlens[b + 1] - cu_seqlens[b];
    if (q <= 0) return;
    int first = 0;
    for (int s = 0; s < b; ++s) first += (cu_seqlens[s + 1] - cu_seqlens[s] + chunk - 1) / chunk;
    const int nc = (q + chunk - 1) / chunk, h = (int)(e / ((int64_t)P * N)), n = (int)(e % N);
    float* rec = state + (int64_t)slots[b] * record + e;
    float S = *rec;
    for (int c0 = 0; c0 < nc; c0 += 8) {                                 // (eight chunks' numbers are on their way at once)
        float local[8], dec[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool in = c0 + k < nc;
            local[k] = in ? chunk_state[(int64_t)(first + c0 + k) * all + e] : 0.f;
            dec[k] = in ? chunk_decay[((int64_t)(first + c0 + k) * H + h) * N + n] : 1.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < nc) chunk_state[(int64_t)(first + c0 + k) * all + e] = S;
            S = fmaf(dec[k], S, local[k]);
        }
    }
    *rec = S;
}

// grid (tokens, groups of heads), a warp per head: o / sqrt(mean(o^2) + eps) * w * silu(g), g from the projection's sums.
template <typename T, bool ONE>
__global__ void __launch_bounds__(256)
gla_norm_gate_kernel(const float* __restrict__ y, const float* __restrict__ parts, int splits, int64_t split_stride, int cols,
                     int g_col, int H, int P, const float* __restrict__ w, float eps, T* __restrict__ out) {
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    parts = fresh(parts);
    const int t = blockIdx.x, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5, warp = blockIdx.y * n_warps + (threadIdx.x >> 5);
    for (int h = warp; h < H; h += n_warps * gridDim.y) {
        const float* row = y + ((int64_t)t * H + h) * P;
        float ss = 0.f;
        for (int j = lane; j < P; j += 32) ss = fmaf(row[j], row[j], ss);
        ss = warp_sum(ss);
        const float f = 1.0f / sqrtf(ss / (float)P + eps);
        for (int j = lane; j < P; j += 32) {
            const int64_t at = (int64_t)t * cols + g_col + h * P + j;
            const float g = ONE ? parts[at] : gla_sum_parts(parts, splits, split_stride, at);
            st(out + ((int64_t)t * H + h) * P + j, (row[j] * f) * w[j] * (g / (1.0f + expf(-g))));
        }
    }
}

struct GlaArgs {
    const float* qkav; int channels, H, P, N; float* state; int64_t record; const int *slots, *cu_seqlens; float* y;
    int run, n_seqs, chunk; float *chunk_state, *chunk_decay; int threads;
};

template <int LN, int MODE>
int gla_launch_mode(const GlaArgs& a, int units, size_t smem, cudaStream_t s) {
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        WICK_CUDA(cudaFuncSetAttribute(gla_scan_kernel<LN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        raised = true;
    }
    WICK_CUDA(launch(gla_scan_kernel<LN, MODE>, dim3(units * a.H, ceil_div(a.P, a.threads / LN * GLA_COLS)), dim3(a.threads), smem, s,
                     a.qkav, a.channels, a.H, a.P, a.N, a.state, a.record, a.slots, a.cu_seqlens, a.y, a.run, a.n_seqs, a.chunk,
                     a.chunk_state, a.chunk_decay));
    return check_launch("gla_scan");
}

template <int LN>
int gla_launch(const GlaArgs& a, int chunks, size_t smem, cudaStream_t s) {
    if (chunks == 0) return gla_launch_mode<LN, 0>(a, a.n_seqs, smem, s);
    if (gla_launch_mode<LN, 1>(a, chunks, smem, s)) return 1;
    const int64_t all = (int64_t)a.H * a.P * a.N;
    WICK_CUDA(launch(gla_chunk_join_kernel, dim3(a.n_seqs, (unsigned)ceil_div(all, (int64_t)256)), dim3(256), 0, s, a.chunk_state,
                     (const float*)a.chunk_decay, a.H, a.P, a.N, a.state, a.record, a.slots, a.cu_seqlens, a.chunk));
    if (check_launch("gla_chunk_join")) return 1;
    return gla_launch_mode<LN, 2>(a, chunks, smem, s);
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

// parts: float32 [splits, n, cols] laid out [q | k | v | g | low]; w2: float32 [H dk, rank]; b2: float32 [H dk] or null;
// state: float32 [slots, H dv dk]; qkav: float32 [n, 3 H dk + H dv] and y: float32 [n, H dv], both written here.
// max_q: the most tokens a sequence can bring (0: unknown).  chunks > 0: the sequences' tokens are scanned in chunks of
// `chunk` tokens side by side; `chunks` is at least the number of chunks (n / chunk + n_seqs is enough), chunk_state float32
// [chunks, H dv dk] and chunk_decay float32 [chunks, H dk] are scratch.
WICK_API int wick_gla_mix(const float* parts, int splits, int n, int cols, int H, int dk, int dv, int rank, const float* w2,
                          const float* b2, float q_scale, float tau, float* state, int64_t record, const int* slots, int n_seqs,
                          const int* cu_seqlens, float* qkav, float* y, int max_q, int chunk, int chunks, float* chunk_state,
                          float* chunk_decay, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    WICK_REQUIRE(H > 0 && dk > 0 && dv > 0 && rank > 0 && tau > 0.f, "gla_mix: bad sizes");
    WICK_REQUIRE(dk <= 32 * GLA_ROWS, "gla_mix: heads of %d key channels (up to %d are built)", dk, 32 * GLA_ROWS);
    const int HK = H * dk, HV = H * dv, channels = 3 * HK + HV;
    WICK_REQUIRE(cols == 2 * HK + 2 * HV + rank, "gla_mix: rows of %d numbers, %d expected", cols, 2 * HK + 2 * HV + rank);
    WICK_REQUIRE(record == (int64_t)HV * dk, "gla_mix: records of another size");
    WICK_REQUIRE(splits >= 1, "gla_mix: partial sums are needed");
    WICK_REQUIRE(chunks == 0 || (chunk > 0 && chunk_state && chunk_decay && (int64_t)chunks >= n / chunk + n_seqs),
                 "gla_mix: the chunked scan needs room for %d chunks", chunk > 0 ? n / chunk + n_seqs : 0);
    WICK_REQUIRE((size_t)rank * 4 <= 48 * 1024, "gla_mix: a rank of %d is beyond one block's shared memory", rank);
    if (n == 0 || n_seqs == 0) return 0;
    const int64_t stride = (int64_t)n * cols;
    // (long steps: eight tokens a block share a thread's row of W2; short ones: a block a token, for more blocks)
    const int prep_tiles = ceil_div(HK, GLA_PREP_THREADS) + ceil_div(HV, GLA_PREP_THREADS);
    const int pb = (n >= 512 && (size_t)rank * 8 * 4 <= 16 * 1024) ? 8 : 1;
    size_t prep_smem = (size_t)pb * rank * 4;
    const size_t staged = (size_t)GLA_PREP_THREADS * (rank | 1) * 4;
    const int stage = prep_smem + staged <= 48 * 1024 ? 1 : 0;          // (else a thread reads its row of W2 from memory)
    if (stage) prep_smem += staged;
    auto prepare = pb == 8 ? (splits == 1 ? gla_prepare_kernel<8, true> : gla_prepare_kernel<8, false>)
                           : (splits == 1 ? gla_prepare_kernel<1, true> : gla_prepare_kernel<1, false>);
    WICK_CUDA(launch(prepare, dim3(ceil_div(n, pb), prep_tiles), dim3(GLA_PREP_THREADS), prep_smem, s, parts, splits, stride, cols, HK, HV,
                     rank, w2, b2, q_scale, 1.0f / tau, qkav, n, stage));
    if (check_launch("gla_prepare")) return 1;
    const int N = dk, P = dv;
    int ln = 1;
    while (ln < 32 && (N + ln - 1) / ln > GLA_ROWS) ln *= 2;
    if (ln < 4 && N >= 16) ln = 4;                                       // (a thread keeps a few numbers, not a whole column)
    int threads = ceil_div(P, GLA_COLS) * ln;
    threads = threads > 128 ? 128 : (threads + 31) / 32 * 32;
    const int cpb = threads / ln * GLA_COLS, np = ceil_div(N, 4 * ln) * 4 * ln;
    const int per_token = 2 * (cpb + 3 * np) + cpb;                       // (two stages of inputs, one of results)
    int run = (52 * 1024 / 4) / per_token;                                // (four blocks of this size share an SM)
    run = run < 1 ? 1 : (run > 64 ? 64 : run);
    if (run > max_q && max_q >= 1) run = max_q;
    if (chunks > 0 && run > chunk) run = chunk;
    if (chunks > 0 && run < chunk) run = ceil_div(chunk, ceil_div(chunk, run));   // (equal runs)
    const size_t smem = (size_t)(2 * ((run * (cpb + 3 * np) + 3) & ~3) + run * cpb) * sizeof(float);
    const GlaArgs a = {qkav, channels, H, P, N, state, record, slots, cu_seqlens, y, run, n_seqs, chunk, chunk_state, chunk_decay,
                       threads};
    switch (ln) {
        case 1: return gla_launch<1>(a, chunks, smem, s);
        case 2: return gla_launch<2>(a, chunks, smem, s);
        case 4: return gla_launch<4>(a, chunks, smem, s);
        case 8: return gla_launch<8>(a, chunks, smem, s);
        case 16: return gla_launch<16>(a, chunks, smem, s);
        default: return gla_launch<32>(a, chunks, smem, s);
    }
}

// y: float32 [n, H dv]; parts as above (g from column g_col on); w: float32 [dv]; out: [n, H dv].
#define WICK_GLA_NORM_GATE(NAME, T)                                                                                            \
    WICK_API int NAME(const float* y, const float* parts, int splits, int n, int cols, int g_col, int H, int dv, const float* w, \
                      float eps, void* out, void* s) {                                                                         \
        WICK_REQUIRE(H > 0 && dv > 0 && g_col >= 0 && g_col + H * dv <= cols, "gla_norm_gate: bad sizes");                     \
        if (n == 0) return 0;                                                                                                  \
        const int warps = H >= 4 ? 4 : H;                                                                                      \
        auto kernel = splits == 1 ? gla_norm_gate_kernel<T, true> : gla_norm_gate_kernel<T, false>;                            \
        WICK_CUDA(launch(kernel, dim3(n, ceil_div(H, warps)), dim3(32 * warps), 0, (cudaStream_t)s, y, parts, splits,          \
                         (int64_t)n * cols, cols, g_col, H, dv, w, eps, (T*)out));                                              \
        return check_launch("gla_norm_gate");                                                                                  \
    }
WICK_GLA_NORM_GATE(wick_gla_norm_gate_bf16, bf16)
WICK_GLA_NORM_GATE(wick_gla_norm_gate_f32, float)
