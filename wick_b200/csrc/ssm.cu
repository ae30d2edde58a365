// A selective state-space recurrence per head (the "state-space duality" form: one decay number per head and
// token), with its short causal convolution, for steps of any shape over per-sequence state records.
//
// The input projection's float32 partial sums hold, per token, [z: inner | x: inner | B: G N | C: G N | dt: H],
// inner = H P (H heads of P numbers), N the state size, G groups of heads that share B and C.
//
//   conv       : u = [x | B | C] (channels = inner + 2 G N);  c_t = silu(b + sum_k w[., k] u_(t - (K - 1) + k)), zeros
//                before position 0; inputs of earlier steps come from the sequence's record
//   conv state : the record's last K - 1 inputs are brought up to date
//   scan       : dt_t = softplus(dt_t + dt_bias_h);  a_t = exp(-exp(A_log_h) dt_t);
//                S_t = a_t S_(t-1) + dt_t B_t x_t^T  (N x P per head);  y_t = S_t^T C_t + D_h x_t
//   gate, norm : g = y * silu(z);  `parts` equal runs of g are each divided by their own root mean square and
//                multiplied by a weight; the result goes out in the activation type
//
// A sequence's record (float32): [K - 1][channels] inputs of the convolution, oldest first, then the state as
// [H][P][N] (a column of S, the N numbers that meet one element of x, lies together).  Everything here is float32
// arithmetic; a token's numbers depend on its own sequence alone.  A step of few tokens adds them in the same order whatever
// its shape; a long prompt step scanned in chunks (below) rounds the state differently, and no more than that.
#include "common.cuh"

namespace wick {

constexpr int SSM_MAX_TAPS = 16;
constexpr int SSM_ROWS = 16;                    // state numbers a thread keeps of one column, at most
constexpr int SSM_COLS = 4;                     // columns of the state a thread keeps

// Which tokens a block of the chunked scan takes.  A sequence's new tokens are cut into runs of `chunk` (the last one may
// be shorter); the runs of all sequences are numbered in a row.  False beyond the last run.
__device__ __forceinline__ bool chunk_of(int slot, int n_seqs, const int* __restrict__ cu_seqlens, int chunk, int& b, int& first,
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

// Asynchronous copies of BYTES (4 or 16) from global into shared memory, in groups a thread waits for.
template <int BYTES>
__device__ __forceinline__ void cp_async(float* dst, const float* src) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(d), "l"(src), "n"(BYTES) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int LEFT>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(LEFT) : "memory"); }

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

__device__ __forceinline__ float sum_parts(const float* __restrict__ parts, int splits, int64_t split_stride, int64_t at) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += parts[s * split_stride + at];
    return v;
}

constexpr int SSM_CONV_TOKENS = 4;              // tokens a thread of the convolution takes (their loads are in flight together)

// grid (ceil(tokens / SSM_CONV_TOKENS), ceil(channels / 256)).  ONE: the projection came as a single set of sums (its loads
// need no loop and go out together).
template <bool ONE>
__global__ void __launch_bounds__(256)
ssm_conv_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, int cols, int first_col, int channels, int taps,
                const float* __restrict__ w, const float* __restrict__ bias, const float* __restrict__ state, int64_t record,
                const int* __restrict__ slots, const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                const int* __restrict__ start, float* __restrict__ out, int n) {
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    state = fresh(state);
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const float b0 = bias ? bias[c] : 0.f;
    float acc[SSM_CONV_TOKENS];
    int pos[SSM_CONV_TOKENS], first[SSM_CONV_TOKENS];
    const float* rec[SSM_CONV_TOKENS];
#pragma unroll
    for (int j = 0; j < SSM_CONV_TOKENS; ++j) {
        const int t = min(blockIdx.x * SSM_CONV_TOKENS + j, n - 1), b = seq_of_token[t];
        pos[j] = positions[t];
        first[j] = start[b];
        rec[j] = state + (int64_t)slots[b] * record;
        acc[j] = b0;
    }
#pragma unroll 4
    for (int k = 0; k < taps; ++k) {
        const float wk = w[(int64_t)c * taps + k];
        float u[SSM_CONV_TOKENS];
#pragma unroll
        for (int j = 0; j < SSM_CONV_TOKENS; ++j) {
            const int t = min(blockIdx.x * SSM_CONV_TOKENS + j, n - 1), sp = pos[j] - (taps - 1) + k;
            u[j] = 0.f;
            const int64_t at = (int64_t)(t - (pos[j] - sp)) * cols + first_col + c;
            if (sp >= first[j]) u[j] = ONE ? parts[at] : sum_parts(parts, splits, split_stride, at);
            else if (sp >= 0) u[j] = rec[j][(int64_t)(sp - (first[j] - (taps - 1))) * channels + c];
        }
#pragma unroll
        for (int j = 0; j < SSM_CONV_TOKENS; ++j) acc[j] = fmaf(wk, u[j], acc[j]);
    }
#pragma unroll
    for (int j = 0; j < SSM_CONV_TOKENS; ++j) {
        const int t = blockIdx.x * SSM_CONV_TOKENS + j;
        if (t < n) out[(int64_t)t * channels + c] = silu_f(acc[j]);
    }
}

// grid (sequences, ceil(channels / 256)).  Runs after the convolution has read the old inputs.
__global__ void __launch_bounds__(256)
ssm_conv_state_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, int cols, int first_col, int channels,
                      int taps, float* __restrict__ state, int64_t record, const int* __restrict__ slots,
                      const int* __restrict__ cu_seqlens) {
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    state = fresh(state);
    const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int t0 = cu_seqlens[b], q = cu_seqlens[b + 1] - t0;
    if (q <= 0) return;
    float* rec = state + (int64_t)slots[b] * record;
    float keep[SSM_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < SSM_MAX_TAPS; ++j) {
        if (j >= taps - 1) break;
        const int from = j + q;                                          // where the input of new place j lies now
        keep[j] = from >= taps - 1 ? sum_parts(parts, splits, split_stride, (int64_t)(t0 + from - (taps - 1)) * cols + first_col + c)
                                   : rec[(int64_t)from * channels + c];
    }
#pragma unroll
    for (int j = 0; j < SSM_MAX_TAPS; ++j) {
        if (j >= taps - 1) break;
        rec[(int64_t)j * channels + c] = keep[j];
    }
}

// The sums of four columns over the LN threads that share them.  Two exchanges halve what a thread carries (it keeps two
// columns, then one), the rest is a butterfly over one number; `col` is the column a thread ends with and `writes` whether
// it is the one of its group that holds it (LN < 4: every column stays, a[0..3] hold the sums).
template <int LN>
__device__ __forceinline__ float sum_columns(float (&a)[4], int sub, int& col, bool& writes) {
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

// A thread keeps a tile of S in registers: SSM_COLS columns (elements of x) by up to SSM_ROWS state rows, the rows in groups
// of four neighbours, group r of thread `sub` being the rows (r LN + sub) 4 .. + 3; the LN threads that share four columns
// are neighbours in a warp.  Tokens pass in runs of `run` through shared memory: x [run][cpb], B and C [run][NP] (NP: N
// rounded up to whole groups, zeros beyond N, so that the loop tests nothing), y [run][cpb], dt and decay [run]; a thread
// reads them as vectors of four.
//   MODE 0, grid (sequences * H, ceil(P / cpb)): a sequence's new tokens one after the other, from its record's state and
//           back into it.
// A long prompt is cut into chunks that run side by side (the recurrence is linear in the state):
//   MODE 1, grid (chunks * H, ...): a chunk from a state of zeros; its last state goes to `chunk_state` [chunks][H][P][N] and
//           the product of its decays to `chunk_decay` [chunks][H].  ssm_chunk_join_kernel then walks a sequence's chunks and
//           leaves in `chunk_state` the state each chunk starts from, and the last one in the record.
//   MODE 2, the same grid: a chunk from the state it starts from, y out.
template <int LN, int MODE>
__global__ void __launch_bounds__(128)
ssm_scan_kernel(const float* __restrict__ xbc, int channels, const float* __restrict__ parts, int splits, int64_t split_stride,
                int cols, int dt_col, int H, int P, int N, int G, const float* __restrict__ dt_bias,
                const float* __restrict__ a_log, const float* __restrict__ d_skip, float* __restrict__ state, int64_t record,
                int64_t state_off, const int* __restrict__ slots, const int* __restrict__ cu_seqlens, float* __restrict__ y,
                int run, int n_seqs, int chunk, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    extern __shared__ float4 smem4[];
    float* smem = reinterpret_cast<float*>(smem4);
    pdl_trigger();
    pdl_wait();
    xbc = fresh(xbc);
    parts = fresh(parts);
    state = fresh(state);
    chunk_state = fresh(chunk_state);
    constexpr int CT = SSM_COLS, R4 = SSM_ROWS / 4;
    const int CPB = (int)blockDim.x / LN * CT;                          // columns a block takes
    const int unit = blockIdx.x / H, h = blockIdx.x - unit * H, g = h / (H / G);
    int b = unit, t0, q;
    if (MODE == 0) {
        t0 = cu_seqlens[b];
        q = cu_seqlens[b + 1] - t0;
        if (q <= 0) return;
    } else if (!chunk_of(unit, n_seqs, cu_seqlens, chunk, b, t0, q)) {
        return;
    }
    const int tid = threadIdx.x, sub = tid % LN, lc = tid / LN, pc0 = blockIdx.y * CPB, col0 = pc0 + lc * CT;
    const int per4 = (N + 4 * LN - 1) / (4 * LN), NP = per4 * 4 * LN, inner = H * P;
    // Two stages of a run's inputs (the next run is copied while this one is computed), then the run's results.
    const int stage = (run * (CPB + 2 * NP + 2) + 3) & ~3;
    float* ys = smem + 2 * stage;                                        // [run][CPB]
    float* sp = MODE == 0 ? state + (int64_t)slots[b] * record + state_off + ((int64_t)h * P + col0) * N
                          : chunk_state + (((int64_t)unit * H + h) * P + col0) * N;
    const bool whole = (N & 3) == 0 && (reinterpret_cast<size_t>(sp) & 15) == 0;     // (a group of rows is one aligned vector)
    // (rows of x, B, C and y start on 16-byte borders: they are copied as vectors of four)
    const bool vec = ((channels | P | N) & 3) == 0 && ((reinterpret_cast<size_t>(xbc) | reinterpret_cast<size_t>(y)) & 15) == 0;
    float S[R4][4][CT];
#pragma unroll
    for (int r = 0; r < R4; ++r)
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
    const float bias = dt_bias[h], rate = -expf(a_log[h]), skip = d_skip ? d_skip[h] : 0.f;
    // What lies beyond the head's columns and the state's rows stays zero in both stages: the copies never write there.
    if (NP != N || pc0 + CPB > P) {
        for (int idx = tid; idx < 2 * stage; idx += blockDim.x) smem[idx] = 0.f;
        __syncthreads();
    }
    // Copies the inputs of the run that starts at token i0 into stage `st` (asynchronously, one group).
    auto copy_run = [&](int st, int i0, int len) {
        float* xs = smem + st * stage;                                   // [run][CPB]
        float* bs = xs + run * CPB;                                      // [run][NP]
        float* cs = bs + run * NP;                                       // [run][NP]
        const float* src = xbc + (int64_t)(t0 + i0) * channels;
        if (vec) {
            const int c4 = CPB / 4, n4 = NP / 4;
            for (int idx = tid; idx < len * c4; idx += blockDim.x) {
                const int i = idx / c4, c = (idx - i * c4) * 4;
                if (pc0 + c < P) cp_async<16>(xs + i * CPB + c, src + (int64_t)i * channels + h * P + pc0 + c);
            }
            for (int idx = tid; idx < len * n4; idx += blockDim.x) {
                const int i = idx / n4, n = (idx - i * n4) * 4;
                if (n < N) {
                    const float* rowp = src + (int64_t)i * channels + inner + g * N + n;
                    cp_async<16>(bs + i * NP + n, rowp);
                    if (MODE != 1) cp_async<16>(cs + i * NP + n, rowp + G * N);
                }
            }
        } else {
            for (int idx = tid; idx < len * CPB; idx += blockDim.x) {
                const int i = idx / CPB, c = idx - i * CPB;
                if (pc0 + c < P) cp_async<4>(xs + idx, src + (int64_t)i * channels + h * P + pc0 + c);
            }
            for (int idx = tid; idx < len * NP; idx += blockDim.x) {
                const int i = idx / NP, n = idx - i * NP;
                if (n < N) {
                    const float* rowp = src + (int64_t)i * channels + inner + g * N + n;
                    cp_async<4>(bs + idx, rowp);
                    if (MODE != 1) cp_async<4>(cs + idx, rowp + G * N);
                }
            }
        }
        cp_async_commit();
    };
    // A run's step sizes: read early (raw), turned into dt and the decay and stored late; two a thread at most (run <= 64).
    auto raw_steps = [&](int i0, int len, float (&raw)[2]) {
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = tid + k * blockDim.x;
            raw[k] = i < len ? sum_parts(parts, splits, split_stride, (int64_t)(t0 + i0 + i) * cols + dt_col + h) : 0.f;
        }
    };
    auto store_steps = [&](int st, int len, const float (&raw)[2]) {
        float* dts = smem + st * stage + run * (CPB + 2 * NP);
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const int i = tid + k * blockDim.x;
            if (i < len) {
                const float dt = softplus_f(raw[k] + bias);
                dts[i] = dt;
                dts[run + i] = expf(rate * dt);
            }
        }
    };
    float decay = 1.f;
    float raw[2];
    copy_run(0, 0, min(run, q));
    raw_steps(0, min(run, q), raw);
    store_steps(0, min(run, q), raw);
    for (int i0 = 0, st = 0; i0 < q; i0 += run, st ^= 1) {
        const int len = min(run, q - i0), next = min(run, q - i0 - run);
        if (next > 0) {
            copy_run(st ^ 1, i0 + run, next);
            raw_steps(i0 + run, next, raw);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float* xs = smem + st * stage;
        const float* bs = xs + run * CPB;
        const float* cs = bs + run * NP;
        const float* dts = cs + run * NP;
        const float* das = dts + run;
        for (int i = 0; i < len; ++i) {
            const float4 xv = *reinterpret_cast<const float4*>(xs + i * CPB + lc * CT);
            const float dt = dts[i], da = das[i];
            const float x[CT] = {xv.x, xv.y, xv.z, xv.w};
            const float4* bi = reinterpret_cast<const float4*>(bs + i * NP) + sub;
            const float4* ci = reinterpret_cast<const float4*>(cs + i * NP) + sub;
            float acc[CT] = {0.f, 0.f, 0.f, 0.f};
            if (MODE == 1) decay *= da;
#pragma unroll
            for (int r = 0; r < R4; ++r) {
                if (r < per4) {
                    const float4 bv = bi[r * LN];
                    const float bd[4] = {dt * bv.x, dt * bv.y, dt * bv.z, dt * bv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
#pragma unroll
                        for (int c = 0; c < CT; ++c) S[r][j][c] = fmaf(da, S[r][j][c], bd[j] * x[c]);
                    if (MODE != 1) {
                        const float4 cv = ci[r * LN];
                        const float cc[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                        for (int j = 0; j < 4; ++j)
#pragma unroll
                            for (int c = 0; c < CT; ++c) acc[c] = fmaf(S[r][j][c], cc[j], acc[c]);
                    }
                }
            }
            if (MODE != 1) {
                int c1;
                bool writes;
                const float m = sum_columns<LN>(acc, sub, c1, writes);
                float* yi = ys + i * CPB + lc * CT;
                if (LN < 4) {
                    if (writes) *reinterpret_cast<float4*>(yi) = make_float4(fmaf(skip, x[0], acc[0]), fmaf(skip, x[1], acc[1]),
                                                                             fmaf(skip, x[2], acc[2]), fmaf(skip, x[3], acc[3]));
                } else if (writes) {
                    yi[c1] = fmaf(skip, c1 == 0 ? x[0] : c1 == 1 ? x[1] : c1 == 2 ? x[2] : x[3], m);
                }
            }
        }
        if (next > 0) store_steps(st ^ 1, next, raw);
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
    if (MODE == 1 && tid == 0 && blockIdx.y == 0) chunk_decay[(int64_t)unit * H + h] = decay;
}

// grid (sequences, ceil(H P N / 256)).  Walks a sequence's chunks in order: what a chunk starts from replaces its own last
// state in `chunk_state`, and S <- (product of the chunk's decays) S + (the chunk's last state from zeros) goes on to the
// next one; after the last chunk S is the record's new state.
__global__ void __launch_bounds__(256)
ssm_chunk_join_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay, int H, int PN, float* __restrict__ state,
                      int64_t record, int64_t state_off, const int* __restrict__ slots, const int* __restrict__ cu_seqlens,
                      int chunk) {
    pdl_trigger();
    pdl_wait();
    chunk_state = fresh(chunk_state);
    chunk_decay = fresh(chunk_decay);
    state = fresh(state);
    const int b = blockIdx.x;
    const int64_t e = (int64_t)blockIdx.y * blockDim.x + threadIdx.x, all = (int64_t)H * PN;
    if (e >= all) return;
    const int q = cu_seqlens[b + 1] - cu_seqlens[b];
    if (q <= 0) return;
    int first = 0;
    for (int s = 0; s < b; ++s) first += (cu_seqlens[s + 1] - cu_seqlens[s] + chunk - 1) / chunk;
    const int nc = (q + chunk - 1) / chunk, h = (int)(e / PN);
    float* rec = state + (int64_t)slots[b] * record + state_off + e;
    float S = *rec;
    for (int c0 = 0; c0 < nc; c0 += 8) {                                 // (eight chunks' numbers are on their way at once)
        float local[8], dec[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const bool in = c0 + k < nc;
            local[k] = in ? chunk_state[(int64_t)(first + c0 + k) * all + e] : 0.f;
            dec[k] = in ? chunk_decay[(int64_t)(first + c0 + k) * H + h] : 1.f;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (c0 + k < nc) chunk_state[(int64_t)(first + c0 + k) * all + e] = S;
            S = fmaf(dec[k], S, local[k]);
        }
    }
    *rec = S;
}

// One block per token: g = y * silu(z) into shared memory; a warp takes whole runs (its lanes a run's elements in
// steps of 32, the 32 sums by the butterfly); then out = g * factor of its run * w.
template <typename T>
__global__ void __launch_bounds__(256)
ssm_gate_norm_kernel(const float* __restrict__ y, const float* __restrict__ parts, int splits, int64_t split_stride, int cols,
                     int z_col, int inner, int n_runs, const float* __restrict__ w, float eps, T* __restrict__ out) {
    extern __shared__ float smem[];
    float* row = smem;                                                   // [inner]
    float* factor = smem + ((inner + 3) & ~3);                           // [n_runs]
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    parts = fresh(parts);
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    for (int j = tid; j < inner; j += blockDim.x)
        row[j] = y[(int64_t)t * inner + j] * silu_f(sum_parts(parts, splits, split_stride, (int64_t)t * cols + z_col + j));
    __syncthreads();
    const int len = inner / n_runs;
    for (int r = warp; r < n_runs; r += n_warps) {
        float ss = 0.f;
        for (int j = lane; j < len; j += 32) ss = fmaf(row[r * len + j], row[r * len + j], ss);
        ss = warp_sum(ss);
        if (lane == 0) factor[r] = 1.0f / sqrtf(ss / (float)len + eps);
    }
    __syncthreads();
    for (int j = tid; j < inner; j += blockDim.x) st(out + (int64_t)t * inner + j, (row[j] * factor[j / len]) * w[j]);
}

struct ScanArgs {
    const float* xbc; int channels; const float* parts; int splits; int64_t split_stride; int cols, dt_col, H, P, N, G;
    const float *dt_bias, *a_log, *d_skip; float* state; int64_t record, state_off; const int *slots, *cu_seqlens; float* y;
    int run, n_seqs, chunk; float *chunk_state, *chunk_decay; int threads;
};

template <int LN, int MODE>
int scan_launch_mode(const ScanArgs& a, int units, size_t smem, cudaStream_t s) {
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        WICK_CUDA(cudaFuncSetAttribute(ssm_scan_kernel<LN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        raised = true;
    }
    WICK_CUDA(launch(ssm_scan_kernel<LN, MODE>, dim3(units * a.H, ceil_div(a.P, a.threads / LN * SSM_COLS)), dim3(a.threads), smem, s, a.xbc, a.channels,
                     a.parts, a.splits, a.split_stride, a.cols, a.dt_col, a.H, a.P, a.N, a.G, a.dt_bias, a.a_log, a.d_skip, a.state,
                     a.record, a.state_off, a.slots, a.cu_seqlens, a.y, a.run, a.n_seqs, a.chunk, a.chunk_state, a.chunk_decay));
    return check_launch("ssm_scan");
}

// chunks == 0: every sequence's tokens one after the other; else the three steps of the chunked scan over `chunks` units.
template <int LN>
int scan_launch(const ScanArgs& a, int chunks, size_t smem, cudaStream_t s) {
    if (chunks == 0) return scan_launch_mode<LN, 0>(a, a.n_seqs, smem, s);
    if (scan_launch_mode<LN, 1>(a, chunks, smem, s)) return 1;
    const int64_t all = (int64_t)a.H * a.P * a.N;
    WICK_CUDA(launch(ssm_chunk_join_kernel, dim3(a.n_seqs, (unsigned)ceil_div(all, (int64_t)256)), dim3(256), 0, s, a.chunk_state,
                     (const float*)a.chunk_decay, a.H, a.P * a.N, a.state, a.record, a.state_off, a.slots, a.cu_seqlens, a.chunk));
    if (check_launch("ssm_chunk_join")) return 1;
    return scan_launch_mode<LN, 2>(a, chunks, smem, s);
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

// parts: float32 [splits, n, cols] laid out [z | x | B | C | dt]; state: float32 [slots, record]; xbc: float32
// [n, channels] and y: float32 [n, H P], both written here.  max_q: the most tokens a sequence can bring (0: unknown).
// chunks > 0: the sequences' tokens are scanned in chunks of `chunk` tokens side by side; `chunks` is at least the number of
// chunks (n / chunk + n_seqs is enough), chunk_state float32 [chunks, H P N] and chunk_decay float32 [chunks, H] are scratch.
WICK_API int wick_ssm_mix(const float* parts, int splits, int n, int cols, int H, int P, int N, int G, int taps, const float* conv_w,
                          const float* conv_b, const float* dt_bias, const float* a_log, const float* d_skip, float* state,
                          int64_t record, const int* slots, int n_seqs, const int* cu_seqlens, const int* start,
                          const int* seq_of_token, const int* positions, float* xbc, float* y, int max_q, int chunk, int chunks,
                          float* chunk_state, float* chunk_decay, void* stream) {
    cudaStream_t s = (cudaStream_t)stream;
    WICK_REQUIRE(H > 0 && P > 0 && N > 0 && G > 0 && H % G == 0, "ssm_mix: bad sizes");
    WICK_REQUIRE(taps >= 1 && taps <= SSM_MAX_TAPS, "ssm_mix: %d taps (1 .. %d are built)", taps, SSM_MAX_TAPS);
    WICK_REQUIRE(N <= SSM_ROWS * 32, "ssm_mix: a state of %d rows (up to %d are built)", N, SSM_ROWS * 32);
    WICK_REQUIRE(N <= 32 * SSM_ROWS, "ssm_mix: a state of %d numbers (up to %d are built)", N, 32 * SSM_ROWS);
    const int inner = H * P, channels = inner + 2 * G * N;
    WICK_REQUIRE(cols == 2 * inner + 2 * G * N + H, "ssm_mix: rows of %d numbers, %d expected", cols, 2 * inner + 2 * G * N + H);
    WICK_REQUIRE(record == (int64_t)(taps - 1) * channels + (int64_t)H * P * N, "ssm_mix: records of another size");
    WICK_REQUIRE(splits >= 1, "ssm_mix: partial sums are needed");
    WICK_REQUIRE(chunks == 0 || (chunk > 0 && chunk_state && chunk_decay && (int64_t)chunks >= n / chunk + n_seqs),
                 "ssm_mix: the chunked scan needs room for %d chunks", chunk > 0 ? n / chunk + n_seqs : 0);
    if (n == 0 || n_seqs == 0) return 0;
    const int64_t stride = (int64_t)n * cols;
    const dim3 conv_grid(ceil_div(n, SSM_CONV_TOKENS), ceil_div(channels, 256));
    if (splits == 1) {
        WICK_CUDA(launch(ssm_conv_kernel<true>, conv_grid, dim3(256), 0, s, parts, splits, stride, cols, inner, channels, taps, conv_w,
                         conv_b, (const float*)state, record, slots, seq_of_token, positions, start, xbc, n));
    } else {
        WICK_CUDA(launch(ssm_conv_kernel<false>, conv_grid, dim3(256), 0, s, parts, splits, stride, cols, inner, channels, taps, conv_w,
                         conv_b, (const float*)state, record, slots, seq_of_token, positions, start, xbc, n));
    }
    if (check_launch("ssm_conv")) return 1;
    if (taps > 1) {
        WICK_CUDA(launch(ssm_conv_state_kernel, dim3(n_seqs, ceil_div(channels, 256)), dim3(256), 0, s, parts, splits, stride, cols,
                         inner, channels, taps, state, record, slots, cu_seqlens));
        if (check_launch("ssm_conv_state")) return 1;
    }
    int ln = 1;
    while (ln < 32 && (N + ln - 1) / ln > SSM_ROWS) ln *= 2;
    if (ln < 4 && N >= 16) ln = 4;                                       // (a thread keeps a few numbers, not a whole column)
    // A block: as many threads as the head's columns need (whole warps, 128 at most), each group of `ln` taking SSM_COLS columns.
    int threads = ceil_div(P, SSM_COLS) * ln;
    threads = threads > 128 ? 128 : (threads + 31) / 32 * 32;
    const int cpb = threads / ln * SSM_COLS, np = ceil_div(N, 4 * ln) * 4 * ln;
    const int per_token = 2 * (cpb + 2 * np + 2) + cpb;                   // (two stages of inputs, one of results)
    int run = (52 * 1024 / 4) / per_token;                                // (four blocks of this size share an SM)
    run = run < 1 ? 1 : (run > 64 ? 64 : run);
    if (run > max_q && max_q >= 1) run = max_q;
    if (chunks > 0 && run > chunk) run = chunk;
    if (chunks > 0 && run < chunk) run = ceil_div(chunk, ceil_div(chunk, run));   // (equal runs)
    const size_t smem = (size_t)(2 * ((run * (cpb + 2 * np + 2) + 3) & ~3) + run * cpb) * sizeof(float);
    const ScanArgs a = {xbc, channels, parts, splits, stride, cols, 2 * inner + 2 * G * N, H, P, N, G, dt_bias, a_log, d_skip, state,
                        record, (int64_t)(taps - 1) * channels, slots, cu_seqlens, y, run, n_seqs, chunk, chunk_state, chunk_decay,
                        threads};
    switch (ln) {
        case 1: return scan_launch<1>(a, chunks, smem, s);
        case 2: return scan_launch<2>(a, chunks, smem, s);
        case 4: return scan_launch<4>(a, chunks, smem, s);
        case 8: return scan_launch<8>(a, chunks, smem, s);
        case 16: return scan_launch<16>(a, chunks, smem, s);
        default: return scan_launch<32>(a, chunks, smem, s);
    }
}

// y: float32 [n, inner]; parts as above (z in its first columns); w: float32 [inner]; out: [n, inner].
#define WICK_SSM_GATE_NORM(NAME, T)                                                                                            \
    WICK_API int NAME(const float* y, const float* parts, int splits, int n, int cols, int inner, int n_runs, const float* w,    \
                      float eps, void* out, void* s) {                                                                         \
        WICK_REQUIRE(n_runs > 0 && inner % n_runs == 0 && inner <= cols, "ssm_gate_norm: bad sizes");                          \
        if (n == 0) return 0;                                                                                                  \
        const size_t smem = (size_t)(((inner + 3) & ~3) + n_runs) * sizeof(float);                                             \
        WICK_REQUIRE(smem <= 48 * 1024, "ssm_gate_norm: a row of %d numbers is beyond one block's shared memory", inner);      \
        WICK_CUDA(launch(ssm_gate_norm_kernel<T>, dim3(n), dim3(256), smem, (cudaStream_t)s, y, parts, splits,                 \
                         (int64_t)n * cols, cols, 0, inner, n_runs, w, eps, (T*)out));                                          \
        return check_launch("ssm_gate_norm");                                                                                  \
    }
WICK_SSM_GATE_NORM(wick_ssm_gate_norm_bf16, bf16)
WICK_SSM_GATE_NORM(wick_ssm_gate_norm_f32, float)
