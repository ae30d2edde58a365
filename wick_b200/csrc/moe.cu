// A mixture of gated experts whose choice is read from a table: token id -> `top` experts,
// each with the same weight.  Expert i: down_i( silu(gate_i x) * (up_i x) ).
//
//   moe_up   : hidden[t][c] = silu(gate x_t) * (up x_t) with the weights of expert table[token_t][c]
//   moe_down : out[t] = base[t] + weight * (down_{e(t,0)} hidden[t][0] + down_{e(t,1)} hidden[t][1] + ...)
//              (choices in table order; base: float32 partial sums of a part that runs for every token)
//
// These kernels are the form of decode steps and of the 32-bit path.  Up to 12,000 (token, choice)
// pairs a step they run by expert (a matrix row is read once for all the pairs that use it); beyond
// that every pair reads its expert's matrices itself (from the L2 cache when pairs share one).  Products accumulate in float32 along the inner dimension in a fixed order (lane l takes
// elements l, l + 32, ... or the 8 neighbours at 8 l, 8 l + 256, ...; the 32 sums by the butterfly).
#include "common.cuh"

namespace wick {

template <typename T> __device__ __forceinline__ float dot_row(const T* __restrict__ w, const float* __restrict__ x, int k, int lane) {
    float s = 0.f;
    constexpr int VN = Vec16<T>::N;
    if (k % VN == 0 && (((uintptr_t)w) & 15) == 0) {
        for (int j = lane * VN; j < k; j += 32 * VN) {
            Vec16<T> v;
            v.load(w + j);
#pragma unroll
            for (int i = 0; i < VN; ++i) s = fmaf(v.v[i], x[j + i], s);
        }
    } else {
        for (int j = lane; j < k; j += 32) s = fmaf(ld(w + j), x[j], s);
    }
    return warp_sum(s);
}

constexpr int ROWS_PER_WARP = 4;

// grid (n * top, ceil(ff / (warps * ROWS_PER_WARP))).  gate_up: [experts][2][ff][width] (gate rows, then up rows); not `gated`:
// [experts][ff][width] and hidden = max(up x, 0)^2.
template <typename T>
__global__ void __launch_bounds__(128)
moe_up_kernel(const T* __restrict__ x, const int* __restrict__ tokens, const int* __restrict__ table, int top, int n_experts,
              const T* __restrict__ gate_up, T* __restrict__ hidden, int width, int ff, int gated) {
    extern __shared__ float xs[];
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    const int t = blockIdx.x / top, c = blockIdx.x - t * top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < width; j += blockDim.x) xs[j] = ld(x + (int64_t)t * width + j);
    __syncthreads();
    const int ex = table[(int64_t)tokens[t] * top + c];
    if (ex < 0 || ex >= n_experts) return;                                   // (a table that names no expert adds nothing)
    const T* wg = gate_up + (int64_t)ex * (gated ? 2 : 1) * ff * width;
    const T* wu = wg + (int64_t)ff * width;
    const int f0 = (blockIdx.y * (blockDim.x >> 5) + warp) * ROWS_PER_WARP;
    for (int f = f0; f < min(f0 + ROWS_PER_WARP, ff); ++f) {
        const float g = dot_row(wg + (int64_t)f * width, xs, width, lane);
        if (gated) {
            const float u = dot_row(wu + (int64_t)f * width, xs, width, lane);
            if (lane == 0) st(hidden + ((int64_t)t * top + c) * ff + f, g / (1.0f + expf(-g)) * u);
        } else if (lane == 0) {
            st(hidden + ((int64_t)t * top + c) * ff + f, fmaxf(g, 0.f) * fmaxf(g, 0.f));
        }
    }
}

// grid (n, ceil(width / (warps * ROWS_PER_WARP))).  down: [experts][width][ff].
template <typename T>
__global__ void __launch_bounds__(128)
moe_down_kernel(const T* __restrict__ hidden, const int* __restrict__ tokens, const int* __restrict__ table, int top,
                int n_experts, const T* __restrict__ down, float weight, const float* __restrict__ base, int base_splits,
                int64_t base_stride, float* __restrict__ out, int width, int ff) {
    extern __shared__ float hs[];                                            // [top][ff]
    pdl_trigger();
    pdl_wait();
    hidden = fresh(hidden);
    base = fresh(base);
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int j = threadIdx.x; j < top * ff; j += blockDim.x) hs[j] = ld(hidden + (int64_t)t * top * ff + j);
    __syncthreads();
    const int o0 = (blockIdx.y * (blockDim.x >> 5) + warp) * ROWS_PER_WARP;
    for (int o = o0; o < min(o0 + ROWS_PER_WARP, width); ++o) {
        float sum = 0.f;
        for (int c = 0; c < top; ++c) {
            const int ex = table[(int64_t)tokens[t] * top + c];
            if (ex < 0 || ex >= n_experts) continue;
            sum += dot_row(down + ((int64_t)ex * width + o) * ff, hs + c * ff, ff, lane);
        }
        if (lane == 0) {
            float v = 0.f;
            for (int s = 0; s < base_splits; ++s) v += base[s * base_stride + (int64_t)t * width + o];
            out[(int64_t)t * width + o] = v + weight * sum;
        }
    }
}

// ---- by expert: every matrix row is read once for all the step's tokens that use it -----------
// grid (experts, ceil(rows / (4 warps x ROWS_PER_WARP))).  A block lists the (token, choice) pairs of its
// expert (in no order: every pair's result is computed on its own), leaves if there are none, and
// then its warps take matrix rows, four each (for the gated pair: four gate rows and four up rows),
// and multiply them with the inputs of two pairs at a time, 16 bytes a lane and trip, float32 sums
// (a lane's elements in index order, the 32 lanes by the butterfly).
//   MODE 1: in = x [n, k], w = [experts][2][rows][k], hidden[pair][row] = silu(g) * u
//   MODE 2: in = x [n, k], w = [experts][rows][k], hidden[pair][row] = max(g, 0)^2
//   MODE 0: in = hidden [n * top, k], w = [experts][rows][k], y[pair][row] = the product (float32)
template <typename T, int MODE>
__global__ void __launch_bounds__(128)
moe_expert_rows_kernel(const T* __restrict__ in, const int* __restrict__ tokens, const int* __restrict__ table, int top,
                       int n_pairs, const T* __restrict__ w, T* __restrict__ hidden_out, float* __restrict__ y_out, int rows,
                       int k) {
    extern __shared__ int list[];
    __shared__ int count;
    constexpr bool GATED = MODE == 1, FROM_X = MODE != 0;
    pdl_trigger();
    pdl_wait();
    in = fresh(in);
    const int ex = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) count = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += blockDim.x)
        if (table[(int64_t)tokens[p / top] * top + (p - p / top * top)] == ex) list[atomicAdd(&count, 1)] = p;
    __syncthreads();
    const int n_list = count;
    if (n_list == 0) return;
    constexpr int VN = Vec16<T>::N;
    const bool vec = k % VN == 0 && ((((uintptr_t)w) | ((uintptr_t)in)) & 15) == 0;
    const int r0 = (blockIdx.y * (blockDim.x >> 5) + warp) * ROWS_PER_WARP;
    if (r0 >= rows) return;
    if (vec && r0 + ROWS_PER_WARP <= rows) {
        // the warp's rows side by side: their loads are in flight together, and an input's 16 bytes serve all of them
        const T* wg = w + (((int64_t)ex * (GATED ? 2 : 1)) * rows + r0) * k;
        const T* wu = wg + (int64_t)rows * k;
        for (int m0 = 0; m0 < n_list; m0 += 2) {
            const T* xin[2];
            float ag[ROWS_PER_WARP][2], au[ROWS_PER_WARP][2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int p = list[min(m0 + u, n_list - 1)];
                xin[u] = in + (int64_t)(FROM_X ? p / top : p) * k;
#pragma unroll
                for (int r = 0; r < ROWS_PER_WARP; ++r) ag[r][u] = au[r][u] = 0.f;
            }
            for (int j = lane * VN; j < k; j += 32 * VN) {
                Vec16<T> g[ROWS_PER_WARP], up[ROWS_PER_WARP], xv[2];
#pragma unroll
                for (int r = 0; r < ROWS_PER_WARP; ++r) {
                    g[r].load(wg + (int64_t)r * k + j);
                    if (GATED) up[r].load(wu + (int64_t)r * k + j);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) xv[u].load(xin[u] + j);
#pragma unroll
                for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
                    for (int u = 0; u < 2; ++u)
#pragma unroll
                        for (int i = 0; i < VN; ++i) {
                            ag[r][u] = fmaf(g[r].v[i], xv[u].v[i], ag[r][u]);
                            if (GATED) au[r][u] = fmaf(up[r].v[i], xv[u].v[i], au[r][u]);
                        }
            }
#pragma unroll
            for (int r = 0; r < ROWS_PER_WARP; ++r)
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float gs = warp_sum(ag[r][u]), us = GATED ? warp_sum(au[r][u]) : 0.f;
                    if (lane == 0 && m0 + u < n_list) {
                        const int p = list[m0 + u];
                        if (GATED) st(hidden_out + (int64_t)p * rows + r0 + r, gs / (1.0f + expf(-gs)) * us);
                        else if (MODE == 2) st(hidden_out + (int64_t)p * rows + r0 + r, fmaxf(gs, 0.f) * fmaxf(gs, 0.f));
                        else y_out[(int64_t)p * rows + r0 + r] = gs;
                    }
                }
        }
        return;
    }
    for (int r = r0; r < min(r0 + ROWS_PER_WARP, rows); ++r) {
        const T* wg = w + (((int64_t)ex * (GATED ? 2 : 1)) * rows + r) * k;
        const T* wu = wg + (int64_t)rows * k;
        for (int m0 = 0; m0 < n_list; m0 += 4) {
            const T* xin[4];
            float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int p = list[min(m0 + u, n_list - 1)];
                xin[u] = in + (int64_t)(FROM_X ? p / top : p) * k;
            }
            for (int j = lane; j < k; j += 32) {
                const float g = ld(wg + j), up = GATED ? ld(wu + j) : 0.f;
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const float xv = ld(xin[u] + j);
                    ag[u] = fmaf(g, xv, ag[u]);
                    if (GATED) au[u] = fmaf(up, xv, au[u]);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float g = warp_sum(ag[u]), up = GATED ? warp_sum(au[u]) : 0.f;
                if (lane == 0 && m0 + u < n_list) {
                    const int p = list[m0 + u];
                    if (GATED) st(hidden_out + (int64_t)p * rows + r, g / (1.0f + expf(-g)) * up);
                    else if (MODE == 2) st(hidden_out + (int64_t)p * rows + r, fmaxf(g, 0.f) * fmaxf(g, 0.f));
                    else y_out[(int64_t)p * rows + r] = g;
                }
            }
        }
    }
}

constexpr int PAIRS_BY_EXPERT = 12000;          // pairs whose list fits one block's shared memory

// ---- the form for many tokens: rows sorted by expert ---------------------------------------
// The (token, choice) pairs of a step, numbered t * top + c, are sorted by expert (pairs of one
// expert keep their order), so that every expert's rows lie together and go through an ordinary
// matrix product.  route: expert_of[pair] and counts[expert]; place: row_of[pair] (a block per
// expert walks all pairs in order and numbers its own); gather: the sorted rows of x; combine:
// out[t] = base[t] + weight * (y[row_of[t, 0]] + y[row_of[t, 1]] + ...), choices in table order.
__global__ void moe_route_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int top, int n_experts,
                                 int* __restrict__ expert_of, int* __restrict__ counts, int n_pairs) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pairs) return;
    const int t = i / top, c = i - t * top;
    int ex = table[(int64_t)tokens[t] * top + c];
    if (ex < 0 || ex >= n_experts) ex = -1;
    expert_of[i] = ex;
    if (ex >= 0) atomicAdd(counts + ex, 1);               // (a count: the order of the additions does not matter)
}

__global__ void __launch_bounds__(1024)
moe_place_kernel(const int* __restrict__ expert_of, const int* __restrict__ counts, int* __restrict__ row_of, int n_pairs, int pad,
                 int* __restrict__ expert_of_tile) {
    __shared__ int warp_count[32];
    pdl_trigger();
    pdl_wait();
    expert_of = fresh(expert_of);
    counts = fresh(counts);
    const int ex = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    // every expert's rows start at a multiple of `pad`; with a table of tiles (of `pad` rows), the expert's tiles are named
    int base = 0;
    for (int e = 0; e < ex; ++e) base += (counts[e] + pad - 1) / pad * pad;
    if (expert_of_tile)
        for (int tile = threadIdx.x; tile < (counts[ex] + pad - 1) / pad; tile += blockDim.x) expert_of_tile[base / pad + tile] = ex;
    // pairs in chunks of one per thread: a pair's row is the expert's first row plus the number of
    // the expert's pairs before it (earlier chunks, earlier warps of the chunk, earlier lanes of the warp)
    for (int i0 = 0; i0 < n_pairs; i0 += blockDim.x) {
        const int i = i0 + threadIdx.x;
        const int mine_ex = i < n_pairs ? expert_of[i] : -2;
        const bool mine = mine_ex == ex;
        const unsigned m = __ballot_sync(0xffffffffu, mine);
        if (lane == 0) warp_count[warp] = __popc(m);
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < n_warps; ++w) {
            const int c = warp_count[w];
            before += w < warp ? c : 0;
            total += c;
        }
        if (mine) row_of[i] = base + before + __popc(m & ((1u << lane) - 1));
        if (ex == 0 && mine_ex == -1) row_of[i] = -1;      // pairs without an expert have no row
        base += total;
        __syncthreads();
    }
}

template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ row_of, int top, T* __restrict__ xs, int width) {
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    row_of = fresh(row_of);
    const int pair = blockIdx.x, row = row_of[pair];
    if (row < 0) return;
    const T* src = x + (int64_t)(pair / top) * width;
    T* dst = xs + (int64_t)row * width;
    constexpr int VN = Vec16<T>::N;
    if (width % VN == 0 && (((uintptr_t)x | (uintptr_t)xs) & 15) == 0) {
        for (int j = threadIdx.x * VN; j < width; j += blockDim.x * VN)
            *reinterpret_cast<uint4*>(dst + j) = *reinterpret_cast<const uint4*>(src + j);
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) dst[j] = src[j];
    }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, const int* __restrict__ row_of, int top, float weight,
                                   const float* __restrict__ base, int base_splits, int64_t base_stride,
                                   float* __restrict__ out, int width) {
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    row_of = fresh(row_of);
    base = fresh(base);
    const int t = blockIdx.x;
    if ((width & 3) == 0 && (base_stride & 3) == 0) {
        // four neighbours a thread; the rows' and the partial sums' loads are independent and issued together
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c = 0; c < top; ++c) {
                const int row = row_of ? row_of[t * top + c] : t * top + c;
                if (row >= 0) {
                    const float4 r = *reinterpret_cast<const float4*>(y + (int64_t)row * width + j);
                    sum.x += r.x; sum.y += r.y; sum.z += r.z; sum.w += r.w;
                }
            }
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < base_splits; ++s) {
                const float4 r = *reinterpret_cast<const float4*>(base + s * base_stride + (int64_t)t * width + j);
                v.x += r.x; v.y += r.y; v.z += r.z; v.w += r.w;
            }
            *reinterpret_cast<float4*>(out + (int64_t)t * width + j) =
                make_float4(v.x + weight * sum.x, v.y + weight * sum.y, v.z + weight * sum.z, v.w + weight * sum.w);
        }
        return;
    }
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float sum = 0.f;
        for (int c = 0; c < top; ++c) {
            const int row = row_of ? row_of[t * top + c] : t * top + c;
            if (row >= 0) sum += y[(int64_t)row * width + j];
        }
        float v = 0.f;
        for (int s = 0; s < base_splits; ++s) v += base[s * base_stride + (int64_t)t * width + j];
        out[(int64_t)t * width + j] = v + weight * sum;
    }
}


// ---- experts chosen by a router ---------------------------------------------------------------
// One warp per token.  z = the router's logits (float32 partial sums, added in index order) over all its outputs;
// s = softmax(z) over the outputs (`scoring` 0) or sigmoid(z) of each (`scoring` 1); the choice score of an output is
// s + correction.  With `groups` > 0 the outputs form that many equal groups of neighbours; a group's score is the sum of
// its two largest choice scores (of its only one, in groups of one); only outputs of the `keep` best groups can be chosen
// (the others' choice scores count as minus infinity).  The `top` outputs with the largest choice scores are chosen (the
// lowest index among equals), one after the other; choice[t][c] = the output's index, weight[t][c] = s of it, divided by
// (the chosen ones' sum + norm_eps) if `renormalize`, times `scale`.  Outputs from n_experts on stand for experts without
// matrices; the kernels that walk the experts' matrices pass them over.  ident[t] = t: with it as "token ids", choice is
// the table those kernels read.
__device__ __forceinline__ void warp_best(float& best, int& at) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (ob > best || (ob == best && oa < at)) {
            best = ob;
            at = oa;
        }
    }
}

__global__ void __launch_bounds__(32)
moe_router_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, int ld, int n_out, const float* __restrict__ correction,
                  int top, int renormalize, int* __restrict__ choice, float* __restrict__ weight, int* __restrict__ ident,
                  int scoring, int groups, int keep, float scale, float norm_eps) {
    extern __shared__ float sm[];
    float* score = sm;                                                  // [n_out]
    float* pick = sm + n_out;                                           // [n_out]: score + correction, -inf once chosen
    float* gscore = pick + n_out;                                       // [groups]: -inf once kept
    float* gkept = gscore + groups;                                     // [groups]: 1 if kept
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    const int t = blockIdx.x, lane = threadIdx.x;
    float m = -INFINITY;
    for (int e = lane; e < n_out; e += 32) {
        float z = 0.f;
        for (int s = 0; s < splits; ++s) z += parts[s * split_stride + (int64_t)t * ld + e];
        score[e] = z;
        m = fmaxf(m, z);
    }
    if (scoring == 0) {
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < n_out; e += 32) {
            const float p = expf(score[e] - m);
            score[e] = p;
            sum += p;
        }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < n_out; e += 32) score[e] *= inv;
    } else {
        for (int e = lane; e < n_out; e += 32) score[e] = 1.0f / (1.0f + expf(-score[e]));
    }
    for (int e = lane; e < n_out; e += 32) pick[e] = score[e] + (correction ? correction[e] : 0.f);
    __syncwarp();
    if (groups > 0) {
        const int per = n_out / groups;
        for (int g = lane; g < groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;                         // the two largest of the group
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = pick[e];
                if (v > a) {
                    b = a;
                    a = v;
                } else if (v > b) {
                    b = v;
                }
            }
            gscore[g] = per > 1 ? a + b : a;
            gkept[g] = 0.f;
        }
        __syncwarp();
        for (int c = 0; c < keep; ++c) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gscore[g] > best) {
                    best = gscore[g];
                    at = g;
                }
            warp_best(best, at);
            if (at >= groups) break;
            if (lane == 0) {
                gscore[at] = -INFINITY;
                gkept[at] = 1.f;
            }
            __syncwarp();
        }
        for (int e = lane; e < n_out; e += 32)
            if (gkept[e / per] == 0.f) pick[e] = -INFINITY;
        __syncwarp();
    }
    float chosen_sum = 0.f;
    for (int c = 0; c < top; ++c) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int e = lane; e < n_out; e += 32)
            if (pick[e] > best) {                                      // (a lane's candidates in index order: the first of equals stays)
                best = pick[e];
                at = e;
            }
        warp_best(best, at);
        if (at >= n_out) at = 0;                                        // (nothing left to choose: scores that are no numbers)
        if (lane == 0) {
            choice[(int64_t)t * top + c] = at;
            weight[(int64_t)t * top + c] = score[at];
            pick[at] = -INFINITY;
        }
        chosen_sum += score[at];
        __syncwarp();
    }
    if (lane == 0)
        for (int c = 0; c < top; ++c) {
            float w = weight[(int64_t)t * top + c];
            if (renormalize) w /= (chosen_sum + norm_eps);
            weight[(int64_t)t * top + c] = w * scale;
        }
    if (lane == 0 && ident) ident[t] = t;
}

// y[pair][o] = down_{e(pair)}[o] . hidden[pair], every pair on its own.  grid (pairs, ceil(width / (warps x ROWS_PER_WARP))).
template <typename T>
__global__ void __launch_bounds__(128)
moe_down_pair_kernel(const T* __restrict__ hidden, const int* __restrict__ tokens, const int* __restrict__ table, int top,
                     int n_experts, const T* __restrict__ down, float* __restrict__ y, int width, int ff) {
    extern __shared__ float hs[];                                       // [ff]
    pdl_trigger();
    pdl_wait();
    hidden = fresh(hidden);
    const int pair = blockIdx.x, t = pair / top, c = pair - t * top;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int ex = table[(int64_t)tokens[t] * top + c];
    if (ex < 0 || ex >= n_experts) return;
    for (int j = threadIdx.x; j < ff; j += blockDim.x) hs[j] = ld(hidden + (int64_t)pair * ff + j);
    __syncthreads();
    const int o0 = (blockIdx.y * (blockDim.x >> 5) + warp) * ROWS_PER_WARP;
    for (int o = o0; o < min(o0 + ROWS_PER_WARP, width); ++o) {
        const float v = dot_row(down + ((int64_t)ex * width + o) * ff, hs, ff, lane);
        if (lane == 0) y[(int64_t)pair * width + o] = v;
    }
}

// out[t] = sum over c of weight[t][c] * r(t, c), choices in index order:  r = the row of y that holds the pair's result
// (row_of[t][c], or the pair's own number where the rows are not sorted) for an expert with matrices; x[t] itself for
// an output that stands for an expert that returns its input; nothing otherwise.
template <typename T>
__global__ void moe_combine_weighted_kernel(const float* __restrict__ y, const int* __restrict__ row_of, const int* __restrict__ choice,
                                            const float* __restrict__ weight, const T* __restrict__ x, int n_experts, int top,
                                            float* __restrict__ out, int width, const float* __restrict__ base, int base_splits,
                                            int64_t base_stride, const float* __restrict__ gate, int gate_splits, int64_t gate_stride,
                                            int gate_ld) {
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    row_of = fresh(row_of);
    choice = fresh(choice);
    weight = fresh(weight);
    x = fresh(x);
    base = fresh(base);
    gate = fresh(gate);
    const int t = blockIdx.x;
    float bf = 1.f;                                                     // the factor of what every token uses: sigmoid of the gate's number
    if (base && gate) {
        float g = 0.f;
        for (int s = 0; s < gate_splits; ++s) g += gate[s * gate_stride + (int64_t)t * gate_ld];
        bf = 1.0f / (1.0f + expf(-g));
    }
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float sum = 0.f;
        for (int c = 0; c < top; ++c) {
            const int ex = choice[(int64_t)t * top + c];
            const float wgt = weight[(int64_t)t * top + c];
            if (ex >= 0 && ex < n_experts) {
                const int64_t row = row_of ? row_of[(int64_t)t * top + c] : (int64_t)t * top + c;
                if (row >= 0) sum = fmaf(wgt, y[row * width + j], sum);
            } else if (ex >= n_experts && x) {
                sum = fmaf(wgt, ld(x + (int64_t)t * width + j), sum);
            }
        }
        if (base) {
            float v = 0.f;
            for (int s = 0; s < base_splits; ++s) v += base[s * base_stride + (int64_t)t * width + j];
            sum = fmaf(bf, v, sum);
        }
        out[(int64_t)t * width + j] = sum;
    }
}

template <typename T>
int moe_up(const void* x, const int* tokens, const int* table, int top, int n_experts, const void* gate_up, void* hidden, int n,
           int width, int ff, int gated, cudaStream_t s) {
    WICK_REQUIRE(top > 0 && n_experts > 0 && width > 0 && ff > 0, "moe_up: bad sizes");
    if (n == 0) return 0;
    const int warps = 4;
    if ((int64_t)n * top <= PAIRS_BY_EXPERT) {
        if (gated) {
            WICK_CUDA(launch(moe_expert_rows_kernel<T, 1>, dim3(n_experts, ceil_div(ff, warps * ROWS_PER_WARP)), dim3(warps * 32),
                             (size_t)n * top * sizeof(int), s, (const T*)x, tokens, table, top, n * top, (const T*)gate_up, (T*)hidden,
                             (float*)nullptr, ff, width));
        } else {
            WICK_CUDA(launch(moe_expert_rows_kernel<T, 2>, dim3(n_experts, ceil_div(ff, warps * ROWS_PER_WARP)), dim3(warps * 32),
                             (size_t)n * top * sizeof(int), s, (const T*)x, tokens, table, top, n * top, (const T*)gate_up, (T*)hidden,
                             (float*)nullptr, ff, width));
        }
        return check_launch("moe_up");
    }
    WICK_REQUIRE((size_t)width * 4 <= 48 * 1024, "moe_up: width %d is beyond %d", width, 48 * 1024 / 4);
    WICK_CUDA(launch(moe_up_kernel<T>, dim3(n * top, ceil_div(ff, warps * ROWS_PER_WARP)), dim3(warps * 32), (size_t)width * 4, s,
                     (const T*)x, tokens, table, top, n_experts, (const T*)gate_up, (T*)hidden, width, ff, gated));
    return check_launch("moe_up");
}

template <typename T>
int moe_down(const void* hidden, const int* tokens, const int* table, int top, int n_experts, const void* down, float weight,
             const float* base, int base_splits, float* y, float* out, int n, int width, int ff, cudaStream_t s) {
    WICK_REQUIRE(top > 0 && n_experts > 0 && width > 0 && ff > 0, "moe_down: bad sizes");
    if (n == 0) return 0;
    const int warps = 4;
    if (y && (int64_t)n * top <= PAIRS_BY_EXPERT) {
        // y [n * top, width] (float32, zero on entry): every pair's product, then the sum per token
        WICK_CUDA(launch(moe_expert_rows_kernel<T, 0>, dim3(n_experts, ceil_div(width, warps * ROWS_PER_WARP)), dim3(warps * 32),
                         (size_t)n * top * sizeof(int), s, (const T*)hidden, tokens, table, top, n * top, (const T*)down, (T*)nullptr,
                         y, width, ff));
        WICK_CUDA(launch(moe_combine_kernel, dim3(n), dim3(256), 0, s, (const float*)y, (const int*)nullptr, top, weight, base,
                         base_splits, (int64_t)n * width, out, width));
        return check_launch("moe_down");
    }
    const size_t smem = (size_t)top * ff * 4;
    WICK_REQUIRE(smem <= 48 * 1024, "moe_down: %d choices of %d numbers are beyond one block's shared memory", top, ff);
    WICK_CUDA(launch(moe_down_kernel<T>, dim3(n, ceil_div(width, warps * ROWS_PER_WARP)), dim3(warps * 32), smem, s,
                     (const T*)hidden, tokens, table, top, n_experts, (const T*)down, weight, base, base_splits,
                     (int64_t)n * width, out, width, ff));
    return check_launch("moe_down");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

WICK_API int wick_moe_up_bf16(const void* x, const int* tokens, const int* table, int top, int n_experts, const void* gate_up,
                              void* hidden, int n, int width, int ff, int gated, void* s) {
    return moe_up<bf16>(x, tokens, table, top, n_experts, gate_up, hidden, n, width, ff, gated, (cudaStream_t)s);
}
WICK_API int wick_moe_up_f32(const void* x, const int* tokens, const int* table, int top, int n_experts, const void* gate_up,
                             void* hidden, int n, int width, int ff, int gated, void* s) {
    return moe_up<float>(x, tokens, table, top, n_experts, gate_up, hidden, n, width, ff, gated, (cudaStream_t)s);
}
WICK_API int wick_moe_down_bf16(const void* hidden, const int* tokens, const int* table, int top, int n_experts, const void* down,
                                float weight, const float* base, int base_splits, float* y, float* out, int n, int width, int ff,
                                void* s) {
    return moe_down<bf16>(hidden, tokens, table, top, n_experts, down, weight, base, base_splits, y, out, n, width, ff,
                          (cudaStream_t)s);
}
WICK_API int wick_moe_down_f32(const void* hidden, const int* tokens, const int* table, int top, int n_experts, const void* down,
                               float weight, const float* base, int base_splits, float* y, float* out, int n, int width, int ff,
                               void* s) {
    return moe_down<float>(hidden, tokens, table, top, n_experts, down, weight, base, base_splits, y, out, n, width, ff,
                           (cudaStream_t)s);
}
WICK_API int wick_moe_pairs_by_expert() { return PAIRS_BY_EXPERT; }

// expert_of, row_of: int32 [n * top]; counts: int32 [experts], zero on entry.
// pad: every expert's rows start at a multiple of it (1: no gaps); expert_of_tile: null, or int32 [enough tiles of
// pad rows]: which expert a tile's rows belong to.
WICK_API int wick_moe_route(const int* tokens, const int* table, int top, int n_experts, int* expert_of, int* counts,
                            int* row_of, int n, int pad, int* expert_of_tile, void* s) {
    WICK_REQUIRE(pad >= 1, "moe_route: bad padding");
    WICK_REQUIRE(top > 0 && n_experts > 0 && n >= 0, "moe_route: bad sizes");
    if (n == 0) return 0;
    const int pairs = n * top;
    WICK_CUDA(launch(moe_route_kernel, dim3(ceil_div(pairs, 256)), dim3(256), 0, (cudaStream_t)s, tokens, table, top, n_experts,
                     expert_of, counts, pairs));
    WICK_CUDA(launch(moe_place_kernel, dim3(n_experts), dim3(pairs >= 1024 ? 1024 : 256), 0, (cudaStream_t)s, (const int*)expert_of,
                     (const int*)counts, row_of, pairs, pad, expert_of_tile));
    return check_launch("moe_route");
}
WICK_API int wick_moe_gather_bf16(const void* x, const int* row_of, int top, void* xs, int n, int width, void* s) {
    if (n == 0) return 0;
    WICK_CUDA(launch(moe_gather_kernel<bf16>, dim3(n * top), dim3(128), 0, (cudaStream_t)s, (const bf16*)x, row_of, top, (bf16*)xs, width));
    return check_launch("moe_gather");
}
WICK_API int wick_moe_gather_f32(const void* x, const int* row_of, int top, void* xs, int n, int width, void* s) {
    if (n == 0) return 0;
    WICK_CUDA(launch(moe_gather_kernel<float>, dim3(n * top), dim3(128), 0, (cudaStream_t)s, (const float*)x, row_of, top, (float*)xs, width));
    return check_launch("moe_gather");
}
WICK_API int wick_moe_combine(const float* y, const int* row_of, int top, float weight, const float* base, int base_splits,
                              float* out, int n, int width, void* s) {
    if (n == 0) return 0;
    WICK_CUDA(launch(moe_combine_kernel, dim3(n), dim3(256), 0, (cudaStream_t)s, y, row_of, top, weight, base, base_splits,
                     (int64_t)n * width, out, width));
    return check_launch("moe_combine");
}

// parts: float32 [splits, n, ld] (the router's logits as partial sums in a row's first n_out columns; a row may hold further
// columns of the same product); correction: float32 [n_out] or null; choice: int32 [n, top]; weight: float32 [n, top];
// ident: int32 [n] or null.
WICK_API int wick_moe_router(const float* parts, int splits, int n, int ld, int n_out, const float* correction, int top, int renormalize,
                             int* choice, float* weight, int* ident, int scoring, int groups, int keep, float scale, float norm_eps,
                             void* s) {
    WICK_REQUIRE(splits >= 1 && n_out > 0 && ld >= n_out && top > 0 && top <= n_out, "moe_router: bad sizes");
    WICK_REQUIRE(scoring == 0 || scoring == 1, "moe_router: scores are a softmax (0) or sigmoids (1)");
    WICK_REQUIRE(groups == 0 || (groups > 0 && n_out % groups == 0 && keep > 0 && keep <= groups && keep * (n_out / groups) >= top),
                 "moe_router: %d outputs do not form %d equal groups of which %d hold %d choices", n_out, groups, keep, top);
    WICK_REQUIRE((size_t)(n_out + groups) * 8 <= 48 * 1024, "moe_router: %d outputs are beyond one block's shared memory", n_out);
    if (n == 0) return 0;
    WICK_CUDA(launch(moe_router_kernel, dim3(n), dim3(32), (size_t)(n_out + groups) * 2 * sizeof(float), (cudaStream_t)s, parts, splits,
                     (int64_t)n * ld, ld, n_out, correction, top, renormalize, choice, weight, ident, scoring, groups, keep, scale,
                     norm_eps));
    return check_launch("moe_router");
}

// y: float32 [n * top, width], zero on entry where pairs without an expert must read as nothing.
template <typename T>
static int moe_expert_down(const void* hidden, const int* tokens, const int* table, int top, int n_experts, const void* down, float* y,
                           int n, int width, int ff, cudaStream_t s) {
    WICK_REQUIRE(top > 0 && n_experts > 0 && width > 0 && ff > 0, "moe_expert_down: bad sizes");
    if (n == 0) return 0;
    const int warps = 4;
    if ((int64_t)n * top <= PAIRS_BY_EXPERT) {
        WICK_CUDA(launch(moe_expert_rows_kernel<T, 0>, dim3(n_experts, ceil_div(width, warps * ROWS_PER_WARP)), dim3(warps * 32),
                         (size_t)n * top * sizeof(int), s, (const T*)hidden, tokens, table, top, n * top, (const T*)down, (T*)nullptr,
                         y, width, ff));
        return check_launch("moe_expert_down");
    }
    WICK_REQUIRE((size_t)ff * 4 <= 48 * 1024, "moe_expert_down: an inner size of %d is beyond one block's shared memory", ff);
    WICK_CUDA(launch(moe_down_pair_kernel<T>, dim3(n * top, ceil_div(width, warps * ROWS_PER_WARP)), dim3(warps * 32), (size_t)ff * 4, s,
                     (const T*)hidden, tokens, table, top, n_experts, (const T*)down, y, width, ff));
    return check_launch("moe_expert_down");
}
WICK_API int wick_moe_expert_down_bf16(const void* hidden, const int* tokens, const int* table, int top, int n_experts,
                                       const void* down, float* y, int n, int width, int ff, void* s) {
    return moe_expert_down<bf16>(hidden, tokens, table, top, n_experts, down, y, n, width, ff, (cudaStream_t)s);
}
WICK_API int wick_moe_expert_down_f32(const void* hidden, const int* tokens, const int* table, int top, int n_experts,
                                      const void* down, float* y, int n, int width, int ff, void* s) {
    return moe_expert_down<float>(hidden, tokens, table, top, n_experts, down, y, n, width, ff, (cudaStream_t)s);
}

// y: float32 rows; row_of: int32 [n, top] or null (rows in pair order); choice: int32 [n, top]; weight: float32 [n, top];
// x: [n, width] or null (what an expert without matrices returns); out: float32 [n, width].
// base: float32 [base_splits, n, width] or null: what every token uses, added with the factor sigmoid(sum of gate[:, t]) where
// gate is given, else 1.  gate: a column of float32 partial sums [gate_splits, n, gate_ld], the pointer at the column's first
// number (the gate's number may be a further column of the router's product).
#define WICK_MOE_COMBINE_WEIGHTED(NAME, T)                                                                                    \
    WICK_API int NAME(const float* y, const int* row_of, const int* choice, const float* weight, const void* x, int n_experts, \
                      int top, float* out, int n, int width, const float* base, int base_splits, const float* gate,           \
                      int gate_splits, int gate_ld, void* s) {                                                                \
        if (n == 0) return 0;                                                                                                 \
        WICK_REQUIRE(!gate || gate_ld >= 1, "moe_combine_weighted: the gate's rows need a length");                           \
        WICK_CUDA(launch(moe_combine_weighted_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)s, y, row_of, choice, weight,     \
                         (const T*)x, n_experts, top, out, width, base, base_splits, (int64_t)n * width, gate, gate_splits,    \
                         (int64_t)n * gate_ld, gate_ld));                                                                      \
        return check_launch("moe_combine_weighted");                                                                          \
    }
WICK_MOE_COMBINE_WEIGHTED(wick_moe_combine_weighted_bf16, bf16)
WICK_MOE_COMBINE_WEIGHTED(wick_moe_combine_weighted_f32, float)
