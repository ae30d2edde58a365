// Attention with options, for any head sizes (run-time numbers): projection biases, an
// RMS norm of q and k over spans of any length (a head, or the whole projection), a
// rotation of neighbouring or of half-split pairs over the first dims of each head, values
// blended with the values another layer made for the same token, key and value heads of
// different sizes, a visibility rule (all earlier keys, the query's own block of positions,
// or the last positions), and a sink in the softmax's denominator.
//
//   finish  : the q/k/v projection's float32 partial sums -> q (activation type) and the
//             token's key and value in its sequence's cache page
//   attend  : every new token over the cache, one block per (token, query head) or per (token, key/value head)
//
// Cache page of one schedule entry: [kv_head][64][d] keys, then [kv_head][64][e] values.
// Scores, the softmax, its weights and the weighted sum are float32.  A token's work is the
// same whatever else the step holds, up to the number of warps that share its keys.
#include "common.cuh"

namespace wick {

constexpr int MASK_CAUSAL = 0, MASK_BLOCK = 1, MASK_WINDOW = 2;

// First key that the query at position p sees.
__device__ __forceinline__ int first_visible(int p, int mask, int size) {
    if (mask == MASK_BLOCK) return p / size * size;
    if (mask == MASK_WINDOW) return max(0, p - size + 1);
    return 0;
}

// ---------------------------------------------------------------------------
// One block per token.  The row [q | k | v] (H d + G d + G e numbers) is summed into shared
// memory with the biases; the norms' factors follow (all warps); then one pass applies the norm, turns the pairs
// (angles from the step's tables) and stores q and k, and another blends and stores the values.
//   v_mode 0: values as projected; 1: also kept in v_keep [n, G e] (float32) for later layers;
//   2: v <- (1 - lambda) v + lambda v_keep.
//   pairing 0: (2i, 2i + 1) rotate together; 1: (i, i + rot_dims / 2).
//   maps: a q or k head of d numbers is `maps` vectors of d / maps, side by side, each of which is
//   turned on its own (the first rot_dims elements of each); 1: the head is one vector.
//   cols: numbers a token's row of partial sums holds (the projection may carry further columns behind
//   q, k and v, an output gate's for instance, which this kernel leaves alone).
//   flags: FINISH_KEYS_ARE_VALUES: the row holds no values; a head's value is its key as projected, before
//   any norm or rotation (e = d).  FINISH_NORM_AFTER: the norm follows the rotation instead of preceding it.
//   A span without a weight vector (q_span > 0, q_w null) is divided by its root mean square and no more.
constexpr int FINISH_KEYS_ARE_VALUES = 1, FINISH_NORM_AFTER = 2;
constexpr int MAX_SPANS = 512;                  // spans of the two norms together (a span per head at most)

template <typename T>
__global__ void __launch_bounds__(256)
qkv_finish_kernel(const float* __restrict__ parts, int splits, int64_t split_stride, const float* __restrict__ bias,
                  int H, int G, int d, int e, const float* __restrict__ q_w, int q_span, const float* __restrict__ k_w,
                  int k_span, float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dims,
                  int pairing, int maps, float* __restrict__ v_keep, int v_mode, const float* __restrict__ lambda, T* __restrict__ q_out,
                  T* __restrict__ kv, const int* __restrict__ page_table, int table_width,
                  const int* __restrict__ seq_of_token, const int* __restrict__ positions, int write_kv, int cols, int flags) {
    extern __shared__ float row[];
    __shared__ float partial[MAX_SPANS], span_scale[MAX_SPANS];
    pdl_trigger();
    pdl_wait();
    parts = fresh(parts);
    v_keep = fresh(v_keep);
    cos_t = fresh(cos_t);
    sin_t = fresh(sin_t);
    const int t = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, n_warps = blockDim.x >> 5;
    const bool keys_are_values = flags & FINISH_KEYS_ARE_VALUES, norm_after = flags & FINISH_NORM_AFTER;
    const int Wq = H * d, Wk = G * d, Wv = G * e, W = Wq + Wk + (keys_are_values ? 0 : Wv);
    if ((W & 3) == 0 && (cols & 3) == 0 && (split_stride & 3) == 0) {
        // four neighbours a load, the loads of four partial sums issued together (a chain of dependent trips to
        // the L2 cache is what a step of few tokens would otherwise wait for); the sums in index order
        for (int j = tid * 4; j < W; j += blockDim.x * 4) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s0 = 0; s0 < splits; s0 += 4) {
                float4 p4[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    p4[u] = s0 + u < splits ? *reinterpret_cast<const float4*>(parts + (s0 + u) * split_stride + (int64_t)t * cols + j)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    v.x += p4[u].x; v.y += p4[u].y; v.z += p4[u].z; v.w += p4[u].w;
                }
            }
            if (bias) {
                v.x += bias[j]; v.y += bias[j + 1]; v.z += bias[j + 2]; v.w += bias[j + 3];
            }
            *reinterpret_cast<float4*>(row + j) = v;
        }
    } else {
        for (int j = tid; j < W; j += blockDim.x) {
            float v = parts[(int64_t)t * cols + j];
            for (int s = 1; s < splits; ++s) v += parts[s * split_stride + (int64_t)t * cols + j];
            if (bias) v += bias[j];
            row[j] = v;
        }
    }
    __syncthreads();
    const int pos = positions[t];
    const float lam = v_mode == 2 ? *lambda : 0.f;
    T* page = nullptr;
    if (write_kv) {
        const int pg = page_table[(int64_t)seq_of_token[t] * table_width + pos / kPage];
        page = kv + (int64_t)pg * G * kPage * (d + e);
    }
    const int r = pos % kPage;
    const int half = cos_t ? rot_dims >> 1 : 0, rot = 2 * half;
    const int dm = d / maps;                               // a vector that turns on its own (the whole head, or one of its maps)
    // The values first (they read the row as projected): blended where asked, then stored.
    for (int j = tid; j < Wv; j += blockDim.x) {
        float v = row[(keys_are_values ? Wq : Wq + Wk) + j];
        if (v_mode == 1) v_keep[(int64_t)t * Wv + j] = v;
        if (v_mode == 2) v = (1.0f - lam) * v + lam * v_keep[(int64_t)t * Wv + j];
        if (write_kv) {
            const int g = j / e, x = j - g * e;
            st(page + (int64_t)G * kPage * d + ((int64_t)g * kPage + r) * e + x, v);
        }
    }
    if (norm_after && half > 0) {
        // the rotation comes before the norm: the pairs turn in place, and the pass at the end turns nothing
        __syncthreads();
        for (int idx = tid; idx < (H + G) * maps * half; idx += blockDim.x) {
            const int h = idx / half, i = idx - h * half;
            const int j0 = pairing == 0 ? 2 * i : i, j1 = pairing == 0 ? 2 * i + 1 : i + half;
            const float u = row[h * dm + j0], v = row[h * dm + j1];
            const float cs = cos_t[(int64_t)t * half + i], sn = sin_t[(int64_t)t * half + i];
            row[h * dm + j0] = u * cs - v * sn;
            row[h * dm + j1] = v * cs + u * sn;
        }
        __syncthreads();
    }
    // The norms: every span's sum of squares is made by `per` warps (each a slice of the span: lane l its
    // elements l, l + 32, ...; the 32 sums by the butterfly), the slices' sums are added in index order.
    const int nq = q_span > 0 ? Wq / q_span : 0, nk = k_span > 0 ? Wk / k_span : 0, n_spans = nq + nk;
    if (n_spans > 0) {
        const int per = max(1, n_warps / n_spans);
        for (int unit = warp; unit < n_spans * per; unit += n_warps) {
            const int seg = unit / per, part = unit - seg * per;
            const bool is_q = seg < nq;
            const int span = is_q ? q_span : k_span;
            const float* p = row + (is_q ? seg * q_span : Wq + (seg - nq) * k_span);
            const int lo = (int)((int64_t)span * part / per), hi = (int)((int64_t)span * (part + 1) / per);
            float ss = 0.f;
            for (int j = lo + lane; j < hi; j += 32) ss = fmaf(p[j], p[j], ss);
            ss = warp_sum(ss);
            if (lane == 0) partial[unit] = ss;
        }
        __syncthreads();
        for (int seg = tid; seg < n_spans; seg += blockDim.x) {
            float ss = 0.f;
            for (int part = 0; part < per; ++part) ss += partial[seg * per + part];
            span_scale[seg] = 1.0f / sqrtf(ss / (float)(seg < nq ? q_span : k_span) + eps);
        }
        __syncthreads();
    }
    // One pass over the pairs of every q and k head: the norm's factor and weight, the rotation (pairs of the first
    // rot_dims elements; the others pass), and the store.  Nothing goes back to shared memory.
    const int pairs = half + (dm - rot + 1) / 2;           // per vector: the turning pairs, then neighbours of the rest
    for (int idx = tid; idx < (H + G) * maps * pairs; idx += blockDim.x) {
        const int h = idx / pairs, i = idx - h * pairs;     // h counts the vectors: q's, then k's
        int j0, j1;
        if (i < half) {
            j0 = pairing == 0 ? 2 * i : i;
            j1 = pairing == 0 ? 2 * i + 1 : i + half;
        } else {
            j0 = rot + 2 * (i - half);
            j1 = j0 + 1;                                    // (beyond the head when its size is odd)
        }
        const bool is_q = h < H * maps, two = j1 < dm;
        const int base = h * dm;                            // (the k vectors follow the q vectors at the same stride)
        float u = row[base + j0], v = two ? row[base + j1] : 0.f;
        const float* w = is_q ? q_w : k_w;
        const int span = is_q ? q_span : k_span;
        if (span > 0) {
            const int o0 = (is_q ? base : base - Wq) + j0, o1 = (is_q ? base : base - Wq) + j1;   // index inside the projection
            u *= span_scale[(is_q ? 0 : nq) + o0 / span];
            if (two) v *= span_scale[(is_q ? 0 : nq) + o1 / span];
            if (w) {
                u *= w[o0 % span];
                if (two) v *= w[o1 % span];
            }
        }
        if (i < half && !norm_after) {
            const float cs = cos_t[(int64_t)t * half + i], sn = sin_t[(int64_t)t * half + i];
            const float ru = u * cs - v * sn, rv = v * cs + u * sn;
            u = ru;
            v = rv;
        }
        if (is_q) {
            T* o = q_out + (int64_t)t * Wq + base;
            st(o + j0, u);
            if (two) st(o + j1, v);
        } else if (write_kv) {
            const int kh = (h - H * maps) / maps, km = (h - H * maps) - kh * maps;
            T* o = page + ((int64_t)kh * kPage + r) * d + km * dm;
            st(o + j0, u);
            if (two) st(o + j1, v);
        }
    }
}

// ---------------------------------------------------------------------------
// One block per (token, query head); its warps share the visible keys, 32 at a time: warp w
// takes the keys lo + 32 w .., lo + 32 (w + warps) .., and so on.  In a tile, lane l scores key
// j0 + l (a dot product of d numbers, in index order), the warp's running maximum and sum
// follow, then every lane adds the 32 weighted value rows into its own elements of the result.
// At the end the warps' partial results are folded in warp order; a sink joins there as a
// score without a value.  This form runs with one warp a block, for steps of many tokens (the
// 32-bit path's prompts, and the twin of the tensor-core kernel); steps of few tokens take the
// grouped form below, which changes the order of sums only.
constexpr int E_CHUNKS = 2;                    // value sizes up to 256: a lane holds 4 neighbours of every 128

__device__ __forceinline__ void load4(const float* p, float* v) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float* v) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

template <typename T>
__global__ void __launch_bounds__(256)
attn_masked_kernel(const T* __restrict__ q, const T* __restrict__ kv, T* __restrict__ out,
                   const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                   const int* __restrict__ page_table, int table_width, int n_tokens, int H, int G, int d, int e,
                   float scale, int mask, int mask_size, const float* __restrict__ sink) {
    extern __shared__ float smem[];
    pdl_trigger();
    pdl_wait();
    q = fresh(q);
    kv = fresh(kv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    const int t = blockIdx.x / H, h = blockIdx.x - t * H;
    const int g = h / (H / G);
    const int pos = positions[t];
    const int* table = page_table + (int64_t)seq_of_token[t] * table_width;
    const int d_pad = (d + 3) & ~3, e_pad = 128 * E_CHUNKS;
    float* qs = smem;                           // [d]
    float* ms = qs + d_pad;                     // [warps] maxima, then [warps] sums
    float* accs = ms + 2 * n_warps;             // [warps][e_pad]
    for (int x = threadIdx.x; x < d; x += blockDim.x) qs[x] = ld(q + ((int64_t)t * H + h) * d + x);
    __syncthreads();
    const int64_t page_elems = (int64_t)G * kPage * (d + e);
    const int64_t v_off = (int64_t)G * kPage * d;
    constexpr int VN = Vec16<T>::N;
    const bool k_vec = d % VN == 0 && (((uintptr_t)kv) & 15) == 0 && (page_elems * sizeof(T)) % 16 == 0;
    const bool v_vec = e % 4 == 0 && (((uintptr_t)kv) & 15) == 0 && (page_elems * sizeof(T)) % 16 == 0 && (v_off * sizeof(T)) % 16 == 0;
    float m = -INFINITY, l = 0.f;
    float acc[4 * E_CHUNKS];
#pragma unroll
    for (int c = 0; c < 4 * E_CHUNKS; ++c) acc[c] = 0.f;
    for (int j0 = first_visible(pos, mask, mask_size) + 32 * warp; j0 <= pos; j0 += 32 * n_warps) {
        const int j = j0 + lane;
        // a tile of 32 keys lies in one page or in two: both are looked up once, ahead of the rows
        const int first_page = j0 / kPage;
        const int64_t page_a = table[first_page] * page_elems;
        const int64_t page_b = (first_page + 1) * kPage <= min(pos, j0 + 31) ? table[first_page + 1] * page_elems : page_a;
        float s = -INFINITY;
        if (j <= pos) {
            const T* kp = kv + (j / kPage == first_page ? page_a : page_b) + ((int64_t)g * kPage + (j % kPage)) * d;
            float dot = 0.f;
            if (k_vec) {
                for (int x = 0; x < d; x += 4 * VN) {            // four loads of 16 bytes in flight
                    Vec16<T> kk[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (x + u * VN < d) kk[u].load(kp + x + u * VN);
#pragma unroll
                    for (int u = 0; u < 4; ++u)
                        if (x + u * VN < d) {
#pragma unroll
                            for (int i = 0; i < VN; ++i) dot = fmaf(qs[x + u * VN + i], kk[u].v[i], dot);
                        }
                }
            } else {
                for (int x = 0; x < d; ++x) dot = fmaf(qs[x], ld(kp + x), dot);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));            // finite: key j0 is visible
        const float corr = expf(m - m_new);                    // (m = -inf at first: 0)
        const float p = j <= pos ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
        m = m_new;
#pragma unroll
        for (int c = 0; c < 4 * E_CHUNKS; ++c) acc[c] *= corr;
        const int n_keys = min(32, pos - j0 + 1);
        auto add_value = [&](int jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const int key = j0 + jj;
            const T* vp = kv + (key / kPage == first_page ? page_a : page_b) + v_off + ((int64_t)g * kPage + (key % kPage)) * e;
#pragma unroll
            for (int c = 0; c < E_CHUNKS; ++c) {
                const int x = 128 * c + 4 * lane;
                if (v_vec) {
                    if (x < e) {
                        float vv[4];
                        load4(vp + x, vv);
#pragma unroll
                        for (int i = 0; i < 4; ++i) acc[4 * c + i] = fmaf(pj, vv[i], acc[4 * c + i]);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (x + i < e) acc[4 * c + i] = fmaf(pj, ld(vp + x + i), acc[4 * c + i]);
                }
            }
        };
        if (n_keys == 32) {                                      // a whole tile: the 32 rows' loads are in flight together
#pragma unroll
            for (int jj = 0; jj < 32; ++jj) add_value(jj);
        } else {
            for (int jj = 0; jj < n_keys; ++jj) add_value(jj);
        }
    }
    if (lane == 0) {
        ms[warp] = m;
        ms[n_warps + warp] = l;
    }
#pragma unroll
    for (int c = 0; c < E_CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < 4; ++i) accs[warp * e_pad + 128 * c + 4 * lane + i] = acc[4 * c + i];
    __syncthreads();
    if (warp != 0) return;
    float big = sink ? sink[h] : -INFINITY;
    for (int w = 0; w < n_warps; ++w) big = fmaxf(big, ms[w]);              // finite: warp 0 holds the first visible key
    float total = sink ? expf(sink[h] - big) : 0.f;
#pragma unroll
    for (int c = 0; c < 4 * E_CHUNKS; ++c) acc[c] = 0.f;
    for (int w = 0; w < n_warps; ++w) {
        const float f = ms[w] == -INFINITY ? 0.f : expf(ms[w] - big);
        total += ms[n_warps + w] * f;
#pragma unroll
        for (int c = 0; c < E_CHUNKS; ++c)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[4 * c + i] = fmaf(accs[w * e_pad + 128 * c + 4 * lane + i], f, acc[4 * c + i]);
    }
    const float inv = 1.0f / total;
#pragma unroll
    for (int c = 0; c < E_CHUNKS; ++c)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int x = 128 * c + 4 * lane + i;
            if (x < e) st(out + ((int64_t)t * H + h) * e + x, acc[4 * c + i] * inv);
        }
}

// ---------------------------------------------------------------------------
// The form for steps of few tokens (a decode step): one block per (token, key/value head); its
// warps share the visible keys, 32 at a time, and every key and value row is read ONCE, by a whole
// warp (a lane holds the elements 4 l .. 4 l + 3 of every 128), for up to RH query heads of the
// group together: the lanes' partial products are added by the butterfly, lane j keeps key j's
// score of each head, the running maxima and sums follow per head, and every lane adds the weighted
// value rows into its own elements of each head's result.  The warps' partial results are folded
// in warp order (warp r folds head r); a sink joins there.  Groups of more than RH heads take
// several passes over the keys.
template <typename T, int RH>
__global__ void __launch_bounds__(256)
attn_masked_group_kernel(const T* __restrict__ q, const T* __restrict__ kv, T* __restrict__ out,
                         const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                         const int* __restrict__ page_table, int table_width, int H, int G, int d, int e,
                         float scale, int mask, int mask_size, const float* __restrict__ sink, int heads_per_block) {
    extern __shared__ float smem[];
    pdl_trigger();
    pdl_wait();
    q = fresh(q);
    kv = fresh(kv);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = blockDim.x >> 5;
    // the block's query heads h0 .. h0 + R - 1 lie in one group (heads_per_block divides the group's size)
    const int t = blockIdx.y, R = heads_per_block, h0 = blockIdx.x * heads_per_block, g = h0 / (H / G);
    const int pos = positions[t];
    const int* table = page_table + (int64_t)seq_of_token[t] * table_width;
    constexpr int e_pad = 128 * E_CHUNKS;
    float* ms = smem;                               // [warps][RH] maxima, then [warps][RH] sums
    float* accs = ms + 2 * n_warps * RH;            // [warps][RH][e_pad]
    const int64_t page_elems = (int64_t)G * kPage * (d + e);
    const int64_t v_off = (int64_t)G * kPage * d;
    const bool aligned = (((uintptr_t)kv) & 15) == 0 && (page_elems * sizeof(T)) % 16 == 0 && (v_off * sizeof(T)) % 16 == 0;
    const bool k_vec = d % 4 == 0 && aligned, v_vec = e % 4 == 0 && aligned;
    const int lo = first_visible(pos, mask, mask_size);
    for (int r0 = 0; r0 < R; r0 += RH) {
        // this pass's query rows, the lane's elements of each
        float qr[RH][4 * E_CHUNKS];
#pragma unroll
        for (int r = 0; r < RH; ++r)
#pragma unroll
            for (int c = 0; c < E_CHUNKS; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int x = 128 * c + 4 * lane + i;
                    qr[r][4 * c + i] = (r0 + r < R && x < d) ? ld(q + ((int64_t)t * H + h0 + r0 + r) * d + x) : 0.f;
                }
        float m[RH], l[RH], acc[RH][4 * E_CHUNKS];
#pragma unroll
        for (int r = 0; r < RH; ++r) {
            m[r] = -INFINITY;
            l[r] = 0.f;
#pragma unroll
            for (int c = 0; c < 4 * E_CHUNKS; ++c) acc[r][c] = 0.f;
        }
        for (int j0 = lo + 32 * warp; j0 <= pos; j0 += 32 * n_warps) {
            const int first_page = j0 / kPage;
            const int64_t page_a = table[first_page] * page_elems;
            const int64_t page_b = (first_page + 1) * kPage <= min(pos, j0 + 31) ? table[first_page + 1] * page_elems : page_a;
            const int n_keys = min(32, pos - j0 + 1);
            float sc[RH];
#pragma unroll
            for (int r = 0; r < RH; ++r) sc[r] = -INFINITY;
            auto score = [&](int jj) {
                const int key = j0 + jj;
                const T* kp = kv + (key / kPage == first_page ? page_a : page_b) + ((int64_t)g * kPage + (key % kPage)) * d;
                float kk[4 * E_CHUNKS];
#pragma unroll
                for (int c = 0; c < E_CHUNKS; ++c) {
                    const int x = 128 * c + 4 * lane;
                    if (k_vec) {
                        if (x < d) load4(kp + x, kk + 4 * c);
                        else kk[4 * c] = kk[4 * c + 1] = kk[4 * c + 2] = kk[4 * c + 3] = 0.f;
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) kk[4 * c + i] = x + i < d ? ld(kp + x + i) : 0.f;
                    }
                }
#pragma unroll
                for (int r = 0; r < RH; ++r) {
                    float part = 0.f;
#pragma unroll
                    for (int c = 0; c < 4 * E_CHUNKS; ++c) part = fmaf(qr[r][c], kk[c], part);
                    part = warp_sum(part);
                    if (lane == jj) sc[r] = part * scale;
                }
            };
            if (n_keys == 32) {
#pragma unroll 8
                for (int jj = 0; jj < 32; ++jj) score(jj);
            } else {
                for (int jj = 0; jj < n_keys; ++jj) score(jj);
            }
            float p[RH];
#pragma unroll
            for (int r = 0; r < RH; ++r) {
                const float m_new = fmaxf(m[r], warp_max(sc[r]));      // finite: key j0 is visible
                const float corr = expf(m[r] - m_new);                 // (-inf at first: 0)
                p[r] = lane < n_keys ? expf(sc[r] - m_new) : 0.f;
                l[r] = l[r] * corr + warp_sum(p[r]);
                m[r] = m_new;
#pragma unroll
                for (int c = 0; c < 4 * E_CHUNKS; ++c) acc[r][c] *= corr;
            }
            auto add_value = [&](int jj) {
                const int key = j0 + jj;
                const T* vp = kv + (key / kPage == first_page ? page_a : page_b) + v_off + ((int64_t)g * kPage + (key % kPage)) * e;
                float vv[4 * E_CHUNKS];
#pragma unroll
                for (int c = 0; c < E_CHUNKS; ++c) {
                    const int x = 128 * c + 4 * lane;
                    if (v_vec) {
                        if (x < e) load4(vp + x, vv + 4 * c);
                        else vv[4 * c] = vv[4 * c + 1] = vv[4 * c + 2] = vv[4 * c + 3] = 0.f;
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i) vv[4 * c + i] = x + i < e ? ld(vp + x + i) : 0.f;
                    }
                }
#pragma unroll
                for (int r = 0; r < RH; ++r) {
                    const float pj = __shfl_sync(0xffffffffu, p[r], jj);
#pragma unroll
                    for (int c = 0; c < 4 * E_CHUNKS; ++c) acc[r][c] = fmaf(pj, vv[c], acc[r][c]);
                }
            };
            if (n_keys == 32) {
#pragma unroll 8
                for (int jj = 0; jj < 32; ++jj) add_value(jj);
            } else {
                for (int jj = 0; jj < n_keys; ++jj) add_value(jj);
            }
        }
        __syncthreads();                                   // (the pass before is folded)
#pragma unroll
        for (int r = 0; r < RH; ++r) {
            if (lane == 0) {
                ms[warp * RH + r] = m[r];
                ms[(n_warps + warp) * RH + r] = l[r];
            }
#pragma unroll
            for (int c = 0; c < E_CHUNKS; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) accs[((int64_t)warp * RH + r) * e_pad + 128 * c + 4 * lane + i] = acc[r][4 * c + i];
        }
        __syncthreads();
        for (int r = warp; r < RH && r0 + r < R; r += n_warps) {
            const int h = h0 + r0 + r;
            float big = sink ? sink[h] : -INFINITY;
            for (int w = 0; w < n_warps; ++w) big = fmaxf(big, ms[w * RH + r]);     // finite: warp 0 holds the first visible key
            float total = sink ? expf(sink[h] - big) : 0.f;
            float o[4 * E_CHUNKS];
#pragma unroll
            for (int c = 0; c < 4 * E_CHUNKS; ++c) o[c] = 0.f;
            for (int w = 0; w < n_warps; ++w) {
                const float mw = ms[w * RH + r];
                const float f = mw == -INFINITY ? 0.f : expf(mw - big);
                total += ms[(n_warps + w) * RH + r] * f;
#pragma unroll
                for (int c = 0; c < E_CHUNKS; ++c)
#pragma unroll
                    for (int i = 0; i < 4; ++i) o[4 * c + i] = fmaf(accs[((int64_t)w * RH + r) * e_pad + 128 * c + 4 * lane + i], f, o[4 * c + i]);
            }
            const float inv = 1.0f / total;
#pragma unroll
            for (int c = 0; c < E_CHUNKS; ++c)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int x = 128 * c + 4 * lane + i;
                    if (x < e) st(out + ((int64_t)t * H + h) * e + x, o[4 * c + i] * inv);
                }
        }
    }
}

template <typename T>
int qkv_finish(const float* parts, int splits, int n, const float* bias, int H, int G, int d, int e, const float* q_w,
               int q_span, const float* k_w, int k_span, float eps, const float* cos_t, const float* sin_t, int rot_dims,
               int pairing, int maps, float* v_keep, int v_mode, const float* lambda, void* q_out, void* kv, const int* page_table,
               int table_width, const int* seq_of_token, const int* positions, int write_kv, int cols, int flags, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0, "qkv_finish: bad head counts or sizes");
    WICK_REQUIRE(!(flags & FINISH_KEYS_ARE_VALUES) || (d == e && v_mode == 0), "qkv_finish: keys that are values have the values' size and are not blended");
    WICK_REQUIRE(cols >= H * d + G * d + ((flags & FINISH_KEYS_ARE_VALUES) ? 0 : G * e), "qkv_finish: rows of %d numbers are too short", cols);
    WICK_REQUIRE(maps >= 1 && d % maps == 0, "qkv_finish: a head of %d numbers is not %d vectors", d, maps);
    WICK_REQUIRE(splits >= 1, "qkv_finish: partial sums are needed");
    const int Wq = H * d, Wk = G * d;
    if (q_w || q_span) WICK_REQUIRE(q_span > 0 && Wq % q_span == 0, "qkv_finish: a q norm span of %d does not divide %d", q_span, Wq);
    if (k_w || k_span) WICK_REQUIRE(k_span > 0 && Wk % k_span == 0, "qkv_finish: a k norm span of %d does not divide %d", k_span, Wk);
    WICK_REQUIRE(rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= d / maps, "qkv_finish: %d rotated dims of %d", rot_dims, d / maps);
    WICK_REQUIRE((cos_t == nullptr) == (sin_t == nullptr), "qkv_finish: the two angle tables come together");
    WICK_REQUIRE((q_span ? Wq / q_span : 0) + (k_span ? Wk / k_span : 0) <= MAX_SPANS, "qkv_finish: too many norm spans");
    WICK_REQUIRE(v_mode == 0 || v_keep, "qkv_finish: the kept values are missing");
    WICK_REQUIRE(v_mode != 2 || lambda, "qkv_finish: the blend factor is missing");
    if (n == 0) return 0;
    const size_t smem = (size_t)(Wq + Wk + G * e) * sizeof(float);
    WICK_REQUIRE(smem <= 200 * 1024, "qkv_finish: a row of %d numbers is beyond one block's shared memory", Wq + Wk + G * e);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        WICK_CUDA(cudaFuncSetAttribute(qkv_finish_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    WICK_CUDA(launch(qkv_finish_kernel<T>, dim3(n), dim3(256), smem, s, parts, splits, (int64_t)n * cols, bias, H, G,
                     d, e, q_w, q_span, k_w, k_span, eps, cos_t, sin_t, rot_dims, pairing, maps, v_keep, v_mode, lambda, (T*)q_out,
                     (T*)kv, page_table, table_width, seq_of_token, positions, write_kv, cols, flags));
    return check_launch("qkv_finish");
}

template <typename T>
int attn_masked(const void* q, const void* kv, void* out, const int* seq_of_token, const int* positions,
                const int* page_table, int table_width, int n, int H, int G, int d, int e, float scale, int mask,
                int mask_size, const float* sink, cudaStream_t s) {
    WICK_REQUIRE(H > 0 && G > 0 && H % G == 0 && d > 0 && e > 0, "attn_masked: bad head counts or sizes");
    WICK_REQUIRE(e <= 128 * E_CHUNKS, "attn_masked: a value size of %d is beyond %d", e, 128 * E_CHUNKS);
    WICK_REQUIRE(mask == MASK_CAUSAL || mask_size > 0, "attn_masked: the mask needs a positive size");
    if (n == 0) return 0;
    if ((int64_t)n * H <= 8192 && d <= 128 * E_CHUNKS && n <= 65535) {
        // few tokens: a block per (token, key/value head), rows read once for the group's query heads
        // With few blocks the group's heads are spread over several blocks (each reads the rows again, from the L2 cache).
        int hpb = H / G;
        const int warps = 8;
        while (hpb % 2 == 0 && (int64_t)(H / hpb) * n < 148) hpb /= 2;
        if (hpb > 1 && (int64_t)(H / hpb) * n < 148) hpb = 1;
        const int rh = hpb >= 4 ? 4 : (hpb >= 2 ? 2 : 1);
        const size_t smem_g = (size_t)(2 * warps * rh + warps * rh * 128 * E_CHUNKS) * sizeof(float);
        const dim3 grid(H / hpb, n), block(warps * 32);
#define WICK_GROUP(RH)                                                                                                          \
        WICK_CUDA(launch(attn_masked_group_kernel<T, RH>, grid, block, smem_g, s, (const T*)q, (const T*)kv, (T*)out, seq_of_token, \
                         positions, page_table, table_width, H, G, d, e, scale, mask, mask_size, sink, hpb))
        if (rh == 4) WICK_GROUP(4);
        else if (rh == 2) WICK_GROUP(2);
        else WICK_GROUP(1);
#undef WICK_GROUP
        return check_launch("attn_masked");
    }
    const int warps = 1;
    const size_t smem = (size_t)(((d + 3) & ~3) + 2 * warps + warps * 128 * E_CHUNKS) * sizeof(float);
    WICK_REQUIRE(smem <= 48 * 1024, "attn_masked: a head size of %d is beyond one block's shared memory", d);
    WICK_CUDA(launch(attn_masked_kernel<T>, dim3((unsigned)((int64_t)n * H)), dim3(warps * 32), smem, s, (const T*)q,
                     (const T*)kv, (T*)out, seq_of_token, positions, page_table, table_width, n, H, G, d, e, scale, mask,
                     mask_size, sink));
    return check_launch("attn_masked");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

#define WICK_QKV_FINISH(NAME, T)                                                                                              \
    WICK_API int NAME(const float* parts, int splits, int n, const float* bias, int H, int G, int d, int e, const float* q_w,    \
                      int q_span, const float* k_w, int k_span, float eps, const float* cos_t, const float* sin_t,               \
                      int rot_dims, int pairing, int maps, float* v_keep, int v_mode, const float* lambda, void* q_out, void* kv, \
                      const int* page_table, int table_width, const int* seq_of_token, const int* positions, int write_kv,       \
                      int cols, int flags, void* s) {                                                                            \
        return qkv_finish<T>(parts, splits, n, bias, H, G, d, e, q_w, q_span, k_w, k_span, eps, cos_t, sin_t, rot_dims, pairing,  \
                             maps, v_keep, v_mode, lambda, q_out, kv, page_table, table_width, seq_of_token, positions, write_kv,      \
                             cols, flags, (cudaStream_t)s);                                                                      \
    }
WICK_QKV_FINISH(wick_qkv_finish_bf16, bf16)
WICK_QKV_FINISH(wick_qkv_finish_f32, float)

#define WICK_ATTN_MASKED(NAME, T)                                                                                             \
    WICK_API int NAME(const void* q, const void* kv, void* out, const int* seq_of_token, const int* positions,                 \
                      const int* page_table, int table_width, int n, int H, int G, int d, int e, float scale, int mask,        \
                      int mask_size, const float* sink, void* s) {                                                             \
        return attn_masked<T>(q, kv, out, seq_of_token, positions, page_table, table_width, n, H, G, d, e, scale, mask,        \
                              mask_size, sink, (cudaStream_t)s);                                                               \
    }
WICK_ATTN_MASKED(wick_attn_masked_bf16, bf16)
WICK_ATTN_MASKED(wick_attn_masked_f32, float)
