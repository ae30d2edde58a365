// Row-wise kernels of layers that normalise AFTER the residual sum, and two
// element-wise steps: the squared ReLU of a plain feed-forward and the soft cap of
// logits.  All arithmetic is float32; T is the storage type of activations.
//
//   post-norm :  y = rms(alpha * x + d_0 + d_1 + ...) * g,   rms(v) = v / sqrt(mean(v^2) + eps)
//                y replaces x (float32, the residual stream) and is also written
//                in the activation type for the next matrix product.
//   relu^2    :  a <- max(a, 0)^2
//   soft cap  :  z <- c * tanh(z / c)
//   stream    :  x <- x + f(d_0 + d_1 + ...), f the identity, a factor per element, or
//                rms(.) * g (times a factor per element), optionally followed by the
//                norm y = tanh(a x) * w + b or by a copy of x in the activation type
//   gate rows :  g = gelu_tanh(z) * e, e a slice of the token's row in a table
#include "common.cuh"

namespace wick {

// x4 += the partial sums d_s[j .. j + 3], s in index order; the loads of four partial sums are issued together
// (a chain of dependent trips to the L2 cache is what a step of few tokens would otherwise wait for).
__device__ __forceinline__ void add_partials4(float4& v, const float* __restrict__ delta, int splits, int64_t split_stride, int64_t at) {
    for (int s0 = 0; s0 < splits; s0 += 4) {
        float4 d[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            d[u] = s0 + u < splits ? *reinterpret_cast<const float4*>(delta + (s0 + u) * split_stride + at) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            v.x += d[u].x; v.y += d[u].y; v.z += d[u].z; v.w += d[u].w;
        }
    }
}

// One block per row; the row waits in shared memory between the two passes.  First pass:
// v = alpha x + the partial sums (index order) and the sum of its squares (a thread's elements in
// index order, then the block's sum in thread order); second pass: y = v * scale * w to x and out.
// The block's size depends on the width alone, so a row's bits do not depend on the batch.
template <typename TOut>
__global__ void __launch_bounds__(1024)
scaled_add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int splits, int64_t split_stride,
                          float alpha, const float* __restrict__ w, float eps, TOut* __restrict__ out, int n, int width) {
    extern __shared__ float smem[];
    float* row = smem;
    float* red = smem + ((width + 3) & ~3);
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    delta = fresh(delta);
    const int r = blockIdx.x;
    float* xr = x + (int64_t)r * width;
    float ss = 0.f;
    const bool vec = (width & 3) == 0 && (split_stride & 3) == 0;
    if (vec) {
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(xr + j);
            v.x *= alpha; v.y *= alpha; v.z *= alpha; v.w *= alpha;
            add_partials4(v, delta, splits, split_stride, (int64_t)r * width + j);
            *reinterpret_cast<float4*>(row + j) = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            float v = alpha * xr[j];
            for (int s = 0; s < splits; ++s) v += delta[s * split_stride + (int64_t)r * width + j];
            row[j] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)width + eps);
    TOut* o = out ? out + (int64_t)r * width : nullptr;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float y = (row[j] * scale) * w[j];
        xr[j] = y;
        if (o) st(o + j, y);
    }
}

// Eight elements a thread where the array allows 16-byte accesses (vec), else one.
template <typename T>
__global__ void relu_squared_kernel(T* __restrict__ a, int64_t n, int vec) {
    pdl_trigger();
    pdl_wait();
    a = fresh(a);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec) {
        constexpr int VN = Vec16<T>::N;
        if (i * VN >= n) return;
        Vec16<T> v;
        v.load(a + i * VN);
#pragma unroll
        for (int k = 0; k < VN; ++k) {
            const float r = fmaxf(v.v[k], 0.f);
            v.v[k] = r * r;
        }
        v.store(a + i * VN);
        return;
    }
    if (i >= n) return;
    const float v = fmaxf(ld(a + i), 0.f);
    st(a + i, v * v);
}

__global__ void soft_cap_kernel(float* __restrict__ z, int64_t n, float cap) {
    pdl_trigger();
    pdl_wait();
    z = fresh(z);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    z[i] = cap * tanhf(z[i] / cap);
}

// float32 -> activation type (the residual stream as the input of a matrix product).
template <typename T>
__global__ void to_activation_kernel(const float* __restrict__ x, T* __restrict__ out, int64_t n) {
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) st(out + i, x[i]);
}

// One block per output row i; source row r = rows ? rows[i] : i.
//   v = x[r] + f(sum of the partial sums, in index order), where f divides by the root mean square and multiplies
//   by rms_w (if given), then multiplies by scale (if given);  v goes back to x[r] unless rows are selected (a row
//   may be named twice, and nobody reads x afterwards then);  out[i] = tanh(alpha v) * w + b if w and b are given,
//   v / sqrt(mean(v^2) + out_eps) * w if w alone is given, else v.
// With rms_w the sums wait in shared memory between the pass that squares them and the pass that uses them, and so does
// v for the norm by its root mean square; otherwise one pass does everything, four neighbours a thread where the width
// allows.
template <typename TOut>
__global__ void __launch_bounds__(1024)
stream_update_kernel(float* __restrict__ x, const float* __restrict__ delta, int splits, int64_t split_stride,
                     const float* __restrict__ scale, const float* __restrict__ rms_w, float rms_eps,
                     const float* __restrict__ alpha, const float* __restrict__ w, const float* __restrict__ b, float out_eps,
                     const int* __restrict__ rows, TOut* __restrict__ out, int width) {
    extern __shared__ float smem[];
    float* row = smem;
    float* red = smem + ((width + 3) & ~3);
    pdl_trigger();
    const float a = alpha ? *alpha : 0.f;              // (a weight: no kernel writes it)
    pdl_wait();
    x = fresh(x);
    delta = fresh(delta);
    const int i = blockIdx.x;
    const int64_t r = rows ? rows[i] : i;
    float* xr = x + r * width;
    TOut* o = out ? out + (int64_t)i * width : nullptr;
    const bool vec = (width & 3) == 0 && (split_stride & 3) == 0;
    const bool out_rms = o && w && !b;                 // (the new row waits in shared memory for its mean square)
    float f = 1.f, ss_out = 0.f;
    if (delta && rms_w) {
        float ss = 0.f;
        if (vec) {
            for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                add_partials4(v, delta, splits, split_stride, r * width + j);
                *reinterpret_cast<float4*>(row + j) = v;
                ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
            }
        } else {
            for (int j = threadIdx.x; j < width; j += blockDim.x) {
                float v = 0.f;
                for (int s = 0; s < splits; ++s) v += delta[s * split_stride + r * width + j];
                row[j] = v;
                ss = fmaf(v, v, ss);
            }
        }
        ss = block_sum(ss, red);
        f = 1.0f / sqrtf(ss / (float)width + rms_eps);
    }
    auto finish = [&](int j, float xv, float d) -> float {
        if (delta) {
            if (rms_w) d = (d * f) * rms_w[j];
            if (scale) d *= scale[j];
            xv += d;
        }
        return xv;
    };
    if (vec) {
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            const float4 xv = *reinterpret_cast<const float4*>(xr + j);
            float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
            if (delta) {
                if (rms_w) d = *reinterpret_cast<const float4*>(row + j);
                else add_partials4(d, delta, splits, split_stride, r * width + j);
            }
            float4 v;
            v.x = finish(j, xv.x, d.x); v.y = finish(j + 1, xv.y, d.y); v.z = finish(j + 2, xv.z, d.z); v.w = finish(j + 3, xv.w, d.w);
            if (delta && !rows) *reinterpret_cast<float4*>(xr + j) = v;
            if (out_rms) {
                *reinterpret_cast<float4*>(row + j) = v;
                ss_out = fmaf(v.x, v.x, ss_out); ss_out = fmaf(v.y, v.y, ss_out); ss_out = fmaf(v.z, v.z, ss_out); ss_out = fmaf(v.w, v.w, ss_out);
            } else if (o) {
                if (w) {
                    st(o + j, tanhf(a * v.x) * w[j] + b[j]);
                    st(o + j + 1, tanhf(a * v.y) * w[j + 1] + b[j + 1]);
                    st(o + j + 2, tanhf(a * v.z) * w[j + 2] + b[j + 2]);
                    st(o + j + 3, tanhf(a * v.w) * w[j + 3] + b[j + 3]);
                } else {
                    st(o + j, v.x); st(o + j + 1, v.y); st(o + j + 2, v.z); st(o + j + 3, v.w);
                }
            }
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            float d = 0.f;
            if (delta) {
                if (rms_w) d = row[j];
                else for (int s = 0; s < splits; ++s) d += delta[s * split_stride + r * width + j];
            }
            const float v = finish(j, xr[j], d);
            if (delta && !rows) xr[j] = v;
            if (out_rms) {
                row[j] = v;
                ss_out = fmaf(v, v, ss_out);
            } else if (o) {
                st(o + j, w ? tanhf(a * v) * w[j] + b[j] : v);
            }
        }
    }
    if (out_rms) {                                     // (a thread reads back the elements it wrote itself)
        const float g = 1.0f / sqrtf(block_sum(ss_out, red) / (float)width + out_eps);
        if (vec) {
            for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
                const float4 v = *reinterpret_cast<const float4*>(row + j);
                st(o + j, (v.x * g) * w[j]); st(o + j + 1, (v.y * g) * w[j + 1]);
                st(o + j + 2, (v.z * g) * w[j + 2]); st(o + j + 3, (v.w * g) * w[j + 3]);
            }
        } else {
            for (int j = threadIdx.x; j < width; j += blockDim.x) st(o + j, (row[j] * g) * w[j]);
        }
    }
}

// out[t, j] = gelu_tanh(z[t, j]) * table[tokens[t], offset + j]; gelu_tanh(z) = z/2 (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).
template <typename T>
__global__ void gelu_gate_rows_kernel(const float* __restrict__ z, const T* __restrict__ table, const int* __restrict__ tokens,
                                      T* __restrict__ out, int64_t n, int dim, int64_t row_width, int offset) {
    pdl_trigger();
    pdl_wait();
    z = fresh(z);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * dim) return;
    const int64_t t = i / dim;
    const int j = (int)(i - t * dim);
    const float v = z[i];
    const float g = 0.5f * v * (1.0f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    st(out + i, g * ld(table + (int64_t)tokens[t] * row_width + offset + j));
}


// y[t, j] <- y[t, j] * sigmoid(g[t, j]), g the sum of the partial sums at column first_col + j of a token's row of `cols`
// numbers (an output gate that came out of the same product as the projections it gates).  float32 arithmetic.
template <typename T>
__global__ void gate_rows_kernel(T* __restrict__ y, const float* __restrict__ parts, int splits, int64_t split_stride, int64_t n,
                                 int width, int cols, int first_col) {
    pdl_trigger();
    pdl_wait();
    y = fresh(y);
    parts = fresh(parts);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * width) return;
    const int64_t t = i / width;
    const int j = (int)(i - t * width);
    float g = 0.f;
    for (int s = 0; s < splits; ++s) g += parts[s * split_stride + t * cols + first_col + j];
    st(y + i, ld(y + i) / (1.0f + expf(-g)));
}

// ---- an embedding with a factor and the positions' sinusoids ------------------------------------------------------
// out[t][j] = table[token_t][j] * scale + s(p_t, j): s = sin(p f_i) for j = 2 i and cos(p f_i) for j = 2 i + 1, the angle the
// float32 product of the position and the frequency f_i (float32 [ceil(width / 2)]); no sinusoid where `freq` is null.
// One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
embed_sinusoid_kernel(const T* __restrict__ table, const int* __restrict__ tokens, const int* __restrict__ positions,
                      const float* __restrict__ freq, float scale, float* __restrict__ out, int width) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const T* row = table + (int64_t)tokens[t] * width;
    const float p = (float)positions[t];
    for (int i = threadIdx.x; 2 * i < width; i += blockDim.x) {
        float sn = 0.f, cs = 0.f;
        if (freq) sincosf(p * freq[i], &sn, &cs);
        out[(int64_t)t * width + 2 * i] = fmaf(ld(row + 2 * i), scale, sn);
        if (2 * i + 1 < width) out[(int64_t)t * width + 2 * i + 1] = fmaf(ld(row + 2 * i + 1), scale, cs);
    }
}

// x[t][j] += (x0 ? x0[t][j] : 0) + (vec ? vec[j] : 0): what a pass over a range of layers begins with.
__global__ void stream_offset_kernel(float* __restrict__ x, const float* __restrict__ x0, const float* __restrict__ vec, int64_t n,
                                     int width) {
    pdl_trigger();
    pdl_wait();
    x = fresh(x);
    x0 = fresh(x0);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    if (x0) v += x0[i];
    if (vec) v += vec[i % width];
    x[i] = v;
}

// out = f_0 sum(a_0) + f_1 sum(a_1) + ...: up to four terms of partial sums (each added in index order), the terms
// in the order given.
struct SumTerms {
    const float* a[4];
    int splits[4];
    float f[4];
};
__global__ void weighted_sum_kernel(SumTerms terms, float* __restrict__ out, int64_t n) {
    pdl_trigger();
    pdl_wait();
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        if (terms.a[k] == nullptr) continue;
        const float* a = fresh(terms.a[k]);
        float sum = 0.f;
        for (int s = 0; s < terms.splits[k]; ++s) sum += a[s * n + i];
        v = k == 0 ? terms.f[k] * sum : fmaf(terms.f[k], sum, v);
    }
    out[i] = v;
}

// out[t] = [a[t] | b[t]] in the activation type.
template <typename T>
__global__ void concat_activation_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int64_t n,
                                         int wa, int wb) {
    pdl_trigger();
    pdl_wait();
    a = fresh(a);
    b = fresh(b);
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n * (wa + wb)) return;
    const int64_t t = i / (wa + wb);
    const int j = (int)(i - t * (wa + wb));
    st(out + i, j < wa ? a[t * wa + j] : b[t * wb + (j - wa)]);
}

template <typename TOut>
int stream_update(float* x, const float* delta, int splits, const float* scale, const float* rms_w, float rms_eps,
                  const float* alpha, const float* w, const float* b, float out_eps, const int* rows, void* out, int n, int n_out,
                  int width, cudaStream_t s) {
    WICK_REQUIRE(width > 0 && n >= 0 && n_out >= 0 && splits >= 0, "stream_update: bad sizes");
    WICK_REQUIRE((b == nullptr) == (alpha == nullptr) && (w || !b), "stream_update: a tanh norm has three tensors, a norm by the root mean square one");
    WICK_REQUIRE(!w || out, "stream_update: a norm needs a place for its result");
    WICK_REQUIRE(delta || (!scale && !rms_w), "stream_update: nothing to scale or to norm");
    if (n_out == 0) return 0;
    const size_t smem = ((size_t)((width + 3) & ~3) + 40) * sizeof(float);
    WICK_REQUIRE(smem <= 200 * 1024, "stream_update: width %d is beyond one block's shared memory", width);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        WICK_CUDA(cudaFuncSetAttribute(stream_update_kernel<TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    const int threads = min(1024, max(64, ((width + 3) / 4 + 31) / 32 * 32));
    WICK_CUDA(launch(stream_update_kernel<TOut>, dim3(n_out), dim3(threads), smem, s, x, delta, splits, (int64_t)n * width, scale,
                     rms_w, rms_eps, alpha, w, b, out_eps, rows, (TOut*)out, width));
    return check_launch("stream_update");
}

template <typename TOut>
int scaled_add_rmsnorm(float* x, const float* delta, int splits, float alpha, const float* w, float eps, void* out, int n,
                       int width, cudaStream_t s) {
    WICK_REQUIRE(width > 0 && n >= 0 && splits >= 0, "scaled_add_rmsnorm: bad sizes");
    if (n == 0) return 0;
    const size_t smem = ((size_t)((width + 3) & ~3) + 40) * sizeof(float);
    WICK_REQUIRE(smem <= 200 * 1024, "scaled_add_rmsnorm: width %d is beyond one block's shared memory", width);
    static bool raised = false;
    if (smem > 48 * 1024 && !raised) {
        WICK_CUDA(cudaFuncSetAttribute(scaled_add_rmsnorm_kernel<TOut>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        raised = true;
    }
    const int threads = min(1024, max(64, ((width + 3) / 4 + 31) / 32 * 32));
    WICK_CUDA(launch(scaled_add_rmsnorm_kernel<TOut>, dim3(n), dim3(threads), smem, s, x, delta, splits, (int64_t)n * width, alpha,
                     w, eps, (TOut*)out, n, width));
    return check_launch("scaled_add_rmsnorm");
}

}  // namespace wick

using namespace wick;
typedef __nv_bfloat16 bf16;

// x: float32 [n, width], replaced by the normalised rows; delta: float32 [splits, n, width] or
// null; w: float32 [width] (the factor itself: an offset is added by the caller); out: [n, width]
// in the activation type or null.
WICK_API int wick_scaled_add_rmsnorm_bf16(float* x, const float* delta, int splits, float alpha, const float* w, float eps,
                                          void* out, int n, int width, void* s) {
    return scaled_add_rmsnorm<bf16>(x, delta, splits, alpha, w, eps, out, n, width, (cudaStream_t)s);
}
WICK_API int wick_scaled_add_rmsnorm_f32(float* x, const float* delta, int splits, float alpha, const float* w, float eps,
                                         void* out, int n, int width, void* s) {
    return scaled_add_rmsnorm<float>(x, delta, splits, alpha, w, eps, out, n, width, (cudaStream_t)s);
}

// x: float32 [n, width]; delta: float32 [splits, n, width] or null; scale, rms_w: float32 [width] or null; alpha [1], w, b
// [width]: the tanh norm's tensors or null, or w alone with out_eps: a norm by the root mean square; rows: int32 [n_out] or
// null (then n_out = n); out: [n_out, width] or null.
WICK_API int wick_stream_update_bf16(float* x, const float* delta, int splits, const float* scale, const float* rms_w,
                                     float rms_eps, const float* alpha, const float* w, const float* b, float out_eps,
                                     const int* rows, void* out, int n, int n_out, int width, void* s) {
    return stream_update<bf16>(x, delta, splits, scale, rms_w, rms_eps, alpha, w, b, out_eps, rows, out, n, n_out, width,
                          (cudaStream_t)s);
}
WICK_API int wick_stream_update_f32(float* x, const float* delta, int splits, const float* scale, const float* rms_w,
                                     float rms_eps, const float* alpha, const float* w, const float* b, float out_eps,
                                     const int* rows, void* out, int n, int n_out, int width, void* s) {
    return stream_update<float>(x, delta, splits, scale, rms_w, rms_eps, alpha, w, b, out_eps, rows, out, n, n_out, width,
                          (cudaStream_t)s);
}

WICK_API int wick_gelu_gate_rows_bf16(const float* z, const void* table, const int* tokens, void* out, int64_t n, int dim,
                                      int64_t row_width, int offset, void* s) {
    if (n == 0 || dim == 0) return 0;
    WICK_CUDA(launch(gelu_gate_rows_kernel<bf16>, dim3(ceil_div(n * dim, 256)), dim3(256), 0, (cudaStream_t)s, z, (const bf16*)table,
                     tokens, (bf16*)out, n, dim, row_width, offset));
    return check_launch("gelu_gate_rows");
}
WICK_API int wick_gelu_gate_rows_f32(const float* z, const void* table, const int* tokens, void* out, int64_t n, int dim,
                                     int64_t row_width, int offset, void* s) {
    if (n == 0 || dim == 0) return 0;
    WICK_CUDA(launch(gelu_gate_rows_kernel<float>, dim3(ceil_div(n * dim, 256)), dim3(256), 0, (cudaStream_t)s, z, (const float*)table,
                     tokens, (float*)out, n, dim, row_width, offset));
    return check_launch("gelu_gate_rows");
}

WICK_API int wick_relu_squared_bf16(void* a, int64_t n, void* s) {
    if (n == 0) return 0;
    const int vec = n % 8 == 0 && ((uintptr_t)a & 15) == 0;
    WICK_CUDA(launch(relu_squared_kernel<bf16>, dim3(ceil_div(vec ? n / 8 : n, 256)), dim3(256), 0, (cudaStream_t)s, (bf16*)a, n, vec));
    return check_launch("relu_squared");
}
WICK_API int wick_relu_squared_f32(void* a, int64_t n, void* s) {
    if (n == 0) return 0;
    const int vec = n % 4 == 0 && ((uintptr_t)a & 15) == 0;
    WICK_CUDA(launch(relu_squared_kernel<float>, dim3(ceil_div(vec ? n / 4 : n, 256)), dim3(256), 0, (cudaStream_t)s, (float*)a, n, vec));
    return check_launch("relu_squared");
}

WICK_API int wick_soft_cap(float* z, int64_t n, float cap, void* s) {
    WICK_REQUIRE(cap > 0.f, "soft_cap: the cap must be positive");
    if (n == 0) return 0;
    WICK_CUDA(launch(soft_cap_kernel, dim3(ceil_div(n, 256)), dim3(256), 0, (cudaStream_t)s, z, n, cap));
    return check_launch("soft_cap");
}

WICK_API int wick_to_activation_bf16(const float* x, void* out, int64_t n, void* s) {
    if (n == 0) return 0;
    WICK_CUDA(launch(to_activation_kernel<bf16>, dim3(ceil_div(n, 256)), dim3(256), 0, (cudaStream_t)s, x, (bf16*)out, n));
    return check_launch("to_activation");
}

// y: [n, width] in the activation type, gated in place; parts: float32 [splits, n, cols].
#define WICK_GATE_ROWS(NAME, T)                                                                                              \
    WICK_API int NAME(void* y, const float* parts, int splits, int n, int width, int cols, int first_col, void* s) {          \
        WICK_REQUIRE(splits >= 1 && first_col >= 0 && first_col + width <= cols, "gate_rows: bad columns");                  \
        if (n == 0 || width == 0) return 0;                                                                                  \
        WICK_CUDA(launch(gate_rows_kernel<T>, dim3(ceil_div((int64_t)n * width, 256)), dim3(256), 0, (cudaStream_t)s, (T*)y,  \
                         parts, splits, (int64_t)n * cols, (int64_t)n, width, cols, first_col));                              \
        return check_launch("gate_rows");                                                                                    \
    }
WICK_GATE_ROWS(wick_gate_rows_bf16, bf16)
WICK_GATE_ROWS(wick_gate_rows_f32, float)

// a_k: float32 [splits_k, n] or null; out: float32 [n].
WICK_API int wick_weighted_sum(const float* a0, int s0, float f0, const float* a1, int s1, float f1, const float* a2, int s2,
                               float f2, const float* a3, int s3, float f3, float* out, int64_t n, void* s) {
    WICK_REQUIRE(a0 != nullptr, "weighted_sum: the first term is missing");
    if (n == 0) return 0;
    SumTerms t = {{a0, a1, a2, a3}, {s0, s1, s2, s3}, {f0, f1, f2, f3}};
    WICK_CUDA(launch(weighted_sum_kernel, dim3(ceil_div(n, 256)), dim3(256), 0, (cudaStream_t)s, t, out, n));
    return check_launch("weighted_sum");
}

#define WICK_CONCAT_ACTIVATION(NAME, T)                                                                                      \
    WICK_API int NAME(const float* a, const float* b, void* out, int n, int wa, int wb, void* s) {                            \
        if (n == 0 || wa + wb == 0) return 0;                                                                                \
        WICK_CUDA(launch(concat_activation_kernel<T>, dim3(ceil_div((int64_t)n * (wa + wb), 256)), dim3(256), 0,              \
                         (cudaStream_t)s, a, b, (T*)out, (int64_t)n, wa, wb));                                                \
        return check_launch("concat_activation");                                                                            \
    }
WICK_CONCAT_ACTIVATION(wick_concat_activation_bf16, bf16)
WICK_CONCAT_ACTIVATION(wick_concat_activation_f32, float)

#define WICK_EMBED_SINUSOID(NAME, T)                                                                                         \
    WICK_API int NAME(const void* table, const int* tokens, const int* positions, const float* freq, float scale, float* out, \
                      int n, int width, void* s) {                                                                           \
        WICK_REQUIRE(n >= 0 && width > 0, "embed_sinusoid: bad sizes");                                                      \
        if (n == 0) return 0;                                                                                                \
        WICK_CUDA(launch(embed_sinusoid_kernel<T>, dim3(n), dim3(256), 0, (cudaStream_t)s, (const T*)table, tokens,          \
                         positions, freq, scale, out, width));                                                               \
        return check_launch("embed_sinusoid");                                                                               \
    }
WICK_EMBED_SINUSOID(wick_embed_sinusoid_bf16, bf16)
WICK_EMBED_SINUSOID(wick_embed_sinusoid_f32, float)

// x: float32 [n, width], changed in place; x0: float32 [n, width] or null; vec: float32 [width] or null.
WICK_API int wick_stream_offset(float* x, const float* x0, const float* vec, int n, int width, void* s) {
    const int64_t all = (int64_t)n * width;
    if (all == 0) return 0;
    WICK_CUDA(launch(stream_offset_kernel, dim3(ceil_div(all, 256)), dim3(256), 0, (cudaStream_t)s, x, x0, vec, all, width));
    return check_launch("stream_offset");
}
