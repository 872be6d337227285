// Row-wise kernels of models whose residual stream is float32 whatever the engine's dtype: the
// embedding gather into float32, the Dynamic Tanh norm with the residual add fused in front of it, and
// the element-wise activations of a dense feed-forward.
//
// The residual sum is the only place where a layer's result meets all earlier ones; kept in float32,
// a delta that the products computed in bfloat16 is added without a second rounding of the sum.
#include "common.cuh"

namespace dfi {

// out[row] = float(table[ids[row]]) * scale
template <typename T>
__global__ void embedding_float_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ out,
                                       int hidden, int vocab, float scale) {
    pdl_launch_next();
    pdl_wait();
    const int row = blockIdx.x;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* src = table + (size_t)id * hidden;
    float* dst = out + (size_t)row * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_float(src[i]) * scale;
}

// Dynamic Tanh: out = tanh(alpha * x) * w + b, element by element (no mean, no variance), where x is
// the float32 residual row after `delta` (the engine's dtype, or null) has been added to it in place.
// alpha is one float in device memory.  VEC: four elements a thread and step (dim % 4 == 0, aligned).
template <typename T, bool VEC>
__global__ void dynamic_tanh_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                    const float* __restrict__ alpha_p, const float* __restrict__ w,
                                    const float* __restrict__ b, T* __restrict__ out, int dim) {
    pdl_launch_next();
    const float alpha = alpha_p[0];
    pdl_wait();
    float* x = residual + (size_t)blockIdx.x * dim;
    const T* d = delta != nullptr ? delta + (size_t)blockIdx.x * dim : nullptr;
    T* o = out + (size_t)blockIdx.x * dim;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(x + i);
            if (d != nullptr) {
                v.x += to_float(d[i]); v.y += to_float(d[i + 1]); v.z += to_float(d[i + 2]); v.w += to_float(d[i + 3]);
                *reinterpret_cast<float4*>(x + i) = v;
            }
            const float4 wv = *reinterpret_cast<const float4*>(w + i), bv = *reinterpret_cast<const float4*>(b + i);
            o[i] = from_float<T>(tanhf(alpha * v.x) * wv.x + bv.x);
            o[i + 1] = from_float<T>(tanhf(alpha * v.y) * wv.y + bv.y);
            o[i + 2] = from_float<T>(tanhf(alpha * v.z) * wv.z + bv.z);
            o[i + 3] = from_float<T>(tanhf(alpha * v.w) * wv.w + bv.w);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            float v = x[i];
            if (d != nullptr) {
                v += to_float(d[i]);
                x[i] = v;
            }
            o[i] = from_float<T>(tanhf(alpha * v) * w[i] + b[i]);
        }
    }
}

// residual (float32) += delta (engine dtype): the residual sum where no norm follows it.
template <typename T>
__global__ void add_to_float_kernel(float* __restrict__ residual, const T* __restrict__ delta, long long n) {
    pdl_launch_next();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        residual[i] += to_float(delta[i]);
}

// Activations of a dense feed-forward, in place on its inner rows (`activate` of common.cuh).
template <typename T>
__global__ void activation_kernel(T* __restrict__ x, long long n, int kind) {
    pdl_launch_next();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        x[i] = from_float<T>(activate(to_float(x[i]), kind));
}

// out = a * sa + b * sb, element by element (the sum of two mixers that read the same rows)
template <typename T>
__global__ void weighted_sum_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long long n,
                                    float sa, float sb) {
    pdl_launch_next();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        out[i] = from_float<T>(to_float(a[i]) * sa + to_float(b[i]) * sb);
}

static inline int blocks_for(long long n) {
    const long long want = (n + 255) / 256;
    return (int)(want < 4096 ? want : 4096);
}

}  // namespace dfi

using namespace dfi;

DFI_EXPORT int dfi_embedding_float(const void* table, const int* ids, float* out, int rows, int hidden, int vocab,
                                   float scale, int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (hidden <= 0 || vocab <= 0) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch(embedding_float_kernel<float>, rows, 128, 0, st, (const float*)table, ids, out, hidden, vocab, scale);
    else if (dtype == DFI_DTYPE_BF16) launch(embedding_float_kernel<bf16>, rows, 128, 0, st, (const bf16*)table, ids, out, hidden, vocab, scale);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// residual [rows, dim] float32 (+= delta in place if delta is given), out [rows, dim] in `dtype`.
DFI_EXPORT int dfi_dynamic_tanh(float* residual, const void* delta, const float* alpha, const float* weight,
                                const float* bias, void* out, int rows, int dim, int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (dim <= 0) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = dim % 4 == 0 && aligned16(residual) && aligned16(weight) && aligned16(bias);
    int threads = 32;
    while (threads < 256 && threads * (vec ? 4 : 1) < dim) threads <<= 1;
    if (dtype == DFI_DTYPE_F32) {
        if (vec) launch(dynamic_tanh_kernel<float, true>, rows, threads, 0, st, residual, (const float*)delta, alpha, weight, bias, (float*)out, dim);
        else launch(dynamic_tanh_kernel<float, false>, rows, threads, 0, st, residual, (const float*)delta, alpha, weight, bias, (float*)out, dim);
    } else if (dtype == DFI_DTYPE_BF16) {
        if (vec) launch(dynamic_tanh_kernel<bf16, true>, rows, threads, 0, st, residual, (const bf16*)delta, alpha, weight, bias, (bf16*)out, dim);
        else launch(dynamic_tanh_kernel<bf16, false>, rows, threads, 0, st, residual, (const bf16*)delta, alpha, weight, bias, (bf16*)out, dim);
    } else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_add_to_float(float* residual, const void* delta, long long n, int dtype, void* stream) {
    if (n <= 0) return DFI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch(add_to_float_kernel<float>, blocks_for(n), 256, 0, st, residual, (const float*)delta, n);
    else if (dtype == DFI_DTYPE_BF16) launch(add_to_float_kernel<bf16>, blocks_for(n), 256, 0, st, residual, (const bf16*)delta, n);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_activation(void* x, long long n, int kind, int dtype, void* stream) {
    if (n <= 0) return DFI_OK;
    if (kind < 0 || kind > 4) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch(activation_kernel<float>, blocks_for(n), 256, 0, st, (float*)x, n, kind);
    else if (dtype == DFI_DTYPE_BF16) launch(activation_kernel<bf16>, blocks_for(n), 256, 0, st, (bf16*)x, n, kind);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_weighted_sum(const void* a, const void* b, void* out, long long n, float sa, float sb, int dtype,
                                void* stream) {
    if (n <= 0) return DFI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch(weighted_sum_kernel<float>, blocks_for(n), 256, 0, st, (const float*)a, (const float*)b, (float*)out, n, sa, sb);
    else if (dtype == DFI_DTYPE_BF16) launch(weighted_sum_kernel<bf16>, blocks_for(n), 256, 0, st, (const bf16*)a, (const bf16*)b, (bf16*)out, n, sa, sb);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
