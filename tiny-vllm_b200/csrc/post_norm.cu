// Layer norm behind the residual sum (post-norm), over a float32 residual stream.
//
//   s   = alpha * x + y          (x: the stream, float32 or of the storage type; y: a sublayer's
//                                 output, optional; the sum in float32)
//   out = (s - mean(s)) / sqrt(mean((s - mean)^2) + eps) * w
//
// `out` is written twice: as the new stream in float32, and rounded once to the storage type as
// the input of the next sublayer's products.  One block per row.  With `gather` only the named
// rows are produced (the last norm of a model, on the wanted rows).  The mean and the variance
// are two passes over the row held in shared memory; the order of additions depends on the width
// alone, so a row's result does not depend on the batch it is in.
#include "common.cuh"

template <typename S, typename A, typename T, typename W>
__global__ void post_layer_norm_kernel(const S* x, float alpha, const A* add, const W* __restrict__ weight,
                                       T* __restrict__ y, float* stream_out, const int* __restrict__ gather,
                                       int width, float eps) {
    extern __shared__ float row_values[];
    __shared__ float scratch[32];
    const int out_row = blockIdx.x;
    const int64_t in_row = gather ? gather[out_row] : out_row;
    const S* xr = x + in_row * width;
    const A* ar = add ? add + in_row * width : nullptr;
    float part = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = to_float<S>(xr[i]);
        if (alpha != 1.0f) v = ar ? __fmaf_rn(alpha, v, to_float<A>(ar[i])) : __fmul_rn(alpha, v);
        else if (ar) v = __fadd_rn(v, to_float<A>(ar[i]));
        row_values[i] = v;
        part = __fadd_rn(part, v);
    }
    const float mean = __fdiv_rn(block_sum(part, scratch), (float)width);
    part = 0.0f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float d = __fsub_rn(row_values[i], mean);
        part = __fmaf_rn(d, d, part);
    }
    const float variance = __fdiv_rn(block_sum(part, scratch), (float)width);
    const float inverse = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(variance, eps)));
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float o = __fmul_rn(__fmul_rn(__fsub_rn(row_values[i], mean), inverse), to_float<W>(weight[i]));
        if (stream_out) stream_out[(int64_t)out_row * width + i] = o;
        if (y) y[(int64_t)out_row * width + i] = from_float<T>(o);
    }
}

template <typename S, typename A, typename T, typename W>
static int launch_post_norm(const void* x, float alpha, const void* add, const void* weight, void* y,
                            float* stream_out, const int* gather, int rows, int width, float eps, cudaStream_t s) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TVB_BAD_ARGUMENT;
    auto kernel = post_layer_norm_kernel<S, A, T, W>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = width >= 2048 ? 512 : (width >= 512 ? 256 : (width >= 128 ? 128 : 32));
    kernel<<<rows, threads, smem, s>>>((const S*)x, alpha, (const A*)add, (const W*)weight, (T*)y, stream_out,
                                       gather, width, eps);
    return tvb_last_error();
}

// x_dtype: type of x; add_dtype: type of add; dtype: type of y; weight_dtype: type of the weight.
// In the float32 path everything is float32; in the bfloat16 path y is bfloat16 and each of x, add
// and the weight is bfloat16 or float32.
extern "C" int tvb_post_layer_norm(const void* x, int x_dtype, float alpha, const void* add, int add_dtype,
                                   const void* weight, int weight_dtype, void* y, int dtype, float* stream_out,
                                   const int* gather, int rows, int width, float eps, void* stream) {
    if (rows <= 0) return 0;
    if (width <= 0 || !x || !weight || (!y && !stream_out)) return TVB_BAD_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (!add) add_dtype = TVB_F32;
#define GO(S, A, T, W) return launch_post_norm<S, A, T, W>(x, alpha, add, weight, y, stream_out, gather, rows, width, eps, s)
    if (dtype == TVB_F32) {
        if (x_dtype == TVB_F32 && add_dtype == TVB_F32 && weight_dtype == TVB_F32) GO(float, float, float, float);
        return TVB_BAD_ARGUMENT;
    }
    if (dtype != TVB_BF16) return TVB_BAD_ARGUMENT;
    const int key = (x_dtype == TVB_BF16 ? 4 : 0) | (add_dtype == TVB_BF16 ? 2 : 0) | (weight_dtype == TVB_BF16 ? 1 : 0);
    switch (key) {
        case 0: GO(float, float, bf16, float);
        case 1: GO(float, float, bf16, bf16);
        case 2: GO(float, bf16, bf16, float);
        case 3: GO(float, bf16, bf16, bf16);
        case 4: GO(bf16, float, bf16, float);
        case 5: GO(bf16, float, bf16, bf16);
        case 6: GO(bf16, bf16, bf16, float);
        default: GO(bf16, bf16, bf16, bf16);
    }
#undef GO
}

// ------------------------------------------------------------ x *= factor (float32, in place)
__global__ void scale_float32_kernel(float* x, int64_t count, float factor) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) x[i] = __fmul_rn(x[i], factor);
}

extern "C" int tvb_scale_float32(float* x, long long count, float factor, void* stream) {
    if (count <= 0) return 0;
    scale_float32_kernel<<<(unsigned)((count + 255) / 256), 256, 0, (cudaStream_t)stream>>>(x, count, factor);
    return tvb_last_error();
}
