// Layer norm with weight and bias, float32 statistics: y = (v - mean) / sqrt(var + eps) * w + b, var the mean of the
// squared deviations from the mean (two passes over the row, which sits in shared memory).
//
// Two uses, one kernel.  (1) A norm on a sublayer's output: v is the sublayer's update; y is added to the float32
// residual stream in place and the new stream is also written in the type the next sublayer's products read
// (`act`), so the sum, the norm and the cast read and write each row once.  (2) A norm of the stream itself
// (a model's last norm): v = x[rows[r]], y goes to `act`, nothing is added.
#include "common.cuh"

struct LayerNormParams {
    const float* in;        // [R, width] rows to norm
    const int* rows;        // null, or for each output row the row of `in` it norms
    const float* weight;    // [width]
    const float* bias;      // [width] or null
    float* stream;          // null, or [R, width]: stream[r] += y
    void* act;              // null, or [R, width]: the new stream (or y when there is no stream) in ActT
    float eps;
    int width;
};

template <typename ActT, int BLOCK>
__global__ void __launch_bounds__(BLOCK) layernorm_kernel(LayerNormParams p) {
    extern __shared__ float row[];           // [width]
    __shared__ float scratch[32];
    // the weights do not depend on the kernel before this one
    let_next_kernel_start();
    const int r = blockIdx.x;
    const int width = p.width;
    wait_for_previous_kernel();
    const int src = p.rows ? p.rows[r] : r;
    const float* in = p.in + (size_t)src * width;
    float sum = 0.f;
    for (int i = threadIdx.x; i < width; i += BLOCK) {
        const float v = in[i];
        row[i] = v;
        sum += v;
    }
    const float mean = block_sum<BLOCK>(sum, scratch) / (float)width;
    float dev = 0.f;
    for (int i = threadIdx.x; i < width; i += BLOCK) {
        const float d = row[i] - mean;
        dev += d * d;
    }
    const float rinv = 1.0f / sqrtf(block_sum<BLOCK>(dev, scratch) / (float)width + p.eps);
    float* stream = p.stream ? p.stream + (size_t)r * width : nullptr;
    ActT* act = p.act ? (ActT*)p.act + (size_t)r * width : nullptr;
    for (int i = threadIdx.x; i < width; i += BLOCK) {
        float y = (row[i] - mean) * rinv * p.weight[i] + (p.bias ? p.bias[i] : 0.f);
        if (stream) {
            y += stream[i];
            stream[i] = y;
        }
        if (act) act[i] = from_f32<ActT>(y);
    }
}

FRB_API int frb_layernorm(const float* in, const int* rows, const float* weight, const float* bias, float eps,
                          float* stream, void* act, int act_dtype, int num_rows, int width, cudaStream_t stream_handle) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(width >= 1 && (size_t)width * sizeof(float) <= 200 * 1024, "layernorm: a row of %d does not fit shared memory", width);
    FRB_CHECK_ARG(!(stream && rows), "layernorm: a norm that adds to the stream takes every row in order");
    LayerNormParams p;
    p.in = in; p.rows = rows; p.weight = weight; p.bias = bias; p.stream = stream; p.act = act; p.eps = eps; p.width = width;
    const size_t smem = (size_t)width * sizeof(float);
    FRB_DISPATCH_DTYPE(act_dtype, ActT, {
        if (num_rows <= 64 && width >= 2048) {
            auto kernel = layernorm_kernel<ActT, 1024>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_rows), dim3(1024), smem, stream_handle, p);
        } else {
            auto kernel = layernorm_kernel<ActT, 256>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_rows), dim3(256), smem, stream_handle, p);
        }
    });
    FRB_RETURN_LAUNCH("layernorm");
}
