// Layer norm fused with the sums in front of it, for pre-norm layers whose sublayers may hand over more than one output:
//
//   res[r, :] <- res_coef * res[r, :] + c0 * d0[r, :] + c1 * d1[r, :]        (float32 stream, updated in place)
//   out[r, :]  = (res[r, :] - mean) / sqrt(var + eps) * w[:]                  var = mean of the squared deviations
//
// d0 and d1 are optional and may each be float32 or bfloat16 (outputs that enter the stream's sum arrive in float32); with
// `center` 0 the mean is taken as 0 and the same kernel is an RMS norm over a sum of several outputs.  One block per row; the
// summed row stays in shared memory between the passes (sum, squared deviations, output), so every input is read once and
// the variance is that of the deviations, not a difference of two large numbers.  Statistics and sums are float32; only
// `out` is rounded to the activation type.  `rows` (optional) gathers: output row b comes from input row rows[b] and the
// stream is left untouched (the selection in front of the output head).
//
// stream_join: out[t] = [ res_coef * res[t] + c0 * d0[t] + c1 * d1[t] | extra[t] ] in the activation type, the operand of a
// product that mixes the stream with a second float32 stream of the same width (the stream itself is not written).
//
// tanh_cap: x <- cap * tanh(x / cap) in place, float32 (a soft limit on logits).
#include "common.cuh"
#include "range_check.cuh"

#define MIE_K_LAYER_NORM 11

template <typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ res, float res_coef, const void* __restrict__ d0, int tag0, float c0,
                                     const void* __restrict__ d1, int tag1, float c1, const float* __restrict__ w,
                                     TO* __restrict__ out, const int* __restrict__ rows, int n, float eps, int center,
                                     int num_in_rows, int* report) {
    extern __shared__ float row_cache[];
    __shared__ float red[33];
    pdl_enter();
    const int b = blockIdx.x;
    const int64_t r = rows ? rows[b] : b;
    if (rows && range_row(r, num_in_rows) != MIE_RANGE_OK) {      // a gathered row that does not exist: reported, not read
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_ROW, MIE_K_LAYER_NORM, b, (int)r);
        return;
    }
    float* res_row = res + r * n;
    const bool sums = d0 || d1 || res_coef != 1.0f;
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = res_row[i];
        if (sums) {
            v *= res_coef;
            if (d0) v = fmaf(c0, load_tagged(d0, r * n + i, tag0), v);
            if (d1) v = fmaf(c1, load_tagged(d1, r * n + i, tag1), v);
            if (!rows) res_row[i] = v;
        }
        row_cache[i] = v;
        s += v;
    }
    float mean = 0.f;
    if (center) {
        mean = block_sum(s, red) / (float)n;
        __syncthreads();                                           // `red` is used again below
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float dv = row_cache[i] - mean; ss += dv * dv; }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    TO* o_row = out + (int64_t)b * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) o_row[i] = from_f32<TO>((row_cache[i] - mean) * rstd * w[i]);
}

template <typename TO>
__global__ void stream_join_kernel(const float* __restrict__ res, float res_coef, const void* __restrict__ d0, int tag0, float c0,
                                   const void* __restrict__ d1, int tag1, float c1, const float* __restrict__ extra,
                                   TO* __restrict__ out, int64_t total, int n) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / n;
        const int i = (int)(idx - t * n);
        float v = res_coef * res[idx];
        if (d0) v = fmaf(c0, load_tagged(d0, idx, tag0), v);
        if (d1) v = fmaf(c1, load_tagged(d1, idx, tag1), v);
        out[t * 2 * n + i] = from_f32<TO>(v);
        out[t * 2 * n + n + i] = from_f32<TO>(extra[idx]);
    }
}

__global__ void tanh_cap_kernel(float* __restrict__ x, int64_t total, float cap) {
    pdl_enter();
    const float inv = 1.0f / cap;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x)
        x[idx] = cap * tanhf(x[idx] * inv);
}

static inline int grid_for(int64_t total, int threads) {
    int64_t blocks = (total + threads - 1) / threads;
    const int64_t cap = (int64_t)device_sm_count() * 16;
    return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// act_tag: type of out.  d0 / d1 may be null; their tags say float32 or bfloat16.  w is float32 [n].
extern "C" int mie_add_layernorm(float* res, float res_coef, const void* d0, int tag0, float c0, const void* d1, int tag1, float c1,
                                 const float* w, void* out, int act_tag, const int* rows, int num_rows, int n, float eps,
                                 int center, int num_in_rows, cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (n <= 0) return MIE_ERR_BAD_ARG;
    const size_t smem = (size_t)n * sizeof(float);
    if (smem > 200 * 1024) return MIE_ERR_TOO_LARGE;
    int threads = 32;
    while (threads < 512 && threads * 4 < n) threads <<= 1;
    cudaError_t e;
    if (act_tag == MIE_F32) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(add_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_kernel(add_layernorm_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, res, res_coef, d0, tag0, c0, d1,
                             tag1, c1, w, (float*)out, rows, n, eps, center, num_in_rows, g_range_report);
    } else if (act_tag == MIE_BF16) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(add_layernorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_kernel(add_layernorm_kernel<bf16>, dim3(num_rows), dim3(threads), smem, stream, res, res_coef, d0, tag0, c0, d1,
                             tag1, c1, w, (bf16*)out, rows, n, eps, center, num_in_rows, g_range_report);
    }
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_stream_join(const float* res, float res_coef, const void* d0, int tag0, float c0, const void* d1, int tag1, float c1,
                               const float* extra, void* out, int act_tag, int num_tokens, int n, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (n <= 0) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * n;
    if (act_tag == MIE_F32)
        return launch_kernel(stream_join_kernel<float>, dim3(grid_for(total, 256)), dim3(256), 0, stream, res, res_coef, d0, tag0, c0, d1,
                             tag1, c1, extra, (float*)out, total, n);
    else if (act_tag == MIE_BF16)
        return launch_kernel(stream_join_kernel<bf16>, dim3(grid_for(total, 256)), dim3(256), 0, stream, res, res_coef, d0, tag0, c0, d1,
                             tag1, c1, extra, (bf16*)out, total, n);
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_tanh_cap(float* x, long long total, float cap, cudaStream_t stream) {
    if (total <= 0) return 0;
    if (!(cap > 0.f)) return MIE_ERR_BAD_ARG;
    return launch_kernel(tanh_cap_kernel, dim3(grid_for(total, 256)), dim3(256), 0, stream, x, (int64_t)total, cap);
}
