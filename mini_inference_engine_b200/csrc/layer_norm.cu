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

__device__ __forceinline__ void store4(float* p, float a, float b, float c, float d) { *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d); }
__device__ __forceinline__ void store4(bf16* p, float a, float b, float c, float d) {
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(a, b);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(c, d);
    *reinterpret_cast<uint2*>(p) = o;
}

template <typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ res, float res_coef, const void* __restrict__ d0, int tag0, float c0,
                                     const void* __restrict__ d1, int tag1, float c1, const float* __restrict__ w,
                                     TO* __restrict__ out, const int* __restrict__ rows, int n, float eps, int center,
                                     int num_in_rows, int* report, int vec4) {
    extern __shared__ __align__(16) float row_cache[];
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
    if (vec4) {
        // 16 bytes a load: rows of whole float4 (the caller has checked sizes, alignment and that the addends are float32)
        const float4* r4 = reinterpret_cast<const float4*>(res_row);
        const float4* a4 = d0 ? reinterpret_cast<const float4*>(reinterpret_cast<const float*>(d0) + r * n) : nullptr;
        const float4* b4 = d1 ? reinterpret_cast<const float4*>(reinterpret_cast<const float*>(d1) + r * n) : nullptr;
        for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
            float4 v = r4[i];
            if (sums) {
                v.x *= res_coef; v.y *= res_coef; v.z *= res_coef; v.w *= res_coef;
                if (a4) { const float4 a = a4[i]; v.x = fmaf(c0, a.x, v.x); v.y = fmaf(c0, a.y, v.y); v.z = fmaf(c0, a.z, v.z); v.w = fmaf(c0, a.w, v.w); }
                if (b4) { const float4 a = b4[i]; v.x = fmaf(c1, a.x, v.x); v.y = fmaf(c1, a.y, v.y); v.z = fmaf(c1, a.z, v.z); v.w = fmaf(c1, a.w, v.w); }
                if (!rows) reinterpret_cast<float4*>(res_row)[i] = v;
            }
            reinterpret_cast<float4*>(row_cache)[i] = v;
            s += (v.x + v.y) + (v.z + v.w);
        }
    } else
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
    } else {
        __syncthreads();                                           // the row is read back by other threads than wrote it
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) { const float dv = row_cache[i] - mean; ss += dv * dv; }
    const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
    TO* o_row = out + (int64_t)b * n;
    if (vec4) {
        for (int i = threadIdx.x; i < (n >> 2); i += blockDim.x) {
            const float4 v = reinterpret_cast<const float4*>(row_cache)[i], ww = reinterpret_cast<const float4*>(w)[i];
            store4(o_row + 4 * i, (v.x - mean) * rstd * ww.x, (v.y - mean) * rstd * ww.y, (v.z - mean) * rstd * ww.z, (v.w - mean) * rstd * ww.w);
        }
        return;
    }
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
    const auto aligned = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec4 = n % 4 == 0 && aligned(res) && aligned(w) && aligned(out) && (!d0 || (tag0 == MIE_F32 && aligned(d0))) &&
                     (!d1 || (tag1 == MIE_F32 && aligned(d1)));
    cudaError_t e;
    if (act_tag == MIE_F32) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(add_layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_kernel(add_layernorm_kernel<float>, dim3(num_rows), dim3(threads), smem, stream, res, res_coef, d0, tag0, c0, d1,
                             tag1, c1, w, (float*)out, rows, n, eps, center, num_in_rows, g_range_report, vec4);
    } else if (act_tag == MIE_BF16) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(add_layernorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_kernel(add_layernorm_kernel<bf16>, dim3(num_rows), dim3(threads), smem, stream, res, res_coef, d0, tag0, c0, d1,
                             tag1, c1, w, (bf16*)out, rows, n, eps, center, num_in_rows, g_range_report, vec4);
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
