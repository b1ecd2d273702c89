// SwiGLU on a fused gate/up projection: out[t, i] = silu(gu[t, i]) * gu[t, I + i],
// silu(z) = z / (1 + exp(-z)), computed in float32 (inference_engine/model.py:180-181, where the
// two halves come from `.chunk(2)` of the fused projection).  With `interleaved` the projection's
// columns alternate gate_i, up_i (the layout the tensor-core product's fused epilogue wants of the
// weight): out[t, i] = silu(gu[t, 2i]) * gu[t, 2i + 1].
#include "common.cuh"

template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int inter, int interleaved) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / inter;
        const int i = (int)(idx - t * inter);
        const float g = to_f32<T>(gu[t * 2 * inter + (interleaved ? 2 * i : i)]);
        const float u = to_f32<T>(gu[t * 2 * inter + (interleaved ? 2 * i + 1 : inter + i)]);
        out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// Eight outputs per thread with 16-byte loads and stores (bfloat16, inter % 8 == 0).  The result is
// rounded to bfloat16, so the exponential and the division are the hardware approximations (two ulp
// each in float32): with the library's the kernel issued instructions all the time and reached 0.6 of
// the memory bandwidth on 2,048 tokens.  Token and place within it are counted along the grid-stride
// loop instead of divided out of a 64-bit index every time.
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int64_t total8, int inter8,
                                     int interleaved) {
    pdl_enter();
    const unsigned stride = gridDim.x * blockDim.x, first = blockIdx.x * blockDim.x + threadIdx.x;   // the grid is capped: both fit
    const unsigned stride_t = stride / (unsigned)inter8, stride_i = stride - stride_t * (unsigned)inter8;
    int64_t t = first / (unsigned)inter8;
    int i8 = (int)(first - (unsigned)t * (unsigned)inter8);
    for (int64_t idx = first; idx < total8; idx += stride, t += stride_t, i8 += (int)stride_i) {
        if (i8 >= inter8) { i8 -= inter8; ++t; }
        const bf16* row = gu + t * 16 * inter8;
        float g[8], u[8];
        if (interleaved) {
            const uint4 a = *reinterpret_cast<const uint4*>(row + 16 * i8), b = *reinterpret_cast<const uint4*>(row + 16 * i8 + 8);
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(ha[j]), y = __bfloat1622float2(hb[j]);
                g[j] = x.x; u[j] = x.y; g[4 + j] = y.x; u[4 + j] = y.y;
            }
        } else {
            const uint4 a = *reinterpret_cast<const uint4*>(row + 8 * i8), b = *reinterpret_cast<const uint4*>(row + 8 * inter8 + 8 * i8);
            const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
            const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 x = __bfloat1622float2(ha[j]), y = __bfloat1622float2(hb[j]);
                g[2 * j] = x.x; g[2 * j + 1] = x.y; u[2 * j] = y.x; u[2 * j + 1] = y.y;
            }
        }
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j)
            ho[j] = __floats2bfloat162_rn(__fdividef(g[2 * j], 1.0f + __expf(-g[2 * j])) * u[2 * j],
                                          __fdividef(g[2 * j + 1], 1.0f + __expf(-g[2 * j + 1])) * u[2 * j + 1]);
        *reinterpret_cast<uint4*>(out + idx * 8) = o;
    }
}

extern "C" int mie_swiglu(const void* gu, void* out, int act_tag, int num_tokens, int inter, int interleaved,
                          cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (inter <= 0) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * inter;
    const int threads = 256;
    if (act_tag == MIE_BF16 && inter % 8 == 0 && (reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
        int64_t blocks8 = (total / 8 + threads - 1) / threads;
        if (blocks8 > device_sm_count() * 16) blocks8 = device_sm_count() * 16;
        return launch_kernel(swiglu_bf16x8_kernel, dim3((int)blocks8), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out,
                             total / 8, inter / 8, interleaved);
    }
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (act_tag == MIE_F32)
        return launch_kernel(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out, total, inter, interleaved);
    else if (act_tag == MIE_BF16)
        return launch_kernel(swiglu_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out, total, inter, interleaved);
    return MIE_ERR_BAD_ARG;
}

// A gated feed-forward activation with clamps, on a fused projection [gate | up] (gate first, `inter` columns each; with
// `interleaved`, columns alternate gate_i, up_i as for SwiGLU above):
//   g = min(gate, limit), u = clamp(up, -limit, limit);  out = g * sigmoid(slope * g) * (u + shift)
// computed in float32 and rounded once.  limit <= 0 means no clamp; limit < 0 also puts a cubic term into the sigmoid's
// argument, slope * g * (1 - limit * g^2): with slope 2 sqrt(2/pi) and limit -0.044715 the gate is gelu in its tanh form.
template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, int64_t total, int inter, float limit,
                                   float slope, float shift, int interleaved) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / inter;
        const int i = (int)(idx - t * inter);
        float g = to_f32<T>(gu[t * 2 * inter + (interleaved ? 2 * i : i)]);
        float u = to_f32<T>(gu[t * 2 * inter + (interleaved ? 2 * i + 1 : inter + i)]);
        if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
        const float z = limit < 0.f ? slope * g * fmaf(-limit * g, g, 1.0f) : slope * g;
        out[idx] = from_f32<T>(g / (1.0f + expf(-z)) * (u + shift));
    }
}

// Eight outputs a thread with 16-byte accesses (bfloat16, inter % 8 == 0)
__global__ void glu_clamped_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int64_t total8, int inter8,
                                          float limit, float slope, float shift, int interleaved) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / inter8;
        const int i8 = (int)(idx - t * inter8);
        const bf16* row = gu + t * 16 * inter8;
        // concatenated: a holds eight gates, b eight values; interleaved: a and b hold (gate, value) pairs 0 - 3 and 4 - 7
        const uint4 a = *reinterpret_cast<const uint4*>(row + (interleaved ? 16 : 8) * i8);
        const uint4 b = *reinterpret_cast<const uint4*>(row + (interleaved ? 16 * i8 + 8 : 8 * inter8 + 8 * i8));
        const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* hb = reinterpret_cast<const __nv_bfloat162*>(&b);
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 g, u;
            if (interleaved) {
                const float2 p0 = __bfloat1622float2(j < 2 ? ha[2 * j] : hb[2 * j - 4]), p1 = __bfloat1622float2(j < 2 ? ha[2 * j + 1] : hb[2 * j - 3]);
                g = make_float2(p0.x, p1.x);
                u = make_float2(p0.y, p1.y);
            } else {
                g = __bfloat1622float2(ha[j]);
                u = __bfloat1622float2(hb[j]);
            }
            if (limit > 0.f) {
                g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
                u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
            }
            float2 z = make_float2(slope * g.x, slope * g.y);
            if (limit < 0.f) { z.x *= fmaf(-limit * g.x, g.x, 1.0f); z.y *= fmaf(-limit * g.y, g.y, 1.0f); }
            ho[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.0f + __expf(-z.x)) * (u.x + shift),
                                          __fdividef(g.y, 1.0f + __expf(-z.y)) * (u.y + shift));
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = o;
    }
}

extern "C" int mie_glu_clamped(const void* gu, void* out, int act_tag, int num_tokens, int inter, float limit, float slope,
                               float shift, int interleaved, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (inter <= 0) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * inter;
    const int threads = 256;
    if (act_tag == MIE_BF16 && inter % 8 == 0 && (reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
        int64_t blocks8 = (total / 8 + threads - 1) / threads;
        if (blocks8 > device_sm_count() * 16) blocks8 = device_sm_count() * 16;
        return launch_kernel(glu_clamped_bf16x8_kernel, dim3((int)blocks8), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out,
                             total / 8, inter / 8, limit, slope, shift, interleaved);
    }
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (act_tag == MIE_F32)
        return launch_kernel(glu_clamped_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gu, (float*)out, total, inter, limit, slope, shift, interleaved);
    else if (act_tag == MIE_BF16)
        return launch_kernel(glu_clamped_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)gu, (bf16*)out, total, inter, limit, slope, shift, interleaved);
    return MIE_ERR_BAD_ARG;
}

// An output gate on attention heads: out[t, h * Dv + c] = attn[t, h, c] * sigmoid(g[t, h * Dv + c]) for c < Dv, where
// attn rows hold H heads of DP >= Dv entries (the padded tail is dropped) and g is a part of a fused projection
// with row stride `g_stride`.
template <typename T>
__global__ void sigmoid_gate_kernel(const T* __restrict__ attn, const T* __restrict__ g, int64_t g_stride, T* __restrict__ out,
                                    int64_t total, int H, int Dv, int DP) {
    pdl_enter();
    const int n = H * Dv;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / n;
        const int i = (int)(idx - t * n);
        const int h = i / Dv, c = i - h * Dv;
        const float z = to_f32<T>(g[t * g_stride + i]);
        out[idx] = from_f32<T>(to_f32<T>(attn[(t * H + h) * DP + c]) / (1.0f + expf(-z)));
    }
}

__global__ void sigmoid_gate_bf16x8_kernel(const bf16* __restrict__ attn, const bf16* __restrict__ g, int64_t g_stride,
                                           bf16* __restrict__ out, int64_t total8, int H, int Dv8, int DP) {
    pdl_enter();
    const int n8 = H * Dv8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / n8;
        const int i8 = (int)(idx - t * n8);
        const int h = i8 / Dv8, c8 = i8 - h * Dv8;
        const uint4 a = *reinterpret_cast<const uint4*>(attn + (t * H + h) * DP + 8 * c8);
        const uint4 z = *reinterpret_cast<const uint4*>(g + t * g_stride + 8 * i8);
        const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* hz = reinterpret_cast<const __nv_bfloat162*>(&z);
        uint4 o;
        __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 x = __bfloat1622float2(ha[j]), y = __bfloat1622float2(hz[j]);
            ho[j] = __floats2bfloat162_rn(__fdividef(x.x, 1.0f + __expf(-y.x)), __fdividef(x.y, 1.0f + __expf(-y.y)));
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = o;
    }
}

extern "C" int mie_sigmoid_gate(const void* attn, const void* g, long long g_stride, void* out, int act_tag, int num_tokens,
                                int H, int Dv, int DP, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || Dv <= 0 || DP < Dv) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * H * Dv;
    const int threads = 256;
    if (act_tag == MIE_BF16 && Dv % 8 == 0 && DP % 8 == 0 && g_stride % 8 == 0 &&
        (reinterpret_cast<uintptr_t>(attn) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
        int64_t blocks8 = (total / 8 + threads - 1) / threads;
        if (blocks8 > device_sm_count() * 16) blocks8 = device_sm_count() * 16;
        return launch_kernel(sigmoid_gate_bf16x8_kernel, dim3((int)blocks8), dim3(threads), 0, stream, (const bf16*)attn, (const bf16*)g,
                             (int64_t)g_stride, (bf16*)out, total / 8, H, Dv / 8, DP);
    }
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (act_tag == MIE_F32)
        return launch_kernel(sigmoid_gate_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)attn, (const float*)g, (int64_t)g_stride, (float*)out, total, H, Dv, DP);
    else if (act_tag == MIE_BF16)
        return launch_kernel(sigmoid_gate_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)attn, (const bf16*)g, (int64_t)g_stride, (bf16*)out, total, H, Dv, DP);
    return MIE_ERR_BAD_ARG;
}

// xIELU, an activation with two constants: for z > 0 a quadratic arm, ap z^2 + z / 2; for z <= 0 an exponential arm,
// an (exp(z) - 1 - z) + z / 2.  Both arms have slope 1/2 at 0.  The caller derives ap and an from the learned numbers.
// Computed in float32 and rounded once.
__device__ __forceinline__ float xielu_f(float z, float ap, float an) {
    return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(an, expm1f(z) - z, 0.5f * z);
}
template <typename T>
__global__ void xielu_kernel(const T* __restrict__ x, T* __restrict__ out, int64_t total, float ap, float an) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x)
        out[idx] = from_f32<T>(xielu_f(to_f32<T>(x[idx]), ap, an));
}
__global__ void xielu_bf16x8_kernel(const bf16* __restrict__ x, bf16* __restrict__ out, int64_t total8, float ap, float an) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (int64_t)gridDim.x * blockDim.x) {
        uint4 u = *reinterpret_cast<const uint4*>(x + idx * 8);
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            h[j] = __floats2bfloat162_rn(xielu_f(f.x, ap, an), xielu_f(f.y, ap, an));
        }
        *reinterpret_cast<uint4*>(out + idx * 8) = u;
    }
}

extern "C" int mie_xielu(const void* x, void* out, int act_tag, long long total, float ap, float an, cudaStream_t stream) {
    if (total <= 0) return 0;
    const int threads = 256;
    if (act_tag == MIE_BF16 && total % 8 == 0 && (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) % 16 == 0) {
        int64_t blocks8 = (total / 8 + threads - 1) / threads;
        if (blocks8 > device_sm_count() * 16) blocks8 = device_sm_count() * 16;
        return launch_kernel(xielu_bf16x8_kernel, dim3((int)blocks8), dim3(threads), 0, stream, (const bf16*)x, (bf16*)out, (int64_t)(total / 8), ap, an);
    }
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (act_tag == MIE_F32)
        return launch_kernel(xielu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)x, (float*)out, (int64_t)total, ap, an);
    else if (act_tag == MIE_BF16)
        return launch_kernel(xielu_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)x, (bf16*)out, (int64_t)total, ap, an);
    return MIE_ERR_BAD_ARG;
}

// A gate on rows gathered from a per-token table: out[t, d] = gelu_tanh(g[t, d]) * table[ids[t], first + d] for d < n, where a
// table row has `table_width` entries.  ids are vocabulary entries (already resolved); one outside [0, vocab) gives zeros.
template <typename T>
__global__ void gelu_gate_rows_kernel(const T* __restrict__ g, const T* __restrict__ table, const int* __restrict__ ids,
                                      T* __restrict__ out, int64_t total, int n, int table_width, int first, int vocab) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / n;
        const int d = (int)(idx - t * n);
        const int id = ids[t];
        const float z = to_f32<T>(g[idx]);
        const float e = id >= 0 && id < vocab ? to_f32<T>(table[(int64_t)id * table_width + first + d]) : 0.f;
        out[idx] = from_f32<T>(0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z))) * e);
    }
}

extern "C" int mie_gelu_gate_rows(const void* g, const void* table, const int* ids, void* out, int act_tag, int num_tokens, int n,
                                  int table_width, int first, int vocab, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (n <= 0 || first < 0 || first + n > table_width || vocab <= 0) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * n;
    const int threads = 256;
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > device_sm_count() * 16) blocks = device_sm_count() * 16;
    if (act_tag == MIE_F32)
        return launch_kernel(gelu_gate_rows_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)g, (const float*)table, ids, (float*)out, total, n, table_width, first, vocab);
    else if (act_tag == MIE_BF16)
        return launch_kernel(gelu_gate_rows_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)g, (const bf16*)table, ids, (bf16*)out, total, n, table_width, first, vocab);
    return MIE_ERR_BAD_ARG;
}
