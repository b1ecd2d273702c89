// The stream's update for layers whose norm sits on the sublayer's OUTPUT, and the depth-weighted average of the layers'
// results.  With y[t, :] the sum of up to three branches (float32 or bfloat16) and, optionally, row_scale[t] * h[t, :]:
//
//   x[t, :] = res[t, :] + y / sqrt(mean(y^2) + eps) * gain * vec[:]          gain: one number (optional), vec: optional
//
// and, when a history of the stream is kept (hist[j] = X_j, the result of layer j - 1; X_0 the embedding):
//
//   hist[slot][t, :] = x;      x <- sum over j <= slot of coef[j] * hist[j][t, :]
//
// then res <- x and, optionally, act <- x rounded to bfloat16 for the next reader.  Without branches nothing is normed
// or added (the average alone).  One block per token; y stays in shared memory between the statistics and the update, so
// every input is read once.  Everything is float32 but `act`.
#include "common.cuh"

struct Addend { const void* p; int tag; };

__device__ __forceinline__ float4 load4(const void* p, int tag, int64_t i) {       // entries i .. i+3, i a multiple of 4
    if (tag == MIE_F32) return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p) + i);
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(p) + i);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

template <int VEC>      // VEC 4: rows of whole float4, all pointers 16-byte aligned (8 for bfloat16)
__global__ void normed_add_kernel(float* __restrict__ res, Addend b0, Addend b1, Addend b2, int num_addends, Addend scaled,
                                  const float* __restrict__ row_scale, const float* __restrict__ gain, const float* __restrict__ vec,
                                  float eps, bf16* __restrict__ act, float* __restrict__ hist, int64_t hist_stride, int slot,
                                  const float* __restrict__ coef, int W) {
    extern __shared__ __align__(16) float ys[];
    __shared__ float red[33];
    pdl_enter();
    const int t = blockIdx.x;
    const int64_t base = (int64_t)t * W;
    const bool normed = num_addends > 0 || scaled.p != nullptr;
    float r = 0.f;
    // the thread's first piece of the stream is asked for before the statistics, so that its latency hides under them
    float4 x_first = make_float4(0.f, 0.f, 0.f, 0.f);
    if (VEC == 4 && threadIdx.x * 4 < W) x_first = *reinterpret_cast<const float4*>(res + base + threadIdx.x * 4);
    if (normed) {
        const float rs = scaled.p ? row_scale[t] : 0.f;
        float ss = 0.f;
        if (VEC == 4) {
            for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
                float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
                if (num_addends > 0) { const float4 a = load4(b0.p, b0.tag, base + i); y = a; }
                if (num_addends > 1) { const float4 a = load4(b1.p, b1.tag, base + i); y.x += a.x; y.y += a.y; y.z += a.z; y.w += a.w; }
                if (num_addends > 2) { const float4 a = load4(b2.p, b2.tag, base + i); y.x += a.x; y.y += a.y; y.z += a.z; y.w += a.w; }
                if (scaled.p) { const float4 a = load4(scaled.p, scaled.tag, base + i); y.x = fmaf(rs, a.x, y.x); y.y = fmaf(rs, a.y, y.y); y.z = fmaf(rs, a.z, y.z); y.w = fmaf(rs, a.w, y.w); }
                *reinterpret_cast<float4*>(ys + i) = y;
                ss += y.x * y.x + y.y * y.y + y.z * y.z + y.w * y.w;
            }
        } else {
            for (int i = threadIdx.x; i < W; i += blockDim.x) {
                float y = 0.f;
                if (num_addends > 0) y = load_tagged(b0.p, base + i, b0.tag);
                if (num_addends > 1) y += load_tagged(b1.p, base + i, b1.tag);
                if (num_addends > 2) y += load_tagged(b2.p, base + i, b2.tag);
                if (scaled.p) y = fmaf(rs, load_tagged(scaled.p, base + i, scaled.tag), y);
                ys[i] = y;
                ss += y * y;
            }
        }
        r = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
        if (gain) r *= gain[0];
    }
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
            float4 x = i == threadIdx.x * 4 ? x_first : *reinterpret_cast<const float4*>(res + base + i);
            if (normed) {
                const float4 y = *reinterpret_cast<const float4*>(ys + i);
                float4 v = make_float4(r, r, r, r);
                if (vec) { const float4 w = *reinterpret_cast<const float4*>(vec + i); v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w; }
                x.x = fmaf(y.x, v.x, x.x); x.y = fmaf(y.y, v.y, x.y); x.z = fmaf(y.z, v.z, x.z); x.w = fmaf(y.w, v.w, x.w);
            }
            if (hist) {
                *reinterpret_cast<float4*>(hist + (int64_t)slot * hist_stride + base + i) = x;
                const float c = coef[slot];
                x.x *= c; x.y *= c; x.z *= c; x.w *= c;
                for (int j = 0; j < slot; ++j) {
                    const float4 p = *reinterpret_cast<const float4*>(hist + (int64_t)j * hist_stride + base + i);
                    const float cj = coef[j];
                    x.x = fmaf(cj, p.x, x.x); x.y = fmaf(cj, p.y, x.y); x.z = fmaf(cj, p.z, x.z); x.w = fmaf(cj, p.w, x.w);
                }
            }
            *reinterpret_cast<float4*>(res + base + i) = x;
            if (act) {
                uint2 u;
                *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(x.x, x.y);
                *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(x.z, x.w);
                *reinterpret_cast<uint2*>(act + base + i) = u;
            }
        }
    } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            float x = res[base + i];
            if (normed) x = fmaf(ys[i], vec ? r * vec[i] : r, x);
            if (hist) {
                hist[(int64_t)slot * hist_stride + base + i] = x;
                x *= coef[slot];
                for (int j = 0; j < slot; ++j) x = fmaf(coef[j], hist[(int64_t)j * hist_stride + base + i], x);
            }
            res[base + i] = x;
            if (act) act[base + i] = __float2bfloat16_rn(x);
        }
    }
}

static inline bool aligned_to(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// addends: up to three [T, W] tensors with their type tags; scaled / row_scale: one more, multiplied by a float32 number per
// row; gain: one float32 on the device; vec: float32 [W]; act: bfloat16 [T, W]; hist: float32 [slots, T, W] with
// hist_stride = T * W entries between slots; coef: float32 [slot + 1].
extern "C" int mie_normed_add(float* res, const void* a0, int t0, const void* a1, int t1, const void* a2, int t2, int num_addends,
                              const void* scaled, int ts, const float* row_scale, const float* gain, const float* vec, float eps,
                              void* act, float* hist, long long hist_stride, int slot, const float* coef, int num_tokens, int W,
                              cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (W <= 0 || num_addends < 0 || num_addends > 3 || (scaled && !row_scale) || (hist && (slot < 0 || !coef))) return MIE_ERR_BAD_ARG;
    if ((size_t)W * sizeof(float) > 200 * 1024) return MIE_ERR_TOO_LARGE;
    const Addend b0{a0, t0}, b1{a1, t1}, b2{a2, t2}, sc{scaled, ts};
    bool vec4 = W % 4 == 0 && aligned_to(res, 16) && aligned_to(vec, 16) && aligned_to(act, 8) && aligned_to(hist, 16) &&
                (hist_stride % 4 == 0);
    const Addend all[4] = {b0, b1, b2, sc};
    for (int i = 0; i < 4; ++i)
        if (i == 3 ? scaled != nullptr : i < num_addends) vec4 = vec4 && aligned_to(all[i].p, all[i].tag == MIE_F32 ? 16 : 8);
    const size_t smem = (size_t)W * sizeof(float);
    const int per = vec4 ? 4 : 1;
    int threads = (W / per + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
    auto kernel = vec4 ? normed_add_kernel<4> : normed_add_kernel<1>;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    return launch_kernel(kernel, dim3(num_tokens), dim3(threads), smem, stream, res, b0, b1, b2, num_addends, sc, row_scale, gain, vec,
                         eps, (bf16*)act, hist, (int64_t)hist_stride, slot, coef, W);
}
