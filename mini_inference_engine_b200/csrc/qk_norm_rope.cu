// What happens to a fused q|k|v projection between the product and attention, for mixers whose queries and keys
// are normed as whole projections and whose heads may be narrower than the pages that hold them:
//
//   qkv[t] = [ q: H x D | k: G x D | v: G x Dv | anything else ]         (row stride `qkv_stride`)
//   q <- q * rsqrt(mean over all H*D entries of q^2 + eps) * qw[:]       (if qw; the same for k with kw over G*D)
//   rotation (rotate-half pairing over the first `rot` dims of every head): with a = position * freq[i],
//       (x_i, x_{i + rot/2}) <- (x_i cos a - x_{i + rot/2} sin a,  x_{i + rot/2} cos a + x_i sin a)
//   q[h] <- q[h] * q_scale * temp[h]    (if temp: a per-head factor on the scores, folded into the query)
//   k    <- k * k_scale
//   q is written to q_out [T, H, DP], k and v to their cache slot [page, G, page_size, DP]; DP >= max(D, Dv), the tail of
//   every head is zero, so that kernels written for one head size serve heads whose key and value sizes differ.
//
// Options: `head_norm` -- the RMS statistics are per head (over its D entries) and qw / kw hold D weights shared by all heads;
// `interleaved` -- the rotation pairs entry 2i with 2i + 1 instead of i with i + rot/2 (the same angle position * freq[i]);
// `temp_coef`, `temp_every` -- the query of position p is also multiplied by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)
// (a temperature that grows with the position; temp_every <= 0: none).
//
// `freq` holds rot/2 float32 frequencies (the host computes them, with whatever rescaling the model asks for);
// angles, cosines and sines are float32 and computed here from the position (once per token, for all heads), so no
// table bounds the positions.
// Statistics and all arithmetic are float32; outputs are rounded to the activation type once.  One block per token.
#include "common.cuh"
#include "range_check.cuh"

#define MIE_K_QK_NORM_ROPE 10

template <typename T>
__global__ void qk_norm_rope_kernel(const T* __restrict__ qkv, int64_t qkv_stride, const int* __restrict__ positions,
                                    const int* __restrict__ slots, const float* __restrict__ freq,
                                    const void* __restrict__ qw, const void* __restrict__ kw, const void* __restrict__ temp,
                                    int w_tag, float eps, float q_scale, float k_scale, T* __restrict__ q_out,
                                    T* __restrict__ k_cache, T* __restrict__ v_cache, int H, int G, int D, int Dv, int DP,
                                    int rot, int page_size, int64_t num_pages, int write_cache, int* report, int head_norm,
                                    int interleaved, float temp_coef, int temp_every) {
    __shared__ float red[33];
    extern __shared__ float cs[];                 // cos [rot/2], sin [rot/2]: once per token, for all heads
    pdl_enter();
    const int t = blockIdx.x;
    const T* q = qkv + (int64_t)t * qkv_stride;
    const T* k = q + H * D;
    const T* v = k + G * D;
    const float pos = (float)positions[t];
    float sq = 1.f, sk = 1.f;
    if (qw && !head_norm) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H * D; i += blockDim.x) { const float x = to_f32<T>(q[i]); ss += x * x; }
        sq = 1.0f / sqrtf(block_sum(ss, red) / (float)(H * D) + eps);
    }
    if (kw && !head_norm) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < G * D; i += blockDim.x) { const float x = to_f32<T>(k[i]); ss += x * x; }
        sk = 1.0f / sqrtf(block_sum(ss, red) / (float)(G * D) + eps);
    }
    const int half = rot >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float a = pos * freq[i];
        cs[i] = cosf(a);
        cs[half + i] = sinf(a);
    }
    __syncthreads();
    // one entry of a rotated projection: x normed, then turned with its partner
    auto entry = [&](const T* x, const void* w, float s, int h, int d) -> float {
        const int wb = head_norm ? 0 : h * D;                     // per-head norms share one weight vector
        float own = to_f32<T>(x[h * D + d]) * s;
        if (w) own *= load_tagged(w, wb + d, w_tag);
        if (d >= rot) return own;
        const bool first = interleaved ? !(d & 1) : d < half;    // the pair's first entry turns with a minus
        const int pd = interleaved ? (d ^ 1) : (d < half ? d + half : d - half);
        const int fi = interleaved ? (d >> 1) : (d < half ? d : d - half);
        float other = to_f32<T>(x[h * D + pd]) * s;
        if (w) other *= load_tagged(w, wb + pd, w_tag);
        const float c = cs[fi], sn = cs[half + fi];
        return first ? own * c - other * sn : own * c + other * sn;
    };
    // a head's own statistic, by the head's warp
    auto head_scale = [&](const T* x, int h, int lane) -> float {
        float ss = 0.f;
        for (int d = lane; d < D; d += 32) { const float v = to_f32<T>(x[h * D + d]); ss += v * v; }
        return 1.0f / sqrtf(warp_sum(ss) / (float)D + eps);
    };
    float pos_temp = 1.f;
    if (temp_every > 0) pos_temp = 1.0f + temp_coef * logf((float)((positions[t] + 1) / temp_every) + 1.0f);
    T* qo = q_out + (int64_t)t * H * DP;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int h = warp; h < H; h += nw) {                      // a head a warp, a dimension a lane: no divisions
        const float hs = (temp ? q_scale * load_tagged(temp, h, w_tag) : q_scale) * pos_temp;
        const float s_h = (qw && head_norm) ? head_scale(q, h, lane) : sq;
        for (int d = lane; d < DP; d += 32) qo[h * DP + d] = from_f32<T>(d < D ? entry(q, qw, s_h, h, d) * hs : 0.f);
    }
    if (!write_cache) return;
    const int slot = slots[t];
    if (range_slot(slot, num_pages, page_size) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_SLOT, MIE_K_QK_NORM_ROPE, t, slot);
        return;
    }
    const int page = slot / page_size, off = slot - page * page_size;
    for (int g = warp; g < G; g += nw) {
        const int64_t row = (((int64_t)page * G + g) * page_size + off) * DP;
        const float s_g = (kw && head_norm) ? head_scale(k, g, lane) : sk;
        for (int d = lane; d < DP; d += 32) {
            k_cache[row + d] = from_f32<T>(d < D ? entry(k, kw, s_g, g, d) * k_scale : 0.f);
            v_cache[row + d] = d < Dv ? v[g * Dv + d] : from_f32<T>(0.f);
        }
    }
}

extern "C" int mie_qk_norm_rope(const void* qkv, int tag, long long qkv_stride, const int* positions, const int* slots,
                                const float* freq, const void* qw, const void* kw, const void* temp, int w_tag, float eps,
                                float q_scale, float k_scale, void* q_out, void* k_cache, void* v_cache, int num_tokens, int H,
                                int G, int D, int Dv, int DP, int rot, int page_size, long long num_pages, int write_cache,
                                int head_norm, int interleaved, float temp_coef, int temp_every, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || G <= 0 || D <= 0 || Dv <= 0 || DP < D || DP < Dv || rot < 0 || rot > D || (rot & 1) || page_size <= 0)
        return MIE_ERR_BAD_ARG;
    const int threads = H * DP >= 2048 ? 256 : 128;
    if (tag == MIE_F32)
        return launch_kernel(qk_norm_rope_kernel<float>, dim3(num_tokens), dim3(threads), (size_t)rot * sizeof(float), stream, (const float*)qkv,
                             (int64_t)qkv_stride, positions, slots, freq, qw, kw, temp, w_tag, eps, q_scale, k_scale,
                             (float*)q_out, (float*)k_cache, (float*)v_cache, H, G, D, Dv, DP, rot, page_size,
                             (int64_t)num_pages, write_cache, g_range_report, head_norm, interleaved, temp_coef, temp_every);
    else if (tag == MIE_BF16)
        return launch_kernel(qk_norm_rope_kernel<bf16>, dim3(num_tokens), dim3(threads), (size_t)rot * sizeof(float), stream, (const bf16*)qkv,
                             (int64_t)qkv_stride, positions, slots, freq, qw, kw, temp, w_tag, eps, q_scale, k_scale,
                             (bf16*)q_out, (bf16*)k_cache, (bf16*)v_cache, H, G, D, Dv, DP, rot, page_size,
                             (int64_t)num_pages, write_cache, g_range_report, head_norm, interleaved, temp_coef, temp_every);
    return MIE_ERR_BAD_ARG;
}
