// A routed mixture of experts: the router's choice, and the experts' activation for the form in which all experts are
// one wide feed-forward.
//
//   router     route with the logits computed in the same kernel: z = W_router x in float32 (float32 weights, the token's
//              input widened), a block per eight tokens, a warp per expert in turn.
//   route      per token, from float32 router logits z [T, E]: the `top` experts with the largest logits (ties: the lower
//              index first), weights = softmax over the chosen logits only.  ids [T, top] int32, wts [T, top] float32.
//   dense_act  with up[t] = [expert 0: F | expert 1: F | ...] the up-projections of ALL experts (one product with the
//              experts' matrices stacked): act[t, e, :] = weight(t, e) f(up[t, e, :]) for a chosen expert, 0 for the others,
//              so that one product with the experts' down matrices side by side gives the weighted sum of the chosen
//              experts' outputs.  f: 0 relu(x)^2, 1 silu, 2 gelu (tanh form).
//   pairs_up / pairs_down   the same layer for a handful of tokens (decoding): a (token, chosen expert) pair streams only
//              its expert's rows -- one warp a matrix row, 16-byte loads -- so a step reads the experts that were chosen
//              and no others.  up: hid[pair, :] = weight f(W_up[e] x_t); down: out[t, :] = sum_k W_down[e_k] hid[pair_k, :]
//              (float32, the k in order).  The matrices are the stacked ones of the wide form: W_up [E * F, h] and
//              W_down [h, E * F].
//   sort / gather / act_rows / combine   the same layer for many tokens with the products done expert by expert (a grouped
//              product over rows sorted by expert): sort gives every (token, expert) pair its place among its expert's
//              rows and the experts' row ranges; gather copies the tokens' inputs to those places; act_rows applies
//              weight f(.) row by row; combine adds a token's rows up in float32, the pairs in order.
//
// A second routing rule (RouteRule.mode 1) and gated experts: scores s = softmax(z) over ALL router outputs; the choice is by
// s + correction (optional), limited to the experts of the `keep` best of `groups` equal groups of neighbours (a group's value is
// its largest choice score; the other groups count as minus infinity); the weights are the chosen s, not renormalized.  Router
// outputs from `real` on are identity experts: no matrices, output = input; the expert kernels skip them and `rest[t]` receives
// the sum of their weights for the caller to add rest[t] * x[t].  A gated expert is down(silu(gate x) * (up x)) with the stacked
// matrix [expert 0: gate F rows, up F rows | expert 1: ...].
#include "common.cuh"

struct RouteRule {
    int mode;                    // 0: the largest logits, softmax over the chosen; 1: softmax over all, see above;
                                 // 2: the largest logits, each chosen one's weight its own sigmoid (not renormalized)
    const float* correction;     // [outputs] added for the choice only (mode 1), or null
    int groups, keep;            // groups <= 1 or keep >= groups: no limit
    int real;                    // router outputs below this have matrices; the others are identity experts
    float* rest;                 // [tokens] sum of the chosen identity experts' weights, or null
};

// Mode 1 for one token.  `ready`: zt already holds softmax scores (made by the block together); else logits.
__device__ __forceinline__ void route_scored(const float* zt, int* ids, float* wts, int n, int top, const RouteRule& rr, bool ready,
                                             float* rest) {
    float m = 0.f, inv = 1.f;
    if (!ready) {
        m = -INFINITY;
        for (int e = 0; e < n; ++e) m = fmaxf(m, zt[e]);
        float sum = 0.f;
        for (int e = 0; e < n; ++e) sum += expf(zt[e] - m);
        inv = 1.0f / sum;
    }
    auto score = [&](int e) { return ready ? zt[e] : expf(zt[e] - m) * inv; };
    auto choice = [&](int e) { return rr.correction ? score(e) + rr.correction[e] : score(e); };
    unsigned long long allowed = ~0ull;
    const int per = rr.groups > 1 ? n / rr.groups : n;
    if (rr.groups > 1 && rr.keep < rr.groups) {
        allowed = 0ull;
        float prev_v = INFINITY;
        int prev_g = -1;
        for (int k = 0; k < rr.keep; ++k) {
            float best = -INFINITY;
            int bg = -1;
            for (int g = 0; g < rr.groups; ++g) {
                float v = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) v = fmaxf(v, choice(e));
                const bool after_prev = v < prev_v || (v == prev_v && g > prev_g);
                if (after_prev && (bg < 0 || v > best)) { best = v; bg = g; }
            }
            if (bg < 0) break;
            allowed |= 1ull << bg;
            prev_v = best;
            prev_g = bg;
        }
    }
    float prev_v = INFINITY, idw = 0.f;
    int prev_i = -1;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int e = 0; e < n; ++e) {
            if (!((allowed >> (rr.groups > 1 ? e / per : 0)) & 1ull)) continue;
            const float v = choice(e);
            const bool after_prev = v < prev_v || (v == prev_v && e > prev_i);
            if (after_prev && (bi < 0 || v > best)) { best = v; bi = e; }
        }
        float w = 0.f;
        if (bi < 0) bi = 0; else w = score(bi);               // scores that are not numbers: keep the ids in range, weight 0
        ids[k] = bi;
        wts[k] = w;
        if (bi >= rr.real) idw += w;
        prev_v = best;
        prev_i = bi;
    }
    if (rest) *rest = idw;
}

// Mode 1 for one token by a whole warp: zt holds the softmax scores (shared memory, made by this warp).  The same choice as
// route_scored, outcome for outcome: a group is kept if fewer than `keep` groups come before it in the order (value falling,
// index rising), which is what picking the best group `keep` times gives; each of the `top` picks is a maximum over the lanes'
// own outputs and then over the lanes, ties to the lower index.  A thread alone walks these loops at a dependent instruction
// every few cycles (16 us of a 26 us launch for one token, twenty outputs, four groups); a warp takes a few hundred cycles.
__device__ __forceinline__ void route_scored_warp(const float* zt, int* ids, float* wts, int n, int top, const RouteRule& rr, float* rest,
                                                  int lane) {
    const unsigned full = 0xffffffffu;
    auto choice = [&](int e) { return rr.correction ? zt[e] + rr.correction[e] : zt[e]; };
    unsigned long long allowed = ~0ull;
    const int per = rr.groups > 1 ? n / rr.groups : n;
    if (rr.groups > 1 && rr.keep < rr.groups) {             // at most 64 groups: a lane holds groups lane and lane + 32
        float v[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int g = lane + 32 * r;
            float m = -INFINITY;
            if (g < rr.groups)
                for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, choice(e));
            v[r] = m;
        }
        int ahead[2] = {0, 0};
        for (int g2 = 0; g2 < rr.groups; ++g2) {
            const float o = __shfl_sync(full, g2 < 32 ? v[0] : v[1], g2 & 31);
#pragma unroll
            for (int r = 0; r < 2; ++r)
                if (o > v[r] || (o == v[r] && g2 < lane + 32 * r)) ++ahead[r];
        }
        const unsigned lo = __ballot_sync(full, lane < rr.groups && ahead[0] < rr.keep);
        const unsigned hi = __ballot_sync(full, lane + 32 < rr.groups && ahead[1] < rr.keep);
        allowed = (unsigned long long)lo | ((unsigned long long)hi << 32);
    }
    float prev_v = INFINITY, idw = 0.f;
    int prev_i = -1;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int e = lane; e < n; e += 32) {
            if (!((allowed >> (rr.groups > 1 ? e / per : 0)) & 1ull)) continue;
            const float c = choice(e);
            const bool after_prev = c < prev_v || (c == prev_v && e > prev_i);
            if (after_prev && (bi < 0 || c > best)) { best = c; bi = e; }
        }
#pragma unroll
        for (int off = 16; off; off >>= 1) {
            const float ob = __shfl_xor_sync(full, best, off);
            const int oi = __shfl_xor_sync(full, bi, off);
            if (oi >= 0 && (bi < 0 || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
        }
        float w = 0.f;
        if (bi < 0) bi = 0; else w = zt[bi];                  // scores that are not numbers: keep the ids in range, weight 0
        if (lane == 0) { ids[k] = bi; wts[k] = w; }
        if (bi >= rr.real) idw += w;
        prev_v = best;
        prev_i = bi;
    }
    if (rest && lane == 0) *rest = idw;
}

// The `top` largest of zt[0 .. E) in order (ties: the lower index first) and the softmax over them.
__device__ __forceinline__ void route_one(const float* zt, int* ids, float* wts, int E, int top) {
    float prev_v = INFINITY;
    int prev_i = -1;
    float first = 0.f, sum = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int e = 0; e < E; ++e) {
            const float v = zt[e];
            const bool after_prev = v < prev_v || (v == prev_v && e > prev_i);      // not chosen yet
            if (after_prev && (bi < 0 || v > best)) { best = v; bi = e; }
        }
        if (bi < 0) { bi = 0; best = -INFINITY; }              // logits that are not numbers: keep the ids in range
        if (k == 0) first = best;
        const float p = expf(best - first);
        ids[k] = bi;
        wts[k] = p;
        sum += p;
        prev_v = best;
        prev_i = bi;
    }
    for (int k = 0; k < top; ++k) wts[k] /= sum;
}

__device__ __forceinline__ void route_by_rule(const float* zt, int* ids, float* wts, int E, int top, const RouteRule& rr, bool ready,
                                              int64_t t) {
    if (rr.mode == 1) { route_scored(zt, ids, wts, E, top, rr, ready, rr.rest ? rr.rest + t : nullptr); return; }
    route_one(zt, ids, wts, E, top);
    if (rr.mode == 2)                                          // the sigmoid keeps the logits' order: the same choice, other weights
        for (int k = 0; k < top; ++k) wts[k] = 1.0f / (1.0f + expf(-zt[ids[k]]));
    if (rr.rest) {
        float idw = 0.f;
        for (int k = 0; k < top; ++k) if (ids[k] >= rr.real) idw += wts[k];
        rr.rest[t] = idw;
    }
}

__global__ void moe_route_kernel(const float* __restrict__ z, int* __restrict__ ids, float* __restrict__ wts, int num_tokens, int E,
                                 int top, RouteRule rr) {
    pdl_enter();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= num_tokens) return;
    route_by_rule(z + (int64_t)t * E, ids + (int64_t)t * top, wts + (int64_t)t * top, E, top, rr, false, t);
}

#define ROUTER_TOKENS 8      // tokens a block: the router's matrix is read once for all of them
#define ROUTER_THREADS 512

// Column segments a row's dot product is cut into, so that a block's warps all have work when there are few outputs: a
// function of the sizes only (never of the batch), so a token's logits are summed in one order whatever runs beside it.
static __host__ __device__ inline int router_segments(int E, int h, int warps) {
    int S = 1;
    while (S < 8 && E * S < 4 * warps && (h + 2 * S - 1) / (2 * S) >= 128) S <<= 1;
    return S;
}

// A block per ROUTER_TOKENS tokens: their inputs into shared memory as float32, a warp per (output, column segment) in turn
// for the logits of all of them (the output's row is read once a block), the segments' sums added in their order, then a
// warp per token for the scores and, by the second rule, the choice (by the first rule a thread per token chooses).  `logits`
// (optional) receives z.
template <typename TA>
__global__ void __launch_bounds__(ROUTER_THREADS)
moe_router_kernel(const TA* __restrict__ x, const float* __restrict__ w, int* __restrict__ ids, float* __restrict__ wts,
                  float* __restrict__ logits, int num_tokens, int h, int E, int top, int tpb, int S, RouteRule rr) {
    extern __shared__ __align__(16) float rs[];               // x [tpb, h], then z [tpb, E], then the segments' sums [S, tpb, E]
    float* z = rs + (size_t)tpb * h;
    float* zp = z + (size_t)tpb * E;
    pdl_enter();
    const int t0 = blockIdx.x * tpb, nt = min(tpb, num_tokens - t0);
    const TA* xb = x + (int64_t)t0 * h;
    if (sizeof(TA) == 2 && (h & 7) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {      // eight inputs a load
        for (int c = threadIdx.x * 8; c < nt * h; c += blockDim.x * 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(xb) + c);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
            const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]), c2 = __bfloat1622float2(p[2]), d = __bfloat1622float2(p[3]);
            *reinterpret_cast<float4*>(rs + c) = make_float4(a.x, a.y, b.x, b.y);
            *reinterpret_cast<float4*>(rs + c + 4) = make_float4(c2.x, c2.y, d.x, d.y);
        }
    } else {
        for (int c = threadIdx.x; c < nt * h; c += blockDim.x) rs[c] = to_f32<TA>(xb[c]);
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const bool vec = (h & 3) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    const int seg = ((h + S - 1) / S + 127) / 128 * 128;      // columns a segment, whole 128-column steps
    for (int item = warp; item < E * S; item += nw) {
        const int e = item / S, s = item - e * S;
        const int c_begin = s * seg, c_end = min(h, c_begin + seg);
        const float* row = w + (int64_t)e * h;
        float acc[ROUTER_TOKENS];
#pragma unroll
        for (int i = 0; i < ROUTER_TOKENS; ++i) acc[i] = 0.f;
        if (vec) {
            for (int c0 = c_begin + lane * 4; c0 < c_end; c0 += 512) {           // four 16-byte loads of the row in flight
                float4 a[4];
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    a[u] = c0 + 128 * u < c_end ? *reinterpret_cast<const float4*>(row + c0 + 128 * u) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int c = c0 + 128 * u;
                    if (c >= c_end) break;
#pragma unroll
                    for (int i = 0; i < ROUTER_TOKENS; ++i)
                        if (i < nt) {
                            const float4 b = *reinterpret_cast<const float4*>(rs + (size_t)i * h + c);
                            acc[i] = fmaf(a[u].x, b.x, acc[i]); acc[i] = fmaf(a[u].y, b.y, acc[i]);
                            acc[i] = fmaf(a[u].z, b.z, acc[i]); acc[i] = fmaf(a[u].w, b.w, acc[i]);
                        }
                }
            }
        } else {
            for (int c = c_begin + lane; c < c_end; c += 32) {
                const float a = row[c];
#pragma unroll
                for (int i = 0; i < ROUTER_TOKENS; ++i)
                    if (i < nt) acc[i] = fmaf(a, rs[(size_t)i * h + c], acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < ROUTER_TOKENS; ++i) {
            const float v = warp_sum(acc[i]);
            if (lane == 0 && i < nt) zp[((size_t)s * tpb + i) * E + e] = v;
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < nt * E; c += blockDim.x) {
        float v = zp[c];
        for (int s = 1; s < S; ++s) v += zp[(size_t)s * tpb * E + c];
        z[c] = v;
    }
    __syncthreads();
    if (logits)
        for (int c = threadIdx.x; c < nt * E; c += blockDim.x) logits[(int64_t)t0 * E + c] = z[c];
    if (rr.mode == 1) {                          // the scores of all outputs, a warp per token: the choice then reads them
        __syncthreads();
        for (int i = warp; i < nt; i += nw) {
            float m = -INFINITY;
            for (int e = lane; e < E; e += 32) m = fmaxf(m, z[i * E + e]);
            m = warp_max(m);
            float sum = 0.f;
            for (int e = lane; e < E; e += 32) { const float p = expf(z[i * E + e] - m); z[i * E + e] = p; sum += p; }
            sum = warp_sum(sum);
            __syncwarp();
            for (int e = lane; e < E; e += 32) z[i * E + e] /= sum;
            __syncwarp();
            route_scored_warp(z + i * E, ids + (int64_t)(t0 + i) * top, wts + (int64_t)(t0 + i) * top, E, top, rr,
                              rr.rest ? rr.rest + t0 + i : nullptr, lane);
        }
        return;
    }
    if (threadIdx.x < nt)
        route_by_rule(z + threadIdx.x * E, ids + (int64_t)(t0 + threadIdx.x) * top, wts + (int64_t)(t0 + threadIdx.x) * top, E, top, rr,
                      false, t0 + threadIdx.x);
}

__device__ __forceinline__ float expert_act(float x, int kind) {
    if (kind == 0) { const float r = fmaxf(x, 0.f); return r * r; }
    if (kind == 1) return x / (1.0f + expf(-x));
    return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
}

// A gated expert's hidden value from its gate and up sums g, u and the token's weight w.  Kinds 0 - 2: w act(g) u.  Kind 3:
// the expert runs on the token times its weight (a factor on both sums), and the gate is clamped: with g' = min(w g, limit),
// u' = clamp(w u, -limit, limit) the value is g' sigmoid(1.702 g') (u' + 1), and nothing multiplies the output.
__device__ __forceinline__ float gated_value(float g, float u, float w, int kind, float limit) {
    if (kind != 3) return w * expert_act(g, kind) * u;
    g *= w; u *= w;
    if (limit > 0.f) { g = fminf(g, limit); u = fminf(fmaxf(u, -limit), limit); }
    return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}

template <typename T>
__global__ void moe_dense_act_kernel(const T* __restrict__ up, const int* __restrict__ ids, const float* __restrict__ wts,
                                     T* __restrict__ act, int64_t total, int E, int F, int top, int kind) {
    pdl_enter();
    const int64_t EF = (int64_t)E * F;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / EF;
        const int e = (int)((idx - t * EF) / F);
        float w = 0.f;
        for (int k = 0; k < top; ++k)
            if (ids[t * top + k] == e) w = wts[t * top + k];
        act[idx] = from_f32<T>(w != 0.f ? w * expert_act(to_f32<T>(up[idx]), kind) : 0.f);
    }
}

// Eight consecutive matrix entries as float32 (16 bytes of bfloat16, or two 16-byte loads of float32).
template <typename T> __device__ __forceinline__ void load8(const T* p, float* v);
template <> __device__ __forceinline__ void load8<bf16>(const bf16* p, float* v) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
template <> __device__ __forceinline__ void load8<float>(const float* p, float* v) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// The dot products of R matrix rows (`stride` entries apart, the last ones repeated past `rows`) of each of M matrices (`gap`
// entries apart) with one float32 vector in shared memory, added to acc[m * R + r]: U column steps of 256 entries are taken at a
// time, and all R * U * M 16-byte loads of a lane are issued before any is used, so a warp keeps that many in flight.  acc[] holds
// the lane's partial sums (a row's columns in their order); the caller adds the lanes up once a row.
template <typename TW, int R, int U, int M>
__device__ __forceinline__ void rows_dot(const TW* __restrict__ first, int64_t gap, int64_t stride, int rows, const float* __restrict__ x,
                                         int n, int lane, float* acc) {
    for (int c0 = lane * 8; c0 < n; c0 += 256 * U) {
        float w[M][R][U][8];
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int c = c0 + 256 * u;
                    if (c < n) load8<TW>(first + m * gap + (int64_t)min(r, rows - 1) * stride + c, w[m][r][u]);
                    else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) w[m][r][u][i] = 0.f;
                    }
                }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int c = c0 + 256 * u;
            if (c >= n) break;
            const float4 xa = *reinterpret_cast<const float4*>(x + c), xb = *reinterpret_cast<const float4*>(x + c + 4);
            const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
            for (int m = 0; m < M; ++m)
#pragma unroll
                for (int r = 0; r < R; ++r)
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[m * R + r] = fmaf(w[m][r][u][i], xv[i], acc[m * R + r]);
        }
    }
}

// n entries (a multiple of 8) of a row into shared memory as float32 by the whole block, 16 bytes a load where the row allows:
// a thread's loads do not depend on one another, so they are in flight together.
template <typename TA>
__device__ __forceinline__ void fill_f32(float* __restrict__ dst, const TA* __restrict__ src, int n) {
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        for (int c = threadIdx.x * 8; c < n; c += blockDim.x * 8) {
            float v[8];
            load8<TA>(src + c, v);
            *reinterpret_cast<float4*>(dst + c) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(dst + c + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    } else {
        for (int c = threadIdx.x; c < n; c += blockDim.x) dst[c] = to_f32<TA>(src[c]);
    }
}

// R rows a warp and U column steps at a time: (4, 1) where the batch gives every SM its fill of warps, (1, 4) for a handful of
// tokens, where more and narrower warps keep as many bytes in flight.  A row's sum runs over its columns in the same order
// either way, so the result does not depend on the choice.
template <typename TA, typename TW, int R, int U>
__global__ void moe_pairs_up_kernel(const TA* __restrict__ x, const TW* __restrict__ w_up, const int* __restrict__ ids,
                                    const float* __restrict__ wts, TA* __restrict__ hid, int h, int E, int F, int top, int kind,
                                    int gated, float limit) {
    extern __shared__ __align__(16) float xs[];               // the token's input, float32
    pdl_enter();
    const int pair = blockIdx.x, t = pair / top;
    const int e = ids[pair];
    const float weight = wts[pair];
    if (e >= E) return;                                        // an identity expert: the down kernel skips the pair
    fill_f32<TA>(xs, x + (int64_t)t * h, h);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int f0 = (blockIdx.y * nw + warp) * R, rows = min(R, F - f0);
    if (rows <= 0) return;
    float gu[2 * R];                                           // gate sums, then up sums
#pragma unroll
    for (int r = 0; r < 2 * R; ++r) gu[r] = 0.f;
    const TW* base = w_up + ((int64_t)e * (gated ? 2 : 1) * F + f0) * h;
    if (gated) rows_dot<TW, R, U, 2>(base, (int64_t)F * h, h, rows, xs, h, lane, gu);
    else rows_dot<TW, R, U, 1>(base, 0, h, rows, xs, h, lane, gu);
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float gs = warp_sum(gu[r]);
        const float v = gated ? gated_value(gs, warp_sum(gu[R + r]), weight, kind, limit) : weight * expert_act(gs, kind);
        if (lane == 0 && r < rows) hid[(int64_t)pair * F + f0 + r] = from_f32<TA>(v);
    }
}

template <typename TA, typename TW, int R, int U>
__global__ void moe_pairs_down_kernel(const TA* __restrict__ hid, const TW* __restrict__ w_down, const int* __restrict__ ids,
                                      float* __restrict__ out, int h, int E, int F, int top) {
    extern __shared__ __align__(16) float hs[];               // the token's `top` hidden rows, float32 [top, F]
    pdl_enter();
    const int t = blockIdx.x;
    for (int k = 0; k < top; ++k)                             // an identity expert's row is never read: the loop below skips it
        if (ids[t * top + k] < E) fill_f32<TA>(hs + k * F, hid + ((int64_t)t * top + k) * F, F);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int n0 = (blockIdx.y * nw + warp) * R, rows = min(R, h - n0);
    if (rows <= 0) return;
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.f;
    for (int k = 0; k < top; ++k) {                           // a lane's sums run over the choices in their order, then the lanes are added
        const int e = ids[t * top + k];
        if (e < E) rows_dot<TW, R, U, 1>(w_down + (int64_t)n0 * E * F + (int64_t)e * F, 0, (int64_t)E * F, rows, hs + k * F, F, lane, acc);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float v = warp_sum(acc[r]);
        if (lane == 0 && r < rows) out[(int64_t)t * h + n0 + r] = v;
    }
}

template <typename TA, typename TW, int R, int U>
static int launch_pairs_as(const void* x, const void* w_up, const void* w_down, const int* ids, const float* wts, void* hid, float* out,
                           int T, int h, int E, int F, int top, int kind, int gated, int threads, float limit, cudaStream_t stream) {
    const int rows = (threads / 32) * R;
    const size_t smem_up = (size_t)h * sizeof(float), smem_down = (size_t)top * F * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(moe_pairs_up_kernel<TA, TW, R, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_up);
    if (e != cudaSuccess) return (int)e;
    e = cudaFuncSetAttribute(moe_pairs_down_kernel<TA, TW, R, U>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_down);
    if (e != cudaSuccess) return (int)e;
    int rc = launch_kernel(moe_pairs_up_kernel<TA, TW, R, U>, dim3(T * top, (F + rows - 1) / rows), dim3(threads), smem_up, stream,
                           (const TA*)x, (const TW*)w_up, ids, wts, (TA*)hid, h, E, F, top, kind, gated, limit);
    if (rc != 0) return rc;
    return launch_kernel(moe_pairs_down_kernel<TA, TW, R, U>, dim3(T, (h + rows - 1) / rows), dim3(threads), smem_down, stream,
                         (const TA*)hid, (const TW*)w_down, ids, out, h, E, F, top);
}

template <typename TA, typename TW>
static int launch_pairs(const void* x, const void* w_up, const void* w_down, const int* ids, const float* wts, void* hid, float* out,
                        int T, int h, int E, int F, int top, int kind, int gated, float limit, cudaStream_t stream) {
    // fewer warps a block where a handful of tokens would leave SMs without one (the warps' work does not depend on it)
    const int threads = (int64_t)T * ((h + 31) / 32) < 2 * device_sm_count() ? 128 : 256;
    // the output rows of the smaller of the two products, four a warp: under 12 warps an SM the narrow form (measured at width
    // 2,048, four experts of 960 a token: one token 52 against 64 us, eight tokens 94 against 81 us)
    const int64_t quads = (int64_t)T * ((h < (int64_t)top * F ? h : top * F) / 4);
    if (quads < 12 * (int64_t)device_sm_count())
        return launch_pairs_as<TA, TW, 1, 4>(x, w_up, w_down, ids, wts, hid, out, T, h, E, F, top, kind, gated, threads, limit, stream);
    return launch_pairs_as<TA, TW, 4, 1>(x, w_up, w_down, ids, wts, hid, out, T, h, E, F, top, kind, gated, threads, limit, stream);
}

// Whether the pair kernels take these sizes: rows of whole 16-byte pieces, and a token's hidden rows within shared memory.
extern "C" int mie_moe_pairs_fit(int h, int F, int top) {
    return h % 8 == 0 && F % 8 == 0 && (size_t)h * sizeof(float) <= 200 * 1024 && (size_t)top * F * sizeof(float) <= 200 * 1024;
}

// x [T, h] and hid [T * top, F] in the activation type (act_tag), w_up [E * F, h] and w_down [h, E * F] in w_tag, out [T, h] float32.
extern "C" int mie_moe_pairs(const void* x, int act_tag, const void* w_up, const void* w_down, int w_tag, const int* ids, const float* wts,
                             void* hid, float* out, int num_tokens, int h, int E, int F, int top, int kind, int gated, float limit,
                             cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || kind < 0 || kind > 3 || (kind == 3 && !gated) || !mie_moe_pairs_fit(h, F, top)) return MIE_ERR_BAD_ARG;
    if (((reinterpret_cast<uintptr_t>(w_up) | reinterpret_cast<uintptr_t>(w_down)) & 15) != 0) return MIE_ERR_BAD_ARG;
    if (act_tag == MIE_F32 && w_tag == MIE_F32)
        return launch_pairs<float, float>(x, w_up, w_down, ids, wts, hid, out, num_tokens, h, E, F, top, kind, gated, limit, stream);
    if (act_tag == MIE_BF16 && w_tag == MIE_BF16)
        return launch_pairs<bf16, bf16>(x, w_up, w_down, ids, wts, hid, out, num_tokens, h, E, F, top, kind, gated, limit, stream);
    if (act_tag == MIE_BF16 && w_tag == MIE_F32)
        return launch_pairs<bf16, float>(x, w_up, w_down, ids, wts, hid, out, num_tokens, h, E, F, top, kind, gated, limit, stream);
    return MIE_ERR_BAD_ARG;
}

#define MOE_SORT_MAX_EXPERTS 1024

// One block.  ends[e] = one past the last sorted row of expert e (the running sum of the experts' pair counts);
// place[p] = the sorted row of pair p = (token p / top, choice p % top); row_weight[place[p]] = wts[p].  Which of an
// expert's rows a pair gets depends on the order the threads arrive in; no result depends on it, since every row is
// computed by itself and read back through place[].
__global__ void moe_sort_kernel(const int* __restrict__ ids, const float* __restrict__ wts, int* __restrict__ ends,
                                int* __restrict__ place, float* __restrict__ row_weight, int pairs, int E) {
    __shared__ int count[MOE_SORT_MAX_EXPERTS];
    __shared__ int start[MOE_SORT_MAX_EXPERTS];
    pdl_enter();
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[min(max(ids[p], 0), E - 1)], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) { start[e] = run; run += count[e]; ends[e] = run; }
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int at = atomicAdd(&start[min(max(ids[p], 0), E - 1)], 1);
        place[p] = at;
        row_weight[at] = wts[p];
    }
}

// rows[place[p]] = x[p / top] for every pair p; 16 bytes a thread where rows allow it.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, const int* __restrict__ place, T* __restrict__ rows, int pairs, int h,
                                  int top, int vec) {
    pdl_enter();
    const int per = 16 / (int)sizeof(T);
    const int n = vec ? h / per : h;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (int64_t)pairs * n; idx += (int64_t)gridDim.x * blockDim.x) {
        const int p = (int)(idx / n), c = (int)(idx - (int64_t)p * n);
        const T* src = x + (int64_t)(p / top) * h;
        T* dst = rows + (int64_t)place[p] * h;
        if (vec) reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
        else dst[c] = src[c];
    }
}

// up[r, :] <- row_weight[r] f(up[r, :]) in place.
template <typename T>
__global__ void moe_act_rows_kernel(T* __restrict__ up, const float* __restrict__ row_weight, int64_t total, int F, int kind) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x)
        up[idx] = from_f32<T>(row_weight[idx / F] * expert_act(to_f32<T>(up[idx]), kind));
}
__global__ void moe_act_rows_bf16x8_kernel(bf16* __restrict__ up, const float* __restrict__ row_weight, int64_t total8, int F8, int kind) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (int64_t)gridDim.x * blockDim.x) {
        const float w = row_weight[idx / F8];
        uint4 u = *reinterpret_cast<const uint4*>(up + idx * 8);
        __nv_bfloat162* hu = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(hu[i]);
            hu[i] = __floats2bfloat162_rn(w * expert_act(f.x, kind), w * expert_act(f.y, kind));
        }
        *reinterpret_cast<uint4*>(up + idx * 8) = u;
    }
}

// out[t, :] = sum over k < top of rows[place[t * top + k], :], float32, k in order.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, const int* __restrict__ place, float* __restrict__ out, int num_tokens,
                                   int h, int top, const int* __restrict__ ids, int real) {
    pdl_enter();
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (int64_t)num_tokens * h; idx += (int64_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / h), c = (int)(idx - (int64_t)t * h);
        float acc = 0.f;
        for (int k = 0; k < top; ++k)
            if (!ids || ids[t * top + k] < real) acc += to_f32<T>(rows[(int64_t)place[t * top + k] * h + c]);
        out[idx] = acc;
    }
}

// The same, eight bfloat16 a thread (16-byte loads, two 16-byte stores); h8 = h / 8.
__global__ void moe_combine_bf16x8_kernel(const bf16* __restrict__ rows, const int* __restrict__ place, float* __restrict__ out,
                                          int num_tokens, int h8, int top, const int* __restrict__ ids, int real) {
    pdl_enter();
    const int64_t total = (int64_t)num_tokens * h8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / h8), c = (int)(idx - (int64_t)t * h8);
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.f;
        for (int k = 0; k < top; ++k) {
            if (ids && ids[t * top + k] >= real) continue;
            const uint4 u = *reinterpret_cast<const uint4*>(rows + ((int64_t)place[t * top + k] * h8 + c) * 8);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(p[i]);
                acc[2 * i] += f.x;
                acc[2 * i + 1] += f.y;
            }
        }
        float4* o = reinterpret_cast<float4*>(out + idx * 8);
        o[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
        o[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
}

static int capped_blocks(int64_t items, int threads) {
    int64_t blocks = (items + threads - 1) / threads;
    if (blocks > (int64_t)device_sm_count() * 16) blocks = (int64_t)device_sm_count() * 16;
    return (int)(blocks < 1 ? 1 : blocks);
}

extern "C" int mie_moe_sort(const int* ids, const float* wts, int* ends, int* place, float* row_weight, int pairs, int E,
                            cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (E <= 0) return MIE_ERR_BAD_ARG;
    if (E > MOE_SORT_MAX_EXPERTS) return MIE_ERR_TOO_LARGE;
    return launch_kernel(moe_sort_kernel, dim3(1), dim3(1024), 0, stream, ids, wts, ends, place, row_weight, pairs, E);
}

extern "C" int mie_moe_gather(const void* x, const int* place, void* rows, int tag, int pairs, int h, int top, cudaStream_t stream) {
    if (pairs <= 0) return 0;
    if (h <= 0 || top <= 0) return MIE_ERR_BAD_ARG;
    const int el = tag == MIE_F32 ? 4 : 2;
    const int vec = (h * el) % 16 == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(rows)) & 15) == 0;
    const int64_t items = (int64_t)pairs * (vec ? h * el / 16 : h);
    if (tag == MIE_F32)
        return launch_kernel(moe_gather_kernel<float>, dim3(capped_blocks(items, 256)), dim3(256), 0, stream, (const float*)x, place,
                             (float*)rows, pairs, h, top, vec);
    else if (tag == MIE_BF16)
        return launch_kernel(moe_gather_kernel<bf16>, dim3(capped_blocks(items, 256)), dim3(256), 0, stream, (const bf16*)x, place,
                             (bf16*)rows, pairs, h, top, vec);
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_moe_act_rows(void* up, const float* row_weight, int tag, int rows, int F, int kind, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (F <= 0 || kind < 0 || kind > 2) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)rows * F;
    if (tag == MIE_BF16 && F % 8 == 0 && (reinterpret_cast<uintptr_t>(up) & 15) == 0)
        return launch_kernel(moe_act_rows_bf16x8_kernel, dim3(capped_blocks(total / 8, 256)), dim3(256), 0, stream, (bf16*)up, row_weight,
                             total / 8, F / 8, kind);
    if (tag == MIE_F32)
        return launch_kernel(moe_act_rows_kernel<float>, dim3(capped_blocks(total, 256)), dim3(256), 0, stream, (float*)up, row_weight, total, F, kind);
    else if (tag == MIE_BF16)
        return launch_kernel(moe_act_rows_kernel<bf16>, dim3(capped_blocks(total, 256)), dim3(256), 0, stream, (bf16*)up, row_weight, total, F, kind);
    return MIE_ERR_BAD_ARG;
}

// ids / real (optional): pairs whose expert id is `real` or more have no row to add (identity experts).
extern "C" int mie_moe_combine(const void* rows, const int* place, float* out, int tag, int num_tokens, int h, int top, const int* ids,
                               int real, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (h <= 0 || top <= 0) return MIE_ERR_BAD_ARG;
    const int64_t items = (int64_t)num_tokens * h;
    if (tag == MIE_BF16 && h % 8 == 0 && ((reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(out)) & 15) == 0)
        return launch_kernel(moe_combine_bf16x8_kernel, dim3(capped_blocks(items / 8, 256)), dim3(256), 0, stream, (const bf16*)rows, place,
                             out, num_tokens, h / 8, top, ids, real);
    if (tag == MIE_F32)
        return launch_kernel(moe_combine_kernel<float>, dim3(capped_blocks(items, 256)), dim3(256), 0, stream, (const float*)rows, place, out,
                             num_tokens, h, top, ids, real);
    else if (tag == MIE_BF16)
        return launch_kernel(moe_combine_kernel<bf16>, dim3(capped_blocks(items, 256)), dim3(256), 0, stream, (const bf16*)rows, place, out,
                             num_tokens, h, top, ids, real);
    return MIE_ERR_BAD_ARG;
}

static bool rule_ok(const RouteRule& rr, int E, int top) {
    if (rr.mode < 0 || rr.mode > 2) return false;
    if (rr.real < 0 || rr.real > E) return false;
    if (rr.mode == 1 && rr.groups > 1) {
        if (rr.groups > 64 || E % rr.groups || rr.keep < 1 || (rr.keep < rr.groups && top > rr.keep * (E / rr.groups))) return false;
    }
    return true;
}

extern "C" int mie_moe_router(const void* x, int tag, const float* w, int* ids, float* wts, float* logits, int num_tokens, int h, int E,
                              int top, int mode, const float* correction, int groups, int keep, int real, float* rest,
                              cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || h <= 0) return MIE_ERR_BAD_ARG;
    const RouteRule rr{mode, correction, groups, keep, real, rest};
    if (!rule_ok(rr, E, top)) return MIE_ERR_BAD_ARG;
    const int threads = ROUTER_THREADS;
    const int S = router_segments(E, h, threads / 32);
    int tpb = ROUTER_TOKENS;                                   // fewer where the tokens' inputs would not fit in 96 KB ...
    while (tpb > 1 && (size_t)tpb * (h + (S + 1) * E) * sizeof(float) > 96 * 1024) tpb >>= 1;
    while (tpb > 1 && (num_tokens + tpb - 1) / tpb < device_sm_count()) tpb >>= 1;      // ... or would leave SMs without a block
    const size_t smem = (size_t)tpb * (h + (S + 1) * E) * sizeof(float);
    if (smem > 200 * 1024) return MIE_ERR_TOO_LARGE;
    const int blocks = (num_tokens + tpb - 1) / tpb;
    cudaError_t e;
    if (tag == MIE_F32) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(moe_router_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_kernel(moe_router_kernel<float>, dim3(blocks), dim3(threads), smem, stream, (const float*)x, w, ids, wts, logits, num_tokens, h, E, top, tpb, S, rr);
    } else if (tag == MIE_BF16) {
        if (smem > 48 * 1024 && (e = cudaFuncSetAttribute(moe_router_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)) != cudaSuccess) return (int)e;
        return launch_kernel(moe_router_kernel<bf16>, dim3(blocks), dim3(threads), smem, stream, (const bf16*)x, w, ids, wts, logits, num_tokens, h, E, top, tpb, S, rr);
    }
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_moe_route(const float* z, int* ids, float* wts, int num_tokens, int E, int top, int mode, const float* correction,
                             int groups, int keep, int real, float* rest, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E) return MIE_ERR_BAD_ARG;
    const RouteRule rr{mode, correction, groups, keep, real, rest};
    if (!rule_ok(rr, E, top)) return MIE_ERR_BAD_ARG;
    const int threads = 64;
    return launch_kernel(moe_route_kernel, dim3((num_tokens + threads - 1) / threads), dim3(threads), 0, stream, z, ids, wts, num_tokens,
                         E, top, rr);
}

// The same, eight bfloat16 a thread; an expert the token did not choose is written as zeros without reading its inputs.
__global__ void moe_dense_act_bf16x8_kernel(const bf16* __restrict__ up, const int* __restrict__ ids, const float* __restrict__ wts,
                                            bf16* __restrict__ act, int64_t total8, int E, int F8, int top, int kind) {
    pdl_enter();
    const int64_t EF8 = (int64_t)E * F8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / EF8;
        const int e = (int)((idx - t * EF8) / F8);
        float w = 0.f;
        for (int k = 0; k < top; ++k)
            if (ids[t * top + k] == e) w = wts[t * top + k];
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (w != 0.f) {
            const uint4 u = *reinterpret_cast<const uint4*>(up + idx * 8);
            const __nv_bfloat162* hu = reinterpret_cast<const __nv_bfloat162*>(&u);
            __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(hu[i]);
                ho[i] = __floats2bfloat162_rn(w * expert_act(f.x, kind), w * expert_act(f.y, kind));
            }
        }
        *reinterpret_cast<uint4*>(act + idx * 8) = o;
    }
}

extern "C" int mie_moe_dense_act(const void* up, const int* ids, const float* wts, void* act, int tag, int num_tokens, int E, int F,
                                 int top, int kind, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (E <= 0 || F <= 0 || top <= 0 || kind < 0 || kind > 2) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)num_tokens * E * F;
    const int threads = 256;
    if (tag == MIE_BF16 && F % 8 == 0 && ((reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(act)) & 15) == 0) {
        int64_t blocks8 = (total / 8 + threads - 1) / threads;
        if (blocks8 > (int64_t)device_sm_count() * 16) blocks8 = (int64_t)device_sm_count() * 16;
        return launch_kernel(moe_dense_act_bf16x8_kernel, dim3((int)blocks8), dim3(threads), 0, stream, (const bf16*)up, ids, wts,
                             (bf16*)act, total / 8, E, F / 8, top, kind);
    }
    int64_t blocks = (total + threads - 1) / threads;
    if (blocks > (int64_t)device_sm_count() * 16) blocks = (int64_t)device_sm_count() * 16;
    if (tag == MIE_F32)
        return launch_kernel(moe_dense_act_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)up, ids, wts,
                             (float*)act, total, E, F, top, kind);
    else if (tag == MIE_BF16)
        return launch_kernel(moe_dense_act_kernel<bf16>, dim3((int)blocks), dim3(threads), 0, stream, (const bf16*)up, ids, wts,
                             (bf16*)act, total, E, F, top, kind);
    return MIE_ERR_BAD_ARG;
}

// Gated experts, the activation between the two products.  rows form: hid[r, f] = row_weight[r] f(gu[r, f]) gu[r, F + f] with
// gu [R, 2F] (the sorted pairs' rows); wide form: act[t, e, f] = weight(t, e) f(gu[t, e, f]) gu[t, e, F + f] for a chosen
// expert and 0 for the others, with gu [T, E, 2F].  `per_row` = 1 for the rows form (E = 1, the weight by row).
template <typename T>
__global__ void moe_glu_kernel(const T* __restrict__ gu, const int* __restrict__ ids, const float* __restrict__ wts, T* __restrict__ act,
                               int64_t total, int E, int F, int top, int kind, int per_row, float limit) {
    pdl_enter();
    const int64_t EF = (int64_t)E * F;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / EF;
        const int e = (int)((idx - t * EF) / F), f = (int)(idx - t * EF - (int64_t)e * F);
        float w = 0.f;
        if (per_row) w = wts[t];
        else
            for (int k = 0; k < top; ++k)
                if (ids[t * top + k] == e) w = wts[t * top + k];
        const int64_t at = (t * E + e) * 2 * F + f;
        act[idx] = from_f32<T>(w != 0.f ? gated_value(to_f32<T>(gu[at]), to_f32<T>(gu[at + F]), w, kind, limit) : 0.f);
    }
}
__global__ void moe_glu_bf16x8_kernel(const bf16* __restrict__ gu, const int* __restrict__ ids, const float* __restrict__ wts,
                                      bf16* __restrict__ act, int64_t total8, int E, int F8, int top, int kind, int per_row, float limit) {
    pdl_enter();
    const int64_t EF8 = (int64_t)E * F8;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t t = idx / EF8;
        const int e = (int)((idx - t * EF8) / F8), f8 = (int)(idx - t * EF8 - (int64_t)e * F8);
        float w = 0.f;
        if (per_row) w = wts[t];
        else
            for (int k = 0; k < top; ++k)
                if (ids[t * top + k] == e) w = wts[t * top + k];
        uint4 o = make_uint4(0u, 0u, 0u, 0u);
        if (w != 0.f) {
            const bf16* at = gu + ((t * E + e) * 2 * F8 + f8) * 8;
            const uint4 g = *reinterpret_cast<const uint4*>(at), u = *reinterpret_cast<const uint4*>(at + (int64_t)F8 * 8);
            const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&g);
            const __nv_bfloat162* hu = reinterpret_cast<const __nv_bfloat162*>(&u);
            __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 a = __bfloat1622float2(hg[i]), b = __bfloat1622float2(hu[i]);
                ho[i] = __floats2bfloat162_rn(gated_value(a.x, b.x, w, kind, limit), gated_value(a.y, b.y, w, kind, limit));
            }
        }
        *reinterpret_cast<uint4*>(act + idx * 8) = o;
    }
}

// gu [rows, E, 2F] -> act [rows, E, F]; per_row: E must be 1 and wts holds one weight a row (ids unused).
extern "C" int mie_moe_glu(const void* gu, const int* ids, const float* wts, void* act, int tag, int rows, int E, int F, int top, int kind,
                           int per_row, float limit, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (E <= 0 || F <= 0 || kind < 0 || kind > 3 || (per_row ? E != 1 : (top <= 0 || !ids))) return MIE_ERR_BAD_ARG;
    const int64_t total = (int64_t)rows * E * F;
    if (tag == MIE_BF16 && F % 8 == 0 && ((reinterpret_cast<uintptr_t>(gu) | reinterpret_cast<uintptr_t>(act)) & 15) == 0)
        return launch_kernel(moe_glu_bf16x8_kernel, dim3(capped_blocks(total / 8, 256)), dim3(256), 0, stream, (const bf16*)gu, ids, wts,
                             (bf16*)act, total / 8, E, F / 8, top, kind, per_row, limit);
    if (tag == MIE_F32)
        return launch_kernel(moe_glu_kernel<float>, dim3(capped_blocks(total, 256)), dim3(256), 0, stream, (const float*)gu, ids, wts,
                             (float*)act, total, E, F, top, kind, per_row, limit);
    else if (tag == MIE_BF16)
        return launch_kernel(moe_glu_kernel<bf16>, dim3(capped_blocks(total, 256)), dim3(256), 0, stream, (const bf16*)gu, ids, wts,
                             (bf16*)act, total, E, F, top, kind, per_row, limit);
    return MIE_ERR_BAD_ARG;
}
