// Linear attention with a fixed decay per head and no softmax or denominator, as a recurrence over a
// float32 state per request and head (prompt portions and single tokens through the same kernels):
//
//   S_t = gamma_h * S_{t-1} + k_t v_t^T        S: [D, Dv],  S before a request's first token is zero
//   o_t = S_t^T q_t
//
// q and k come from the fused projection [ q: H x D | k: H x D | v: H x Dv | ... ], are rotated (rotate-half pairing
// over the first `rot` dims, angle = position * freq[i], float32) and k is multiplied by `k_scale` after the
// rotation: the `prepare` kernel, one block per token, writes both as float32 [T, H, D]; a token's cosines and sines
// are computed once and serve all heads.  The state lives in `state[slot, h, c, d]` (value column c, key dimension
// d: transposed, so that the threads that share a column read neighbouring words).
//
// A request's new tokens are cut into chunks of RET_L.  The recurrence is linear in S, so a chunk's effect on the
// state is (gamma^len, the state it builds from zero), and the chunks of a long portion run side by side:
//   pass 0   every chunk j but the last of a row of two or more: the state it builds from zero     -> scratch[j + 1]
//   combine  per such row, in order: scratch[0] = the request's state, scratch[j + 1] += gamma^RET_L * scratch[j]
//   pass 1   every chunk from its start (scratch[j]; the request's state for a row of one chunk): outputs; a row's
//            last chunk stores the state (no block reads the state of a row whose other blocks may write it)
// A step whose rows all fit one chunk (decoding) runs pass 1 only.  Blocks find their (row, chunk) from the rows'
// lengths on the device, so the launch is laid out for the step's token count, not for what the host knows of its rows.
//
// Work split of a pass: one block = one chunk, one head and a slice of value columns (one or two a thread).  A column's state is held in
// the registers of P threads of one warp (thread p holds the key dimensions 4 (p + P j) .. 4 (p + P j) + 3, j = 0 ..:
// RET_DPT of them, read from shared memory as float4), which add up their parts of o_t by shuffles.  Tokens are staged in shared memory RET_TT at a time.
// Everything is float32.
//
// The last kernel finishes the mixer's head stage: every head's o is divided by its root mean square (no
// weight) and multiplied by silu(g), g being another part of the fused projection.
#include "common.cuh"

#define RET_DPT 16      // key dimensions per thread
#define RET_TT 16       // tokens staged at a time
#define RET_L 64        // tokens per chunk

// `act` 1: q and k pass silu first (a linear attention over activated projections).  `q_scale` multiplies q; `k_tok`
// (optional, [T, H] float32) is one more factor on a token's key per head (a write gate folded into the key).
template <typename T>
__global__ void retention_prepare_kernel(const T* __restrict__ qkv, int64_t stride, const int* __restrict__ positions,
                                         const float* __restrict__ freq, float k_scale, float* __restrict__ qr,
                                         float* __restrict__ kr, int H, int D, int rot, int act, float q_scale,
                                         const float* __restrict__ k_tok) {
    extern __shared__ float cs[];                 // cos [rot/2], sin [rot/2]
    pdl_enter();
    const int t = blockIdx.x, half = rot >> 1;
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float a = pos * freq[i];
        cs[i] = cosf(a);
        cs[half + i] = sinf(a);
    }
    __syncthreads();
    const T* src = qkv + (int64_t)t * stride;
    for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
        const int d = i % D;
        float qo = to_f32<T>(src[i]), ko = to_f32<T>(src[H * D + i]);
        if (act) { qo = qo / (1.0f + expf(-qo)); ko = ko / (1.0f + expf(-ko)); }
        if (d < rot) {
            const int j = d < half ? d : d - half;
            const int pi = d < half ? i + half : i - half;
            const float c = cs[j], sn = cs[half + j];
            const float qp = to_f32<T>(src[pi]), kp = to_f32<T>(src[H * D + pi]);
            qo = d < half ? qo * c - qp * sn : qo * c + qp * sn;
            ko = d < half ? ko * c - kp * sn : ko * c + kp * sn;
        }
        qr[(int64_t)t * H * D + i] = qo * q_scale;
        kr[(int64_t)t * H * D + i] = ko * (k_tok ? k_scale * k_tok[(int64_t)t * H + i / D] : k_scale);
    }
}

// Which (row, chunk) has number `index`, counting every row's chunks (numbering 1: max(1, ceil(len / RET_L)) a row) or
// only the chunks of rows that have two or more (numbering 0: these have a scratch slot each).  Returns the row (-1: none), the chunk within the row, the row's
// count in that numbering, and how many chunks of numbering 0 lie in front of the row.  Asked by whole warps.
__device__ __forceinline__ int find_chunk(const int* __restrict__ row_q_len, int num_rows, int index, int numbering,
                                          int& within, int& items, int& before0) {
    const int lane = threadIdx.x & 31;
    int seen0 = 0;
    for (int base = 0; base < num_rows; base += 32) {
        const int r = base + lane;
        const int n1 = r < num_rows ? max(1, (row_q_len[r] + RET_L - 1) / RET_L) : 0;
        const int n0 = n1 > 1 ? n1 : 0;
        const int n = numbering ? n1 : n0;
        int incl = n, incl0 = n0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o), up0 = __shfl_up_sync(0xffffffffu, incl0, o);
            if (lane >= o) { incl += up; incl0 += up0; }
        }
        const int total = __shfl_sync(0xffffffffu, incl, 31), total0 = __shfl_sync(0xffffffffu, incl0, 31);
        if (index < total) {
            const int l = __ffs(__ballot_sync(0xffffffffu, incl > index)) - 1;
            items = __shfl_sync(0xffffffffu, n, l);
            within = index - (__shfl_sync(0xffffffffu, incl, l) - items);
            before0 = seen0 + __shfl_sync(0xffffffffu, incl0, l) - __shfl_sync(0xffffffffu, n0, l);
            return base + l;
        }
        index -= total;
        seen0 += total0;
    }
    within = 0; items = 0; before0 = 0;
    return -1;
}

template <typename T, int PASS, int P, int NC>
__global__ void retention_chunk_kernel(const float* __restrict__ qr, const float* __restrict__ kr, const T* __restrict__ v,
                                       int64_t v_stride, const int* __restrict__ row_q_start,
                                       const int* __restrict__ row_q_len, const int* __restrict__ state_slots,
                                       const float* __restrict__ decay, float* __restrict__ state,
                                       float* __restrict__ scratch, float* __restrict__ out, int num_rows, int H, int D, int Dv,
                                       int CW, int slices, const float* __restrict__ tok_decay, float* __restrict__ chunk_decay,
                                       int Dv_in, int v_act) {
    // `tok_decay` (optional, [T, H]): the decay of every token instead of one per head; pass 0 then leaves the product of
    // a chunk's decays in `chunk_decay` for the combine.  `Dv_in` < Dv: v has Dv_in columns a head and the state's column
    // Dv_in is fed with ones (the sum of the keys under the same decays: a normalizer).  `v_act`: v passes silu.
    constexpr int DPAD = P * RET_DPT;        // key dimensions as the threads of a column hold them: D padded with zeros
    extern __shared__ float smem[];
    float* q_s = smem;                       // [RET_TT][DPAD]
    float* k_s = q_s + RET_TT * DPAD;        // [RET_TT][DPAD]
    float* v_s = k_s + RET_TT * DPAD;        // [RET_TT][CW]
    float* a_s = v_s + RET_TT * CW;          // [RET_TT] the tokens' decays
    pdl_enter();
    int within, items, before0;
    const int r = find_chunk(row_q_len, num_rows, (int)blockIdx.y, PASS, within, items, before0);
    if (r < 0 || (PASS == 0 && within == items - 1)) return;          // nobody needs what a row's last chunk builds from zero
    const int h = blockIdx.x / slices, slice = blockIdx.x - h * slices;
    const int q_len = row_q_len[r], q_start = row_q_start[r];
    const int t_lo = within * RET_L, t_hi = min(q_len, t_lo + RET_L);
    // a thread holds NC value columns, CW / NC apart (the key and query it reads from shared memory serve all of them)
    const int p = threadIdx.x % P, cl = threadIdx.x / P, cstep = CW / NC;
    const float gamma = decay ? decay[h] : 1.f;
    const int64_t per_state = (int64_t)H * Dv * D;
    int c[NC];
    bool col_ok[NC];
    int64_t hcol[NC];
    float S[NC][RET_DPT];
    // pass 0 builds from zero; pass 1 starts from the request's state or from what the combine left for this chunk
    const float* from = PASS == 0 ? nullptr : (items == 1 ? state + (int64_t)state_slots[r] * per_state
                                                           : scratch + (int64_t)(before0 + within) * per_state);
#pragma unroll
    for (int n = 0; n < NC; ++n) {
        c[n] = slice * CW + cl + n * cstep;
        col_ok[n] = cl < cstep && c[n] < Dv;
        hcol[n] = ((int64_t)h * Dv + (col_ok[n] ? c[n] : 0)) * D;
#pragma unroll
        for (int j = 0; j < RET_DPT; ++j) {
            const int d = 4 * (p + P * (j >> 2)) + (j & 3);
            S[n][j] = (from && col_ok[n] && d < D) ? from[hcol[n] + d] : 0.f;
        }
    }
    // S[4 j4 + e] is key dimension 4 (p + P j4) + e: a thread reads its dimensions of a token as RET_DPT / 4 float4,
    // the P threads of a column 16 P contiguous bytes at a time, at offsets known at compile time
    const float4* k_mine = reinterpret_cast<const float4*>(k_s) + p;
    const float4* q_mine = reinterpret_cast<const float4*>(q_s) + p;
    const float* v_mine = v_s + (cl < cstep ? cl : 0);
    for (int t0 = t_lo; t0 < t_hi; t0 += RET_TT) {
        const int nt = min(RET_TT, t_hi - t0);
        __syncthreads();
        const int64_t row0 = ((int64_t)(q_start + t0) * H + h) * D;
        for (int i = threadIdx.x; i < nt * DPAD; i += blockDim.x) {
            const int tt = i / DPAD, d = i % DPAD;
            k_s[i] = d < D ? kr[row0 + (int64_t)tt * H * D + d] : 0.f;
            if (PASS) q_s[i] = d < D ? qr[row0 + (int64_t)tt * H * D + d] : 0.f;
        }
        for (int i = threadIdx.x; i < nt * CW; i += blockDim.x) {
            const int tt = i / CW, cc = i - tt * CW;
            const int col = slice * CW + cc;
            float vv = 0.f;
            if (col < Dv_in) {
                vv = to_f32<T>(v[(int64_t)(q_start + t0 + tt) * v_stride + h * Dv_in + col]);
                if (v_act) vv = vv / (1.0f + expf(-vv));
            } else if (col < Dv) vv = 1.0f;
            v_s[i] = vv;
        }
        if (threadIdx.x < nt) a_s[threadIdx.x] = tok_decay ? tok_decay[(int64_t)(q_start + t0 + threadIdx.x) * H + h] : gamma;
        __syncthreads();
        float* o_ptr = out + (int64_t)(q_start + t0) * H * Dv + h * Dv;
        for (int tt = 0; tt < nt; ++tt) {
            float vv[NC], acc0[NC], acc1[NC];
            const float gamma_t = a_s[tt];
#pragma unroll
            for (int n = 0; n < NC; ++n) { vv[n] = v_mine[tt * CW + n * cstep]; acc0[n] = 0.f; acc1[n] = 0.f; }
            const float4* kt = k_mine + tt * (DPAD / 4);
            const float4* qt = q_mine + tt * (DPAD / 4);
#pragma unroll
            for (int j4 = 0; j4 < RET_DPT / 4; ++j4) {              // padded dimensions hold zeros and stay zero
                const float4 kk = kt[P * j4];
                float4 qq = make_float4(0.f, 0.f, 0.f, 0.f);
                if (PASS) qq = qt[P * j4];
#pragma unroll
                for (int n = 0; n < NC; ++n) {
                    S[n][4 * j4 + 0] = fmaf(gamma_t, S[n][4 * j4 + 0], kk.x * vv[n]);
                    S[n][4 * j4 + 1] = fmaf(gamma_t, S[n][4 * j4 + 1], kk.y * vv[n]);
                    S[n][4 * j4 + 2] = fmaf(gamma_t, S[n][4 * j4 + 2], kk.z * vv[n]);
                    S[n][4 * j4 + 3] = fmaf(gamma_t, S[n][4 * j4 + 3], kk.w * vv[n]);
                    if (PASS) {
                        acc0[n] = fmaf(S[n][4 * j4 + 0], qq.x, acc0[n]);
                        acc1[n] = fmaf(S[n][4 * j4 + 1], qq.y, acc1[n]);
                        acc0[n] = fmaf(S[n][4 * j4 + 2], qq.z, acc0[n]);
                        acc1[n] = fmaf(S[n][4 * j4 + 3], qq.w, acc1[n]);
                    }
                }
            }
            if (PASS) {
#pragma unroll
                for (int n = 0; n < NC; ++n) {
                    float acc = acc0[n] + acc1[n];
#pragma unroll
                    for (int o = P >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
                    if (p == 0 && col_ok[n]) o_ptr[(int64_t)tt * H * Dv + c[n]] = acc;
                }
            }
        }
    }
    if (PASS == 0 && tok_decay && slice == 0 && threadIdx.x == 0) {      // what this chunk does to the state it starts from
        float prod = 1.f;
        for (int t = t_lo; t < t_hi; ++t) prod *= tok_decay[(int64_t)(q_start + t) * H + h];
        chunk_decay[(int64_t)(before0 + within + 1) * H + h] = prod;
    }
    float* to = PASS == 0 ? scratch + (int64_t)(before0 + within + 1) * per_state
                          : (within == items - 1 ? state + (int64_t)state_slots[r] * per_state : nullptr);
    if (to) {
#pragma unroll
        for (int n = 0; n < NC; ++n) {
            if (!col_ok[n]) continue;
#pragma unroll
            for (int j = 0; j < RET_DPT; ++j) {
                const int d = 4 * (p + P * (j >> 2)) + (j & 3);
                if (d < D) to[hcol[n] + d] = S[n][j];
            }
        }
    }
}

// scratch[j] becomes the state at the start of chunk j, for every row with two chunks or more.  One thread per state
// entry; every thread walks the rows (their lengths are the same few cached words for all) and, for a long row, the
// row's chunks in order, eight loads ahead of the dependent multiply-adds.
__global__ void retention_combine_kernel(const int* __restrict__ row_q_len, const int* __restrict__ state_slots,
                                         const float* __restrict__ decay, const float* __restrict__ state,
                                         float* __restrict__ scratch, int num_rows, int H, int Dv, int D,
                                         const float* __restrict__ chunk_decay) {
    pdl_enter();
    const int64_t per_state = (int64_t)H * Dv * D;
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= per_state) return;
    const int h = (int)(e / ((int64_t)Dv * D));
    const float g_head = chunk_decay ? 0.f : exp2f((float)RET_L * log2f(decay[h]));      // (decay may be null with token decays)
    int before0 = 0;
    for (int r = 0; r < num_rows; ++r) {
        const int items = (row_q_len[r] + RET_L - 1) / RET_L;
        if (items < 2) continue;
        float cur = state[(int64_t)state_slots[r] * per_state + e];
        float* slot = scratch + (int64_t)before0 * per_state + e;
        slot[0] = cur;
        for (int j0 = 1; j0 < items; j0 += 8) {
            float add[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) add[k] = j0 + k < items ? slot[(int64_t)(j0 + k) * per_state] : 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (j0 + k < items) {
                    const float g = chunk_decay ? chunk_decay[(int64_t)(before0 + j0 + k) * H + h] : g_head;
                    cur = fmaf(g, cur, add[k]);
                    slot[(int64_t)(j0 + k) * per_state] = cur;
                }
        }
        before0 += items;
    }
}

// out[t, h, :] = o[t, h, :] * rsqrt(mean(o[t, h, :]^2) + eps) * silu(g[t, h, :]); a warp per (token, head)
template <typename T>
__global__ void head_rms_gate_kernel(const float* __restrict__ o, const T* __restrict__ g, int64_t g_stride, T* __restrict__ out,
                                     int num_tokens, int H, int Dv, float eps) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)num_tokens * H) return;
    const int64_t t = item / H;
    const int h = (int)(item - t * H);
    const float* src = o + item * Dv;
    float ss = 0.f;
    for (int i = lane; i < Dv; i += 32) { const float v = src[i]; ss += v * v; }
    const float s = 1.0f / sqrtf(warp_sum(ss) / (float)Dv + eps);
    const T* gate = g + t * g_stride + h * Dv;
    for (int i = lane; i < Dv; i += 32) {
        const float z = to_f32<T>(gate[i]);
        out[item * Dv + i] = from_f32<T>(src[i] * s * (z / (1.0f + expf(-z))));
    }
}

// The general entry.  `rows_in` holds [ q: H x D | k: H x D | v: H x Dv_in | ... ] per token.  `act`: q, k and v pass silu
// (no rotation then).  `tok_decay` / `k_tok` (optional, float32 [T, H]): a decay and a factor on the key per token and head,
// in place of `decay` [H].  `ones`: the state and the output have one more column per head, Dv_in + 1 in all, fed with ones.
// state [slots, H, Dv, D], out [T, H, Dv] with Dv = Dv_in + ones; `chunk_decay`: scratch of (scratch_chunks + 1) * H floats.
extern "C" int mie_decay_scan(const void* qkv, int tag, long long stride, const int* positions, const int* row_q_start,
                              const int* row_q_len, const int* state_slots, const float* decay, const float* freq,
                              float q_scale, float k_scale, const float* tok_decay, const float* k_tok, int act, int ones,
                              float* state, float* qr, float* kr, float* scratch, long long scratch_chunks, float* chunk_decay,
                              float* out, int num_tokens, int num_rows, int max_q_len, int H, int D, int Dv_in, int rot,
                              cudaStream_t stream) {
    if (num_rows <= 0 || num_tokens <= 0) return 0;
    if (H <= 0 || D <= 0 || Dv_in <= 0 || rot < 0 || rot > D || (rot & 1) || (act && rot) || (!decay && !tok_decay) || ones < 0 || ones > 1)
        return MIE_ERR_BAD_ARG;
    const int Dv = Dv_in + ones;
    int P = 1;
    while (P * RET_DPT < D) P <<= 1;
    if (P > 32) return MIE_ERR_TOO_LARGE;                      // key dimensions beyond 32 x RET_DPT
    // Value columns a thread.  Pass 0 (no outputs): two where the head has enough of them to fill 256 threads that way --
    // its shared-memory reads of k then serve twice the multiply-adds (107 -> 90 us at 8 heads of 128 x 256, 2,048
    // tokens).  Pass 1 stays with one: with two it takes 72 registers, three blocks an SM instead of six, and was
    // measured slower (188 -> 231 us).  The state's layout does not depend on how a pass cuts the columns.
    struct Cut { int NC, CW, slices, threads; size_t smem; };
    auto cut = [&](int nc) {
        Cut c;
        c.NC = nc;
        c.CW = nc * (256 / P);                                 // columns a block
        if (c.CW > Dv) c.CW = Dv;
        if (nc == 2 && (c.CW & 1)) c.CW += 1;                  // two columns a thread: an even count (the odd one out is masked)
        c.slices = (Dv + c.CW - 1) / c.CW;
        c.threads = (c.CW / nc * P + 31) / 32 * 32;
        c.smem = (size_t)RET_TT * (2 * P * RET_DPT + c.CW + 1) * sizeof(float);
        return c;
    };
    const Cut cut0 = cut(Dv >= 2 * (256 / P) ? 2 : 1), cut1 = cut(1);
    // chunks the step can have at most: every row one, and one more per RET_L tokens; those of rows with two or more
    // (such a row has more than RET_L tokens): two per RET_L tokens
    const int chunks1 = num_rows + num_tokens / RET_L, chunks0 = max_q_len > RET_L ? 2 * (num_tokens / RET_L) : 0;
    if (chunks0 > scratch_chunks) return MIE_ERR_BAD_ARG;
    if (chunks0 > 0 && tok_decay && !chunk_decay) return MIE_ERR_BAD_ARG;
    float* cdec = tok_decay ? chunk_decay : nullptr;
    const int prep_threads = H * D >= 1024 ? 256 : 128;
    int rc;
#define RET_PASS(T, PASS, PP, ny)                                                                                             \
    ((PASS == 0 && cut0.NC == 2) ? RET_PASS_N(T, 0, PP, 2, ny, cut0) : RET_PASS_N(T, PASS, PP, 1, ny, (PASS == 0 ? cut0 : cut1)))
#define RET_PASS_N(T, PASS, PP, NN, ny, CUT)                                                                                  \
    launch_kernel(retention_chunk_kernel<T, PASS, PP, NN>, dim3(H * CUT.slices, ny), dim3(CUT.threads), CUT.smem, stream, qr, \
                  kr, (const T*)qkv + 2 * H * D, (int64_t)stride, row_q_start, row_q_len, state_slots, decay, state, scratch, \
                  out, num_rows, H, D, Dv, CUT.CW, CUT.slices, tok_decay, cdec, Dv_in, act)
#define RET_PASS_P(T, PASS, ny)                                                                                               \
    (P == 1 ? RET_PASS(T, PASS, 1, ny) : P == 2 ? RET_PASS(T, PASS, 2, ny) : P == 4 ? RET_PASS(T, PASS, 4, ny)                \
     : P == 8 ? RET_PASS(T, PASS, 8, ny) : P == 16 ? RET_PASS(T, PASS, 16, ny) : RET_PASS(T, PASS, 32, ny))
#define RET_LAUNCH(T)                                                                                                         \
    rc = launch_kernel(retention_prepare_kernel<T>, dim3(num_tokens), dim3(prep_threads), (size_t)rot * sizeof(float), stream, \
                       (const T*)qkv, (int64_t)stride, positions, freq, k_scale, qr, kr, H, D, rot, act, q_scale, k_tok);     \
    if (rc) return rc;                                                                                                        \
    if (chunks0 > 0) {                                                                                                        \
        rc = RET_PASS_P(T, 0, chunks0);                                                                                       \
        if (rc) return rc;                                                                                                    \
        rc = launch_kernel(retention_combine_kernel, dim3((unsigned)(((int64_t)H * Dv * D + 255) / 256)), dim3(256), 0, stream, \
                           row_q_len, state_slots, decay, (const float*)state, scratch, num_rows, H, Dv, D, (const float*)cdec); \
        if (rc) return rc;                                                                                                    \
    }                                                                                                                         \
    return RET_PASS_P(T, 1, chunks1);
    if (tag == MIE_F32) { RET_LAUNCH(float) }
    else if (tag == MIE_BF16) { RET_LAUNCH(bf16) }
#undef RET_LAUNCH
#undef RET_PASS_P
#undef RET_PASS
#undef RET_PASS_N
    return MIE_ERR_BAD_ARG;
}

extern "C" int mie_retention_scan(const void* qkv, int tag, long long stride, const int* positions, const int* row_q_start,
                                  const int* row_q_len, const int* state_slots, const float* decay, const float* freq,
                                  float k_scale, float* state, float* qr, float* kr, float* scratch, long long scratch_chunks,
                                  float* out, int num_tokens, int num_rows, int max_q_len, int H, int D, int Dv, int rot,
                                  cudaStream_t stream) {
    return mie_decay_scan(qkv, tag, stride, positions, row_q_start, row_q_len, state_slots, decay, freq, 1.0f, k_scale, nullptr, nullptr,
                          0, 0, state, qr, kr, scratch, scratch_chunks, nullptr, out, num_tokens, num_rows, max_q_len, H, D, Dv, rot,
                          stream);
}

extern "C" int mie_retention_chunk_tokens() { return RET_L; }

extern "C" int mie_head_rms_gate(const float* o, const void* g, int tag, long long g_stride, void* out, int num_tokens, int H,
                                 int Dv, float eps, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (H <= 0 || Dv <= 0) return MIE_ERR_BAD_ARG;
    const int warps = 4;
    const int64_t items = (int64_t)num_tokens * H;
    const int blocks = (int)((items + warps - 1) / warps);
    if (tag == MIE_F32)
        return launch_kernel(head_rms_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o, (const float*)g,
                             (int64_t)g_stride, (float*)out, num_tokens, H, Dv, eps);
    else if (tag == MIE_BF16)
        return launch_kernel(head_rms_gate_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, o, (const bf16*)g,
                             (int64_t)g_stride, (bf16*)out, num_tokens, H, Dv, eps);
    return MIE_ERR_BAD_ARG;
}

// ---------------------------------------------------------------------------------------------------------------------
// Exponential gates with a running maximum, for a matrix memory whose decay and write strength change with the token
// (the scan above then runs with `tok_decay` = keep and `k_tok` = write):
//   i_t = cap tanh((zi_t + bi) / cap)          f_t = logsigmoid(cap tanh((zf_t + bf) / cap))        (cap <= 0: no cap)
//   m_t = max(f_t + m_{t-1}, i_t)              keep_t = exp(f_t + m_{t-1} - m_t)      write_t = exp(i_t - m_t)
// z [T, 2H] float32 holds [zi: H | zf: H] per token; m_state [slots, H] carries m between steps (0 for a fresh request).
// A warp per (row, head) takes 32 tokens at a time: with L_j the sum of f over the tile up to token j and m_c the maximum carried
// into the tile, m_j - L_j = max(m_c, max over s <= j of (i_s - L_s)), so a prefix sum and a prefix maximum by shuffles give all 32
// maxima at once, and the sums never run over more than a tile (no large numbers are subtracted from one another).
__global__ void gate_scan_kernel(const float* __restrict__ z, const float* __restrict__ bi, const float* __restrict__ bf, float cap,
                                 const int* __restrict__ row_q_start, const int* __restrict__ row_q_len,
                                 const int* __restrict__ state_slots, float* __restrict__ m_state, float* __restrict__ keep,
                                 float* __restrict__ write, float* __restrict__ m_out, int num_rows, int H) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= num_rows * H) return;
    const int r = item / H, h = item - r * H;
    const int start = row_q_start[r], len = row_q_len[r];
    float* ms = m_state + (int64_t)state_slots[r] * H + h;
    float m_c = *ms;
    const float b_i = bi ? bi[h] : 0.f, b_f = bf ? bf[h] : 0.f, inv = cap > 0.f ? 1.0f / cap : 0.f;
    // four tiles' pre-activations are loaded before the first of them is scanned: the loads of a tile would otherwise stand
    // in front of every tile's chain
    for (int t00 = 0; t00 < len; t00 += 128) {
        float zi4[4], zf4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int tt = t00 + 32 * k + lane;
            const int64_t t = start + tt;
            zi4[k] = tt < len ? z[t * 2 * H + h] : 0.f;
            zf4[k] = tt < len ? z[t * 2 * H + H + h] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int t0 = t00 + 32 * k;
            if (t0 >= len) break;
            const bool ok = t0 + lane < len;
            const int64_t t = start + t0 + lane;
            float gi = -INFINITY, f = 0.f;                         // lanes beyond the row: nothing is written, nothing forgotten
            if (ok) {
                float zi = zi4[k] + b_i, zf = zf4[k] + b_f;
                if (cap > 0.f) { zi = cap * tanhf(zi * inv); zf = cap * tanhf(zf * inv); }
                gi = zi;
                f = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));     // log sigmoid
            }
            float L = f;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const float up = __shfl_up_sync(0xffffffffu, L, o); if (lane >= o) L += up; }
            const float own = gi - L;
            float a = own;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) { const float up = __shfl_up_sync(0xffffffffu, a, o); if (lane >= o) a = fmaxf(a, up); }
            // u_j = m_j - L_j never falls, and f_j + m_{j-1} - m_j = u_{j-1} - u_j: where a token only forgets, its keep factor is
            // exactly 1, and where it sets the maximum, its write factor is; no difference of large sums enters a factor that the
            // state multiplies up over many tokens
            const float u = fmaxf(m_c, a);
            float u_prev = __shfl_up_sync(0xffffffffu, u, 1);
            if (lane == 0) u_prev = m_c;
            const float m = L + u;
            if (ok) {
                keep[t * H + h] = expf(u_prev - u);
                write[t * H + h] = expf(own - u);
                m_out[t * H + h] = m;
            }
            m_c = __shfl_sync(0xffffffffu, m, min(31, len - t0 - 1));
        }
    }
    if (lane == 0) *ms = m_c;
}

extern "C" int mie_gate_scan(const float* z, const float* bi, const float* bf, float cap, const int* row_q_start, const int* row_q_len,
                             const int* state_slots, float* m_state, float* keep, float* write, float* m_out, int num_rows, int H,
                             cudaStream_t stream) {
    if (num_rows <= 0) return 0;
    if (H <= 0) return MIE_ERR_BAD_ARG;
    const int items = num_rows * H, warps = 2;
    return launch_kernel(gate_scan_kernel, dim3((items + warps - 1) / warps), dim3(warps * 32), 0, stream, z, bi, bf, cap, row_q_start,
                         row_q_len, state_slots, m_state, keep, write, m_out, num_rows, H);
}

// What follows a linear-attention scan in several mixers, as one kernel: o [T, groups, stride] float32 holds `size` outputs per
// group (stride >= size; with `normalizer` the entry behind them is n . q and `m` [T, groups] the running maximum: the group is
// first divided by max(|n . q|, exp(-m)) + 1e-6); each group is divided by its root mean square (eps inside the root),
// multiplied by a weight (`w_len` entries, indexed by the output's place in the row modulo w_len: one weight per head, or one
// for the whole row; null: none) and by a gate read from `gate` (sigmoid, or silu with `gate_silu`).  groups = 1 norms the
// whole row at once.  A warp per (token, group).
template <typename T>
__global__ void group_norm_gate_kernel(const float* __restrict__ o, int stride, const float* __restrict__ m, const float* __restrict__ w,
                                       int w_len, const T* __restrict__ gate, int64_t g_stride, T* __restrict__ out, int num_tokens,
                                       int groups, int size, float eps, int normalizer, int gate_silu) {
    pdl_enter();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)num_tokens * groups) return;
    const int64_t t = item / groups;
    const int g = (int)(item - t * groups);
    const float* src = o + item * stride;
    float scale = 1.f;
    if (normalizer) scale = 1.0f / (fmaxf(fabsf(src[size]), expf(-m[item])) + 1e-6f);
    float ss = 0.f;
    for (int i = lane; i < size; i += 32) { const float v = src[i] * scale; ss += v * v; }
    const float s = scale / sqrtf(warp_sum(ss) / (float)size + eps);
    const T* gt = gate ? gate + t * g_stride + (int64_t)g * size : nullptr;
    for (int i = lane; i < size; i += 32) {
        float v = src[i] * s;
        if (w) v *= w[(g * size + i) % w_len];
        if (gt) {
            const float zz = to_f32<T>(gt[i]);
            v *= gate_silu ? zz / (1.0f + expf(-zz)) : 1.0f / (1.0f + expf(-zz));
        }
        out[(t * groups + g) * size + i] = from_f32<T>(v);
    }
}

extern "C" int mie_group_norm_gate(const float* o, int stride, const float* m, const float* w, int w_len, const void* gate, int tag,
                                   long long g_stride, void* out, int num_tokens, int groups, int size, float eps, int normalizer,
                                   int gate_silu, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (groups <= 0 || size <= 0 || stride < size + (normalizer ? 1 : 0) || (w && w_len <= 0) || (normalizer && !m)) return MIE_ERR_BAD_ARG;
    const int warps = 4;
    const int64_t items = (int64_t)num_tokens * groups;
    const int blocks = (int)((items + warps - 1) / warps);
    if (tag == MIE_F32)
        return launch_kernel(group_norm_gate_kernel<float>, dim3(blocks), dim3(warps * 32), 0, stream, o, stride, m, w, w_len,
                             (const float*)gate, (int64_t)g_stride, (float*)out, num_tokens, groups, size, eps, normalizer, gate_silu);
    else if (tag == MIE_BF16)
        return launch_kernel(group_norm_gate_kernel<bf16>, dim3(blocks), dim3(warps * 32), 0, stream, o, stride, m, w, w_len,
                             (const bf16*)gate, (int64_t)g_stride, (bf16*)out, num_tokens, groups, size, eps, normalizer, gate_silu);
    return MIE_ERR_BAD_ARG;
}
