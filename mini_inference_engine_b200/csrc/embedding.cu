// Embedding gather: res[t, :] = table[ids[t], :], written as float32 because the gathered row
// opens the residual stream, which this engine keeps in 32-bit
// (what F.embedding does at inference_engine/model.py:168).
// A negative id -(k+1) stands for "the k-th token the previous step sampled": it is read from the
// `feedback` buffer on the device, so a step can be launched before the host has seen that token.
// `scale` multiplies the row (in float32) and `copies` writes it that many times side by side (a model that carries
// several copies of its stream: out is [tokens, copies, hidden]).
#include "common.cuh"
#include "range_check.cuh"

template <typename TT>
__global__ void embedding_kernel(const TT* __restrict__ table, const int* __restrict__ ids,
                                 const int* __restrict__ feedback, float* __restrict__ out, int hidden, int vocab,
                                 int feedback_len, float scale, int copies, int* report) {
    pdl_enter();
    const int t = blockIdx.x;
    int id = ids[t];
    // ids are checked on the host when a request is added; one out of range here is reported and its
    // row left as it is (both the id in the batch and the token it may stand for are checked)
    bool ok = range_token(id, vocab, feedback ? feedback_len : 0) == MIE_RANGE_OK;
    if (ok && id < 0) { id = feedback[-id - 1]; ok = id >= 0 && id < vocab; }
    if (!ok) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_TOKEN, MIE_K_EMBEDDING, t, id);
        return;
    }
    const TT* src = table + (int64_t)id * hidden;
    float* dst = out + (int64_t)t * copies * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        const float v = to_f32<TT>(src[i]) * scale;
        for (int c = 0; c < copies; ++c) dst[(int64_t)c * hidden + i] = v;
    }
}

extern "C" int mie_embedding(const void* table, int table_tag, const int* ids, const int* feedback, float* out,
                             int num_tokens, int hidden, int vocab, int feedback_len, float scale, int copies, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0 || copies < 1) return MIE_ERR_BAD_ARG;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    if (table_tag == MIE_F32)
        return launch_kernel(embedding_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)table, ids, feedback, out, hidden, vocab, feedback_len, scale, copies, g_range_report);
    else if (table_tag == MIE_BF16)
        return launch_kernel(embedding_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream, (const bf16*)table, ids, feedback, out, hidden, vocab, feedback_len, scale, copies, g_range_report);
    return MIE_ERR_BAD_ARG;
}

// The same gather with a second table indexed by a hash of the token and the token before it:
//   out[t, :] = table[id, :] * scale + pair_table[(prev * mul_prev + id * mul_cur) mod buckets, :]
// and row `buckets` (the table's last) for the first token of a sequence.  The token before is the one in front of it
// in the batch row, or, for the first token of a row that continues a sequence (position > 0), the sequence's
// `last_token` state (one int32 per state slot); the block of a row's first token also leaves the row's last token
// there for the next step, so that no other block reads or writes that slot.  Also written: the ids with fed-back
// tokens resolved (`resolved`, for parts that read other per-token tables), a second copy of the row (`first`: entry 0 of
// a history of the stream, optional) and its rounding to the activation type (`act`, optional).  All sums in float32.
template <typename TT>
__global__ void pair_embedding_kernel(const TT* __restrict__ table, const TT* __restrict__ pair_table, const int* __restrict__ ids,
                                      const int* __restrict__ feedback, const int* __restrict__ positions,
                                      const int* __restrict__ token_row, const int* __restrict__ row_q_start,
                                      const int* __restrict__ row_q_len, const int* __restrict__ state_slots,
                                      int* __restrict__ last_token, float* __restrict__ out, float* __restrict__ first,
                                      bf16* __restrict__ act, int* __restrict__ resolved, int hidden, int vocab, int feedback_len,
                                      float scale, int buckets, long long mul_prev, long long mul_cur, int num_rows, int num_slots,
                                      int* report) {
    pdl_enter();
    const int t = blockIdx.x;
    auto resolve = [&](int at, int& id) -> bool {
        id = ids[at];
        bool ok = range_token(id, vocab, feedback ? feedback_len : 0) == MIE_RANGE_OK;
        if (ok && id < 0) { id = feedback[-id - 1]; ok = id >= 0 && id < vocab; }
        return ok;
    };
    int id;
    if (!resolve(t, id)) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_TOKEN, MIE_K_EMBEDDING, t, id);
        return;
    }
    const int row = token_row[t];
    if (range_row(row, num_rows) != MIE_RANGE_OK) {
        if (threadIdx.x == 0) range_report(report, MIE_RANGE_ROW, MIE_K_EMBEDDING, t, row);
        return;
    }
    const int start = row_q_start[row];
    int prev = -1;                                   // -1: the sequence starts here
    if (t > start) {
        if (!resolve(t - 1, prev)) return;           // reported by that token's own block
    } else {
        const int slot = state_slots[row];
        if (slot < 0 || slot >= num_slots) {
            if (threadIdx.x == 0) range_report(report, MIE_RANGE_ROW, MIE_K_EMBEDDING, t, slot);
            return;
        }
        if (positions[t] > 0) prev = last_token[slot];
        int last;
        const bool ok = resolve(start + row_q_len[row] - 1, last);
        __syncthreads();                              // every thread has read the state before one of them replaces it
        if (threadIdx.x == 0 && ok) last_token[slot] = last;
        if (prev < 0 && positions[t] > 0) prev = 0;   // (a state that was never written: keep the index in range)
        if (prev >= vocab) prev = vocab - 1;
    }
    if (threadIdx.x == 0 && resolved) resolved[t] = id;
    const TT* src = table + (int64_t)id * hidden;
    const TT* pair = nullptr;
    if (pair_table) {
        const long long b = prev < 0 ? (long long)buckets : ((long long)prev * mul_prev + (long long)id * mul_cur) % (long long)buckets;
        pair = pair_table + b * hidden;
    }
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
        float v = to_f32<TT>(src[i]) * scale;
        if (pair) v += to_f32<TT>(pair[i]);
        out[(int64_t)t * hidden + i] = v;
        if (first) first[(int64_t)t * hidden + i] = v;
        if (act) act[(int64_t)t * hidden + i] = __float2bfloat16_rn(v);
    }
}

extern "C" int mie_pair_embedding(const void* table, const void* pair_table, int table_tag, const int* ids, const int* feedback,
                                  const int* positions, const int* token_row, const int* row_q_start, const int* row_q_len,
                                  const int* state_slots, int* last_token, float* out, float* first, void* act, int* resolved,
                                  int num_tokens, int hidden, int vocab, int feedback_len, float scale, int buckets,
                                  long long mul_prev, long long mul_cur, int num_rows, int num_slots, cudaStream_t stream) {
    if (num_tokens <= 0) return 0;
    if (hidden <= 0 || vocab <= 0 || num_rows <= 0 || num_slots <= 0 || (pair_table && (buckets <= 0 || mul_prev < 0 || mul_cur < 0)))
        return MIE_ERR_BAD_ARG;
    const int threads = hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64);
    if (table_tag == MIE_F32)
        return launch_kernel(pair_embedding_kernel<float>, dim3(num_tokens), dim3(threads), 0, stream, (const float*)table,
                             (const float*)pair_table, ids, feedback, positions, token_row, row_q_start, row_q_len, state_slots,
                             last_token, out, first, (bf16*)act, resolved, hidden, vocab, feedback_len, scale, buckets, mul_prev,
                             mul_cur, num_rows, num_slots, g_range_report);
    else if (table_tag == MIE_BF16)
        return launch_kernel(pair_embedding_kernel<bf16>, dim3(num_tokens), dim3(threads), 0, stream, (const bf16*)table,
                             (const bf16*)pair_table, ids, feedback, positions, token_row, row_q_start, row_q_len, state_slots,
                             last_token, out, first, (bf16*)act, resolved, hidden, vocab, feedback_len, scale, buckets, mul_prev,
                             mul_cur, num_rows, num_slots, g_range_report);
    return MIE_ERR_BAD_ARG;
}
