// Inputs that depend on the token ids beyond the plain embedding row.
//
// embed_pair_rows: out[t] = table[tok_t] * scale + pair[row_t], where row_t is a hash of the token before and the
//   token itself, row_t = (tok_{t-1} * mul_prev + tok_t * mul_cur) mod buckets, and the extra row `buckets` for a
//   sequence's first token.  The token before a step's first token is state of the sequence: an int32 pair per slot,
//   a step that begins at position p reads copy p & 1 and writes copy (p + n) & 1 (n: its new tokens), so that a
//   one-token step never writes what it reads and a row that a recorded step holds twice computes the same twice.
//
// token_side_gate: g[t, j] = gelu_tanh(lin[t, j]) * side[tok_t, column0 + j], the gate of a per-layer token input.
// add_rms_normed:  x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w, the sum in float32 in place.
// add_typed_copy:  x[t] += delta[t] (if given), act[t] = x[t] in the model type.
#include "common.cuh"

template <typename WT, typename AT>
__global__ void __launch_bounds__(256)
embed_pair_rows_kernel(const int* __restrict__ tokens, const WT* __restrict__ table, const WT* __restrict__ pair,
                       float* __restrict__ out, AT* __restrict__ act, int width, int vocab, float scale, int buckets,
                       long long mul_prev, long long mul_cur, const int* __restrict__ tok_pos,
                       const int* __restrict__ tok_seq, const int* __restrict__ tok_slot,
                       const int* __restrict__ cu_q_len, int* __restrict__ state) {
    after_previous_kernel();
    const int t = blockIdx.x;
    int token = tokens[t];
    if (token < 0 || token >= vocab) token = 0;      // ids are checked on the host before any launch
    const int pos = tok_pos[t], seq = tok_seq[t], slot = tok_slot[t];
    const int first_row = cu_q_len[seq], end_row = cu_q_len[seq + 1];
    const bool opens_step = t == first_row;
    int row = buckets;
    if (pos > 0) {
        const int before = opens_step ? state[2 * slot + (pos & 1)] : tokens[t - 1];
        row = (int)(((long long)before * mul_prev + (long long)token * mul_cur) % (long long)buckets);
    }
    const WT* a = table + (size_t)token * width;
    const WT* b = pair + (size_t)row * width;
    float* dst = out + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = to_f32<WT>(a[i]) * scale + to_f32<WT>(b[i]);
        dst[i] = v;
        if (act) act[(size_t)t * width + i] = from_f32<AT>(v);
    }
    if (opens_step) {
        // the block of a sequence's first new row is the only one that reads its state, and the only one that writes it
        __syncthreads();
        if (threadIdx.x == 0) state[2 * slot + ((pos + end_row - first_row) & 1)] = tokens[end_row - 1];
    }
}

FRB_API int frb_embed_pair_rows(const int* tokens, const void* table, const void* pair, int table_dtype, float* out,
                                int num_tokens, int width, int vocab, float scale, int buckets, long long mul_prev,
                                long long mul_cur, const int* tok_pos, const int* tok_seq, const int* tok_slot,
                                const int* cu_q_len, int* state, void* act, int act_dtype, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(buckets >= 1, "embedding: a pair table of %d hashed rows", buckets);
    FRB_DISPATCH_DTYPE(table_dtype, WT, FRB_DISPATCH_DTYPE(act_dtype, AT, {
        launch_dependent(embed_pair_rows_kernel<WT, AT>, dim3(num_tokens), dim3(256), 0, stream, tokens, (const WT*)table,
                         (const WT*)pair, out, (AT*)act, width, vocab, scale, buckets, mul_prev, mul_cur, tok_pos, tok_seq,
                         tok_slot, cu_q_len, state);
    }));
    FRB_RETURN_LAUNCH("embed_pair_rows");
}

__device__ __forceinline__ float gelu_tanh_f(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <typename WT, typename OutT>
__global__ void token_side_gate_kernel(const float* __restrict__ lin, const int* __restrict__ tokens,
                                       const WT* __restrict__ side, OutT* __restrict__ out, int dim, int side_width,
                                       int column0, int vocab, size_t total) {
    after_previous_kernel();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / dim;
    const int j = (int)(i - t * dim);
    int token = tokens[t];
    if (token < 0 || token >= vocab) token = 0;
    const float e = to_f32<WT>(side[(size_t)token * side_width + column0 + j]);
    out[i] = from_f32<OutT>(gelu_tanh_f(lin[i]) * e);
}

FRB_API int frb_token_side_gate(const float* lin, const int* tokens, const void* side, int side_dtype, void* out,
                                int out_dtype, int num_tokens, int dim, int side_width, int column0, int vocab,
                                cudaStream_t stream) {
    const size_t total = (size_t)num_tokens * dim;
    if (total == 0) return 0;
    FRB_CHECK_ARG(column0 >= 0 && column0 + dim <= side_width, "token side input: columns %d..%d of a table of %d", column0,
                  column0 + dim, side_width);
    FRB_DISPATCH_DTYPE(side_dtype, WT, FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(token_side_gate_kernel<WT, OutT>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, lin,
                         tokens, (const WT*)side, (OutT*)out, dim, side_width, column0, vocab, total);
    }));
    FRB_RETURN_LAUNCH("token_side_gate");
}

// One block per row; the row is read twice (statistic, then the sum), from L1/L2 the second time.
template <int BLOCK>
__global__ void __launch_bounds__(BLOCK)
add_rms_normed_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ weight, int width, float eps) {
    after_previous_kernel();
    __shared__ float scratch[32];
    const size_t base = (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += BLOCK) { const float v = y[base + i]; ss += v * v; }
    const float rinv = 1.0f / sqrtf(block_sum<BLOCK>(ss, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += BLOCK) x[base + i] += y[base + i] * rinv * weight[i];
}

FRB_API int frb_add_rms_normed(float* x, const float* y, const float* weight, int rows, int width, float eps,
                               cudaStream_t stream) {
    if (rows == 0) return 0;
    launch_dependent(add_rms_normed_kernel<256>, dim3(rows), dim3(256), 0, stream, x, y, weight, width, eps);
    FRB_RETURN_LAUNCH("add_rms_normed");
}

template <typename OutT>
__global__ void add_typed_copy_kernel(float* __restrict__ x, const float* __restrict__ delta, OutT* __restrict__ act, size_t n) {
    after_previous_kernel();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = x[i];
    if (delta) { v += delta[i]; x[i] = v; }
    act[i] = from_f32<OutT>(v);
}

FRB_API int frb_add_typed_copy(float* x, const float* delta, void* act, int act_dtype, long long n, cudaStream_t stream) {
    if (n == 0) return 0;
    FRB_DISPATCH_DTYPE(act_dtype, OutT, {
        launch_dependent(add_typed_copy_kernel<OutT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x, delta,
                         (OutT*)act, (size_t)n);
    });
    FRB_RETURN_LAUNCH("add_typed_copy");
}
