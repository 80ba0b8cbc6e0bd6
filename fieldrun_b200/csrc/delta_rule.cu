// The gated delta rule: a recurrence over a float32 state S [dim, vdim] per head and sequence.
//
//   q, k  unit vectors per head (v / sqrt(sum v^2 + 1e-6)), q also times dim^(-1/2); head h uses q/k head h / (heads / kv_heads)
//   beta = sigmoid(b),  g = exp(-exp(a_log_h) * softplus(a + dt_bias_h))                       one of each per head and token
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                                the read-out sees the token's own write
//   out = o / sqrt(mean(o^2) + eps) * w * silu(gate)                                            w [vdim] shared by the heads
//
// Everything here is float32 whatever the model's type: the inputs are the float32 results of the projections (behind
// their short convolution), and only `out` is rounded.  A block takes one (sequence, head), or a slice of the head's value
// columns.  C neighbouring columns of the state belong to P neighbouring lanes, each with R rows of them in registers, so
// the two sums over the rows that a token needs (S^T k and S^T q, taken before the decay and the write and corrected
// afterwards: o = g S_old^T q + u (k . q)) are one round of shuffles among P lanes and nothing crosses a warp.  Tokens go
// in chunks of DELTA_TOKENS: their rows come into shared memory as asynchronous copies while the chunk before them runs,
// are normed side by side (a warp a token), the pass along the chunk runs without a barrier, and the chunk's outputs are
// normed and gated side by side again.  The state of a slot exists twice: a step that begins at position p reads copy
// p & 1 and writes copy (p + n) & 1, so a step of one token never writes what it reads.
//
// The state's columns do not depend on one another, so every head's columns may be cut into slices over blocks
// (blockIdx.z); only the output's root mean square spans a head, and the sliced blocks leave o unnormed in a float32
// buffer that a second kernel norms and gates with the same sums in the same order: a token's output has the same bits
// however its step was cut.  The pass along a chunk is bound by what a thread reads from shared memory (its rows of k and
// q for every token: a 16-byte load serves four multiply-adds a column) and by the few warps that a long dependent chain
// leaves to hide behind.
#include "common.cuh"

#define DELTA_TOKENS 16

struct DeltaParams {
    const float* conv;       // [T, conv_stride]: q at q_off (kv_heads * dim), k at k_off, v at v_off (heads * vdim), behind conv and silu
    const float* proj;       // [T, proj_stride]: b at b_off (heads), a at a_off (heads), gate at g_off (heads * vdim), as projected
    const float* a_log;      // [heads]
    const float* dt_bias;    // [heads]
    const float* norm;       // [vdim]
    const int* seq_slot;     // [B]
    const int* seq_start;    // [B]
    const int* cu_q_len;     // [B + 1]
    float* state;            // [slots][2][copy_floats]
    long long copy_floats, state_offset;
    void* out;               // [T, heads * vdim]
    float* raw;              // [T, heads * vdim] float32: o before its norm, when a head's columns are cut over blocks (cols < vdim)
    int cols;                // value columns a block takes
    int conv_stride, q_off, k_off, v_off, proj_stride, b_off, a_off, g_off;
    int heads, kv_heads, dim, vdim, lanes;      // lanes: P
    float eps;
};

__device__ __forceinline__ float delta_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

__device__ __forceinline__ void delta_copy_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void delta_copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most `pending` of this thread's groups of copies are still on their way (0 or 1)
__device__ __forceinline__ void delta_copies_wait(int pending) {
    if (pending) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
}

template <int R, int C, typename OutT>
__global__ void __launch_bounds__(512) gated_delta_rule_kernel(DeltaParams p) {
    extern __shared__ __align__(16) float sm[];
    after_previous_kernel();
    constexpr int SEG = R + 4;                         // a lane's rows of k and q, padded so that neighbours miss each other's banks
    const int P = p.lanes, dim = p.dim, vdim = p.vdim;
    const int row_floats = P * SEG;
    const int cols = p.cols, col0 = blockIdx.z * p.cols;
    const bool fused = p.raw == nullptr;               // the block has all of the head's columns: it norms and gates its outputs itself
    float* s_q = sm;                                   // [DELTA_TOKENS][row_floats]
    float* s_k = s_q + DELTA_TOKENS * row_floats;      // [DELTA_TOKENS][row_floats]
    float* s_o = s_k + DELTA_TOKENS * row_floats;      // [DELTA_TOKENS][cols]
    float* s_beta = s_o + DELTA_TOKENS * cols;         // [DELTA_TOKENS]
    float* s_g = s_beta + DELTA_TOKENS;
    float* s_kq = s_g + DELTA_TOKENS;
    // the rows of a chunk as they come from memory, twice: the next chunk's are on their way while this one runs
    float* s_in0 = s_kq + DELTA_TOKENS;
    const int in_floats = DELTA_TOKENS * (2 * dim + 2 * cols + 2);       // q, k [dim] each; v, gate [cols] each; beta's and the decay's logits
    const int b = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (p.heads / p.kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int group = threadIdx.x / P, part = threadIdx.x - group * P;     // the thread's C columns (within the block's slice) and its share of their rows
    const int jl = group * C, j = col0 + jl;
    const int row0 = p.cu_q_len[b], n_tok = p.cu_q_len[b + 1] - row0;
    const int start = p.seq_start[b], slot = p.seq_slot[b];
    const int chunks = (n_tok + DELTA_TOKENS - 1) / DELTA_TOKENS;

    // asks for the rows of chunk n into its buffer
    auto fetch = [&](int n) {
        float* in = s_in0 + (n & 1) * in_floats;
        float* in_q = in;
        float* in_k = in_q + DELTA_TOKENS * dim;
        float* in_v = in_k + DELTA_TOKENS * dim;
        float* in_gate = in_v + DELTA_TOKENS * cols;
        float* in_ba = in_gate + DELTA_TOKENS * cols;
        const int t0 = n * DELTA_TOKENS, count = min(DELTA_TOKENS, n_tok - t0);
        // (token, entry) of this thread's copies step by step, without a division a copy
        {
            int t = threadIdx.x / dim, d = threadIdx.x - t * dim;
            const int step_t = blockDim.x / dim, step_d = blockDim.x - step_t * dim;
            for (int i = threadIdx.x; i < count * dim; i += blockDim.x) {
                const float* row = p.conv + (size_t)(row0 + t0 + t) * p.conv_stride + kvh * dim + d;
                delta_copy_async4(in_q + i, row + p.q_off);
                delta_copy_async4(in_k + i, row + p.k_off);
                t += step_t;
                d += step_d;
                if (d >= dim) { d -= dim; ++t; }
            }
        }
        {
            int t = threadIdx.x / cols, d = threadIdx.x - t * cols;
            const int step_t = blockDim.x / cols, step_d = blockDim.x - step_t * cols;
            for (int i = threadIdx.x; i < count * cols; i += blockDim.x) {
                if (col0 + d < vdim) {
                    const size_t row = (size_t)(row0 + t0 + t);
                    delta_copy_async4(in_v + i, p.conv + row * p.conv_stride + p.v_off + h * vdim + col0 + d);
                    if (fused) delta_copy_async4(in_gate + i, p.proj + row * p.proj_stride + p.g_off + h * vdim + col0 + d);
                }
                t += step_t;
                d += step_d;
                if (d >= cols) { d -= cols; ++t; }
            }
        }
        if (threadIdx.x < 2 * count) {
            const int t = threadIdx.x >> 1, which = threadIdx.x & 1;
            delta_copy_async4(in_ba + threadIdx.x, p.proj + (size_t)(row0 + t0 + t) * p.proj_stride + (which ? p.a_off : p.b_off) + h);
        }
        delta_copies_commit();
    };
    if (chunks > 0) fetch(0);

    const size_t head_floats = (size_t)dim * vdim;
    const float* s_in = p.state + ((size_t)slot * 2 + (start & 1)) * p.copy_floats + p.state_offset + h * head_floats;
    float* s_out = p.state + ((size_t)slot * 2 + ((start + n_tok) & 1)) * p.copy_floats + p.state_offset + h * head_floats;
    bool live[C];
#pragma unroll
    for (int c = 0; c < C; ++c) live[c] = jl + c < cols && j + c < vdim;
    float S[R][C];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = part * R + i;
#pragma unroll
        for (int c = 0; c < C; ++c) S[i][c] = (live[c] && row < dim) ? s_in[(size_t)row * vdim + j + c] : 0.f;
    }
    const float rate = expf(p.a_log[h]), dt_bias = p.dt_bias[h];
    const float q_scale = 1.0f / sqrtf((float)dim);
    for (int i = threadIdx.x; i < 2 * DELTA_TOKENS * row_floats; i += blockDim.x) sm[i] = 0.f;       // the padding stays zero

    for (int n = 0; n < chunks; ++n) {
        const int t0 = n * DELTA_TOKENS, count = min(DELTA_TOKENS, n_tok - t0);
        if (n + 1 < chunks) fetch(n + 1);
        delta_copies_wait(n + 1 < chunks ? 1 : 0);
        __syncthreads();                               // this chunk's rows are here for every thread (and the zeros, the first time)
        const float* in = s_in0 + (n & 1) * in_floats;
        const float* in_q = in;
        const float* in_k = in_q + DELTA_TOKENS * dim;
        const float* in_v = in_k + DELTA_TOKENS * dim;
        const float* in_gate = in_v + DELTA_TOKENS * cols;
        const float* in_ba = in_gate + DELTA_TOKENS * cols;
        // -- the chunk's rows, normed: a warp a token
        for (int t = warp; t < count; t += nwarps) {
            const float* qr = in_q + t * dim;
            const float* kr = in_k + t * dim;
            float qq = 0.f, kk = 0.f;
            for (int d = lane; d < dim; d += 32) { const float a = qr[d], c = kr[d]; qq += a * a; kk += c * c; }
            qq = warp_sum(qq);
            kk = warp_sum(kk);
            const float q_inv = q_scale / sqrtf(qq + 1e-6f), k_inv = 1.0f / sqrtf(kk + 1e-6f);
            float dot = 0.f;
            for (int d = lane; d < dim; d += 32) {
                const float a = qr[d] * q_inv, c = kr[d] * k_inv;
                const int at = t * row_floats + (d / R) * SEG + (d % R);
                s_q[at] = a;
                s_k[at] = c;
                dot += a * c;
            }
            dot = warp_sum(dot);
            if (lane == 0) {
                s_beta[t] = 1.0f / (1.0f + expf(-in_ba[2 * t]));
                s_g[t] = expm1f(-rate * delta_softplus(in_ba[2 * t + 1] + dt_bias));      // the decay less one
                s_kq[t] = dot;
            }
        }
        __syncthreads();
        // -- along the chunk
        for (int t = 0; t < count; ++t) {
            const float4* k4 = reinterpret_cast<const float4*>(s_k + t * row_floats + part * SEG);
            const float4* q4 = reinterpret_cast<const float4*>(s_q + t * row_floats + part * SEG);
            float sk[C], sq[C];
#pragma unroll
            for (int c = 0; c < C; ++c) sk[c] = sq[c] = 0.f;
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 kk = k4[i], qq = q4[i];
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    sk[c] = fmaf(S[4 * i][c], kk.x, sk[c]); sk[c] = fmaf(S[4 * i + 1][c], kk.y, sk[c]);
                    sk[c] = fmaf(S[4 * i + 2][c], kk.z, sk[c]); sk[c] = fmaf(S[4 * i + 3][c], kk.w, sk[c]);
                    sq[c] = fmaf(S[4 * i][c], qq.x, sq[c]); sq[c] = fmaf(S[4 * i + 1][c], qq.y, sq[c]);
                    sq[c] = fmaf(S[4 * i + 2][c], qq.z, sq[c]); sq[c] = fmaf(S[4 * i + 3][c], qq.w, sq[c]);
                }
            }
#pragma unroll
            for (int round = 0; round < 5; ++round) {          // P is the same for the whole block: no branch diverges
                const int o = 1 << round;
                if (o < P) {
#pragma unroll
                    for (int c = 0; c < C; ++c) {
                        sk[c] += __shfl_xor_sync(0xffffffffu, sk[c], o);
                        sq[c] += __shfl_xor_sync(0xffffffffu, sq[c], o);
                    }
                }
            }
            // the decay is kept as g - 1 and applied as S + (g - 1) S: rounded to float32, a decay close to one would lose
            // its distance from one by the same amount at every token
            const float gm1 = s_g[t], beta = s_beta[t], kq = s_kq[t];
            float u[C];
#pragma unroll
            for (int c = 0; c < C; ++c) {
                sk[c] = fmaf(gm1, sk[c], sk[c]);
                sq[c] = fmaf(gm1, sq[c], sq[c]);
                u[c] = live[c] ? beta * (in_v[t * cols + jl + c] - sk[c]) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 kk = k4[i];
#pragma unroll
                for (int c = 0; c < C; ++c) {
                    S[4 * i][c] = fmaf(kk.x, u[c], fmaf(gm1, S[4 * i][c], S[4 * i][c]));
                    S[4 * i + 1][c] = fmaf(kk.y, u[c], fmaf(gm1, S[4 * i + 1][c], S[4 * i + 1][c]));
                    S[4 * i + 2][c] = fmaf(kk.z, u[c], fmaf(gm1, S[4 * i + 2][c], S[4 * i + 2][c]));
                    S[4 * i + 3][c] = fmaf(kk.w, u[c], fmaf(gm1, S[4 * i + 3][c], S[4 * i + 3][c]));
                }
            }
            if (part == 0) {
#pragma unroll
                for (int c = 0; c < C; ++c)
                    if (live[c]) s_o[t * cols + jl + c] = fmaf(u[c], kq, sq[c]);
            }
        }
        __syncthreads();
        if (!fused) {                                  // a slice of the head: o as it is, for the kernel that norms whole heads
            for (int i = threadIdx.x; i < count * cols; i += blockDim.x) {
                const int t = i / cols, d = i - t * cols;
                if (col0 + d < vdim) p.raw[((size_t)(row0 + t0 + t) * p.heads + h) * vdim + col0 + d] = s_o[i];
            }
        } else {
            // -- the chunk's outputs: root mean square over the head, weight, gate
            for (int t = warp; t < count; t += nwarps) {
                const size_t row = (size_t)(row0 + t0 + t);
                float ss = 0.f;
                for (int d = lane; d < vdim; d += 32) { const float o = s_o[t * cols + d]; ss += o * o; }
                const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + p.eps);
                OutT* out = (OutT*)p.out + (row * p.heads + h) * vdim;
                for (int d = lane; d < vdim; d += 32) {
                    const float z = in_gate[t * cols + d];
                    out[d] = from_f32<OutT>(s_o[t * cols + d] * rinv * p.norm[d] * (z / (1.0f + expf(-z))));
                }
            }
        }
        // The next round's copies go into the buffer that this chunk was read from, and its rows overwrite s_q and s_k: behind
        // the barrier at the top of the next round, which no thread passes before all are done here.
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = part * R + i;
#pragma unroll
        for (int c = 0; c < C; ++c)
            if (live[c] && row < dim) s_out[(size_t)row * vdim + j + c] = S[i][c];
    }
}

// Norms and gates the outputs that sliced blocks left in `raw`: a warp per (token, head), the same sums in the same order
// as the unsliced kernel's last phase.
template <typename OutT>
__global__ void __launch_bounds__(128) delta_output_kernel(DeltaParams p, int num_rows) {
    after_previous_kernel();
    const int lane = threadIdx.x & 31, item = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= num_rows * p.heads) return;
    const size_t row = item / p.heads;
    const int h = item - (int)row * p.heads, vdim = p.vdim;
    const float* o = p.raw + (row * p.heads + h) * vdim;
    float ss = 0.f;
    for (int d = lane; d < vdim; d += 32) { const float v = o[d]; ss += v * v; }
    const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + p.eps);
    const float* gr = p.proj + row * p.proj_stride + p.g_off + h * vdim;
    OutT* out = (OutT*)p.out + (row * p.heads + h) * vdim;
    for (int d = lane; d < vdim; d += 32) {
        const float z = gr[d];
        out[d] = from_f32<OutT>(o[d] * rinv * p.norm[d] * (z / (1.0f + expf(-z))));
    }
}

// How a head's state is shared out: `lanes` (a power of two up to 32) neighbouring lanes take `columns` neighbouring value
// columns, each lane `rows` (4, 8, 16 or 32) key rows of them.  `many_warps`: up to eight rows of two columns a thread;
// else up to 64 state elements a thread (four columns of up to 16 rows; two of 32).  0 lanes: more keys than 32 lanes of
// 32 rows hold.
static long frb_dependent_launch_blocks_or_sms() {
    static const long sms = [] {
        int device = 0, count = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
        return (long)(count > 0 ? count : 148);
    }();
    return sms;
}

static void delta_shape(int dim, bool many_warps, int& lanes, int& rows, int& columns) {
    const int most = many_warps ? 8 : 16;
    lanes = 1;
    while (lanes < 32 && (dim + lanes - 1) / lanes > most) lanes *= 2;
    const int need = (dim + lanes - 1) / lanes;
    rows = need <= 4 ? 4 : need <= 8 ? 8 : need <= 16 ? 16 : 32;
    columns = rows == 32 ? 2 : (many_warps && rows <= 8) ? 2 : 4;
    if (dim < 1 || need > 32) lanes = 0;
}

FRB_API int frb_gated_delta_rule(const float* conv, int conv_stride, int q_off, int k_off, int v_off, const float* proj,
                                 int proj_stride, int b_off, int a_off, int g_off, const float* a_log, const float* dt_bias,
                                 const float* norm, const int* seq_slot, const int* seq_start, const int* cu_q_len, float* state,
                                 long long copy_floats, long long state_offset, void* out, int out_dtype, float* raw, int num_rows,
                                 int slices, int num_seqs, int heads, int kv_heads, int dim, int vdim, float eps, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(heads >= 1 && kv_heads >= 1 && heads % kv_heads == 0, "gated delta rule: %d heads are not a multiple of %d key heads",
                  heads, kv_heads);
    FRB_CHECK_ARG(heads <= 65535, "gated delta rule: %d heads exceed the grid", heads);
    int lanes, rows, columns;
    // A prompt's tokens go one after the other through every thread of their head, and what hides one thread's latencies
    // is other warps: eight rows of two columns a thread, sixteen warps a block.  A step of single tokens is bound by the
    // state it reads and writes: up to 64 elements a thread, fewer loads of k and q from shared memory.  (Measured on a
    // B200, 16 heads of 128 x 128, four prompts of 2,048 tokens: eight rows of one, two, four columns a thread 1.69, 1.40,
    // 1.98 ms, sixteen rows of four columns 2.64; 64 single tokens: 0.153 with eight rows of one column, 0.072 with sixteen
    // of four.)
    const bool prompt = num_rows > num_seqs;
    delta_shape(dim, prompt, lanes, rows, columns);
    FRB_CHECK_ARG(vdim >= 1 && lanes > 0, "gated delta rule: heads of %d keys and %d values (the kernel takes up to 1024 keys)", dim, vdim);
    DeltaParams p;
    p.conv = conv; p.proj = proj; p.a_log = a_log; p.dt_bias = dt_bias; p.norm = norm; p.seq_slot = seq_slot;
    p.seq_start = seq_start; p.cu_q_len = cu_q_len; p.state = state; p.copy_floats = copy_floats; p.state_offset = state_offset;
    p.out = out; p.conv_stride = conv_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.proj_stride = proj_stride;
    p.b_off = b_off; p.a_off = a_off; p.g_off = g_off; p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim;
    p.lanes = lanes; p.eps = eps;
    // A head's value columns go over `slices` blocks, in multiples of four columns; more than one: the outputs pass through
    // `raw`.  slices 0: blocks of up to 512 threads, and for single tokens narrower ones (down to 128 threads) while the
    // step has fewer than two blocks an SM.
    const int most_cols = (512 / lanes) * columns;          // 512 threads
    const int all_cols = (vdim + 3) / 4 * 4;
    int cols;
    if (slices >= 1) {
        cols = ((vdim + slices - 1) / slices + 3) / 4 * 4;
    } else {
        cols = most_cols < all_cols ? most_cols : all_cols;
        const long wanted = 2 * frb_dependent_launch_blocks_or_sms();
        while (!prompt && (long)num_seqs * heads * ((vdim + cols - 1) / cols) < wanted && cols >= 8 && (cols / 2 / columns) * lanes >= 128)
            cols = (cols / 2 + 3) / 4 * 4;
    }
    if (cols > most_cols) cols = most_cols;
    if (cols > all_cols) cols = all_cols;
    slices = (vdim + cols - 1) / cols;
    FRB_CHECK_ARG(slices == 1 || raw != nullptr, "gated delta rule: heads of %d x %d go over %d blocks each, which needs the "
                  "float32 buffer for their outputs", dim, vdim, slices);
    FRB_CHECK_ARG(slices <= 65535, "gated delta rule: %d slices exceed the grid", slices);
    p.cols = cols;
    p.raw = slices > 1 ? raw : nullptr;
    const int threads = ((lanes * ((cols + columns - 1) / columns) + 31) / 32) * 32;
    const size_t smem = ((size_t)2 * DELTA_TOKENS * lanes * (rows + 4) + (size_t)DELTA_TOKENS * cols + 3 * DELTA_TOKENS +
                         (size_t)2 * DELTA_TOKENS * (2 * dim + 2 * cols + 2)) * sizeof(float);
    FRB_CHECK_ARG(smem <= 200 * 1024, "gated delta rule: heads of %d x %d need %zu bytes of shared memory", dim, vdim, smem);
    FRB_CHECK_ARG(threads <= 512, "gated delta rule: %d value columns a block with %d lanes each", cols, lanes);
    dim3 grid(num_seqs, heads, slices);
#define FRB_LAUNCH_DELTA(R, C)                                                                                       \
    do {                                                                                                             \
        auto kernel = gated_delta_rule_kernel<R, C, OutT>;                                                           \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        launch_dependent(kernel, grid, dim3(threads), smem, stream, p);                                              \
    } while (0)
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        if (rows == 4 && columns == 2) FRB_LAUNCH_DELTA(4, 2);
        else if (rows == 8 && columns == 2) FRB_LAUNCH_DELTA(8, 2);
        else if (rows == 4) FRB_LAUNCH_DELTA(4, 4);
        else if (rows == 8) FRB_LAUNCH_DELTA(8, 4);
        else if (rows == 16) FRB_LAUNCH_DELTA(16, 4);
        else FRB_LAUNCH_DELTA(32, 2);
    });
#undef FRB_LAUNCH_DELTA
    if (slices > 1) {
        FRB_DISPATCH_DTYPE(out_dtype, OutT, {
            launch_dependent(delta_output_kernel<OutT>, dim3((num_rows * heads + 3) / 4), dim3(128), 0, stream, p, num_rows);
        });
    }
    FRB_RETURN_LAUNCH("gated_delta_rule");
}
