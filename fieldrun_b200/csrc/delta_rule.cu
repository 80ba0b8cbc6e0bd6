// The gated delta rule: a recurrence over a float32 state S [dim, vdim] per head and sequence.
//
//   q, k  unit vectors per head (v / sqrt(sum v^2 + 1e-6)), q also times dim^(-1/2); head h uses q/k head h / (heads / kv_heads)
//   beta = sigmoid(b),  g = exp(-exp(a_log_h) * softplus(a + dt_bias_h))                       one of each per head and token
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q                                the read-out sees the token's own write
//   out = o / sqrt(mean(o^2) + eps) * w * silu(gate)                                            w [vdim] shared by the heads
//
// Everything here is float32 whatever the model's type: the inputs are the float32 results of the projections (behind
// their short convolution), and only `out` is rounded.  A block takes one (sequence, head).  Column j of the state
// belongs to P neighbouring lanes, each with R rows of it in registers, so the two sums over the rows that a token needs
// (S^T k and S^T q, taken before the decay and the write and corrected afterwards: o = g S_old^T q + u (k . q)) are one
// round of shuffles among P lanes and nothing crosses a warp.  Tokens go in chunks of DELTA_TOKENS: their rows are
// normed side by side (a warp a token), the pass along the chunk runs without a barrier, and the chunk's outputs are
// normed and gated side by side again.  The state of a slot exists twice: a step that begins at position p reads copy
// p & 1 and writes copy (p + n) & 1, so a step of one token never writes what it reads.
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
    int conv_stride, q_off, k_off, v_off, proj_stride, b_off, a_off, g_off;
    int heads, kv_heads, dim, vdim, lanes;      // lanes: P
    float eps;
};

__device__ __forceinline__ float delta_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

template <int R, int MAX_THREADS, typename OutT>
__global__ void __launch_bounds__(MAX_THREADS) gated_delta_rule_kernel(DeltaParams p) {
    extern __shared__ __align__(16) float sm[];
    after_previous_kernel();
    constexpr int SEG = R + 4;                         // a lane's rows of k and q, padded so that neighbours miss each other's banks
    const int P = p.lanes, dim = p.dim, vdim = p.vdim;
    const int row_floats = P * SEG;
    float* s_q = sm;                                   // [DELTA_TOKENS][row_floats]
    float* s_k = s_q + DELTA_TOKENS * row_floats;      // [DELTA_TOKENS][row_floats]
    float* s_v = s_k + DELTA_TOKENS * row_floats;      // [DELTA_TOKENS][vdim]
    float* s_o = s_v + DELTA_TOKENS * vdim;            // [DELTA_TOKENS][vdim]
    float* s_beta = s_o + DELTA_TOKENS * vdim;         // [DELTA_TOKENS]
    float* s_g = s_beta + DELTA_TOKENS;
    float* s_kq = s_g + DELTA_TOKENS;
    const int b = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (p.heads / p.kv_heads);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const int j = threadIdx.x / P, part = threadIdx.x - j * P;       // the state's column and this lane's share of its rows
    const bool live = j < vdim;
    const int row0 = p.cu_q_len[b], n_tok = p.cu_q_len[b + 1] - row0;
    const int start = p.seq_start[b], slot = p.seq_slot[b];
    const size_t head_floats = (size_t)dim * vdim;
    const float* s_in = p.state + ((size_t)slot * 2 + (start & 1)) * p.copy_floats + p.state_offset + h * head_floats;
    float* s_out = p.state + ((size_t)slot * 2 + ((start + n_tok) & 1)) * p.copy_floats + p.state_offset + h * head_floats;
    float S[R];
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = part * R + i;
        S[i] = (live && row < dim) ? s_in[(size_t)row * vdim + j] : 0.f;
    }
    const float rate = expf(p.a_log[h]), dt_bias = p.dt_bias[h];
    const float q_scale = rsqrtf((float)dim);
    for (int i = threadIdx.x; i < 2 * DELTA_TOKENS * row_floats; i += blockDim.x) sm[i] = 0.f;       // the padding stays zero
    __syncthreads();

    for (int t0 = 0; t0 < n_tok; t0 += DELTA_TOKENS) {
        const int count = min(DELTA_TOKENS, n_tok - t0);
        // -- the chunk's rows, normed: a warp a token
        for (int t = warp; t < count; t += nwarps) {
            const size_t row = (size_t)(row0 + t0 + t);
            const float* qr = p.conv + row * p.conv_stride + p.q_off + kvh * dim;
            const float* kr = p.conv + row * p.conv_stride + p.k_off + kvh * dim;
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
            const float* vr = p.conv + row * p.conv_stride + p.v_off + h * vdim;
            for (int d = lane; d < vdim; d += 32) s_v[t * vdim + d] = vr[d];
            if (lane == 0) {
                const float* pr = p.proj + row * p.proj_stride;
                s_beta[t] = 1.0f / (1.0f + expf(-pr[p.b_off + h]));
                s_g[t] = expm1f(-rate * delta_softplus(pr[p.a_off + h] + dt_bias));      // the decay less one
                s_kq[t] = dot;
            }
        }
        __syncthreads();
        // -- along the chunk
        for (int t = 0; t < count; ++t) {
            const float4* k4 = reinterpret_cast<const float4*>(s_k + t * row_floats + part * SEG);
            const float4* q4 = reinterpret_cast<const float4*>(s_q + t * row_floats + part * SEG);
            float sk = 0.f, sq = 0.f;
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 kk = k4[i], qq = q4[i];
                sk = fmaf(S[4 * i], kk.x, sk); sk = fmaf(S[4 * i + 1], kk.y, sk);
                sk = fmaf(S[4 * i + 2], kk.z, sk); sk = fmaf(S[4 * i + 3], kk.w, sk);
                sq = fmaf(S[4 * i], qq.x, sq); sq = fmaf(S[4 * i + 1], qq.y, sq);
                sq = fmaf(S[4 * i + 2], qq.z, sq); sq = fmaf(S[4 * i + 3], qq.w, sq);
            }
            for (int o = 1; o < P; o <<= 1) {
                sk += __shfl_xor_sync(0xffffffffu, sk, o);
                sq += __shfl_xor_sync(0xffffffffu, sq, o);
            }
            // the decay is kept as g - 1 and applied as S + (g - 1) S: rounded to float32, a decay close to one would lose
            // its distance from one by the same amount at every token
            const float gm1 = s_g[t];
            sk = fmaf(gm1, sk, sk);
            sq = fmaf(gm1, sq, sq);
            const float u = live ? s_beta[t] * (s_v[t * vdim + j] - sk) : 0.f;
#pragma unroll
            for (int i = 0; i < R / 4; ++i) {
                const float4 kk = k4[i];
                S[4 * i] = fmaf(kk.x, u, fmaf(gm1, S[4 * i], S[4 * i]));
                S[4 * i + 1] = fmaf(kk.y, u, fmaf(gm1, S[4 * i + 1], S[4 * i + 1]));
                S[4 * i + 2] = fmaf(kk.z, u, fmaf(gm1, S[4 * i + 2], S[4 * i + 2]));
                S[4 * i + 3] = fmaf(kk.w, u, fmaf(gm1, S[4 * i + 3], S[4 * i + 3]));
            }
            if (live && part == 0) s_o[t * vdim + j] = fmaf(u, s_kq[t], sq);
        }
        __syncthreads();
        // -- the chunk's outputs: root mean square over the head, weight, gate
        for (int t = warp; t < count; t += nwarps) {
            const size_t row = (size_t)(row0 + t0 + t);
            float ss = 0.f;
            for (int d = lane; d < vdim; d += 32) { const float o = s_o[t * vdim + d]; ss += o * o; }
            const float rinv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + p.eps);
            const float* gr = p.proj + row * p.proj_stride + p.g_off + h * vdim;
            OutT* out = (OutT*)p.out + (row * p.heads + h) * vdim;
            for (int d = lane; d < vdim; d += 32) {
                const float z = gr[d];
                out[d] = from_f32<OutT>(s_o[t * vdim + d] * rinv * p.norm[d] * (z / (1.0f + expf(-z))));
            }
        }
        // the next chunk's rows overwrite s_q, s_k, s_v, which every thread is done with (the barrier above); s_o is
        // written again only behind the next barrier
    }
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int row = part * R + i;
        if (live && row < dim) s_out[(size_t)row * vdim + j] = S[i];
    }
}

// How the rows of a head's state are shared out: `lanes` neighbouring lanes a column, `rows` (4, 8, 16 or 32) rows a lane.
// 0 lanes: a state the kernel does not take.
static void delta_shape(int dim, int vdim, int& lanes, int& rows) {
    lanes = 0;
    rows = 0;
    for (int P = 4; P <= 32; P *= 2) {
        if (P * 32 < dim) continue;
        if ((long)P * vdim > 1024) break;
        lanes = P;
        const int need = (dim + P - 1) / P;
        rows = need <= 4 ? 4 : need <= 8 ? 8 : need <= 16 ? 16 : 32;
        return;
    }
}

FRB_API int frb_gated_delta_rule(const float* conv, int conv_stride, int q_off, int k_off, int v_off, const float* proj,
                                 int proj_stride, int b_off, int a_off, int g_off, const float* a_log, const float* dt_bias,
                                 const float* norm, const int* seq_slot, const int* seq_start, const int* cu_q_len, float* state,
                                 long long copy_floats, long long state_offset, void* out, int out_dtype, int num_seqs, int heads,
                                 int kv_heads, int dim, int vdim, float eps, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    FRB_CHECK_ARG(heads >= 1 && kv_heads >= 1 && heads % kv_heads == 0, "gated delta rule: %d heads are not a multiple of %d key heads",
                  heads, kv_heads);
    FRB_CHECK_ARG(heads <= 65535, "gated delta rule: %d heads exceed the grid", heads);
    int lanes, rows;
    delta_shape(dim, vdim, lanes, rows);
    FRB_CHECK_ARG(dim >= 1 && vdim >= 1 && lanes > 0,
                  "gated delta rule: a state of %d x %d per head is more than a block's registers hold (keys up to 1024 and "
                  "keys x values up to 32768 with 32 rows a lane)", dim, vdim);
    DeltaParams p;
    p.conv = conv; p.proj = proj; p.a_log = a_log; p.dt_bias = dt_bias; p.norm = norm; p.seq_slot = seq_slot;
    p.seq_start = seq_start; p.cu_q_len = cu_q_len; p.state = state; p.copy_floats = copy_floats; p.state_offset = state_offset;
    p.out = out; p.conv_stride = conv_stride; p.q_off = q_off; p.k_off = k_off; p.v_off = v_off; p.proj_stride = proj_stride;
    p.b_off = b_off; p.a_off = a_off; p.g_off = g_off; p.heads = heads; p.kv_heads = kv_heads; p.dim = dim; p.vdim = vdim;
    p.lanes = lanes; p.eps = eps;
    const int threads = ((lanes * vdim + 31) / 32) * 32;
    const size_t smem = ((size_t)2 * DELTA_TOKENS * lanes * (rows + 4) + (size_t)2 * DELTA_TOKENS * vdim + 3 * DELTA_TOKENS) * sizeof(float);
    FRB_CHECK_ARG(smem <= 200 * 1024, "gated delta rule: heads of %d x %d need %zu bytes of shared memory", dim, vdim, smem);
    dim3 grid(num_seqs, heads);
#define FRB_LAUNCH_DELTA(R, MAX_THREADS)                                                                             \
    do {                                                                                                             \
        auto kernel = gated_delta_rule_kernel<R, MAX_THREADS, OutT>;                                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
        launch_dependent(kernel, grid, dim3(threads), smem, stream, p);                                              \
    } while (0)
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        // 32 rows a lane want more than the 64 registers that a block of 1024 threads leaves a thread
        if (rows == 4) FRB_LAUNCH_DELTA(4, 1024);
        else if (rows == 8) FRB_LAUNCH_DELTA(8, 1024);
        else if (rows == 16) FRB_LAUNCH_DELTA(16, 1024);
        else if (threads <= 512) FRB_LAUNCH_DELTA(32, 512);
        else FRB_LAUNCH_DELTA(32, 1024);
    });
#undef FRB_LAUNCH_DELTA
    FRB_RETURN_LAUNCH("gated_delta_rule");
}
