// Operations on whole rows of the float32 residual stream that need no statistics, or only a row's mean square:
//
//   dyt_norm     the dynamic-tanh norm, y = tanh(alpha v) * w + b, of v = x + updates, for up to two norms of the same
//                v at once (a block whose two sublayers read the same x), with the sum stored back into x;
//                the updates are up to two float32 tensors and the weighted rows of routed experts, added in a
//                fixed order: x + ((d0 + d1) + sum over ranks of weight * row)
//   rms_blend    out = share * (a / rms(a) * wa + b / rms(b) * wb), two mixers' outputs side by side
//   concat_rows  out = [a | b] row by row in the model dtype (a may get an update added first)
//   add_row_vector  out = y + vec, the same vector on every row
#include "common.cuh"

#define ROW_BLOCK 256
#define DYT_MAX_ROWS 64      // the most weighted rows that the norm sums for a token

struct DytParams {
    float* x;                 // [T, width]
    const float* delta0;      // [T, width] or null
    const float* delta1;      // [T, width] or null
    const float* y;           // [N, width] or null: expert outputs
    const float* ew;          // [T, top_k]
    const int* rowmap;        // [T * top_k]
    const int* rows;          // [R] or null: the rows to norm
    const float *w1, *b1, *alpha1;
    void* out1;
    const float *w2, *b2, *alpha2;   // null: one norm only
    void* out2;
    float* out2_32;           // null, or the second norm's result in float32 as well
    int top_k, width, write_back;
};

template <typename OutT>
__global__ void __launch_bounds__(ROW_BLOCK) dyt_norm_kernel(DytParams p) {
    __shared__ float s_weight[DYT_MAX_ROWS];
    __shared__ int s_row[DYT_MAX_ROWS];
    after_previous_kernel();
    const int r = blockIdx.x;
    const int src = p.rows ? p.rows[r] : r;
    const size_t base = (size_t)src * p.width, obase = (size_t)r * p.width;
    const float a1 = *p.alpha1, a2 = p.w2 ? *p.alpha2 : 0.f;
    if (p.y) {                                          // the row's experts: weights and rows once, not per element
        if (threadIdx.x < p.top_k) {
            s_weight[threadIdx.x] = p.ew[(size_t)src * p.top_k + threadIdx.x];
            s_row[threadIdx.x] = p.rowmap[(size_t)src * p.top_k + threadIdx.x];
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < p.width; i += ROW_BLOCK) {
        float v = p.x[base + i];
        float d = 0.f;
        bool any = false;
        if (p.delta0) { d = p.delta0[base + i]; any = true; }
        if (p.delta1) { d += p.delta1[base + i]; any = true; }
        if (p.y) {
            float e = 0.f;
            for (int k = 0; k < p.top_k; ++k) e += s_weight[k] * p.y[(size_t)s_row[k] * p.width + i];
            d += e;
            any = true;
        }
        if (any) {
            v += d;
            if (p.write_back) p.x[base + i] = v;
        }
        ((OutT*)p.out1)[obase + i] = from_f32<OutT>(tanhf(a1 * v) * p.w1[i] + p.b1[i]);
        if (p.w2) {
            const float o2 = tanhf(a2 * v) * p.w2[i] + p.b2[i];
            ((OutT*)p.out2)[obase + i] = from_f32<OutT>(o2);
            if (p.out2_32) p.out2_32[obase + i] = o2;
        }
    }
}

FRB_API int frb_dyt_norm(float* x, const float* delta0, const float* delta1, const float* y, const float* ew,
                         const int* rowmap, int top_k, const int* rows, const float* w1, const float* b1,
                         const float* alpha1, void* out1, const float* w2, const float* b2, const float* alpha2, void* out2,
                         float* out2_32, int out_dtype, int num_rows, int width, int write_back, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(!(rows && write_back), "dyt_norm: chosen rows cannot be stored back");
    FRB_CHECK_ARG(!y || (top_k >= 1 && top_k <= DYT_MAX_ROWS), "dyt_norm: %d weighted rows a token are outside 1..%d", top_k, DYT_MAX_ROWS);
    DytParams p;
    p.x = x; p.delta0 = delta0; p.delta1 = delta1; p.y = y; p.ew = ew; p.rowmap = rowmap; p.rows = rows;
    p.w1 = w1; p.b1 = b1; p.alpha1 = alpha1; p.out1 = out1; p.w2 = w2; p.b2 = b2; p.alpha2 = alpha2; p.out2 = out2;
    p.out2_32 = out2_32; p.top_k = top_k; p.width = width; p.write_back = write_back;
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(dyt_norm_kernel<OutT>, dim3(num_rows), dim3(ROW_BLOCK), 0, stream, p);
    });
    FRB_RETURN_LAUNCH("dyt_norm");
}

// ---------------------------------------------------------------------------------------------------- rms_blend

__global__ void __launch_bounds__(ROW_BLOCK) rms_blend_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                              const float* __restrict__ wa, const float* __restrict__ wb,
                                                              float* __restrict__ out, int width, float eps, float share) {
    __shared__ float scratch[64];
    after_previous_kernel();
    const size_t base = (size_t)blockIdx.x * width;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < width; i += ROW_BLOCK) {
        const float va = a[base + i], vb = b[base + i];
        sa += va * va;
        sb += vb * vb;
    }
    block_sum_pair<ROW_BLOCK>(sa, sb, scratch);
    const float ra = 1.0f / sqrtf(sa / (float)width + eps), rb = 1.0f / sqrtf(sb / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += ROW_BLOCK)
        out[base + i] = share * (a[base + i] * ra * wa[i] + b[base + i] * rb * wb[i]);
}

FRB_API int frb_rms_blend(const float* a, const float* b, const float* wa, const float* wb, float* out, int num_rows,
                          int width, float eps, float share, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    launch_dependent(rms_blend_kernel, dim3(num_rows), dim3(ROW_BLOCK), 0, stream, a, b, wa, wb, out, width, eps, share);
    FRB_RETURN_LAUNCH("rms_blend");
}

// ---------------------------------------------------------------------------------------------------- concat, add

template <typename OutT>
__global__ void __launch_bounds__(ROW_BLOCK) concat_rows_kernel(float* a, const float* __restrict__ delta,
                                                                const float* __restrict__ b, OutT* __restrict__ out, int wa,
                                                                int wb) {
    after_previous_kernel();
    const size_t r = blockIdx.x;
    for (int i = threadIdx.x; i < wa + wb; i += ROW_BLOCK) {
        float v;
        if (i < wa) {
            v = a[r * wa + i];
            if (delta) v += delta[r * wa + i];
        } else {
            v = b[r * wb + i - wa];
        }
        out[r * (wa + wb) + i] = from_f32<OutT>(v);
    }
}

FRB_API int frb_concat_rows(float* a, const float* delta, const float* b, void* out, int out_dtype, int num_rows, int wa,
                            int wb, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(concat_rows_kernel<OutT>, dim3(num_rows), dim3(ROW_BLOCK), 0, stream, a, delta, b, (OutT*)out, wa, wb);
    });
    FRB_RETURN_LAUNCH("concat_rows");
}

__global__ void __launch_bounds__(ROW_BLOCK) add_row_vector_kernel(const float* __restrict__ y, const float* __restrict__ vec,
                                                                   float* __restrict__ out, int width) {
    after_previous_kernel();
    const size_t base = (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += ROW_BLOCK) out[base + i] = y[base + i] + vec[i];
}

FRB_API int frb_add_row_vector(const float* y, const float* vec, float* out, int num_rows, int width, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    launch_dependent(add_row_vector_kernel, dim3(num_rows), dim3(ROW_BLOCK), 0, stream, y, vec, out, width);
    FRB_RETURN_LAUNCH("add_row_vector");
}

// out[t, h * vd + d] *= sigmoid(gate[t * stride + h]): a gate per token and head on an attention's output
template <typename T>
__global__ void __launch_bounds__(ROW_BLOCK) head_gate_kernel(T* __restrict__ out, const float* __restrict__ gate, int stride,
                                                              int heads, int vd) {
    after_previous_kernel();
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < heads * vd; i += ROW_BLOCK) {
        const float g = 1.0f / (1.0f + expf(-gate[t * stride + i / vd]));
        out[t * heads * vd + i] = from_f32<T>(to_f32<T>(out[t * heads * vd + i]) * g);
    }
}

FRB_API int frb_head_gate(void* out, int dtype, const float* gate, int stride, int num_rows, int heads, int vd,
                          cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_DISPATCH_DTYPE(dtype, T, {
        launch_dependent(head_gate_kernel<T>, dim3(num_rows), dim3(ROW_BLOCK), 0, stream, (T*)out, gate, stride, heads, vd);
    });
    FRB_RETURN_LAUNCH("head_gate");
}

// ---------------------------------------------------------------------------------------------------- weighted_pair

// out = ca * a + cb * b: two mixers' outputs side by side, each with a constant weight.
__global__ void __launch_bounds__(ROW_BLOCK) weighted_pair_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                                  float* __restrict__ out, size_t total, float ca, float cb) {
    after_previous_kernel();
    const size_t i = (size_t)blockIdx.x * ROW_BLOCK + threadIdx.x;
    if (i < total) out[i] = ca * a[i] + cb * b[i];
}

FRB_API int frb_weighted_pair(const float* a, const float* b, float* out, long long total, float ca, float cb, cudaStream_t stream) {
    if (total == 0) return 0;
    launch_dependent(weighted_pair_kernel, dim3((unsigned)((total + ROW_BLOCK - 1) / ROW_BLOCK)), dim3(ROW_BLOCK), 0, stream, a, b, out,
                     (size_t)total, ca, cb);
    FRB_RETURN_LAUNCH("weighted_pair");
}
