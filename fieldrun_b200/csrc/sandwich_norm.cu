// A sublayer's output norm, the residual sum and the next norm of the stream in one pass over a row, for blocks that
// have a norm in front of and behind each sublayer:
//
//   u = ca * a + cb * b + sum over ranks r, in rank order, of weight[r] * y[row[r]]      (each of the three may be absent)
//   v = x + u / sqrt(mean(u^2) + eps) * wu                                                the sum is stored back into x
//   out = v / sqrt(mean(v^2) + eps) * w                                                   (left out when `out` is null)
//
// All in float32; `out` is rounded to the model's type (and given in float32 as well when `out32` is set).  One block
// per output row r, src = rows ? rows[r] : r.  The row stays in shared memory between the two statistics, so the
// stream is read once and written once.  The order of every sum is fixed by the block's size, which follows the number
// of rows in the step (as the plain norm's does).
#include "common.cuh"

// A step of few rows takes blocks of 1024 threads (the row's latency is the step's), a step of many rows blocks of 256.
#define SANDWICH_FEW_ROWS 64
#define SANDWICH_MAX_TOP_K 32

struct SandwichParams {
    float* x;                 // [T, width]
    const float* a;           // [T, width] or null
    const float* b;           // [T, width] or null
    const float* y;           // [N, width] or null: expert outputs
    const float* ew;          // [T, top_k]
    const int* rowmap;        // [T * top_k]
    const int* rows;          // [R] or null
    const float* wu;          // [width]: weight of the update's norm
    const float* w;           // [width]: weight of the stream's norm (unused without out)
    void* out;                // [R, width] or null
    float* out32;             // [R, width] or null
    float ca, cb, eps_u, eps;
    int top_k, width, write_back;
};

template <typename OutT, int SANDWICH_BLOCK>
__global__ void __launch_bounds__(SANDWICH_BLOCK) sandwich_norm_kernel(SandwichParams p) {
    extern __shared__ __align__(16) float row[];         // [width]: u, then v
    __shared__ float scratch[32];
    __shared__ float s_weight[SANDWICH_MAX_TOP_K];
    __shared__ const float* s_row[SANDWICH_MAX_TOP_K];
    after_previous_kernel();
    const int r = blockIdx.x;
    const int src = p.rows ? p.rows[r] : r;
    const size_t base = (size_t)src * p.width, obase = (size_t)r * p.width;
    if (p.y) {
        if (threadIdx.x < p.top_k) {
            const size_t at = (size_t)src * p.top_k + threadIdx.x;
            s_weight[threadIdx.x] = p.ew[at];
            s_row[threadIdx.x] = p.y + (size_t)p.rowmap[at] * p.width;
        }
        __syncthreads();
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.width; i += SANDWICH_BLOCK) {
        float u = 0.f;
        if (p.a) u = p.ca * p.a[base + i];
        if (p.b) u = p.a ? fmaf(p.cb, p.b[base + i], u) : p.cb * p.b[base + i];
        if (p.y) {
            float sum = 0.f;
            for (int k = 0; k < p.top_k; ++k) sum = fmaf(s_weight[k], s_row[k][i], sum);
            u += sum;
        }
        row[i] = u;
        ss += u * u;
    }
    const float rinv_u = 1.0f / sqrtf(block_sum<SANDWICH_BLOCK>(ss, scratch) / (float)p.width + p.eps_u);
    ss = 0.f;
    for (int i = threadIdx.x; i < p.width; i += SANDWICH_BLOCK) {
        const float v = p.x[base + i] + row[i] * rinv_u * p.wu[i];
        row[i] = v;
        ss += v * v;
        if (p.write_back) p.x[base + i] = v;
    }
    if (!p.out) return;
    const float rinv = 1.0f / sqrtf(block_sum<SANDWICH_BLOCK>(ss, scratch) / (float)p.width + p.eps);
    OutT* out = (OutT*)p.out;
    for (int i = threadIdx.x; i < p.width; i += SANDWICH_BLOCK) {
        const float yv = row[i] * rinv * p.w[i];
        out[obase + i] = from_f32<OutT>(yv);
        if (p.out32) p.out32[obase + i] = yv;
    }
}

FRB_API int frb_sandwich_norm(float* x, const float* a, const float* b, float ca, float cb, const float* expert_y,
                              const float* expert_weights, const int* row_of_assign, int top_k, const int* rows, const float* wu,
                              float eps_u, const float* w, float eps, int num_rows, int width, void* out, int out_dtype, float* out32,
                              int write_back, cudaStream_t stream) {
    if (num_rows == 0) return 0;
    FRB_CHECK_ARG(a || b || expert_y, "sandwich_norm: no update was given");
    FRB_CHECK_ARG(expert_y == nullptr || (top_k >= 1 && top_k <= SANDWICH_MAX_TOP_K), "sandwich_norm: %d experts per token exceed %d",
                  top_k, SANDWICH_MAX_TOP_K);
    FRB_CHECK_ARG(out != nullptr || write_back, "sandwich_norm: neither a normed output nor the stream is to be written");
    const size_t smem = (size_t)width * sizeof(float);
    FRB_CHECK_ARG(smem <= 200 * 1024, "sandwich_norm: width %d needs %zu bytes of shared memory, more than 200 KB", width, smem);
    SandwichParams p;
    p.x = x; p.a = a; p.b = b; p.y = expert_y; p.ew = expert_weights; p.rowmap = row_of_assign; p.rows = rows; p.wu = wu; p.w = w;
    p.out = out; p.out32 = out32; p.ca = ca; p.cb = cb; p.eps_u = eps_u; p.eps = eps; p.top_k = top_k; p.width = width;
    p.write_back = write_back;
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        if (num_rows <= SANDWICH_FEW_ROWS && width >= 1024) {
            auto kernel = sandwich_norm_kernel<OutT, 1024>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_rows), dim3(1024), smem, stream, p);
        } else {
            auto kernel = sandwich_norm_kernel<OutT, 256>;
            if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            launch_dependent(kernel, dim3(num_rows), dim3(256), smem, stream, p);
        }
    });
    FRB_RETURN_LAUNCH("sandwich_norm");
}
