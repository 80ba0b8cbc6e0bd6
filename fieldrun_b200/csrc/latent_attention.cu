// Attention through latents: a token keeps one normed latent row c [R] and one rotated key part r [P] for all heads;
// head h's key is [U_h c ; r] and its value V_h c.  The products with U_h and V_h are moved to the query and to the
// output, so the kernels here attend with one shared key row [c ; r] of D = R + P entries per token and return
// sum_j p_j c_j, R entries per head:
//
//   score(i, j, h) = (a_h(i) . c_j + b_h(i) . r_j) * scale,   a_h = U_h^T q_h (unrotated part), b_h = rotated part
//   o_h(i) = sum_j softmax_j(score) c_j                        (the caller multiplies by V_h)
//
// The cache line holds key pages only, [pages][1][64][D]; the value of a key is the first R entries of its row.
//
// latent_prepare:  per token, from the float32 result of the down projections [q latent | kv latent | key part | ...]:
//                  RMS norms of both latents (float32), rotation of the key part, the key row into its page.
// latent_queries:  splits the up-projected queries into the unrotated parts [H][T][dim] (for the product with U_h) and
//                  the rotated parts [T][H][P], rotated at the token's position.
// latent_attention: the general kernel, float32 arithmetic, any sizes up to R = 1024.
// latent_gate:     o[h][t][:] * sigmoid(gate) -> [T][H * vdim], a gate per head or per element.
#include "common.cuh"

struct LatentPrepareParams {
    const float* down;          // [T, stride]
    int stride, q_rank, kv_rank, rot_dim, rotary_dims, interleaved;
    const float* q_weight;      // [q_rank]
    const float* kv_weight;     // [kv_rank]; null: the layer reads another layer's latents
    float eps;
    const float* cos_table;     // [positions, rotary_dims / 2]
    const float* sin_table;
    int table_positions;
    const int* tok_pos;
    const int* tok_slot;
    const int* page_table;
    int max_pages;
    void* cq_out;               // [T, q_rank]
    void* k_pages;              // [pages, 1, 64, kv_rank + rot_dim]
};

template <typename OutT, int BLOCK>
__global__ void __launch_bounds__(BLOCK) latent_prepare_kernel(LatentPrepareParams p) {
    after_previous_kernel();
    __shared__ float scratch[64];
    const int t = blockIdx.x;
    const float* row = p.down + (size_t)t * p.stride;
    const bool own = p.kv_weight != nullptr;
    float ssq = 0.f, ssk = 0.f;
    for (int i = threadIdx.x; i < p.q_rank; i += BLOCK) { const float v = row[i]; ssq += v * v; }
    if (own)
        for (int i = threadIdx.x; i < p.kv_rank; i += BLOCK) { const float v = row[p.q_rank + i]; ssk += v * v; }
    block_sum_pair<BLOCK>(ssq, ssk, scratch);
    const float rinv_q = 1.0f / sqrtf(ssq / (float)p.q_rank + p.eps);
    OutT* cq = (OutT*)p.cq_out + (size_t)t * p.q_rank;
    for (int i = threadIdx.x; i < p.q_rank; i += BLOCK) cq[i] = from_f32<OutT>(row[i] * rinv_q * p.q_weight[i]);
    if (!own) return;
    const float rinv_k = 1.0f / sqrtf(ssk / (float)p.kv_rank + p.eps);
    const int pos = p.tok_pos[t];
    const int page = p.page_table[(size_t)p.tok_slot[t] * p.max_pages + pos / FRB_PAGE];
    if (page < 0) return;
    const int width = p.kv_rank + p.rot_dim;
    OutT* key = (OutT*)p.k_pages + ((size_t)page * FRB_PAGE + pos % FRB_PAGE) * width;
    for (int i = threadIdx.x; i < p.kv_rank; i += BLOCK) key[i] = from_f32<OutT>(row[p.q_rank + i] * rinv_k * p.kv_weight[i]);
    const float* part = row + p.q_rank + p.kv_rank;
    const int half = p.rotary_dims / 2;
    const int table_row = pos < p.table_positions ? pos : p.table_positions - 1;   // positions are checked on the host
    for (int i = threadIdx.x; i < p.rot_dim; i += BLOCK) {
        float value = part[i];
        if (i < p.rotary_dims) {
            int j, partner;
            bool first;
            if (p.interleaved) { j = i >> 1; first = (i & 1) == 0; partner = first ? i + 1 : i - 1; }
            else { first = i < half; j = first ? i : i - half; partner = first ? i + half : i - half; }
            const float c = p.cos_table[(size_t)table_row * half + j], s = p.sin_table[(size_t)table_row * half + j];
            const float other = part[partner];
            value = first ? value * c - other * s : value * c + other * s;
        }
        key[p.kv_rank + i] = from_f32<OutT>(value);
    }
}

FRB_API int frb_latent_prepare(const float* down, int stride, int q_rank, int kv_rank, int rot_dim, int rotary_dims,
                               int interleaved, const float* q_weight, const float* kv_weight, float eps,
                               const float* cos_table, const float* sin_table, int table_positions, const int* tok_pos,
                               const int* tok_slot, const int* page_table, int max_pages, void* cq_out, void* k_pages,
                               int out_dtype, int num_tokens, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(rotary_dims % 2 == 0 && rotary_dims <= rot_dim, "latent attention: %d rotated entries of a key part of %d",
                  rotary_dims, rot_dim);
    FRB_CHECK_ARG(rotary_dims == 0 || (cos_table && sin_table), "latent attention: a rotation without tables");
    LatentPrepareParams p;
    p.down = down; p.stride = stride; p.q_rank = q_rank; p.kv_rank = kv_rank; p.rot_dim = rot_dim; p.rotary_dims = rotary_dims;
    p.interleaved = interleaved; p.q_weight = q_weight; p.kv_weight = kv_weight; p.eps = eps; p.cos_table = cos_table;
    p.sin_table = sin_table; p.table_positions = table_positions; p.tok_pos = tok_pos; p.tok_slot = tok_slot;
    p.page_table = page_table; p.max_pages = max_pages; p.cq_out = cq_out; p.k_pages = k_pages;
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(latent_prepare_kernel<OutT, 256>, dim3(num_tokens), dim3(256), 0, stream, p);
    });
    FRB_RETURN_LAUNCH("latent_prepare");
}

// q [T][H][dim + P] float32 -> plain [H][T][dim] and rotated [T][H][P], both OutT.
template <typename OutT>
__global__ void latent_queries_kernel(const float* __restrict__ q, OutT* __restrict__ plain, OutT* __restrict__ rotated,
                                      const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                      int table_positions, const int* __restrict__ tok_pos, int num_tokens, int heads,
                                      int dim, int rot_dim, int rotary_dims, int interleaved) {
    after_previous_kernel();
    const int per_head = dim + rot_dim;
    const size_t total = (size_t)num_tokens * heads * per_head;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t th = i / per_head;
    const int d = (int)(i - th * per_head);
    const int t = (int)(th / heads), h = (int)(th - (size_t)t * heads);
    if (d < dim) {
        plain[((size_t)h * num_tokens + t) * dim + d] = from_f32<OutT>(q[i]);
        return;
    }
    const int r = d - dim;
    float value = q[i];
    if (r < rotary_dims) {
        const int half = rotary_dims / 2;
        const int pos = tok_pos[t];
        const int table_row = pos < table_positions ? pos : table_positions - 1;
        int j, partner;
        bool first;
        if (interleaved) { j = r >> 1; first = (r & 1) == 0; partner = first ? 1 : -1; }
        else { first = r < half; j = first ? r : r - half; partner = first ? half : -half; }
        const float c = cos_table[(size_t)table_row * half + j], s = sin_table[(size_t)table_row * half + j];
        const float other = q[i + partner];
        value = first ? value * c - other * s : value * c + other * s;
    }
    rotated[((size_t)t * heads + h) * rot_dim + r] = from_f32<OutT>(value);
}

FRB_API int frb_latent_queries(const float* q, void* plain, void* rotated, int out_dtype, const float* cos_table,
                               const float* sin_table, int table_positions, const int* tok_pos, int num_tokens, int heads,
                               int dim, int rot_dim, int rotary_dims, int interleaved, cudaStream_t stream) {
    const size_t total = (size_t)num_tokens * heads * (dim + rot_dim);
    if (total == 0) return 0;
    FRB_CHECK_ARG(rotary_dims % 2 == 0 && rotary_dims <= rot_dim, "latent attention: %d rotated entries of a query part of %d",
                  rotary_dims, rot_dim);
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(latent_queries_kernel<OutT>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, q,
                         (OutT*)plain, (OutT*)rotated, cos_table, sin_table, table_positions, tok_pos, num_tokens, heads, dim,
                         rot_dim, rotary_dims, interleaved);
    });
    FRB_RETURN_LAUNCH("latent_queries");
}

struct LatentAttnParams {
    const void* q_lat;          // [H, T, R]
    const void* q_rot;          // [T, H, P]
    const void* k_pages;        // [pages, 1, 64, R + P]
    const int* page_table;      // [slots, max_pages]
    const int* tok_pos;
    const int* tok_slot;
    void* out;                  // [H, T, R]
    float scale;
    int window, max_pages, num_tokens, num_heads, rank, rot_dim;
};

#define LAT_KEYS 32
#define LAT_WARPS 8

// grid (token, blocks of LAT_WARPS heads); one warp per head, the warps share the staged key rows.
template <typename T, int ACC>
__global__ void __launch_bounds__(32 * LAT_WARPS) latent_attention_kernel(LatentAttnParams p) {
    after_previous_kernel();
    extern __shared__ float sm[];
    const int R = p.rank, P = p.rot_dim, D = R + P;
    float* k_tile = sm;                                  // [LAT_KEYS][D + 1]
    float* q_rows = k_tile + LAT_KEYS * (D + 1);         // [LAT_WARPS][D]
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y * LAT_WARPS + warp;
    const bool active = head < p.num_heads;
    const int pos = p.tok_pos[t];
    const int lo = first_visible_key(pos, p.window, 0);
    const int* table = p.page_table + (size_t)p.tok_slot[t] * p.max_pages;
    const T* k_pages = (const T*)p.k_pages;
    if (active) {
        const T* a = (const T*)p.q_lat + ((size_t)head * p.num_tokens + t) * R;
        const T* b = (const T*)p.q_rot + ((size_t)t * p.num_heads + head) * P;
        for (int d = lane; d < R; d += 32) q_rows[warp * D + d] = to_f32<T>(a[d]);
        for (int d = lane; d < P; d += 32) q_rows[warp * D + R + d] = to_f32<T>(b[d]);
    }
    float m = -INFINITY, l = 0.f;
    float acc[ACC];
#pragma unroll
    for (int i = 0; i < ACC; ++i) acc[i] = 0.f;

    for (int j0 = (lo / LAT_KEYS) * LAT_KEYS; j0 <= pos; j0 += LAT_KEYS) {
        __syncthreads();
        const int page = table[j0 / FRB_PAGE];
        const size_t base = ((size_t)page * FRB_PAGE + j0 % FRB_PAGE) * D;
        for (int i = threadIdx.x; i < LAT_KEYS * D; i += 32 * LAT_WARPS) {
            const int r = i / D, d = i - r * D;
            const bool valid = (j0 + r >= lo) && (j0 + r <= pos) && page >= 0;
            k_tile[r * (D + 1) + d] = valid ? to_f32<T>(k_pages[base + i]) : 0.f;
        }
        __syncthreads();
        if (active) {
            const int j = j0 + lane;
            const bool valid = (j >= lo) && (j <= pos);
            float s = 0.f;
            const float* qr = q_rows + warp * D;
            const float* kr = k_tile + lane * (D + 1);
            for (int d = 0; d < D; ++d) s += qr[d] * kr[d];
            s = valid ? s * p.scale : -INFINITY;
            const float m_new = fmaxf(m, warp_max(s));
            const float corr = expf(m - m_new);
            const float pj = valid ? expf(s - m_new) : 0.f;
            l = l * corr + warp_sum(pj);
#pragma unroll
            for (int i = 0; i < ACC; ++i) acc[i] *= corr;
            for (int kk = 0; kk < LAT_KEYS; ++kk) {
                const float pk = __shfl_sync(0xffffffffu, pj, kk);
#pragma unroll
                for (int i = 0; i < ACC; ++i) {
                    const int d = lane + 32 * i;
                    if (d < R) acc[i] += pk * k_tile[kk * (D + 1) + d];
                }
            }
            m = m_new;
        }
    }
    if (active) {
        const float inv = 1.0f / l;
        T* out = (T*)p.out + ((size_t)head * p.num_tokens + t) * R;
#pragma unroll
        for (int i = 0; i < ACC; ++i) {
            const int d = lane + 32 * i;
            if (d < R) out[d] = from_f32<T>(acc[i] * inv);
        }
    }
}

FRB_API int frb_latent_attention(const void* q_lat, const void* q_rot, const void* k_pages, int dtype, const int* page_table,
                                 int max_pages, const int* tok_pos, const int* tok_slot, void* out, int num_tokens,
                                 int num_heads, int rank, int rot_dim, float scale, int window, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(rank >= 1 && rank <= 1024, "latent attention: a latent of %d entries is outside 1..1024", rank);
    FRB_CHECK_ARG(rot_dim >= 0 && rot_dim <= 1024, "latent attention: a rotated key part of %d entries", rot_dim);
    LatentAttnParams p;
    p.q_lat = q_lat; p.q_rot = q_rot; p.k_pages = k_pages; p.page_table = page_table; p.tok_pos = tok_pos; p.tok_slot = tok_slot;
    p.out = out; p.scale = scale; p.window = window; p.max_pages = max_pages; p.num_tokens = num_tokens; p.num_heads = num_heads;
    p.rank = rank; p.rot_dim = rot_dim;
    const int D = rank + rot_dim;
    const size_t smem = ((size_t)LAT_KEYS * (D + 1) + (size_t)LAT_WARPS * D) * sizeof(float);
    dim3 grid(num_tokens, (num_heads + LAT_WARPS - 1) / LAT_WARPS);
#define FRB_LATENT_LAUNCH(T, ACC)                                                                                      \
    do {                                                                                                               \
        auto kernel = latent_attention_kernel<T, ACC>;                                                                 \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        launch_dependent(kernel, grid, dim3(32 * LAT_WARPS), smem, stream, p);                                         \
    } while (0)
    FRB_DISPATCH_DTYPE(dtype, T, {
        if (rank <= 128) FRB_LATENT_LAUNCH(T, 4);
        else if (rank <= 256) FRB_LATENT_LAUNCH(T, 8);
        else if (rank <= 512) FRB_LATENT_LAUNCH(T, 16);
        else FRB_LATENT_LAUNCH(T, 32);
    });
    FRB_RETURN_LAUNCH("latent_attention");
}

// o [H][T][vdim] float32, gate logits in rows of `gate_stride` floats from column `gate_column` on: one per head
// (per_head) or one per output element; out [T][H * vdim].
template <typename OutT>
__global__ void latent_gate_kernel(const float* __restrict__ o, const float* __restrict__ gate, int gate_stride,
                                   int gate_column, int per_head, OutT* __restrict__ out, int num_tokens, int heads, int vdim) {
    after_previous_kernel();
    const size_t total = (size_t)num_tokens * heads * vdim;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t th = i / vdim;
    const int j = (int)(i - th * vdim);
    const int t = (int)(th / heads), h = (int)(th - (size_t)t * heads);
    const float logit = gate[(size_t)t * gate_stride + gate_column + (per_head ? h : h * vdim + j)];
    const float value = o[((size_t)h * num_tokens + t) * vdim + j];
    out[i] = from_f32<OutT>(value / (1.0f + expf(-logit)));
}

FRB_API int frb_latent_gate(const float* o, const float* gate, int gate_stride, int gate_column, int per_head, void* out,
                            int out_dtype, int num_tokens, int heads, int vdim, cudaStream_t stream) {
    const size_t total = (size_t)num_tokens * heads * vdim;
    if (total == 0) return 0;
    FRB_DISPATCH_DTYPE(out_dtype, OutT, {
        launch_dependent(latent_gate_kernel<OutT>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, o, gate,
                         gate_stride, gate_column, per_head, (OutT*)out, num_tokens, heads, vdim);
    });
    FRB_RETURN_LAUNCH("latent_gate");
}
