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

// ---------------------------------------------------------------------------------------------------------------------
// latent_attention_mma: the same attention on tensor cores (mma.sync m16n8k16, bfloat16 operands, float32 scores,
// statistics and sums), for prompts and for single tokens.
//
// A block of 16 warps takes M = 16 MT rows: TQ neighbouring tokens x M / TQ heads.  All rows of one sequence read the same
// key rows, so a tile of 32 key rows [c ; r] in shared memory serves every head and every token of the block; the next
// tile is on its way (cp.async) while this one is used.  Per tile:
//   scores   warp w takes the 8 keys (w & 3) of the tile and a quarter of the row tiles: S = Q K^T over all D entries,
//            two steps of 16 entries at a time (their loads first, two sums a row tile);
//   softmax  the four warps of a row exchange their maxima through shared memory; p = exp2(s - m) goes to shared
//            memory as bfloat16, the factor for what was summed before beside it;
//   sums     warp w takes the latent entries 8 (w + 16 n) .. + 7 of all rows: O = O * factor + P C, C being the first R
//            entries of the same key rows, read transposed (ldmatrix.trans).
// Tokens of a block that belong to different sequences are taken one sequence after the other.
// Single tokens over long contexts: the keys are cut at fixed multiples of `chunk_keys`, a block per (token, chunk), and
// latent_combine_kernel joins the chunks' parts in their order.  Where the cuts lie depends on nothing but the
// positions, so a token's result is the same bit for bit whatever else the step holds.
// Sizes: R a multiple of 8 up to 512, R + P a multiple of 16.
#define LM_THREADS 512
#define LM_KEYS 32
#define LM_PSTRIDE 40
#define LM_DECODE_QSTEPS 9      // steps of 16 entries a warp takes of the scores: a quarter of (R + P) / 16 <= 36
#define LM_DECODE_STAGES 4     // tiles of key rows in shared memory in the form for single tokens of at most 16 heads

struct LatentMmaParams {
    const bf16* q_lat;          // [H, T, R]
    const bf16* q_rot;          // [T, H, P]
    const bf16* k_pages;        // [pages, 1, 64, R + P]
    const int* page_table;
    const int* tok_pos;
    const int* tok_slot;
    bf16* out;                  // [H, T, R]
    float scale2;               // softmax scale * log2(e)
    int window, max_pages, num_tokens, num_heads, rank, rot_dim;
    int tokens_per_block;       // TQ; a block's rows are TQ tokens x (M / TQ) heads
    int chunk_keys;             // > 0 (single tokens only): block z takes the keys [z, z + 1) * chunk_keys and leaves its
    float* part_o;              // unnormalised sums [Z, H, T, R] and
    float* part_ml;             // (maximum, sum of weights) [Z, H, T, 2] for latent_combine_kernel
};

__device__ __forceinline__ void lm_ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const bf16* at) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(at);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void lm_ldmatrix_x2(uint32_t& r0, uint32_t& r1, const bf16* at) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(at);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void lm_ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const bf16* at) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(at);
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(a));
}
__device__ __forceinline__ void lm_mma(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void lm_copy16(bf16* to, const bf16* from) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(to);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(a), "l"(from) : "memory");
}
// 2^x by the special-function unit (relative error about 2^-22; -inf and anything below -126 give 0)
__device__ __forceinline__ float lm_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void lm_copies_done() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

template <int MT, int NTW>
__global__ void __launch_bounds__(LM_THREADS, 1) latent_attention_mma_kernel(LatentMmaParams p) {
    after_previous_kernel();
    if (p.chunk_keys > 0) {                              // single tokens in chunks of keys: a chunk without a visible key ends here
        const int pos = p.tok_pos[blockIdx.x], z = (int)blockIdx.z;
        if (pos < z * p.chunk_keys || (z + 1) * p.chunk_keys - 1 < first_visible_key(pos, p.window, 0) / LM_KEYS * LM_KEYS) return;
    }
    constexpr int M = 16 * MT;
    constexpr int RT_S = MT >= 4 ? MT / 4 : 1;           // row tiles of a warp in the score phase
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int R = p.rank, D = p.rank + p.rot_dim, DS = D + 8, chunks = D / 8;
    bf16* q_s = reinterpret_cast<bf16*>(lm_smem);        // [M][DS]
    bf16* k_s = q_s + (size_t)M * DS;                    // [2][LM_KEYS][DS]
    bf16* p_s = k_s + (size_t)2 * LM_KEYS * DS;          // [M][LM_PSTRIDE]
    float* pmax = reinterpret_cast<float*>(p_s + M * LM_PSTRIDE);     // [4][M]
    float* corr = pmax + 4 * M;                          // [M]
    float* lsum = corr + M;                              // [4][M]
    float* mfin = lsum + 4 * M;                          // [M]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;
    const int TQ = p.tokens_per_block, HB = M / TQ;
    const int t0 = blockIdx.x * TQ, h0 = blockIdx.y * HB;
    const int T = p.num_tokens, H = p.num_heads;

    // the queries of all rows: [a_h ; b_h] per row, zeros for rows without a token or head
    for (int i = tid; i < M * chunks; i += LM_THREADS) {
        const int r = i / chunks, c = i - r * chunks;
        const int tok = t0 + r / HB, head = h0 + r % HB;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (tok < T && head < H) {
            const int d = c * 8;
            const bf16* src = d < R ? p.q_lat + ((size_t)head * T + tok) * R + d
                                    : p.q_rot + ((size_t)tok * H + head) * p.rot_dim + (d - R);
            v = *reinterpret_cast<const uint4*>(src);
        }
        *reinterpret_cast<uint4*>(q_s + (size_t)r * DS + c * 8) = v;
    }

    const int nt = warp & 3, rg = warp >> 2;
    const bool scores_here = rg * RT_S < MT;

    int seg = 0;
    while (seg < TQ && t0 + seg < T) {
        // the run of tokens of one sequence that starts at token t0 + seg
        const int slot = p.tok_slot[t0 + seg];
        int seg_end = seg + 1;
        while (seg_end < TQ && t0 + seg_end < T && p.tok_slot[t0 + seg_end] == slot) ++seg_end;
        int lo_min = 0x7fffffff, hi_max = -1;
        for (int i = seg; i < seg_end; ++i) {
            const int pos = p.tok_pos[t0 + i];
            lo_min = min(lo_min, first_visible_key(pos, p.window, 0));
            hi_max = max(hi_max, pos);
        }
        const int* table = p.page_table + (size_t)slot * p.max_pages;
        int j_begin = lo_min / LM_KEYS * LM_KEYS, j_last = hi_max;
        if (p.chunk_keys > 0) {
            j_begin = max(j_begin, (int)blockIdx.z * p.chunk_keys);
            j_last = min(j_last, ((int)blockIdx.z + 1) * p.chunk_keys - 1);
        }
        if (j_last < j_begin) { seg = seg_end; continue; }   // no key of this chunk is visible (the same for every thread)
        const int tiles = (j_last - j_begin) / LM_KEYS + 1;

        // rows of this warp in the score phase: row tile rg * RT_S + i, rows g and g + 8 of it
        int row_lo[RT_S][2], row_hi[RT_S][2];
        float m_run[RT_S][2], l_run[RT_S][2];
#pragma unroll
        for (int i = 0; i < RT_S; ++i)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = (rg * RT_S + i) * 16 + g + 8 * h;
                const int ti = r / HB, head = h0 + r % HB;
                const bool valid = scores_here && ti >= seg && ti < seg_end && head < H;
                const int pos = valid ? p.tok_pos[t0 + ti] : -1;
                row_hi[i][h] = pos;
                row_lo[i][h] = valid ? first_visible_key(pos, p.window, 0) : 0;
                m_run[i][h] = -INFINITY;
                l_run[i][h] = 0.f;
            }
        float o[MT][NTW][4];
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int n = 0; n < NTW; ++n)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[a][n][e] = 0.f;

        auto fetch_tile = [&](int tile) {
            const int j0 = j_begin + tile * LM_KEYS;
            const int page = table[j0 / FRB_PAGE];
            bf16* dst = k_s + (size_t)(tile & 1) * LM_KEYS * DS;
            const bf16* src = p.k_pages + ((size_t)(page < 0 ? 0 : page) * FRB_PAGE + j0 % FRB_PAGE) * D;
            for (int i = tid; i < LM_KEYS * chunks; i += LM_THREADS) {
                const int key = i / chunks, c = i - key * chunks;
                if (page >= 0) lm_copy16(dst + (size_t)key * DS + c * 8, src + (size_t)key * D + c * 8);
                else *reinterpret_cast<uint4*>(dst + (size_t)key * DS + c * 8) = make_uint4(0u, 0u, 0u, 0u);
            }
            asm volatile("cp.async.commit_group;\n" ::: "memory");
        };

        fetch_tile(0);
        for (int tile = 0; tile < tiles; ++tile) {
            lm_copies_done();
            __syncthreads();                             // the tile is here; everyone is done with the tile before
            if (tile + 1 < tiles) fetch_tile(tile + 1);
            const bf16* kb = k_s + (size_t)(tile & 1) * LM_KEYS * DS;
            const int j0 = j_begin + tile * LM_KEYS;

            float s[RT_S][4];
            if (scores_here) {
                float s_odd[RT_S][4];                    // every second step of 16 entries sums here: two chains a row tile
#pragma unroll
                for (int i = 0; i < RT_S; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[i][e] = s_odd[i][e] = 0.f;
                const bf16* k_at = kb + (size_t)(nt * 8 + (lane & 7)) * DS + (lane >> 3) * 8;
                const bf16* q_at = q_s + (size_t)(rg * RT_S * 16 + (lane & 15)) * DS + (lane >> 4) * 8;
                int k0 = 0;
                for (; k0 + 32 <= D; k0 += 32) {         // all loads of two steps, then their products
                    uint32_t b0, b1, b2, b3, a[RT_S][8];
                    lm_ldmatrix_x4(b0, b1, b2, b3, k_at + k0);
#pragma unroll
                    for (int i = 0; i < RT_S; ++i) {
                        lm_ldmatrix_x4(a[i][0], a[i][1], a[i][2], a[i][3], q_at + (size_t)i * 16 * DS + k0);
                        lm_ldmatrix_x4(a[i][4], a[i][5], a[i][6], a[i][7], q_at + (size_t)i * 16 * DS + k0 + 16);
                    }
#pragma unroll
                    for (int i = 0; i < RT_S; ++i) {
                        lm_mma(s[i], a[i][0], a[i][1], a[i][2], a[i][3], b0, b1);
                        lm_mma(s_odd[i], a[i][4], a[i][5], a[i][6], a[i][7], b2, b3);
                    }
                }
                if (k0 < D) {                            // D = 16 (2 n + 1): one step is left
                    uint32_t b0, b1;
                    lm_ldmatrix_x2(b0, b1, kb + (size_t)(nt * 8 + (lane & 7)) * DS + ((lane >> 3) & 1) * 8 + k0);
#pragma unroll
                    for (int i = 0; i < RT_S; ++i) {
                        uint32_t a0, a1, a2, a3;
                        lm_ldmatrix_x4(a0, a1, a2, a3, q_at + (size_t)i * 16 * DS + k0);
                        lm_mma(s[i], a0, a1, a2, a3, b0, b1);
                    }
                }
#pragma unroll
                for (int i = 0; i < RT_S; ++i)
#pragma unroll
                    for (int e = 0; e < 4; ++e) s[i][e] += s_odd[i][e];
#pragma unroll
                for (int i = 0; i < RT_S; ++i)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float mx = -INFINITY;
#pragma unroll
                        for (int d = 0; d < 2; ++d) {
                            const int j = j0 + nt * 8 + 2 * tq + d;
                            const bool seen = j >= row_lo[i][h] && j <= row_hi[i][h];
                            const float v = seen ? s[i][2 * h + d] * p.scale2 : -INFINITY;
                            s[i][2 * h + d] = v;
                            mx = fmaxf(mx, v);
                        }
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                        if (tq == 0) pmax[nt * M + (rg * RT_S + i) * 16 + g + 8 * h] = mx;
                    }
            }
            __syncthreads();
            if (scores_here) {
#pragma unroll
                for (int i = 0; i < RT_S; ++i)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int r = (rg * RT_S + i) * 16 + g + 8 * h;
                        const float m_new = fmaxf(fmaxf(m_run[i][h], fmaxf(pmax[r], pmax[M + r])), fmaxf(pmax[2 * M + r], pmax[3 * M + r]));
                        const float factor = m_new == -INFINITY ? 1.f : exp2f(m_run[i][h] - m_new);
                        const float p0 = s[i][2 * h] == -INFINITY ? 0.f : exp2f(s[i][2 * h] - m_new);
                        const float p1 = s[i][2 * h + 1] == -INFINITY ? 0.f : exp2f(s[i][2 * h + 1] - m_new);
                        l_run[i][h] = l_run[i][h] * factor + p0 + p1;
                        m_run[i][h] = m_new;
                        *reinterpret_cast<__nv_bfloat162*>(p_s + r * LM_PSTRIDE + nt * 8 + 2 * tq) = __floats2bfloat162_rn(p0, p1);
                        if (nt == 0 && tq == 0) corr[r] = factor;
                    }
            }
            __syncthreads();
            // sums: O = O * factor + P C for this warp's latent entries
#pragma unroll
            for (int a = 0; a < MT; ++a) {
                const float f0 = corr[a * 16 + g], f1 = corr[a * 16 + g + 8];
#pragma unroll
                for (int n = 0; n < NTW; ++n) { o[a][n][0] *= f0; o[a][n][1] *= f0; o[a][n][2] *= f1; o[a][n][3] *= f1; }
            }
#pragma unroll
            for (int kk = 0; kk < LM_KEYS; kk += 16) {
                uint32_t pa[MT][4];
#pragma unroll
                for (int a = 0; a < MT; ++a)
                    lm_ldmatrix_x4(pa[a][0], pa[a][1], pa[a][2], pa[a][3], p_s + (a * 16 + (lane & 15)) * LM_PSTRIDE + kk + (lane >> 4) * 8);
                uint32_t pb[NTW][2];
#pragma unroll
                for (int n = 0; n < NTW; ++n) {
                    const int d0 = (warp + LM_THREADS / 32 * n) * 8;
                    if (d0 < R) lm_ldmatrix_x2_trans(pb[n][0], pb[n][1], kb + (size_t)(kk + (lane & 15)) * DS + d0);
                }
#pragma unroll
                for (int n = 0; n < NTW; ++n) {
                    const int d0 = (warp + LM_THREADS / 32 * n) * 8;
                    if (d0 < R) {
#pragma unroll
                        for (int a = 0; a < MT; ++a) lm_mma(o[a][n], pa[a][0], pa[a][1], pa[a][2], pa[a][3], pb[n][0], pb[n][1]);
                    }
                }
            }
        }
        // the rows' sums of weights, then the output of this run's rows
        if (scores_here) {
#pragma unroll
            for (int i = 0; i < RT_S; ++i)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float l = l_run[i][h];
                    l += __shfl_xor_sync(0xffffffffu, l, 1);
                    l += __shfl_xor_sync(0xffffffffu, l, 2);
                    if (tq == 0) lsum[nt * M + (rg * RT_S + i) * 16 + g + 8 * h] = l;
                    if (tq == 0 && nt == 0) mfin[(rg * RT_S + i) * 16 + g + 8 * h] = m_run[i][h];
                }
        }
        __syncthreads();
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int r = a * 16 + g + 8 * h;
                const int ti = r / HB, head = h0 + r % HB;
                if (ti < seg || ti >= seg_end || head >= H) continue;
                const float l = lsum[r] + lsum[M + r] + lsum[2 * M + r] + lsum[3 * M + r];
                if (p.chunk_keys > 0) {
                    const size_t row = ((size_t)blockIdx.z * H + head) * T + t0 + ti;
                    if (warp == 0 && tq == 0) { p.part_ml[2 * row] = mfin[r]; p.part_ml[2 * row + 1] = l; }
#pragma unroll
                    for (int n = 0; n < NTW; ++n) {
                        const int d0 = (warp + LM_THREADS / 32 * n) * 8;
                        if (d0 < R) *reinterpret_cast<float2*>(p.part_o + row * R + d0 + 2 * tq) = make_float2(o[a][n][2 * h], o[a][n][2 * h + 1]);
                    }
                    continue;
                }
                const float inv = l > 0.f ? 1.0f / l : 0.f;
                bf16* dst = p.out + ((size_t)head * T + t0 + ti) * R;
#pragma unroll
                for (int n = 0; n < NTW; ++n) {
                    const int d0 = (warp + LM_THREADS / 32 * n) * 8;
                    if (d0 < R)
                        *reinterpret_cast<__nv_bfloat162*>(dst + d0 + 2 * tq) = __floats2bfloat162_rn(o[a][n][2 * h] * inv, o[a][n][2 * h + 1] * inv);
                }
            }
        __syncthreads();                                 // the next run writes the same shared tables
        seg = seg_end;
    }
}

// latent_decode_mma: single tokens, at most 16 heads a block (one row tile).  The form above leaves twelve of sixteen
// warps idle while four compute the scores, and passes maxima, weights and factors through shared memory with three
// barriers a tile.  Here every warp takes a key tile (w & 3) and a quarter of the D entries (w >> 2): S = sum of four
// partial products, exchanged once through shared memory.  Every warp then holds the whole 16 x 32 tile of scores in
// the accumulator layout, computes the same maxima, weights and sums, and uses its weights directly as the A operand
// of O += P C for its own latent entries (the accumulator layout of two key tiles is the A layout of sixteen keys).
// Two barriers a tile: the tile has landed, the partial products are there.
template <int NTW>
__global__ void __launch_bounds__(LM_THREADS, 1) latent_decode_mma_kernel(LatentMmaParams p) {
    after_previous_kernel();
    const int tok = blockIdx.x, h0 = blockIdx.y * 16, T = p.num_tokens, H = p.num_heads;
    const int pos = p.tok_pos[tok];
    const int lo = first_visible_key(pos, p.window, 0);
    int j_begin = lo / LM_KEYS * LM_KEYS, j_last = pos;
    if (p.chunk_keys > 0) {                              // a chunk without a visible key ends here
        j_begin = max(j_begin, (int)blockIdx.z * p.chunk_keys);
        j_last = min(j_last, ((int)blockIdx.z + 1) * p.chunk_keys - 1);
        if (j_last < j_begin) return;
    }
    extern __shared__ __align__(16) unsigned char lm_smem[];
    const int R = p.rank, D = p.rank + p.rot_dim, DS = D + 8, chunks = D / 8;
    bf16* q_s = reinterpret_cast<bf16*>(lm_smem);        // [16][DS]
    bf16* k_s = q_s + (size_t)16 * DS;                   // [LM_DECODE_STAGES][LM_KEYS][DS]
    float4* part = reinterpret_cast<float4*>(k_s + (size_t)LM_DECODE_STAGES * LM_KEYS * DS);     // [4 quarters][4 key tiles][32 lanes]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, tq = lane & 3;

    for (int i = tid; i < 16 * chunks; i += LM_THREADS) {
        const int r = i / chunks, c = i - r * chunks, head = h0 + r;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (head < H) {
            const int d = c * 8;
            const bf16* src = d < R ? p.q_lat + ((size_t)head * T + tok) * R + d
                                    : p.q_rot + ((size_t)tok * H + head) * p.rot_dim + (d - R);
            v = *reinterpret_cast<const uint4*>(src);
        }
        *reinterpret_cast<uint4*>(q_s + (size_t)r * DS + c * 8) = v;
    }
    const int* table = p.page_table + (size_t)p.tok_slot[tok] * p.max_pages;
    const int tiles = (j_last - j_begin) / LM_KEYS + 1;
    const int nt = warp & 3, quarter = warp >> 2;
    const int steps = D / 16, steps_each = (steps + 3) / 4;
    const int step_lo = min(steps, quarter * steps_each), step_hi = min(steps, step_lo + steps_each);

    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[NTW][4];
#pragma unroll
    for (int n = 0; n < NTW; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    const int my_steps = step_hi - step_lo;              // at most LM_DECODE_QSTEPS (D <= 576)
    uint32_t qf[LM_DECODE_QSTEPS][4];                    // the A operands of this warp's steps, the same for every tile

    // A tile of 32 key rows is 37 KB; one of them on its way at a time leaves the memory idle most of the time (a block
    // per SM, about a microsecond from request to arrival).  So LM_DECODE_STAGES - 1 tiles are on their way while one
    // is used.  Every turn commits one group of copies, an empty one after the last tile, so that "all but the newest
    // LM_DECODE_STAGES - 2 groups have landed" always means "this turn's tile has landed".
    // a thread's copies of a tile: 16 bytes c of key row `key`, the next one LM_THREADS places on (no division a copy)
    const int copy_key0 = tid / chunks, copy_c0 = tid - copy_key0 * chunks;
    const int copy_key_step = LM_THREADS / chunks, copy_c_step = LM_THREADS - copy_key_step * chunks;
    auto fetch_tile = [&](int tile) {
        if (tile < tiles) {
            const int j0 = j_begin + tile * LM_KEYS;
            const int page = table[j0 / FRB_PAGE];
            bf16* dst = k_s + (size_t)(tile % LM_DECODE_STAGES) * LM_KEYS * DS;
            const bf16* src = p.k_pages + ((size_t)(page < 0 ? 0 : page) * FRB_PAGE + j0 % FRB_PAGE) * D;
            for (int key = copy_key0, c = copy_c0; key < LM_KEYS;) {
                if (page >= 0) lm_copy16(dst + (size_t)key * DS + c * 8, src + (size_t)key * D + c * 8);
                else *reinterpret_cast<uint4*>(dst + (size_t)key * DS + c * 8) = make_uint4(0u, 0u, 0u, 0u);
                key += copy_key_step;
                c += copy_c_step;
                if (c >= chunks) { c -= chunks; ++key; }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    for (int ahead = 0; ahead < LM_DECODE_STAGES - 1; ++ahead) fetch_tile(ahead);
    __syncthreads();                                     // the queries are in shared memory
#pragma unroll
    for (int i = 0; i < LM_DECODE_QSTEPS; ++i) {
        qf[i][0] = qf[i][1] = qf[i][2] = qf[i][3] = 0u;
        if (i < my_steps) lm_ldmatrix_x4(qf[i][0], qf[i][1], qf[i][2], qf[i][3], q_s + (size_t)(lane & 15) * DS + (lane >> 4) * 8 + (step_lo + i) * 16);
    }
    for (int tile = 0; tile < tiles; ++tile) {
        asm volatile("cp.async.wait_group %0;\n" ::"n"(LM_DECODE_STAGES - 2) : "memory");
        __syncthreads();                                 // the tile is here; everyone is done with the tile before
        fetch_tile(tile + LM_DECODE_STAGES - 1);         // into the stage of the tile before
        const bf16* kb = k_s + (size_t)(tile % LM_DECODE_STAGES) * LM_KEYS * DS;
        const int j0 = j_begin + tile * LM_KEYS;

        // this warp's part of the scores: key tile nt, entries [16 step_lo, 16 step_hi); its queries wait in registers
        float s_even[4] = {0.f, 0.f, 0.f, 0.f}, s_odd[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const bf16* k_at = kb + (size_t)(nt * 8 + (lane & 7)) * DS + (lane >> 3) * 8 + step_lo * 16;
#pragma unroll
            for (int i = 0; i < LM_DECODE_QSTEPS; i += 2) {
                if (i + 1 < my_steps) {
                    uint32_t b0, b1, b2, b3;
                    lm_ldmatrix_x4(b0, b1, b2, b3, k_at + i * 16);
                    lm_mma(s_even, qf[i][0], qf[i][1], qf[i][2], qf[i][3], b0, b1);
                    if (i + 1 < LM_DECODE_QSTEPS) lm_mma(s_odd, qf[i + 1][0], qf[i + 1][1], qf[i + 1][2], qf[i + 1][3], b2, b3);
                } else if (i < my_steps) {
                    uint32_t b0, b1;
                    lm_ldmatrix_x2(b0, b1, kb + (size_t)(nt * 8 + (lane & 7)) * DS + ((lane >> 3) & 1) * 8 + (step_lo + i) * 16);
                    lm_mma(s_even, qf[i][0], qf[i][1], qf[i][2], qf[i][3], b0, b1);
                }
            }
        }
        part[(quarter * 4 + nt) * 32 + lane] = make_float4(s_even[0] + s_odd[0], s_even[1] + s_odd[1], s_even[2] + s_odd[2], s_even[3] + s_odd[3]);
        __syncthreads();                                 // the partial products are there

        // the whole tile of scores, in every warp: s[j] = key tile j, rows g (entries 0, 1) and g + 8 (entries 2, 3)
        float s[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 p0 = part[(0 * 4 + j) * 32 + lane], p1 = part[(1 * 4 + j) * 32 + lane];
            const float4 p2 = part[(2 * 4 + j) * 32 + lane], p3 = part[(3 * 4 + j) * 32 + lane];
            s[j][0] = (p0.x + p1.x) + (p2.x + p3.x); s[j][1] = (p0.y + p1.y) + (p2.y + p3.y);
            s[j][2] = (p0.z + p1.z) + (p2.z + p3.z); s[j][3] = (p0.w + p1.w) + (p2.w + p3.w);
        }
        float mx[2] = {-INFINITY, -INFINITY};
        if (j0 >= lo && j0 + LM_KEYS - 1 <= pos) {       // every key of the tile is visible (the scale is positive)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = j0 + 8 * j + 2 * tq + (e & 1);
                    if (key < lo || key > pos) s[j][e] = -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], s[j][e]);
                }
        }
        float factor[2], m_sub[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h] * p.scale2);
            factor[h] = m_new == -INFINITY ? 1.f : lm_exp2(m_run[h] - m_new);
            m_run[h] = m_new;
            m_sub[h] = m_new == -INFINITY ? 0.f : m_new;
        }
        float sum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float w = lm_exp2(fmaf(s[j][e], p.scale2, -m_sub[e >> 1]));      // a masked key: 2^-inf = 0
                s[j][e] = w;
                sum[e >> 1] += w;
            }
        l_run[0] = l_run[0] * factor[0] + sum[0];
        l_run[1] = l_run[1] * factor[1] + sum[1];
#pragma unroll
        for (int n = 0; n < NTW; ++n) { o[n][0] *= factor[0]; o[n][1] *= factor[0]; o[n][2] *= factor[1]; o[n][3] *= factor[1]; }
        // sums: O += P C for this warp's latent entries; the weights of key tiles 2 kk and 2 kk + 1 are the A operand
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const __nv_bfloat162 w0 = __floats2bfloat162_rn(s[2 * kk][0], s[2 * kk][1]), w1 = __floats2bfloat162_rn(s[2 * kk][2], s[2 * kk][3]);
            const __nv_bfloat162 w2 = __floats2bfloat162_rn(s[2 * kk + 1][0], s[2 * kk + 1][1]), w3 = __floats2bfloat162_rn(s[2 * kk + 1][2], s[2 * kk + 1][3]);
            const uint32_t a0 = *reinterpret_cast<const uint32_t*>(&w0), a1 = *reinterpret_cast<const uint32_t*>(&w1);
            const uint32_t a2 = *reinterpret_cast<const uint32_t*>(&w2), a3 = *reinterpret_cast<const uint32_t*>(&w3);
            uint32_t pb[NTW][2];
#pragma unroll
            for (int n = 0; n < NTW; ++n) {
                const int d0 = (warp + LM_THREADS / 32 * n) * 8;
                if (d0 < R) lm_ldmatrix_x2_trans(pb[n][0], pb[n][1], kb + (size_t)(kk * 16 + (lane & 15)) * DS + d0);
            }
#pragma unroll
            for (int n = 0; n < NTW; ++n) {
                const int d0 = (warp + LM_THREADS / 32 * n) * 8;
                if (d0 < R) lm_mma(o[n], a0, a1, a2, a3, pb[n][0], pb[n][1]);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int head = h0 + g + 8 * h;
        if (head >= H) continue;
        if (p.chunk_keys > 0) {
            const size_t row = ((size_t)blockIdx.z * H + head) * T + tok;
            if (warp == 0 && tq == 0) { p.part_ml[2 * row] = m_run[h]; p.part_ml[2 * row + 1] = l_run[h]; }
#pragma unroll
            for (int n = 0; n < NTW; ++n) {
                const int d0 = (warp + LM_THREADS / 32 * n) * 8;
                if (d0 < R) *reinterpret_cast<float2*>(p.part_o + row * R + d0 + 2 * tq) = make_float2(o[n][2 * h], o[n][2 * h + 1]);
            }
            continue;
        }
        const float inv = l_run[h] > 0.f ? 1.0f / l_run[h] : 0.f;
        bf16* dst = p.out + ((size_t)head * T + tok) * R;
#pragma unroll
        for (int n = 0; n < NTW; ++n) {
            const int d0 = (warp + LM_THREADS / 32 * n) * 8;
            if (d0 < R)
                *reinterpret_cast<__nv_bfloat162*>(dst + d0 + 2 * tq) = __floats2bfloat162_rn(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
        }
    }
}

// out[h][t][:] = sum_z 2^(m_z - m) o_z / sum_z 2^(m_z - m) l_z over the chunks that hold visible keys of token t (at most
// LM_MAX_CHUNKS).  The threads weigh the chunks, a thread every 128th; then every thread sums four entries over the
// chunks in their order.  The order of every sum depends on the token's position and the window only.
#define LM_MAX_CHUNKS 1024
#define LM_COMBINE_THREADS 128
__global__ void __launch_bounds__(LM_COMBINE_THREADS) latent_combine_kernel(LatentMmaParams p) {
    after_previous_kernel();
    __shared__ float weight[LM_MAX_CHUNKS];
    __shared__ float red[2][LM_COMBINE_THREADS / 32];
    const int t = blockIdx.x, head = blockIdx.y, T = p.num_tokens, H = p.num_heads, R = p.rank;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int pos = p.tok_pos[t];
    const int z_lo = first_visible_key(pos, p.window, 0) / LM_KEYS * LM_KEYS / p.chunk_keys, z_hi = pos / p.chunk_keys;
    const int count = min(z_hi - z_lo + 1, LM_MAX_CHUNKS);
    const float* ml0 = p.part_ml + 2 * (((size_t)z_lo * H + head) * T + t);
    const size_t ml_step = (size_t)2 * H * T;
    float m = -INFINITY;
    for (int z = tid; z < count; z += LM_COMBINE_THREADS) {
        const float2 ml = *reinterpret_cast<const float2*>(ml0 + z * ml_step);
        if (ml.y > 0.f) m = fmaxf(m, ml.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[0][warp] = m;
    __syncthreads();
    m = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
    float total = 0.f;
    for (int z = tid; z < count; z += LM_COMBINE_THREADS) {
        const float2 ml = *reinterpret_cast<const float2*>(ml0 + z * ml_step);
        const float w = ml.y > 0.f ? exp2f(ml.x - m) : 0.f;
        weight[z] = w;
        total += w * ml.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
    if (lane == 0) red[1][warp] = total;
    __syncthreads();
    total = (red[1][0] + red[1][1]) + (red[1][2] + red[1][3]);
    const float inv = total > 0.f ? 1.0f / total : 0.f;
    const float* first = p.part_o + (((size_t)z_lo * H + head) * T + t) * R;
    const size_t step = (size_t)H * T * R;                     // from a chunk's part to the next chunk's
    for (int d = 4 * tid; d < R; d += 4 * LM_COMBINE_THREADS) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int z = 0; z < count; ++z) {
            const float wz = weight[z];
            if (wz == 0.f) continue;
            const float4 v = *reinterpret_cast<const float4*>(first + z * step + d);
            acc.x = fmaf(wz, v.x, acc.x); acc.y = fmaf(wz, v.y, acc.y); acc.z = fmaf(wz, v.z, acc.z); acc.w = fmaf(wz, v.w, acc.w);
        }
        bf16* dst = p.out + ((size_t)head * T + t) * R + d;
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    }
}

// the join for the kernels of this library that leave parts by chunks of keys (latent_attention_tc.cu has one too)
void latent_combine_launch(const int* tok_pos, int window, int chunk_keys, float* part_o, float* part_ml, void* out,
                           int num_tokens, int num_heads, int rank, cudaStream_t stream) {
    LatentMmaParams p = {};
    p.tok_pos = tok_pos; p.window = window; p.chunk_keys = chunk_keys; p.part_o = part_o; p.part_ml = part_ml;
    p.out = (bf16*)out; p.num_tokens = num_tokens; p.num_heads = num_heads; p.rank = rank;
    launch_dependent(latent_combine_kernel, dim3(num_tokens, num_heads), dim3(LM_COMBINE_THREADS), 0, stream, p);
}

FRB_API int frb_latent_attention_mma(const void* q_lat, const void* q_rot, const void* k_pages, const int* page_table,
                                     int max_pages, const int* tok_pos, const int* tok_slot, void* out, int num_tokens,
                                     int num_heads, int rank, int rot_dim, float scale, int window, int single_tokens,
                                     int chunk_keys, int num_chunks, void* part_o, void* part_ml, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(rank >= 8 && rank <= 512 && rank % 8 == 0 && (rank + rot_dim) % 16 == 0 && rot_dim >= 0,
                  "latent attention on tensor cores: a latent of %d and a key part of %d entries", rank, rot_dim);
    FRB_CHECK_ARG(scale > 0.f, "latent attention on tensor cores: a softmax scale of %g is not positive", (double)scale);
    int padded_heads = 1;
    while (padded_heads < num_heads && padded_heads < 64) padded_heads *= 2;
    int rows, per_block;
    if (single_tokens) {                                 // every token is another sequence: a block per token
        rows = padded_heads <= 16 ? 16 : padded_heads;
        per_block = 1;
    } else {
        rows = 64;
        while (rows > 16 && (long long)num_tokens * padded_heads <= rows / 2) rows /= 2;
        if (padded_heads > rows) padded_heads = rows;
        per_block = rows / padded_heads;
    }
    const int heads_per_block = rows / per_block;
    LatentMmaParams p;
    p.q_lat = (const bf16*)q_lat; p.q_rot = (const bf16*)q_rot; p.k_pages = (const bf16*)k_pages; p.page_table = page_table;
    p.tok_pos = tok_pos; p.tok_slot = tok_slot; p.out = (bf16*)out; p.scale2 = scale * 1.4426950408889634f; p.window = window;
    p.max_pages = max_pages; p.num_tokens = num_tokens; p.num_heads = num_heads; p.rank = rank; p.rot_dim = rot_dim;
    p.tokens_per_block = per_block;
    FRB_CHECK_ARG(chunk_keys == 0 || (single_tokens && chunk_keys % LM_KEYS == 0 && num_chunks >= 1 && num_chunks <= LM_MAX_CHUNKS && part_o && part_ml),
                  "latent attention in chunks of %d keys (%d of them, at most 1024): single tokens, a multiple of %d, and room for the parts",
                  chunk_keys, num_chunks, LM_KEYS);
    p.chunk_keys = chunk_keys; p.part_o = (float*)part_o; p.part_ml = (float*)part_ml;
    const int DS = rank + rot_dim + 8;
    const size_t smem = ((size_t)rows * DS + (size_t)2 * LM_KEYS * DS + (size_t)rows * LM_PSTRIDE) * sizeof(bf16) + (size_t)10 * rows * sizeof(float);
    dim3 grid((num_tokens + per_block - 1) / per_block, (num_heads + heads_per_block - 1) / heads_per_block, chunk_keys > 0 ? num_chunks : 1);
#define FRB_LATENT_MMA(MT, NTW)                                                                                        \
    do {                                                                                                               \
        auto kernel = latent_attention_mma_kernel<MT, NTW>;                                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        launch_dependent(kernel, grid, dim3(LM_THREADS), smem, stream, p);                                             \
    } while (0)
#define FRB_LATENT_MMA_ROWS(MT)                                                                                        \
    do {                                                                                                               \
        if (rank <= 128) FRB_LATENT_MMA(MT, 1);                                                                        \
        else if (rank <= 256) FRB_LATENT_MMA(MT, 2);                                                                   \
        else FRB_LATENT_MMA(MT, 4);                                                                                    \
    } while (0)
    if (single_tokens && rows == 16 && ((rank + rot_dim) / 16 + 3) / 4 <= LM_DECODE_QSTEPS) {     // one row tile: the form with every warp on the scores
        const size_t smem_one = ((size_t)16 * DS + (size_t)LM_DECODE_STAGES * LM_KEYS * DS) * sizeof(bf16) + (size_t)16 * 32 * sizeof(float4);
#define FRB_LATENT_DECODE(NTW)                                                                                         \
    do {                                                                                                               \
        auto kernel = latent_decode_mma_kernel<NTW>;                                                                   \
        if (smem_one > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_one); \
        launch_dependent(kernel, grid, dim3(LM_THREADS), smem_one, stream, p);                                         \
    } while (0)
        if (rank <= 128) FRB_LATENT_DECODE(1);
        else if (rank <= 256) FRB_LATENT_DECODE(2);
        else FRB_LATENT_DECODE(4);
#undef FRB_LATENT_DECODE
    } else if (rows == 16) FRB_LATENT_MMA_ROWS(1);
    else if (rows == 32) FRB_LATENT_MMA_ROWS(2);
    else FRB_LATENT_MMA_ROWS(4);
    if (chunk_keys > 0) launch_dependent(latent_combine_kernel, dim3(num_tokens, num_heads), dim3(LM_COMBINE_THREADS), 0, stream, p);
    FRB_RETURN_LAUNCH("latent_attention_mma");
}
