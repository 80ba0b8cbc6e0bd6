// Attention over shared key rows (latent_attention.cu) on the fifth-generation tensor cores, for prompts in bfloat16.
//
// A token keeps one row [c ; r] of R + P entries for all heads; head h's query against it is [a_h ; b_h], and its
// result is the softmax-weighted sum of the rows' first R entries.  So the 128 rows of a block's tile are (head, token)
// pairs of one sequence (HB heads x TQ neighbouring tokens, row = head * TQ + token), and one page of 64 key rows in
// shared memory serves all of them, as the B operand of both products:
//   S = Q K^T      tcgen05.mma 128 x 64 x (R + P): Q and the page in shared memory as pieces of 64 entries (rows of
//                  128 bytes under the 128-byte swizzle that TMA writes), both K-major, S in tensor memory;
//   softmax        four warps, a thread per row: S comes back with tcgen05.ld, P (bfloat16) goes into tensor memory
//                  over the columns of S;
//   O += P C       tcgen05.mma 128 x RH x 64 with P as the tensor-memory operand and the SAME pieces of the page as
//                  an N-major operand (the latent entries of a key row are contiguous).
// Tensor memory holds 512 columns of 32 bits for each of the 128 rows.  A latent of more than 256 entries is therefore
// cut in two: blockIdx.z takes RH = R / 2 of its entries; both blocks compute the same scores.
// Shared memory holds Q (128 rows) and ONE page (147 + 74 KB at R + P = 576).  A page's pieces come in two groups with
// a barrier each.  The pieces that only the scores read (the rotated part, the other half of the latent) are fetched
// again as soon as the scores are done, the block's own pieces of the latent when P C is done; the scores of the next
// page start on the first group while the second is on its way.
// The running maximum of a row is only raised when a page's maximum exceeds it by more than 8 (in units of log2), so O
// is rescaled on few pages.  A block whose tokens belong to several sequences takes one sequence after the other.
//
// Every wait on an mbarrier gives up after about a second (at once when another wait of the block has given up), sets
// `status`, and the block leaves through the common exit, which frees the tensor memory.
#include "tcgen05.cuh"

#define LT_ROWS 128
#define LT_THREADS 192         // warp 0: TMA producer, warp 1: MMA issuer and tensor-memory owner, warps 2-5: softmax
#define LT_Q_PIECE (LT_ROWS * 128)      // bytes of 64 entries of all rows
#define LT_K_PIECE (FRB_PAGE * 128)     // bytes of 64 entries of a page's keys
#define LT_RAISE 8.0f
#define LT_S_COL 0
#define LT_O_COL 64

using namespace frb_tma;
using namespace frb_tc;

namespace {

__device__ __forceinline__ float lt_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// An N-major operand of pieces [keys][64 entries] (rows of 128 bytes, 128-byte swizzle): the next 64 entries along N
// lie `piece_bytes` on (leading byte offset), the next 8 keys along K 1024 bytes on (stride byte offset).
__device__ __forceinline__ uint64_t lt_desc_n_major(uint32_t addr, uint32_t piece_bytes) {
    return (uint64_t)((addr & 0x3FFFF) >> 4) | ((uint64_t)(piece_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}

__device__ __forceinline__ void lt_load_3d(void* dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_addr(dst)), "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}

}  // namespace

struct LatentTcParams {
    const int* page_table;
    const int* tok_pos;
    const int* tok_slot;
    bf16* out;                  // [H, T, R]
    int* status;
    float scale2;               // softmax scale * log2(e)
    int window, max_pages, num_tokens, num_heads, rank, rot_dim;
    int tokens_per_block, heads_per_block;      // TQ x HB = 128
    int half_rank;              // RH: the latent entries of one block
    uint32_t tmem_cols;
    int chunk_pages;            // > 0 (single tokens, TQ = 1): grid.x counts (token, chunk) pairs; a block takes the pages
    int num_chunks;             // [z, z + 1) * chunk_pages of its token and leaves unnormalised sums [Z, H, T, R] and
    float* part_o;              // (maximum in use, sum of weights) [Z, H, T, 2] for the join (latent_combine_kernel)
    float* part_ml;
};

// the run of tokens of one sequence that starts at token `begin` of the block
struct LatentTcRun {
    int begin, end, slot, first_page, pages;
};

__device__ __forceinline__ LatentTcRun lt_run(const LatentTcParams& p, int t0, int begin, int chunk) {
    LatentTcRun r;
    const int TQ = p.tokens_per_block, T = p.num_tokens;
    r.begin = begin;
    r.slot = p.tok_slot[t0 + begin];
    r.end = begin + 1;
    while (r.end < TQ && t0 + r.end < T && p.tok_slot[t0 + r.end] == r.slot) ++r.end;
    int lo = 0x7fffffff, hi = -1;
    for (int i = r.begin; i < r.end; ++i) {
        const int pos = p.tok_pos[t0 + i];
        lo = min(lo, first_visible_key(pos, p.window, 0));
        hi = max(hi, pos);
    }
    r.first_page = lo / FRB_PAGE;
    int last_page = hi / FRB_PAGE;
    if (p.chunk_pages > 0) {
        r.first_page = max(r.first_page, chunk * p.chunk_pages);
        last_page = min(last_page, (chunk + 1) * p.chunk_pages - 1);
    }
    r.pages = last_page - r.first_page + 1;              // none (or less) if the chunk holds no visible key
    return r;
}

__global__ void __launch_bounds__(LT_THREADS)
latent_attention_tc_kernel(const __grid_constant__ CUtensorMap map_ql, const __grid_constant__ CUtensorMap map_qr,
                           const __grid_constant__ CUtensorMap map_k, LatentTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t q_full, first_full, second_full, s_full, p_full, pv_done;
    __shared__ uint32_t tmem_slot;
    __shared__ int failed_flag;
    volatile int* failed = &failed_flag;

    let_next_kernel_start();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int TQ = p.tokens_per_block, HB = p.heads_per_block, T = p.num_tokens, H = p.num_heads;
    const int chunk = p.chunk_pages > 0 ? (int)blockIdx.x % p.num_chunks : 0;
    const int t0 = p.chunk_pages > 0 ? (int)blockIdx.x / p.num_chunks : (int)blockIdx.x * TQ, h0 = blockIdx.y * HB;
    if (p.chunk_pages > 0) {                                   // a chunk without a visible key ends here (every thread
        wait_for_previous_kernel();                            // alike, before any barrier and any tensor memory)
        if (lt_run(p, t0, 0, chunk).pages <= 0) return;
    }
    const int R = p.rank, RH = p.half_rank;
    const int latent_pieces = R / 64, pieces = (R + p.rot_dim) / 64;
    const int own0 = (int)blockIdx.z * (RH / 64), own1 = own0 + RH / 64;      // this block's pieces of the latent

    uint8_t* base = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* q_s = base;                                       // [pieces][128 rows][128 bytes]
    uint8_t* k_s = base + (size_t)pieces * LT_Q_PIECE;         // [pieces][64 keys][128 bytes]

    if (threadIdx.x == 0) {
        bar_init(&q_full, 1);
        bar_init(&first_full, 1);
        bar_init(&second_full, 1);
        bar_init(&s_full, 1);
        bar_init(&p_full, 4);
        bar_init(&pv_done, 1);
        failed_flag = 0;
        bar_init_fence();
    }
    if (warp == 1) tmem_alloc(&tmem_slot, p.tmem_cols);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem = tmem_slot;
    wait_for_previous_kernel();

    if (warp == 0) {
        if (lane == 0) {
            const int heads_here = min(HB, H - h0), rot_pieces = pieces - latent_pieces;
            bar_expect(&q_full, (uint32_t)latent_pieces * LT_Q_PIECE + (uint32_t)heads_here * rot_pieces * TQ * 128);
            for (int c = 0; c < latent_pieces; ++c) lt_load_3d(q_s + (size_t)c * LT_Q_PIECE, &map_ql, c * 64, t0, h0, &q_full);
            for (int c = 0; c < rot_pieces; ++c)
                for (int hh = 0; hh < heads_here; ++hh)
                    load_2d(q_s + (size_t)(latent_pieces + c) * LT_Q_PIECE + (size_t)hh * TQ * 128, &map_qr,
                            (h0 + hh) * p.rot_dim + c * 64, t0, &q_full);
            int n = 0, begin = 0;
            bool ok = true;
            while (ok && begin < TQ && t0 + begin < T) {
                const LatentTcRun run = lt_run(p, t0, begin, chunk);
                const int* table = p.page_table + (size_t)run.slot * p.max_pages;
                for (int j = 0; j < run.pages && ok; ++j, ++n) {
                    const int page = max(table[run.first_page + j], 0);
                    // the pieces that only the scores read: free when the scores of the page before are done
                    if (n > 0 && !bar_wait(&s_full, (n - 1) & 1, failed)) { atomicExch(p.status, 21); ok = false; break; }
                    bar_expect(&first_full, (uint32_t)(pieces - (own1 - own0)) * LT_K_PIECE);
                    for (int c = 0; c < pieces; ++c)
                        if (c < own0 || c >= own1) load_2d(k_s + (size_t)c * LT_K_PIECE, &map_k, c * 64, page * FRB_PAGE, &first_full);
                    // the block's own pieces of the latent: free when P C of the page before is done
                    if (n > 0 && !bar_wait(&pv_done, (n - 1) & 1, failed)) { atomicExch(p.status, 22); ok = false; break; }
                    bar_expect(&second_full, (uint32_t)(own1 - own0) * LT_K_PIECE);
                    for (int c = own0; c < own1; ++c) load_2d(k_s + (size_t)c * LT_K_PIECE, &map_k, c * 64, page * FRB_PAGE, &second_full);
                }
                begin = run.end;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // float32 accumulate, bfloat16 operands.  S: M 128 x N 64, both operands K-major.  O: M 128 x N RH, A from tensor
            // memory, B N-major (bit 16).  The MMAs of this thread run in the order of their issue, so the scores of a page
            // may be asked for over the columns that P C of the page before still reads.
            const uint32_t idesc_s = instr_desc_bf16(LT_ROWS, FRB_PAGE);
            const uint32_t idesc_o = instr_desc_bf16(LT_ROWS, RH) | (1u << 16);
            const uint64_t q_desc = tile_desc(smem_addr(q_s)), k_desc = tile_desc(smem_addr(k_s));
            bool ok = bar_wait(&q_full, 0, failed);
            if (!ok) atomicExch(p.status, 23);
            int n = 0, begin = 0;
            while (ok && begin < TQ && t0 + begin < T) {
                const LatentTcRun run = lt_run(p, t0, begin, chunk);
                for (int j = 0; j < run.pages && ok; ++j, ++n) {
                    if (!bar_wait(&first_full, n & 1, failed)) { atomicExch(p.status, 24); ok = false; break; }
                    fence_after_sync();
                    uint32_t accumulate = 0;
                    for (int c = 0; c < pieces; ++c) {
                        if (c >= own0 && c < own1) continue;
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            mma_ss(tmem + LT_S_COL, q_desc + ((c * LT_Q_PIECE + k * 32) >> 4), k_desc + ((c * LT_K_PIECE + k * 32) >> 4),
                                   idesc_s, accumulate);
                            accumulate = 1;
                        }
                    }
                    if (!bar_wait(&second_full, n & 1, failed)) { atomicExch(p.status, 24); ok = false; break; }
                    fence_after_sync();
                    for (int c = own0; c < own1; ++c)
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            mma_ss(tmem + LT_S_COL, q_desc + ((c * LT_Q_PIECE + k * 32) >> 4), k_desc + ((c * LT_K_PIECE + k * 32) >> 4),
                                   idesc_s, accumulate);
                            accumulate = 1;
                        }
                    mma_commit(&s_full);
                    if (!bar_wait(&p_full, n & 1, failed)) { atomicExch(p.status, 25); ok = false; break; }
                    fence_after_sync();
#pragma unroll
                    for (int k = 0; k < 4; ++k)                // 16 keys per MMA: 8 columns of packed P, 16 rows of the page
                        mma_ts(tmem + LT_O_COL, tmem + LT_S_COL + 8 * k,
                               lt_desc_n_major(smem_addr(k_s + (size_t)own0 * LT_K_PIECE + k * 16 * 128), LT_K_PIECE), idesc_o,
                               (j | k) != 0);
                    mma_commit(&pv_done);
                }
                begin = run.end;
            }
        }
    } else {
        // Softmax: the thread's row of the tile = its lane of tensor memory.  A wait that gives up does not end the loops:
        // the block's later waits then return at once, and every thread reaches the barriers of the end.
        const int quarter = warp & 3, row = quarter * 32 + lane;
        const int ti = row % TQ, head = h0 + row / TQ, tok = t0 + ti;
        const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_mine = lane_base + LT_S_COL, o_mine = lane_base + LT_O_COL;
        bool ok = true;
        int n = 0, begin = 0;
        while (begin < TQ && t0 + begin < T) {
            const LatentTcRun run = lt_run(p, t0, begin, chunk);
            const bool valid = tok < T && head < H && ti >= run.begin && ti < run.end;
            const int hi = valid ? p.tok_pos[tok] : -1;
            const int lo = valid ? first_visible_key(hi, p.window, 0) : 0;
            float m_used = -INFINITY, l_sum = 0.f;
            bool begun = false;
            for (int j = 0; j < run.pages; ++j, ++n) {
                if (!bar_wait(&s_full, n & 1, failed)) { if (ok && lane == 0) atomicExch(p.status, 26); ok = false; }
                fence_after_sync();
                const int key0 = (run.first_page + j) * FRB_PAGE;
                uint32_t raw[FRB_PAGE / 16][16];
#pragma unroll
                for (int c = 0; c < FRB_PAGE / 16; ++c) tmem_ld16(s_mine + 16 * c, raw[c]);
                tmem_wait_ld();
                // a page wholly before the run's first query (and inside every window) has no masked key for any row
                const bool open_page = __all_sync(0xffffffffu, valid && key0 + FRB_PAGE - 1 <= hi && key0 >= lo);
                float step_max = -INFINITY;
                if (open_page) {
                    float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                    for (int c = 0; c < FRB_PAGE / 16; ++c)
#pragma unroll
                        for (int i = 0; i < 16; ++i) top[i & 3] = fmaxf(top[i & 3], __uint_as_float(raw[c][i]));
                    step_max = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3])) * p.scale2;      // the scale is positive
                } else {
#pragma unroll
                    for (int c = 0; c < FRB_PAGE / 16; ++c)
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const int key = key0 + 16 * c + i;
                            const float v = key >= lo && key <= hi ? __uint_as_float(raw[c][i]) : -INFINITY;
                            raw[c][i] = __float_as_uint(v);
                            step_max = fmaxf(step_max, v * p.scale2);
                        }
                }
                float corr = 1.f;
                const bool raise = step_max > m_used + LT_RAISE;       // also true on the first page with a visible key
                if (raise) { corr = exp2f(m_used - step_max); m_used = step_max; }
                const float m_sub = m_used == -INFINITY ? 0.f : m_used;
                float sums[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t packed[FRB_PAGE / 32][16];
#pragma unroll
                for (int c = 0; c < FRB_PAGE / 16; ++c)
#pragma unroll
                    for (int i = 0; i < 16; i += 2) {
                        const float a = lt_exp2(fmaf(__uint_as_float(raw[c][i]), p.scale2, -m_sub));       // a masked key: 2^-inf = 0
                        const float b = lt_exp2(fmaf(__uint_as_float(raw[c][i + 1]), p.scale2, -m_sub));
                        sums[(i >> 1) & 3] += a + b;
                        packed[c >> 1][(c & 1) * 8 + (i >> 1)] = pack_bf16x2(a, b);
                    }
                l_sum = l_sum * corr + ((sums[0] + sums[1]) + (sums[2] + sums[3]));
                if (begun && __any_sync(0xffffffffu, raise)) {         // rare: O must follow the new maximum
                    if (!bar_wait(&pv_done, (n - 1) & 1, failed)) { if (ok && lane == 0) atomicExch(p.status, 27); ok = false; }
                    fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < RH / 16; ++c) {
                        uint32_t o[16];
                        tmem_ld16(o_mine + 16 * c, o);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * corr);
                        tmem_st16(o_mine + 16 * c, o);
                    }
                }
                begun = true;
#pragma unroll
                for (int c = 0; c < FRB_PAGE / 32; ++c) tmem_st16(s_mine + 16 * c, packed[c]);
                tmem_wait_st();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) bar_arrive(&p_full);
            }
            // the run's last P C has ended: this row's part of the output
            if (!bar_wait(&pv_done, (n - 1) & 1, failed)) { if (ok && lane == 0) atomicExch(p.status, 28); ok = false; }
            fence_after_sync();
            const float inv = p.chunk_pages > 0 ? 1.f : l_sum > 0.f ? 1.0f / l_sum : 0.f;
            const bool write = valid && ok && !*failed;
            float* part = nullptr;
            if (p.chunk_pages > 0 && write) {
                const size_t part_row = ((size_t)chunk * H + head) * T + tok;
                part = p.part_o + part_row * R + (size_t)blockIdx.z * RH;
                if (blockIdx.z == 0) { p.part_ml[2 * part_row] = m_used; p.part_ml[2 * part_row + 1] = l_sum; }
            }
            bf16* dst = p.out + ((size_t)(valid ? head : 0) * T + (valid ? tok : 0)) * R + (size_t)blockIdx.z * RH;
#pragma unroll 1
            for (int c = 0; c < RH / 16; ++c) {
                uint32_t o[16];
                tmem_ld16(o_mine + 16 * c, o);
                tmem_wait_ld();
                if (part) {
#pragma unroll
                    for (int i = 0; i < 16; i += 4)
                        *reinterpret_cast<float4*>(part + 16 * c + i) = make_float4(__uint_as_float(o[i]), __uint_as_float(o[i + 1]),
                                                                                   __uint_as_float(o[i + 2]), __uint_as_float(o[i + 3]));
                } else if (write) {
                    uint4 lo4, hi4;
                    lo4.x = pack_bf16x2(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv);
                    lo4.y = pack_bf16x2(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv);
                    lo4.z = pack_bf16x2(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv);
                    lo4.w = pack_bf16x2(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv);
                    hi4.x = pack_bf16x2(__uint_as_float(o[8]) * inv, __uint_as_float(o[9]) * inv);
                    hi4.y = pack_bf16x2(__uint_as_float(o[10]) * inv, __uint_as_float(o[11]) * inv);
                    hi4.z = pack_bf16x2(__uint_as_float(o[12]) * inv, __uint_as_float(o[13]) * inv);
                    hi4.w = pack_bf16x2(__uint_as_float(o[14]) * inv, __uint_as_float(o[15]) * inv);
                    reinterpret_cast<uint4*>(dst + 16 * c)[0] = lo4;
                    reinterpret_cast<uint4*>(dst + 16 * c)[1] = hi4;
                }
            }
            fence_before_sync();
            begin = run.end;
        }
    }
    fence_before_sync();
    __syncthreads();
    if (failed_flag && warp == 0 && lane == 0) {
        // copies may still be on their way into this block's shared memory: give them a bounded time to land
        int zero = 0;
        bar_wait(&q_full, 0, &zero);
        zero = 0;
        bar_wait(&first_full, 0, &zero);
        zero = 0;
        bar_wait(&second_full, 0, &zero);
    }
    __syncthreads();
    if (warp == 1) tmem_free(tmem, p.tmem_cols);
}

// ----------------------------------------------------------------------------- host side

// A map over bfloat16 [heads, tokens, cols] with boxes of [box_heads, box_tokens, 64 columns]: in shared memory a box
// is [head][token] rows of 128 bytes under the 128-byte swizzle; zeros outside.
static bool lt_map_heads_tokens(CUtensorMap* map, const void* base, uint64_t heads, uint64_t tokens, uint64_t cols,
                                uint32_t box_heads, uint32_t box_tokens) {
    EncodeFn fn = encoder();
    if (!fn) return false;
    cuuint64_t dims[3] = {cols, tokens, heads};
    cuuint64_t strides[2] = {cols * 2, tokens * cols * 2};
    cuuint32_t box[3] = {64, box_tokens, box_heads};
    cuuint32_t elem[3] = {1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

void latent_combine_launch(const int* tok_pos, int window, int chunk_keys, float* part_o, float* part_ml, void* out,
                           int num_tokens, int num_heads, int rank, cudaStream_t stream);     // latent_attention.cu

// q_lat bf16 [H, T, R]; q_rot bf16 [T, H, P]; k_pages bf16 [pages, 1, 64, R + P]; out bf16 [H, T, R].  A sequence's
// tokens lie together, in rising positions.  R and P multiples of 64, R + P at most 576, R a multiple of 128 beyond 256.
// chunk_keys > 0: every token is another sequence; a block takes one token's heads (of 128 rows the heads fill the
// first ones: the tensor cores have time to spare where the key rows come from memory once for a single token) and
// the keys [z, z + 1) * chunk_keys (a multiple of 64) for one of num_chunks z; the chunks cover every position;
// part_o float32 [num_chunks, H, T, R] and part_ml float32 [num_chunks, H, T, 2] take the parts, a second kernel joins
// them.  status: one int on the device, zero before the call.
FRB_API int frb_latent_attention_tc(const void* q_lat, const void* q_rot, const void* k_pages, int num_pages,
                                    const int* page_table, int max_pages, const int* tok_pos, const int* tok_slot, void* out,
                                    int num_tokens, int num_heads, int rank, int rot_dim, float scale, int window, int* status,
                                    int chunk_keys, int num_chunks, void* part_o, void* part_ml, cudaStream_t stream) {
    if (num_tokens == 0) return 0;
    FRB_CHECK_ARG(rank >= 64 && rank % 64 == 0 && rot_dim >= 64 && rot_dim % 64 == 0 && rank + rot_dim <= 576 &&
                  (rank <= 256 || rank % 128 == 0),
                  "tcgen05 latent attention: a latent of %d and a key part of %d entries", rank, rot_dim);
    FRB_CHECK_ARG(scale > 0.f, "tcgen05 latent attention: a softmax scale of %g is not positive", (double)scale);
    FRB_CHECK_ARG(chunk_keys == 0 || (chunk_keys % FRB_PAGE == 0 && num_chunks >= 1 && num_chunks <= 1024 && part_o && part_ml &&
                                      num_heads <= LT_ROWS),
                  "tcgen05 latent attention in chunks of %d keys (%d of them, at most 1024): a multiple of %d, at most %d heads, and room for the parts",
                  chunk_keys, num_chunks, FRB_PAGE, LT_ROWS);
    int heads_per_block = 1;
    while (heads_per_block < num_heads && heads_per_block < LT_ROWS) heads_per_block *= 2;
    if (chunk_keys > 0) heads_per_block = LT_ROWS;
    const int tokens_per_block = LT_ROWS / heads_per_block;
    const int halves = rank > 256 ? 2 : 1, half_rank = rank / halves, pieces = (rank + rot_dim) / 64;
    CUtensorMap map_ql, map_qr, map_k;
    FRB_CHECK_ARG(lt_map_heads_tokens(&map_ql, q_lat, num_heads, num_tokens, rank, heads_per_block, tokens_per_block) &&
                  map_rows_of_64(&map_qr, q_rot, num_tokens, (uint64_t)num_heads * rot_dim, tokens_per_block) &&
                  map_rows_of_64(&map_k, k_pages, (uint64_t)num_pages * FRB_PAGE, rank + rot_dim, FRB_PAGE),
                  "tcgen05 latent attention: cuTensorMapEncodeTiled failed or is not available");
    LatentTcParams p;
    p.page_table = page_table; p.tok_pos = tok_pos; p.tok_slot = tok_slot; p.out = (bf16*)out; p.status = status;
    p.scale2 = scale * 1.4426950408889634f; p.window = window; p.max_pages = max_pages; p.num_tokens = num_tokens;
    p.num_heads = num_heads; p.rank = rank; p.rot_dim = rot_dim; p.tokens_per_block = tokens_per_block;
    p.heads_per_block = heads_per_block; p.half_rank = half_rank;
    p.tmem_cols = LT_O_COL + half_rank <= 128 ? 128 : LT_O_COL + half_rank <= 256 ? 256 : 512;
    p.chunk_pages = chunk_keys / FRB_PAGE; p.num_chunks = num_chunks; p.part_o = (float*)part_o; p.part_ml = (float*)part_ml;
    const size_t smem = (size_t)pieces * (LT_Q_PIECE + LT_K_PIECE) + 1024;
    dim3 grid(chunk_keys > 0 ? num_tokens * num_chunks : (num_tokens + tokens_per_block - 1) / tokens_per_block,
              (num_heads + heads_per_block - 1) / heads_per_block, halves);
    cudaFuncSetAttribute(latent_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_dependent(latent_attention_tc_kernel, grid, dim3(LT_THREADS), smem, stream, map_ql, map_qr, map_k, p);
    if (chunk_keys > 0) latent_combine_launch(tok_pos, window, chunk_keys, p.part_o, p.part_ml, out, num_tokens, num_heads, rank, stream);
    FRB_RETURN_LAUNCH("latent_attention_tc");
}
