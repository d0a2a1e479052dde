// Paged causal attention for steps that bring prompt portions (alone or beside decoded tokens), bfloat16.
//
// Same contract as the reference's kernel (csrc/ops/paged_attention.cu:133-383): a request's queries are the
// last n positions of its seq_len, keys 0..position come from its pages, and the rows of a tile are
// (query token x query head of one kv head) folded together (:50-74), so that a decoded token with g heads per
// kv head and a 2,048-token portion use the same code.  Built anew: 64-row tiles (16 rows per warp), 64-key
// tiles copied page row by page row with cp.async into two XOR-swizzled shared-memory stages, ldmatrix +
// mma.sync m16n8k16 (bf16 in, f32 out), running softmax in base 2 with the scores never leaving registers, an
// optional window, and the request of a tile found by a scan of query_start_loc instead of a search per thread.
//
// Cache layout of one layer: [page][0 = keys, 1 = values][kv head][slot in page][D].
#include "mma_utils.cuh"

namespace cib {

constexpr int kPfWarps = 4;
constexpr int kPfM = 64;     // rows per CTA
constexpr int kPfN = 64;     // keys per tile
constexpr int kPfStages = 2;

template <int D>
__device__ __forceinline__ void pf_load_kv_tile(__nv_bfloat16* sK, __nv_bfloat16* sV, const __nv_bfloat16* cache,
                                                const int* table, int key0, int key_end, int page_size, int num_pages,
                                                int nkv, int kvh, int tid) {
    constexpr int kChunks = D / 8;
    constexpr int kRowsPerPass = (kPfWarps * 32) / kChunks;
    constexpr int kPasses = kPfN / kRowsPerPass;
    const size_t head_stride = (size_t)page_size * D;
    const int sub_row = tid / kChunks, chunk = tid % kChunks;
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
        const int row = pass * kRowsPerPass + sub_row;
        const int j = key0 + row;
        bool valid = j < key_end;
        int page = 0, off = 0;
        if (valid) {
            page = table[j / page_size];
            off = j % page_size;
            valid = page >= 0 && page < num_pages;
        }
        const __nv_bfloat16* kp = cache + (((size_t)(valid ? page : 0) * 2) * nkv + kvh) * head_stride + (size_t)(valid ? off : 0) * D;
        const __nv_bfloat16* vp = kp + (size_t)nkv * head_stride;
        const int sw = (chunk ^ (row & 7)) * 8;
        cp_async16(sK + row * D + sw, kp + chunk * 8, valid);
        cp_async16(sV + row * D + sw, vp + chunk * 8, valid);
    }
}

template <int D>
__global__ void __launch_bounds__(kPfWarps * 32, 3)
paged_attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_stride, __nv_bfloat16* __restrict__ out,
                               int out_stride, const __nv_bfloat16* __restrict__ cache, int num_pages, int page_size,
                               const int* __restrict__ block_table, int table_stride,
                               const int* __restrict__ query_start_loc, const int* __restrict__ seq_lens,
                               int num_requests, int nq, int nkv, float scale_log2, int window, int pair) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ int s_req, s_tile, s_ntiles;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int quad = lane & 3, qrow = lane >> 2;
    const int kvh = blockIdx.y;
    const int g = nq / nkv;

    // ---- which request and which of its row tiles is this CTA? ----
    if (tid == 0) {
        // A CTA takes a pair of row tiles of one request: tile p and tile (tiles - 1 - p).  Under the causal mask
        // tile i sees about i + 1 key tiles, so every pair carries the same work and the launch ends evenly.
        int t = blockIdx.x, r = 0, tiles = 0;
        for (; r < num_requests; ++r) {
            tiles = ((query_start_loc[r + 1] - query_start_loc[r]) * g + kPfM - 1) / kPfM;
            const int pairs = pair ? (tiles + 1) / 2 : tiles;
            if (t < pairs) break;
            t -= pairs;
        }
        s_req = r;
        s_tile = t;
        s_ntiles = tiles;
    }
    __syncthreads();
    const int r = s_req;
    if (r >= num_requests) return;
    const int pair_first = s_tile, pair_second = pair ? s_ntiles - 1 - s_tile : s_tile;
    for (int which = 0; which < 2; ++which) {
    if (which == 1 && pair_second == pair_first) break;
    const int tile_index = which == 0 ? pair_second : pair_first;      // the longer one first
    __syncthreads();                                                    // shared memory of the first tile is free
    const int q0 = query_start_loc[r];
    const int n = query_start_loc[r + 1] - q0;
    const int seq_len = seq_lens[r];
    const int rows_total = n * g;
    const int row0 = tile_index * kPfM;
    const int* table = block_table + (size_t)r * table_stride;

    // two stages of (K [64][D], V [64][D]); the query tile borrows stage 1 until its fragments are in registers
    __nv_bfloat16* sKV = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* sQ = sKV + (size_t)2 * kPfN * D;
    auto stage_k = [&](int s) { return sKV + (size_t)s * 2 * kPfN * D; };
    auto stage_v = [&](int s) { return sKV + (size_t)s * 2 * kPfN * D + kPfN * D; };

    // ---- key range of the tile ----
    const int last_row = min(row0 + kPfM, rows_total) - 1;
    const int pos_first = seq_len - n + row0 / g;
    const int pos_last = seq_len - n + last_row / g;
    int k_lo = window > 0 ? max(0, pos_first - window + 1) : 0;
    k_lo = k_lo / kPfN * kPfN;
    const int k_hi = pos_last + 1;                       // keys < k_hi
    const int num_tiles = (k_hi - k_lo + kPfN - 1) / kPfN;

    // ---- Q tile -> shared (row = token_local * g + head_in_group) ----
    {
        constexpr int kChunks = D / 8;
        for (int idx = tid; idx < kPfM * kChunks; idx += kPfWarps * 32) {
            const int row = idx / kChunks, chunk = idx % kChunks;
            const int grow = row0 + row;
            const bool valid = grow < rows_total;
            const int tl = valid ? grow / g : 0, hi = valid ? grow % g : 0;
            const __nv_bfloat16* src = q + (size_t)(q0 + tl) * q_stride + (size_t)(kvh * g + hi) * D + chunk * 8;
            cp_async16(sQ + row * D + ((chunk ^ (row & 7)) * 8), src, valid);
        }
        cp_async_commit();
    }
    pf_load_kv_tile<D>(stage_k(0), stage_v(0), cache, table, k_lo, k_hi, page_size, num_pages, nkv, kvh, tid);
    cp_async_commit();

    // Q fragments of this warp's 16 rows
    cp_async_wait<1>();
    __syncthreads();
    uint32_t qf[D / 16][4];
    {
        const int mat = lane >> 3, rr = lane & 7;
        const int row = warp * 16 + (mat & 1) * 8 + rr;
#pragma unroll
        for (int kt = 0; kt < D / 16; ++kt) {
            const int chunk = 2 * kt + (mat >> 1);
            ldmatrix_x4(qf[kt], smem_u32(sQ + row * D + ((chunk ^ (row & 7)) * 8)));
        }
    }
    __syncthreads();          // every warp has its query fragments: stage 1 may now take keys and values
    // positions of this lane's two rows
    int pos_row[2];
    bool row_ok[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int grow = row0 + warp * 16 + qrow + 8 * h;
        row_ok[h] = grow < rows_total;
        pos_row[h] = row_ok[h] ? seq_len - n + grow / g : -1;
    }
    const int warp_pos_min = seq_len - n + min(row0 + warp * 16, max(rows_total - 1, 0)) / g;

    float o[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY};
    float l_run[2] = {0.f, 0.f};

    for (int t = 0; t < num_tiles; ++t) {
        const int key0 = k_lo + t * kPfN;
        if (t + 1 < num_tiles)
            pf_load_kv_tile<D>(stage_k((t + 1) % kPfStages), stage_v((t + 1) % kPfStages), cache, table, key0 + kPfN, k_hi,
                               page_size, num_pages, nkv, kvh, tid);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const __nv_bfloat16* sK = stage_k(t % kPfStages);
        const __nv_bfloat16* sV = stage_v(t % kPfStages);

        // ---- S = Q K^T : 16 x 64 per warp ----
        float s[kPfN / 8][4];
#pragma unroll
        for (int nt = 0; nt < kPfN / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
        {
            const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int kt = 0; kt < D / 16; ++kt) {
#pragma unroll
                for (int np = 0; np < kPfN / 16; ++np) {
                    const int krow = np * 16 + (mat >> 1) * 8 + rr;
                    const int chunk = 2 * kt + (mat & 1);
                    uint32_t b[4];
                    ldmatrix_x4(b, smem_u32(sK + krow * D + ((chunk ^ (krow & 7)) * 8)));
                    mma_bf16_16816(s[2 * np], qf[kt], b[0], b[1]);
                    mma_bf16_16816(s[2 * np + 1], qf[kt], b[2], b[3]);
                }
            }
        }
        // ---- scale, mask (only where the tile touches the diagonal or the window's edge) ----
        const bool need_mask = key0 + kPfN - 1 > warp_pos_min || window > 0;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < kPfN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                float v = s[nt][e] * scale_log2;
                if (need_mask) {
                    const int key = key0 + nt * 8 + quad * 2 + (e & 1);
                    const bool vis = key <= pos_row[h] && (window <= 0 || key > pos_row[h] - window);
                    v = vis ? v : -INFINITY;
                }
                s[nt][e] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            corr[h] = m_run[h] == -INFINITY ? 0.f : exp2f(m_run[h] - m_new);
            m_run[h] = m_new;
            l_run[h] *= corr[h];
        }
#pragma unroll
        for (int nt = 0; nt < kPfN / 8; ++nt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float mref = m_run[e >> 1];
                const float p = (s[nt][e] == -INFINITY || mref == -INFINITY) ? 0.f : exp2f(s[nt][e] - mref);
                s[nt][e] = p;
                l_run[e >> 1] += p;
            }
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) { o[i][0] *= corr[0]; o[i][1] *= corr[0]; o[i][2] *= corr[1]; o[i][3] *= corr[1]; }
        // ---- O += P V ----
        {
            const int mat = lane >> 3, rr = lane & 7;
#pragma unroll
            for (int kp = 0; kp < kPfN / 16; ++kp) {
                uint32_t pf[4];
                pf[0] = pack_bf16(s[2 * kp][0], s[2 * kp][1]);
                pf[1] = pack_bf16(s[2 * kp][2], s[2 * kp][3]);
                pf[2] = pack_bf16(s[2 * kp + 1][0], s[2 * kp + 1][1]);
                pf[3] = pack_bf16(s[2 * kp + 1][2], s[2 * kp + 1][3]);
                const int vrow = kp * 16 + (mat & 1) * 8 + rr;
#pragma unroll
                for (int nt = 0; nt < D / 16; ++nt) {
                    const int chunk = 2 * nt + (mat >> 1);
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, smem_u32(sV + vrow * D + ((chunk ^ (vrow & 7)) * 8)));
                    mma_bf16_16816(o[2 * nt], pf, b[0], b[1]);
                    mma_bf16_16816(o[2 * nt + 1], pf, b[2], b[3]);
                }
            }
        }
        __syncthreads();      // every warp is done with this stage before it is filled again
    }
    cp_async_wait<0>();

    // ---- normalise and store ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float l = l_run[h];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (!row_ok[h]) continue;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const int grow = row0 + warp * 16 + qrow + 8 * h;
        const int tl = grow / g, hi = grow % g;
        __nv_bfloat16* dst = out + (size_t)(q0 + tl) * out_stride + (size_t)(kvh * g + hi) * D;
#pragma unroll
        for (int nt = 0; nt < D / 8; ++nt) {
            *reinterpret_cast<uint32_t*>(dst + nt * 8 + quad * 2) = pack_bf16(o[nt][2 * h] * inv, o[nt][2 * h + 1] * inv);
        }
    }
    }   // the pair's second tile
}

template <int D>
static int launch_prefill(const void* q, int q_stride, void* out, int out_stride, const void* cache, int num_pages,
                          int page_size, const int* block_table, int table_stride, const int* query_start_loc,
                          const int* seq_lens, int num_requests, int num_tiles, int nq, int nkv, float scale, int window,
                          int pair, cudaStream_t stream) {
    const size_t smem = (size_t)(kPfStages * 2 * kPfN * D) * sizeof(__nv_bfloat16);
    static SmemLimit limit;
    if (int rc = raise_smem_limit(limit, paged_attention_prefill_kernel<D>, smem, "paged_attention_prefill")) return rc;
    dim3 grid(num_tiles, nkv);
    paged_attention_prefill_kernel<D><<<grid, kPfWarps * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)cache, num_pages,
        page_size, block_table, table_stride, query_start_loc, seq_lens, num_requests, nq, nkv,
        scale * 1.4426950408889634f, window, pair);
    CIB_LAUNCH_CHECK("paged_attention_prefill");
    return 0;
}

}  // namespace cib

using namespace cib;

extern "C" int cib_paged_attention_prefill_supports(int head_dim, int nq, int nkv) {
    return (head_dim == 64 || head_dim == 128) && nkv > 0 && nq % nkv == 0;
}

// num_tiles = number of CTAs along x: with pair = 0 the sum over requests of t_r = ceil(tokens_r * (nq / nkv) / 64);
// with pair = 1 a CTA takes the row tiles p and t_r - 1 - p of a request (equal work under the causal mask) and
// num_tiles is the sum of ceil(t_r / 2).
extern "C" int cib_paged_attention_prefill(const void* q, int q_stride, void* out, int out_stride, const void* cache,
                                           int num_pages, int page_size, const int* block_table, int table_stride,
                                           const int* query_start_loc, const int* seq_lens, int num_requests,
                                           int num_tiles, int nq, int nkv, int head_dim, float scale, int window,
                                           int pair, cudaStream_t stream) {
    CIB_REQUIRE(cib_paged_attention_prefill_supports(head_dim, nq, nkv),
                "paged_attention_prefill: head_dim %d is not taken by this kernel (64 or 128)", head_dim);
    CIB_REQUIRE(num_requests >= 0 && num_tiles >= 0 && nkv <= 65535, "paged_attention_prefill: bad sizes");
    CIB_REQUIRE(page_size > 0 && num_pages > 0 && table_stride > 0, "paged_attention_prefill: bad cache geometry");
    CIB_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && out_stride % 2 == 0 && ((uintptr_t)out % 4) == 0,
                "paged_attention_prefill: q rows must be 16-byte aligned and out rows 4-byte aligned");
    if (num_requests == 0 || num_tiles == 0) return 0;
    if (head_dim == 64)
        return launch_prefill<64>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, query_start_loc, seq_lens, num_requests, num_tiles, nq, nkv, scale, window, pair, stream);
    return launch_prefill<128>(q, q_stride, out, out_stride, cache, num_pages, page_size, block_table, table_stride, query_start_loc, seq_lens, num_requests, num_tiles, nq, nkv, scale, window, pair, stream);
}
