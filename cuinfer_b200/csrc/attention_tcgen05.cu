// Paged causal attention for prompt portions on the 5th-generation tensor cores (head size 128, bfloat16).
//
// Same contract as csrc/ops/paged_attention.cu:133-383 of the reference (queries are the last n positions of a
// request, keys 0..position come from its pages, rows of a tile are query token x query head of one kv head), on
// Blackwell's own path instead of mma.sync:
//
//   * a CTA owns a 128-row query tile (128 / g tokens x g heads of one kv head) and walks over 128-key tiles;
//   * keys and values come page by page through TMA (`cp.async.bulk.tensor.2d`, one box of 64 columns x one page per
//     copy, 128-byte swizzle: the layout the tensor cores read), issued by the lanes of the producer warps,
//     double-buffered, completion counted in bytes on mbarriers.  (Copies issued by ordinary loads or `cp.async` kept
//     too few bytes in flight per SM: a tile took longer to arrive than its softmax takes.)  The page size must be a
//     power of two of at least 8 slots, so that a box starts on a 1024-byte swizzle atom;
//   * S = Q K^T and O += P V are `tcgen05.mma.cta_group::1.kind::f16` with accumulators in tensor memory; K is a
//     K-major operand, V an MN-major one, straight from the page layout; P is the A operand of P V straight from tensor
//     memory (bfloat16, written with `tcgen05.st` over the scores it was made from), so it never touches shared memory;
//   * key tiles alternate between two sets of S, running maximum, running sum and O in tensor memory (4 x 128 columns),
//     merged at the end like the splits of a split-key kernel: S of tile j+1 is computed and P V of tile j-1 runs while
//     the sixteen softmax warps take the exponentials of tile j.  Four threads share a row (TMEM lane = row, 32 columns
//     each): they read S with one `tcgen05.ld`, keep the running maximum in base 2 and raise it only when it grows by
//     more than 8 (so O is rescaled rarely, with `tcgen05.ld`/`tcgen05.st`);
//   * a seventeenth warp's first lane issues the MMAs.
//
// Every mbarrier wait is bounded; on a time-out the kernel raises the error flag, stops, frees its tensor memory
// and returns.
#include <type_traits>

#include "common.cuh"
#include "mma_utils.cuh"
#include "tcgen05_utils.cuh"

namespace cib {
namespace fa {

constexpr int kD = 128;          // head size
constexpr int kM = 128;          // rows per CTA
constexpr int kN = 128;          // keys per tile
constexpr int kPanel = kM * 128; // bytes of one 64-column panel of a 128-row tile

// MN-major operand (values: [key][d], d contiguous), 128-byte swizzle: 64-element panels `panel_bytes` apart (leading
// offset), 8-key groups 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t desc_mnmajor(const void* smem, uint32_t panel_bytes) {
    return (uint64_t)((tc_smem_u32(smem) & 0x3ffff) >> 4) | ((uint64_t)(panel_bytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D = F32, A = B = BF16, M = 128, N = 128; b_mn: B is MN-major.
__host__ __device__ constexpr uint32_t idesc(bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void tst32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tst16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tst_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// shared memory: Q | K0 | K1 | V0 | V1, each 128 rows x 128 columns bf16 = 32 KB as two 64-column panels.  (A third key
// buffer changed nothing: what a tile waits for is the 64 KB of its keys and values crossing from the L2.)
constexpr int kTileBytes = 2 * kPanel;
constexpr int kKBufs = 2, kVBufs = 2;
constexpr int kSmemBytes = (1 + kKBufs + kVBufs) * kTileBytes + 1024 + 256;

constexpr int kMmaWarp = 16;                       // warps 0-15: the softmax
constexpr int kThreads = (kMmaWarp + 3) * 32;      // + the MMA warp, a producer warp for keys and one for values

// A operand from tensor memory (P, bfloat16, two keys to a column), B from shared memory
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a_tmem, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a_tmem), "l"(b), "r"(id), "r"(acc) : "memory");
}

__global__ void __launch_bounds__(kThreads)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap kv_map, int num_pages, const __nv_bfloat16* __restrict__ q, int q_stride,
                         __nv_bfloat16* __restrict__ out, int out_stride, int page_size,
                         const int* __restrict__ block_table, int table_stride, const int* __restrict__ query_start_loc,
                         const int* __restrict__ seq_lens, int num_requests, int nq, int nkv, float scale_log2, int window,
                         int* __restrict__ error_flag) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = base;
    unsigned char* sK = base + kTileBytes;                      // kKBufs buffers: tile j in buffer j % kKBufs
    unsigned char* sV = base + (1 + kKBufs) * kTileBytes;       // kVBufs buffers
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + (1 + kKBufs + kVBufs) * kTileBytes);
    // one barrier per buffer; key tile j uses key and value buffer and tensor-memory set j % 2
    uint64_t* k_full = bars;           // [kKBufs <= 3] a key tile has landed (bytes counted)
    uint64_t* v_full = bars + 3;       // [2] a value tile has landed
    uint64_t* s_full = bars + 5;       // [2] S of a tile is in tensor memory
    uint64_t* p_ready = bars + 7;      // [2] P of a tile is in tensor memory (16 warps arrive)
    uint64_t* pv_done = bars + 9;      // [2] the set's O includes a tile
    // With two key and two value buffers, tile j's buffers are free again exactly when s_full[j % 2] (S has read the
    // keys) and pv_done[j % 2] (P V has read the values) complete: the producers wait on those, and the thread that
    // issues the MMAs, which every tile waits for in turn, has two commits fewer per tile to issue.
    static_assert(kKBufs == 2 && kVBufs == 2, "the producers take s_full and pv_done for the buffers' release");
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    __shared__ int s_req, s_tile, s_abort, s_q0, s_n, s_seq;
    __shared__ float s_mx[2][4][128];      // [tile parity][column quarter][row]: the quarters' maxima
    __shared__ float s_l[2][4][128];       // [tile parity][column quarter][row]: the quarters' sums at the end

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x;     // heads vary fastest: every head's longest tile starts before any shorter one
    const int g = nq / nkv;

    const int g_shift = 31 - __clz(g);      // g divides 128: a power of two

    if (warp == 0) {
        // which request and which of its row tiles: the whole warp looks, 32 requests at a time (one thread walking up
        // to 64 requests took 6 us, and nothing else of the tile can start before this is known)
        int t = gridDim.y - 1 - blockIdx.y;     // later (longer) tiles first
        int req = num_requests, tile = 0;
        for (int r0 = 0; r0 < num_requests; r0 += 32) {
            const int r = r0 + lane;
            int tiles = 0;
            if (r < num_requests) tiles = ((query_start_loc[r + 1] - query_start_loc[r]) * g + kM - 1) / kM;
            int upto = tiles;                   // tiles of the requests r0 .. r
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int o = __shfl_up_sync(0xffffffffu, upto, d);
                if (lane >= d) upto += o;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, r < num_requests && t < upto);
            if (hit) {
                const int first = __ffs(hit) - 1;
                req = r0 + first;
                tile = t - (__shfl_sync(0xffffffffu, upto, first) - __shfl_sync(0xffffffffu, tiles, first));
                break;
            }
            t -= __shfl_sync(0xffffffffu, upto, 31);
        }
        if (lane == 0) {
            s_req = req; s_tile = tile; s_abort = 0;
            if (req < num_requests) {   // read here once, so that the other threads need no round trip of their own after the barrier
                s_q0 = query_start_loc[req];
                s_n = query_start_loc[req + 1] - query_start_loc[req];
                s_seq = seq_lens[req];
            }
            asm volatile("prefetch.tensormap [%0];" ::"l"(&kv_map) : "memory");
        }
    } else if (warp == 1 && lane < 16) {
        // a thread per barrier: p_ready (at 7 and 8) counts the sixteen softmax warps, all others one arrival
        mbar_init(&bars[lane], lane == 7 || lane == 8 ? kMmaWarp : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // stale shared memory must at least be finite: rows of a tile that no page covers are multiplied by P = 0
    for (int i = tid; i < (kKBufs + kVBufs) * kTileBytes / 16; i += blockDim.x) reinterpret_cast<uint4*>(sK)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // before the bulk copies write the same bytes
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    // everything so far read only what the host wrote for this step; queries, keys and values come from the kernel before
    griddep_launch();
    griddep_wait();
    const uint32_t tmem = *tmem_slot;
    const int r = s_req;
    const bool active = r < num_requests;

    int q0 = 0, n = 0, seq_len = 0, row0 = 0, rows_total = 0, num_tiles = 0, k_lo = 0;
    if (active) {
        q0 = s_q0;
        n = s_n;
        seq_len = s_seq;
        rows_total = n * g;
        row0 = s_tile * kM;
        const int last_row = min(row0 + kM, rows_total) - 1;
        const int pos_first = seq_len - n + (row0 >> g_shift), pos_last = seq_len - n + (last_row >> g_shift);
        k_lo = window > 0 ? max(0, pos_first - window + 1) / kN * kN : 0;
        num_tiles = (pos_last + 1 - k_lo + kN - 1) / kN;
    }

    if (active && warp < kMmaWarp) {
        // ---- the query tile: row = token_local * g + head_in_group, two swizzled 64-column panels ----
        // (a thread's four loads are all on their way before the first is stored: one round trip, not four)
        constexpr int kPer = kM * 16 / (kMmaWarp * 32);
        uint4 v[kPer];
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int idx = tid + u * kMmaWarp * 32;
            const int row = idx >> 4, c = idx & 15;
            const int grow = row0 + row;
            v[u] = make_uint4(0, 0, 0, 0);
            if (grow < rows_total) {
                const int tl = grow >> g_shift, hi = grow & (g - 1);
                v[u] = *reinterpret_cast<const uint4*>(q + (size_t)(q0 + tl) * q_stride + (size_t)(kvh * g + hi) * kD + c * 8);
            }
        }
#pragma unroll
        for (int u = 0; u < kPer; ++u) {
            const int idx = tid + u * kMmaWarp * 32;
            const int row = idx >> 4, c = idx & 15;
            *reinterpret_cast<uint4*>(sQ + (c >> 3) * kPanel + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = v[u];
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // the MMA warp waits for the query tile; the producer warps do not, so that the first keys and values are on their
    // way while the queries are still being copied
    if (warp <= kMmaWarp) asm volatile("bar.sync 10, %0;" ::"r"((kMmaWarp + 1) * 32) : "memory");

    // tensor memory: S of set 0 | S of set 1 | O of set 0 | O of set 1, 128 columns each; P of a set (bfloat16,
    // two keys to a column) takes the first 64 columns of the set's S once the softmax holds S in registers
    if (active && warp == kMmaWarp) {
        // ---- the MMAs: the whole warp walks the loop, lane 0 issues ----
        auto issue_s = [&](int j) {
            if (lane != 0) return;
            const int b = j & 1;
            const uint64_t qd = umma_desc_k_major_sw128(sQ), kd = umma_desc_k_major_sw128(sK + (j % kKBufs) * kTileBytes);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint64_t off = (uint64_t)(((k >> 2) * kPanel + (k & 3) * 32) >> 4);
                umma_bf16(tmem + (uint32_t)(b * kN), qd + off, kd + off, idesc(false), k != 0);
            }
            umma_commit(&s_full[b]);            // also: the key buffer can be refilled
        };
        auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
            bool ok = mbar_wait(bar, parity);
            if (!ok && lane == 0) { atomicExch(error_flag, code); s_abort = 1; }
            return __all_sync(0xffffffffu, ok);
        };
        bool ok = true;
        ok = wait_all(&k_full[0], 0, 11);
        if (ok) { tcgen05_fence_after(); issue_s(0); }
        for (int j = 0; j < num_tiles && ok; ++j) {
            const int b = j & 1;
            const uint32_t parity = (j >> 1) & 1;
            if (j + 1 < num_tiles) {
                // S(j+1) overwrites S and P of tile j-1 (same set): P V(j-1) was issued before, and the tensor pipe
                // runs what one thread issues in order
                ok = wait_all(&k_full[(j + 1) % kKBufs], ((j + 1) / kKBufs) & 1, 12);
                if (!ok) break;
                tcgen05_fence_after();
                issue_s(j + 1);
            }
            ok = wait_all(&p_ready[b], parity, 13) && wait_all(&v_full[b], parity, 14);
            if (!ok) break;
            {
                // the last page of the request came whole: value rows past its last token may hold anything, and
                // 0 x NaN is NaN, so they are cleared (their columns of P are 0)
                const int valid_rows = seq_len - (k_lo + j * kN);
                if (valid_rows < kN) {
                    const int box_rows = min(page_size, kN);
                    const int end = min(kN, (valid_rows + box_rows - 1) / box_rows * box_rows);
                    unsigned char* vb = sV + b * kTileBytes;
                    for (int idx = valid_rows * 16 + lane; idx < end * 16; idx += 32) {
                        const int row = idx >> 4, c = idx & 15;
                        *reinterpret_cast<uint4*>(vb + (c >> 3) * kPanel + row * 128 + (((c & 7) ^ (row & 7)) << 4)) = make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                }
            }
            tcgen05_fence_after();
            if (lane == 0) {
                // O_b += P V: P is the A operand straight from tensor memory (16 keys = 8 columns per step)
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const uint64_t vd = desc_mnmajor(sV + b * kTileBytes + k * 16 * 128, kPanel);
                    mma_ts(tmem + (uint32_t)(2 * kN + b * kN), tmem + (uint32_t)(b * kN + k * 8), vd, idesc(true), (j >= 2) || k != 0);
                }
                umma_commit(&pv_done[b]);        // also: the value buffer can be refilled
            }
            __syncwarp();
        }
    } else if (active && warp > kMmaWarp) {
        // ---- producer warps (first: keys, second: values; two more warps did not make the copies of a tile land sooner:
        // 64 KB per tile is what an SM fetches from the L2 in about 1.6 k cycles): a lane issues one TMA copy per (page
        // of the tile, 64-column panel); keys of tile j+2 as soon as S(j) has read its buffer, values of tile j+2 after P V(j).  Rows of a tile past the
        // request's last page are not copied: their columns of S are masked and P is 0 there.  A page number outside the
        // pool turns into a row outside the tensor map, which reads as zeros and still counts its bytes. ----
        const int* table = block_table + (size_t)r * table_stride;
        const int box_rows = min(page_size, kN);
        const int boxes = kN / box_rows;
        const long long total_rows = (long long)num_pages * 2 * nkv * page_size;
        // a tile has at most 32 boxes (16 pages of 8 slots x 2 panels): lane = box * 2 + panel.  The page number of
        // a lane's box is fetched a tile ahead, so that no copy waits for a round trip to the table.
        const int kv = warp - kMmaWarp - 1;
        const int box = lane >> 1, panel = lane & 1;
        int page = -1;
        auto lookup = [&](int t) {
            const int key = k_lo + t * kN + box * box_rows;
            page = t < num_tiles && box < boxes && key < seq_len ? __ldg(table + key / page_size) : -1;
        };
        const int depth = kv ? kVBufs : kKBufs;
        auto fill = [&](int t) {
            const int b = t % depth;
            const int key0 = k_lo + t * kN;
            uint64_t* bar = kv ? &v_full[b] : &k_full[b];
            const int nvalid = min(boxes, max(0, (seq_len - key0 + box_rows - 1) / box_rows));
            if (lane == 0) mbar_expect_tx(bar, (uint32_t)(nvalid * 2 * box_rows * 128));
            __syncwarp();
            if (box < nvalid) {
                const int off = (key0 + box * box_rows) % page_size;        // not 0 only for pages longer than a tile
                const long long row = page >= 0 && page < num_pages
                                          ? (((long long)page * 2 + kv) * nkv + kvh) * page_size + off : total_rows;
                tma_load_2d((kv ? sV : sK) + b * kTileBytes + panel * kPanel + box * box_rows * 128, &kv_map, bar, panel * 64, (int)row);
            }
        };
        auto wait_all = [&](uint64_t* bar, uint32_t parity, int code) {
            bool ok = mbar_wait(bar, parity);
            if (!ok && lane == 0) { atomicExch(error_flag, code); s_abort = 1; }
            return __all_sync(0xffffffffu, ok);
        };
        uint64_t* free_bar = kv ? pv_done : s_full;
        for (int t = 0; t < depth && t < num_tiles; ++t) {
            lookup(t);
            fill(t);
        }
        lookup(depth);
        for (int j = 0; j + depth < num_tiles; ++j) {
            if (!wait_all(&free_bar[j % depth], (j / depth) & 1, 18 + kv)) break;      // S(j) / P V(j) has read the buffer
            fill(j + depth);
            lookup(j + depth + 1);
        }
    } else if (active && warp < kMmaWarp) {
        // ---- softmax: all sixteen warps take every key tile, four threads to a row (TMEM lane) with 32 of the 128
        // columns each; warps w, w + 4, w + 8 and w + 12 share the lanes 32 * (w % 4) .. + 31 and meet at a named barrier
        // to combine a row's maxima.  Tiles alternate between two sets of scores, running maximum, running sum and
        // output accumulator (set j % 2), so that the scores of tile j + 1 are computed and the P V of tile j - 1 runs
        // while the exponentials of tile j are taken; the two sets are merged at the end. ----
        const int quarter = warp & 3, cq = warp >> 2;
        const int cb = cq * 32;
        const int row_local = quarter * 32 + lane;
        const int grow = row0 + row_local;
        const bool row_ok = grow < rows_total;
        const int pos = row_ok ? seq_len - n + (grow >> g_shift) : -1;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
        auto row_barrier = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(1 + quarter) : "memory"); };
        float m_set[2] = {-INFINITY, -INFINITY}, l_set[2] = {0.f, 0.f};     // indexed by constants only
        bool ok = true;
        // one key tile of set B (a constant after inlining); false if a wait ran out
        auto softmax_tile = [&](int j, auto set) -> bool {
            constexpr int B = decltype(set)::value;
            float& m_used = m_set[B];
            float& l = l_set[B];
            const uint32_t s_col = (uint32_t)(B * kN), o_col = (uint32_t)(2 * kN + B * kN);
            const int done = j >> 1;                    // tiles of this set before this one
            const int key0 = k_lo + j * kN;
            bool good = mbar_wait(&s_full[B], (uint32_t)(done & 1));
            if (!good && lane == 0) { atomicExch(error_flag, 15); s_abort = 1; }
            good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0 && !(*(volatile int*)&s_abort);
            if (!good) {
                row_barrier();      // a warp that gives up still meets the row's other warps at every barrier they reach
                return false;
            }
            tcgen05_fence_after();
            const bool need_mask = key0 + kN - 1 > pos || window > 0;
            const int hi = pos - key0;                              // columns <= hi are visible ...
            const int lo = window > 0 ? hi - window : -1;           // ... and > lo
            // this thread's 32 scores, read from tensor memory once; masked ones become -inf here, so that the
            // maximum (the scale is positive: applied afterwards) and the exponentials need no second look at the mask
            uint32_t v[32];
            tmem_ld_32x32b_x32(lane_addr + s_col + (uint32_t)cb, v);
            tmem_ld_wait();
            float mx = -INFINITY;
            if (need_mask) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    const int col = cb + e;
                    if (!(col <= hi && col > lo)) v[e] = __float_as_uint(-INFINITY);
                }
            }
#pragma unroll
            for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(v[e]));
            s_mx[B][cq][row_local] = mx;
            row_barrier();                          // all four threads of the row hold their scores in registers from here on
            mx = fmaxf(fmaxf(s_mx[B][0][row_local], s_mx[B][1][row_local]), fmaxf(s_mx[B][2][row_local], s_mx[B][3][row_local])) * scale_log2;
            // raise the reference maximum only when it would grow by more than 8 (values stay below 2^8); the
            // threads of a row see the same numbers and decide alike
            float corr = 1.f;
            bool rescale = false;
            if (mx > m_used + 8.f || (m_used == -INFINITY && mx != -INFINITY)) {
                corr = m_used == -INFINITY ? 0.f : exp2f(m_used - mx);
                m_used = mx;
                l *= corr;
                rescale = done > 0;
            }
            // P = 2^(s * scale - m): one fused multiply-add and one ex2 per score, packed two to a register
            const float m_eff = m_used == -INFINITY ? 0.f : m_used;
            uint32_t p[16];
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                float pe[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const float x = fmaf(__uint_as_float(v[e + u]), scale_log2, -m_eff);
                    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(pe[u]) : "f"(x));
                }
                l += pe[0] + pe[1];
                __nv_bfloat162 pk = __floats2bfloat162_rn(pe[0], pe[1]);
                p[e / 2] = *reinterpret_cast<uint32_t*>(&pk);
            }
            // the set's O is only touched once P V of its tile before has finished
            if (done > 0 && __any_sync(0xffffffffu, rescale)) {
                good = mbar_wait(&pv_done[B], (uint32_t)((done - 1) & 1));
                if (!good && lane == 0) { atomicExch(error_flag, 16); s_abort = 1; }
                good = __shfl_sync(0xffffffffu, good ? 1 : 0, 0) != 0;
                if (!good) return false;
                tcgen05_fence_after();
                uint32_t o[32];
                tmem_ld_32x32b_x32(lane_addr + o_col + (uint32_t)cb, o);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * (rescale ? corr : 1.f));
                tst32(lane_addr + o_col + (uint32_t)cb, o);
            }
            // P (bfloat16, two keys to a column): this thread's 32 keys take the columns 16 cq .. + 15, over scores
            // that the row's threads hold in registers since the barrier above
            tst16(lane_addr + s_col + (uint32_t)(cq * 16), p);
            tst_wait();
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_ready[B]);
            return true;
        };
        for (int j = 0; j < num_tiles; j += 2) {
            // after a wait has run out (never in a healthy run) only the tiles' barriers are kept, so that no warp of
            // the row is left waiting at one
            if (ok) ok = softmax_tile(j, std::integral_constant<int, 0>{});
            else row_barrier();
            if (j + 1 < num_tiles) {
                if (ok) ok = softmax_tile(j + 1, std::integral_constant<int, 1>{});
                else row_barrier();
            }
        }
        // ---- merge the two sets: O = (O_0 2^(m_0 - m) + O_1 2^(m_1 - m)) / (l_0 2^(m_0 - m) + l_1 2^(m_1 - m)) ----
        // every thread waits for the last P V of both sets itself: behind them no MMA reads shared or tensor memory
#pragma unroll
        for (int B = 0; B < 2; ++B) {
            if (ok && num_tiles > B) {
                const int last = ((num_tiles - 1 - B) >> 1);        // the set's last tile is its (last + 1)-th
                ok = mbar_wait(&pv_done[B], (uint32_t)(last & 1));
                if (!ok && lane == 0) { atomicExch(error_flag, 17); s_abort = 1; }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
        }
        s_l[0][cq][row_local] = l_set[0];
        s_l[1][cq][row_local] = l_set[1];
        tcgen05_fence_before();
        row_barrier();                  // the four threads of a row
        tcgen05_fence_after();
        if (!(*(volatile int*)&s_abort) && num_tiles > 0) {
            // this thread stores the output columns 32 cq .. + 31 of its row
            const float m0 = m_set[0], m1 = m_set[1];
            const float l0 = (s_l[0][0][row_local] + s_l[0][1][row_local]) + (s_l[0][2][row_local] + s_l[0][3][row_local]);
            const float l1 = (s_l[1][0][row_local] + s_l[1][1][row_local]) + (s_l[1][2][row_local] + s_l[1][3][row_local]);
            const float m = fmaxf(m0, m1);
            const float w0 = m0 == -INFINITY ? 0.f : exp2f(m0 - m), w1 = m1 == -INFINITY ? 0.f : exp2f(m1 - m);
            const float total = l0 * w0 + l1 * w1;
            // (total is at least 2^-8 for a row with a visible key and at most a few thousand)
            const float inv = total > 0.f ? __fdividef(1.f, total) : 0.f;
            const float f0 = w0 * inv, f1 = w1 * inv;
            const bool has1 = num_tiles > 1;        // set 1 has an accumulator only if there was a second tile
            uint32_t a[32], b[32];
            tmem_ld_32x32b_x32(lane_addr + (uint32_t)(2 * kN + cb), a);
            if (has1) tmem_ld_32x32b_x32(lane_addr + (uint32_t)(3 * kN + cb), b);
            tmem_ld_wait();
            // into the query tile's shared memory (every S has read it), a row's 256 bytes together, its 16-byte pieces
            // swapped by the row number so that neither these stores nor the loads below meet in a bank
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
                float y[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    y[u] = __uint_as_float(a[e + u]) * f0;
                    if (has1) y[u] = fmaf(__uint_as_float(b[e + u]), f1, y[u]);
                }
                uint4 pk;
                __nv_bfloat162 t0 = __floats2bfloat162_rn(y[0], y[1]), t1 = __floats2bfloat162_rn(y[2], y[3]);
                __nv_bfloat162 t2 = __floats2bfloat162_rn(y[4], y[5]), t3 = __floats2bfloat162_rn(y[6], y[7]);
                pk.x = *reinterpret_cast<uint32_t*>(&t0); pk.y = *reinterpret_cast<uint32_t*>(&t1);
                pk.z = *reinterpret_cast<uint32_t*>(&t2); pk.w = *reinterpret_cast<uint32_t*>(&t3);
                const int piece = (cb + e) >> 3;
                *reinterpret_cast<uint4*>(sQ + row_local * 256 + ((piece ^ (row_local & 15)) << 4)) = pk;
            }
        }
        // out to global memory sixteen threads to a row: a thread that stored its own row's pieces sent 32 partial
        // sectors with every instruction, and the tile's 2 048 of them took 1.5 us
        asm volatile("bar.sync 9, %0;" ::"r"(kMmaWarp * 32) : "memory");
        if (!(*(volatile int*)&s_abort) && num_tiles > 0) {
#pragma unroll
            for (int u = 0; u < kM * 16 / (kMmaWarp * 32); ++u) {
                const int idx = tid + u * kMmaWarp * 32;
                const int row = idx >> 4, c = idx & 15;
                const int grow_out = row0 + row;
                if (grow_out < rows_total) {
                    const uint4 pk = *reinterpret_cast<const uint4*>(sQ + row * 256 + ((c ^ (row & 15)) << 4));
                    const int tl = grow_out >> g_shift, hh = grow_out & (g - 1);
                    *reinterpret_cast<uint4*>(out + (size_t)(q0 + tl) * out_stride + (size_t)(kvh * g + hh) * kD + c * 8) = pk;
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
}

}  // namespace fa
}  // namespace cib

using namespace cib;


extern "C" int cib_attention_tcgen05_supports(int head_dim, int nq, int nkv, int page_size) {
    if (head_dim != 128 || nkv <= 0 || nq % nkv != 0) return 0;
    const int g = nq / nkv;
    return 128 % g == 0 && page_size >= 8 && (page_size & (page_size - 1)) == 0;
}

// num_tiles = sum over requests of ceil(tokens_r * (nq / nkv) / 128).  error_flag: one zero int in device memory.
extern "C" int cib_attention_tcgen05(const void* q, int q_stride, void* out, int out_stride, const void* cache, int num_pages,
                                     int page_size, const int* block_table, int table_stride, const int* query_start_loc,
                                     const int* seq_lens, int num_requests, int num_tiles, int nq, int nkv, int head_dim,
                                     float scale, int window, int* error_flag, cudaStream_t stream) {
    CIB_REQUIRE(cib_attention_tcgen05_supports(head_dim, nq, nkv, page_size),
                "attention_tcgen05: head_dim %d, %d/%d heads, page size %d are not taken (head size 128, heads per kv head dividing 128, pages of 8, 16, 32, ... slots)",
                head_dim, nq, nkv, page_size);
    CIB_REQUIRE(num_requests >= 0 && num_tiles >= 0 && num_tiles <= 65535 && num_pages > 0 && table_stride > 0, "attention_tcgen05: bad sizes");
    CIB_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && out_stride % 8 == 0 && ((uintptr_t)out % 16) == 0 && ((uintptr_t)cache % 16) == 0,
                "attention_tcgen05: rows must be 16-byte aligned");
    CIB_REQUIRE(error_flag != nullptr, "attention_tcgen05: error flag missing");
    if (num_requests == 0 || num_tiles == 0) return 0;
    // the cache as rows of one head's slot: [pages * 2 * kv heads * page_size, 128]; a box is one page x 64 columns
    const long long total_rows = (long long)num_pages * 2 * nkv * page_size;
    CIB_REQUIRE(total_rows < (1ll << 31), "attention_tcgen05: %lld cache rows do not fit a 32-bit coordinate", total_rows);
    CUtensorMap kv_map;
    if (encode_tensor_map_bf16_2d(&kv_map, cache, (unsigned long long)total_rows, fa::kD, fa::kD, 64,
                                  page_size < fa::kN ? page_size : fa::kN, "attention_tcgen05") != 0)
        return -1;
    static SmemLimit limit;
    if (int rc = raise_smem_limit(limit, fa::attention_tcgen05_kernel, fa::kSmemBytes, "attention_tcgen05")) return rc;
    dim3 grid(nkv, num_tiles);
    cudaError_t e = launch_pdl(fa::attention_tcgen05_kernel, grid, dim3(fa::kThreads), (size_t)fa::kSmemBytes, stream, prompt_pdl(),
                               kv_map, num_pages, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)out, out_stride, page_size,
                               block_table, table_stride, query_start_loc, seq_lens, num_requests, nq, nkv,
                               scale * 1.4426950408889634f, window, error_flag);
    if (e != cudaSuccess) {
        set_error("attention_tcgen05: launch failed: %s", cudaGetErrorString(e));
        return -2;
    }
    return 0;
}
