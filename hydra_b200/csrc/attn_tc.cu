// attn_tc.cu — attention on the 5th-generation tensor cores (sm_100a only): chunked prefill and
// split decode over the bf16 KV cache, one persistent kernel for both.
//
// Replaces attention_prefill (Sources/HydraMetal/Shaders/batch.metal:307-427) and
// attention_decode_split (Sources/HydraMetal/Shaders/attention.metal:307-415).  Where the reference
// gives every (token, query head) its own threadgroup that streams the whole key range, this kernel
// packs the G query heads that share a KV head and 128/G consecutive tokens into one 128-row tile,
// so each K/V tile fetched by TMA serves 128 query rows, and both contractions run as tcgen05.mma
// with accumulators in tensor memory.  A CTA is persistent: it walks a static list of work items
// (row tile x kv head for prefill; run of key tiles x kv head x sequence for decode) and keeps its
// TMA ring, tensor memory and barriers across items, so one item's ramp-up hides behind the
// previous item's tail.
//
//   warp 0      producer: TMA loads of K and V tiles (128 keys x d, 128-byte swizzle) into a ring
//   warp 1      MMA issuer: S = Q K^T (A, B from shared memory), O_j = P V (A = P from tensor memory)
//   warps 2-5   softmax: S from tensor memory, causal / window mask, row maximum, P = bf16(exp2(..)),
//               row sum, P back into tensor memory over S
//   warps 6-9   fold: stages the next item's Q tile in shared memory; O_j from tensor memory folded
//               into the row's running (M, L, A) in registers (prefill) or written out as the
//               tile's partial (decode); the epilogue (divide, gate, store)
//
// The arithmetic is the canonical tile-partial + fold of common.cuh: every key tile yields an
// independent partial with its own maximum and the partials are folded in ascending tile order
// seeded with the sink.  A row's result depends only on that row's query and on the key tiles, not
// on the chunk it arrived in nor on its position inside the 128-row tile, which is what makes
// chunked prefill, one-shot prefill and token-by-token decode agree bit for bit.
//
// Every wait on an mbarrier is bounded: after about a second it records HC_TIMEOUT in the
// context's status word, raises a CTA-wide abort flag that all other waits observe, and the CTA
// drains and frees its tensor memory before returning.

#include <algorithm>

#include "internal.hpp"
#include "tc_ptx.cuh"

namespace hc {
namespace {

struct TcArgs {
    const uint16_t* q;        // bf16 [rows][q_heads][d], prepared
    int tokens;               // prefill: tokens of the chunk
    int first_position;
    int q_heads;
    int kv_heads;
    int log_group;
    int window;
    float c;
    const uint16_t* sinks;
    int count_sink;
    int seq;
    RowMap map;
    EpilogueArgs ep;
    int* status;
    int n_items;              // work items in the list
    int mtiles;               // prefill: row tiles per kv head
    // Decode (split over key tiles): one query token per batch entry; an item is a run of
    // `tiles_per_item` consecutive key tiles of one (sequence, kv head) whose partials it writes.
    int decode;
    int chunks;               // decode: items per (sequence, kv head)
    int tiles_per_item;
    float* part_o;            // fp32 [rows][part_tiles][d]
    float* part_ml;           // fp32 [rows][part_tiles][2]
    int part_tiles;
    BatchMeta meta;
};

template <int D>
struct TcLayout {
    static constexpr int kBlocks = D / 64;                   // 64-element (128-byte) column blocks
    static constexpr int kTileBytes = kTileKeys * D * 2;     // one K or V tile
    static constexpr int kStages = D == 64 ? 4 : 2;
    static constexpr int kQBytes = kRows * D * 2;            // one Q tile; two are kept
    // Tensor memory: two S buffers of 128 columns (P overwrites the first 64 of its S), then two
    // O buffers; d = 64 leaves room beside each for 16 columns of row sums computed by the tensor core.
    static constexpr int kOCol0 = 2 * kTileKeys;
    static constexpr bool kSumOnTensor = D == 64;
    static constexpr int kOStride = kSumOnTensor ? D + 16 : D;
    static constexpr int kTmemCols = 512;
    static constexpr int kOnesBytes = 2048;
    static constexpr int kSmemBytes = 1024 /*align slack*/ + 2 * kQBytes + 2 * kStages * kTileBytes + kOnesBytes;
};

struct TcBarriers {
    uint64_t q_full[2], q_empty[2];
    uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
    uint64_t s_full[2], p_full[2], o_full[2], o_free[2];
    uint32_t tmem_base;
    int abort_flag;
    float mm[4][kRows];       // per-tile scaled maxima, softmax -> fold (ring of 4 tiles)
    float l[4][kRows];        // per-tile row sums (when they are not computed on the tensor core)
};

// One unit of work of a CTA.
struct TcItem {
    int kv_head;
    int seq;
    int row0;          // first row of q / out (token index of the chunk, or batch entry)
    int valid_tokens;  // query tokens in this row tile
    int first_pos;     // position of the first query token
    int tile_first;    // absolute index of the first key tile
    int n_tiles;       // key tiles to visit (stride `world` apart); <= 0: nothing to do
    int ordinal0;      // decode: ordinal of the first tile among the row's tiles
};

__device__ __forceinline__ TcItem decode_item(const TcArgs& args, int index) {
    TcItem w;
    const int tokens_per_tile = kRows >> args.log_group;
    int chunk = 0;
    if (args.decode) {
        chunk = index % args.chunks;
        const int rest = index / args.chunks;
        w.kv_head = rest % args.kv_heads;
        const int b = rest / args.kv_heads;
        w.row0 = b;
        w.valid_tokens = 1;
        w.first_pos = args.meta.pos[b];
        w.seq = args.meta.seq[b];
    } else {
        // Longest key ranges first: descending row tile, the kv heads of one row tile adjacent.
        w.kv_head = index % args.kv_heads;
        const int mtile = args.mtiles - 1 - index / args.kv_heads;
        w.row0 = mtile * tokens_per_tile;
        w.valid_tokens = min(tokens_per_tile, args.tokens - w.row0);
        w.first_pos = args.first_position + w.row0;
        w.seq = args.seq;
    }
    const int last_pos = w.first_pos + w.valid_tokens - 1;
    const int lo_first = args.window > 0 ? max(0, w.first_pos - args.window + 1) : 0;
    const int world = max(args.map.world, 1);
    int tile_first = lo_first / kTileKeys;
    const int tile_last = last_pos / kTileKeys;
    if (world > 1) tile_first += ((args.map.rank - tile_first % world) + world) % world;
    int n_tiles = tile_first > tile_last ? 0 : (tile_last - tile_first) / world + 1;
    w.ordinal0 = 0;
    if (args.decode) {
        w.ordinal0 = chunk * args.tiles_per_item;
        tile_first += w.ordinal0 * world;
        n_tiles = min(args.tiles_per_item, n_tiles - w.ordinal0);
    }
    w.tile_first = tile_first;
    w.n_tiles = n_tiles;
    return w;
}

// The next item of this CTA's list that has work, or n_items.
__device__ __forceinline__ int next_item(const TcArgs& args, int index) {
    for (index += gridDim.x; index < args.n_items; index += gridDim.x) {
        if (decode_item(args, index).n_tiles > 0) return index;
    }
    return args.n_items;
}
__device__ __forceinline__ int first_item(const TcArgs& args) {
    int index = blockIdx.x;
    if (index < args.n_items && decode_item(args, index).n_tiles > 0) return index;
    return index < args.n_items ? next_item(args, index) : args.n_items;
}

// bf16x2 of two softmax weights: `lo` in the low half (the earlier key), `hi` in the high half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    return packed;
}

// Optional timeline for bring-up builds (-DHC_TC_TRACE): nanosecond stamps of a few events per CTA.
#ifdef HC_TC_TRACE
__device__ unsigned long long hc_tc_trace[256 * 16 * 4];
__device__ __forceinline__ void tc_trace(int slot) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    if (blockIdx.x < 256 && hc_tc_trace[blockIdx.x * 16 + slot] == 0) hc_tc_trace[blockIdx.x * 16 + slot] = now;
}
#define TC_TRACE(slot) tc_trace(slot)
// Cycle accounting of one thread: TC_LAP(k) adds the cycles since the previous lap to bucket k.
#define TC_LAP_DECL long long lap_last = clock64(); long long lap_acc[6] = {0, 0, 0, 0, 0, 0};
#define TC_LAP(k) { const long long lap_now = clock64(); lap_acc[k] += lap_now - lap_last; lap_last = lap_now; }
#define TC_LAP_STORE(base) { for (int lap_i = 0; lap_i < 6; ++lap_i) hc_tc_trace[(blockIdx.x & 255) * 16 + 16 * 256 * (base) + lap_i] = (unsigned long long)lap_acc[lap_i]; }
#else
#define TC_TRACE(slot)
#define TC_LAP_DECL
#define TC_LAP(k)
#define TC_LAP_STORE(base)
#endif

// A position in the stream of key tiles a CTA processes: tile j of the item with ordinal `it`.
struct TcCursor {
    int item;          // index in the work list, or n_items at the end
    TcItem w;
    int j;             // tile within the item
    uint32_t t;        // ordinal of the tile in the CTA's stream
    uint32_t it;       // ordinal of the item
};
__device__ __forceinline__ TcCursor cursor_begin(const TcArgs& args) {
    TcCursor c{};
    c.item = first_item(args);
    if (c.item < args.n_items) c.w = decode_item(args, c.item);
    return c;
}
__device__ __forceinline__ bool cursor_valid(const TcArgs& args, const TcCursor& c) { return c.item < args.n_items; }
__device__ __forceinline__ void cursor_advance(const TcArgs& args, TcCursor& c) {
    ++c.t;
    if (++c.j >= c.w.n_tiles) {
        c.item = next_item(args, c.item);
        if (c.item < args.n_items) c.w = decode_item(args, c.item);
        c.j = 0;
        ++c.it;
    }
}

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                    const TcArgs args) {
    using LT = TcLayout<D>;
    extern __shared__ unsigned char raw_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = base;                                  // two Q tiles
    unsigned char* k_smem = q_smem + 2 * LT::kQBytes;
    unsigned char* v_smem = k_smem + LT::kStages * LT::kTileBytes;
    unsigned char* ones_smem = v_smem + LT::kStages * LT::kTileBytes;   // 2 KiB of bf16 1.0
    TcBarriers* bars = reinterpret_cast<TcBarriers*>(ones_smem + LT::kOnesBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int wg = warp >> 2;                                      // 0 control, 1-2 softmax (even / odd tiles), 3 fold
    const int G = 1 << args.log_group;
    const int world = max(args.map.world, 1);
    volatile int* abort_flag = &bars->abort_flag;

    if (threadIdx.x == 0) {
        TC_TRACE(0);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->q_full[i], 128);
            mbar_init(&bars->q_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->p_full[i], 128);
            mbar_init(&bars->o_full[i], 1);
            mbar_init(&bars->o_free[i], 128);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&bars->k_full[i], 1);
            mbar_init(&bars->k_empty[i], 1);
            mbar_init(&bars->v_full[i], 1);
            mbar_init(&bars->v_empty[i], 1);
        }
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    // The constant B operand of the row-sum MMA: every element is bf16 1.0, so any layout reads it.
    for (int i = threadIdx.x; i < LT::kOnesBytes / 4; i += kTcThreads) {
        reinterpret_cast<uint32_t*>(ones_smem)[i] = 0x3F803F80u;
    }
    fence_proxy_async();
    if (warp == 1) tmem_alloc(&bars->tmem_base, LT::kTmemCols);
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    if (threadIdx.x == 0) TC_TRACE(1);

    // Registers follow the work (setmaxnreg, first thing in each warpgroup's branch): the fold
    // warpgroup holds a row of O per thread, the control warpgroup needs almost none.
    if (wg == 0) {
    reg_dealloc<48>();
    if (warp == 0) {
        // ===== producer: one stream of tiles across all of this CTA's items =====
        if (lane == 0) {
            for (TcCursor c = cursor_begin(args); cursor_valid(args, c); cursor_advance(args, c)) {
                const int plane = c.w.seq * args.kv_heads + c.w.kv_head;
                const int slot = int(c.t % LT::kStages);
                const uint32_t round = c.t / LT::kStages;
                const int row0 = row_of_tile(args.map, c.w.tile_first + c.j * world);
                if (round > 0 && !mbar_wait(&bars->k_empty[slot], (round - 1) & 1, abort_flag, args.status, 1)) break;
                mbar_expect_tx(&bars->k_full[slot], LT::kTileBytes);
                for (int b = 0; b < LT::kBlocks; ++b) {
                    tma_load_3d(k_smem + slot * LT::kTileBytes + b * (kTileKeys * 128), &tmap_k,
                                &bars->k_full[slot], b * 64, row0, plane);
                }
                if (round > 0 && !mbar_wait(&bars->v_empty[slot], (round - 1) & 1, abort_flag, args.status, 2)) break;
                mbar_expect_tx(&bars->v_full[slot], LT::kTileBytes);
                for (int b = 0; b < LT::kBlocks; ++b) {
                    tma_load_3d(v_smem + slot * LT::kTileBytes + b * (kTileKeys * 128), &tmap_v,
                                &bars->v_full[slot], b * 64, row0, plane);
                }
                TC_TRACE(2);
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: S runs up to two tiles ahead of P V, across item boundaries too =====
        if (lane == 0) {
            constexpr uint32_t idesc_qk = instr_desc(kTileKeys, false);
            constexpr uint32_t idesc_pv = instr_desc(D, true);
            constexpr uint32_t idesc_sum = instr_desc(16, false);
            const uint64_t ones_desc = smem_desc(smem_u32(ones_smem), 16);
            // S = Q K^T of the tile under cursor `c`.
            auto issue_qk = [&](const TcCursor& c) -> bool {
                const int slot = int(c.t % LT::kStages);
                const int qb = int(c.it & 1);
                const int sb = int(c.t & 1);
                if (c.j == 0 && !mbar_wait(&bars->q_full[qb], (c.it >> 1) & 1, abort_flag, args.status, 4)) return false;
                TC_TRACE(3);
                if (!mbar_wait(&bars->k_full[slot], (c.t / LT::kStages) & 1, abort_flag, args.status, 3)) return false;
                TC_TRACE(4);
                tc_fence_after();
                const uint32_t q_addr = smem_u32(q_smem + qb * LT::kQBytes);
                const uint32_t k_addr = smem_u32(k_smem + slot * LT::kTileBytes);
                const uint32_t s_tmem = tmem + sb * kTileKeys;
                #pragma unroll
                for (int b = 0; b < LT::kBlocks; ++b) {
                    #pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint32_t off = b * (kRows * 128) + ks * 32;
                        mma_ss(s_tmem, smem_desc(q_addr + off, 16), smem_desc(k_addr + off, 16), idesc_qk,
                               (b | ks) != 0 ? 1u : 0u);
                    }
                }
                tc_commit(&bars->k_empty[slot]);
                tc_commit(&bars->s_full[sb]);
                if (c.j + 1 == c.w.n_tiles) tc_commit(&bars->q_empty[qb]);   // the item's Q tile was read for the last time
                return true;
            };
            TcCursor ahead = cursor_begin(args);          // next tile whose S is to be issued
            bool ok = true;
            for (TcCursor c = cursor_begin(args); ok && cursor_valid(args, c); cursor_advance(args, c)) {
                // S of tile t + 1 goes to the buffer tile t - 1 used; its P V is already queued.  The
                // look-ahead never waits for a Q tile beyond the next item's: that one is staged only
                // after the fold warpgroup has seen this item's outputs.
                while (ok && cursor_valid(args, ahead) && ahead.t < c.t + 2 && ahead.it <= c.it + 1) {
                    ok = issue_qk(ahead);
                    cursor_advance(args, ahead);
                }
                if (!ok) break;
                const int slot = int(c.t % LT::kStages);
                const int sb = int(c.t & 1);
                if (!mbar_wait(&bars->p_full[sb], (c.t >> 1) & 1, abort_flag, args.status, 5)) break;
                if (!mbar_wait(&bars->v_full[slot], (c.t / LT::kStages) & 1, abort_flag, args.status, 6)) break;
                if (c.t >= 2 && !mbar_wait(&bars->o_free[sb], ((c.t >> 1) - 1) & 1, abort_flag, args.status, 7)) break;
                tc_fence_after();
                const uint32_t v_addr = smem_u32(v_smem + slot * LT::kTileBytes);
                const uint32_t p_tmem = tmem + sb * kTileKeys;
                const uint32_t o_tmem = tmem + LT::kOCol0 + sb * LT::kOStride;
                #pragma unroll
                for (int ks = 0; ks < kTileKeys / 16; ++ks) {
                    mma_ts(o_tmem, p_tmem + ks * 8, smem_desc(v_addr + ks * 2048, kTileKeys * 128), idesc_pv,
                           ks != 0 ? 1u : 0u);
                }
                if (LT::kSumOnTensor) {
                    // Row sums of P on the tensor core: P x ones, 16 identical columns beside O.
                    #pragma unroll
                    for (int ks = 0; ks < kTileKeys / 16; ++ks) {
                        mma_ts(o_tmem + D, p_tmem + ks * 8, ones_desc, idesc_sum, ks != 0 ? 1u : 0u);
                    }
                }
                tc_commit(&bars->v_empty[slot]);
                tc_commit(&bars->o_full[sb]);
            }
        }
    }
    } else if (wg == 1 || wg == 2) {
        // ===== softmax: warpgroup 1 takes the even tiles of the stream, warpgroup 2 the odd ones, so
        // one group's exp2 phase overlaps the other's loads and maximum.  Thread = row. =====
        reg_dealloc<112>();
        const int parity = wg - 1;
        const int quad = warp & 3;                           // the TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        const float neg_inf = __int_as_float(0xff800000);
        TC_LAP_DECL
        for (TcCursor c = cursor_begin(args); cursor_valid(args, c); cursor_advance(args, c)) {
            if (int(c.t & 1) != parity) continue;
            const bool valid = t_local < c.w.valid_tokens;
            const bool warp_has_rows = quad * 32 < (c.w.valid_tokens << args.log_group);   // warp-uniform
            const int pos = valid ? c.w.first_pos + t_local : -1;
            const int lo = args.window > 0 ? max(0, pos - args.window + 1) : 0;
            const int sb = int(c.t & 1);
            TC_LAP(5)
            if (!mbar_wait(&bars->s_full[sb], (c.t >> 1) & 1, abort_flag, args.status, 8)) break;
            TC_LAP(0)
            if (threadIdx.x == 128) TC_TRACE(5);
            tc_fence_after();
            if (!warp_has_rows) {
                // No query row lives in this quadrant: its P rows stay whatever they were and the
                // O rows they produce are never read (rows are independent).
                tc_fence_before();
                mbar_arrive(&bars->p_full[sb]);
                continue;
            }
            const uint32_t s_tmem = tmem + lane_base + sb * kTileKeys;
            const int key0 = (c.w.tile_first + c.j * world) * kTileKeys;
            const int c_lo = lo - key0;                      // visible columns: [c_lo, c_hi]
            const int c_hi = pos - key0;
            const bool full = c_lo <= 0 && c_hi >= kTileKeys - 1;
            // Pass 1: the row maximum, 64 columns at a time (exact under any association).
            float m = neg_inf;
            #pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                uint32_t s[2][32];
                HC_TMEM_LD32(s_tmem + hb * 64, s[0]);
                HC_TMEM_LD32(s_tmem + hb * 64 + 32, s[1]);
                tc_wait_ld();
                if (!full) {
                    #pragma unroll
                    for (int idx = 0; idx < 64; ++idx) {
                        const int col = hb * 64 + idx;
                        if (col < c_lo || col > c_hi) s[idx >> 5][idx & 31] = __float_as_uint(neg_inf);
                    }
                }
                float mx[4];
                #pragma unroll
                for (int u = 0; u < 4; ++u) {
                    float acc = __uint_as_float(s[0][u]);
                    #pragma unroll
                    for (int k = 1; k < 15; k += 2) {
                        const int i0 = u + 4 * k, i1 = u + 4 * (k + 1);
                        acc = fmax3(acc, __uint_as_float(s[i0 >> 5][i0 & 31]), __uint_as_float(s[i1 >> 5][i1 & 31]));
                    }
                    mx[u] = fmaxf(acc, __uint_as_float(s[1][28 + u]));
                }
                m = fmax3(m, fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
            }
            const float neg_mc = -__fmul_rn((m == neg_inf) ? 0.0f : m, args.c);
            TC_LAP(2)
            // Pass 2: weights, 64 columns at a time; P overwrites the S columns already consumed.
            float sum = 0.0f;
            #pragma unroll
            for (int hb = 0; hb < 2; ++hb) {
                uint32_t s[2][32];
                HC_TMEM_LD32(s_tmem + hb * 64, s[0]);
                HC_TMEM_LD32(s_tmem + hb * 64 + 32, s[1]);
                tc_wait_ld();
                if (!full) {
                    #pragma unroll
                    for (int idx = 0; idx < 64; ++idx) {
                        const int col = hb * 64 + idx;
                        if (col < c_lo || col > c_hi) s[idx >> 5][idx & 31] = __float_as_uint(neg_inf);
                    }
                }
                #pragma unroll
                for (int q2 = 0; q2 < 2; ++q2) {
                    uint32_t packed[16];
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float e0 = tile_weight_raw(__uint_as_float(s[q2][2 * i]), neg_mc, args.c);
                        const float e1 = tile_weight_raw(__uint_as_float(s[q2][2 * i + 1]), neg_mc, args.c);
                        packed[i] = pack_bf16x2(e0, e1);
                    }
                    HC_TMEM_ST16(s_tmem + hb * 32 + q2 * 16, packed);
                    if (!LT::kSumOnTensor) {
                        // Group of 32 columns by the butterfly tree (i with i + 16, + 8, + 4, + 2, + 1);
                        // the four groups of the row are then added in order.
                        float a[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const uint32_t lo_word = packed[i >> 1], hi_word = packed[(i + 16) >> 1];
                            const float x = __uint_as_float((i & 1) ? (lo_word & 0xffff0000u) : (lo_word << 16));
                            const float y = __uint_as_float((i & 1) ? (hi_word & 0xffff0000u) : (hi_word << 16));
                            a[i] = __fadd_rn(x, y);
                        }
                        #pragma unroll
                        for (int i = 0; i < 8; ++i) a[i] = __fadd_rn(a[i], a[i + 8]);
                        #pragma unroll
                        for (int i = 0; i < 4; ++i) a[i] = __fadd_rn(a[i], a[i + 4]);
                        a[0] = __fadd_rn(a[0], a[2]);
                        a[1] = __fadd_rn(a[1], a[3]);
                        const float group = __fadd_rn(a[0], a[1]);
                        sum = (hb == 0 && q2 == 0) ? group : __fadd_rn(sum, group);
                    }
                }
            }
            bars->mm[c.t & 3][row] = __fmul_rn(m, args.c);
            if (!LT::kSumOnTensor) bars->l[c.t & 3][row] = sum;
            TC_LAP(3)
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(&bars->p_full[sb]);
            TC_LAP(4)
            if (threadIdx.x == 128) TC_TRACE(6);
        }
        if (threadIdx.x == 128) { TC_LAP_STORE(1) }
    } else {
        // ===== fold + epilogue: thread = row; also stages the Q tiles =====
        reg_alloc<232>();
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const int g = row & (G - 1);
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        // This thread copies its own row of an item's Q tile into the swizzled K-major layout.
        auto stage_q = [&](const TcItem& w, int qb) {
            const bool valid = t_local < w.valid_tokens;
            const uint16_t* src = args.q + (size_t(w.row0 + t_local) * args.q_heads + size_t(w.kv_head) * G + g) * D;
            unsigned char* dst = q_smem + qb * LT::kQBytes;
            #pragma unroll
            for (int b = 0; b < LT::kBlocks; ++b) {
                #pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    uint4 value = make_uint4(0, 0, 0, 0);
                    if (valid) value = *reinterpret_cast<const uint4*>(src + b * 64 + ch * 8);
                    *reinterpret_cast<uint4*>(dst + b * (kRows * 128) + row * 128 + ((ch ^ (row & 7)) << 4)) = value;
                }
            }
            fence_proxy_async();
            mbar_arrive(&bars->q_full[qb]);
        };
        uint32_t t = 0, it = 0;
        bool ok = true;
        int item = first_item(args);
        if (item < args.n_items) stage_q(decode_item(args, item), 0);
        while (ok && item < args.n_items) {
            const TcItem w = decode_item(args, item);
            const int nxt = next_item(args, item);
            if (nxt < args.n_items) {
                // Stage the next item's Q now; its buffer was last read by item it - 1.
                const int qb = int((it + 1) & 1);
                if (it >= 1 && !mbar_wait(&bars->q_empty[qb], (((it + 1) >> 1) - 1) & 1, abort_flag, args.status, 10)) {
                    ok = false;
                    break;
                }
                stage_q(decode_item(args, nxt), qb);
            }
            const int head = w.kv_head * G + g;
            const bool valid = t_local < w.valid_tokens;
            const bool warp_has_rows = quad * 32 < (w.valid_tokens << args.log_group);   // warp-uniform
            float M, L;
            if (args.count_sink) {
                const uint16_t bits = args.sinks ? args.sinks[head] : kNoSinkBits;
                M = __fmul_rn(bf16_bits_to_float(bits), kLog2e);
                L = 1.0f;
            } else {
                M = kEmptyMax;
                L = 0.0f;
            }
            float A[D];
            #pragma unroll
            for (int i = 0; i < D; ++i) A[i] = 0.0f;
            for (int j = 0; j < w.n_tiles; ++j, ++t) {
                const int ob = int(t & 1);
                const uint32_t o_tmem = tmem + lane_base + LT::kOCol0 + ob * LT::kOStride;
                if (!mbar_wait(&bars->o_full[ob], (t >> 1) & 1, abort_flag, args.status, 9)) { ok = false; break; }
                if (threadIdx.x == 384) TC_TRACE(7);
                tc_fence_after();
                if (!warp_has_rows) {
                    tc_fence_before();
                    mbar_arrive(&bars->o_free[ob]);
                    continue;
                }
                // The tile's row sum: column D of the O buffer (tensor core) or the softmax thread's sum.
                float l_tile;
                if (LT::kSumOnTensor) {
                    const uint32_t bits = tmem_ld1(o_tmem + D);
                    tc_wait_ld();
                    l_tile = __uint_as_float(bits);
                } else {
                    l_tile = bars->l[t & 3][row];
                }
                const float mm_tile = bars->mm[t & 3][row];
                if (args.decode) {
                    // Split decode: the tile's partial goes to the workspace; merge_tiles_kernel folds.
                    const size_t prow = (size_t(w.row0) * args.q_heads + head) * args.part_tiles + (w.ordinal0 + j);
                    #pragma unroll
                    for (int hb = 0; hb < D / 64; ++hb) {
                        uint32_t o[2][32];
                        HC_TMEM_LD32(o_tmem + hb * 64, o[0]);
                        HC_TMEM_LD32(o_tmem + hb * 64 + 32, o[1]);
                        tc_wait_ld();
                        if (hb == D / 64 - 1) {
                            tc_fence_before();
                            mbar_arrive(&bars->o_free[ob]);
                        }
                        if (valid) {
                            float* dst = args.part_o + prow * D + hb * 64;
                            #pragma unroll
                            for (int u = 0; u < 2; ++u) {
                                #pragma unroll
                                for (int i = 0; i < 32; i += 4) {
                                    *reinterpret_cast<uint4*>(dst + u * 32 + i) =
                                        make_uint4(o[u][i], o[u][i + 1], o[u][i + 2], o[u][i + 3]);
                                }
                            }
                        }
                    }
                    if (valid) {
                        args.part_ml[prow * 2] = mm_tile;
                        args.part_ml[prow * 2 + 1] = l_tile;
                    }
                    continue;
                }
                float Mn, a, b;
                fold_coefficients(M, mm_tile, Mn, a, b);
                L = __fmaf_rn(L, a, __fmul_rn(l_tile, b));
                M = Mn;
                #pragma unroll
                for (int hb = 0; hb < D / 64; ++hb) {
                    uint32_t o[2][32];
                    HC_TMEM_LD32(o_tmem + hb * 64, o[0]);
                    HC_TMEM_LD32(o_tmem + hb * 64 + 32, o[1]);
                    tc_wait_ld();
                    if (hb == D / 64 - 1) {
                        tc_fence_before();
                        mbar_arrive(&bars->o_free[ob]);
                    }
                    #pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int col = hb * 64 + u * 32 + i;
                            A[col] = fold_value(A[col], a, __uint_as_float(o[u][i]), b);
                        }
                    }
                }
            }
            if (!ok) break;
            if (valid && !args.decode) {
                const size_t out_row = size_t(w.row0 + t_local);
                if (args.ep.write_partial) {
                    float* dst = reinterpret_cast<float*>(args.ep.out) + (out_row * args.q_heads + head) * size_t(D + 2);
                    // A partial row is D + 2 floats: its start is 8-byte aligned, not 16.
                    #pragma unroll
                    for (int i = 0; i < D; i += 2) {
                        *reinterpret_cast<float2*>(dst + i) = make_float2(A[i], A[i + 1]);
                    }
                    dst[D] = M;
                    dst[D + 1] = L;
                } else {
                    const bool gated = args.ep.gate_layout != HC_GATE_NONE;
                    const size_t vec = out_row * args.q_heads + head;
                    const size_t gate_base = args.ep.gate_layout == HC_GATE_INTERLEAVED ? vec * size_t(2 * D) + D : vec * size_t(D);
                    #pragma unroll
                    for (int i = 0; i < D; i += 8) {
                        float r[8];
                        #pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float gv = gated ? load_io(args.ep.gate, gate_base + i + u, args.ep.io_dtype) : 0.0f;
                            r[u] = finish_value(A[i + u], L, gated, gv);
                        }
                        if (args.ep.io_dtype == HC_F32) {
                            float* dst = reinterpret_cast<float*>(args.ep.out) + vec * D + i;
                            *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
                            *reinterpret_cast<float4*>(dst + 4) = make_float4(r[4], r[5], r[6], r[7]);
                        } else {
                            uint4 packed;
                            packed.x = pack_bf16x2(r[0], r[1]);
                            packed.y = pack_bf16x2(r[2], r[3]);
                            packed.z = pack_bf16x2(r[4], r[5]);
                            packed.w = pack_bf16x2(r[6], r[7]);
                            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(args.ep.out) + vec * D + i) = packed;
                        }
                    }
                }
            }
            if (threadIdx.x == 384) TC_TRACE(8);
            item = nxt;
            ++it;
        }
        if (threadIdx.x == 384) {
#ifdef HC_TC_TRACE
            hc_tc_trace[(blockIdx.x & 255) * 16 + 9] = 0;
#endif
            TC_TRACE(9);
        }
    }

    // Teardown.  On the abort path the producer first lets its copies in flight land (bounded).
    if (warp == 0 && lane == 0 && *abort_flag != 0) {
        const long long start = clock64();
        while (static_cast<unsigned long long>(clock64() - start) < 200000000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) TC_TRACE(10);
    if (warp == 1) tmem_dealloc(tmem, LT::kTmemCols);
}

// ---- host side ------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) == cudaSuccess &&
            result == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
        }
    }
    return fn;
}

bool dim_ok(int d) { return d == 64 || d == 128; }

}  // namespace

bool tc_supported(const AttnShape& shape) { return dim_ok(shape.head_dim) && shape.group <= 16; }

hc_status tc_make_tensor_maps(hc_kv_cache* cache, hc_layer_store& layer) {
    if (!dim_ok(layer.desc.head_dim)) return HC_OK;
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return fail(HC_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    const int d = layer.desc.head_dim;
    for (int which = 0; which < 2; ++which) {
        CUtensorMap* map = new CUtensorMap;
        const cuuint64_t dims[3] = {cuuint64_t(d), cuuint64_t(layer.capacity),
                                    cuuint64_t(cache->max_seqs) * layer.desc.kv_heads};
        const cuuint64_t strides[2] = {cuuint64_t(d) * 2, cuuint64_t(layer.capacity) * d * 2};
        const cuuint32_t box[3] = {64, cuuint32_t(kTileKeys), 1};
        const cuuint32_t elem[3] = {1, 1, 1};
        const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, which == 0 ? layer.k : layer.v, dims,
                                   strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) {
            delete map;
            return fail(HC_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(rc)));
        }
        (which == 0 ? layer.tmap_k : layer.tmap_v) = map;
    }
    return HC_OK;
}

void tc_free_tensor_maps(hc_layer_store& layer) {
    delete static_cast<CUtensorMap*>(layer.tmap_k);
    delete static_cast<CUtensorMap*>(layer.tmap_v);
    layer.tmap_k = layer.tmap_v = nullptr;
}

template <int D>
static hc_status launch_tc(hc_context* ctx, const TcArgs& args, const hc_layer_store& layer, cudaStream_t stream) {
    using LT = TcLayout<D>;
    const int smem = LT::kSmemBytes + int(sizeof(TcBarriers));
    static bool configured[64] = {};                 // per device: the attribute is set once
    if (!configured[ctx->device & 63]) {
        cudaError_t err = cudaFuncSetAttribute(attention_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return check_cuda(err, "attention_tc_kernel shared memory");
        configured[ctx->device & 63] = true;
    }
    // Persistent: one CTA per SM at most, each walking items blockIdx.x, blockIdx.x + gridDim.x, ...
    const int grid = std::max(1, std::min(args.n_items, std::max(ctx->sm_count, 1)));
    attention_tc_kernel<D><<<grid, kTcThreads, smem, stream>>>(*static_cast<const CUtensorMap*>(layer.tmap_k),
                                                              *static_cast<const CUtensorMap*>(layer.tmap_v), args);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "attention_tc_kernel launch");
}

hc_status tc_prefill(hc_context* ctx, const AttnShape& shape, const hc_layer_store& layer, const CacheView& cache,
                     int seq, const uint16_t* q, int tokens, int first_position, const EpilogueArgs& ep,
                     cudaStream_t stream) {
    if (!layer.tmap_k || !layer.tmap_v) return fail(HC_UNSUPPORTED, "this layer has no tensor maps");
    if (tokens <= 0) return HC_OK;
    TcArgs args{};
    args.q = q;
    args.tokens = tokens;
    args.first_position = first_position;
    args.q_heads = shape.q_heads;
    args.kv_heads = shape.kv_heads;
    int log_group = 0;
    while ((1 << log_group) < shape.group) ++log_group;
    args.log_group = log_group;
    args.window = shape.window;
    args.c = shape.c;
    args.sinks = shape.sinks;
    args.count_sink = shape.count_sink;
    args.seq = seq;
    args.map = cache.map;
    args.ep = ep;
    args.status = ctx->status_dev;
    const int tokens_per_tile = kRows / shape.group;
    args.mtiles = (tokens + tokens_per_tile - 1) / tokens_per_tile;
    args.n_items = args.mtiles * shape.kv_heads;
    if (shape.head_dim == 64) return launch_tc<64>(ctx, args, layer, stream);
    return launch_tc<128>(ctx, args, layer, stream);
}

hc_status tc_decode(hc_context* ctx, const AttnShape& shape, const hc_layer_store& layer, const CacheView& cache,
                    const BatchMeta& meta, int n_seq, const uint16_t* q, const Workspace& ws,
                    const EpilogueArgs& ep, cudaStream_t stream) {
    if (!layer.tmap_k || !layer.tmap_v) return fail(HC_UNSUPPORTED, "this layer has no tensor maps");
    if (n_seq <= 0) return HC_OK;
    const int world = cache.map.world > 1 ? cache.map.world : 1;
    int max_tiles = 0;
    long long total_tiles = 0;
    for (int b = 0; b < n_seq; ++b) {
        const int lo = shape.window > 0 ? std::max(0, meta.pos[b] - shape.window + 1) : 0;
        int n = meta.pos[b] / kTileKeys - lo / kTileKeys + 1;
        if (world > 1) n = (n + world - 1) / world + 1;
        max_tiles = std::max(max_tiles, n);
        total_tiles += n;
    }
    const size_t rows = size_t(n_seq) * shape.q_heads;
    if (rows * max_tiles * shape.head_dim > ws.part_o_floats || rows * max_tiles * 2 > ws.part_ml_floats) {
        return fail(HC_KV_OVERFLOW, "decode: the split-attention workspace is too small for this call");
    }
    TcArgs args{};
    args.q = q;
    args.tokens = n_seq;
    args.q_heads = shape.q_heads;
    args.kv_heads = shape.kv_heads;
    int log_group = 0;
    while ((1 << log_group) < shape.group) ++log_group;
    args.log_group = log_group;
    args.window = shape.window;
    args.c = shape.c;
    args.sinks = shape.sinks;
    args.count_sink = shape.count_sink;
    args.map = cache.map;
    args.ep = ep;
    args.status = ctx->status_dev;
    args.decode = 1;
    // Items of consecutive tiles, about eight per CTA so that the static round-robin balances.
    const long long target = 8LL * std::max(ctx->sm_count, 1);
    long long per = (total_tiles * shape.kv_heads + target - 1) / target;
    args.tiles_per_item = int(std::min<long long>(std::max<long long>(per, 1), 64));
    args.part_o = ws.part_o;
    args.part_ml = ws.part_ml;
    args.part_tiles = max_tiles;
    args.meta = meta;
    args.chunks = (max_tiles + args.tiles_per_item - 1) / args.tiles_per_item;
    args.n_items = args.chunks * shape.kv_heads * n_seq;
    hc_status st = shape.head_dim == 64 ? launch_tc<64>(ctx, args, layer, stream)
                                        : launch_tc<128>(ctx, args, layer, stream);
    if (st != HC_OK) return st;
    return launch_merge(ctx, shape, meta, n_seq, ws, max_tiles, world, cache.map.rank, ep, stream);
}

#ifdef HC_TC_TRACE
extern "C" __attribute__((visibility("default"))) int hc_debug_read_trace(unsigned long long* out, int clear) {
    cudaDeviceSynchronize();
    if (cudaMemcpyFromSymbol(out, hc_tc_trace, sizeof(hc_tc_trace)) != cudaSuccess) return -1;
    if (clear) {
        static unsigned long long zeros[256 * 16 * 4];
        cudaMemcpyToSymbol(hc_tc_trace, zeros, sizeof(zeros));
    }
    return 0;
}
#endif

}  // namespace hc
