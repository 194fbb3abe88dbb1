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
//   warpgroup 0 (warps 0-3)    control.  Warp 0: TMA loads of K and V tiles (128 keys x d, 128-byte
//                              swizzle) into a ring.  Warp 1: issues S = Q K^T (A, B from shared
//                              memory) up to three tiles ahead.  Warp 2: issues O_j = P V (A = P from
//                              tensor memory) and, for d = 64, the row sums of P in the same
//                              instruction.  Warp 3: copies each item's Q tile into the swizzled
//                              operand layout, two items ahead.
//   warpgroups 1-2 (warps 4-11) softmax, thread = row; the groups take alternate tiles.  S from
//                              tensor memory, causal / window mask, row maximum, then
//                              P = bf16(exp2(..)) back into tensor memory over S.  What paces a
//                              tile is the exp2 unit: 16 results per clock per SM, 1024 clocks for
//                              128 x 128; the two groups' exp2 phases are left free to overlap.  In decode the 16 real rows are read with the 16x256b shape,
//                              four threads per row.
//   warpgroup 3 (warps 12-15)   fold: O_j from tensor memory folded into the row's running (M, L, A)
//                              in registers (prefill) or written out as the tile's partial
//                              (decode); the epilogue
//
// Tensor memory: three S / P buffers of 128 columns and one O buffer.  Registers are moved between
// the warpgroups with setmaxnreg (48 / 152 / 152 / 160 per thread at d = 64, 48 / 112 / 112 / 232
// at d = 128).
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
#include "tc_common.cuh"
#include "tc_ptx.cuh"

namespace hc {
namespace {

template <int D>
struct TcLayout {
    static constexpr int kBlocks = D / 64;                   // 64-element (128-byte) column blocks
    static constexpr int kTileBytes = kTileKeys * D * 2;     // one K or V tile
    static constexpr int kStages = D == 64 ? 4 : 2;
    static constexpr int kSBufs = 3;                         // S / P buffers of 128 columns at 0, 128, 256
    static constexpr int kQBytes = kRows * D * 2;            // one Q tile; two are kept
    static constexpr int kOCol0 = kSBufs * kTileKeys;        // the one O buffer
    // d = 64 leaves room beside O for 16 columns of row sums computed by the tensor core.
    static constexpr bool kSumOnTensor = D == 64;
    // Registers per thread after setmaxnreg (control / softmax / fold); 128 x their sum with the
    // softmax counted twice is the 64 K register file.
    // With d = 64 the fold needs less and a softmax thread can hold its whole row of S.
    static constexpr bool kRowInRegs = D == 64;
    static constexpr int kRegsControl = 48;
    static constexpr int kRegsSoftmax = kRowInRegs ? 152 : 112;
    static constexpr int kRegsFold = kRowInRegs ? 160 : 232;
    static constexpr int kTmemCols = 512;
    static constexpr int kOnesBytes = kTileKeys * 128;       // a 128-row block of bf16 1.0 (16 KiB)
    // Staging for the epilogue's coalesced stores: 4 warps x 32 rows x 128 bytes.  With d = 128 the
    // block of ones is not used by any MMA and serves.
    static constexpr int kEpiWarpBytes = 32 * 128;
    static constexpr int kEpiBytes = kSumOnTensor ? 4 * kEpiWarpBytes : 0;
    static constexpr int kSmemBytes = 1024 /*align slack*/ + 2 * kQBytes + 2 * kStages * kTileBytes + kOnesBytes + kEpiBytes;
};

struct TcBarriers {
    uint64_t q_full[2], q_empty[2];
    uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
    uint64_t s_full[3], p_full[3], pv_done[3];   // per S buffer; pv_done: P V has read the buffer's P
    uint64_t o_full, o_free;
    uint32_t tmem_base;
    int abort_flag;
    float mm[8][kRows];       // per-tile scaled maxima, softmax -> fold (ring of 8 tiles)
    float l[8][kRows];        // per-tile row sums (when not summed on the tensor core)
    float m2[kRows], l2[kRows];   // the rows' second fold between segments
};


// MODE says what becomes of an item's rows (TcArgs: finish, tile_partials), so that a launch carries
// the code of its own way only: 0 = the kernel finishes them, 1 = segment partials, 2 = tile partials.
constexpr int kModeFinish = 0, kModeSegments = 1, kModeTiles = 2;

template <int D, int MODE>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                    const TcArgs args) {
    constexpr bool kFinish = MODE == kModeFinish;
    constexpr bool kTilePartials = MODE == kModeTiles;
    using LT = TcLayout<D>;
    extern __shared__ unsigned char raw_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = base;                                  // two Q tiles
    unsigned char* k_smem = q_smem + 2 * LT::kQBytes;
    unsigned char* v_smem = k_smem + LT::kStages * LT::kTileBytes;
    unsigned char* ones_smem = v_smem + LT::kStages * LT::kTileBytes;   // 128 rows of bf16 1.0
    unsigned char* epi_smem = LT::kEpiBytes > 0 ? ones_smem + LT::kOnesBytes : ones_smem;
    TcBarriers* bars = reinterpret_cast<TcBarriers*>(ones_smem + LT::kOnesBytes + LT::kEpiBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int wg = warp >> 2;                                      // 0 control, 1-2 softmax halves, 3 fold
    const int G = 1 << args.log_group;
    const int world = max(args.map.world, 1);
    volatile int* abort_flag = &bars->abort_flag;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->q_full[i], 1);
            mbar_init(&bars->q_empty[i], 1);
        }
        for (int i = 0; i < 3; ++i) {
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->p_full[i], 128);
            mbar_init(&bars->pv_done[i], 1);
        }
        mbar_init(&bars->o_full, 1);
        mbar_init(&bars->o_free, 128);
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
    // Everything above touched only this CTA's shared and tensor memory; from here on the kernel
    // reads what earlier kernels of the stream wrote (prepared q, the cache) and writes its outputs.
    pdl_wait();

    // Registers follow the work (setmaxnreg, first thing in each warpgroup's branch): the fold
    // warpgroup holds a row of O per thread, the control warpgroup needs almost none.
    if (wg == 0) {
    reg_dealloc<LT::kRegsControl>();
    if (warp == 0) {
        // ===== producer: one stream of tiles across all of this CTA's items =====
        if (LT::kStages >= 4 && lane == 0) {
            // K(t) then V(t), tile by tile.
            uint32_t t = 0;
            bool ok = true;
            for (TcItemIter walk = items_begin(args); ok && walk.item < args.n_items; items_next(args, walk)) {
                const TcItem& w = walk.w;
                const int plane = cache_plane(args.map, w.seq, args.kv_heads, w.kv_head);
                for (int j = 0; j < w.n_tiles; ++j, ++t) {
                    const int slot = int(t % LT::kStages);
                    const uint32_t round = t / LT::kStages;
                    const int row0 = cache_row(args.map, w.seq, (w.tile_first + j * world) * kTileKeys);
                    if (round > 0 && !mbar_wait(&bars->k_empty[slot], (round - 1) & 1, abort_flag, args.status, 1)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&bars->k_full[slot], LT::kTileBytes);
                    for (int b = 0; b < LT::kBlocks; ++b) {
                        tma_load_3d(k_smem + slot * LT::kTileBytes + b * (kTileKeys * 128), &tmap_k,
                                    &bars->k_full[slot], b * 64, row0, plane);
                    }
                    if (round > 0 && !mbar_wait(&bars->v_empty[slot], (round - 1) & 1, abort_flag, args.status, 2)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&bars->v_full[slot], LT::kTileBytes);
                    for (int b = 0; b < LT::kBlocks; ++b) {
                        tma_load_3d(v_smem + slot * LT::kTileBytes + b * (kTileKeys * 128), &tmap_v,
                                    &bars->v_full[slot], b * 64, row0, plane);
                    }
                }
            }
        }
        // With the two stages of d = 128 that lockstep leaves the K ring idle: the S issuer takes a K tile
        // up to three tiles before the O issuer takes the V tile of the same keys.  There the K tiles
        // run ahead of the V tiles, each stream with its own walk over the items (measured: 61 -> 57 us
        // on a 512-token chunk at context 4096; with the four stages of d = 64 it is slower, 72 -> 74 us
        // and 77 -> 85 us in decode, where the second walk's item decoding sits in the producer's path).
        if (LT::kStages < 4 && lane == 0) {
            constexpr int kKeysAhead = 3;
            struct Cursor {
                TcItemIter walk;
                int j;
                uint32_t t;
            };
            Cursor ck, cv;
            ck.walk = items_begin(args);
            ck.j = 0;
            ck.t = 0;
            cv = ck;
            bool ok = true;
            while (ok && (ck.walk.item < args.n_items || cv.walk.item < args.n_items)) {
                const bool keys = ck.walk.item < args.n_items && (ck.t < cv.t + kKeysAhead || cv.walk.item >= args.n_items);
                Cursor& c = keys ? ck : cv;
                const int slot = int(c.t % LT::kStages);
                const uint32_t round = c.t / LT::kStages;
                uint64_t* empty = keys ? &bars->k_empty[slot] : &bars->v_empty[slot];
                if (round > 0 && !mbar_wait(empty, (round - 1) & 1, abort_flag, args.status, keys ? 1 : 2)) {
                    ok = false;
                    break;
                }
                const TcItem& w = c.walk.w;
                const int plane = cache_plane(args.map, w.seq, args.kv_heads, w.kv_head);
                const int row0 = cache_row(args.map, w.seq, (w.tile_first + c.j * world) * kTileKeys);
                uint64_t* full = keys ? &bars->k_full[slot] : &bars->v_full[slot];
                unsigned char* dst = (keys ? k_smem : v_smem) + slot * LT::kTileBytes;
                mbar_expect_tx(full, LT::kTileBytes);
                for (int b = 0; b < LT::kBlocks; ++b) {
                    tma_load_3d(dst + b * (kTileKeys * 128), keys ? &tmap_k : &tmap_v, full, b * 64, row0, plane);
                }
                ++c.t;
                if (++c.j == w.n_tiles) {
                    c.j = 0;
                    items_next(args, c.walk);
                }
            }
        }
    } else if (warp == 1) {
        // ===== S issuer: S = Q K^T, up to three tiles ahead of the softmax, across item boundaries.
        // The whole warp walks the loop and waits, so control flow stays warp-uniform; one elected
        // lane issues the tcgen05 instructions. =====
        constexpr uint32_t idesc_qk = instr_desc(kTileKeys, false);
        const uint64_t q_desc0 = smem_desc(smem_u32(q_smem), 16);
        const uint64_t k_desc0 = smem_desc(smem_u32(k_smem), 16);
        uint32_t t = 0, it = 0;
        bool ok = true;
        for (TcItemIter walk = items_begin(args); ok && walk.item < args.n_items; items_next(args, walk), ++it) {
          const int n_tiles = walk.w.n_tiles;
          for (int j = 0; j < n_tiles; ++j, ++t) {
            const int slot = int(t % LT::kStages);
            const int qb = int(it & 1);
            const int sb = int(t % LT::kSBufs);
            // The buffer's previous contents, P of tile t - 3, must have been consumed.
            if (t >= LT::kSBufs &&
                !mbar_wait(&bars->pv_done[sb], (t / LT::kSBufs - 1) & 1, abort_flag, args.status, 12)) { ok = false; break; }
            if (j == 0 && !mbar_wait(&bars->q_full[qb], (it >> 1) & 1, abort_flag, args.status, 4)) { ok = false; break; }
            if (!mbar_wait(&bars->k_full[slot], (t / LT::kStages) & 1, abort_flag, args.status, 3)) { ok = false; break; }
            tc_fence_after();
            if (elect_one()) {
                // Descriptors differ from the precomputed bases only in the 16-byte address field.
                const uint64_t q_desc = q_desc0 + uint64_t((qb * LT::kQBytes) >> 4);
                const uint64_t k_desc = k_desc0 + uint64_t((slot * LT::kTileBytes) >> 4);
                const uint32_t s_tmem = tmem + sb * kTileKeys;
                #pragma unroll
                for (int b = 0; b < LT::kBlocks; ++b) {
                    #pragma unroll
                    for (int ks = 0; ks < 4; ++ks) {
                        const uint64_t off = uint64_t((b * (kRows * 128) + ks * 32) >> 4);
                        mma_ss(s_tmem, q_desc + off, k_desc + off, idesc_qk, (b | ks) != 0 ? 1u : 0u);
                    }
                }
                tc_commit(&bars->k_empty[slot]);
                tc_commit(&bars->s_full[sb]);
                if (j + 1 == n_tiles) tc_commit(&bars->q_empty[qb]);   // the item's Q tile was read for the last time
            }
            __syncwarp();
          }
        }
    } else if (warp == 2) {
        // ===== O issuer: O_t = P_t V_t (A = P from tensor memory) as soon as the tile's weights are
        // written and the fold has taken the previous tile out of the O buffer. =====
        // With the row sums on the tensor core, P V and P x ones are one instruction: the B operand
        // is the V tile (64 columns) followed by a block of ones that the descriptor's
        // column-block stride points at, so O gets 16 more columns, each the row's sum.
        constexpr uint32_t idesc_pv = instr_desc(LT::kSumOnTensor ? D + 16 : D, true);
        const uint32_t ones_addr = smem_u32(ones_smem);
        const uint32_t v_base = smem_u32(v_smem);
        uint32_t t = 0;
        bool ok = true;
        for (TcItemIter walk = items_begin(args); ok && walk.item < args.n_items; items_next(args, walk)) {
            const int n_tiles = walk.w.n_tiles;
            for (int j = 0; j < n_tiles; ++j, ++t) {
                const int slot = int(t % LT::kStages);
                const int sb = int(t % LT::kSBufs);
                if (!mbar_wait(&bars->p_full[sb], (t / LT::kSBufs) & 1, abort_flag, args.status, 5)) { ok = false; break; }
                if (!mbar_wait(&bars->v_full[slot], (t / LT::kStages) & 1, abort_flag, args.status, 6)) { ok = false; break; }
                if (t >= 1 && !mbar_wait(&bars->o_free, (t - 1) & 1, abort_flag, args.status, 7)) { ok = false; break; }
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t v_addr = v_base + slot * LT::kTileBytes;
                    const uint32_t p_tmem = tmem + sb * kTileKeys;
                    const uint32_t o_tmem = tmem + LT::kOCol0;
                    const uint32_t block_stride = LT::kSumOnTensor ? ones_addr - v_addr : uint32_t(kTileKeys * 128);
                    const uint64_t v_desc = smem_desc(v_addr, block_stride);
                    #pragma unroll
                    for (int ks = 0; ks < kTileKeys / 16; ++ks) {
                        mma_ts(o_tmem, p_tmem + ks * 8, v_desc + uint64_t((ks * 2048) >> 4), idesc_pv, ks != 0 ? 1u : 0u);
                    }
                    tc_commit(&bars->o_full);
                    tc_commit(&bars->pv_done[sb]);
                    tc_commit(&bars->v_empty[slot]);
                }
                __syncwarp();
            }
        }
    } else {
        // ===== Q stager: copies each item's Q tile (128 rows of the prepared q) into the swizzled
        // K-major layout, up to two items ahead of the S issuer, so the global-memory latency of a
        // new item never sits in another role's path.  Lane l copies rows l, l + 32, l + 64, l + 96. =====
        uint32_t it = 0;
        for (TcItemIter walk = items_begin(args); walk.item < args.n_items; items_next(args, walk), ++it) {
            const TcItem& w = walk.w;
            const int qb = int(it & 1);
            // The buffer was last read by item it - 2.
            if (it >= 2 && !mbar_wait(&bars->q_empty[qb], ((it >> 1) - 1) & 1, abort_flag, args.status, 10)) break;
            // All of the tile's 16-byte pieces are put in flight at once (cp.async, no registers), so
            // an item costs one round trip to global memory rather than one per row.
            const uint32_t dst = smem_u32(q_smem + qb * LT::kQBytes);
            #pragma unroll 1
            for (int r = 0; r < 4; ++r) {
                const int row = r * 32 + lane;
                const int t_local = row >> args.log_group;
                const int g = row & (G - 1);
                const bool valid = t_local < w.valid_tokens;
                const uint16_t* src = valid
                    ? args.q + (size_t(w.row0 + t_local) * args.q_heads + size_t(w.kv_head) * G + g) * D
                    : args.q;
                #pragma unroll
                for (int b = 0; b < LT::kBlocks; ++b) {
                    #pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        cp_async16(dst + b * (kRows * 128) + row * 128 + ((ch ^ (row & 7)) << 4), src + b * 64 + ch * 8,
                                   valid ? 16u : 0u);
                    }
                }
            }
            cp_async_wait_all();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->q_full[qb]);
        }
    }
    } else if (wg == 1 || wg == 2) {
        // ===== softmax: warpgroup 1 takes the even tiles of the stream (S buffer 0), warpgroup 2 the
        // odd ones (S buffer 1), so one group's exp2 phase overlaps the other's wait, load and
        // maximum.  Thread = row; the row is read twice (maximum, then weights) to stay in registers. =====
        if constexpr (LT::kRegsSoftmax > 128) reg_alloc<LT::kRegsSoftmax>(); else reg_dealloc<LT::kRegsSoftmax>();
        const int parity = wg - 1;
        const int quad = warp & 3;                           // the TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        const float neg_inf = __int_as_float(0xff800000);
        uint32_t t = 0;
        bool ok = true;
        for (TcItemIter walk = items_begin(args); ok && walk.item < args.n_items; items_next(args, walk)) {
            const TcItem& w = walk.w;
            const bool valid = t_local < w.valid_tokens;
            const bool warp_has_rows = quad * 32 < (w.valid_tokens << args.log_group);   // warp-uniform
            int pos = valid ? w.first_pos + t_local : -1;
            const int lo = args.window > 0 ? max(0, pos - args.window + 1) : 0;
            // From here on `pos` is the last key the row sees: its own, or the end of its bidirectional
            // block (Sources/HydraMetal/Shaders/batch.metal:351-352) as far as keys have been appended.
            if (!args.decode && args.block_ends != nullptr && valid) {
                pos = max(pos, min(__ldg(args.block_ends + (w.first_pos - args.first_position) + t_local), args.appended) - 1);
            }
            for (int j = 0; j < w.n_tiles; ++j, ++t) {
                if (int(t & 1) != parity) continue;
                const int sb = int(t % LT::kSBufs);
                const uint32_t s_tmem = tmem + lane_base + sb * kTileKeys;
                if (!mbar_wait(&bars->s_full[sb], (t / LT::kSBufs) & 1, abort_flag, args.status, 8)) { ok = false; break; }
                tc_fence_after();
                if (!warp_has_rows) {
                    // No query row lives in this quadrant: its P rows stay whatever they were and the
                    // O rows they produce are never read (rows are independent).
                    tc_fence_before();
                    mbar_arrive(&bars->p_full[sb]);
                    continue;
                }
                const int key0 = (w.tile_first + j * world) * kTileKeys;
                if (args.decode && LT::kSumOnTensor) {
                    // Decode has at most 16 real rows, all in quadrant 0 and all at one position.  The
                    // 16x256b shape spreads each row over four threads, so a warp computes 16 x 128
                    // weights instead of 32 x 128.  Element for element the weights are the
                    // ones the prefill layout computes; the row sums come from the tensor core either way.
                    const int q4 = lane & 3;
                    const int tile_key0 = key0;
                    const int c_lo = (args.window > 0 ? max(0, w.first_pos - args.window + 1) : 0) - tile_key0;
                    const int c_hi = w.first_pos - tile_key0;
                    const bool upper = G > 8;                // rows 8-15 hold heads only when the group is 16
                    uint32_t v[2][32];
                    HC_TMEM_LD_16x256b_x8(s_tmem, v[0]);
                    HC_TMEM_LD_16x256b_x8(s_tmem + 64, v[1]);
                    tc_wait_ld();
                    if (!(c_lo <= 0 && c_hi >= kTileKeys - 1)) {
                        #pragma unroll
                        for (int hb = 0; hb < 2; ++hb) {
                            #pragma unroll
                            for (int n = 0; n < 8; ++n) {
                                #pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int col = 64 * hb + 8 * n + 2 * q4 + e;
                                    if (col < c_lo || col > c_hi) {
                                        v[hb][4 * n + e] = __float_as_uint(neg_inf);
                                        v[hb][4 * n + 2 + e] = __float_as_uint(neg_inf);
                                    }
                                }
                            }
                        }
                    }
                    // Row maxima: this thread's 32 columns, then the four threads of the row.
                    float neg_mc[2] = {0.0f, 0.0f};
                    #pragma unroll
                    for (int rs = 0; rs < 2; ++rs) {
                        if (rs == 0 || upper) {
                            float m0 = __uint_as_float(v[0][2 * rs]), m1 = __uint_as_float(v[0][2 * rs + 1]);
                            float m2 = __uint_as_float(v[1][2 * rs]), m3 = __uint_as_float(v[1][2 * rs + 1]);
                            #pragma unroll
                            for (int n = 1; n < 7; n += 2) {
                                m0 = fmax3(m0, __uint_as_float(v[0][4 * n + 2 * rs]), __uint_as_float(v[0][4 * (n + 1) + 2 * rs]));
                                m1 = fmax3(m1, __uint_as_float(v[0][4 * n + 2 * rs + 1]), __uint_as_float(v[0][4 * (n + 1) + 2 * rs + 1]));
                                m2 = fmax3(m2, __uint_as_float(v[1][4 * n + 2 * rs]), __uint_as_float(v[1][4 * (n + 1) + 2 * rs]));
                                m3 = fmax3(m3, __uint_as_float(v[1][4 * n + 2 * rs + 1]), __uint_as_float(v[1][4 * (n + 1) + 2 * rs + 1]));
                            }
                            m0 = fmax3(m0, __uint_as_float(v[0][28 + 2 * rs]), m1);
                            m2 = fmax3(m2, __uint_as_float(v[1][28 + 2 * rs]), m3);
                            float m = fmax3(fmaxf(m0, m2), __uint_as_float(v[0][29 + 2 * rs]), __uint_as_float(v[1][29 + 2 * rs]));
                            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                            m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
                            neg_mc[rs] = -__fmul_rn((m == neg_inf) ? 0.0f : m, args.c);
                            if (q4 == 0) bars->mm[t & 7][(lane >> 2) + 8 * rs] = __fmul_rn(m, args.c);
                        }
                    }
                    // st[2n + rs]: P column 4n + q4 of row lane/4 + 8 rs, the layout of the 16x128b store.
                    #pragma unroll
                    for (int hb = 0; hb < 2; ++hb) {
                        uint32_t st[16];
                        #pragma unroll
                        for (int rs = 0; rs < 2; ++rs) {
                            #pragma unroll
                            for (int n = 0; n < 8; ++n) {
                                if (rs == 0 || upper) {
                                    const float e0 = tile_weight_raw(__uint_as_float(v[hb][4 * n + 2 * rs]), neg_mc[rs], args.c);
                                    const float e1 = tile_weight_raw(__uint_as_float(v[hb][4 * n + 2 * rs + 1]), neg_mc[rs], args.c);
                                    st[2 * n + rs] = pack_bf16x2(e0, e1);
                                } else {
                                    st[2 * n + rs] = 0u;
                                }
                            }
                        }
                        HC_TMEM_ST_16x128b_x8(s_tmem + hb * 32, st);
                    }
                    tc_wait_st();
                    tc_fence_before();
                    mbar_arrive(&bars->p_full[sb]);
                    continue;
                }
                const int c_lo = lo - key0;                  // visible columns: [c_lo, c_hi]
                const int c_hi = pos - key0;
                const bool full = c_lo <= 0 && c_hi >= kTileKeys - 1;
                if constexpr (LT::kRowInRegs) {
                    // The whole row of S in registers: one load, the maximum, the scaled differences
                    // (two per instruction), and then the exp2 unit's
                    // share: exp2, rounding to bf16 and the store of P.
                    uint32_t s[4][32];
                    HC_TMEM_LD32(s_tmem, s[0]);
                    HC_TMEM_LD32(s_tmem + 32, s[1]);
                    HC_TMEM_LD32(s_tmem + 64, s[2]);
                    HC_TMEM_LD32(s_tmem + 96, s[3]);
                    tc_wait_ld();
                    if (!full) {
                        #pragma unroll
                        for (int col = 0; col < kTileKeys; ++col) {
                            if (col < c_lo || col > c_hi) s[col >> 5][col & 31] = __float_as_uint(neg_inf);
                        }
                    }
                    float mx[8];
                    #pragma unroll
                    for (int u = 0; u < 8; ++u) {
                        float acc = __uint_as_float(s[0][u]);
                        #pragma unroll
                        for (int k = 1; k < 15; k += 2) {
                            const int i0 = u + 8 * k, i1 = u + 8 * (k + 1);
                            acc = fmax3(acc, __uint_as_float(s[i0 >> 5][i0 & 31]), __uint_as_float(s[i1 >> 5][i1 & 31]));
                        }
                        mx[u] = fmaxf(acc, __uint_as_float(s[3][24 + u]));
                    }
                    const float m = fmaxf(fmax3(mx[0], mx[1], mx[2]), fmax3(fmaxf(mx[3], mx[4]), fmaxf(mx[5], mx[6]), mx[7]));
                    const float neg_mc = -__fmul_rn((m == neg_inf) ? 0.0f : m, args.c);
                    #pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) fma2_inplace(s[q][2 * i], s[q][2 * i + 1], args.c, neg_mc);
                    }
                    #pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        #pragma unroll
                        for (int i = 0; i < 32; ++i) s[q][i] = __float_as_uint(ex2(__uint_as_float(s[q][i])));
                        uint32_t packed[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            packed[i] = pack_bf16x2(__uint_as_float(s[q][2 * i]), __uint_as_float(s[q][2 * i + 1]));
                        }
                        HC_TMEM_ST16(s_tmem + q * 16, packed);
                    }
                    bars->mm[t & 7][row] = __fmul_rn(m, args.c);
                    tc_wait_st();
                    tc_fence_before();
                    mbar_arrive(&bars->p_full[sb]);
                    continue;
                }
                // The row is read twice, 32 columns at a time, in rolled loops: the maximum, then the
                // weights.  Rolled on purpose: the loop bodies of the four roles have to stay resident
                // in the instruction cache together.  Each load is in flight while the previous group
                // is worked on.  P overwrites S columns already consumed (the bf16 weights of columns
                // 32 q .. 32 q + 31 land in 32-bit columns 16 q .. 16 q + 15).
                auto mask_group = [&](uint32_t (&s)[32], int base_col) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = base_col + i;
                        if (col < c_lo || col > c_hi) s[i] = __float_as_uint(neg_inf);
                    }
                };
                auto group_max = [&](const uint32_t (&s)[32]) -> float {
                    float mx[4];
                    #pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        float acc = __uint_as_float(s[u]);
                        #pragma unroll
                        for (int k = 1; k < 7; k += 2) {
                            acc = fmax3(acc, __uint_as_float(s[u + 4 * k]), __uint_as_float(s[u + 4 * (k + 1)]));
                        }
                        mx[u] = fmaxf(acc, __uint_as_float(s[u + 28]));
                    }
                    return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                };
                float m = neg_inf;
                {
                    uint32_t cur[32], nxt[32];
                    HC_TMEM_LD32(s_tmem, cur);
                    tc_wait_ld();
                    #pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        HC_TMEM_LD32(s_tmem + 64 * h + 32, nxt);
                        if (!full) mask_group(cur, 64 * h);
                        m = fmaxf(m, group_max(cur));
                        tc_wait_ld();
                        if (h == 0) HC_TMEM_LD32(s_tmem + 64, cur);
                        if (!full) mask_group(nxt, 64 * h + 32);
                        m = fmaxf(m, group_max(nxt));
                        tc_wait_ld();
                    }
                }
                const float neg_mc = -__fmul_rn((m == neg_inf) ? 0.0f : m, args.c);
                // Weights of one group of 32 columns; returns their sum when the tensor core does not.
                auto group_weights = [&](const uint32_t (&s)[32], uint32_t dst) -> float {
                    uint32_t packed[16];
                    #pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float e0 = tile_weight_raw(__uint_as_float(s[2 * i]), neg_mc, args.c);
                        const float e1 = tile_weight_raw(__uint_as_float(s[2 * i + 1]), neg_mc, args.c);
                        packed[i] = pack_bf16x2(e0, e1);
                    }
                    HC_TMEM_ST16(dst, packed);
                    if (LT::kSumOnTensor) return 0.0f;
                    // Sum of the 32 weights by the butterfly tree (i with i + 16, then + 8, + 4, + 2, + 1).
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
                    return __fadd_rn(a[0], a[1]);
                };
                // A half of the row is its two groups added, the row its two halves.
                float half_sum[2] = {0.0f, 0.0f};
                {
                    uint32_t cur[32], nxt[32];
                    HC_TMEM_LD32(s_tmem, cur);
                    tc_wait_ld();
                    #pragma unroll 1
                    for (int h = 0; h < 2; ++h) {
                        HC_TMEM_LD32(s_tmem + 64 * h + 32, nxt);
                        if (!full) mask_group(cur, 64 * h);
                        const float g0 = group_weights(cur, s_tmem + 32 * h);
                        tc_wait_ld();
                        if (h == 0) HC_TMEM_LD32(s_tmem + 64, cur);
                        if (!full) mask_group(nxt, 64 * h + 32);
                        const float g1 = group_weights(nxt, s_tmem + 32 * h + 16);
                        tc_wait_ld();
                        const float hs = __fadd_rn(g0, g1);
                        if (h == 0) half_sum[0] = hs; else half_sum[1] = hs;
                    }
                }
                if (!LT::kSumOnTensor) bars->l[t & 7][row] = __fadd_rn(half_sum[0], half_sum[1]);
                bars->mm[t & 7][row] = __fmul_rn(m, args.c);
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(&bars->p_full[sb]);
            }
        }
    } else {
        // ===== fold + epilogue: thread = row =====
        reg_alloc<LT::kRegsFold>();
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const int g = row & (G - 1);
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        // Where this thread's row keeps the values of its second fold between segments.
        constexpr int kStateStride = kRows;
        auto state_of_row = [&]() -> float* {
            return args.row_state + size_t(blockIdx.x) * (D * kRows) + row;
        };
        // (M, L) the second fold stands at: what the last segment end left, or the seed.
        auto second_fold_state = [&](bool state_holds, uint16_t sink, float& M2, float& L2) {
            if (state_holds) {
                M2 = bars->m2[row];
                L2 = bars->l2[row];
            } else if (args.count_sink) {
                M2 = __fmul_rn(bf16_bits_to_float(sink), kLog2e);
                L2 = 1.0f;
            } else {
                M2 = kEmptyMax;
                L2 = 0.0f;
            }
        };
        // The tile's row sum: from the tensor core (column D of the O buffer) or the two halves' sums.
        // Issued before the loads of O so that one wait covers both.
        auto tile_sum = [&](uint32_t o_tmem, uint32_t t) -> uint32_t {
            if (LT::kSumOnTensor) return tmem_ld1(o_tmem + D);
            return __float_as_uint(bars->l[t & 7][row]);
        };
        uint32_t t = 0, it = 0;
        bool ok = true;
        TcItemIter walk = items_begin(args);
        // The head's sink is fetched one item ahead (only when this kernel runs the second fold), so its
        // latency never sits at an item's start.
        const bool wants_sink = kFinish && args.count_sink && args.sinks != nullptr;
        uint16_t sink_bits = kNoSinkBits;
        if (wants_sink && walk.item < args.n_items) sink_bits = args.sinks[walk.w.kv_head * G + g];
        while (ok && walk.item < args.n_items) {
            const TcItem w = walk.w;
            items_next(args, walk);
            const int head = w.kv_head * G + g;
            const bool valid = t_local < w.valid_tokens;
            const bool warp_has_rows = quad * 32 < (w.valid_tokens << args.log_group);   // warp-uniform
            const uint16_t item_sink = sink_bits;
            if (wants_sink && walk.item < args.n_items) sink_bits = args.sinks[walk.w.kv_head * G + g];
            if constexpr (kTilePartials) {
                // Finely split decode: every tile's own partial goes to the workspace, both folds to the merge.
                for (int j = 0; j < w.n_tiles; ++j, ++t) {
                    if (!mbar_wait(&bars->o_full, t & 1, abort_flag, args.status, 9)) { ok = false; break; }
                    tc_fence_after();
                    if (!warp_has_rows) {
                        tc_fence_before();
                        mbar_arrive(&bars->o_free);
                        continue;
                    }
                    const uint32_t o_tmem = tmem + lane_base + LT::kOCol0;
                    const uint32_t l_bits = tile_sum(o_tmem, t);   // valid after the first wait below
                    const size_t prow = (size_t(w.row0) * args.q_heads + head) * args.slots + (w.slot + j);
                    #pragma unroll
                    for (int hb = 0; hb < D / 64; ++hb) {
                        uint32_t o[2][32];
                        HC_TMEM_LD32(o_tmem + hb * 64, o[0]);
                        HC_TMEM_LD32(o_tmem + hb * 64 + 32, o[1]);
                        tc_wait_ld();
                        if (hb == D / 64 - 1) {
                            tc_fence_before();
                            mbar_arrive(&bars->o_free);
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
                        *reinterpret_cast<float2*>(args.part_ml + prow * 2) =
                            make_float2(bars->mm[t & 7][row], __uint_as_float(l_bits));
                    }
                }
                ++it;
                continue;
            }
            // The running segment's partial: a fold over its tiles from the empty state.
            float M = kEmptyMax, L = 0.0f;
            float A[D];
            #pragma unroll
            for (int i = 0; i < D; ++i) A[i] = 0.0f;
            // One pass per segment the item touches.  With finish, the row's second fold runs between
            // the passes.  Its state is kept out of the registers: (M2, L2) in shared memory, the values
            // in global memory (element i of this thread's row at state[i * kStateStride]; it stays in L2);
            // both are untouched
            // until the item's first segment is complete, which a tile's segment index tells.
            for (int j = 0; ok && j < w.n_tiles;) {
                const int pass_tile = w.tile_first + j * world;
                const int pass_last = (((pass_tile >> args.map.log_segment) + 1) << args.map.log_segment) - 1;
                const int pass_end = min(w.n_tiles, j + (pass_last - pass_tile) / world + 1);
                // The first fold over the segment's tiles.
                for (; j < pass_end; ++j, ++t) {
                    if (!mbar_wait(&bars->o_full, t & 1, abort_flag, args.status, 9)) { ok = false; break; }
                    tc_fence_after();
                    if (!warp_has_rows) {
                        tc_fence_before();
                        mbar_arrive(&bars->o_free);
                        continue;
                    }
                    const uint32_t o_tmem = tmem + lane_base + LT::kOCol0;
                    const uint32_t l_bits = tile_sum(o_tmem, t);   // valid after the first wait below
                    float Mn, a, b;
                    #pragma unroll
                    for (int hb = 0; hb < D / 64; ++hb) {
                        uint32_t o[2][32];
                        HC_TMEM_LD32(o_tmem + hb * 64, o[0]);
                        HC_TMEM_LD32(o_tmem + hb * 64 + 32, o[1]);
                        if (hb == 0) fold_coefficients(M, bars->mm[t & 7][row], Mn, a, b);   // while the loads fly
                        tc_wait_ld();
                        if (hb == D / 64 - 1) {
                            tc_fence_before();
                            mbar_arrive(&bars->o_free);
                        }
                        if (hb == 0) {
                            L = __fmaf_rn(L, a, __fmul_rn(__uint_as_float(l_bits), b));
                            M = Mn;
                        }
                        #pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            #pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                const int col = hb * 64 + u * 32 + i;
                                fold_value2(A[col], A[col + 1], a, o[u][i], o[u][i + 1], b);
                            }
                        }
                    }
                }
                if constexpr (!kFinish) {
                    // The segment's partial goes to the workspace (a merge kernel runs the second fold), and
                    // the next segment of the run starts over.
                    if (ok && valid) {
                        const int slot = (pass_tile >> args.map.log_segment) - w.first_segment;
                        const size_t prow = ((size_t(w.row0 + t_local)) * args.q_heads + head) * args.slots + slot;
                        float* dst = args.part_o + prow * D;
                        #pragma unroll
                        for (int i = 0; i < D; i += 4) {
                            *reinterpret_cast<float4*>(dst + i) = make_float4(A[i], A[i + 1], A[i + 2], A[i + 3]);
                        }
                        *reinterpret_cast<float2*>(args.part_ml + prow * 2) = make_float2(M, L);
                    }
                    if (j < w.n_tiles) {
                        #pragma unroll
                        for (int i = 0; i < D; ++i) A[i] = 0.0f;
                        M = kEmptyMax;
                        L = 0.0f;
                    }
                }
                if (kFinish && ok && warp_has_rows && j < w.n_tiles) {
                    // A segment is complete and another follows: fold it into the row's state and start over.
                    const int tile = w.tile_first + (j - 1) * world;
                    const bool state_holds = (tile >> args.map.log_segment) != (w.tile_first >> args.map.log_segment);
                    float M2, L2;
                    second_fold_state(state_holds, item_sink, M2, L2);
                    float Mn2, a2, b2;
                    fold_coefficients(M2, M, Mn2, a2, b2);
                    bars->m2[row] = Mn2;
                    bars->l2[row] = __fmaf_rn(L2, a2, __fmul_rn(L, b2));
                    float* const state = state_of_row();
                    #pragma unroll
                    for (int i0 = 0; i0 < D; i0 += 16) {
                        float before[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) before[i] = state_holds ? state[(i0 + i) * kStateStride] : 0.0f;
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            state[(i0 + i) * kStateStride] = fold_value(before[i], a2, A[i0 + i], b2);
                            A[i0 + i] = 0.0f;
                        }
                        asm volatile("" ::: "memory");      // sixteen values in flight, not all of them
                    }
                    M = kEmptyMax;
                    L = 0.0f;
                }
            }
            if (!ok) break;
            const size_t out_row = size_t(w.row0 + t_local);
            if constexpr (!kFinish) {
                ++it;
                continue;
            }
            // The row's last segment: the last step of the second fold, which started from the sink (or,
            // on the ranks of a sequence-sharded cache that do not count it, from the empty state).
            {
                const int last_tile = w.tile_first + (w.n_tiles - 1) * world;
                const bool state_holds = warp_has_rows && (last_tile >> args.map.log_segment) != (w.tile_first >> args.map.log_segment);
                float M2, L2;
                second_fold_state(state_holds, item_sink, M2, L2);
                float Mn, a, b;
                fold_coefficients(M2, M, Mn, a, b);
                L = __fmaf_rn(L2, a, __fmul_rn(L, b));
                M = Mn;
                const float* const state = state_of_row();
                if (state_holds) {
                    #pragma unroll
                    for (int i0 = 0; i0 < D; i0 += 16) {
                        float before[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) before[i] = state[(i0 + i) * kStateStride];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) A[i0 + i] = fold_value(before[i], a, A[i0 + i], b);
                        asm volatile("" ::: "memory");
                    }
                } else {
                    // fold_value(0, a, A, b) = 0 * a + A * b = A * b exactly: one multiply.
                    #pragma unroll
                    for (int i = 0; i < D; ++i) A[i] = __fmul_rn(A[i], b);
                }
            }
            if (warp_has_rows && !args.ep.write_partial && args.ep.gate_layout == HC_GATE_NONE &&
                args.ep.io_dtype != HC_F32) {
                // bf16 output without a gate (warp-uniform): rows go through shared memory so that a
                // store instruction writes whole 128-byte lines (the G heads of a token are adjacent
                // in memory) instead of 16 bytes of 32 different rows.
                unsigned char* stage = epi_smem + (warp & 3) * LT::kEpiWarpBytes;
                uint16_t* out16 = reinterpret_cast<uint16_t*>(args.ep.out);
                #pragma unroll
                for (int b = 0; b < D / 64; ++b) {
                    #pragma unroll
                    for (int ch = 0; ch < 8; ++ch) {
                        float r[8];
                        #pragma unroll
                        for (int u = 0; u < 8; ++u) r[u] = finish_value(A[b * 64 + ch * 8 + u], L, false, 0.0f);
                        uint4 packed;
                        packed.x = pack_bf16x2(r[0], r[1]);
                        packed.y = pack_bf16x2(r[2], r[3]);
                        packed.z = pack_bf16x2(r[4], r[5]);
                        packed.w = pack_bf16x2(r[6], r[7]);
                        *reinterpret_cast<uint4*>(stage + lane * 128 + ((ch ^ (lane & 7)) << 4)) = packed;
                    }
                    __syncwarp();
                    #pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const int rl = k * 4 + (lane >> 3), ch = lane & 7;
                        const int row2 = quad * 32 + rl;
                        const int t2 = row2 >> args.log_group;
                        if (t2 < w.valid_tokens) {
                            const size_t vec2 = size_t(w.row0 + t2) * args.q_heads + size_t(w.kv_head) * G + (row2 & (G - 1));
                            const uint4 value = *reinterpret_cast<const uint4*>(stage + rl * 128 + ((ch ^ (rl & 7)) << 4));
                            *reinterpret_cast<uint4*>(out16 + vec2 * D + b * 64 + ch * 8) = value;
                        }
                    }
                    __syncwarp();
                }
            } else if (valid) {
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
            ++it;
        }
    }

    // Teardown.  On the abort path the producer first lets its copies in flight land (bounded).
    if (warp == 0 && lane == 0 && *abort_flag != 0) {
        const long long start = clock64();
        while (static_cast<unsigned long long>(clock64() - start) < 200000000ull) { }
    }
    tc_fence_before();
    __syncthreads();
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

bool dim_ok(int d) { return d == 64 || d == 128 || d == 256; }

}  // namespace

hc_status tc_encode_2d(void* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return fail(HC_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {cuuint64_t(cols), cuuint64_t(rows)};
    const cuuint64_t strides[1] = {cuuint64_t(cols) * 2};
    const cuuint32_t box[2] = {64, cuuint32_t(box_rows)};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(static_cast<CUtensorMap*>(map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                               strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(HC_CUDA_ERROR, "cuTensorMapEncodeTiled failed with code " + std::to_string(int(rc)));
    return HC_OK;
}

bool tc_supported(const AttnShape& shape) { return dim_ok(shape.head_dim) && shape.group <= 16; }

hc_status tc_make_tensor_maps(hc_kv_cache* cache, hc_layer_store& layer) {
    if (!dim_ok(layer.desc.head_dim)) return HC_OK;
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return fail(HC_CUDA_ERROR, "cuTensorMapEncodeTiled is not available from this driver");
    const int d = layer.desc.head_dim;
    for (int which = 0; which < 2; ++which) {
        CUtensorMap* map = new CUtensorMap;
        const bool paged = cache->pages_dev != nullptr && layer.ring == 0;       // one plane per head, shared
        const cuuint64_t dims[3] = {cuuint64_t(d), cuuint64_t(layer.capacity),
                                    cuuint64_t(paged ? 1 : cache->max_seqs) * layer.desc.kv_heads};
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

template <int D, int MODE>
static hc_status launch_tc_mode(hc_context* ctx, const TcArgs& args, const hc_layer_store& layer, cudaStream_t stream) {
    using LT = TcLayout<D>;
    const int smem = LT::kSmemBytes + int(sizeof(TcBarriers));
    static bool configured[64] = {};                 // per device: the attribute is set once
    if (!configured[ctx->device & 63]) {
        cudaError_t err = cudaFuncSetAttribute(attention_tc_kernel<D, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return check_cuda(err, "attention_tc_kernel shared memory");
        configured[ctx->device & 63] = true;
    }
    // Persistent: one CTA per SM at most, each walking items blockIdx.x, blockIdx.x + gridDim.x, ...
    const int grid = std::max(1, std::min(args.n_items, std::max(ctx->sm_count, 1)));
    const cudaError_t launched = launch_pdl(attention_tc_kernel<D, MODE>, grid, kTcThreads, size_t(smem), stream,
                                            *static_cast<const CUtensorMap*>(layer.tmap_k),
                                            *static_cast<const CUtensorMap*>(layer.tmap_v), args);
    ctx->launches += 1;
    if (launched != cudaSuccess) return check_cuda(launched, "attention_tc_kernel launch");
    return check_cuda(cudaGetLastError(), "attention_tc_kernel launch");
}

template <int D>
static hc_status launch_tc(hc_context* ctx, const TcArgs& args, const hc_layer_store& layer, cudaStream_t stream) {
    if (args.finish) return launch_tc_mode<D, kModeFinish>(ctx, args, layer, stream);
    if (args.tile_partials) return launch_tc_mode<D, kModeTiles>(ctx, args, layer, stream);
    return launch_tc_mode<D, kModeSegments>(ctx, args, layer, stream);
}

// What the two launchers share.
static void fill_common_args(TcArgs& args, hc_context* ctx, const AttnShape& shape, const CacheView& cache,
                             const uint16_t* q, const Workspace& ws, const EpilogueArgs& ep) {
    args.q = q;
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
    args.part_o = ws.part_o;
    args.part_ml = ws.part_ml;
    args.row_state = ws.part_o;       // a launch uses one or the other
}

// Floats of row state a whole-row launch needs.
static size_t row_state_floats(const hc_context* ctx, const AttnShape& shape) {
    return size_t(std::max(ctx->sm_count, 1)) * shape.head_dim * kRows;
}

static hc_status launch_any(hc_context* ctx, const AttnShape& shape, const TcArgs& args, const hc_layer_store& layer,
                            cudaStream_t stream) {
    if (shape.head_dim == 64) return launch_tc<64>(ctx, args, layer, stream);
    if (shape.head_dim == 128) return launch_tc<128>(ctx, args, layer, stream);
    return launch_tc256(ctx, layer.tmap_k, layer.tmap_v, &args, args.n_items, stream);
}

hc_status tc_prefill(hc_context* ctx, const AttnShape& shape, const hc_layer_store& layer, const CacheView& cache,
                     int seq, const uint16_t* q, int tokens, int first_position, const Workspace& ws,
                     const EpilogueArgs& ep, cudaStream_t stream, const int* block_ends) {
    if (!layer.tmap_k || !layer.tmap_v) return fail(HC_UNSUPPORTED, "this layer has no tensor maps");
    if (tokens <= 0) return HC_OK;
    TcArgs args{};
    fill_common_args(args, ctx, shape, cache, q, ws, ep);
    args.tokens = tokens;
    args.first_position = first_position;
    args.seq = seq;
    args.log_run = cache.map.log_segment;
    const int tokens_per_tile = kRows / shape.group;
    args.mtiles = (tokens + tokens_per_tile - 1) / tokens_per_tile;
    // Segments and key tiles a row tile spans, at most.
    int slots = 1, most_tiles = 1;
    for (int mtile = 0; mtile < args.mtiles; ++mtile) {
        const int first = first_position + mtile * tokens_per_tile;
        const int last = first_position + (block_ends ? tokens : std::min((mtile + 1) * tokens_per_tile, tokens)) - 1;
        slots = std::max(slots, visible_groups(first, last, shape.window, cache.map.log_segment));
        most_tiles = std::max(most_tiles, row_tiles(cache.map, first, last, shape.window).count);
    }
    // Whole rows per item, or one item per (row tile, kv head, segment) merged afterwards: whichever
    // the longest thread block finishes first, in units of one key tile's time.  An item costs its
    // tiles plus a start and an end (about four tiles' worth; eight for head_dim 256, whose kernel
    // does not look ahead across items), the merge and its launch about ten.  Measured on one
    // GPT-OSS chunk of 512 tokens with 1, 2 and 4 kv heads: the model picks the faster of the two
    // in all but ties.
    const int whole_items = args.mtiles * shape.kv_heads;
    const size_t rows = size_t(tokens) * shape.q_heads;
    const bool can_split = slots > 1 && rows * slots * shape.head_dim <= ws.part_o_floats && rows * slots * 2 <= ws.part_ml_floats;
    const bool can_finish = slots == 1 || row_state_floats(ctx, shape) <= ws.part_o_floats;
    const int sms = std::max(ctx->sm_count, 1);
    const int item_cost = shape.head_dim == 256 ? 8 : 4;
    const int whole_time = ((whole_items + sms - 1) / sms) * (most_tiles + item_cost);
    const int split_time = ((whole_items * slots + sms - 1) / sms) * (std::min(most_tiles, 1 << cache.map.log_segment) + item_cost) + 10;
    // With bidirectional blocks a row's last key is known on the device only: whole rows per item, no
    // merge over per-row segment lists (or the general kernel, if the row state does not fit).
    if (block_ends && !can_finish) return simt_prefill(ctx, shape, cache, seq, q, tokens, first_position, ep, stream, block_ends);
    args.block_ends = block_ends;
    args.appended = first_position + tokens;
    const bool whole = block_ends != nullptr || !can_split || (can_finish && whole_time <= split_time);
    if (whole && !can_finish) {
        return fail(HC_KV_OVERFLOW, "prefill: the attention workspace is too small for this chunk (" + std::to_string(tokens) +
                                        " tokens over " + std::to_string(slots) + " segments)");
    }
    args.finish = whole ? 1 : 0;
    if (whole) slots = 1;
    args.slots = slots;
    args.n_items = whole_items * slots;
    args.magic_slots = division_magic(uint32_t(slots), uint32_t(args.n_items));
    args.magic_kv_heads = division_magic(uint32_t(shape.kv_heads), uint32_t(args.n_items));
    const hc_status st = launch_any(ctx, shape, args, layer, stream);
    if (st != HC_OK || args.finish) return st;
    return launch_merge_prefill(ctx, shape, cache.map, tokens, first_position, ws, slots, ep, stream);
}

DecodePlan tc_plan_decode(const hc_context* ctx, const AttnShape& shape, const RowMap& map, const BatchMeta& meta, int n_seq,
                          size_t part_o_floats) {
    // About six items per thread block, so that the static round-robin balances (measured best of
    // 3 .. 12 on uniform and ragged batches); the head_dim 256 kernel does not look ahead across
    // items: about one per thread block.
    const int target = (shape.head_dim == 256 ? 1 : 6) * std::max(ctx->sm_count, 1);
    DecodePlan plan = plan_decode(shape, map, meta, n_seq, target, true, 64);
    if (plan.finish && row_state_floats(ctx, shape) > part_o_floats) {
        // A whole row that spans two segments needs the second fold's state, for which there is no room.
        bool spans = false;
        for (int b = 0; b < n_seq; ++b) spans = spans || visible_groups(meta.pos[b], meta.pos[b], shape.window, map.log_segment) > 1;
        if (spans) plan = plan_decode(shape, map, meta, n_seq, target, false, 64);
    }
    return plan;
}

hc_status tc_decode(hc_context* ctx, const AttnShape& shape, const hc_layer_store& layer, const CacheView& cache,
                    const BatchMeta& meta, int n_seq, const uint16_t* q, const Workspace& ws,
                    const EpilogueArgs& ep, cudaStream_t stream) {
    if (!layer.tmap_k || !layer.tmap_v) return fail(HC_UNSUPPORTED, "this layer has no tensor maps");
    if (n_seq <= 0) return HC_OK;
    TcArgs args{};
    fill_common_args(args, ctx, shape, cache, q, ws, ep);
    args.tokens = n_seq;
    args.decode = 1;
    args.meta = meta;
    const DecodePlan plan = tc_plan_decode(ctx, shape, cache.map, meta, n_seq, ws.part_o_floats);
    args.finish = plan.finish;
    args.log_run = plan.log_run;
    args.tile_partials = plan.tile_partials;
    args.slots = plan.slots;
    // One item per (sequence, kv head, run of the sequence's visible key tiles).
    int next = 0;
    for (int b = 0; b < n_seq; ++b) {
        int n = 1;
        if (plan.tile_partials) {
            n = visible_groups(meta.pos[b], meta.pos[b], shape.window, plan.log_run);
        } else if (!plan.finish) {
            // The sequence's segments in runs of one size, about plan.run_segments each.
            const int segments = visible_groups(meta.pos[b], meta.pos[b], shape.window, cache.map.log_segment);
            const int want = (segments + plan.run_segments - 1) / plan.run_segments;
            const int run = (segments + want - 1) / want;
            n = (segments + run - 1) / run;
            args.seq_run[b] = static_cast<unsigned short>(run);
        }
        args.item_start[b] = next;
        args.seq_slots[b] = static_cast<unsigned short>(n);
        args.seq_magic[b] = division_magic(uint32_t(n), uint32_t(n) * uint32_t(shape.kv_heads));
        next += n * shape.kv_heads;
    }
    for (int b = n_seq; b <= kMaxBatch; ++b) args.item_start[b] = next;
    args.n_items = next;
    if (!args.finish) {
        const size_t rows = size_t(n_seq) * shape.q_heads;
        if (rows * plan.slots * shape.head_dim > ws.part_o_floats || rows * plan.slots * 2 > ws.part_ml_floats) {
            return fail(HC_KV_OVERFLOW, "decode: the split-attention workspace is too small for this call");
        }
    }
    const hc_status st = launch_any(ctx, shape, args, layer, stream);
    if (st != HC_OK || args.finish) return st;
    return launch_merge_decode(ctx, shape, cache.map, meta, n_seq, ws, plan, ep, stream);
}

}  // namespace hc
