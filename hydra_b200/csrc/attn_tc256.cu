// attn_tc256.cu — the tcgen05 attention kernel for head_dim 256 (Gemma- and Qwen-shaped layers).
//
// Same arithmetic and the same item list as attn_tc.cu; what changes is how a 128 x 256 output row
// tile fits the machine.  Tensor memory holds two S buffers (2 x 128 columns) and ONE O buffer
// (256 columns): all 512 columns.  Shared memory holds one Q tile (64 KB), one K tile and one V tile
// (64 KB each).  A row of O is 256 floats, too many for one thread, so two warpgroups fold it, one
// per 128-column half.
//
//   warpgroup 0   warp 0 producer (TMA), warp 1 MMA issuer
//   warpgroup 1   softmax, thread = row, the row walked in 64-column passes (maximum, then weights)
//   warpgroup 2   fold of O columns 0-127, stages the next item's Q tile
//   warpgroup 3   fold of O columns 128-255
//
// Registers per thread after setmaxnreg: 48 / 112 / 176 / 176.  Every mbarrier wait is bounded.

#include <algorithm>

#include "internal.hpp"
#include "tc_common.cuh"
#include "tc_ptx.cuh"

namespace hc {
namespace {


constexpr int kD = 256;
constexpr int kBlocks256 = kD / 64;
constexpr int kTileBytes256 = kTileKeys * kD * 2;        // 64 KB
constexpr int kQBytes256 = kRows * kD * 2;               // 64 KB
constexpr int kOCol256 = 2 * kTileKeys;

struct Tc256Barriers {
    uint64_t q_full, q_empty;
    uint64_t k_full, k_empty, v_full, v_empty;
    uint64_t s_full[2], p_full[2], o_full, o_free;
    uint32_t tmem_base;
    int abort_flag;
    float mm[4][kRows];
    float l[4][kRows];
    float m2[2][kRows], l2[2][kRows];   // the rows' second fold between segments, per half
};

// MODE says what becomes of an item's rows (TcArgs: finish, tile_partials), so that a launch carries
// the code of its own way only: 0 = the kernel finishes them, 1 = segment partials, 2 = tile partials.
template <int MODE>
__global__ void __launch_bounds__(kTcThreads, 1)
attention_tc256_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       const TcArgs args) {
    constexpr bool kFinish = MODE == 0;
    constexpr bool kTilePartials = MODE == 2;
    extern __shared__ unsigned char raw_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = base;
    unsigned char* k_smem = q_smem + kQBytes256;
    unsigned char* v_smem = k_smem + kTileBytes256;
    Tc256Barriers* bars = reinterpret_cast<Tc256Barriers*>(v_smem + kTileBytes256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int wg = warp >> 2;
    const int G = 1 << args.log_group;
    const int world = max(args.map.world, 1);
    volatile int* abort_flag = &bars->abort_flag;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 128);
        mbar_init(&bars->q_empty, 1);
        mbar_init(&bars->k_full, 1);
        mbar_init(&bars->k_empty, 1);
        mbar_init(&bars->v_full, 1);
        mbar_init(&bars->v_empty, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->p_full[i], 128);
        }
        mbar_init(&bars->o_full, 1);
        mbar_init(&bars->o_free, 256);
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(&bars->tmem_base, 512);
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tmap_k);
        prefetch_tensormap(&tmap_v);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    pdl_wait();        // set-up done; from here on the kernel reads what earlier kernels wrote

    if (wg == 0) {
    reg_dealloc<48>();
    if (warp == 0) {
        // ===== producer =====
        if (lane == 0) {
            uint32_t t = 0;
            bool ok = true;
            for (TcItemIter walk = items_begin(args); ok && walk.item < args.n_items; items_next(args, walk)) {
                const TcItem& w = walk.w;
                const int plane = cache_plane(args.map, w.seq, args.kv_heads, w.kv_head);
                for (int j = 0; j < w.n_tiles; ++j, ++t) {
                    const int row0 = cache_row(args.map, w.seq, (w.tile_first + j * world) * kTileKeys);
                    if (t > 0 && !mbar_wait(&bars->k_empty, (t - 1) & 1, abort_flag, args.status, 1)) { ok = false; break; }
                    mbar_expect_tx(&bars->k_full, kTileBytes256);
                    for (int b = 0; b < kBlocks256; ++b) {
                        tma_load_3d(k_smem + b * (kTileKeys * 128), &tmap_k, &bars->k_full, b * 64, row0, plane);
                    }
                    if (t > 0 && !mbar_wait(&bars->v_empty, (t - 1) & 1, abort_flag, args.status, 2)) { ok = false; break; }
                    mbar_expect_tx(&bars->v_full, kTileBytes256);
                    for (int b = 0; b < kBlocks256; ++b) {
                        tma_load_3d(v_smem + b * (kTileKeys * 128), &tmap_v, &bars->v_full, b * 64, row0, plane);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: S(t + 1) is issued before P(t) is awaited, inside an item.  The whole warp
        // walks the loop and waits, so control flow stays warp-uniform; one elected lane issues the
        // tcgen05 instructions (a lane in a divergent branch pays several times more per instruction). =====
        {
            constexpr uint32_t idesc_qk = instr_desc(kTileKeys, false);
            constexpr uint32_t idesc_pv = instr_desc(kD, true);
            const uint64_t q_desc0 = smem_desc(smem_u32(q_smem), 16);
            const uint64_t k_desc0 = smem_desc(smem_u32(k_smem), 16);
            const uint64_t v_desc0 = smem_desc(smem_u32(v_smem), kTileKeys * 128);
            auto issue_qk = [&](uint32_t t, bool last) -> bool {
                if (!mbar_wait(&bars->k_full, t & 1, abort_flag, args.status, 3)) return false;
                tc_fence_after();
                if (elect_one()) {
                    const uint32_t s_tmem = tmem + (t & 1) * kTileKeys;
                    #pragma unroll
                    for (int b = 0; b < kBlocks256; ++b) {
                        #pragma unroll
                        for (int ks = 0; ks < 4; ++ks) {
                            const uint64_t off = uint64_t((b * (kRows * 128) + ks * 32) >> 4);
                            mma_ss(s_tmem, q_desc0 + off, k_desc0 + off, idesc_qk, (b | ks) != 0 ? 1u : 0u);
                        }
                    }
                    tc_commit(&bars->k_empty);
                    tc_commit(&bars->s_full[t & 1]);
                    if (last) tc_commit(&bars->q_empty);
                }
                __syncwarp();
                return true;
            };
            uint32_t t = 0, it = 0;
            bool ok = true;
            for (TcItemIter walk = items_begin(args); ok && walk.item < args.n_items; items_next(args, walk), ++it) {
                const int n_tiles = walk.w.n_tiles;
                if (!mbar_wait(&bars->q_full, it & 1, abort_flag, args.status, 4)) break;
                tc_fence_after();
                ok = issue_qk(t, n_tiles == 1);
                for (int j = 0; ok && j < n_tiles; ++j, ++t) {
                    if (j + 1 < n_tiles) {
                        ok = issue_qk(t + 1, j + 2 == n_tiles);
                        if (!ok) break;
                    }
                    if (!mbar_wait(&bars->p_full[t & 1], (t >> 1) & 1, abort_flag, args.status, 5)) { ok = false; break; }
                    if (!mbar_wait(&bars->v_full, t & 1, abort_flag, args.status, 6)) { ok = false; break; }
                    if (t > 0 && !mbar_wait(&bars->o_free, (t - 1) & 1, abort_flag, args.status, 7)) { ok = false; break; }
                    tc_fence_after();
                    if (elect_one()) {
                        const uint32_t p_tmem = tmem + (t & 1) * kTileKeys;
                        #pragma unroll
                        for (int ks = 0; ks < kTileKeys / 16; ++ks) {
                            mma_ts(tmem + kOCol256, p_tmem + ks * 8, v_desc0 + uint64_t((ks * 2048) >> 4), idesc_pv,
                                   ks != 0 ? 1u : 0u);
                        }
                        tc_commit(&bars->v_empty);
                        tc_commit(&bars->o_full);
                    }
                    __syncwarp();
                }
            }
        }
    }
    } else if (wg == 1) {
        // ===== softmax: thread = row =====
        reg_dealloc<112>();
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        const float neg_inf = __int_as_float(0xff800000);
        uint32_t t = 0;
        bool ok = true;
        for (TcItemIter walk = items_begin(args); ok && walk.item < args.n_items; items_next(args, walk)) {
            const TcItem& w = walk.w;
            const bool valid = t_local < w.valid_tokens;
            const bool warp_has_rows = quad * 32 < (w.valid_tokens << args.log_group);
            int pos = valid ? w.first_pos + t_local : -1;
            const int lo = args.window > 0 ? max(0, pos - args.window + 1) : 0;
            // From here on the last key the row sees: its own, or the end of its bidirectional block.
            if (!args.decode && args.block_ends != nullptr && valid) {
                pos = max(pos, min(__ldg(args.block_ends + (w.first_pos - args.first_position) + t_local), args.appended) - 1);
            }
            for (int j = 0; j < w.n_tiles; ++j, ++t) {
                const int sb = int(t & 1);
                if (!mbar_wait(&bars->s_full[sb], (t >> 1) & 1, abort_flag, args.status, 8)) { ok = false; break; }
                tc_fence_after();
                if (!warp_has_rows) {
                    tc_fence_before();
                    mbar_arrive(&bars->p_full[sb]);
                    continue;
                }
                const uint32_t s_tmem = tmem + lane_base + sb * kTileKeys;
                const int key0 = (w.tile_first + j * world) * kTileKeys;
                const int c_lo = lo - key0;
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
                // Pass 2: weights; P overwrites the S columns already consumed.  The row sum has a
                // fixed shape: groups of 32 columns by the butterfly tree, the four groups in order.
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
                bars->mm[t & 3][row] = __fmul_rn(m, args.c);
                bars->l[t & 3][row] = sum;
                tc_wait_st();
                tc_fence_before();
                mbar_arrive(&bars->p_full[sb]);
            }
        }
    } else {
        // ===== fold + epilogue: two threads per row, one per 128-column half of O =====
        reg_alloc<176>();
        const int half = wg - 2;
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const int g = row & (G - 1);
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        const uint32_t o_tmem = tmem + lane_base + kOCol256 + half * 128;
        auto state_of_row = [&]() -> float* {
            return args.row_state + size_t(blockIdx.x) * (kD * kRows) + size_t(half * 128) * kRows + row;
        };
        // (M, L) the second fold stands at: what the last segment end left, or the seed.
        auto second_fold_state = [&](bool state_holds, uint16_t sink, float& M2, float& L2) {
            if (state_holds) {
                M2 = bars->m2[half][row];
                L2 = bars->l2[half][row];
            } else if (args.count_sink) {
                M2 = __fmul_rn(bf16_bits_to_float(sink), kLog2e);
                L2 = 1.0f;
            } else {
                M2 = kEmptyMax;
                L2 = 0.0f;
            }
        };
        auto stage_q = [&](const TcItem& w) {
            const bool valid = t_local < w.valid_tokens;
            const uint16_t* src = args.q + (size_t(w.row0 + t_local) * args.q_heads + size_t(w.kv_head) * G + g) * kD;
            // The row's 32 pieces of 16 bytes go global -> shared in one flight (cp.async, no registers).
            const uint32_t dst = smem_u32(q_smem);
            const uint16_t* from = valid ? src : args.q;
            #pragma unroll
            for (int b = 0; b < kBlocks256; ++b) {
                #pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    cp_async16(dst + b * (kRows * 128) + row * 128 + ((ch ^ (row & 7)) << 4), from + b * 64 + ch * 8,
                               valid ? 16u : 0u);
                }
            }
            cp_async_wait_all();
            fence_proxy_async();
            mbar_arrive(&bars->q_full);
        };
        uint32_t t = 0, it = 0;
        bool ok = true;
        TcItemIter walk = items_begin(args);
        if (half == 0 && walk.item < args.n_items) stage_q(walk.w);
        // The head's sink is fetched one item ahead (only when this kernel runs the second fold).
        const bool wants_sink = kFinish && args.count_sink && args.sinks != nullptr;
        uint16_t sink_bits = kNoSinkBits;
        if (wants_sink && walk.item < args.n_items) sink_bits = args.sinks[walk.w.kv_head * G + g];
        while (ok && walk.item < args.n_items) {
            const TcItem w = walk.w;
            items_next(args, walk);
            const int head = w.kv_head * G + g;
            const bool valid = t_local < w.valid_tokens;
            const bool warp_has_rows = quad * 32 < (w.valid_tokens << args.log_group);
            const uint16_t item_sink = sink_bits;
            if (wants_sink && walk.item < args.n_items) sink_bits = args.sinks[walk.w.kv_head * G + g];
            // Half 0 also stages the next item's Q tile once this item's last S has been issued.
            auto stage_next_q = [&](int j) -> bool {
                if (half == 0 && j == w.n_tiles - 1 && walk.item < args.n_items) {
                    if (!mbar_wait(&bars->q_empty, it & 1, abort_flag, args.status, 10)) return false;
                    stage_q(walk.w);
                }
                return true;
            };
            if constexpr (kTilePartials) {
                // Finely split decode: every tile's own partial goes to the workspace, both folds to the merge.
                for (int j = 0; j < w.n_tiles; ++j, ++t) {
                    if (!stage_next_q(j)) { ok = false; break; }
                    if (!mbar_wait(&bars->o_full, t & 1, abort_flag, args.status, 9)) { ok = false; break; }
                    tc_fence_after();
                    if (!warp_has_rows) {
                        tc_fence_before();
                        mbar_arrive(&bars->o_free);
                        continue;
                    }
                    const size_t prow = (size_t(w.row0) * args.q_heads + head) * args.slots + (w.slot + j);
                    #pragma unroll
                    for (int chunk = 0; chunk < 4; ++chunk) {
                        uint32_t o[32];
                        HC_TMEM_LD32(o_tmem + chunk * 32, o);
                        tc_wait_ld();
                        if (chunk == 3) {
                            tc_fence_before();
                            mbar_arrive(&bars->o_free);
                        }
                        if (valid) {
                            float* dst = args.part_o + prow * kD + half * 128 + chunk * 32;
                            #pragma unroll
                            for (int i = 0; i < 32; i += 4) {
                                *reinterpret_cast<uint4*>(dst + i) = make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                            }
                        }
                    }
                    if (valid && half == 0) {
                        *reinterpret_cast<float2*>(args.part_ml + prow * 2) = make_float2(bars->mm[t & 3][row], bars->l[t & 3][row]);
                    }
                }
                if (!ok) break;
                ++it;
                continue;
            }
            // The running segment's partial: a fold over its tiles from the empty state (both halves of
            // the row carry M and L, the same chain, the same bits).
            float M = kEmptyMax, L = 0.0f;
            float A[128];
            #pragma unroll
            for (int i = 0; i < 128; ++i) A[i] = 0.0f;
            // One pass per segment the item touches.  With finish, the row's second fold runs between
            // the passes.  Its state is kept out of the registers: (M2, L2) in shared memory (one copy per
            // half), the values in global memory (element i of this thread's half row at
            // state[i * kRows]); both are untouched until the item's first segment is complete, which
            // a tile's segment index tells.
            for (int j = 0; ok && j < w.n_tiles;) {
                const int pass_tile = w.tile_first + j * world;
                const int pass_last = (((pass_tile >> args.map.log_segment) + 1) << args.map.log_segment) - 1;
                const int pass_end = min(w.n_tiles, j + (pass_last - pass_tile) / world + 1);
                // The first fold over the segment's tiles.
                for (; j < pass_end; ++j, ++t) {
                    if (!stage_next_q(j)) { ok = false; break; }
                    if (!mbar_wait(&bars->o_full, t & 1, abort_flag, args.status, 9)) { ok = false; break; }
                    tc_fence_after();
                    if (!warp_has_rows) {
                        tc_fence_before();
                        mbar_arrive(&bars->o_free);
                        continue;
                    }
                    float Mn, a, b;
                    fold_coefficients(M, bars->mm[t & 3][row], Mn, a, b);
                    L = __fmaf_rn(L, a, __fmul_rn(bars->l[t & 3][row], b));
                    M = Mn;
                    #pragma unroll
                    for (int chunk = 0; chunk < 4; ++chunk) {
                        uint32_t o[32];
                        HC_TMEM_LD32(o_tmem + chunk * 32, o);
                        tc_wait_ld();
                        if (chunk == 3) {
                            tc_fence_before();
                            mbar_arrive(&bars->o_free);
                        }
                        #pragma unroll
                        for (int i = 0; i < 32; i += 2) {
                            fold_value2(A[chunk * 32 + i], A[chunk * 32 + i + 1], a, o[i], o[i + 1], b);
                        }
                    }
                }
                if constexpr (!kFinish) {
                    // The segment's partial goes to the workspace (a merge kernel runs the second fold), and
                    // the next segment of the run starts over.
                    if (ok && valid) {
                        const int slot = (pass_tile >> args.map.log_segment) - w.first_segment;
                        const size_t prow = ((size_t(w.row0 + t_local)) * args.q_heads + head) * args.slots + slot;
                        float* dst = args.part_o + prow * kD + half * 128;
                        #pragma unroll
                        for (int i = 0; i < 128; i += 4) {
                            *reinterpret_cast<float4*>(dst + i) = make_float4(A[i], A[i + 1], A[i + 2], A[i + 3]);
                        }
                        if (half == 0) *reinterpret_cast<float2*>(args.part_ml + prow * 2) = make_float2(M, L);
                    }
                    if (j < w.n_tiles) {
                        #pragma unroll
                        for (int i = 0; i < 128; ++i) A[i] = 0.0f;
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
                    bars->m2[half][row] = Mn2;
                    bars->l2[half][row] = __fmaf_rn(L2, a2, __fmul_rn(L, b2));
                    float* const state = state_of_row();
                    #pragma unroll
                    for (int i0 = 0; i0 < 128; i0 += 16) {
                        float before[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) before[i] = state_holds ? state[(i0 + i) * kRows] : 0.0f;
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            state[(i0 + i) * kRows] = fold_value(before[i], a2, A[i0 + i], b2);
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
            const int col0 = half * 128;
            if constexpr (!kFinish) {
                ++it;
                continue;
            }
            // The row's last segment: the last step of the second fold, which started from the sink (or
            // from the empty state).
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
                    for (int i0 = 0; i0 < 128; i0 += 16) {
                        float before[16];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) before[i] = state[(i0 + i) * kRows];
                        #pragma unroll
                        for (int i = 0; i < 16; ++i) A[i0 + i] = fold_value(before[i], a, A[i0 + i], b);
                        asm volatile("" ::: "memory");
                    }
                } else {
                    // fold_value(0, a, A, b) = 0 * a + A * b = A * b exactly: one multiply.
                    #pragma unroll
                    for (int i = 0; i < 128; ++i) A[i] = __fmul_rn(A[i], b);
                }
            }
            if (valid) {
                if (args.ep.write_partial) {
                    float* dst = reinterpret_cast<float*>(args.ep.out) + (out_row * args.q_heads + head) * size_t(kD + 2) + col0;
                    #pragma unroll
                    for (int i = 0; i < 128; i += 2) {
                        *reinterpret_cast<float2*>(dst + i) = make_float2(A[i], A[i + 1]);
                    }
                    if (half == 0) {
                        float* tail = reinterpret_cast<float*>(args.ep.out) + (out_row * args.q_heads + head) * size_t(kD + 2) + kD;
                        tail[0] = M;
                        tail[1] = L;
                    }
                } else {
                    const bool gated = args.ep.gate_layout != HC_GATE_NONE;
                    const size_t vec = out_row * args.q_heads + head;
                    const size_t gate_base = (args.ep.gate_layout == HC_GATE_INTERLEAVED ? vec * size_t(2 * kD) + kD : vec * size_t(kD)) + col0;
                    #pragma unroll
                    for (int i = 0; i < 128; i += 8) {
                        float r[8];
                        #pragma unroll
                        for (int u = 0; u < 8; ++u) {
                            const float gv = gated ? load_io(args.ep.gate, gate_base + i + u, args.ep.io_dtype) : 0.0f;
                            r[u] = finish_value(A[i + u], L, gated, gv);
                        }
                        if (args.ep.io_dtype == HC_F32) {
                            float* dst = reinterpret_cast<float*>(args.ep.out) + vec * kD + col0 + i;
                            *reinterpret_cast<float4*>(dst) = make_float4(r[0], r[1], r[2], r[3]);
                            *reinterpret_cast<float4*>(dst + 4) = make_float4(r[4], r[5], r[6], r[7]);
                        } else {
                            uint4 packed;
                            packed.x = pack_bf16x2(r[0], r[1]);
                            packed.y = pack_bf16x2(r[2], r[3]);
                            packed.z = pack_bf16x2(r[4], r[5]);
                            packed.w = pack_bf16x2(r[6], r[7]);
                            *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(args.ep.out) + vec * kD + col0 + i) = packed;
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
    if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace

hc_status launch_tc256(hc_context* ctx, const void* tmap_k, const void* tmap_v, const void* args_ptr,
                       int n_items, cudaStream_t stream) {
    const TcArgs& args = *static_cast<const TcArgs*>(args_ptr);
    const int smem = 1024 + kQBytes256 + 2 * kTileBytes256 + int(sizeof(Tc256Barriers));
    auto kernel = args.finish ? attention_tc256_kernel<0> : args.tile_partials ? attention_tc256_kernel<2> : attention_tc256_kernel<1>;
    static bool configured[64][3] = {};
    const int mode = args.finish ? 0 : args.tile_partials ? 2 : 1;
    if (!configured[ctx->device & 63][mode]) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return check_cuda(err, "attention_tc256_kernel shared memory");
        configured[ctx->device & 63][mode] = true;
    }
    const int grid = std::max(1, std::min(n_items, std::max(ctx->sm_count, 1)));
    const cudaError_t launched = launch_pdl(kernel, grid, kTcThreads, size_t(smem), stream,
                                            *static_cast<const CUtensorMap*>(tmap_k),
                                            *static_cast<const CUtensorMap*>(tmap_v), args);
    ctx->launches += 1;
    if (launched != cudaSuccess) return check_cuda(launched, "attention_tc256_kernel launch");
    return check_cuda(cudaGetLastError(), "attention_tc256_kernel launch");
}

}  // namespace hc
