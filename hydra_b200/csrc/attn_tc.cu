// attn_tc.cu — chunked-prefill attention on the 5th-generation tensor cores (sm_100a only).
//
// Replaces attention_prefill (Sources/HydraMetal/Shaders/batch.metal:307-427).  Where the reference
// gives every (token, query head) its own threadgroup that streams the whole key range, this kernel
// packs the G query heads that share a KV head and 128/G consecutive tokens into one 128-row tile,
// so each K/V tile fetched by TMA serves 128 query rows, and both contractions run as tcgen05.mma
// with accumulators in tensor memory:
//
//   warp 0      producer: TMA loads of K and V tiles (128 keys x d, 128-byte swizzle) into a ring
//   warp 1      MMA issuer: S = Q K^T (A, B from shared memory), O_j = P V (A = P from tensor memory)
//   warps 2-5   softmax: S from tensor memory, causal / window mask, row maximum, P = bf16(exp2(..)),
//               row sum, P back into tensor memory over S
//   warps 6-9   fold: O_j from tensor memory folded into the row's running (M, L, A) in registers,
//               then the epilogue (divide, gate, store)
//
// The arithmetic is the canonical tile-partial + fold of common.cuh: every key tile yields an
// independent partial with its own maximum and the partials are folded in ascending tile order
// seeded with the sink.  A row's result depends only on that row's query and on the key tiles, not
// on the chunk it arrived in nor on its position inside the 128-row tile.
//
// Every wait on an mbarrier is bounded: after about a second it records HC_TIMEOUT in the
// context's status word, raises a CTA-wide abort flag that all other waits observe, and the CTA
// drains and frees its tensor memory before returning.

#include <cuda.h>

#include <algorithm>

#include "internal.hpp"

namespace hc {
namespace {

constexpr int kTcThreads = 320;          // 10 warps
constexpr int kRows = 128;               // query rows per CTA (MMA M)
constexpr unsigned long long kWaitCycles = 3000000000ull;   // ~1.5 s at 1.9 GHz

// ---- PTX wrappers ---------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return done != 0;
}
// Bounded wait.  Returns false if the CTA is aborting (this wait or another one ran out of time).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status_word, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long start = clock64();
    for (;;) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag != 0) return false;
        if (static_cast<unsigned long long>(clock64() - start) > kWaitCycles) {
            *abort_flag = 1;
            atomicCAS(status_word, 0, 0x100 + where);
            return false;
        }
    }
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

#define HC_TMEM_LD32(taddr, v)                                                                              \
    asm volatile(                                                                                           \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                           \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                          \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"          \
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),  \
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),         \
          "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),       \
          "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),       \
          "=r"(v[29]), "=r"(v[30]), "=r"(v[31])                                                             \
        : "r"(taddr) : "memory")

#define HC_TMEM_ST16(taddr, v)                                                                              \
    asm volatile(                                                                                           \
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "                                                     \
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"                          \
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]),         \
          "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]),     \
          "r"(v[15]) : "memory")

// ---- descriptors ----------------------------------------------------------------------------------

// Shared-memory matrix descriptor, 128-byte swizzle, version 1 (sm_100).  Addresses and offsets in
// units of 16 bytes.  K-major operands: rows of 128 bytes, 8-row groups 1024 bytes apart (SBO).
// MN-major operands (V): the same rows, and 64-element column blocks `lbo_bytes` apart.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes) {
    uint64_t desc = 0;
    desc |= uint64_t((addr & 0x3FFFF) >> 4);
    desc |= uint64_t((lbo_bytes >> 4) & 0x3FFF) << 16;
    desc |= uint64_t((1024 >> 4) & 0x3FFF) << 32;
    desc |= uint64_t(1) << 46;             // descriptor version
    desc |= uint64_t(2) << 61;             // SWIZZLE_128B
    return desc;
}
// Instruction descriptor: bf16 x bf16 -> f32, M = 128, N = n; B MN-major when b_mn is set.
__host__ __device__ constexpr uint32_t instr_desc(int n, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | (uint32_t(n >> 3) << 17) |
           (uint32_t(kRows >> 4) << 24);
}

// ---- kernel ---------------------------------------------------------------------------------------

struct TcArgs {
    const uint16_t* q;        // bf16 [tokens][q_heads][d], prepared
    int tokens;
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
    // Decode (split over key tiles): one query token per batch entry, each CTA takes
    // `tiles_per_cta` consecutive tiles of one (sequence, kv head) and writes their partials.
    int decode;
    int tiles_per_cta;
    float* part_o;            // fp32 [rows][part_tiles][d]
    float* part_ml;           // fp32 [rows][part_tiles][2]
    int part_tiles;
    BatchMeta meta;
};

template <int D>
struct TcLayout {
    static constexpr int kBlocks = D / 64;                   // 64-element (128-byte) column blocks
    static constexpr int kTileBytes = kTileKeys * D * 2;     // one K or V tile
    static constexpr int kStages = D == 64 ? 4 : (D == 128 ? 2 : 1);
    static constexpr int kOBufs = D <= 128 ? 2 : 1;
    static constexpr int kQBytes = kRows * D * 2;
    static constexpr int kSCol0 = 0, kSCol1 = 128;
    static constexpr int kOCol0 = 256;
    static constexpr int kTmemCols = 512;
    static constexpr int kSmemBytes = 1024 /*align slack*/ + kQBytes + 2 * kStages * kTileBytes + 4096;
};

struct TcBarriers {
    uint64_t q_full;
    uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
    uint64_t s_full[2], p_full[2], o_full[2], o_free[2];
    uint32_t tmem_base;
    int abort_flag;
    float mm[4][kRows];       // per-tile scaled maxima and sums, softmax -> fold (ring of 4 tiles)
    float l[4][kRows];
};
static_assert(sizeof(TcBarriers) <= 4096 + 4096, "barrier block must fit its reservation");

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                  const TcArgs args) {
    using LT = TcLayout<D>;
    extern __shared__ unsigned char raw_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
    unsigned char* q_smem = base;
    unsigned char* k_smem = q_smem + LT::kQBytes;
    unsigned char* v_smem = k_smem + LT::kStages * LT::kTileBytes;
    TcBarriers* bars = reinterpret_cast<TcBarriers*>(v_smem + LT::kStages * LT::kTileBytes);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int G = 1 << args.log_group;
    const int tokens_per_tile = kRows >> args.log_group;
    const int kv_head = blockIdx.y;
    int token0, valid_tokens, first_pos, seq;
    if (args.decode) {
        token0 = blockIdx.z;                                   // row of q / partial = batch entry
        valid_tokens = 1;
        first_pos = args.meta.pos[blockIdx.z];
        seq = args.meta.seq[blockIdx.z];
    } else {
        const int n_mtiles = (args.tokens + tokens_per_tile - 1) / tokens_per_tile;
        const int mtile = n_mtiles - 1 - int(blockIdx.x);      // longest key ranges first
        token0 = mtile * tokens_per_tile;
        valid_tokens = min(tokens_per_tile, args.tokens - token0);
        first_pos = args.first_position + token0;
        seq = args.seq;
    }
    const int last_pos = first_pos + valid_tokens - 1;
    const int lo_first = args.window > 0 ? max(0, first_pos - args.window + 1) : 0;
    // Key tiles of this row tile, restricted to the tiles this rank owns (sequence sharding).
    const int world = max(args.map.world, 1);
    int tile_first = lo_first / kTileKeys;
    const int tile_last = last_pos / kTileKeys;
    if (world > 1) tile_first += ((args.map.rank - tile_first % world) + world) % world;
    int n_tiles = tile_first > tile_last ? 0 : (tile_last - tile_first) / world + 1;
    int ordinal0 = 0;                                          // ordinal of this CTA's first tile
    if (args.decode) {
        ordinal0 = int(blockIdx.x) * args.tiles_per_cta;
        if (ordinal0 >= n_tiles) return;                       // uniform: before any barrier or allocation
        tile_first += ordinal0 * world;
        n_tiles = min(args.tiles_per_cta, n_tiles - ordinal0);
    }
    const int valid_rows = valid_tokens << args.log_group;

    volatile int* abort_flag = &bars->abort_flag;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 128);
        for (int i = 0; i < 4; ++i) {
            mbar_init(&bars->k_full[i], 1);
            mbar_init(&bars->k_empty[i], 1);
            mbar_init(&bars->v_full[i], 1);
            mbar_init(&bars->v_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->s_full[i], 1);
            mbar_init(&bars->p_full[i], 128);
            mbar_init(&bars->o_full[i], 1);
            mbar_init(&bars->o_free[i], 128);
        }
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(&bars->tmem_base, LT::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;

    if (warp == 0) {
        // ===== producer =====
        if (lane == 0 && n_tiles > 0) {
            const int plane = seq * args.kv_heads + kv_head;
            for (int j = 0; j < n_tiles; ++j) {
                const int slot = j % LT::kStages;
                const uint32_t round = uint32_t(j / LT::kStages);
                const int row0 = row_of_tile(args.map, tile_first + j * world);
                if (j >= LT::kStages &&
                    !mbar_wait(&bars->k_empty[slot], (round - 1) & 1, abort_flag, args.status, 1)) break;
                mbar_expect_tx(&bars->k_full[slot], LT::kTileBytes);
                for (int b = 0; b < LT::kBlocks; ++b) {
                    tma_load_3d(k_smem + slot * LT::kTileBytes + b * (kTileKeys * 128), &tmap_k,
                                &bars->k_full[slot], b * 64, row0, plane);
                }
                if (j >= LT::kStages &&
                    !mbar_wait(&bars->v_empty[slot], (round - 1) & 1, abort_flag, args.status, 2)) break;
                mbar_expect_tx(&bars->v_full[slot], LT::kTileBytes);
                for (int b = 0; b < LT::kBlocks; ++b) {
                    tma_load_3d(v_smem + slot * LT::kTileBytes + b * (kTileKeys * 128), &tmap_v,
                                &bars->v_full[slot], b * 64, row0, plane);
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer =====
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t idesc_qk = instr_desc(kTileKeys, false);
            constexpr uint32_t idesc_pv = instr_desc(D, true);
            const uint32_t q_addr = smem_u32(q_smem);
            auto issue_qk = [&](int j) -> bool {
                const int slot = j % LT::kStages;
                if (!mbar_wait(&bars->k_full[slot], uint32_t(j / LT::kStages) & 1, abort_flag, args.status, 3)) return false;
                tc_fence_after();
                const uint32_t k_addr = smem_u32(k_smem + slot * LT::kTileBytes);
                const uint32_t s_tmem = tmem + ((j & 1) ? LT::kSCol1 : LT::kSCol0);
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
                tc_commit(&bars->s_full[j & 1]);
                return true;
            };
            bool ok = mbar_wait(&bars->q_full, 0, abort_flag, args.status, 4);
            if (ok) {
                tc_fence_after();
                ok = issue_qk(0);
            }
            for (int j = 0; ok && j < n_tiles; ++j) {
                if (j + 1 < n_tiles) {
                    ok = issue_qk(j + 1);
                    if (!ok) break;
                }
                const int slot = j % LT::kStages;
                const int ob = LT::kOBufs == 2 ? (j & 1) : 0;
                if (!mbar_wait(&bars->p_full[j & 1], uint32_t(j >> 1) & 1, abort_flag, args.status, 5)) break;
                if (!mbar_wait(&bars->v_full[slot], uint32_t(j / LT::kStages) & 1, abort_flag, args.status, 6)) break;
                if (j >= LT::kOBufs) {
                    const uint32_t use = uint32_t(j / LT::kOBufs) - 1;      // the read of the buffer's previous use
                    if (!mbar_wait(&bars->o_free[ob], use & 1, abort_flag, args.status, 7)) break;
                }
                tc_fence_after();
                const uint32_t v_addr = smem_u32(v_smem + slot * LT::kTileBytes);
                const uint32_t p_tmem = tmem + ((j & 1) ? LT::kSCol1 : LT::kSCol0);
                const uint32_t o_tmem = tmem + LT::kOCol0 + ob * D;
                #pragma unroll
                for (int ks = 0; ks < kTileKeys / 16; ++ks) {
                    mma_ts(o_tmem, p_tmem + ks * 8, smem_desc(v_addr + ks * 2048, kTileKeys * 128), idesc_pv,
                           ks != 0 ? 1u : 0u);
                }
                tc_commit(&bars->v_empty[slot]);
                tc_commit(&bars->o_full[ob]);
            }
        }
    } else if (warp < 6) {
        // ===== softmax: thread = row =====
        const int quad = warp & 3;                           // the TMEM lane quadrant this warp may touch
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const int g = row & (G - 1);
        const bool valid = t_local < valid_tokens;
        // Q tile: this thread copies its own row into the swizzled K-major layout.
        {
            const uint16_t* src = args.q + (size_t(token0 + t_local) * args.q_heads + size_t(kv_head) * G + g) * D;
            #pragma unroll
            for (int b = 0; b < LT::kBlocks; ++b) {
                #pragma unroll
                for (int ch = 0; ch < 8; ++ch) {
                    uint4 value = make_uint4(0, 0, 0, 0);
                    if (valid) value = *reinterpret_cast<const uint4*>(src + b * 64 + ch * 8);
                    *reinterpret_cast<uint4*>(q_smem + b * (kRows * 128) + row * 128 + ((ch ^ (row & 7)) << 4)) = value;
                }
            }
            fence_proxy_async();
            mbar_arrive(&bars->q_full);
        }
        const int pos = valid ? first_pos + t_local : -1;
        const int lo = args.window > 0 ? max(0, pos - args.window + 1) : 0;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        const float neg_inf = __int_as_float(0xff800000);
        const bool warp_has_rows = quad * 32 < valid_rows;     // warp-uniform
        for (int j = 0; j < n_tiles; ++j) {
            const int sb = j & 1;
            if (!mbar_wait(&bars->s_full[sb], uint32_t(j >> 1) & 1, abort_flag, args.status, 8)) break;
            tc_fence_after();
            if (!warp_has_rows) {
                // No query row lives in this quadrant: its P rows stay whatever they were and the
                // O rows they produce are never read (rows are independent).
                tc_fence_before();
                mbar_arrive(&bars->p_full[sb]);
                continue;
            }
            const uint32_t s_tmem = tmem + lane_base + (sb ? LT::kSCol1 : LT::kSCol0);
            const int key0 = (tile_first + j * world) * kTileKeys;
            const int c_lo = lo - key0;                      // visible columns: [c_lo, c_hi]
            const int c_hi = pos - key0;
            uint32_t s[4][32];
            HC_TMEM_LD32(s_tmem + 0, s[0]);
            HC_TMEM_LD32(s_tmem + 32, s[1]);
            HC_TMEM_LD32(s_tmem + 64, s[2]);
            HC_TMEM_LD32(s_tmem + 96, s[3]);
            tc_wait_ld();
            float m = neg_inf;
            if (c_lo <= 0 && c_hi >= kTileKeys - 1) {
                #pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) m = fmaxf(m, __uint_as_float(s[q4][i]));
                }
            } else {
                #pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = q4 * 32 + i;
                        const float value = (col >= c_lo && col <= c_hi) ? __uint_as_float(s[q4][i]) : neg_inf;
                        s[q4][i] = __float_as_uint(value);
                        m = fmaxf(m, value);
                    }
                }
            }
            const float m_safe = (m == neg_inf) ? 0.0f : m;
            float sum = 0.0f;
            #pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                uint32_t packed[16];
                #pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float p0 = tile_weight(__uint_as_float(s[q4][2 * i]), m_safe, args.c);
                    const float p1 = tile_weight(__uint_as_float(s[q4][2 * i + 1]), m_safe, args.c);
                    sum = __fadd_rn(sum, p0);
                    sum = __fadd_rn(sum, p1);
                    packed[i] = (__float_as_uint(p0) >> 16) | (__float_as_uint(p1) & 0xffff0000u);
                }
                HC_TMEM_ST16(s_tmem + q4 * 16, packed);
            }
            bars->mm[j & 3][row] = __fmul_rn(m, args.c);
            bars->l[j & 3][row] = sum;
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(&bars->p_full[sb]);
        }
    } else {
        // ===== fold + epilogue: thread = row =====
        const int quad = warp & 3;
        const int row = quad * 32 + lane;
        const int t_local = row >> args.log_group;
        const int g = row & (G - 1);
        const int head = kv_head * G + g;
        const bool valid = t_local < valid_tokens;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
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
        bool ok = true;
        const bool warp_has_rows = quad * 32 < valid_rows;     // warp-uniform
        for (int j = 0; j < n_tiles; ++j) {
            const int ob = LT::kOBufs == 2 ? (j & 1) : 0;
            if (!mbar_wait(&bars->o_full[ob], uint32_t(j / LT::kOBufs) & 1, abort_flag, args.status, 9)) {
                ok = false;
                break;
            }
            tc_fence_after();
            if (!warp_has_rows) {
                tc_fence_before();
                mbar_arrive(&bars->o_free[ob]);
                continue;
            }
            if (args.decode) {
                // Split decode: the tile's partial goes to the workspace; merge_tiles_kernel folds.
                const size_t prow = (size_t(token0) * args.q_heads + head) * args.part_tiles + (ordinal0 + j);
                const uint32_t o_tmem = tmem + lane_base + LT::kOCol0 + ob * D;
                #pragma unroll
                for (int half = 0; half < D / 64; ++half) {
                    uint32_t o[2][32];
                    HC_TMEM_LD32(o_tmem + half * 64, o[0]);
                    HC_TMEM_LD32(o_tmem + half * 64 + 32, o[1]);
                    tc_wait_ld();
                    if (half == D / 64 - 1) {
                        tc_fence_before();
                        mbar_arrive(&bars->o_free[ob]);
                    }
                    if (valid) {
                        float* dst = args.part_o + prow * D + half * 64;
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
                    args.part_ml[prow * 2] = bars->mm[j & 3][row];
                    args.part_ml[prow * 2 + 1] = bars->l[j & 3][row];
                }
                continue;
            }
            float Mn, a, b;
            fold_coefficients(M, bars->mm[j & 3][row], Mn, a, b);
            L = __fmaf_rn(L, a, __fmul_rn(bars->l[j & 3][row], b));
            M = Mn;
            const uint32_t o_tmem = tmem + lane_base + LT::kOCol0 + ob * D;
            #pragma unroll
            for (int half = 0; half < D / 64; ++half) {
                uint32_t o[2][32];
                HC_TMEM_LD32(o_tmem + half * 64, o[0]);
                HC_TMEM_LD32(o_tmem + half * 64 + 32, o[1]);
                tc_wait_ld();
                if (half == D / 64 - 1) {
                    tc_fence_before();
                    mbar_arrive(&bars->o_free[ob]);
                }
                #pragma unroll
                for (int u = 0; u < 2; ++u) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int col = half * 64 + u * 32 + i;
                        A[col] = fold_value(A[col], a, __uint_as_float(o[u][i]), b);
                    }
                }
            }
        }
        if (ok && valid && !args.decode) {
            const size_t out_row = size_t(token0 + t_local);
            if (args.ep.write_partial) {
                float* dst = reinterpret_cast<float*>(args.ep.out) + (out_row * args.q_heads + head) * size_t(D + 2);
                #pragma unroll
                for (int i = 0; i < D; i += 4) {
                    *reinterpret_cast<float4*>(dst + i) = make_float4(A[i], A[i + 1], A[i + 2], A[i + 3]);
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
                        packed.x = uint32_t(float_to_bf16_bits(r[0])) | (uint32_t(float_to_bf16_bits(r[1])) << 16);
                        packed.y = uint32_t(float_to_bf16_bits(r[2])) | (uint32_t(float_to_bf16_bits(r[3])) << 16);
                        packed.z = uint32_t(float_to_bf16_bits(r[4])) | (uint32_t(float_to_bf16_bits(r[5])) << 16);
                        packed.w = uint32_t(float_to_bf16_bits(r[6])) | (uint32_t(float_to_bf16_bits(r[7])) << 16);
                        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(args.ep.out) + vec * D + i) = packed;
                    }
                }
            }
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
static hc_status launch_tc(hc_context* ctx, const TcArgs& args, const hc_layer_store& layer, int grid_x,
                           cudaStream_t stream, int grid_z = 1) {
    using LT = TcLayout<D>;
    const int smem = LT::kSmemBytes + int(sizeof(TcBarriers));
    cudaError_t err = cudaFuncSetAttribute(prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return check_cuda(err, "prefill_tc_kernel shared memory");
    dim3 grid(grid_x, args.kv_heads, grid_z);
    prefill_tc_kernel<D><<<grid, kTcThreads, smem, stream>>>(*static_cast<const CUtensorMap*>(layer.tmap_k),
                                                            *static_cast<const CUtensorMap*>(layer.tmap_v), args);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "prefill_tc_kernel launch");
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
    const int n_mtiles = (tokens + tokens_per_tile - 1) / tokens_per_tile;
    if (shape.head_dim == 64) return launch_tc<64>(ctx, args, layer, n_mtiles, stream);
    return launch_tc<128>(ctx, args, layer, n_mtiles, stream);
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
    // Enough CTAs to cover the machine about twice, each with a run of consecutive tiles.
    const long long target = 2LL * std::max(ctx->sm_count, 1);
    long long per = (total_tiles * shape.kv_heads + target - 1) / target;
    args.tiles_per_cta = int(std::min<long long>(std::max<long long>(per, 1), 64));
    args.part_o = ws.part_o;
    args.part_ml = ws.part_ml;
    args.part_tiles = max_tiles;
    args.meta = meta;
    const int grid_x = (max_tiles + args.tiles_per_cta - 1) / args.tiles_per_cta;
    hc_status st = shape.head_dim == 64 ? launch_tc<64>(ctx, args, layer, grid_x, stream, n_seq)
                                        : launch_tc<128>(ctx, args, layer, grid_x, stream, n_seq);
    if (st != HC_OK) return st;
    return launch_merge(ctx, shape, meta, n_seq, ws, max_tiles, world, cache.map.rank, ep, stream);
}

}  // namespace hc
