// linear_tc.cu — the projections around the attention path on the 5th-generation tensor cores:
// y[t][o] = sum_i x[t][i] * w[o][i] (+ bias[o]), bf16 x bf16 -> fp32.
//
// Replaces bf16_gemv (Sources/HydraMetal/Shaders/dense.metal:14-60) and its batched and tiled
// forms (Sources/HydraMetal/Shaders/batch.metal:36-88, tiled.metal:48-120) for the Q, K, V and O
// projections; the CPU statement is ReferenceLayer.matVec
// (Sources/HydraReference/ReferenceLayer.swift:104-113).  The weight keeps the reference's layout:
// row-major [out_features][in_features] bf16, so both operands are K-major and no transpose is
// needed.  Where the reference gives every output row its own threadgroup that streams that row
// of the weight once per token, this kernel computes a 128 x 256 tile of y per step, so a weight
// tile fetched by TMA serves 128 tokens.
//
// One persistent CTA per SM walks the output tiles (all row tiles of one 256-wide column tile are
// adjacent in the walk, so the CTAs running at one time share a weight tile in L2):
//   warp 0      TMA producer: x tile (128 x 64) and w tile (256 x 64) per K step into a 4-stage ring
//               (a launch may carry up to four projections of the same x: one list of tiles)
//   warp 1      MMA issuer: four tcgen05.mma (M 128, N 256, K 16) per K step into one of two
//               accumulators in tensor memory (2 x 256 columns)
//   warps 4-7   epilogue: the finished accumulator from tensor memory, + bias (+ residual), to y (fp32 or bf16),
//               thread = row, while the next tile's MMAs fill the other accumulator
// Every mbarrier wait is bounded and reports through the context's status word.

#include <algorithm>

#include "internal.hpp"
#include "tc_ptx.cuh"

namespace hc {
namespace {

constexpr int kLinM = 128;
constexpr int kLinK = 64;                       // one 128-byte swizzled row of bf16
constexpr int kLinABytes = kLinM * kLinK * 2;   // 16 KB
constexpr int kLinThreads = 256;
constexpr int kLinMaxStages = 9;

// Two shapes of the same kernel.  Wide: 128 x 256 output tiles, 4 stages: tensor-bound, for prompts.
// Narrow: 128 x 32 tiles, 9 stages: when there are at most 128 tokens (decode) the work is reading
// the weight once, and narrow column tiles spread its rows over all SMs with enough of them in
// flight (9 x 4 KB per SM).  An output element is the same sum in the same order in both, so a token
// projected alone and inside a prompt gets the same bits.
template <int BN>
struct LinShape {
    static constexpr int kStages = BN == 256 ? 4 : kLinMaxStages;
    static constexpr int kBBytes = BN * kLinK * 2;
    static constexpr int kTmemCols = BN == 256 ? 512 : 64;      // two accumulators
    static constexpr int kSmemBytes = 1024 + kStages * (kLinABytes + kBBytes);
};

struct LinBarriers {
    uint64_t full[kLinMaxStages], empty[kLinMaxStages];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

constexpr int kLinJobs = 4;

// One launch may carry several projections of the same x (q, k and v of a layer): their output tiles
// form one list, job after job.
struct LinJob {
    const uint16_t* bias;     // bf16 [out_features] or null
    const float* residual;    // fp32 [tokens][out_features] added to the result, or null (may be y itself)
    void* y;                  // [tokens][out_features]
    int out_features;
    int first_tile;           // of this job in the launch's list; its tiles: column tile major, row tiles adjacent
};

struct LinArgs {
    LinJob job[kLinJobs];
    int n_jobs;
    int y_dtype;              // HC_F32 or HC_BF16
    int tokens;
    int tiles_m, n_tiles, k_steps;
    int a_bytes;              // of one x box: 128 rows x 128 bytes, fewer rows for a call of few tokens
    int* status;
};

struct LinTile {
    int job, tn, tm;
};
__device__ __forceinline__ LinTile decode_tile(const LinArgs& args, int tile) {
    LinTile t;
    t.job = 0;
    #pragma unroll
    for (int j = 1; j < kLinJobs; ++j) {
        if (j < args.n_jobs && tile >= args.job[j].first_tile) t.job = j;
    }
    const int local = tile - args.job[t.job].first_tile;
    t.tn = local / args.tiles_m;
    t.tm = local - t.tn * args.tiles_m;
    return t;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

template <int BN>
__global__ void __launch_bounds__(kLinThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w0,
                 const __grid_constant__ CUtensorMap tmap_w1, const __grid_constant__ CUtensorMap tmap_w2,
                 const __grid_constant__ CUtensorMap tmap_w3, const LinArgs args) {
    using LS = LinShape<BN>;
    constexpr int kLinN = BN;
    constexpr int kLinStages = LS::kStages;
    constexpr int kLinBBytes = LS::kBBytes;
    extern __shared__ unsigned char raw_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
    unsigned char* a_smem = base;                                   // [stages][128 x 64]
    unsigned char* b_smem = a_smem + kLinStages * kLinABytes;       // [stages][256 x 64]
    LinBarriers* bars = reinterpret_cast<LinBarriers*>(b_smem + kLinStages * kLinBBytes);
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    volatile int* abort_flag = &bars->abort_flag;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int i = 0; i < kLinStages; ++i) {
            mbar_init(&bars->full[i], 1);
            mbar_init(&bars->empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->acc_full[i], 1);
            mbar_init(&bars->acc_empty[i], 128);
        }
        bars->abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(&bars->tmem_base, LS::kTmemCols);
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tmap_x);
        prefetch_tensormap(&tmap_w0);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    pdl_wait();

    const int n_tiles = args.n_tiles;
    if (warp == 0) {
        // ===== producer =====
        if (lane == 0) {
            uint32_t step = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const LinTile where = decode_tile(args, tile);
                const int tn = where.tn, tm = where.tm;
                const CUtensorMap* tmap_w = where.job == 0 ? &tmap_w0 : where.job == 1 ? &tmap_w1 : where.job == 2 ? &tmap_w2 : &tmap_w3;
                for (int k = 0; k < args.k_steps; ++k, ++step) {
                    const int slot = int(step % kLinStages);
                    const uint32_t round = step / kLinStages;
                    if (round > 0 && !mbar_wait(&bars->empty[slot], (round - 1) & 1, abort_flag, args.status, 21)) { ok = false; break; }
                    mbar_expect_tx(&bars->full[slot], uint32_t(args.a_bytes) + kLinBBytes);
                    tma_load_2d(a_smem + slot * kLinABytes, &tmap_x, &bars->full[slot], k * kLinK, tm * kLinM);
                    tma_load_2d(b_smem + slot * kLinBBytes, tmap_w, &bars->full[slot], k * kLinK, tn * kLinN);
                }
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer (the warp walks the loop converged; one elected lane issues) =====
        constexpr uint32_t idesc = instr_desc(kLinN, false);
        const uint64_t a_desc0 = smem_desc(smem_u32(a_smem), 16);
        const uint64_t b_desc0 = smem_desc(smem_u32(b_smem), 16);
        uint32_t step = 0, count = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++count) {
            const int acc = int(count & 1);
            // The epilogue must have taken this accumulator's previous tile out.
            if (count >= 2 && !mbar_wait(&bars->acc_empty[acc], ((count >> 1) - 1) & 1, abort_flag, args.status, 22)) break;
            tc_fence_after();
            for (int k = 0; k < args.k_steps; ++k, ++step) {
                const int slot = int(step % kLinStages);
                if (!mbar_wait(&bars->full[slot], (step / kLinStages) & 1, abort_flag, args.status, 23)) { ok = false; break; }
                tc_fence_after();
                if (elect_one()) {
                    const uint64_t a_desc = a_desc0 + uint64_t((slot * kLinABytes) >> 4);
                    const uint64_t b_desc = b_desc0 + uint64_t((slot * kLinBBytes) >> 4);
                    #pragma unroll
                    for (int ks = 0; ks < kLinK / 16; ++ks) {
                        mma_ss(tmem + acc * kLinN, a_desc + uint64_t((ks * 32) >> 4), b_desc + uint64_t((ks * 32) >> 4), idesc,
                               (k | ks) != 0 ? 1u : 0u);
                    }
                    tc_commit(&bars->empty[slot]);
                    if (k + 1 == args.k_steps) tc_commit(&bars->acc_full[acc]);
                }
                __syncwarp();
            }
        }
    } else if (warp >= 4) {
        // ===== epilogue: thread = row of the tile =====
        const int quad = warp & 3;
        const int row_in_tile = quad * 32 + lane;
        const uint32_t lane_base = uint32_t(quad * 32) << 16;
        uint32_t count = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++count) {
            const LinTile where = decode_tile(args, tile);
            const int tn = where.tn, tm = where.tm;
            const LinJob& job = args.job[where.job];
            const int acc = int(count & 1);
            if (!mbar_wait(&bars->acc_full[acc], (count >> 1) & 1, abort_flag, args.status, 24)) break;
            tc_fence_after();
            const int row = tm * kLinM + row_in_tile;
            const bool row_ok = row < args.tokens;
            #pragma unroll 1
            for (int chunk = 0; chunk < kLinN / 32; ++chunk) {
                uint32_t v[32];
                HC_TMEM_LD32(tmem + lane_base + acc * kLinN + chunk * 32, v);
                tc_wait_ld();
                const int col0 = tn * kLinN + chunk * 32;
                if (row_ok && col0 < job.out_features) {
                float r[32];
                #pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int col = col0 + i;
                    const float b = (job.bias != nullptr && col < job.out_features) ? bf16_bits_to_float(__ldg(job.bias + col)) : 0.0f;
                    r[i] = __fadd_rn(__uint_as_float(v[i]), b);
                }
                const size_t offset = size_t(row) * job.out_features + col0;
                if (job.residual != nullptr) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (col0 + i < job.out_features) r[i] = __fadd_rn(r[i], __ldg(job.residual + offset + i));
                    }
                }
                const bool whole = col0 + 32 <= job.out_features && (job.out_features & 7) == 0;
                if (args.y_dtype == HC_F32) {
                    float* dst = reinterpret_cast<float*>(job.y) + offset;
                    if (whole) {
                        #pragma unroll
                        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(r[i], r[i + 1], r[i + 2], r[i + 3]);
                    } else {
                        for (int i = 0; i < 32 && col0 + i < job.out_features; ++i) dst[i] = r[i];
                    }
                } else {
                    uint16_t* dst = reinterpret_cast<uint16_t*>(job.y) + offset;
                    if (whole) {
                        #pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 packed;
                            packed.x = uint32_t(float_to_bf16_bits(r[i])) | (uint32_t(float_to_bf16_bits(r[i + 1])) << 16);
                            packed.y = uint32_t(float_to_bf16_bits(r[i + 2])) | (uint32_t(float_to_bf16_bits(r[i + 3])) << 16);
                            packed.z = uint32_t(float_to_bf16_bits(r[i + 4])) | (uint32_t(float_to_bf16_bits(r[i + 5])) << 16);
                            packed.w = uint32_t(float_to_bf16_bits(r[i + 6])) | (uint32_t(float_to_bf16_bits(r[i + 7])) << 16);
                            *reinterpret_cast<uint4*>(dst + i) = packed;
                        }
                    } else {
                        for (int i = 0; i < 32 && col0 + i < job.out_features; ++i) dst[i] = float_to_bf16_bits(r[i]);
                    }
                }
                }
                __syncwarp();          // the next tcgen05.ld is warp-wide
            }
            tc_fence_before();
            mbar_arrive(&bars->acc_empty[acc]);
        }
    }

    // Teardown.  On the abort path the producer first lets its copies in flight land (bounded).
    if (warp == 0 && lane == 0 && *abort_flag != 0) {
        const long long start = clock64();
        while (static_cast<unsigned long long>(clock64() - start) < 200000000ull) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, LS::kTmemCols);
}

}  // namespace

// Encoding a tensor map costs a few microseconds of host time, as much as a decode-sized call's
// kernel; weights and activation buffers recur from call to call, so the last maps are kept, keyed
// by what determines them.  One caller thread per context: the cache is per thread.
static hc_status cached_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows) {
    struct Entry {
        const void* base;
        uint64_t rows, cols;
        uint32_t box_rows;
        CUtensorMap map;
    };
    constexpr int kEntries = 32;
    static thread_local Entry entries[kEntries];
    static thread_local int used = 0, next = 0;
    for (int i = 0; i < used; ++i) {
        const Entry& e = entries[i];
        if (e.base == base && e.rows == rows && e.cols == cols && e.box_rows == box_rows) {
            *out = e.map;
            return HC_OK;
        }
    }
    Entry& e = entries[next];
    const hc_status st = tc_encode_2d(&e.map, base, rows, cols, box_rows);
    if (st != HC_OK) {
        e.base = nullptr;
        return st;
    }
    e.base = base;
    e.rows = rows;
    e.cols = cols;
    e.box_rows = box_rows;
    *out = e.map;
    next = (next + 1) % kEntries;
    used = std::min(used + 1, kEntries);
    return HC_OK;
}

template <int BN>
static hc_status launch_linear(hc_context* ctx, const void* x, const void* const* w, LinArgs args, int in_features,
                               cudaStream_t stream) {
    using LS = LinShape<BN>;
    CUtensorMap tmap_x, tmap_w[kLinJobs];
    // A box that reaches past the last token is filled with zeros, and that fill measured slower than
    // reading real rows (one token: 21 us against 13 us for 128): a call of few tokens loads only the
    // rows it has.  The rows of the 128-row operand tile it leaves unwritten feed accumulator rows that
    // are never stored (a row of the result depends on its own row of x alone).
    const int x_rows = std::min(kLinM, (args.tokens + 7) & ~7);
    args.a_bytes = x_rows * kLinK * 2;
    hc_status st = cached_map(&tmap_x, x, uint64_t(args.tokens), uint64_t(in_features), uint32_t(x_rows));
    args.tiles_m = (args.tokens + kLinM - 1) / kLinM;
    int tiles = 0;
    for (int j = 0; j < kLinJobs && st == HC_OK; ++j) {
        const int source = j < args.n_jobs ? j : 0;            // unused maps repeat the first
        st = cached_map(&tmap_w[j], w[source], uint64_t(args.job[source].out_features), uint64_t(in_features), BN);
        if (j < args.n_jobs) {
            args.job[j].first_tile = tiles;
            tiles += args.tiles_m * ((args.job[j].out_features + BN - 1) / BN);
        }
    }
    if (st != HC_OK) return st;
    args.n_tiles = tiles;
    const int smem = LS::kSmemBytes + int(sizeof(LinBarriers));
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        cudaError_t err = cudaFuncSetAttribute(linear_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return check_cuda(err, "linear_tc_kernel shared memory");
        configured[ctx->device & 63] = true;
    }
    const int grid = std::max(1, std::min(tiles, std::max(ctx->sm_count, 1)));
    const cudaError_t launched = launch_pdl(linear_tc_kernel<BN>, grid, kLinThreads, size_t(smem), stream, tmap_x, tmap_w[0],
                                            tmap_w[1], tmap_w[2], tmap_w[3], args);
    ctx->launches += 1;
    if (launched != cudaSuccess) return check_cuda(launched, "linear_tc_kernel launch");
    return check_cuda(cudaGetLastError(), "linear_tc_kernel launch");
}

hc_status linear_tc(hc_context* ctx, const void* x, int n_jobs, const void* const* w, const void* const* bias,
                    const float* const* residual, void* const* y, const int* out_features, int tokens, int in_features,
                    int y_dtype, cudaStream_t stream) {
    LinArgs args{};
    args.n_jobs = n_jobs;
    for (int j = 0; j < n_jobs; ++j) {
        args.job[j].bias = bias ? static_cast<const uint16_t*>(bias[j]) : nullptr;
        args.job[j].residual = residual ? residual[j] : nullptr;
        args.job[j].y = y[j];
        args.job[j].out_features = out_features[j];
    }
    args.y_dtype = y_dtype;
    args.tokens = tokens;
    args.k_steps = in_features / kLinK;
    args.status = ctx->status_dev;
    if (tokens <= kLinM) return launch_linear<32>(ctx, x, w, args, in_features, stream);
    return launch_linear<256>(ctx, x, w, args, in_features, stream);
}

}  // namespace hc
