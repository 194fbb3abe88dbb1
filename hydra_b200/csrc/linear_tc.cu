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
constexpr int kLinN = 256;
constexpr int kLinK = 64;                       // one 128-byte swizzled row of bf16
constexpr int kLinStages = 4;
constexpr int kLinABytes = kLinM * kLinK * 2;   // 16 KB
constexpr int kLinBBytes = kLinN * kLinK * 2;   // 32 KB
constexpr int kLinThreads = 256;

struct LinBarriers {
    uint64_t full[kLinStages], empty[kLinStages];
    uint64_t acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

struct LinArgs {
    const uint16_t* bias;     // bf16 [out_features] or null
    const float* residual;    // fp32 [tokens][out_features] added to the result, or null (may be y itself)
    void* y;                  // [tokens][out_features]
    int y_dtype;              // HC_F32 or HC_BF16
    int tokens, out_features;
    int tiles_m, tiles_n, k_steps;
    int* status;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

__global__ void __launch_bounds__(kLinThreads, 1)
linear_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                 const LinArgs args) {
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
    if (warp == 1) tmem_alloc(&bars->tmem_base, 512);
    if (warp == 0 && lane == 0) {
        prefetch_tensormap(&tmap_x);
        prefetch_tensormap(&tmap_w);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = bars->tmem_base;
    pdl_wait();

    const int n_tiles = args.tiles_m * args.tiles_n;
    if (warp == 0) {
        // ===== producer =====
        if (lane == 0) {
            uint32_t step = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const int tn = tile / args.tiles_m, tm = tile - tn * args.tiles_m;
                for (int k = 0; k < args.k_steps; ++k, ++step) {
                    const int slot = int(step % kLinStages);
                    const uint32_t round = step / kLinStages;
                    if (round > 0 && !mbar_wait(&bars->empty[slot], (round - 1) & 1, abort_flag, args.status, 21)) { ok = false; break; }
                    mbar_expect_tx(&bars->full[slot], kLinABytes + kLinBBytes);
                    tma_load_2d(a_smem + slot * kLinABytes, &tmap_x, &bars->full[slot], k * kLinK, tm * kLinM);
                    tma_load_2d(b_smem + slot * kLinBBytes, &tmap_w, &bars->full[slot], k * kLinK, tn * kLinN);
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
            const int tn = tile / args.tiles_m, tm = tile - tn * args.tiles_m;
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
                if (row_ok && col0 < args.out_features) {
                float r[32];
                #pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int col = col0 + i;
                    const float b = (args.bias != nullptr && col < args.out_features) ? bf16_bits_to_float(__ldg(args.bias + col)) : 0.0f;
                    r[i] = __fadd_rn(__uint_as_float(v[i]), b);
                }
                const size_t offset = size_t(row) * args.out_features + col0;
                if (args.residual != nullptr) {
                    #pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        if (col0 + i < args.out_features) r[i] = __fadd_rn(r[i], __ldg(args.residual + offset + i));
                    }
                }
                const bool whole = col0 + 32 <= args.out_features && (args.out_features & 7) == 0;
                if (args.y_dtype == HC_F32) {
                    float* dst = reinterpret_cast<float*>(args.y) + offset;
                    if (whole) {
                        #pragma unroll
                        for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(r[i], r[i + 1], r[i + 2], r[i + 3]);
                    } else {
                        for (int i = 0; i < 32 && col0 + i < args.out_features; ++i) dst[i] = r[i];
                    }
                } else {
                    uint16_t* dst = reinterpret_cast<uint16_t*>(args.y) + offset;
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
                        for (int i = 0; i < 32 && col0 + i < args.out_features; ++i) dst[i] = float_to_bf16_bits(r[i]);
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
    if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace

hc_status linear_tc(hc_context* ctx, const void* x, const void* w, const void* bias, const float* residual, void* y,
                    int tokens, int in_features, int out_features, int y_dtype, cudaStream_t stream) {
    CUtensorMap tmap_x, tmap_w;
    hc_status st = tc_encode_2d(&tmap_x, x, uint64_t(tokens), uint64_t(in_features), kLinM);
    if (st == HC_OK) st = tc_encode_2d(&tmap_w, w, uint64_t(out_features), uint64_t(in_features), kLinN);
    if (st != HC_OK) return st;
    LinArgs args{};
    args.bias = static_cast<const uint16_t*>(bias);
    args.residual = residual;
    args.y = y;
    args.y_dtype = y_dtype;
    args.tokens = tokens;
    args.out_features = out_features;
    args.tiles_m = (tokens + kLinM - 1) / kLinM;
    args.tiles_n = (out_features + kLinN - 1) / kLinN;
    args.k_steps = in_features / kLinK;
    args.status = ctx->status_dev;
    const int smem = 1024 + kLinStages * (kLinABytes + kLinBBytes) + int(sizeof(LinBarriers));
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        cudaError_t err = cudaFuncSetAttribute(linear_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return check_cuda(err, "linear_tc_kernel shared memory");
        configured[ctx->device & 63] = true;
    }
    const int grid = std::max(1, std::min(args.tiles_m * args.tiles_n, std::max(ctx->sm_count, 1)));
    const cudaError_t launched = launch_pdl(linear_tc_kernel, grid, kLinThreads, size_t(smem), stream, tmap_x, tmap_w, args);
    ctx->launches += 1;
    if (launched != cudaSuccess) return check_cuda(launched, "linear_tc_kernel launch");
    return check_cuda(cudaGetLastError(), "linear_tc_kernel launch");
}

}  // namespace hc
