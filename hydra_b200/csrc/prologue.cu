// prologue.cu — everything that happens to q, k and v before attention, in one kernel:
// per-head RMSNorm, half-split rotation, rounding to bf16 and, for k and v, the store into the
// cache.  Also the stand-alone element-wise kernels of the protocol.
//
// Replaces, fused: rms_norm_heads (Sources/HydraMetal/Shaders/gemma.metal:785-821), rope_apply /
// rope_apply_batch / rope_apply_batched (attention.metal:48-72, batch.metal:224-251,
// gemma.metal:961-984) and kv_cache_write / kv_cache_write_batch (dense.metal:66-86,
// batch.metal:254-277).  The order is the reference's: norm, then rotation, then the cast
// (Sources/HydraReference/Gemma4ReferenceLayer.swift:154-157, 234-246); v is normalised without a
// weight and never rotated.
//
// One warp handles one head vector.  HBM-bound and tiny: a chunk of 512 tokens moves a few MB.

#include <algorithm>

#include "internal.hpp"

namespace hc {
namespace {

constexpr int kPrepWarps = 8;
constexpr int kMaxHeadDim = 512;

// One head vector of 32 * PER elements handled by one warp with no staging: lane l holds elements
// l + 32 j, so both members of every rotation pair (i, i + d/2) sit in one lane.  The arithmetic and
// its order are those of the staged path below.
template <int PER>
__device__ __forceinline__ void prepare_in_lanes(const PrepJob& job, size_t src_base, uint16_t* dst16,
                                                 const float* cos_row, const float* sin_row, float eps, int lane) {
    constexpr int kHalfPer = PER / 2;
    constexpr int d = 32 * PER;
    constexpr int half = d / 2;
    float xv[PER], cv[kHalfPer], sv[kHalfPer];
    #pragma unroll
    for (int j = 0; j < PER; ++j) xv[j] = load_io(job.src, src_base + lane + 32 * j, job.src_dtype);
    if (cos_row) {
        #pragma unroll
        for (int j = 0; j < kHalfPer; ++j) {
            cv[j] = cos_row[lane + 32 * j];
            sv[j] = sin_row[lane + 32 * j];
        }
    }
    if (job.norm != 0) {
        float sum = 0.0f;
        #pragma unroll
        for (int j = 0; j < PER; ++j) sum = __fmaf_rn(xv[j], xv[j], sum);
        #pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, offset));
        }
        const float inverse = __frsqrt_rn(__fadd_rn(__fdiv_rn(sum, float(d)), eps));
        #pragma unroll
        for (int j = 0; j < PER; ++j) {
            float value = __fmul_rn(xv[j], inverse);
            if (job.norm == 1) value = __fmul_rn(value, bf16_bits_to_float(job.weight[lane + 32 * j]));
            xv[j] = value;
        }
    }
    #pragma unroll
    for (int j = 0; j < kHalfPer; ++j) {
        float x1 = xv[j], x2 = xv[j + kHalfPer];
        if (cos_row) {
            const float r1 = __fmaf_rn(x1, cv[j], -__fmul_rn(x2, sv[j]));
            const float r2 = __fmaf_rn(x2, cv[j], __fmul_rn(x1, sv[j]));
            x1 = r1;
            x2 = r2;
        }
        const int i = lane + 32 * j;
        if (job.kind == 3) {
            store_io(job.dst, src_base + i, job.src_dtype, x1);
            store_io(job.dst, src_base + half + i, job.src_dtype, x2);
        } else {
            dst16[i] = float_to_bf16_bits(x1);
            dst16[half + i] = float_to_bf16_bits(x2);
        }
    }
}

__global__ void __launch_bounds__(kPrepWarps * 32)
prepare_heads_kernel(const PrepArgs args) {
    __shared__ float stage[kPrepWarps][kMaxHeadDim];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int d = args.head_dim;
    const int half = d >> 1;

    int total_heads = 0;
    for (int j = 0; j < args.n_jobs; ++j) total_heads += args.job[j].heads;
    // Warps stride over the (token, head) vectors of the call.
    // 32-bit indices: a launch covers at most 32768 tokens x a few hundred heads.
    const unsigned vectors = unsigned(args.tokens) * unsigned(total_heads);
    const unsigned stride = gridDim.x * kPrepWarps;
    for (unsigned vec = blockIdx.x * kPrepWarps + warp; vec < vectors; vec += stride) {
    const int token = int(vec / unsigned(total_heads));
    const int slot = int(vec - unsigned(token) * unsigned(total_heads));
    int job_index = 0, head = slot;
    while (head >= args.job[job_index].heads) {
        head -= args.job[job_index].heads;
        ++job_index;
    }
    const PrepJob& job = args.job[job_index];

    const int position = args.batched ? args.meta.pos[token] : args.first_position + token;
    const int seq = args.batched ? args.meta.seq[token] : args.seq;
    if (job.kind == 1 || job.kind == 2) {
        if (!row_is_local(args.cache.map, position)) continue;   // another rank owns this key tile
    }

    const size_t src_base = size_t(token) * size_t(job.token_stride) + size_t(head) * job.head_stride;
    const bool rotate = job.rope != 0;
    const int table_row = position < args.table_positions ? position : args.table_positions - 1;
    // Destination of this head vector.
    uint16_t* dst16 = nullptr;
    if (job.kind == 0) {
        dst16 = reinterpret_cast<uint16_t*>(job.dst) + (size_t(token) * job.heads + head) * d;
    } else if (job.kind == 1 || job.kind == 2) {
        const int row = row_of_position(args.cache.map, position);
        uint16_t* base = job.kind == 1 ? args.cache.k : args.cache.v;
        dst16 = base + ((size_t(seq) * args.cache.kv_heads + head) * args.cache.capacity + row) * d;
    }

    if ((half & 31) == 0) {
        // Fast path (head_dim 64, 128, 256, 512): no staging, all loads issued up front.
        const float* cos_row = rotate ? args.cos + size_t(table_row) * half : nullptr;
        const float* sin_row = rotate ? args.sin + size_t(table_row) * half : nullptr;
        switch (d >> 5) {
            case 2: prepare_in_lanes<2>(job, src_base, dst16, cos_row, sin_row, args.eps, lane); break;
            case 4: prepare_in_lanes<4>(job, src_base, dst16, cos_row, sin_row, args.eps, lane); break;
            case 8: prepare_in_lanes<8>(job, src_base, dst16, cos_row, sin_row, args.eps, lane); break;
            default: prepare_in_lanes<16>(job, src_base, dst16, cos_row, sin_row, args.eps, lane); break;
        }
        continue;
    }

    // General path (small or odd head dims): stage the vector in shared memory.
    __syncwarp();                                  // the staging row is reused
    float* x = stage[warp];
    float sum = 0.0f;
    for (int i = lane; i < d; i += 32) {
        const float value = load_io(job.src, src_base + i, job.src_dtype);
        x[i] = value;
        sum = __fmaf_rn(value, value, sum);
    }
    if (job.norm != 0) {
        #pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) {
            sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, offset));
        }
        const float inverse = __frsqrt_rn(__fadd_rn(__fdiv_rn(sum, float(d)), args.eps));
        for (int i = lane; i < d; i += 32) {
            float value = __fmul_rn(x[i], inverse);
            if (job.norm == 1) value = __fmul_rn(value, bf16_bits_to_float(job.weight[i]));
            x[i] = value;
        }
    }
    __syncwarp();
    for (int i = lane; i < half; i += 32) {
        float x1 = x[i], x2 = x[half + i];
        if (rotate) {
            const float c = args.cos[size_t(table_row) * half + i];
            const float s = args.sin[size_t(table_row) * half + i];
            const float r1 = __fmaf_rn(x1, c, -__fmul_rn(x2, s));
            const float r2 = __fmaf_rn(x2, c, __fmul_rn(x1, s));
            x1 = r1;
            x2 = r2;
        }
        if (job.kind == 3) {
            store_io(job.dst, src_base + i, job.src_dtype, x1);
            store_io(job.dst, src_base + half + i, job.src_dtype, x2);
        } else {
            dst16[i] = float_to_bf16_bits(x1);
            dst16[half + i] = float_to_bf16_bits(x2);
        }
    }
    }
}

__global__ void split_query_gate_kernel(const void* combined, void* query, void* gate, size_t count,
                                        int d, int dtype) {
    // count = tokens * heads * d; element e = (token*heads + head) * d + i
    const size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count) return;
    const size_t vec = e / d;
    const int i = int(e % d);
    store_io(query, e, dtype, load_io(combined, vec * 2 * d + i, dtype));
    store_io(gate, e, dtype, load_io(combined, vec * 2 * d + d + i, dtype));
}

__global__ void output_gate_kernel(void* output, const void* gate, size_t count, int dtype) {
    const size_t e = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (e >= count) return;
    const float value = load_io(output, e, dtype);
    store_io(output, e, dtype, __fmul_rn(value, sigmoid_gate(load_io(gate, e, dtype))));
}

}  // namespace

hc_status launch_prepare(hc_context* ctx, const PrepArgs& args, cudaStream_t stream) {
    int total_heads = 0;
    for (int j = 0; j < args.n_jobs; ++j) total_heads += args.job[j].heads;
    if (total_heads == 0 || args.tokens == 0) return HC_OK;
    const long long vectors = (long long)args.tokens * total_heads;
    const long long wanted = (vectors + kPrepWarps - 1) / kPrepWarps;
    const int grid = int(std::min<long long>(wanted, (long long)std::max(ctx->sm_count, 1) * 16));
    prepare_heads_kernel<<<grid, kPrepWarps * 32, 0, stream>>>(args);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "prepare_heads_kernel launch");
}

hc_status launch_split_query_gate(hc_context* ctx, const void* combined, void* query, void* gate,
                                  int tokens, int heads, int d, int dtype, cudaStream_t stream) {
    const size_t count = size_t(tokens) * heads * d;
    if (count == 0) return HC_OK;
    split_query_gate_kernel<<<unsigned((count + 255) / 256), 256, 0, stream>>>(combined, query, gate,
                                                                               count, d, dtype);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "split_query_gate_kernel launch");
}

hc_status launch_output_gate(hc_context* ctx, void* output, const void* gate, size_t count,
                             int dtype, cudaStream_t stream) {
    if (count == 0) return HC_OK;
    output_gate_kernel<<<unsigned((count + 255) / 256), 256, 0, stream>>>(output, gate, count, dtype);
    ctx->launches += 1;
    return check_cuda(cudaGetLastError(), "output_gate_kernel launch");
}

}  // namespace hc
